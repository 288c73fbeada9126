// Element-wise companions of the expert products: routing-weighted sum and the SwiGLU gate.
#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
// out[t, h0..h0+7] = sum_j w[t, j] * Y[t * K + j, h0..h0+7]: fp32, experts in order j = 0..K-1, BF16 round at the end
template <bool WBF16>
__global__ void __launch_bounds__(256) wsum_kernel(const uint4* __restrict__ Y, const void* __restrict__ w,
                                                   uint4* __restrict__ out, long long T, int K, int H8) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= T * H8) return;
  const long long t = i / H8;
  const int c = (int)(i % H8);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < K; ++j) {
    const float wt = WBF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[t * K + j])
                           : reinterpret_cast<const float*>(w)[t * K + j];
    const uint4 v = Y[(t * K + j) * H8 + c];
    const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc[2 * q] += wt * __uint_as_float(p[q] << 16);
      acc[2 * q + 1] += wt * __uint_as_float(p[q] & 0xFFFF0000u);
    }
  }
  uint4 o;
  o.x = st::pack_bf16(acc[0], acc[1]); o.y = st::pack_bf16(acc[2], acc[3]);
  o.z = st::pack_bf16(acc[4], acc[5]); o.w = st::pack_bf16(acc[6], acc[7]);
  out[t * H8 + c] = o;
}

// act[s, i] = bf16(silu(gate)) * up with gate = gu[s, i], up = gu[s, I + i]
__device__ __forceinline__ __nv_bfloat16 silu_mul_one(__nv_bfloat16 gate, __nv_bfloat16 up) {
  const float gte = __bfloat162float(gate);
  return __hmul(__float2bfloat16_rn(gte / (1.f + __expf(-gte))), up);
}
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ gu,
                                                       __nv_bfloat16* __restrict__ act, long long S, long long I) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= S * I) return;
  const long long s = i / I, c = i % I;
  act[i] = silu_mul_one(gu[s * 2 * I + c], gu[s * 2 * I + I + c]);
}
// eight values per thread, 16-byte loads and stores (I a multiple of 8, 16-byte aligned rows); blockIdx.y = row
__global__ void __launch_bounds__(256) silu_mul_vec_kernel(const uint4* __restrict__ gu, uint4* __restrict__ act, int I8) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= I8) return;
  const size_t s = blockIdx.y;
  const uint4 g = gu[s * 2 * I8 + c], u = gu[s * 2 * I8 + I8 + c];
  const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(&gs[j]);
    const __nv_bfloat162 uv = *reinterpret_cast<const __nv_bfloat162*>(&us[j]);
    __nv_bfloat162 r;
    r.x = silu_mul_one(gv.x, uv.x);
    r.y = silu_mul_one(gv.y, uv.y);
    o[j] = *reinterpret_cast<const uint32_t*>(&r);
  }
  act[s * I8 + c] = make_uint4(o[0], o[1], o[2], o[3]);
}
// Groups the S (token, expert) pairs by expert in blocks of bs (8 for the grouped GEMV, 64 / 128 for the grouped
// tcgen05 GEMM; the layout vLLM's moe_align_block_size produces and
// the grouped expert kernels consume): sorted[nblk * bs] holds pair indices, expert-major, original order inside an
// expert, every expert's run padded to a multiple of bs with the value S; bexp[b] = expert of block b; npost = entries
// in use.  One CTA does the whole job in shared memory: histogram, padded prefix sum, one warp per expert placing its
// pairs in order with ballots, a binary search per block.  Expert ids outside [0, E) count as E - 1 / 0 (clamped).
constexpr int ALIGN_MAX_E = 1024;
template <bool IDS64>
__global__ void __launch_bounds__(1024) moe_align_kernel(const void* __restrict__ ids_, int S, int E, int used_bins,
                                                         int nblk, int bs, int* __restrict__ sorted,
                                                         int* __restrict__ bexp, int* __restrict__ npost) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  __shared__ int cnt[ALIGN_MAX_E], end_[ALIGN_MAX_E], wsum[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto id_of = [&](int i) {
    long long v = IDS64 ? reinterpret_cast<const long long*>(ids_)[i] : (long long)reinterpret_cast<const int*>(ids_)[i];
    return (int)(v < 0 ? 0 : (v >= E ? E - 1 : v));
  };
  for (int e = tid; e < E; e += 1024) cnt[e] = 0;
  for (int i = tid; i < nblk * bs; i += 1024) sorted[i] = S;               // padding value
  __syncthreads();
  for (int i = tid; i < S; i += 1024) atomicAdd(&cnt[id_of(i)], 1);
  __syncthreads();
  // inclusive prefix sum of the padded counts: thread e < E (E <= 1024), warp scans + a scan of the warp totals
  int room = tid < E ? (cnt[tid] + bs - 1) / bs * bs : 0;
  int v = room;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(st::FULL, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = wsum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(st::FULL, w, o);
      if (lane >= o) w += n;
    }
    wsum[lane] = w;
  }
  __syncthreads();
  if (tid < E) end_[tid] = v + (warp ? wsum[warp - 1] : 0);
  __syncthreads();
  // placement: warp w takes experts w, w + 32, ...; pairs in original order (ballot prefix inside each 32-pair chunk)
  for (int e = warp; e < E; e += 32) {
    if (cnt[e] == 0) continue;
    int at = end_[e] - (cnt[e] + bs - 1) / bs * bs;
    for (int base = 0; base < S; base += 32) {
      const int i = base + lane;
      const bool hit = i < S && id_of(i) == e;
      const unsigned m = __ballot_sync(st::FULL, hit);
      if (hit) sorted[at + __popc(m & ((1u << lane) - 1u))] = i;
      at += __popc(m);
    }
  }
  // expert of every block: first expert whose end lies beyond the block's first slot (clamped for the unused tail)
  for (int b = tid; b < nblk; b += 1024) {
    const int slot = b * bs;
    int lo = 0, hi = E;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (end_[mid] <= slot) lo = mid + 1; else hi = mid;
    }
    bexp[b] = lo < E ? lo : E - 1;
  }
  if (tid == 0) npost[0] = end_[used_bins - 1];                            // entries of the first used_bins experts
}

// Xg[i, :] = X[sorted[i] / xdiv, :] for the used entries of sorted (padding entries are skipped: their columns of the
// grouped product are never stored).  One warp per row, 16-byte vectors.
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint4* __restrict__ X, const int* __restrict__ sorted,
                                                         const int* __restrict__ npost, int S, int xdiv, int n16,
                                                         long long rows, uint4* __restrict__ Xg) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows || r >= npost[0]) return;
  const int src = sorted[r];
  if (src < 0 || src >= S) return;
  const uint4* in = X + (size_t)(src / xdiv) * n16;
  uint4* out = Xg + (size_t)r * n16;
  for (int c = threadIdx.x & 31; c < n16; c += 32) out[c] = in[c];
}
}  // namespace

extern "C" int st_moe_align(const void* ids, int ids64, int64_t S, int64_t E, int64_t used_bins, int64_t bs,
                            int32_t* sorted, int32_t* bexp, int32_t* npost, int64_t nblk, void* stream) {
  ST_REQUIRE(S >= 1 && S <= (1 << 20) && E >= 1 && E <= ALIGN_MAX_E, "st_moe_align: 1..%d experts, up to 2^20 pairs",
             ALIGN_MAX_E);
  ST_REQUIRE(bs >= 1 && bs <= 1024, "st_moe_align: block size in [1, 1024]");
  ST_REQUIRE(nblk >= S / bs + (S < E ? S : E) && nblk * bs < (1ll << 31),
             "st_moe_align: nblk must cover S / bs + min(S, E) blocks");
  ST_REQUIRE(used_bins >= 1 && used_bins <= E, "st_moe_align: used_bins must be in [1, E]");
  ST_REQUIRE(ids && sorted && bexp && npost, "st_moe_align: null pointer");
  return st::launch("st_moe_align launch", ids64 ? moe_align_kernel<true> : moe_align_kernel<false>, dim3(1), dim3(1024), 0,
                    (cudaStream_t)stream, ids, (int)S, (int)E, (int)used_bins, (int)nblk, (int)bs, (int*)sorted, (int*)bexp,
                    (int*)npost);
}

extern "C" int st_moe_gather(const void* X, const int32_t* sorted, const int32_t* npost, int64_t rows, int64_t S,
                             int64_t xdiv, int64_t N, void* Xg, void* stream) {
  ST_REQUIRE(rows >= 0 && S >= 0 && xdiv >= 1 && N > 0 && N % 8 == 0, "st_moe_gather: sizes (N %% 8 == 0)");
  if (rows == 0 || S == 0) return 0;
  ST_REQUIRE(X && sorted && npost && Xg && st::aligned16(X) && st::aligned16(Xg), "st_moe_gather: null or unaligned pointer");
  return st::launch("st_moe_gather launch", moe_gather_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0,
                    (cudaStream_t)stream, (const uint4*)X, sorted, npost, (int)S, (int)xdiv, (int)(N / 8), (long long)rows,
                    (uint4*)Xg);
}

// Router of a mixture-of-experts layer for a decode step: softmax over the E expert logits of a token, the K largest
// probabilities (ties: the lower expert first) and, optionally, their renormalisation to sum 1, in one launch of one
// warp per token (PyTorch takes five).  expert_map (optional, int32 [E]) turns the ids into this rank's local ids;
// a pair routed to another rank's expert gets id 0 and weight 0 (it then contributes nothing).
__global__ void __launch_bounds__(128) moe_route_kernel(const void* logits, int f32, int T, int E, int K, int renorm,
                                                        const int* expert_map, int* ids, float* w) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  const int lane = threadIdx.x & 31, t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  constexpr int PER = 32;                                            // E <= 1024
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    float x = -INFINITY;
    if (e < E)
      x = f32 ? reinterpret_cast<const float*>(logits)[(size_t)t * E + e]
              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[(size_t)t * E + e]);
    v[i] = x;
    mx = fmaxf(mx, x);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(st::FULL, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : -1.f;          // (-1 marks "no expert" and "already taken")
    sum += fmaxf(v[i], 0.f);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(st::FULL, sum, o);
  const float inv = 1.f / sum;
  float mine_w = 0.f;                                                // lane k keeps the k-th pick
  int mine_e = 0;
  float tot = 0.f;
  for (int k = 0; k < K; ++k) {
    float best = -1.f;
    int be = 0x7FFFFFFF;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (v[i] > best) { best = v[i]; be = i * 32 + lane; }         // ascending e per lane: ties keep the lower expert
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(st::FULL, best, o);
      const int oe = __shfl_xor_sync(st::FULL, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if ((be & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == (be >> 5)) v[i] = -1.f;
    }
    const float p = best * inv;
    tot += p;
    if (lane == k) { mine_w = p; mine_e = be; }
  }
  if (lane < K) {
    float p = renorm ? mine_w / tot : mine_w;
    int e = mine_e;
    if (expert_map != nullptr) {
      const int local = expert_map[e];
      if (local < 0) { e = 0; p = 0.f; } else { e = local; }
    }
    ids[(size_t)t * K + lane] = e;
    w[(size_t)t * K + lane] = p;
  }
}

extern "C" int st_moe_route(const void* logits, int logits_f32, int64_t T, int64_t E, int64_t K, int renorm,
                            const int32_t* expert_map, int32_t* ids, float* w, void* stream) {
  ST_REQUIRE(T >= 0 && E >= 1 && E <= 1024 && K >= 1 && K <= 32 && K <= E,
             "st_moe_route: 1..1024 experts, 1..32 picks per token (got E = %lld, K = %lld)", (long long)E, (long long)K);
  if (T == 0) return 0;
  ST_REQUIRE(logits && ids && w, "st_moe_route: null pointer");
  return st::launch("st_moe_route launch", moe_route_kernel, dim3((unsigned)((T + 3) / 4)), dim3(128), 0,
                    (cudaStream_t)stream, logits, logits_f32, (int)T, (int)E, (int)K, renorm, (const int*)expert_map,
                    (int*)ids, w);
}

extern "C" int st_wsum(const void* Y, const void* w, int w_bf16, void* out, int64_t T, int64_t K, int64_t H,
                       void* stream) {
  ST_REQUIRE(T >= 0 && K >= 1 && H > 0 && H % 8 == 0, "st_wsum: H must be a multiple of 8, K >= 1");
  if (T == 0) return 0;
  ST_REQUIRE(Y && w && out && st::aligned16(Y) && st::aligned16(out), "st_wsum: null or unaligned pointer");
  const long long n = T * (H / 8);
  const unsigned grid = (unsigned)((n + 255) / 256);
  return st::launch("st_wsum launch", w_bf16 ? wsum_kernel<true> : wsum_kernel<false>, dim3(grid), dim3(256), 0,
                    (cudaStream_t)stream, (const uint4*)Y, w, (uint4*)out, (long long)T, (int)K, (int)(H / 8));
}

extern "C" int st_silu_mul(const void* gu, void* act, int64_t S, int64_t I, void* stream) {
  ST_REQUIRE(S >= 0 && I > 0, "st_silu_mul: sizes");
  if (S == 0) return 0;
  ST_REQUIRE(gu && act, "st_silu_mul: null pointer");
  if (I % 8 == 0 && S <= 65535 && st::aligned16(gu) && st::aligned16(act))
    return st::launch("st_silu_mul launch", silu_mul_vec_kernel, dim3((unsigned)((I / 8 + 255) / 256), (unsigned)S),
                      dim3(256), 0, (cudaStream_t)stream, (const uint4*)gu, (uint4*)act, (int)(I / 8));
  const long long n = S * I;
  return st::launch("st_silu_mul launch", silu_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                    (cudaStream_t)stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, (long long)S, (long long)I);
}
