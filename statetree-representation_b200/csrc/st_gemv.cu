// Small-batch fused tree-decode GEMV for sm_100a: Y[B, M] = X[B, N] W[M, N]^T, B <= 32, W stored as state-tree records.
//
// The record stream is consumed in MEMORY ORDER.  Work unit = up to 8 consecutive records of one 16-row tile
// (12 416 B); the U units of the (virtual) matrix are cut into one contiguous range per CTA, so every CTA streams one
// contiguous span of HBM.  A producer warp moves each unit into a ring of shared-memory stages with 1-D bulk copies
// (TMA, mbarrier byte counting, L2 evict-first): the records, the unit's 64-byte escape block, and the matching
// 512-column slice of every activation row.  Eight consumer warps each take one record of the unit: three 128-bit
// shared loads per lane give the lane's fragment of the record, five integer ops per four weights decode it into the
// mma.m16n8k16 A fragment, escapes are patched in registers, and the activations come in as B fragments by ldmatrix.
// Accumulators stay in registers across the units of a tile; at the end of a tile the eight warps are summed in warp
// order in shared memory.  A tile whose units span several CTAs is finished by the last CTA to arrive, which adds
// the partial sums in CTA order, so results are bit-identical from run to run.
//
// The same kernel serves the mixture-of-experts products: MODE 1 makes every (token, expert) slot its own problem
// with one activation row; MODE 2 makes every block of 8 slots of one expert (moe_align_block_size layout) a problem.
#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
using namespace st;

constexpr int CW = 8;                     // consumer warps = records per unit
constexpr int UNIT_BYTES = CW * REC;      // 12416
constexpr int SIDE_BYTES = 64;            // escape block of a unit
constexpr int XROW = CW * 128 + 16;       // bytes per staged activation row (512 columns + pad: conflict-free ldmatrix)
constexpr int MODE_DENSE = 0, MODE_SLOT = 1, MODE_GROUP = 2;

struct GemvArgs {
  // dense: one matrix; MoE: per-expert device address tables
  const uint8_t* tree; const int* eo; const uint32_t* eb; const uint32_t* el;
  const long long* tp; const long long* eop; const long long* ebp; const long long* elp;
  const uint16_t* X; uint16_t* Y; float* Yf;
  float* ws; int* cnt; int* status;
  const void* ids; int ids64;             // MODE_SLOT: expert of each slot
  const int* sorted; const int* bexp; const int* npost;   // MODE_GROUP
  long long M, N;
  int B;                                  // activation rows (dense) / slots S (MoE)
  int E, xdiv;
  int NG, CPT, T;                         // column groups, units per tile, tiles per problem
  long long U;                            // units over all problems
  int nprob, maxcover, stages;
};

struct Prob {                             // what a unit's problem resolves to
  const uint8_t* tree; const int* eo; const uint32_t* eb; const uint32_t* el;
  bool skip;
};

template <int MODE>
__device__ __forceinline__ Prob resolve(const GemvArgs& a, int p) {
  Prob r;
  r.skip = false;
  if (MODE == MODE_DENSE) {
    r.tree = a.tree; r.eo = a.eo; r.eb = a.eb; r.el = a.el;
    return r;
  }
  long long e;
  if (MODE == MODE_SLOT) {
    e = a.ids64 ? ((const long long*)a.ids)[p] : (long long)((const int*)a.ids)[p];
    e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
  } else {
    e = a.bexp[p];
    r.skip = e < 0 || e >= a.E || p * 8 >= a.npost[0];
    if (r.skip) e = 0;
  }
  r.tree = reinterpret_cast<const uint8_t*>(a.tp[e]);
  r.eo = reinterpret_cast<const int*>(a.eop[e]);
  r.eb = reinterpret_cast<const uint32_t*>(a.ebp[e]);
  r.el = reinterpret_cast<const uint32_t*>(a.elp[e]);
  return r;
}

// activation row / output row of column n of problem p; -1 = unused column
template <int MODE>
__device__ __forceinline__ long long out_row(const GemvArgs& a, int p, int n) {
  if (MODE == MODE_DENSE) return n < a.B ? n : -1;
  if (MODE == MODE_SLOT) return n == 0 ? p : -1;
  const int s = a.sorted[p * 8 + n];
  return (n < 8 && s >= 0 && s < a.B) ? s : -1;
}

__device__ __forceinline__ int cta_of_unit(long long u, long long U, int C) { return (int)(((u + 1) * C - 1) / U); }

template <int NT, int MODE>
__global__ void __launch_bounds__((CW + 1) * 32, 1) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int NB = 8 * NT;                                   // activation columns of the mma
  constexpr int STAGE = UNIT_BYTES + SIDE_BYTES + NB * XROW;   // bytes per ring stage
  constexpr int EL = 16 * NB;                                  // outputs of one tile
  const int S = a.stages;
  uint8_t* ring = smem;
  float* red = reinterpret_cast<float*>(smem + (size_t)S * STAGE);          // [CW][EL]
  float* tot = red + CW * EL;                                               // [EL]
  uint64_t* full = reinterpret_cast<uint64_t*>(tot + EL);
  uint64_t* empty = full + S;
  int* s_last = reinterpret_cast<int*>(empty + S);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = gridDim.x;
  const long long u0 = (long long)blockIdx.x * a.U / C, u1 = (long long)(blockIdx.x + 1) * a.U / C;
  const int UPP = a.T * a.CPT;                                 // units per problem

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, CW); }
    fence_barrier_init();
  }
  // activation rows that no copy ever fills must not hold NaN patterns
  for (int i = tid; i < S * NB * (XROW / 16); i += blockDim.x) {
    const int s = i / (NB * (XROW / 16)), j = i % (NB * (XROW / 16));
    reinterpret_cast<uint4*>(ring + (size_t)s * STAGE + UNIT_BYTES + SIDE_BYTES)[j] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();
  __syncthreads();

  if (warp == CW) {
    // ------------------------------------------------------------------ producer: one elected lane drives the ring
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      long long it = 0;
      for (long long u = u0; u < u1; ++u) {
        const int p = (int)(u / UPP), ul = (int)(u % UPP);
        const Prob pr = resolve<MODE>(a, p);
        if (pr.skip) continue;
        const int tile = ul / a.CPT, c = ul % a.CPT;
        const int nrec = min(CW, a.NG - c * CW);
        const int s = (int)(it % S);
        const long long k = it / S;
        if (k > 0 && !mbar_wait(empty + s, (uint32_t)(k - 1) & 1u)) { atomicExch(a.status, ERR_WAIT_EMPTY); break; }
        uint8_t* st = ring + (size_t)s * STAGE;
        int nx = 0;
        long long rows[NB];
#pragma unroll
        for (int n = 0; n < NB; ++n) {
          const long long r = out_row<MODE>(a, p, n);
          rows[n] = r < 0 ? -1 : (MODE == MODE_DENSE ? r : r / a.xdiv);
          nx += r >= 0;
        }
        mbar_expect_tx(full + s, (uint32_t)(nrec * REC + SIDE_BYTES + nx * nrec * 128));
        bulk_g2s(st, pr.tree + ((size_t)tile * a.NG + (size_t)c * CW) * REC, (uint32_t)(nrec * REC), full + s, pol_w);
        bulk_g2s(st + UNIT_BYTES, pr.eb + ((size_t)tile * a.CPT + c) * 16, SIDE_BYTES, full + s, pol_w);
#pragma unroll
        for (int n = 0; n < NB; ++n)
          if (rows[n] >= 0)
            bulk_g2s(st + UNIT_BYTES + SIDE_BYTES + n * XROW, a.X + rows[n] * a.N + (size_t)c * CW * 64,
                     (uint32_t)(nrec * 128), full + s, pol_x);
        ++it;
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int g = lane >> 2;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  long long it = 0;
  for (long long u = u0; u < u1; ++u) {
    const int p = (int)(u / UPP), ul = (int)(u % UPP);
    const Prob pr = resolve<MODE>(a, p);
    if (pr.skip) continue;
    const int tile = ul / a.CPT, c = ul % a.CPT;
    const int nrec = min(CW, a.NG - c * CW);
    const int s = (int)(it % S);
    if (!mbar_wait(full + s, (uint32_t)(it / S) & 1u)) {
      if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
      return;
    }
    ++it;
    const uint8_t* st = ring + (size_t)s * STAGE;
    if (warp < nrec) {
      uint32_t A[4][4];
      decode_frag(load_rec_shared(st + warp * REC, lane), A);
      const uint32_t* side = reinterpret_cast<const uint32_t*>(st + UNIT_BYTES);
      const uint32_t ne = side[0];
      if (ne) {
        if (ne <= 14u) {
          for (uint32_t i = 0; i < ne; ++i) {
            const uint32_t e = side[2 + i];
            if (((e >> 10) & 7u) == (uint32_t)warp) patch_entry(A, e, lane);
          }
        } else {                                               // crowded unit: this record's own list
          const size_t r = (size_t)tile * a.NG + (size_t)c * CW + warp;
          const int lo = __ldg(pr.eo + r), hi = __ldg(pr.eo + r + 1);
          for (int base = lo; base < hi; base += 32) {
            const int n = min(32, hi - base);
            const uint32_t mine = (lane < n) ? __ldg(pr.el + base + lane) : 0u;
            for (int i = 0; i < n; ++i) patch_entry(A, __shfl_sync(FULL, mine, i), lane);
          }
        }
      }
      const uint32_t xs = smem_addr(st + UNIT_BYTES + SIDE_BYTES) + (uint32_t)((lane & 7) * XROW + warp * 128 + (lane >> 3) * 16);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        uint32_t b[8];
        ldmatrix_x4(xs + nt * 8 * XROW, b[0], b[1], b[2], b[3]);
        ldmatrix_x4(xs + nt * 8 * XROW + 64, b[4], b[5], b[6], b[7]);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_bf16(acc[nt], A[ks], b[2 * ks], b[2 * ks + 1]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);

    // ---- end of this CTA's share of the tile: reduce the warps, then store or hand over a partial sum
    const bool tile_end = (c == a.CPT - 1) || (u + 1 == u1);
    if (!tile_end) continue;
    float* mine = red + warp * EL;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int n0 = nt * 8 + 2 * (lane & 3);
      mine[n0 * 16 + g] = acc[nt][0];
      mine[(n0 + 1) * 16 + g] = acc[nt][1];
      mine[n0 * 16 + g + 8] = acc[nt][2];
      mine[(n0 + 1) * 16 + g + 8] = acc[nt][3];
      acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    }
    named_bar_sync(1, CW * 32);
    const long long tbase = (long long)p * UPP + (long long)tile * a.CPT;      // first unit of the tile
    const int cfirst = cta_of_unit(tbase, a.U, C), clast = cta_of_unit(tbase + a.CPT - 1, a.U, C);
    const int ncover = clast - cfirst + 1;
    const long long tg = (long long)p * a.T + tile;
    for (int idx = tid; idx < EL; idx += CW * 32) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < CW; ++w) sum += red[w * EL + idx];
      if (ncover == 1) tot[idx] = sum;
      else a.ws[((size_t)tg * a.maxcover + (blockIdx.x - cfirst)) * EL + idx] = sum;
    }
    bool finish = ncover == 1;
    if (ncover > 1) {
      __threadfence();
      named_bar_sync(1, CW * 32);
      if (tid == 0) *s_last = (atomicAdd(a.cnt + tg, 1) == ncover - 1);
      named_bar_sync(1, CW * 32);
      finish = *s_last != 0;
      if (finish) {
        __threadfence();
        for (int idx = tid; idx < EL; idx += CW * 32) {
          float sum = 0.f;
          for (int k = 0; k < ncover; ++k) sum += __ldcg(a.ws + ((size_t)tg * a.maxcover + k) * EL + idx);
          tot[idx] = sum;
        }
        if (tid == 0) a.cnt[tg] = 0;
      }
    }
    if (finish) {
      for (int idx = tid; idx < EL; idx += CW * 32) {
        const int n = idx >> 4, r = idx & 15;
        const long long row = out_row<MODE>(a, p, n);
        if (row >= 0) {
          const float v = tot[idx];
          const __nv_bfloat16 hv = __float2bfloat16_rn(v);
          a.Y[row * a.M + (size_t)tile * 16 + r] = *reinterpret_cast<const uint16_t*>(&hv);
          if (a.Yf) a.Yf[row * a.M + (size_t)tile * 16 + r] = v;
        }
      }
    }
    named_bar_sync(1, CW * 32);                                  // red / tot / s_last are free again
  }
}

struct Plan { int C, stages, maxcover; size_t smem; long long U; int CPT, T, NG, nprob; };

template <int NT>
Plan make_plan(long long M, long long N, int nprob) {
  Plan p;
  p.NG = (int)(N / 64);
  p.CPT = (p.NG + CW - 1) / CW;
  p.T = (int)(M / 16);
  p.nprob = nprob;
  p.U = (long long)nprob * p.T * p.CPT;
  const int sms = st::sm_count();
  p.C = (int)(p.U < sms ? p.U : sms);
  const long long per = p.U / p.C;
  long long mc = (p.CPT + per - 1) / per + 1;
  if (mc > p.CPT) mc = p.CPT;
  p.maxcover = (int)(mc < 1 ? 1 : mc);
  constexpr int NB = 8 * NT, STAGE = UNIT_BYTES + SIDE_BYTES + NB * XROW, EL = 16 * NB;
  const size_t fixed = (size_t)(CW + 1) * EL * 4 + 2 * 16 * 8 + 16;
  int stages = (int)((200 * 1024 - fixed) / STAGE);
  if (stages > 8) stages = 8;
  p.stages = stages;
  p.smem = (size_t)stages * STAGE + fixed;
  return p;
}

template <int NT, int MODE>
int launch(GemvArgs& a, int nprob, long long ws_bytes, cudaStream_t stream, const char* who) {
  const Plan p = make_plan<NT>(a.M, a.N, nprob);
  a.NG = p.NG; a.CPT = p.CPT; a.T = p.T; a.U = p.U; a.nprob = nprob; a.maxcover = p.maxcover; a.stages = p.stages;
  const long long need = (long long)nprob * p.T * p.maxcover * 16 * 8 * NT * 4;
  ST_REQUIRE(p.maxcover == 1 || (a.ws && ws_bytes >= need), "%s: workspace of %lld bytes needed, %lld given", who, need,
             ws_bytes);
  ST_REQUIRE(p.stages >= 2, "%s: internal: ring does not fit", who);
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "%s: no device status word", who);
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    if (int e = st::cuda_fail(cudaFuncSetAttribute(gemv_kernel<NT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   200 * 1024), who))
      return e;
    set[dev] = true;
  }
  gemv_kernel<NT, MODE><<<p.C, (CW + 1) * 32, p.smem, stream>>>(a);
  ST_LAUNCH_CHECK(who);
  return 0;
}

template <int NT>
long long ws_need(long long M, long long N, int nprob) {
  const Plan p = make_plan<NT>(M, N, nprob);
  return p.maxcover == 1 ? 0 : (long long)nprob * p.T * p.maxcover * 16 * 8 * NT * 4;
}
}  // namespace

extern "C" int64_t st_gemv_workspace_bytes(int64_t M, int64_t N, int64_t B) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || B < 1 || B > 32) return -1;
  return B <= 8 ? ws_need<1>(M, N, 1) : (B <= 16 ? ws_need<2>(M, N, 1) : ws_need<4>(M, N, 1));
}

extern "C" int st_gemv(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X,
                       void* Y, float* Yf32, int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt,
                       void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 16 == 0 && N % 64 == 0, "st_gemv: M %% 16 and N %% 64 must be 0 (got %lld x %lld)",
             (long long)M, (long long)N);
  ST_REQUIRE(B >= 1 && B <= 32, "st_gemv: batch must be in [1, 32] (got %lld)", (long long)B);
  ST_REQUIRE(tree && eo && eb && el && X && Y && cnt, "st_gemv: null pointer");
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(eb) && st::aligned16(X), "st_gemv: tree, eb and X must be 16-byte aligned");
  ST_REQUIRE((M / 16) * ((N / 64 + 7) / 8) < (1ll << 31), "st_gemv: too many units");
  GemvArgs a = {};
  a.tree = (const uint8_t*)tree; a.eo = eo; a.eb = eb; a.el = el;
  a.X = (const uint16_t*)X; a.Y = (uint16_t*)Y; a.Yf = Yf32; a.ws = (float*)ws; a.cnt = cnt;
  a.M = M; a.N = N; a.B = (int)B; a.E = 1; a.xdiv = 1;
  cudaStream_t s = (cudaStream_t)stream;
  if (B <= 8) return launch<1, MODE_DENSE>(a, 1, ws_bytes, s, "st_gemv");
  if (B <= 16) return launch<2, MODE_DENSE>(a, 1, ws_bytes, s, "st_gemv");
  return launch<4, MODE_DENSE>(a, 1, ws_bytes, s, "st_gemv");
}

extern "C" int64_t st_moe_gemv_workspace_bytes(int64_t S, int64_t M, int64_t N) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || S < 1) return -1;
  return ws_need<1>(M, N, (int)S);
}

static int moe_common_checks(const char* who, const int64_t* tp, const int64_t* eop, const int64_t* ebp,
                             const int64_t* elp, int64_t E, const void* X, void* Y, int64_t S, int64_t M, int64_t N,
                             int64_t xdiv, int32_t* cnt) {
  ST_REQUIRE(M > 0 && N > 0 && M % 16 == 0 && N % 64 == 0, "%s: M %% 16 and N %% 64 must be 0", who);
  ST_REQUIRE(E >= 1 && S >= 0 && xdiv >= 1, "%s: E >= 1, S >= 0, xdiv >= 1", who);
  ST_REQUIRE(tp && eop && ebp && elp && X && Y && cnt, "%s: null pointer", who);
  ST_REQUIRE(st::aligned16(X), "%s: X must be 16-byte aligned", who);
  ST_REQUIRE(N % 8 == 0, "%s: N", who);
  return 0;
}

extern "C" int st_moe_gemv(const int64_t* tp, const int64_t* eop, const int64_t* ebp, const int64_t* elp, int64_t E,
                           const void* X, const void* ids, int ids64, void* Y, int64_t S, int64_t M, int64_t N,
                           int64_t xdiv, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream) {
  if (int e = moe_common_checks("st_moe_gemv", tp, eop, ebp, elp, E, X, Y, S, M, N, xdiv, cnt)) return e;
  if (S == 0) return 0;
  ST_REQUIRE(ids != nullptr, "st_moe_gemv: null ids");
  ST_REQUIRE(S * (M / 16) * ((N / 64 + 7) / 8) < (1ll << 31), "st_moe_gemv: too many units");
  GemvArgs a = {};
  a.tp = (const long long*)tp; a.eop = (const long long*)eop; a.ebp = (const long long*)ebp; a.elp = (const long long*)elp;
  a.X = (const uint16_t*)X; a.Y = (uint16_t*)Y; a.ws = (float*)ws; a.cnt = cnt; a.ids = ids; a.ids64 = ids64;
  a.M = M; a.N = N; a.B = (int)S; a.E = (int)E; a.xdiv = (int)xdiv;
  return launch<1, MODE_SLOT>(a, (int)S, ws_bytes, (cudaStream_t)stream, "st_moe_gemv");
}

extern "C" int64_t st_moe_group_workspace_bytes(int64_t nblk, int64_t M, int64_t N) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || nblk < 1) return -1;
  return ws_need<1>(M, N, (int)nblk);
}

extern "C" int st_moe_group_gemv(const int64_t* tp, const int64_t* eop, const int64_t* ebp, const int64_t* elp,
                                 int64_t E, const void* X, const int32_t* sorted, const int32_t* bexp,
                                 const int32_t* npost, int64_t nblk, void* Y, int64_t S, int64_t M, int64_t N,
                                 int64_t xdiv, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream) {
  if (int e = moe_common_checks("st_moe_group_gemv", tp, eop, ebp, elp, E, X, Y, S, M, N, xdiv, cnt)) return e;
  if (S == 0 || nblk == 0) return 0;
  ST_REQUIRE(sorted && bexp && npost, "st_moe_group_gemv: null alignment tables");
  ST_REQUIRE(nblk * (M / 16) * ((N / 64 + 7) / 8) < (1ll << 31), "st_moe_group_gemv: too many units");
  GemvArgs a = {};
  a.tp = (const long long*)tp; a.eop = (const long long*)eop; a.ebp = (const long long*)ebp; a.elp = (const long long*)elp;
  a.X = (const uint16_t*)X; a.Y = (uint16_t*)Y; a.ws = (float*)ws; a.cnt = cnt;
  a.sorted = sorted; a.bexp = bexp; a.npost = npost;
  a.M = M; a.N = N; a.B = (int)S; a.E = (int)E; a.xdiv = (int)xdiv;
  return launch<1, MODE_GROUP>(a, (int)nblk, ws_bytes, (cudaStream_t)stream, "st_moe_group_gemv");
}
