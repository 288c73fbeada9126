// Small fused glue kernels of the decode step (between the tree-stored linears and the KV kernels): residual add +
// RMSNorm, and per-head q/k RMSNorm + rotary embedding.  BF16 in and out, fp32 arithmetic.  They keep a decode step at
// about ten launches per layer; the reference's measurement harness (statetree/bench.py:74-99) leaves this work to
// PyTorch element-wise kernels.
#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(st::FULL, v, o);
  return v;
}

// one CTA (256 threads) per row: x += delta (optional, written back), out = x * rsqrt(mean(x^2) + eps) * w.
// Any even width; the row is read twice.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ delta,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ out, int cols, float eps) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  __shared__ float part[8];
  const size_t base = (size_t)blockIdx.x * cols;
  float ss = 0.f;
  for (int c = threadIdx.x * 2; c < cols; c += 512) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + base + c));
    if (delta) {
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(delta + base + c));
      const __nv_bfloat162 s = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);      // the residual stream stays BF16
      *reinterpret_cast<__nv_bfloat162*>(x + base + c) = s;
      v = __bfloat1622float2(s);
    }
    ss += v.x * v.x + v.y * v.y;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += part[i];
  const float r = rsqrtf(tot / (float)cols + eps);
  for (int c = threadIdx.x * 2; c < cols; c += 512) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + base + c));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + c));
    const __nv_bfloat162 n = __floats2bfloat162_rn(v.x * r, v.y * r);           // normalised value rounded, then scaled
    const float2 nf = __bfloat1622float2(n);
    *reinterpret_cast<__nv_bfloat162*>(out + base + c) = __floats2bfloat162_rn(nf.x * g.x, nf.y * g.y);
  }
}

// The same for rows of up to K * 4096 columns (a multiple of 8, 16-byte aligned): 512 threads, eight values per thread
// and pass, every operand requested up front with 16-byte loads and the row kept in registers, so the kernel is one
// round trip to memory, one block reduction and the stores (a decode step runs it twice per layer on a single row).
template <int K>
__global__ void __launch_bounds__(512) add_rmsnorm_vec_kernel(__nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ delta,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              __nv_bfloat16* __restrict__ out, int cols, float eps) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  __shared__ float part[16];
  const size_t base = (size_t)blockIdx.x * cols;
  uint4 xv[K], dv[K], wv[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = (threadIdx.x + k * 512) * 8;
    if (c < cols) {
      xv[k] = *reinterpret_cast<const uint4*>(x + base + c);
      if (delta) dv[k] = *reinterpret_cast<const uint4*>(delta + base + c);
      wv[k] = *reinterpret_cast<const uint4*>(w + c);
    }
  }
  float f[K][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = (threadIdx.x + k * 512) * 8;
    if (c < cols) {
      const uint32_t xs[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
      const uint32_t ds[4] = {dv[k].x, dv[k].y, dv[k].z, dv[k].w};
      uint32_t so[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xs[j]));
        if (delta) {
          const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ds[j]));
          const __nv_bfloat162 s = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);  // the residual stream stays BF16
          so[j] = *reinterpret_cast<const uint32_t*>(&s);
          v = __bfloat1622float2(s);
        }
        f[k][2 * j] = v.x;
        f[k][2 * j + 1] = v.y;
        ss += v.x * v.x + v.y * v.y;
      }
      if (delta) *reinterpret_cast<uint4*>(x + base + c) = make_uint4(so[0], so[1], so[2], so[3]);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) tot += part[i];
  const float r = rsqrtf(tot / (float)cols + eps);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = (threadIdx.x + k * 512) * 8;
    if (c < cols) {
      const uint32_t ws[4] = {wv[k].x, wv[k].y, wv[k].z, wv[k].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ws[j]));
        const float2 nf = __bfloat1622float2(__floats2bfloat162_rn(f[k][2 * j] * r, f[k][2 * j + 1] * r));
        const __nv_bfloat162 y = __floats2bfloat162_rn(nf.x * g.x, nf.y * g.y);  // normalised value rounded, then scaled
        o[j] = *reinterpret_cast<const uint32_t*>(&y);
      }
      *reinterpret_cast<uint4*>(out + base + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// one warp per (token, head) of q and k inside a fused qkv row: RMSNorm over the 128 dims, then rotary embedding of
// interleaved pairs (2i, 2i+1) with the angle table row of the step's position (a device scalar: graph-safe)
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride,
                                                           const __nv_bfloat16* __restrict__ wq,
                                                           const __nv_bfloat16* __restrict__ wk,
                                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                           const long long* __restrict__ pos, long long max_pos,
                                                           __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                                                           int B, int hq, int hkv, float eps) {
  st::pdl_wait();
  st::pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int heads = hq + hkv;
  if (wid >= (long long)B * heads) return;
  const int b = (int)(wid / heads), h = (int)(wid % heads);
  const bool is_k = h >= hq;
  const __nv_bfloat16* src = qkv + (size_t)b * row_stride + (size_t)h * 128 + 4 * lane;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  const float ss = warp_sum(st::sumsq4(a.x, a.y, c.x, c.y));
  const float r = rsqrtf(__fmaf_rn(ss, 1.f / 128.f, eps));
  const __nv_bfloat16* w = (is_k ? wk : wq) + 4 * lane;
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + 2));
  // normalised values rounded to BF16 as a separate norm layer would, then rotated in fp32
  const float2 n0 = __bfloat1622float2(__floats2bfloat162_rn(
      __bfloat162float(__float2bfloat16_rn(a.x * r)) * g0.x, __bfloat162float(__float2bfloat16_rn(a.y * r)) * g0.y));
  const float2 n1 = __bfloat1622float2(__floats2bfloat162_rn(
      __bfloat162float(__float2bfloat16_rn(c.x * r)) * g1.x, __bfloat162float(__float2bfloat16_rn(c.y * r)) * g1.y));
  long long p = pos[0];
  p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
  const float c0 = cos_t[p * 64 + 2 * lane], s0 = sin_t[p * 64 + 2 * lane];
  const float c1 = cos_t[p * 64 + 2 * lane + 1], s1 = sin_t[p * 64 + 2 * lane + 1];
  uint2 o;
  o.x = st::rope_pair(n0.x, n0.y, c0, s0);
  o.y = st::rope_pair(n1.x, n1.y, c1, s1);
  __nv_bfloat16* dst = is_k ? k_out + ((size_t)b * hkv + (h - hq)) * 128 : q_out + ((size_t)b * hq + h) * 128;
  *reinterpret_cast<uint2*>(dst + 4 * lane) = o;
}
}  // namespace

extern "C" int st_add_rmsnorm(void* x, const void* delta, const void* w, void* out, int64_t rows, int64_t cols, double eps,
                              void* stream) {
  ST_REQUIRE(rows >= 0 && cols > 0 && cols % 2 == 0, "st_add_rmsnorm: cols must be even");
  if (rows == 0) return 0;
  ST_REQUIRE(x && w && out, "st_add_rmsnorm: null pointer");
  ST_REQUIRE(((uintptr_t)x & 3u) == 0 && ((uintptr_t)out & 3u) == 0 && ((uintptr_t)w & 3u) == 0 &&
             (!delta || ((uintptr_t)delta & 3u) == 0), "st_add_rmsnorm: pointers must be 4-byte aligned");
  const bool vec = cols % 8 == 0 && cols <= 8192 && st::aligned16(x) && st::aligned16(out) && st::aligned16(w) &&
                   (!delta || st::aligned16(delta));
  auto* kern = !vec ? add_rmsnorm_kernel : (cols <= 4096 ? add_rmsnorm_vec_kernel<1> : add_rmsnorm_vec_kernel<2>);
  return st::launch("st_add_rmsnorm launch", kern, dim3((unsigned)rows), dim3(vec ? 512 : 256), 0, (cudaStream_t)stream,
                    (__nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w, (__nv_bfloat16*)out,
                    (int)cols, (float)eps);
}

extern "C" int st_qk_norm_rope(const void* qkv, int64_t row_stride, const void* wq, const void* wk, const float* cos_t,
                               const float* sin_t, const int64_t* pos, int64_t max_pos, void* q_out, void* k_out, int64_t B,
                               int64_t hq, int64_t hkv, double eps, void* stream) {
  ST_REQUIRE(B >= 0 && hq > 0 && hkv > 0 && max_pos > 0, "st_qk_norm_rope: sizes");
  if (B == 0) return 0;
  ST_REQUIRE(qkv && wq && wk && cos_t && sin_t && pos && q_out && k_out, "st_qk_norm_rope: null pointer");
  ST_REQUIRE(((uintptr_t)qkv & 7u) == 0 && row_stride % 4 == 0 && ((uintptr_t)q_out & 7u) == 0 && ((uintptr_t)k_out & 7u) == 0,
             "st_qk_norm_rope: 8-byte alignment");
  const long long warps = B * (hq + hkv);
  return st::launch("st_qk_norm_rope launch", qk_norm_rope_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0,
                    (cudaStream_t)stream, (const __nv_bfloat16*)qkv, (long long)row_stride, (const __nv_bfloat16*)wq,
                    (const __nv_bfloat16*)wk, cos_t, sin_t, (const long long*)pos, (long long)max_pos,
                    (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, (int)B, (int)hq, (int)hkv, (float)eps);
}
