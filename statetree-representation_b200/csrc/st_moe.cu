// Element-wise companions of the expert products: routing-weighted sum and the SwiGLU gate.
#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
// out[t, h0..h0+7] = sum_j w[t, j] * Y[t * K + j, h0..h0+7]: fp32, experts in order j = 0..K-1, BF16 round at the end
template <bool WBF16>
__global__ void __launch_bounds__(256) wsum_kernel(const uint4* __restrict__ Y, const void* __restrict__ w,
                                                   uint4* __restrict__ out, long long T, int K, int H8) {
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
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ gu,
                                                       __nv_bfloat16* __restrict__ act, long long S, long long I) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= S * I) return;
  const long long s = i / I, c = i % I;
  const float gte = __bfloat162float(gu[s * 2 * I + c]);
  const __nv_bfloat16 sg = __float2bfloat16_rn(gte / (1.f + __expf(-gte)));
  act[i] = __hmul(sg, gu[s * 2 * I + I + c]);
}
}  // namespace

extern "C" int st_wsum(const void* Y, const void* w, int w_bf16, void* out, int64_t T, int64_t K, int64_t H,
                       void* stream) {
  ST_REQUIRE(T >= 0 && K >= 1 && H > 0 && H % 8 == 0, "st_wsum: H must be a multiple of 8, K >= 1");
  if (T == 0) return 0;
  ST_REQUIRE(Y && w && out && st::aligned16(Y) && st::aligned16(out), "st_wsum: null or unaligned pointer");
  const long long n = T * (H / 8);
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (w_bf16)
    wsum_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)Y, w, (uint4*)out, T, (int)K, (int)(H / 8));
  else
    wsum_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)Y, w, (uint4*)out, T, (int)K, (int)(H / 8));
  ST_LAUNCH_CHECK("st_wsum launch");
  return 0;
}

extern "C" int st_silu_mul(const void* gu, void* act, int64_t S, int64_t I, void* stream) {
  ST_REQUIRE(S >= 0 && I > 0, "st_silu_mul: sizes");
  if (S == 0) return 0;
  ST_REQUIRE(gu && act, "st_silu_mul: null pointer");
  const long long n = S * I;
  silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, S, I);
  ST_LAUNCH_CHECK("st_silu_mul launch");
  return 0;
}
