// tree -> dense BF16 (st_dec) and row gather (st_rows): one warp per record, fragments transposed through shared
// memory so that every row leaves as full 128-byte lines.
#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
using namespace st;

__device__ __forceinline__ void apply_list(uint32_t (&A)[4][4], const uint32_t* el, int lo, int hi, int lane) {
  for (int base = lo; base < hi; base += 32) {
    const int n = min(32, hi - base);
    const uint32_t mine = (lane < n) ? __ldg(el + base + lane) : 0u;
    for (int i = 0; i < n; ++i) patch_entry(A, __shfl_sync(FULL, mine, i), lane);
  }
}

// one warp per record; block = 8 warps; each warp owns a 16 x 64 bf16 staging tile (row stride 144 B: conflict-free
// 4-byte fragment stores and 16-byte row reads)
__global__ void __launch_bounds__(256) dec_kernel(const uint8_t* __restrict__ tree, const int* __restrict__ eo,
                                                  const uint32_t* __restrict__ el, long long nrec, int NG, int N,
                                                  __nv_bfloat16* __restrict__ W) {
  __shared__ __align__(16) uint8_t tile[8][16 * 144];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const long long r = (long long)blockIdx.x * 8 + warp;
  if (r >= nrec) return;
  const long long T = r / NG;
  const int G = (int)(r % NG);
  uint32_t A[4][4];
  decode_frag(load_rec_global(tree + r * REC, lane), A);
  const int lo = __ldg(eo + r), hi = __ldg(eo + r + 1);
  if (lo < hi) apply_list(A, el, lo, hi, lane);
  uint8_t* my = tile[warp];
#pragma unroll
  for (int s = 0; s < 4; ++s)
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<uint32_t*>(my + (g + 8 * (q & 1)) * 144 + (16 * s + 8 * (q >> 1) + 2 * t) * 2) = A[s][q];
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 4 * i + (lane >> 3), seg = lane & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(my + row * 144 + seg * 16);
    *reinterpret_cast<uint4*>(W + (T * 16 + row) * (long long)N + G * 64 + seg * 8) = v;
  }
}

// one warp per (id, column group): decodes the record that holds the row and writes its 64 values
__global__ void __launch_bounds__(256) rows_kernel(const uint8_t* __restrict__ tree, const int* __restrict__ eo,
                                                   const uint32_t* __restrict__ el, const long long* __restrict__ ids,
                                                   long long n, int NG, int N, long long M,
                                                   __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= n * NG) return;
  const long long i = w / NG;
  const int G = (int)(w % NG);
  long long id = ids[i];
  const bool valid = id >= 0 && id < M;
  id = valid ? id : 0;
  const long long r = (id >> 4) * NG + G;
  const int row = (int)(id & 15);
  uint32_t A[4][4];
  decode_frag(load_rec_global(tree + r * REC, lane), A);
  const int lo = __ldg(eo + r), hi = __ldg(eo + r + 1);
  if (lo < hi) apply_list(A, el, lo, hi, lane);
  if (g == (row & 7)) {
    uint32_t* o = reinterpret_cast<uint32_t*>(out + i * (long long)N + G * 64);
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int hi2 = 0; hi2 < 2; ++hi2) {
        const uint32_t v = (row >> 3) ? A[s][1 + 2 * hi2] : A[s][2 * hi2];
        o[(16 * s + 8 * hi2 + 2 * t) >> 1] = valid ? v : 0u;
      }
  }
}
}  // namespace

extern "C" int st_dec(const void* tree, const int32_t* eo, const uint32_t* el, int64_t M, int64_t N, void* W,
                      void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 16 == 0 && N % 64 == 0, "st_dec: M %% 16 and N %% 64 must be 0 (got %lld x %lld)",
             (long long)M, (long long)N);
  ST_REQUIRE(tree && eo && el && W, "st_dec: null pointer");
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(W), "st_dec: tree and W must be 16-byte aligned");
  const long long nrec = (M / 16) * (N / 64);
  ST_REQUIRE(nrec < (1ll << 31), "st_dec: too many records");
  dec_kernel<<<(unsigned)((nrec + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)tree, eo, el, nrec, (int)(N / 64), (int)N, (__nv_bfloat16*)W);
  ST_LAUNCH_CHECK("st_dec launch");
  return 0;
}

extern "C" int st_rows(const void* tree, const int32_t* eo, const uint32_t* el, int64_t M, int64_t N,
                       const int64_t* ids, int64_t n, void* out, void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 16 == 0 && N % 64 == 0, "st_rows: M %% 16 and N %% 64 must be 0");
  ST_REQUIRE(n >= 0, "st_rows: negative count");
  if (n == 0) return 0;
  ST_REQUIRE(tree && eo && el && ids && out, "st_rows: null pointer");
  ST_REQUIRE(st::aligned16(tree) && ((uintptr_t)out & 3u) == 0, "st_rows: alignment");
  const long long nw = n * (N / 64);
  ST_REQUIRE(nw < (1ll << 34), "st_rows: too many rows");
  rows_kernel<<<(unsigned)((nw + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)tree, eo, el, (const long long*)ids, n, (int)(N / 64), (int)N, M, (__nv_bfloat16*)out);
  ST_LAUNCH_CHECK("st_rows launch");
  return 0;
}
