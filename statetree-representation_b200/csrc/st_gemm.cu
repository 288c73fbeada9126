// Large-batch fused tree-decode + GEMM on the 5th-generation tensor cores (tcgen05 / TMEM) of sm_100a.
//   Y[B, M] = X[B, N] W[M, N]^T,  W as state-tree records, fp32 accumulation in tensor memory, BF16 output.
//
// One CTA computes a 128-row block of W against one tile of NT tokens (NT = 64, 128 or 256) over a contiguous range
// of 64-column k-tiles.  Warp roles (10 warps):
//   warp 8   producer: per k-tile, eight 1552-byte bulk copies (the records of the block's eight 16-row tiles) and
//            one tiled TMA load of the activation tile X[tok0 .. tok0+NT, 64 cols] with the 128-byte swizzle
//   warps 0-7 decode: each turns one record into its mma-fragment registers (five integer ops per four weights),
//            patches escapes, and writes the 16 x 64 BF16 sub-tile into the K-major, 128-byte-swizzled A tile with
//            stmatrix; fence.proxy.async hands the tile to the tensor core
//   warp 9   MMA: one elected thread issues four tcgen05.mma (128 x NT x 16, kind::f16) per k-tile, A and B read
//            from shared memory through descriptors, D in TMEM; tcgen05.commit releases the stage
// Epilogue: warps 0-7 read the accumulator with tcgen05.ld (32 lanes x 32 columns per instruction) and either store
// BF16 results or, when the k range is split over several CTAs, store fp32 partials; the last CTA to arrive for a
// tile adds the partials in split order (deterministic) and stores the result.
// Every mbarrier wait is bounded; a wait that runs out sets the device status word and the CTA leaves after
// releasing its tensor memory.
#include <cuda.h>

#include <mutex>

#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
using namespace st;

constexpr int A_TILE = 128 * 128;            // 128 rows x 64 bf16, one swizzle atom wide
constexpr int RAW = 13 * 1024;               // 8 records (12416 B) padded to keep stages 1024-byte aligned
constexpr int NDEC = 8;                      // decode warps = records per k-tile

struct GemmArgs {
  const uint8_t* tree; const int* eo; const uint32_t* el;
  uint16_t* Y; float* Yf; float* ws; int* cnt; int* status;
  long long M, N;
  int B, NG, NT, KS, RB, TT, stages;
  uint32_t idesc;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               :: "r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_addr(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               :: "r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                 "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                 "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__global__ void __launch_bounds__(320, 1) gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int NT = a.NT, S = a.stages;
  const int XT = NT * 128;                       // bytes of an activation tile
  const int STAGE = A_TILE + XT + RAW;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)S * STAGE);
  uint64_t* ready = full + S;
  uint64_t* empty = ready + S;
  uint64_t* accbar = empty + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accbar + 1);
  int* flags = reinterpret_cast<int*>(tmem_slot + 1);        // [0] abort, [1] last arriver

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // unit of this CTA
  const int ks = blockIdx.x % a.KS, rt = blockIdx.x / a.KS;
  const int rb = rt % a.RB, tt = rt / a.RB;
  const int k0 = (int)((long long)a.NG * ks / a.KS), k1 = (int)((long long)a.NG * (ks + 1) / a.KS);
  const int nk = k1 - k0;
  const int tok0 = tt * NT;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(full + s, 1); mbar_init(ready + s, NDEC); mbar_init(empty + s, 1); }
    mbar_init(accbar, 1);
    flags[0] = 0; flags[1] = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, (uint32_t)(NT < 32 ? 32 : NT));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_first();
      for (int i = 0; i < nk; ++i) {
        const int s = i % S, k = i / S;
        if (k > 0 && !mbar_wait(empty + s, (uint32_t)(k - 1) & 1u)) { atomicExch(a.status, ERR_WAIT_EMPTY); break; }
        uint8_t* st = smem + (size_t)s * STAGE;
        mbar_expect_tx(full + s, (uint32_t)(NDEC * REC + XT));
        tma_load_2d(st + A_TILE, &xmap, (k0 + i) * 64, tok0, full + s);
#pragma unroll
        for (int w = 0; w < NDEC; ++w)
          bulk_g2s(st + A_TILE + XT + w * REC, a.tree + ((size_t)(rb * 8 + w) * a.NG + (k0 + i)) * REC, REC, full + s, pol);
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int s = i % S, k = i / S;
        if (!mbar_wait(ready + s, (uint32_t)k & 1u)) { atomicExch(a.status, ERR_WAIT_MMA); ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_addr(smem + (size_t)s * STAGE), sb = sa + A_TILE;
        const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb);
#pragma unroll
        for (int j = 0; j < 4; ++j) tc_mma(tmem, da + 2 * j, db + 2 * j, a.idesc, (i | j) ? 1u : 0u);
        tc_commit(empty + s);
      }
      tc_commit(accbar);                                          // arrives when every MMA above has completed
    }
  } else {
    // ---------------------------------------------------------------- decode warps
    const size_t rbase = (size_t)(rb * 8 + warp) * a.NG;
    int lo = 0, hi = 0;
    if (nk > 0) { lo = __ldg(a.eo + rbase + k0); hi = __ldg(a.eo + rbase + k0 + 1); }
    for (int i = 0; i < nk; ++i) {
      const int s = i % S, k = i / S;
      int nlo = hi, nhi = hi;
      if (i + 1 < nk) nhi = __ldg(a.eo + rbase + k0 + i + 2);    // next record's list end (lists are contiguous)
      if (!mbar_wait(full + s, (uint32_t)k & 1u)) {
        if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
        break;
      }
      uint8_t* st = smem + (size_t)s * STAGE;
      uint32_t A[4][4];
      decode_frag(load_rec_shared(st + A_TILE + XT + warp * REC, lane), A);
      for (int base = lo; base < hi; base += 32) {
        const int n = min(32, hi - base);
        const uint32_t mine = (lane < n) ? __ldg(a.el + base + lane) : 0u;
        for (int e = 0; e < n; ++e) patch_entry(A, __shfl_sync(FULL, mine, e), lane);
      }
      // lane l addresses row (l & 7) of matrix (l >> 3): matrices = (rows 0-7 | 8-15) x (16-byte chunk 2ks | 2ks+1)
      const int mrow = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
      const uint32_t rowaddr = smem_addr(st) + mrow * 128;
      const int chalf = lane >> 4;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        stmatrix_x4(rowaddr + (uint32_t)(((2 * q + chalf) ^ (mrow & 7)) << 4), A[q][0], A[q][1], A[q][2], A[q][3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ready + s);
      lo = nlo; hi = nhi;
    }
    // ---------------------------------------------------------------- epilogue
    const bool acc_ok = mbar_wait(accbar, 0u);
    if (!acc_ok && lane == 0) atomicExch(a.status, ERR_WAIT_ACC);
    tc_fence_after();
    const int q4 = warp & 3, half = warp >> 2;
    const int row = rb * 128 + q4 * 32 + lane;
    const int cper = NT / 2;                                      // columns of this warp
    const int unit = tt * a.RB + rb;
    if (acc_ok && nk > 0) {
      for (int c0 = half * cper; c0 < (half + 1) * cper; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0, v);
        if (a.KS == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok < a.B) {
              const float f = __uint_as_float(v[j]);
              const __nv_bfloat16 hv = __float2bfloat16_rn(f);
              a.Y[(size_t)tok * a.M + row] = *reinterpret_cast<const uint16_t*>(&hv);
              if (a.Yf) a.Yf[(size_t)tok * a.M + row] = f;
            }
          }
        } else {
          float* part = a.ws + ((size_t)unit * a.KS + ks) * NT * 128;
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(size_t)(c0 + j) * 128 + q4 * 32 + lane] = __uint_as_float(v[j]);
        }
      }
    }
    if (a.KS > 1) {
      __threadfence();
      named_bar_sync(1, NDEC * 32);
      if (tid == 0) flags[1] = (atomicAdd(a.cnt + unit, 1) == a.KS - 1);
      named_bar_sync(1, NDEC * 32);
      if (flags[1]) {
        __threadfence();
        // the last CTA to arrive adds the KS partial tiles in split order; eight token columns per thread are kept in
        // flight so the L2 latency of the partial reads overlaps
        const int r = tid & 127;
        const int ncol = min(NT, a.B - tok0);
        const float* base = a.ws + (size_t)unit * a.KS * NT * 128 + r;
        for (int c0 = tid >> 7; c0 < ncol; c0 += 16) {
          float sum[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) sum[u] = 0.f;
          for (int p = 0; p < a.KS; ++p) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = c0 + 2 * u;
              if (c < ncol) sum[u] += __ldcg(base + ((size_t)p * NT + c) * 128);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int c = c0 + 2 * u;
            if (c < ncol) {
              const __nv_bfloat16 hv = __float2bfloat16_rn(sum[u]);
              a.Y[(size_t)(tok0 + c) * a.M + rb * 128 + r] = *reinterpret_cast<const uint16_t*>(&hv);
              if (a.Yf) a.Yf[(size_t)(tok0 + c) * a.M + rb * 128 + r] = sum[u];
            }
          }
        }
        if (tid == 0) a.cnt[unit] = 0;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem, (uint32_t)(NT < 32 ? 32 : NT));
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct GemmPlan { int NT, TT, RB, KS, stages; size_t smem; };

GemmPlan gemm_plan(long long M, long long N, long long B) {
  GemmPlan p;
  p.NT = B <= 64 ? 64 : (B <= 128 ? 128 : 256);
  p.TT = (int)((B + p.NT - 1) / p.NT);
  p.RB = (int)(M / 128);
  const int NG = (int)(N / 64), sms = st::sm_count();
  const long long units = (long long)p.RB * p.TT;
  int best = 1;
  double best_score = -1.0;
  const int ksmax = NG / 4 < 1 ? 1 : (NG / 4 > 32 ? 32 : NG / 4);
  for (int ks = 1; ks <= ksmax; ++ks) {
    const long long ctas = units * ks;
    const long long waves = (ctas + sms - 1) / sms;
    const double score = (double)ctas / (double)(waves * sms) - 0.03 * ks * p.NT / 256.0;   // partial-sum traffic
    if (score > best_score + 1e-9) { best_score = score; best = ks; }
  }
  p.KS = best;
  const int stage = A_TILE + p.NT * 128 + RAW;
  int s = (int)((212 * 1024) / stage);
  p.stages = s > 6 ? 6 : s;
  p.smem = (size_t)p.stages * stage + 1024 /* alignment slack */ + 256 /* barriers */;
  return p;
}
}  // namespace

extern "C" int64_t st_gemm_workspace_bytes(int64_t M, int64_t N, int64_t B) {
  if (M <= 0 || N <= 0 || M % 128 || N % 64 || B < 1) return -1;
  const GemmPlan p = gemm_plan(M, N, B);
  return p.KS == 1 ? 0 : (int64_t)p.RB * p.TT * p.KS * p.NT * 128 * 4;
}

extern "C" int st_gemm(const void* tree, const int32_t* eo, const uint32_t* el, const void* X, void* Y, float* Yf32,
                       int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 128 == 0 && N % 64 == 0,
             "st_gemm: M %% 128 and N %% 64 must be 0 (got %lld x %lld)", (long long)M, (long long)N);
  ST_REQUIRE(B >= 1 && B < (1ll << 24), "st_gemm: batch out of range");
  ST_REQUIRE(tree && eo && el && X && Y && cnt, "st_gemm: null pointer");
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(X), "st_gemm: tree and X must be 16-byte aligned");
  const GemmPlan p = gemm_plan(M, N, B);
  const long long need = p.KS == 1 ? 0 : (long long)p.RB * p.TT * p.KS * p.NT * 128 * 4;
  ST_REQUIRE(need == 0 || (ws && ws_bytes >= need), "st_gemm: workspace of %lld bytes needed, %lld given", need,
             (long long)ws_bytes);
  ST_REQUIRE((long long)p.RB * p.TT * p.KS < (1ll << 31), "st_gemm: grid too large");
  EncodeTiledFn enc = encode_fn();
  ST_REQUIRE(enc != nullptr, "st_gemm: cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)B};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)p.NT};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult cr = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ST_REQUIRE(cr == CUDA_SUCCESS, "st_gemm: cuTensorMapEncodeTiled failed (%d)", (int)cr);
  GemmArgs a;
  a.tree = (const uint8_t*)tree; a.eo = eo; a.el = el; a.Y = (uint16_t*)Y; a.Yf = Yf32; a.ws = (float*)ws; a.cnt = cnt;
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "st_gemm: no device status word");
  a.M = M; a.N = N; a.B = (int)B; a.NG = (int)(N / 64); a.NT = p.NT; a.KS = p.KS; a.RB = p.RB; a.TT = p.TT;
  a.stages = p.stages;
  // instruction descriptor: D fp32, A and B bf16, both K-major, N = NT, M = 128
  a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    if (int e = st::cuda_fail(cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024),
                              "st_gemm: shared memory attribute"))
      return e;
    set[dev] = true;
  }
  gemm_kernel<<<(unsigned)(p.RB * p.TT * p.KS), 320, p.smem, (cudaStream_t)stream>>>(a, xmap);
  ST_LAUNCH_CHECK("st_gemm launch");
  return 0;
}
