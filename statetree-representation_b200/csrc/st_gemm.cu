// Large-batch fused tree-decode + GEMM on the 5th-generation tensor cores (tcgen05 / TMEM) of sm_100a.
//   Y[B, M] = X[B, N] W[M, N]^T,  W as state-tree records, fp32 accumulation in tensor memory, BF16 output.
//
// One CTA computes a 128-row block of W against one tile of NT tokens (NT = 64, 128 or 256) over a contiguous range
// of 64-column k-tiles.  Warp roles (20 warps):
//   warps 0-15  decode, in two groups of eight (group g takes every second k-tile): each warp turns one record into
//               its mma-fragment registers (five integer ops per four weights), patches escapes, and writes the
//               16 x 64 BF16 sub-tile into the K-major, 128-byte-swizzled A tile with stmatrix; fence.proxy.async
//               hands the tile to the tensor core
//   warp 16     record producer: one 3-D tiled TMA load per k-tile brings the eight 1552-byte records of the block's
//               eight 16-row tiles into a deep ring
//   warp 17     activation producer: one tiled TMA load of X[tok0 .. tok0 + NT, 64 cols] with the 128-byte swizzle
//   warps 18-19 MMA issuers: one elected thread each issues four tcgen05.mma (128 x NT x 16, kind::f16) per k-tile of
//               its decode group, A and B read from shared memory through descriptors, D in its own TMEM
//               accumulator; tcgen05.commit releases the stage
// Epilogue: the decode warps read the accumulators with tcgen05.ld, add the two issuers' tiles in a fixed order and
// park the fp32 tile in shared memory; the CTAs that split a k range form a thread-block cluster and add their tiles
// through distributed shared memory in rank order (deterministic), then store BF16.
// The grouped (mixture-of-experts) variant runs the same pipeline per (block of NT routed pairs, 128-row block): the
// block's expert selects the weight tensor map and escape tables, the activation tile comes from rows gathered in
// block order, and the result rows are scattered back to their pair indices.
// Every mbarrier wait is bounded; a wait that runs out sets the device status word and the CTA leaves after
// releasing its tensor memory.
#include <cuda.h>

#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
using namespace st;

constexpr int A_TILE = 128 * 128;            // 128 rows x 64 bf16, one swizzle atom wide
constexpr int NDEC = 8;                      // decode warps = records per k-tile

constexpr int MAXL = 4;                       // matrices in one list launch

struct GemmArgs {
  const uint8_t* tree; const int* eo; const uint32_t* el;
  uint16_t* Y; float* Yf; int* status;
  // grouped (mixture of experts): per-expert weight tensor maps and escape tables, pairs in moe_align layout
  const CUtensorMap* maps; const long long* eop; const long long* elp;
  const int* sorted; const int* bexp; const int* npost; int E;
  long long M, N;
  int B, NG, NT, KS, RB, TT, stages, rstages, nmma, bar_off;
  uint32_t idesc;
  // list of matrices that share the activations (q / k / v, gate / up as separate trees): member of each row block
  int nlist; int rbend[MAXL];                 // first row block after each member in the concatenation
  const int* leo[MAXL]; const uint32_t* lel[MAXL]; uint16_t* lY[MAXL]; float* lYf[MAXL]; long long lM[MAXL];
};
struct WMaps { CUtensorMap m[MAXL]; };        // weight tensor maps: one, or one per member of a list

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               :: "r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               :: "r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_addr(bar)) : "memory");
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Two decode groups of eight warps (group g takes the k-tiles g, g + 2, ...), a record producer, an activation
// producer and two MMA issuer warps: one CTA per SM.
constexpr int DG = 2;
constexpr int NDW = DG * NDEC;                                              // decode warps
constexpr int W_RAW = NDW, W_X = NDW + 1, W_MMA = NDW + 2;                  // role warps
constexpr int THREADS = (NDW + 2 + DG) * 32;
#define GW mbar_wait_look
__device__ __forceinline__ bool wait_decode(uint64_t* bar, uint32_t parity) { return GW(bar, parity); }
constexpr int RAW_SLOT = NDEC * REC;         // 12416 B: the eight records of one k-tile

// Two rings.  The RAW ring (R slots of eight records) faces HBM: its depth sets the bytes in flight.  The TILE ring
// (S stages of decoded weight tile + activation tile) covers the decode -> MMA hand-over and the L2 latency of the
// activation loads; one mbarrier per stage counts both operands so the MMA thread waits once and commits once.
// The KS CTAs that split the k range of one (row block, token tile) form a thread-block cluster (blockIdx.x % KS is
// the rank).  After its main loop every CTA parks its fp32 accumulator tile in its own shared memory; after a cluster
// barrier CTA j adds the KS tiles for its share of the token columns through distributed shared memory, in rank
// order (bit-identical from run to run), and stores BF16.  No partial sums travel through global memory.
template <bool GROUPED>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ WMaps wmaps) {
  constexpr int NMMA = DG;                                     // issuer warps; a.nmma of them work
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int NT = a.NT, S = a.stages, R = a.rstages;
  const int XT = NT * 128;                       // bytes of an activation tile
  const int STAGE = A_TILE + XT;                 // tile stage: decoded weight tile + activation tile
  uint8_t* rawring = smem + (size_t)S * STAGE;                       // [R] record slots (deep: covers HBM latency)
  // one barrier per tile stage collects both operands: 8 decode-warp arrivals + the activation tile's TMA bytes
  uint64_t* ready = reinterpret_cast<uint64_t*>(smem + a.bar_off);   // [S] both operands of the stage are in place
  uint64_t* empty = ready + S;                                       // [S] MMAs that read the stage have completed
  uint64_t* rfull = empty + S;                                       // [R] records landed
  uint64_t* rempty = rfull + R;                                      // [R] records copied to registers
  uint64_t* accbar = rempty + R;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accbar + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // unit of this CTA
  const int ks = blockIdx.x % a.KS, rt = blockIdx.x / a.KS;
  const int rb = rt % a.RB, tt = rt / a.RB;
  const int k0 = (int)((long long)a.NG * ks / a.KS), k1 = (int)((long long)a.NG * (ks + 1) / a.KS);
  const int nk = k1 - k0;
  const int tok0 = tt * NT;
  // the matrix this CTA multiplies by: the one of the call, or (grouped) the expert of pair block tt
  const int* eo = a.eo;
  const uint32_t* el = a.el;
  const CUtensorMap* wm = &wmaps.m[0];
  int lrb = rb;                                                  // row block inside its matrix
  uint16_t* Yp = a.Y;
  float* Yfp = a.Yf;
  long long Mp = a.M;
  if (!GROUPED && a.nlist > 0) {                                 // a list: the member this row block belongs to
    int m = 0;
    while (m + 1 < a.nlist && rb >= a.rbend[m]) ++m;
    lrb = rb - (m ? a.rbend[m - 1] : 0);
    eo = a.leo[m]; el = a.lel[m]; wm = &wmaps.m[m];
    Yp = a.lY[m]; Yfp = a.lYf[m]; Mp = a.lM[m];
  }
  if (GROUPED) {
    pdl_wait();                                                  // the block table comes from an earlier kernel
    if (tok0 >= a.npost[0]) return;                              // beyond the blocks the routing filled
    const int expert = a.bexp[tt];
    if (expert < 0 || expert >= a.E) return;                     // another rank's expert
    eo = reinterpret_cast<const int*>(a.eop[expert]);
    el = reinterpret_cast<const uint32_t*>(a.elp[expert]);
    wm = a.maps + expert;
  }

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(ready + s, NDEC + 1); mbar_init(empty + s, 1); }
    for (int r = 0; r < R; ++r) { mbar_init(rfull + r, 1); mbar_init(rempty + r, NDEC); }
    mbar_init(accbar, NMMA);                                       // every issuer warp arrives, working or not
    fence_barrier_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(tmem_slot, (uint32_t)(a.nmma * NT));              // 64 .. 256 columns: one accumulator per working issuer
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();

  if (warp == W_RAW) {
    // ---------------------------------------------------------------- record producer: one tiled TMA load per k-tile
    // fetches the eight records (row tiles rb * 8 .. + 7 of column group k0 + i) through a 3-D view of the tree
    // [row tile][column group][194 x u64]; eight separate 1552-byte bulk copies per k-tile would cost far more issue time
    if (lane == 0) {
      for (int i = 0, r = 0, k = 0; i < nk; ++i, r = (r + 1 == R ? 0 : r + 1), k += (r == 0)) {
        if (k > 0 && !GW(rempty + r, (uint32_t)(k - 1) & 1u)) { atomicExch(a.status, ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(rfull + r, (uint32_t)RAW_SLOT);
        tma_load_3d(rawring + (size_t)r * RAW_SLOT, wm, 0, k0 + i, lrb * 8, rfull + r);
      }
    }
  } else if (warp == W_X) {
    // ---------------------------------------------------------------- activation producer.  The activations are the
    // only input an earlier kernel of the stream may still be writing: with programmatic dependent launch the CTA
    // starts (and its record producer streams weights) under the tail of that kernel, and this thread is the one that
    // waits for it.  Everything that touches the output is downstream of the first activation tile.
    if (lane == 0) {
      pdl_wait();
      for (int i = 0, s = 0, k = 0; i < nk; ++i, s = (s + 1 == S ? 0 : s + 1), k += (s == 0)) {
        if (k > 0 && !GW(empty + s, (uint32_t)(k - 1) & 1u)) { atomicExch(a.status, ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(ready + s, (uint32_t)XT);
        tma_load_2d(smem + (size_t)s * STAGE + A_TILE, &xmap, (k0 + i) * 64, tok0, ready + s);
      }
    }
  } else if (warp >= W_MMA) {
    // ---------------------------------------------------------------- MMA issuers.  The serial cost of one thread
    // per k-tile (its barrier wait, four tcgen05.mma and the commit) is of the order of a k-tile's share of the decode
    // time, so one issuer would hold the pipeline back.  Two issuers alternate k-tiles, each into its own accumulator (the epilogue adds the two in a
    // fixed order), so the serial cost per k-tile halves and the result does not depend on which issuer ran first.
    // This needs an even number of tile stages and record slots: then every stage and slot belongs to one decode group
    // and one issuer, which use it in their own program order.  (A waiter may be at most one phase ahead of an mbarrier:
    // with shared stages an issuer could ask for use k of a stage whose use k - 1, the other issuer's, has not
    // completed, and the parity test would pass on use k - 2.)  With three stages (256-token tiles) one issuer works.
    const int m = warp - W_MMA;
    if (lane == 0 && m >= a.nmma) mbar_arrive(accbar);
    if (lane == 0 && m < a.nmma) {
      const uint32_t acc = tmem + (uint32_t)(m * NT);
      int s = m % S, k = m / S;
      for (int i = m; i < nk; i += a.nmma) {
        if (!GW(ready + s, (uint32_t)k & 1u)) {
          atomicExch(a.status, ERR_WAIT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_addr(smem + (size_t)s * STAGE);
        const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_TILE);
#pragma unroll
        for (int j = 0; j < 4; ++j) tc_mma(acc, da + 2 * j, db + 2 * j, a.idesc, (i >= a.nmma || j) ? 1u : 0u);
        tc_commit(empty + s);
        s += a.nmma; while (s >= S) { s -= S; ++k; }
      }
      tc_commit(accbar);                                          // arrives when every MMA of this issuer has completed
    }
  } else {
    // ---------------------------------------------------------------- decode warps: group g = warp / 8 takes the
    // k-tiles i = g, g + DG, ...; warp r of a group decodes record r (rows 16 r .. 16 r + 15 of the block)
    const int grp = warp / NDEC, rec = warp % NDEC;
    const size_t rbase = (size_t)(lrb * 8 + rec) * a.NG + k0;
    // Escape entries are fetched one k-tile ahead: the list offsets of this warp's records come 32 k-tiles at a time
    // (lane l holds the offsets of k-tile eo_base + l) and the first 32 entries of the next record are requested before
    // this record is decoded, so no global-load latency sits between the records landing and the tile being handed
    // to the tensor core (one record in six has an escape; eight warps must all arrive before the MMA can start)
    int eo_base = 0, eo_lo = 0, eo_hi = 0;
    unsigned emask = 0u;                                           // bit l: k-tile eo_base + l of this warp has escapes
    auto load_offsets = [&](int first) {
      eo_base = first;
      const int j = first + lane;
      eo_lo = j < nk ? __ldg(eo + rbase + j) : 0;
      eo_hi = j < nk ? __ldg(eo + rbase + j + 1) : 0;
      emask = __ballot_sync(FULL, eo_hi > eo_lo);
    };
    int lo = 0, hi = 0;
    uint32_t ent = 0u;
    if (grp < nk) {
      load_offsets(grp);
      if (emask & 1u) {
        lo = __shfl_sync(FULL, eo_lo, 0);
        hi = __shfl_sync(FULL, eo_hi, 0);
        if (lane < hi - lo) ent = __ldg(el + lo + lane);
      }
    }
    int s = grp % S, k = grp / S, r = grp % R, rk = grp / R;          // tile stage / use count, record slot / use count
    for (int i = grp; i < nk; i += DG) {
      int nlo = 0, nhi = 0;
      uint32_t nent = 0u;
      if (i + DG < nk) {
        if (i + DG - eo_base >= 32) load_offsets(i + DG);
        const int off = i + DG - eo_base;
        if ((emask >> off) & 1u) {                                // five records in six have none: one bit test
          nlo = __shfl_sync(FULL, eo_lo, off);
          nhi = __shfl_sync(FULL, eo_hi, off);
          if (lane < nhi - nlo) nent = __ldg(el + nlo + lane);
        }
      }
      if (!wait_decode(rfull + r, (uint32_t)rk & 1u)) {
        if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
        break;
      }
      const RecRegs rr = load_rec_shared(rawring + (size_t)r * RAW_SLOT + rec * REC, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(rempty + r);                     // the slot can be refilled while we decode
      uint32_t A[4][4];
      decode_frag(rr, A);
      {
        const int n = min(32, hi - lo);
        for (int e = 0; e < n; ++e) patch_entry(A, __shfl_sync(FULL, ent, e), lane);
      }
      for (int base = lo + 32; base < hi; base += 32) {          // a crowded record: the rest of its list
        const int n = min(32, hi - base);
        const uint32_t mine = (lane < n) ? __ldg(el + base + lane) : 0u;
        for (int e = 0; e < n; ++e) patch_entry(A, __shfl_sync(FULL, mine, e), lane);
      }
      lo = nlo; hi = nhi; ent = nent;
      if (k > 0 && !wait_decode(empty + s, (uint32_t)(k - 1) & 1u)) {   // the MMAs of the stage's last use are done
        if (lane == 0) atomicExch(a.status, ERR_WAIT_EMPTY);
        break;
      }
      uint8_t* st = smem + (size_t)s * STAGE;
      // lane l addresses row (l & 7) of matrix (l >> 3): matrices = (rows 0-7 | 8-15) x (16-byte chunk 2q | 2q+1)
      const int mrow = rec * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
      const uint32_t rowaddr = smem_addr(st) + mrow * 128;
      const int chalf = lane >> 4;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        stmatrix_x4(rowaddr + (uint32_t)(((2 * q + chalf) ^ (mrow & 7)) << 4), A[q][0], A[q][1], A[q][2], A[q][3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ready + s);
      s += DG; while (s >= S) { s -= S; ++k; }
      r += DG; while (r >= R) { r -= R; ++rk; }
    }
    // ---------------------------------------------------------------- epilogue 1: accumulator -> own shared memory
    const bool acc_ok = GW(accbar, 0u);
    if (!acc_ok && lane == 0) atomicExch(a.status, ERR_WAIT_ACC);
    tc_fence_after();
    float* stg = reinterpret_cast<float*>(smem);                 // [NT][128] fp32, over the (now idle) ring
    const int q4 = warp & 3, cg = warp >> 2;                     // TMEM lane quadrant, column share of the warp
    const int cper = NT / (NDW / 4);
    const bool two = a.nmma > 1 && nk > 1;                       // the second issuer had a k-tile
    for (int c0 = cg * cper; c0 < (cg + 1) * cper; c0 += 16) {
      uint32_t v[32], w[32];                                     // (the x16 load fills the first sixteen)
      const uint32_t t0 = tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0;
      tmem_ld16(t0, v);
      if (two) {
        tmem_ld16(t0 + (uint32_t)NT, w);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) stg[(size_t)(c0 + j) * 128 + q4 * 32 + lane] = __uint_as_float(v[j]);
    }
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();                                            // every CTA of the cluster has parked its tile
  if (warp < NDW) {
    // ---------------------------------------------------------------- epilogue 2: add the KS tiles, rank order
    const int ncol = GROUPED ? NT : min(NT, a.B - tok0);        // grouped: padding pairs are filtered per column
    const int c_lo = (int)((long long)NT * ks / a.KS), c_hi = (int)((long long)NT * (ks + 1) / a.KS);
    const uint32_t mine = smem_addr(smem);
    const int c_end = min(c_hi, ncol);
    // two columns per pass, every partial tile's float4 requested before the first add: distributed-shared-memory
    // reads have a long latency, so the loads of a pass must all be in flight together
    for (int c = c_lo + warp; c < c_end; c += 2 * NDW) {
      const int c2 = c + NDW;
      float4 v0[8], v1[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        if (p < a.KS) {
          v0[p] = ld_cluster_f4(map_to_cta(mine + (uint32_t)((c * 128 + 4 * lane) * 4), (uint32_t)p));
          if (c2 < c_end) v1[p] = ld_cluster_f4(map_to_cta(mine + (uint32_t)((c2 * 128 + 4 * lane) * 4), (uint32_t)p));
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int cc = h ? c2 : c;
        if (cc >= c_end) break;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          if (p < a.KS) {
            const float4 v = h ? v1[p] : v0[p];
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
          }
        }
        long long row = tok0 + cc;
        if (GROUPED) {                                            // result rows go back to their pair index
          row = a.sorted[tok0 + cc];
          if (row < 0 || row >= a.B) continue;
        }
        const size_t o = (size_t)row * Mp + lrb * 128 + 4 * lane;
        uint2 packed;
        packed.x = pack_bf16(sum.x, sum.y);
        packed.y = pack_bf16(sum.z, sum.w);
        *reinterpret_cast<uint2*>(Yp + o) = packed;
        if (Yfp) *reinterpret_cast<float4*>(Yfp + o) = sum;
      }
    }
  }
  __syncwarp();
  cluster_sync_all();                                            // nobody leaves while a peer still reads its tile
  if (warp == W_MMA) {
    __syncwarp();
    tmem_dealloc(tmem, (uint32_t)(a.nmma * NT));
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

struct GemmPlan { int NT, TT, RB, KS, stages, rstages, nmma, bar_off; size_t smem; };

template <bool GROUPED>
int gemm_attr() {                                                // once per device: opt in to the large dynamic shared memory
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    if (int e = st::cuda_fail(cudaFuncSetAttribute(gemm_kernel<GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   220 * 1024), "st_gemm: shared memory attribute"))
      return e;
    set[dev] = true;
  }
  return 0;
}

// CTAs that can be resident at once when launched as clusters of ks (one CTA per SM): a cluster lives inside one GPC,
// so sizes that do not divide a GPC's SM count strand SMs (clusters of 3 fit 44 times, not 49: a 48-cluster grid then
// runs as two waves).  Asked from the driver once per (device, cluster size, token tile).
long long resident_ctas(int ks, int NT, size_t smem, int sms) {
  static int cache[64][9][3] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int ti = NT <= 64 ? 0 : (NT <= 128 ? 1 : 2);
  if (ks == 1 || dev < 0 || dev >= 64) return sms;
  if (cache[dev][ks][ti] == 0) {
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(ks * sms));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (gemm_attr<false>() != 0 || cudaOccupancyMaxActiveClusters(&n, gemm_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sms / ks;                                              // no answer (no device): assume perfect packing
    }
    cache[dev][ks][ti] = n;
  }
  return (long long)cache[dev][ks][ti] * ks;
}

// rings and issuers for a token tile of NT
void gemm_rings(GemmPlan& p) {
  const size_t stage = A_TILE + (size_t)p.NT * 128;
  const size_t stg = (size_t)p.NT * 128 * 4;                      // the parked accumulator tile reuses the rings
  // tile stages (decoded weight tile + activation tile): enough to cover the L2 latency of the activation loads; the
  // rest of the shared memory goes to the record ring, which covers the HBM latency
  p.stages = p.NT >= 256 ? 3 : 4;
  p.rstages = (int)((212 * 1024 - p.stages * stage) / RAW_SLOT);
  if (p.rstages > 12) p.rstages = 12;
  // The two decode groups alternate k-tiles.  A decode warp waits for the fill of a record slot by the parity of that
  // slot's use count, and an mbarrier tells only the current phase from the previous one, so a waiter must never be
  // two fills ahead.  With an even slot count every slot belongs to one group, whose own program order guarantees
  // that; with an odd count the groups share slots, and a group that runs ahead while a bulk copy of the other
  // group's k-tile is still in flight passes its wait on the stale phase, reads old records and releases the slot a
  // second time.  So: always an even number of record slots.  (Tile stages may be odd: their waits are on the
  // previous use of a stage.)
  p.rstages &= ~1;
  // two MMA issuers need every tile stage owned by one decode group as well: an even count of stages
  p.nmma = (p.stages % 2 == 0 && p.rstages >= 4) ? 2 : 1;
  size_t ring = (size_t)p.stages * stage + (size_t)p.rstages * RAW_SLOT;
  ring = (ring + 15) & ~(size_t)15;
  if (ring < stg) ring = stg;
  p.bar_off = (int)ring;
  p.smem = ring + 1024 /* alignment slack */ + 512 /* barriers */;
}

GemmPlan gemm_plan(long long M, long long N, long long B) {
  GemmPlan p;
  p.NT = B <= 64 ? 64 : (B <= 128 ? 128 : 256);
  p.TT = (int)((B + p.NT - 1) / p.NT);
  p.RB = (int)(M / 128);
  const int NG = (int)(N / 64), sms = st::sm_count();
  const long long units = (long long)p.RB * p.TT;
  gemm_rings(p);
  // Split of the k range = cluster size (<= 8).  A CTA's time is its k-tiles plus a fixed part (start-up, pipeline fill,
  // epilogue; the epilogue grows with the tiles to add through distributed shared memory); a grid larger than the
  // CTAs that are resident at once runs in waves, each paying all of it again.  Take the split with the least
  // estimated time (the constants are in units of one k-tile of a 64-token tile).
  int best = 1;
  double best_t = 1e30;
  const int ksmax = NG / 4 < 1 ? 1 : (NG / 4 > 8 ? 8 : NG / 4);
  const double tile = p.NT >= 256 ? 1.4 : (p.NT >= 128 ? 1.08 : 1.0);
  for (int ks = 1; ks <= ksmax; ++ks) {
    const long long ctas = units * ks;
    const long long slots = resident_ctas(ks, p.NT, p.smem, sms);
    if (slots <= 0) continue;
    const long long waves = (ctas + slots - 1) / slots;
    const double t = (double)waves * ((double)((NG + ks - 1) / ks) * tile + 14.0 + 0.8 * ks * p.NT / 64.0);
    if (t < best_t - 1e-9) { best_t = t; best = ks; }
  }
  p.KS = best;
  return p;
}

template <bool GROUPED>
int gemm_launch(const GemmPlan& p, const GemmArgs& a, const CUtensorMap& xmap, const WMaps& wmaps, cudaStream_t stream) {
  if (int e = gemm_attr<GROUPED>()) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.RB * p.TT * p.KS));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.KS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = st::pdl_enabled() ? 2 : 1;
  return st::cuda_fail(cudaLaunchKernelEx(&cfg, gemm_kernel<GROUPED>, a, xmap, wmaps), GROUPED ? "st_moe_group_gemm launch" : "st_gemm launch");
}

// activations [rows, N] BF16 as 64-column x NT-row boxes with the 128-byte swizzle
int make_xmap(CUtensorMap* map, const void* X, long long rows, long long N, int NT, const char* who) {
  EncodeTiledFn enc = encode_fn();
  ST_REQUIRE(enc != nullptr, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)NT};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult cr = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ST_REQUIRE(cr == CUDA_SUCCESS, "%s: cuTensorMapEncodeTiled failed (%d)", who, (int)cr);
  return 0;
}

// a tree [M/16][N/64][1552 B] as 194 x u64 rows, boxes of eight row tiles of one column group
int make_wmap(CUtensorMap* map, const void* tree, long long M, long long N, const char* who) {
  EncodeTiledFn enc = encode_fn();
  ST_REQUIRE(enc != nullptr, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
  const cuuint64_t wd[3] = {194u, (cuuint64_t)(N / 64), (cuuint64_t)(M / 16)};
  const cuuint64_t wst[2] = {(cuuint64_t)REC, (cuuint64_t)(N / 64) * REC};
  const cuuint32_t wbox[3] = {194u, 1u, 8u};
  const cuuint32_t we[3] = {1u, 1u, 1u};
  const CUresult wr = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void*>(tree), wd, wst, wbox, we,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ST_REQUIRE(wr == CUDA_SUCCESS, "%s: cuTensorMapEncodeTiled (tree) failed (%d)", who, (int)wr);
  return 0;
}

// instruction descriptor: D fp32, A and B bf16, both K-major, N = NT, M = 128
uint32_t mma_idesc(int NT) { return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); }
}  // namespace

extern "C" int64_t st_gemm_workspace_bytes(int64_t M, int64_t N, int64_t B) {
  if (M <= 0 || N <= 0 || M % 128 || N % 64 || B < 1) return -1;
  return 0;                                                      // split partial sums stay in shared memory
}

extern "C" int st_gemm(const void* tree, const int32_t* eo, const uint32_t* el, const void* X, void* Y, float* Yf32,
                       int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 128 == 0 && N % 64 == 0,
             "st_gemm: M %% 128 and N %% 64 must be 0 (got %lld x %lld)", (long long)M, (long long)N);
  ST_REQUIRE(B >= 1 && B < (1ll << 24), "st_gemm: batch out of range");
  ST_REQUIRE(tree && eo && el && X && Y && cnt, "st_gemm: null pointer");
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(X), "st_gemm: tree and X must be 16-byte aligned");
  const GemmPlan p = gemm_plan(M, N, B);
  (void)ws; (void)ws_bytes;
  ST_REQUIRE((long long)p.RB * p.TT * p.KS < (1ll << 31), "st_gemm: grid too large");
  CUtensorMap xmap;
  WMaps wmaps;
  memset(&wmaps, 0, sizeof(wmaps));
  if (int e = make_xmap(&xmap, X, B, N, p.NT, "st_gemm")) return e;
  if (int e = make_wmap(&wmaps.m[0], tree, M, N, "st_gemm")) return e;
  GemmArgs a = {};
  a.tree = (const uint8_t*)tree; a.eo = eo; a.el = el; a.Y = (uint16_t*)Y; a.Yf = Yf32;
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "st_gemm: no device status word");
  a.M = M; a.N = N; a.B = (int)B; a.NG = (int)(N / 64); a.NT = p.NT; a.KS = p.KS; a.RB = p.RB; a.TT = p.TT;
  a.stages = p.stages; a.rstages = p.rstages; a.nmma = p.nmma; a.bar_off = p.bar_off;
  a.idesc = mma_idesc(p.NT);
  return gemm_launch<false>(p, a, xmap, wmaps, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------- list of matrices
extern "C" int st_gemm_list(int64_t n, const void* const* trees, const int32_t* const* eo, const uint32_t* const* el,
                            const void* X, void* const* Y, float* const* Yf32, int64_t B, const int64_t* M, int64_t N,
                            int32_t* cnt, void* stream) {
  const char* who = "st_gemm_list";
  ST_REQUIRE(n >= 1 && n <= MAXL, "%s: 1 to %d matrices per call (got %lld)", who, MAXL, (long long)n);
  ST_REQUIRE(trees && eo && el && X && Y && M && cnt, "%s: null pointer", who);
  ST_REQUIRE(N > 0 && N % 64 == 0, "%s: N %% 64 must be 0", who);
  ST_REQUIRE(B >= 1 && B < (1ll << 24), "%s: batch out of range", who);
  ST_REQUIRE(st::aligned16(X), "%s: X must be 16-byte aligned", who);
  GemmArgs a = {};
  WMaps wmaps;
  memset(&wmaps, 0, sizeof(wmaps));
  long long total = 0;
  for (int i = 0; i < (int)n; ++i) {
    ST_REQUIRE(trees[i] && eo[i] && el[i] && Y[i], "%s: null pointer in member %d", who, i);
    ST_REQUIRE(st::aligned16(trees[i]), "%s: tree of member %d must be 16-byte aligned", who, i);
    ST_REQUIRE(M[i] > 0 && M[i] % 128 == 0, "%s: rows of member %d must be a positive multiple of 128", who, i);
    if (int e = make_wmap(&wmaps.m[i], trees[i], M[i], N, who)) return e;
    a.leo[i] = eo[i]; a.lel[i] = el[i]; a.lY[i] = (uint16_t*)Y[i]; a.lYf[i] = Yf32 ? Yf32[i] : nullptr; a.lM[i] = M[i];
    total += M[i];
    a.rbend[i] = (int)(total / 128);
  }
  a.nlist = (int)n;
  const GemmPlan p = gemm_plan(total, N, B);
  ST_REQUIRE((long long)p.RB * p.TT * p.KS < (1ll << 31), "%s: grid too large", who);
  CUtensorMap xmap;
  if (int e = make_xmap(&xmap, X, B, N, p.NT, who)) return e;
  a.eo = eo[0]; a.el = el[0]; a.Y = (uint16_t*)Y[0];
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "%s: no device status word", who);
  a.M = total; a.N = N; a.B = (int)B; a.NG = (int)(N / 64); a.NT = p.NT; a.KS = p.KS; a.RB = p.RB; a.TT = p.TT;
  a.stages = p.stages; a.rstages = p.rstages; a.nmma = p.nmma; a.bar_off = p.bar_off;
  a.idesc = mma_idesc(p.NT);
  return gemm_launch<false>(p, a, xmap, wmaps, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------- grouped (MoE)
extern "C" int64_t st_moe_tensor_map_bytes(void) { return (int64_t)sizeof(CUtensorMap); }

extern "C" int st_moe_tensor_maps(const int64_t* trees_host, int64_t E, int64_t M, int64_t N, void* maps_dev,
                                  void* stream) {
  ST_REQUIRE(E >= 1 && E <= 4096 && M > 0 && N > 0 && M % 128 == 0 && N % 64 == 0,
             "st_moe_tensor_maps: 1..4096 experts of M %% 128 == 0 rows and N %% 64 == 0 columns");
  ST_REQUIRE(trees_host && maps_dev && ((uintptr_t)maps_dev & 63u) == 0, "st_moe_tensor_maps: null or unaligned pointer");
  static thread_local CUtensorMap staging[4096];
  for (int64_t e = 0; e < E; ++e) {
    const void* tree = reinterpret_cast<const void*>(trees_host[e]);
    ST_REQUIRE(tree != nullptr && st::aligned16(tree), "st_moe_tensor_maps: tree %lld is null or unaligned", (long long)e);
    if (int r = make_wmap(&staging[e], tree, M, N, "st_moe_tensor_maps")) return r;
  }
  // pageable source: the copy is staged by the driver before the call returns, so `staging` may be reused at once
  return st::cuda_fail(cudaMemcpyAsync(maps_dev, staging, (size_t)E * sizeof(CUtensorMap), cudaMemcpyHostToDevice,
                                       (cudaStream_t)stream), "st_moe_tensor_maps: copy");
}

extern "C" int st_moe_group_gemm(const void* maps, const int64_t* eop, const int64_t* elp, int64_t E, const void* Xg,
                                 const int32_t* sorted, const int32_t* bexp, const int32_t* npost, int64_t nblk,
                                 int64_t bs, void* Y, float* Yf32, int64_t S, int64_t M, int64_t N, void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 128 == 0 && N % 64 == 0, "st_moe_group_gemm: M %% 128 and N %% 64 must be 0");
  ST_REQUIRE(bs == 64 || bs == 128, "st_moe_group_gemm: block size must be 64 or 128 (got %lld)", (long long)bs);
  ST_REQUIRE(E >= 1 && S >= 0 && nblk >= 0, "st_moe_group_gemm: sizes");
  if (S == 0 || nblk == 0) return 0;
  ST_REQUIRE(maps && eop && elp && Xg && sorted && bexp && npost && Y, "st_moe_group_gemm: null pointer");
  ST_REQUIRE(((uintptr_t)maps & 63u) == 0 && st::aligned16(Xg), "st_moe_group_gemm: maps 64-byte, Xg 16-byte aligned");
  GemmPlan p;
  p.NT = (int)bs;
  p.TT = (int)nblk;
  p.RB = (int)(M / 128);
  p.KS = 1;
  gemm_rings(p);
  ST_REQUIRE((long long)p.RB * p.TT < (1ll << 31), "st_moe_group_gemm: grid too large");
  CUtensorMap xmap;
  WMaps unused;
  if (int e = make_xmap(&xmap, Xg, nblk * bs, N, p.NT, "st_moe_group_gemm")) return e;
  memset(&unused, 0, sizeof(unused));
  GemmArgs a = {};
  a.Y = (uint16_t*)Y; a.Yf = Yf32;
  a.maps = reinterpret_cast<const CUtensorMap*>(maps); a.eop = (const long long*)eop; a.elp = (const long long*)elp;
  a.sorted = sorted; a.bexp = bexp; a.npost = npost; a.E = (int)E;
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "st_moe_group_gemm: no device status word");
  a.M = M; a.N = N; a.B = (int)S; a.NG = (int)(N / 64); a.NT = p.NT; a.KS = 1; a.RB = p.RB; a.TT = p.TT;
  a.stages = p.stages; a.rstages = p.rstages; a.nmma = p.nmma; a.bar_off = p.bar_off;
  a.idesc = mma_idesc(p.NT);
  return gemm_launch<true>(p, a, xmap, unused, (cudaStream_t)stream);
}
