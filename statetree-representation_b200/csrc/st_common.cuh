// Shared device helpers of the sm_100a state-tree kernels: record geometry, the 4-weight decode step, escape
// patches on mma fragments, mbarrier / bulk-copy (TMA) wrappers with bounded waits, and the status word.
//
// Record (1552 B per 16 rows x 64 columns; reference: statetree/format.py:9-12):
//   [0, 1024)    leaves, two 512-byte halves; lane L = (g, t) owns 16 B in each: k-steps 2h, 2h+1, rows g / g+8
//   [1024, 1536) states, lane L owns 16 B: word s = k-step s, low nibbles row g, high nibbles row g+8
//   [1536, 1552) nodes: byte 2g = exponent of row g, byte 2g+1 = exponent of row g+8
// A lane's 4 registers of k-step s are the mma.m16n8k16 A fragment of the 16 x 16 sub-block (columns 16s..16s+15).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace st {

constexpr int REC = 1552;          // bytes per weight record
constexpr int RKV = 1600;          // bytes per KV record (record + header + 11 escape slots)
constexpr int PAGE = 16;           // tokens per KV page
constexpr int HD = 128;            // head dimension of the KV kernels
constexpr int NSLOT = 11;          // in-record escape slots of a KV record
constexpr int XSLOT = 15;          // escape slots of a pool extension block
constexpr unsigned FULL = 0xFFFFFFFFu;

// status word codes written by kernels that gave up on a bounded wait
constexpr int ERR_WAIT_FULL = 1, ERR_WAIT_EMPTY = 2, ERR_WAIT_MMA = 3, ERR_WAIT_ACC = 4, ERR_WAIT_PEER = 5;
constexpr uint32_t SPIN_LIMIT = 1u << 24;   // mbarrier try_wait rounds before a kernel gives up (~seconds)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------------------------------------ decode
// Four weights from one leaf word (bytes: cols c, c+1, c+8, c+9 of one row), their four 4-bit states spread one per
// byte, and the row's node exponent replicated in every byte.  Leaf byte = mantissa << 1 | sign of the pair partner,
// so interleaving [leaf, exponent] bytes and rotating the 32-bit pair right by one bit lands each sign on bit 15 / 31
// (reference: statetree/csrc/kernels.cu:45-50).
__device__ __forceinline__ void dec_quad(uint32_t leaf, uint32_t states, uint32_t node4, uint32_t& lo, uint32_t& hi) {
  const uint32_t ex = node4 - states;
  const uint32_t a = __byte_perm(leaf, ex, 0x5140);
  const uint32_t b = __byte_perm(leaf, ex, 0x7362);
  lo = __funnelshift_r(a, a, 1);
  hi = __funnelshift_r(b, b, 1);
}

struct RecRegs { uint4 l0, l1, st; uint32_t nodes; };   // one lane's share of a record

// all four k-steps of a lane's fragment: A[s][q], q = 0: row g cols 2t..; 1: row g+8; 2: row g cols 8+2t..; 3: row g+8
__device__ __forceinline__ void decode_frag(const RecRegs& r, uint32_t (&A)[4][4]) {
  const uint32_t n0 = (r.nodes & 0xFFu) * 0x01010101u, n1 = ((r.nodes >> 8) & 0xFFu) * 0x01010101u;
  const uint32_t lw[8] = {r.l0.x, r.l0.y, r.l0.z, r.l0.w, r.l1.x, r.l1.y, r.l1.z, r.l1.w};
  const uint32_t sw[4] = {r.st.x, r.st.y, r.st.z, r.st.w};
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    dec_quad(lw[2 * s], sw[s] & 0x0F0F0F0Fu, n0, A[s][0], A[s][2]);
    dec_quad(lw[2 * s + 1], (sw[s] >> 4) & 0x0F0F0F0Fu, n1, A[s][1], A[s][3]);
  }
}

// overwrite element (row, col) of the record held as warp fragments with its exact bits; warp-uniform call
__device__ __forceinline__ void patch_frag(uint32_t (&A)[4][4], int row, int col, uint32_t bits, int lane) {
  const int cc = col & 15;
  if (lane == (row & 7) * 4 + ((cc & 7) >> 1)) {
    const int s = col >> 4, q = (row >> 3) + 2 * (cc >> 3);
    const uint32_t sh = 16u * (uint32_t)(cc & 1), msk = 0xFFFFu << sh, v = (bits & 0xFFFFu) << sh;
#pragma unroll
    for (int ss = 0; ss < 4; ++ss)
#pragma unroll
      for (int qq = 0; qq < 4; ++qq)
        if (ss == s && qq == q) A[ss][qq] = (A[ss][qq] & ~msk) | v;
  }
}

// escape list entry: bits << 16 | (record % 8) << 10 | row << 6 | col
__device__ __forceinline__ void patch_entry(uint32_t (&A)[4][4], uint32_t e, int lane) {
  patch_frag(A, (int)((e >> 6) & 15u), (int)(e & 63u), e >> 16, lane);
}

__device__ __forceinline__ RecRegs load_rec_global(const uint8_t* rec, int lane) {
  RecRegs r;
  const uint4* p = reinterpret_cast<const uint4*>(rec);
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.l0.x), "=r"(r.l0.y), "=r"(r.l0.z), "=r"(r.l0.w) : "l"(p + lane));
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.l1.x), "=r"(r.l1.y), "=r"(r.l1.z), "=r"(r.l1.w) : "l"(p + 32 + lane));
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.st.x), "=r"(r.st.y), "=r"(r.st.z), "=r"(r.st.w) : "l"(p + 64 + lane));
  r.nodes = __ldg(reinterpret_cast<const uint16_t*>(rec + 1536) + (lane >> 2));
  return r;
}

__device__ __forceinline__ RecRegs load_rec_shared(const uint8_t* rec, int lane) {
  RecRegs r;
  const uint4* p = reinterpret_cast<const uint4*>(rec);
  r.l0 = p[lane];
  r.l1 = p[32 + lane];
  r.st = p[64 + lane];
  r.nodes = *(reinterpret_cast<const uint16_t*>(rec + 1536) + (lane >> 2));
  return r;
}

// ------------------------------------------------------------------------------------------------ mma / matrices
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_r(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};"
               :: "r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// ------------------------------------------------------------------------------------------------ mbarrier / TMA
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait: false when the barrier did not flip within SPIN_LIMIT rounds (the caller records an error and leaves)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
    if (mbar_try(bar, parity)) return true;
  return false;
}
// the same with a non-blocking look first, for waiters whose barrier has usually flipped already (the tcgen05 GEMM's
// warps, which wait twice per k-tile)
__device__ __forceinline__ bool mbar_wait_look(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return ok ? true : mbar_wait(bar, parity);
}
// non-suspending variant: polls with test_wait, so a waiter notices the flip within a few cycles (try_wait may park the
// thread for a while); for short hand-overs between a few warps
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t i = 0; i < (SPIN_LIMIT << 4); ++i) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may start while
// its predecessor in the stream still runs: griddepcontrol.wait blocks until that predecessor has completed and its
// writes are visible (a no-op for an ordinary launch); launch_dependents lets the successor's CTAs be scheduled early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// thread-block clusters: barrier over all threads of all CTAs, and loads from another CTA's shared memory
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// pieces of the per-head RMSNorm + rotary embedding shared by the stand-alone kernel and the one fused with the KV
// append: written with explicit fused multiply-adds so that both produce the same bits
__device__ __forceinline__ float sumsq4(float a, float b, float c, float d) {
  return __fmaf_rn(d, d, __fmaf_rn(c, c, __fmaf_rn(b, b, __fmul_rn(a, a))));
}
__device__ __forceinline__ uint32_t rope_pair(float n0, float n1, float c, float s) {      // -> packed BF16 pair
  return pack_bf16(__fmaf_rn(n0, c, -__fmul_rn(n1, s)), __fmaf_rn(n0, s, __fmul_rn(n1, c)));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               :: "r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}

}  // namespace st
