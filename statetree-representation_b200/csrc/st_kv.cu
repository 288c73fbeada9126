// Compressed KV pages on sm_100a: append (page encode), dequant, and split decode attention straight over the pages.
//
// Page layout (frozen by the reference, statetree/csrc/kvcache.cu:1-14): uint8 [blocks, H, 2 (K/V), 2 (dim half), 1600];
// one 1600-byte unit = a 1552-byte record of 16 tokens x 64 dims (token = row) + a header word + 11 escape slots
// (bits << 16 | row << 6 | col); further escapes chain through 16-word blocks of a pool.
//
// Attention design: grid = B x Hkv x S; each of the 4 warps of a CTA walks its own pages of the split through a
// private 3-stage ring of 6400-byte bulk copies (one page of one KV head = K half 0/1, V half 0/1, contiguous), so a
// CTA keeps up to 12 pages (75 KB) in flight with no block-level barrier inside the loop.  S = q K^T and O += P V run
// on mma.m16n8k16 with the decoded K fragments as the B operand and the V fragments transposed in registers;
// P is fed as a BF16 high part plus a BF16 residual, so the softmax weights keep ~16 mantissa bits.
#include <math.h>
#include <stdlib.h>

#include "../../include/statetree_b200.h"
#include "st_common.cuh"
#include "st_host.h"

namespace {
using namespace st;

// byte offset of the leaf pair / state pair of columns 2l, 2l+1 of row r (statetree/csrc/kvcache.cu:31-38)
__device__ __forceinline__ int leaf_pair_off(int r, int l) {
  const int s = l >> 3, t = l & 3, hi = (l >> 2) & 1;
  return (s >> 1) * 512 + ((r & 7) * 4 + t) * 16 + ((s & 1) * 2 + (r >> 3)) * 4 + 2 * hi;
}
__device__ __forceinline__ int state_pair_off(int r, int l) {
  const int s = l >> 3, t = l & 3, hi = (l >> 2) & 1;
  return 1024 + ((r & 7) * 4 + t) * 16 + s * 4 + 2 * hi;
}
__device__ __forceinline__ size_t unit_off(long long blk, int H, int h, int kvi, int half) {
  return ((((size_t)blk * H + h) * 2 + kvi) * 2 + half) * RKV;
}

// ------------------------------------------------------------------------------------------------ append
struct AppendArgs {
  const uint16_t* K; const uint16_t* V;
  long long ks, vs;
  const long long* slot;
  uint8_t* kv;
  uint32_t* pool;
  int* pool_cnt;
  long long nblocks;
  int N, H, P, reuse;
  int gsz;                  // tokens of the call scanned per warp for segment starts (1: decode steps, 16: prefill)
};

// escape bookkeeping of one record while a warp appends rows to it (lane 0 owns the chain walk)
struct EscCursor {
  int cnt;   // in-record slots used
  int head;  // first extension block, -1 = none
  int tail;  // block currently appended to, -1 = not located yet
  int fill;  // entries in tail
};

__device__ void chain_put(const AppendArgs& a, EscCursor& c, uint32_t* slots, uint32_t e) {
  if (c.cnt < NSLOT) { slots[c.cnt++] = e; return; }
  if (c.head >= 0 && c.tail < 0) {                 // first use of an existing chain: find its first non-full block
    c.tail = c.head;
    for (int hops = 0; hops < 4096; ++hops) {
      const uint32_t w0 = a.pool[(size_t)c.tail * 16];
      const int nx = (int)(w0 >> 8) - 1;
      c.fill = (int)(w0 & 0xFFu);
      if (c.fill < XSLOT || nx < 0 || nx >= a.P) break;
      c.tail = nx;
    }
  }
  if (c.tail >= 0 && c.fill == XSLOT) {            // full: step to a recycled block that is already linked
    const int nx = (int)(a.pool[(size_t)c.tail * 16] >> 8) - 1;
    if (nx >= 0 && nx < a.P) { c.tail = nx; c.fill = (int)(a.pool[(size_t)nx * 16] & 0xFFu); }
  }
  if (c.tail < 0 || c.fill == XSLOT) {             // take a new block from the pool
    const int nb = atomicAdd(a.pool_cnt, 1);
    if (nb >= a.P) { atomicExch(a.pool_cnt + 1, 1); return; }   // exhausted: flagged for the host, never silent
    a.pool[(size_t)nb * 16] = 0u;
    if (c.tail < 0) c.head = nb;
    else a.pool[(size_t)c.tail * 16] = (a.pool[(size_t)c.tail * 16] & 0xFFu) | ((uint32_t)(nb + 1) << 8);
    c.tail = nb;
    c.fill = 0;
  }
  a.pool[(size_t)c.tail * 16 + 1 + c.fill] = e;
  ++c.fill;
  a.pool[(size_t)c.tail * 16] = (a.pool[(size_t)c.tail * 16] & ~0xFFu) | (uint32_t)c.fill;
}

// Encodes nrow consecutive rows (r0 ..) of one record, whose values are pairs[i] (columns 2 lane, 2 lane + 1 of row i),
// into the 1600-byte unit: staged in `rec` (shared memory, one per warp), written back to `grec` as 100 16-byte stores.
__device__ __forceinline__ void append_rows(const AppendArgs& a, uint8_t* const grec, uint8_t* const rec, const int r0,
                                            const int nrow, const uint32_t (&pairs)[PAGE], const int lane) {
  uint32_t* const hdr = reinterpret_cast<uint32_t*>(rec + REC);
  uint32_t* const slots = hdr + 1;
  EscCursor c;
  if (r0 == 0) {                                                  // row 0: the page starts over
    int keep = -1;
    if (a.reuse) {
      const uint32_t old = *reinterpret_cast<const volatile uint32_t*>(grec + REC);
      if ((old & 16u) && (int)(old >> 8) < a.P) keep = (int)(old >> 8);
    }
    for (int i = lane; i < RKV / 16; i += 32) reinterpret_cast<uint4*>(rec)[i] = make_uint4(0, 0, 0, 0);
    if (keep >= 0 && lane == 0) {                                 // empty the kept chain, links stay
      int b = keep;
      for (int hops = 0; b >= 0 && b < a.P && hops < 4096; ++hops) {
        const uint32_t w0 = a.pool[(size_t)b * 16];
        a.pool[(size_t)b * 16] = w0 & ~0xFFu;
        b = (int)(w0 >> 8) - 1;
      }
    }
    c.cnt = 0;
    c.head = keep;
  } else {                                                        // continue a page: bring the unit in
    for (int i = lane; i < RKV / 16; i += 32) reinterpret_cast<uint4*>(rec)[i] = reinterpret_cast<const uint4*>(grec)[i];
    __syncwarp();
    const uint32_t old = *hdr;
    c.cnt = (int)(old & 15u);
    c.head = (old & 16u) ? (int)(old >> 8) : -1;
  }
  __syncwarp();
  c.tail = -1;
  c.fill = 0;
#pragma unroll
  for (int i = 0; i < PAGE; ++i) {
    if (i >= nrow) break;
    const int r = r0 + i;
    const uint32_t pr = pairs[i];
    const uint32_t b0 = pr & 0xFFFFu, b1 = pr >> 16;
    const int e0 = (int)((b0 >> 7) & 0xFFu), e1 = (int)((b1 >> 7) & 0xFFu);
    int E = max(e0, e1);
#pragma unroll
    for (int o = 16; o; o >>= 1) E = max(E, __shfl_xor_sync(FULL, E, o));
    const int d0 = E - e0, d1 = E - e1;
    const bool x0 = d0 > 14, x1 = d1 > 14;
    const uint32_t leaf0 = ((x0 ? 0u : (b0 & 0x7Fu)) << 1) | (x1 ? 0u : (b1 >> 15));
    const uint32_t leaf1 = ((x1 ? 0u : (b1 & 0x7Fu)) << 1) | (x0 ? 0u : (b0 >> 15));
    *reinterpret_cast<uint16_t*>(rec + leaf_pair_off(r, lane)) = (uint16_t)(leaf0 | (leaf1 << 8));
    uint16_t* const sp = reinterpret_cast<uint16_t*>(rec + state_pair_off(r, lane));
    const int sh = 4 * (r >> 3);
    const uint32_t q0 = x0 ? 15u : (uint32_t)d0, q1 = x1 ? 15u : (uint32_t)d1;
    const uint32_t keepmask = ~((0xFu << sh) | (0xFu << (8 + sh)));
    *sp = (uint16_t)((*sp & keepmask) | (q0 << sh) | (q1 << (8 + sh)));
    if (lane == 0) rec[1536 + 2 * (r & 7) + (r >> 3)] = (uint8_t)E;
    const unsigned m0 = __ballot_sync(FULL, x0), m1 = __ballot_sync(FULL, x1);
    const int tot = __popc(m0) + __popc(m1);
    if (tot == 0) continue;
    const uint32_t en0 = (b0 << 16) | ((uint32_t)r << 6) | (uint32_t)(2 * lane);
    const uint32_t en1 = (b1 << 16) | ((uint32_t)r << 6) | (uint32_t)(2 * lane + 1);
    if (c.cnt + tot <= NSLOT) {                                   // all fit in the record: column order
      const unsigned below = (1u << lane) - 1u;
      const int at = c.cnt + __popc(m0 & below) + __popc(m1 & below);
      if (x0) slots[at] = en0;
      if (x1) slots[at + (x0 ? 1 : 0)] = en1;
      c.cnt += tot;
    } else {                                                      // lane 0 places them one by one
      for (int sl = 0; sl < 32; ++sl) {
        const uint32_t f0 = __shfl_sync(FULL, en0, sl), f1 = __shfl_sync(FULL, en1, sl);
        if (lane == 0) {
          if ((m0 >> sl) & 1u) chain_put(a, c, slots, f0);
          if ((m1 >> sl) & 1u) chain_put(a, c, slots, f1);
        }
      }
      c.cnt = __shfl_sync(FULL, c.cnt, 0);
      c.head = __shfl_sync(FULL, c.head, 0);
      c.tail = __shfl_sync(FULL, c.tail, 0);
      c.fill = __shfl_sync(FULL, c.fill, 0);
    }
  }
  if (lane == 0) *hdr = (uint32_t)c.cnt | (c.head >= 0 ? (16u | ((uint32_t)c.head << 8)) : 0u);
  __syncwarp();
  for (int i = lane; i < RKV / 16; i += 32) reinterpret_cast<uint4*>(grec)[i] = reinterpret_cast<const uint4*>(rec)[i];
  __syncwarp();                                                   // the staging unit is reused by the next segment
}

// One warp per (token, head, K/V, half); only the warp of a segment's first token works: a segment is a run of
// consecutive slots inside one page, and its warp owns the record for the whole launch (rows g and g+8 share state
// bytes, and the header is read-modify-write).  Semantics of statetree/csrc/kvcache.cu:62-192.
// The warp edits the 1600-byte unit in shared memory: the segment's rows are fetched up front (independent loads),
// encoded row by row with shared-memory byte stores, and the unit goes back to the page as 100 16-byte stores.
__global__ void __launch_bounds__(256) kv_append_kernel(const AppendArgs a) {
  __shared__ __align__(16) uint8_t s_unit[8][RKV];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int units = a.H * 4;
  const long long grp = w / units;                                // a.gsz consecutive tokens of the call per warp
  if (grp * a.gsz >= a.N) return;
  const int u = (int)(w % units), h = u >> 2, kvi = (u >> 1) & 1, half = u & 1;
  const long long n_end = min((long long)a.N, (grp + 1) * a.gsz);
  for (long long n = grp * a.gsz; n < n_end; ++n) {
  const long long s0 = a.slot[n];
  if (s0 < 0) continue;
  const long long blk = s0 / PAGE;
  if (blk >= a.nblocks) continue;                                 // outside the cache: dropped, no write
  if (n > 0) {
    const long long sp = a.slot[n - 1];
    if (sp >= 0 && sp + 1 == s0 && sp / PAGE == blk) continue;    // continues the previous token's segment
  }
  uint8_t* const grec = a.kv + unit_off(blk, a.H, h, kvi, half);
  uint8_t* const rec = s_unit[threadIdx.x >> 5];
  const int r0 = (int)(s0 % PAGE);
  // rows of this segment: consecutive slots that stay inside the page
  int nrow = 1;
  while (nrow < PAGE - r0 && n + nrow < a.N && a.slot[n + nrow] == s0 + nrow) ++nrow;
  // fetch every row's pair of values now (independent loads), encode afterwards
  uint32_t pairs[PAGE];
#pragma unroll
  for (int i = 0; i < PAGE; ++i) {
    if (i < nrow) {
      const uint16_t* src = (kvi ? a.V + (n + i) * a.vs : a.K + (n + i) * a.ks) + h * HD + half * 64;
      pairs[i] = *reinterpret_cast<const uint32_t*>(src + 2 * lane);
    }
  }
  append_rows(a, grec, rec, r0, nrow, pairs, lane);
  }
}

// Decode step, one new token per sequence: per-head q/k RMSNorm + rotary embedding and the KV append in one launch.
// Warps [0, B * hq) normalise and rotate a query head into q_out (the arithmetic of qk_norm_rope_kernel, operation for
// operation); the B * hkv * 4 warps after them each own one (sequence, KV head, K/V, half) record as in
// kv_append_kernel, and the K warps compute their 64 normalised, rotated values themselves instead of reading them
// back from a buffer another kernel wrote.  The pages are bit-identical to norm/rope followed by append.
struct RopeArgs {
  const uint16_t* qkv; long long row_stride;
  const uint16_t* wq; const uint16_t* wk;
  const float* cos_t; const float* sin_t;
  const long long* pos; long long max_pos;
  uint16_t* q_out;
  int B, hq;
  float eps;
};
__device__ __forceinline__ float kv_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(256) rope_append_kernel(const RopeArgs r, const AppendArgs a) {
  __shared__ __align__(16) uint8_t s_unit[8][RKV];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long nq = (long long)r.B * r.hq;
  long long p = r.pos[0];
  p = p < 0 ? 0 : (p >= r.max_pos ? r.max_pos - 1 : p);
  if (w < nq) {                                                     // ---- a query head
    const int b = (int)(w / r.hq), h = (int)(w % r.hq);
    const uint16_t* src = r.qkv + (size_t)b * r.row_stride + (size_t)h * HD + 4 * lane;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    const float ss = kv_warp_sum(sumsq4(x0.x, x0.y, x1.x, x1.y));
    const float rn = rsqrtf(__fmaf_rn(ss, 1.f / 128.f, r.eps));
    const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(r.wq + 4 * lane));
    const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(r.wq + 4 * lane + 2));
    const float n00 = bf16_round(bf16_round(x0.x * rn) * g0.x), n01 = bf16_round(bf16_round(x0.y * rn) * g0.y);
    const float n10 = bf16_round(bf16_round(x1.x * rn) * g1.x), n11 = bf16_round(bf16_round(x1.y * rn) * g1.y);
    const float c0 = r.cos_t[p * 64 + 2 * lane], s0 = r.sin_t[p * 64 + 2 * lane];
    const float c1 = r.cos_t[p * 64 + 2 * lane + 1], s1 = r.sin_t[p * 64 + 2 * lane + 1];
    uint2 o;
    o.x = rope_pair(n00, n01, c0, s0);
    o.y = rope_pair(n10, n11, c1, s1);
    *reinterpret_cast<uint2*>(r.q_out + ((size_t)b * r.hq + h) * HD + 4 * lane) = o;
    return;
  }
  const long long u = w - nq;                                        // ---- a record of the new token
  const int units = a.H * 4;
  if (u >= (long long)r.B * units) return;
  const int b = (int)(u / units), uu = (int)(u % units), h = uu >> 2, kvi = (uu >> 1) & 1, half = uu & 1;
  const long long s0 = a.slot[b];
  if (s0 < 0) return;
  const long long blk = s0 / PAGE;
  if (blk >= a.nblocks) return;
  uint32_t pairs[PAGE];
  if (kvi) {
    const uint16_t* src = r.qkv + (size_t)b * r.row_stride + (size_t)(r.hq + a.H + h) * HD + half * 64;
    pairs[0] = *reinterpret_cast<const uint32_t*>(src + 2 * lane);
  } else {
    const uint16_t* src = r.qkv + (size_t)b * r.row_stride + (size_t)(r.hq + h) * HD;
    const uint2 raw = *reinterpret_cast<const uint2*>(src + 4 * lane);         // the whole head, for the norm
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    const float ss = kv_warp_sum(sumsq4(x0.x, x0.y, x1.x, x1.y));
    const float rn = rsqrtf(__fmaf_rn(ss, 1.f / 128.f, r.eps));
    const int d0 = half * 64 + 2 * lane;                                        // this lane's pair of the record row
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + d0));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(r.wk + d0));
    const float n0 = bf16_round(bf16_round(v.x * rn) * g.x), n1 = bf16_round(bf16_round(v.y * rn) * g.y);
    const float c = r.cos_t[p * 64 + (d0 >> 1)], sn = r.sin_t[p * 64 + (d0 >> 1)];
    pairs[0] = rope_pair(n0, n1, c, sn);
  }
  append_rows(a, a.kv + unit_off(blk, a.H, h, kvi, half), s_unit[threadIdx.x >> 5], (int)(s0 % PAGE), 1, pairs, lane);
}

// ------------------------------------------------------------------------------------------------ record decode
// fragments of one KV unit (record + in-record slots + pool chain); `rec` may be shared or global memory
__device__ __forceinline__ void apply_kv_escapes(uint32_t (&A)[4][4], const uint8_t* rec, const uint32_t* pool, int P,
                                                 int lane) {
  const uint32_t head = *reinterpret_cast<const uint32_t*>(rec + REC);
  if ((head & 31u) == 0u) return;
  const int cnt = min((int)(head & 15u), NSLOT);
  const uint32_t* sl = reinterpret_cast<const uint32_t*>(rec + REC + 4);
  for (int i = 0; i < cnt; ++i) {
    const uint32_t e = sl[i];
    patch_frag(A, (int)((e >> 6) & 15u), (int)(e & 63u), e >> 16, lane);
  }
  if (head & 16u) {
    int b = (int)(head >> 8);
    for (int hops = 0; b >= 0 && b < P && hops < 4096; ++hops) {
      const uint32_t w0 = __ldg(pool + (size_t)b * 16);
      const int n = min((int)(w0 & 0xFFu), XSLOT);
      for (int i = 0; i < n; ++i) {
        const uint32_t e = __ldg(pool + (size_t)b * 16 + 1 + i);
        patch_frag(A, (int)((e >> 6) & 15u), (int)(e & 63u), e >> 16, lane);
      }
      b = (int)(w0 >> 8) - 1;
    }
  }
}

// listed pages (blocks != nullptr) or every page -> dense BF16 [n, 16, H, 128]; one warp per unit
__global__ void __launch_bounds__(256) kv_dequant_kernel(const uint8_t* __restrict__ kv, long long nblocks, int H,
                                                         const uint32_t* __restrict__ pool, int P,
                                                         const int* __restrict__ blocks, long long n,
                                                         uint16_t* __restrict__ Kd, uint16_t* __restrict__ Vd) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= n * H * 4) return;
  const int half = (int)(w & 1), kvi = (int)((w >> 1) & 1);
  const long long ih = w >> 2;
  const int h = (int)(ih % H);
  const long long i = ih / H;
  const long long blk = blocks ? (long long)blocks[i] : i;
  uint32_t A[4][4];
  if (blk >= 0 && blk < nblocks) {
    const uint8_t* rec = kv + unit_off(blk, H, h, kvi, half);
    decode_frag(load_rec_global(rec, lane), A);
    apply_kv_escapes(A, rec, pool, P, lane);
  } else {
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int q = 0; q < 4; ++q) A[s][q] = 0u;
  }
  uint16_t* out = (kvi ? Vd : Kd) + ((size_t)i * PAGE * H + h) * HD + half * 64;
#pragma unroll
  for (int s = 0; s < 4; ++s)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int row = g + 8 * (q & 1), col = 16 * s + 8 * (q >> 1) + 2 * t;
      *reinterpret_cast<uint32_t*>(out + (size_t)row * H * HD + col) = A[s][q];
    }
}

// ------------------------------------------------------------------------------------------------ attention
struct AttnArgs {
  const uint16_t* q; long long qs;
  const uint8_t* kv; long long nblocks;
  const uint32_t* pool; int P;
  const int* bt; long long bts;
  const int* lens; const int* starts;
  uint16_t* out; long long os;
  float* wo; float* wml;
  float sl2;
  int Hkv, S, minpps;
  int* status;
};

constexpr int PAGE_BYTES = 4 * RKV;

// ATT_NW warps per CTA, each with ATT_STG pages in flight.  The per-warp partial results reuse the ring once the
// loop is over, so a CTA needs only the ring and its barriers (4 warps x 3 stages = 75 KB measured slightly faster
// than 8 warps x 2 stages = 100 KB; both leave two CTAs per SM).
template <int G, int ATT_NW, int ATT_STG>
__global__ void __launch_bounds__(ATT_NW * 32) kv_attn_kernel(const AttnArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;                                                         // [NW][STG][6400]
  float* red = reinterpret_cast<float*>(smem);                                  // [NW][G * 128 + 2 G], after the loop
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ATT_NW * ATT_STG * PAGE_BYTES);   // [NW][STG]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int j = blockIdx.x % a.S, bh = blockIdx.x / a.S;
  const int h = bh % a.Hkv, b = bh / a.Hkv, Hq = a.Hkv * G;
  pdl_wait();                               // queries, lengths and the pages of this step come from earlier kernels
  pdl_launch_dependents();
  const int len = a.lens[b], st0 = a.starts ? a.starts[b] : 0;
  const int pfirst = st0 / PAGE;
  const int npg = len > st0 ? (int)min((long long)(len + PAGE - 1) / PAGE, a.bts) : 0;
  const int pps = max(a.minpps, (npg - pfirst + a.S - 1) / a.S);
  const int p0 = pfirst + j * pps, p1 = min(npg, p0 + pps);
  const int mine = p1 > p0 + warp ? (p1 - p0 - warp + ATT_NW - 1) / ATT_NW : 0;   // pages of this warp

  uint64_t* mybar = bars + warp * ATT_STG;
  uint8_t* myring = ring + (size_t)warp * ATT_STG * PAGE_BYTES;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < ATT_STG; ++s) mbar_init(mybar + s, 1);
    fence_barrier_init();
  }
  __syncwarp();
  uint64_t pol = 0;
  auto issue = [&](int i) {                        // lane 0: page i of this warp -> stage i % STG
    const int p = p0 + warp + i * ATT_NW;
    long long blk = a.bt[(size_t)b * a.bts + p];
    blk = blk < 0 ? 0 : (blk >= a.nblocks ? a.nblocks - 1 : blk);
    const int s = i % ATT_STG;
    mbar_expect_tx(mybar + s, PAGE_BYTES);
    bulk_g2s(myring + (size_t)s * PAGE_BYTES, a.kv + ((size_t)blk * a.Hkv + h) * PAGE_BYTES, PAGE_BYTES, mybar + s, pol);
  };
  if (lane == 0) {
    pol = policy_evict_first();
    for (int i = 0; i < min(mine, ATT_STG); ++i) issue(i);
  }

  uint32_t qa[8][2];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    if (g < G) {
      const uint16_t* qp = a.q + (size_t)b * a.qs + (size_t)(h * G + g) * HD;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 2 * t);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 8 + 2 * t);
    } else {
      qa[ks][0] = qa[ks][1] = 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m = -INFINITY, l = 0.f;
  int dead_at = -1;

  for (int i = 0; i < mine; ++i) {
    const int p = p0 + warp + i * ATT_NW, s = i % ATT_STG;
    if (!mbar_wait(mybar + s, (uint32_t)(i / ATT_STG) & 1u)) {
      if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
      dead_at = i;
      break;
    }
    const uint8_t* pg = myring + (size_t)s * PAGE_BYTES;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t A[4][4];
      const uint8_t* rec = pg + hf * RKV;
      decode_frag(load_rec_shared(rec, lane), A);
      apply_kv_escapes(A, rec, a.pool, a.P, lane);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        mma_bf16_r(s0, qa[hf * 4 + ks][0], 0u, qa[hf * 4 + ks][1], 0u, A[ks][0], A[ks][2]);   // tokens 0..7
        mma_bf16_r(s1, qa[hf * 4 + ks][0], 0u, qa[hf * 4 + ks][1], 0u, A[ks][1], A[ks][3]);   // tokens 8..15
      }
    }
    const int hiv = len - p * PAGE, lov = st0 - p * PAGE;          // valid rows of this page: [lov, hiv)
    const float x0 = (2 * t < hiv && 2 * t >= lov) ? s0[0] * a.sl2 : -INFINITY;
    const float x1 = (2 * t + 1 < hiv && 2 * t + 1 >= lov) ? s0[1] * a.sl2 : -INFINITY;
    const float x2 = (8 + 2 * t < hiv && 8 + 2 * t >= lov) ? s1[0] * a.sl2 : -INFINITY;
    const float x3 = (9 + 2 * t < hiv && 9 + 2 * t >= lov) ? s1[1] * a.sl2 : -INFINITY;
    float mp = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
    mp = fmaxf(mp, __shfl_xor_sync(FULL, mp, 1));
    mp = fmaxf(mp, __shfl_xor_sync(FULL, mp, 2));
    const float mn = fmaxf(m, mp);                                // finite: every page here holds a valid token
    const float al = exp2f(m - mn);
    const float e0 = exp2f(x0 - mn), e1 = exp2f(x1 - mn), e2 = exp2f(x2 - mn), e3 = exp2f(x3 - mn);
    float ps = (e0 + e1) + (e2 + e3);
    ps += __shfl_xor_sync(FULL, ps, 1);
    ps += __shfl_xor_sync(FULL, ps, 2);
    l = l * al + ps;
    m = mn;
    if (__any_sync(FULL, al != 1.f)) {                             // after the first pages the maxima rarely move
#pragma unroll
      for (int n = 0; n < 16; ++n) { o[n][0] *= al; o[n][1] *= al; }
    }
    // P = high BF16 part + BF16 residual
    const __nv_bfloat16 h0 = __float2bfloat16_rn(e0), h1 = __float2bfloat16_rn(e1), h2 = __float2bfloat16_rn(e2),
                        h3 = __float2bfloat16_rn(e3);
    const uint32_t ph0 = pack_bf16(e0, e1), ph2 = pack_bf16(e2, e3);
    const uint32_t pl0 = pack_bf16(e0 - __bfloat162float(h0), e1 - __bfloat162float(h1));
    const uint32_t pl2 = pack_bf16(e2 - __bfloat162float(h2), e3 - __bfloat162float(h3));
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t A[4][4];
      const uint8_t* rec = pg + (2 + hf) * RKV;
      decode_frag(load_rec_shared(rec, lane), A);
      apply_kv_escapes(A, rec, a.pool, a.P, lane);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const int nt = 2 * (4 * hf + ks);
        const uint32_t v0 = movmatrix_t(A[ks][0]), v1 = movmatrix_t(A[ks][1]);
        const uint32_t v2 = movmatrix_t(A[ks][2]), v3 = movmatrix_t(A[ks][3]);
        mma_bf16_r(o[nt], ph0, 0u, ph2, 0u, v0, v1);               // dims 16 ks .. + 7
        mma_bf16_r(o[nt], pl0, 0u, pl2, 0u, v0, v1);
        mma_bf16_r(o[nt + 1], ph0, 0u, ph2, 0u, v2, v3);           // dims 16 ks + 8 .. + 15
        mma_bf16_r(o[nt + 1], pl0, 0u, pl2, 0u, v2, v3);
      }
    }
    __syncwarp();                                                  // every lane is done with this stage
    if (lane == 0 && i + ATT_STG < mine) {
      fence_proxy_async();
      issue(i + ATT_STG);
    }
  }
  if (dead_at >= 0) {                                              // drain this warp's copies still in flight
    for (int k = dead_at; k < min(mine, dead_at + ATT_STG); ++k)
      (void)mbar_wait(mybar + k % ATT_STG, (uint32_t)(k / ATT_STG) & 1u);
    m = -INFINITY; l = 0.f;
  }

  // merge the warps of the CTA (every warp is done with the ring: its partial result goes where the pages were)
  __syncthreads();
  constexpr int WS = G * 128 + 2 * G;
  static_assert(ATT_NW * WS * 4 <= ATT_NW * ATT_STG * PAGE_BYTES, "partials must fit the ring");
  float* so = red + warp * WS;
  if (g < G) {
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      so[g * 128 + n * 8 + 2 * t] = o[n][0];
      so[g * 128 + n * 8 + 2 * t + 1] = o[n][1];
    }
    if (t == 0) { so[G * 128 + 2 * g] = m; so[G * 128 + 2 * g + 1] = l; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * 128; i += ATT_NW * 32) {
    const int r = i >> 7, d = i & 127;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_NW; ++w) M = fmaxf(M, red[w * WS + G * 128 + 2 * r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_NW; ++w) {
      const float mw = red[w * WS + G * 128 + 2 * r];
      if (mw == -INFINITY) continue;
      const float f = exp2f(mw - M);
      L += f * red[w * WS + G * 128 + 2 * r + 1];
      O += f * red[w * WS + r * 128 + d];
    }
    if (a.S == 1) {
      const __nv_bfloat16 v = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
      a.out[(size_t)b * a.os + (size_t)(h * G + r) * HD + d] = *reinterpret_cast<const uint16_t*>(&v);
    } else {
      const size_t ix = (size_t)(b * Hq + h * G + r) * a.S + j;
      a.wo[ix * HD + d] = O;
      if (d == 0) { a.wml[ix * 2] = M; a.wml[ix * 2 + 1] = L; }
    }
  }
}

__global__ void __launch_bounds__(128) kv_merge_kernel(const float* __restrict__ wo, const float* __restrict__ wml,
                                                       uint16_t* __restrict__ out, long long os, int Hq, int S) {
  const int bq = blockIdx.x, d = threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  float M = -INFINITY;
  for (int j = 0; j < S; ++j) M = fmaxf(M, wml[((size_t)bq * S + j) * 2]);
  float L = 0.f, O = 0.f;
  for (int j = 0; j < S; ++j) {
    const float mj = wml[((size_t)bq * S + j) * 2];
    if (mj == -INFINITY) continue;
    const float f = exp2f(mj - M);
    L += f * wml[((size_t)bq * S + j) * 2 + 1];
    O += f * wo[((size_t)bq * S + j) * HD + d];
  }
  const __nv_bfloat16 v = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
  out[(size_t)(bq / Hq) * os + (size_t)(bq % Hq) * HD + d] = *reinterpret_cast<const uint16_t*>(&v);
}

template <int G, int NW, int STG>
int attn_launch_cfg(const AttnArgs& a, int B, cudaStream_t st) {
  const int smem = NW * STG * PAGE_BYTES + NW * STG * 8;
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    if (int e = st::cuda_fail(cudaFuncSetAttribute(kv_attn_kernel<G, NW, STG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   smem), "st_kv_attn: shared memory attribute"))
      return e;
    set[dev] = true;
  }
  return st::launch("st_kv_attn launch", kv_attn_kernel<G, NW, STG>, dim3((unsigned)(B * a.Hkv * a.S)), dim3(NW * 32),
                    (size_t)smem, st, a);
}

template <int G>
int attn_launch(const AttnArgs& a, int B, cudaStream_t st) {
  // STATETREE_ATTN_CFG (tuning aid): 2 = 4 warps x 2 page stages, three CTAs per SM (default: the kernel is bound by
  // instruction latency, and twelve warps per SM hide more of it than eight with deeper rings; 4.5 TB/s at batch 32 x 4K
  // against 4.0), 1 = 4 warps x 3 stages, 0 = 8 warps x 2
  static int cfg = -1;
  if (cfg < 0) {
    const char* v = getenv("STATETREE_ATTN_CFG");
    cfg = v ? atoi(v) : 2;
  }
  return cfg == 1 ? attn_launch_cfg<G, 4, 3>(a, B, st) : (cfg == 2 ? attn_launch_cfg<G, 4, 2>(a, B, st) : attn_launch_cfg<G, 8, 2>(a, B, st));
}
}  // namespace

extern "C" int64_t st_kv_page_bytes(int64_t H) { return H * 4 * st::RKV; }

extern "C" int st_kv_append(const void* K, const void* V, int64_t ks, int64_t vs, const int64_t* slot, int64_t N,
                            int64_t H, void* kv, int64_t nblocks, uint32_t* pool, int64_t P, int32_t* pool_cnt,
                            int reuse, void* stream) {
  ST_REQUIRE(N >= 0 && H > 0 && nblocks >= 0 && P >= 0, "st_kv_append: negative size");
  if (N == 0) return 0;
  ST_REQUIRE(K && V && slot && kv && pool && pool_cnt, "st_kv_append: null pointer");
  ST_REQUIRE(ks >= H * 128 && vs >= H * 128 && ks % 2 == 0 && vs % 2 == 0,
             "st_kv_append: K / V must be [N, H, 128] with heads contiguous (token stride >= H * 128)");
  ST_REQUIRE(((uintptr_t)K & 3u) == 0 && ((uintptr_t)V & 3u) == 0 && st::aligned16(kv), "st_kv_append: alignment");
  ST_REQUIRE(N * H * 4 < (1ll << 34) && P < (1ll << 23), "st_kv_append: too large");
  AppendArgs a;
  a.K = (const uint16_t*)K; a.V = (const uint16_t*)V; a.ks = ks; a.vs = vs;
  a.slot = (const long long*)slot; a.kv = (uint8_t*)kv; a.pool = pool; a.pool_cnt = pool_cnt;
  a.nblocks = nblocks; a.N = (int)N; a.H = (int)H; a.P = (int)P; a.reuse = reuse ? 1 : 0;
  // long calls are mostly whole pages of consecutive tokens: one warp per 16 tokens finds (typically) one segment
  // and the grid shrinks 16-fold; short calls (decode steps) keep one warp per token
  a.gsz = N >= 1024 ? 16 : 1;
  const long long warps = ((N + a.gsz - 1) / a.gsz) * H * 4;
  return st::launch("st_kv_append launch", kv_append_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0,
                    (cudaStream_t)stream, a);
}

extern "C" int st_rope_kv_append(const void* qkv, int64_t row_stride, const void* wq, const void* wk, const float* cos_t,
                                 const float* sin_t, const int64_t* pos, int64_t max_pos, void* q_out, int64_t B,
                                 int64_t hq, int64_t hkv, double eps, const int64_t* slot, void* kv, int64_t nblocks,
                                 uint32_t* pool, int64_t P, int32_t* pool_cnt, void* stream) {
  ST_REQUIRE(B >= 0 && hq > 0 && hkv > 0 && max_pos > 0 && nblocks >= 0 && P >= 0, "st_rope_kv_append: sizes");
  if (B == 0) return 0;
  ST_REQUIRE(qkv && wq && wk && cos_t && sin_t && pos && q_out && slot && kv && pool && pool_cnt,
             "st_rope_kv_append: null pointer");
  ST_REQUIRE(((uintptr_t)qkv & 7u) == 0 && row_stride % 4 == 0 && row_stride >= (hq + 2 * hkv) * 128 &&
                 ((uintptr_t)q_out & 7u) == 0 && ((uintptr_t)wq & 3u) == 0 && ((uintptr_t)wk & 3u) == 0 && st::aligned16(kv),
             "st_rope_kv_append: alignment / row stride");
  ST_REQUIRE(B * (hq + hkv * 4) < (1ll << 31) && P < (1ll << 23), "st_rope_kv_append: too large");
  RopeArgs r;
  r.qkv = (const uint16_t*)qkv; r.row_stride = row_stride; r.wq = (const uint16_t*)wq; r.wk = (const uint16_t*)wk;
  r.cos_t = cos_t; r.sin_t = sin_t; r.pos = (const long long*)pos; r.max_pos = max_pos; r.q_out = (uint16_t*)q_out;
  r.B = (int)B; r.hq = (int)hq; r.eps = (float)eps;
  AppendArgs a;
  a.K = nullptr; a.V = nullptr; a.ks = 0; a.vs = 0;
  a.slot = (const long long*)slot; a.kv = (uint8_t*)kv; a.pool = pool; a.pool_cnt = pool_cnt;
  a.nblocks = nblocks; a.N = (int)B; a.H = (int)hkv; a.P = (int)P; a.reuse = 0; a.gsz = 1;
  const long long warps = B * (hq + hkv * 4);
  return st::launch("st_rope_kv_append launch", rope_append_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0,
                    (cudaStream_t)stream, r, a);
}

extern "C" int st_kv_dequant_blocks(const void* kv, int64_t nblocks, int64_t H, const uint32_t* pool, int64_t P,
                                    const int32_t* blocks, int64_t n, void* Kd, void* Vd, void* stream) {
  ST_REQUIRE(n >= 0 && H > 0 && nblocks >= 0, "st_kv_dequant_blocks: negative size");
  if (n == 0) return 0;
  ST_REQUIRE(kv && pool && Kd && Vd, "st_kv_dequant_blocks: null pointer");
  ST_REQUIRE(st::aligned16(kv) && ((uintptr_t)Kd & 3u) == 0 && ((uintptr_t)Vd & 3u) == 0, "st_kv_dequant_blocks: alignment");
  const long long nw = n * H * 4;
  kv_dequant_kernel<<<(unsigned)((nw + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)kv, nblocks, (int)H, pool, (int)P, blocks, n, (uint16_t*)Kd, (uint16_t*)Vd);
  ST_LAUNCH_CHECK("st_kv_dequant launch");
  return 0;
}

extern "C" int st_kv_dequant(const void* kv, int64_t nblocks, int64_t H, const uint32_t* pool, int64_t P, void* Kd,
                             void* Vd, void* stream) {
  return st_kv_dequant_blocks(kv, nblocks, H, pool, P, nullptr, nblocks, Kd, Vd, stream);
}

extern "C" int st_kv_attn(const void* q, int64_t qs, int64_t B, int64_t Hq, const void* kv, int64_t nblocks,
                          int64_t Hkv, const uint32_t* pool, int64_t P, const int32_t* bt, int64_t bts,
                          const int32_t* lens, const int32_t* starts, void* out, int64_t os, float* wo, float* wml,
                          double scale, int64_t S, int64_t minpps, void* stream) {
  ST_REQUIRE(B >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "st_kv_attn: heads");
  ST_REQUIRE(S >= 1 && S <= 1024, "st_kv_attn: splits must be in [1, 1024]");
  if (B == 0) return 0;
  ST_REQUIRE(q && kv && pool && bt && lens && out, "st_kv_attn: null pointer");
  ST_REQUIRE(S == 1 || (wo && wml), "st_kv_attn: split workspace (wo, wml) missing");
  ST_REQUIRE(nblocks > 0, "st_kv_attn: empty cache");
  ST_REQUIRE(((uintptr_t)q & 3u) == 0 && qs % 2 == 0 && st::aligned16(kv), "st_kv_attn: alignment");
  ST_REQUIRE(B * Hkv * S < (1ll << 31), "st_kv_attn: grid too large");
  AttnArgs a;
  a.q = (const uint16_t*)q; a.qs = qs; a.kv = (const uint8_t*)kv; a.nblocks = nblocks; a.pool = pool; a.P = (int)P;
  a.bt = bt; a.bts = bts; a.lens = lens; a.starts = starts; a.out = (uint16_t*)out; a.os = os; a.wo = wo; a.wml = wml;
  a.sl2 = (float)(scale * 1.4426950408889634);
  a.Hkv = (int)Hkv; a.S = (int)S; a.minpps = (int)(minpps < 1 ? 1 : minpps);
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "st_kv_attn: no device status word");
  cudaStream_t st_ = (cudaStream_t)stream;
  int e = 0;
  switch (Hq / Hkv) {
    case 1: e = attn_launch<1>(a, (int)B, st_); break;
    case 2: e = attn_launch<2>(a, (int)B, st_); break;
    case 4: e = attn_launch<4>(a, (int)B, st_); break;
    case 8: e = attn_launch<8>(a, (int)B, st_); break;
    default: return st::fail("st_kv_attn: query heads per KV head must be 1, 2, 4 or 8 (got %lld)", (long long)(Hq / Hkv));
  }
  if (e) return e;
  if (S > 1)
    return st::launch("st_kv_attn merge launch", kv_merge_kernel, dim3((unsigned)(B * Hq)), dim3(128), 0, st_,
                      (const float*)wo, (const float*)wml, (uint16_t*)out, (long long)os, (int)Hq, (int)S);
  return 0;
}
