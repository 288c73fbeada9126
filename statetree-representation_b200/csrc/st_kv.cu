// Compressed KV pages on sm_100a: append (page encode), dequant, and split decode attention straight over the pages.
//
// Page layout (frozen by the reference, statetree/csrc/kvcache.cu:1-14): uint8 [blocks, H, 2 (K/V), 2 (dim half), 1600];
// one 1600-byte unit = a 1552-byte record of 16 tokens x 64 dims (token = row) + a header word + 11 escape slots
// (bits << 16 | row << 6 | col); further escapes chain through 16-word blocks of a pool.
//
// The attention kernel's design is described above kv_attn_kernel.
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

// ---- escapes of a record.  A value whose exponent lies more than 14 below its row's largest cannot be held by the
// 4-bit state; its exact bits go to an entry (bits << 16 | row << 6 | col).  The first 11 entries of a record live in
// the unit itself, the rest in a chain of 16-word pool blocks (word 0 = entries used | (next block + 1) << 8, then up to
// 15 entries); the unit's header word is  entries in the unit | 16 if a chain exists | first block << 8.

// lane 0's view of a record's chain while it appends to it
struct ChainTail {
  uint32_t* pool;
  int* pool_cnt;
  int P;
  int first;      // first block of the chain, -1 = the record has none
  int blk;        // block being filled, -1 = not looked for yet
  int used;       // entries in blk

  __device__ uint32_t& word0(int b) const { return pool[(size_t)b * 16]; }
  __device__ static int next_of(uint32_t w0) { return (int)(w0 >> 8) - 1; }

  // an existing chain is entered at its first block that still has room (blocks before it are full)
  __device__ void locate() {
    blk = first;
    for (int hops = 0; hops < 4096; ++hops) {
      const uint32_t w0 = word0(blk);
      used = (int)(w0 & 0xFFu);
      const int nx = next_of(w0);
      if (used < XSLOT || nx < 0 || nx >= P) return;
      blk = nx;
    }
  }
  // the block is full (or there is none): move to the next linked block (a recycled chain keeps its links) or take a
  // fresh block from the pool and link it; false when the pool is exhausted (flagged for the host)
  __device__ bool advance() {
    if (blk >= 0) {
      const int nx = next_of(word0(blk));
      if (nx >= 0 && nx < P) {
        blk = nx;
        used = (int)(word0(nx) & 0xFFu);
        if (used < XSLOT) return true;
      }
    }
    const int fresh = atomicAdd(pool_cnt, 1);
    if (fresh >= P) {
      atomicExch(pool_cnt + 1, 1);
      return false;
    }
    word0(fresh) = 0u;
    if (blk < 0) first = fresh;
    else word0(blk) = (word0(blk) & 0xFFu) | ((uint32_t)(fresh + 1) << 8);
    blk = fresh;
    used = 0;
    return true;
  }
  __device__ void push(uint32_t entry) {
    if (first >= 0 && blk < 0) locate();
    if ((blk < 0 || used >= XSLOT) && !advance()) return;
    pool[(size_t)blk * 16 + 1 + used] = entry;
    ++used;
    word0(blk) = (word0(blk) & ~0xFFu) | (uint32_t)used;
  }
};

// Encodes nrow consecutive rows (r0 ..) of one record, whose values are pairs[i] (columns 2 lane, 2 lane + 1 of row i),
// into the 1600-byte unit: staged in `rec` (shared memory, one per warp), written back to `grec` as 100 16-byte stores.
// Two phases: every row is encoded and its escape entries are queued in `queue` (shared memory, row-major, column
// order, positions from warp ballots); then the queue is placed: into the unit's free slots by all lanes at once, and
// whatever is left into the chain by lane 0.
__device__ __forceinline__ void append_rows(const AppendArgs& a, uint8_t* const grec, uint8_t* const rec,
                                            uint32_t* const queue, const int r0, const int nrow,
                                            const uint32_t (&pairs)[PAGE], const int lane) {
  uint32_t* const header = reinterpret_cast<uint32_t*>(rec + REC);
  uint32_t* const slots = header + 1;
  int in_unit, chain;                                             // entries already in the unit; first chain block or -1
  if (r0 == 0) {
    // the page starts over: an all-zero unit; with `reuse` the old chain is kept, emptied (its links stay)
    chain = -1;
    if (a.reuse) {
      const uint32_t was = *reinterpret_cast<const volatile uint32_t*>(grec + REC);
      if ((was & 16u) && (int)(was >> 8) < a.P) chain = (int)(was >> 8);
    }
    for (int i = lane; i < RKV / 16; i += 32) reinterpret_cast<uint4*>(rec)[i] = make_uint4(0, 0, 0, 0);
    if (chain >= 0 && lane == 0) {
      int b = chain;
      for (int hops = 0; b >= 0 && b < a.P && hops < 4096; ++hops) {
        const uint32_t w0 = a.pool[(size_t)b * 16];
        a.pool[(size_t)b * 16] = w0 & ~0xFFu;
        b = (int)(w0 >> 8) - 1;
      }
    }
    in_unit = 0;
  } else {
    for (int i = lane; i < RKV / 16; i += 32) reinterpret_cast<uint4*>(rec)[i] = reinterpret_cast<const uint4*>(grec)[i];
    __syncwarp();
    const uint32_t was = *header;
    in_unit = (int)(was & 15u);
    chain = (was & 16u) ? (int)(was >> 8) : -1;
  }
  __syncwarp();
  // ---- phase 1: rows
  int queued = 0;
#pragma unroll
  for (int i = 0; i < PAGE; ++i) {
    if (i >= nrow) break;
    const int r = r0 + i;
    const uint32_t v0 = pairs[i] & 0xFFFFu, v1 = pairs[i] >> 16;
    const int e0 = (int)((v0 >> 7) & 0xFFu), e1 = (int)((v1 >> 7) & 0xFFu);
    int top = max(e0, e1);                                        // the row's node: largest exponent of its 64 values
#pragma unroll
    for (int o = 16; o; o >>= 1) top = max(top, __shfl_xor_sync(FULL, top, o));
    const bool out0 = top - e0 > 14, out1 = top - e1 > 14;
    // leaf = mantissa << 1 | sign of the pair partner (zero for a value that escapes), state = exponent distance
    const uint32_t leaf0 = (out0 ? 0u : (v0 & 0x7Fu) << 1) | (out1 ? 0u : v1 >> 15);
    const uint32_t leaf1 = (out1 ? 0u : (v1 & 0x7Fu) << 1) | (out0 ? 0u : v0 >> 15);
    *reinterpret_cast<uint16_t*>(rec + leaf_pair_off(r, lane)) = (uint16_t)(leaf0 | leaf1 << 8);
    const uint32_t st0 = out0 ? 15u : (uint32_t)(top - e0), st1 = out1 ? 15u : (uint32_t)(top - e1);
    uint16_t* const sp = reinterpret_cast<uint16_t*>(rec + state_pair_off(r, lane));
    const int nib = 4 * (r >> 3);                                 // rows 0-7 low nibbles, rows 8-15 high nibbles
    *sp = (uint16_t)((*sp & ~((0xFu << nib) | (0xF00u << nib))) | st0 << nib | st1 << (8 + nib));
    if (lane == 0) rec[1536 + 2 * (r & 7) + (r >> 3)] = (uint8_t)top;
    const unsigned m0 = __ballot_sync(FULL, out0), m1 = __ballot_sync(FULL, out1);
    if ((m0 | m1) == 0u) continue;
    const unsigned below = (1u << lane) - 1u;
    const int at = queued + __popc(m0 & below) + __popc(m1 & below);
    const uint32_t where = (uint32_t)r << 6 | (uint32_t)(2 * lane);
    if (out0) queue[at] = v0 << 16 | where;
    if (out1) queue[at + (out0 ? 1 : 0)] = v1 << 16 | (where + 1u);
    queued += __popc(m0) + __popc(m1);
  }
  __syncwarp();
  // ---- phase 2: place the queued entries
  const int to_unit = min(queued, NSLOT - in_unit);
  if (lane < to_unit) slots[in_unit + lane] = queue[lane];       // at most 11
  in_unit += to_unit;
  if (queued > to_unit) {
    if (lane == 0) {
      ChainTail tail{a.pool, a.pool_cnt, a.P, chain, -1, 0};
      for (int i = to_unit; i < queued; ++i) tail.push(queue[i]);
      chain = tail.first;
    }
    chain = __shfl_sync(FULL, chain, 0);
  }
  if (lane == 0) *header = (uint32_t)in_unit | (chain >= 0 ? 16u | (uint32_t)chain << 8 : 0u);
  __syncwarp();
  for (int i = lane; i < RKV / 16; i += 32) reinterpret_cast<uint4*>(grec)[i] = reinterpret_cast<const uint4*>(rec)[i];
  __syncwarp();                                                   // the staging unit and the queue are reused
}

// One warp per (token, head, K/V, half); only the warp of a segment's first token works: a segment is a run of
// consecutive slots inside one page, and its warp owns the record for the whole launch (rows g and g+8 share state
// bytes, and the header is read-modify-write).  Semantics of statetree/csrc/kvcache.cu:62-192.
// The warp edits the 1600-byte unit in shared memory: the segment's rows are fetched up front (independent loads),
// encoded row by row with shared-memory byte stores, and the unit goes back to the page as 100 16-byte stores.
__global__ void __launch_bounds__(256) kv_append_kernel(const AppendArgs a) {
  __shared__ __align__(16) uint8_t s_unit[8][RKV];
  __shared__ uint32_t s_queue[8][PAGE * 64];                      // a segment's escape entries, worst case all of them
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
  append_rows(a, grec, rec, s_queue[threadIdx.x >> 5], r0, nrow, pairs, lane);
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
  __shared__ uint32_t s_queue[8][64];                             // one row per launch: at most 64 escape entries
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
  append_rows(a, a.kv + unit_off(blk, a.H, h, kvi, half), s_unit[threadIdx.x >> 5], s_queue[threadIdx.x >> 5],
              (int)(s0 % PAGE), 1, pairs, lane);
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
// Decode attention over the pages, one query token per sequence.
//
// Orientation.  A record is stored in mma.m16n8k16 A-fragment order with tokens as rows, and a decode step has only
// G = Hq / Hkv (1..8) query heads per KV head.  So the heads go on the 8-wide N side of the tensor-core shape and the
// big dimensions on the 16-wide M side:
//     S^T [16 tokens x 8 heads]  = K [16 tokens x 128 dims] . Q^T      8 MMAs per page; the decoded K record is the A
//                                                                      operand as it comes out of the decoder
//     O^T [128 dims x 8 heads]  += V^T [128 dims x 16 tokens] . P^T    8 MMAs per page (16 with the residual of P);
//                                                                      V^T fragments are the V record's 8 x 8 blocks
//                                                                      transposed in registers (movmatrix), P^T is the
//                                                                      probability fragment transposed the same way
// With G = 4 half of each MMA is useful (a quarter when the heads sit on the M side), 24 MMAs per page in all.
//
// Softmax.  Scores live in the exp2 domain.  Each head keeps a reference maximum m that is raised only when a page
// holds a score more than 8 above it (one warp vote per page finds out; raising costs the cross-lane reduction and a
// rescale of the accumulators), so probabilities stay below 2^8 and the common page pays no reduction at all.  The
// row sums are kept per lane and reduced once at the end.  P is fed to the tensor cores as a BF16 value plus the BF16
// of its rounding residual (~16 mantissa bits), which keeps the fp32 partial results within 1e-3 of fp64.
//
// Work split.  Grid = sequences x KV heads x splits; a CTA's pages are dealt round-robin to its warps, and every warp
// streams its own pages through a private ring of 6400-byte bulk copies (one page of one KV head = K half 0/1, V
// half 0/1, contiguous), so there is no block-level barrier inside the loop.
struct AttnLaunch {
  const uint16_t* q; long long q_stride;          // [B][Hq][128] BF16, elements between sequences
  const uint8_t* pages; long long n_pages;
  const uint32_t* pool; int pool_blocks;
  const int* table; long long table_stride;       // block table [B][table_stride]
  const int* seq_len; const int* seq_start;       // tokens [seq_start, seq_len) of each sequence take part
  uint16_t* out; long long out_stride;
  float* part_o; float* part_ml;                  // split partials: [B][Hq][splits][128], [B][Hq][splits][2] = (m, l)
  float scale_log2;                               // softmax scale * log2(e)
  int kv_heads, group, splits, min_pages;
  int* status;
};

constexpr int PAGE_BYTES = 4 * RKV;
constexpr float RAISE_MARGIN = 8.f;               // a head's reference maximum is raised when a score exceeds it by this

// exact bits of one element of a decoded record; the entry is the same in every lane, so the register it lands in is
// warp-uniform and only the lane that owns the element takes the (single) branch
__device__ __forceinline__ void put_exact(uint32_t (&R)[4][4], uint32_t entry, int lane) {
  const int row = (int)((entry >> 6) & 15u), col = (int)(entry & 63u);
  if (lane != (row & 7) * 4 + ((col & 7) >> 1)) return;
  const uint32_t sh = 16u * (uint32_t)(col & 1), keep = ~(0xFFFFu << sh), val = (entry >> 16) << sh;
  switch ((col >> 4) * 4 + (row >> 3) + 2 * ((col >> 3) & 1)) {
#define ST_PUT(i) case i: R[(i) >> 2][(i) & 3] = (R[(i) >> 2][(i) & 3] & keep) | val; break;
    ST_PUT(0) ST_PUT(1) ST_PUT(2) ST_PUT(3) ST_PUT(4) ST_PUT(5) ST_PUT(6) ST_PUT(7)
    ST_PUT(8) ST_PUT(9) ST_PUT(10) ST_PUT(11) ST_PUT(12) ST_PUT(13) ST_PUT(14) ST_PUT(15)
#undef ST_PUT
  }
}

// one 1600-byte unit in shared memory -> the lane's fragment registers, escapes (in-record slots, then the pool chain)
// applied
__device__ __forceinline__ void unit_to_frag(const uint8_t* unit, const uint32_t* pool, int pool_blocks, int lane,
                                             uint32_t (&R)[4][4]) {
  decode_frag(load_rec_shared(unit, lane), R);
  const uint32_t head = *reinterpret_cast<const uint32_t*>(unit + REC);
  if ((head & 31u) == 0u) return;
  const uint32_t* slot = reinterpret_cast<const uint32_t*>(unit + REC + 4);
  const int used = min((int)(head & 15u), NSLOT);
  for (int i = 0; i < used; ++i) put_exact(R, slot[i], lane);
  if (head & 16u) {
    int blk = (int)(head >> 8);
    for (int hops = 0; blk >= 0 && blk < pool_blocks && hops < 4096; ++hops) {
      const uint32_t w0 = __ldg(pool + (size_t)blk * 16);
      const int n = min((int)(w0 & 0xFFu), XSLOT);
      for (int i = 0; i < n; ++i) put_exact(R, __ldg(pool + (size_t)blk * 16 + 1 + i), lane);
      blk = (int)(w0 >> 8) - 1;
    }
  }
}

__device__ __forceinline__ float max_over_rows(float v) {        // lanes that differ in g (bits 2..4) hold other tokens
  v = fmaxf(v, __shfl_xor_sync(FULL, v, 4));
  v = fmaxf(v, __shfl_xor_sync(FULL, v, 8));
  return fmaxf(v, __shfl_xor_sync(FULL, v, 16));
}
__device__ __forceinline__ float sum_over_rows(float v) {
  v += __shfl_xor_sync(FULL, v, 4);
  v += __shfl_xor_sync(FULL, v, 8);
  return v + __shfl_xor_sync(FULL, v, 16);
}

template <int NW, int STG>
__global__ void __launch_bounds__(NW * 32) kv_attn_kernel(const AttnLaunch a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NW * STG * PAGE_BYTES);      // [NW][STG]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int G = a.group, Hq = a.kv_heads * G;
  const int split = blockIdx.x % a.splits, bh = blockIdx.x / a.splits;
  const int kvh = bh % a.kv_heads, seq = bh / a.kv_heads;
  pdl_wait();                               // queries, lengths and this step's pages come from earlier kernels
  pdl_launch_dependents();

  // ---- this warp's pages
  const int len = a.seq_len[seq], start = a.seq_start ? a.seq_start[seq] : 0;
  const int first_page = start / PAGE;
  const int end_page = len > start ? (int)min((long long)(len + PAGE - 1) / PAGE, a.table_stride) : 0;
  const int per_split = max(a.min_pages, (end_page - first_page + a.splits - 1) / a.splits);
  const int lo_page = first_page + split * per_split, hi_page = min(end_page, lo_page + per_split);
  const int my_first = lo_page + warp;
  const int my_count = hi_page > my_first ? (hi_page - my_first + NW - 1) / NW : 0;

  uint8_t* ring = smem + (size_t)warp * STG * PAGE_BYTES;
  uint64_t* bar = bars + warp * STG;
  if (lane == 0) {
    for (int s = 0; s < STG; ++s) mbar_init(bar + s, 1);
    fence_barrier_init();
  }
  __syncwarp();
  const uint64_t stream_policy = policy_evict_first();
  auto fetch = [&](int i) {                        // lane 0: this warp's i-th page -> stage i % STG
    long long blk = a.table[(size_t)seq * a.table_stride + my_first + i * NW];
    blk = blk < 0 ? 0 : (blk >= a.n_pages ? a.n_pages - 1 : blk);
    const int s = i % STG;
    mbar_expect_tx(bar + s, PAGE_BYTES);
    bulk_g2s(ring + (size_t)s * PAGE_BYTES, a.pages + ((size_t)blk * a.kv_heads + kvh) * PAGE_BYTES, PAGE_BYTES, bar + s,
             stream_policy);
  };
  if (lane == 0)
    for (int i = 0; i < min(my_count, STG); ++i) fetch(i);

  // ---- Q^T as the B operand: lane (g, t) holds head g, dims 16 ks + 2t, +1 and 16 ks + 8 + 2t, +1
  uint32_t qf[8][2];
  {
    const uint16_t* qrow = a.q + (size_t)seq * a.q_stride + (size_t)(kvh * G + (g < G ? g : 0)) * HD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t v0 = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t);
      const uint32_t v1 = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 8 + 2 * t);
      qf[ks][0] = g < G ? v0 : 0u;
      qf[ks][1] = g < G ? v1 : 0u;
    }
  }
  // ---- running state.  This lane's score columns are heads 2t and 2t + 1; heads beyond G never take part: their
  // scores are masked to -inf and their reference maximum stays 0, so their probabilities are exactly 0
  const bool head0 = 2 * t < G, head1 = 2 * t + 1 < G;
  float m0 = head0 ? -INFINITY : 0.f, m1 = head1 ? -INFINITY : 0.f, l0 = 0.f, l1 = 0.f;
  float acc[8][4];                                 // O^T: tile j = dims 16j .. 16j + 15; [0],[1] dim 16j + g, [2],[3] + 8
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  bool gave_up = false;

  for (int i = 0; i < my_count; ++i) {
    const int s = i % STG, page = my_first + i * NW;
    if (!mbar_wait(bar + s, (uint32_t)(i / STG) & 1u)) {
      if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
      for (int k = i + 1; k < min(my_count, i + STG); ++k)           // let the copies still in flight land
        (void)mbar_wait(bar + k % STG, (uint32_t)(k / STG) & 1u);
      gave_up = true;
      break;
    }
    const uint8_t* pg = ring + (size_t)s * PAGE_BYTES;
    // ---- S^T = K Q^T
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t R[4][4];
      unit_to_frag(pg + half * RKV, a.pool, a.pool_blocks, lane, R);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) mma_bf16(sc, R[ks], qf[half * 4 + ks][0], qf[half * 4 + ks][1]);
    }
    // this lane: tokens g and g + 8 of the page; valid tokens of the sequence are [start, len)
    const int tok = page * PAGE + g;
    const bool v_lo = tok >= start && tok < len, v_hi = tok + 8 >= start && tok + 8 < len;
    const float x00 = (v_lo && head0) ? sc[0] * a.scale_log2 : -INFINITY;
    const float x01 = (v_lo && head1) ? sc[1] * a.scale_log2 : -INFINITY;
    const float x10 = (v_hi && head0) ? sc[2] * a.scale_log2 : -INFINITY;
    const float x11 = (v_hi && head1) ? sc[3] * a.scale_log2 : -INFINITY;
    const float top0 = fmaxf(x00, x10), top1 = fmaxf(x01, x11);
    if (__any_sync(FULL, top0 > m0 + RAISE_MARGIN || top1 > m1 + RAISE_MARGIN)) {
      // raise the reference maxima to the page's true maxima and bring the accumulators along
      const float n0 = fmaxf(m0, max_over_rows(top0)), n1 = fmaxf(m1, max_over_rows(top1));
      const float f0 = n0 == m0 ? 1.f : exp2f(m0 - n0), f1 = n1 == m1 ? 1.f : exp2f(m1 - n1);
      l0 *= f0;
      l1 *= f1;
#pragma unroll
      for (int j = 0; j < 8; ++j) { acc[j][0] *= f0; acc[j][1] *= f1; acc[j][2] *= f0; acc[j][3] *= f1; }
      m0 = n0;
      m1 = n1;
    }
    const float p00 = exp2f(x00 - m0), p01 = exp2f(x01 - m1), p10 = exp2f(x10 - m0), p11 = exp2f(x11 - m1);
    l0 += p00 + p10;
    l1 += p01 + p11;
    // P^T as the B operand: the score fragment is [token][head]; transposed it is [head g][tokens 2t, 2t + 1]
    const uint32_t hi_lo = pack_bf16(p00, p01), hi_hi = pack_bf16(p10, p11);
    const float2 r_lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi_lo));
    const float2 r_hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi_hi));
    const uint32_t pb0 = movmatrix_t(hi_lo), pb1 = movmatrix_t(hi_hi);
    const uint32_t rb0 = movmatrix_t(pack_bf16(p00 - r_lo.x, p01 - r_lo.y));
    const uint32_t rb1 = movmatrix_t(pack_bf16(p10 - r_hi.x, p11 - r_hi.y));
    // ---- O^T += V^T P^T
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t R[4][4];
      unit_to_frag(pg + (2 + half) * RKV, a.pool, a.pool_blocks, lane, R);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        // 8 x 8 blocks of the record (tokens x dims) transposed: rows become dims, the k index becomes tokens
        const uint32_t a0 = movmatrix_t(R[ks][0]), a1 = movmatrix_t(R[ks][2]);
        const uint32_t a2 = movmatrix_t(R[ks][1]), a3 = movmatrix_t(R[ks][3]);
        mma_bf16_r(acc[half * 4 + ks], a0, a1, a2, a3, pb0, pb1);
        mma_bf16_r(acc[half * 4 + ks], a0, a1, a2, a3, rb0, rb1);
      }
    }
    __syncwarp();                                  // every lane has read this stage
    if (lane == 0 && i + STG < my_count) {
      fence_proxy_async();
      fetch(i + STG);
    }
  }
  if (gave_up) { m0 = head0 ? -INFINITY : 0.f; m1 = head1 ? -INFINITY : 0.f; l0 = l1 = 0.f; }
  l0 = sum_over_rows(l0);
  l1 = sum_over_rows(l1);

  // ---- combine the warps of the CTA.  The rings are idle now; each warp parks (O^T, m, l) of its G heads there.
  __syncthreads();
  float* park = reinterpret_cast<float*>(smem);
  constexpr int PER_WARP = 8 * (HD + 2);           // per head: 128 values of O, then m, l
  static_assert(NW * PER_WARP * 4 <= NW * STG * PAGE_BYTES, "parked partials must fit in the ring");
  float* mine = park + warp * PER_WARP;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (head0) { mine[(2 * t) * (HD + 2) + 16 * j + g] = acc[j][0]; mine[(2 * t) * (HD + 2) + 16 * j + 8 + g] = acc[j][2]; }
    if (head1) { mine[(2 * t + 1) * (HD + 2) + 16 * j + g] = acc[j][1]; mine[(2 * t + 1) * (HD + 2) + 16 * j + 8 + g] = acc[j][3]; }
  }
  if (g == 0) {
    if (head0) { mine[(2 * t) * (HD + 2) + HD] = m0; mine[(2 * t) * (HD + 2) + HD + 1] = l0; }
    if (head1) { mine[(2 * t + 1) * (HD + 2) + HD] = m1; mine[(2 * t + 1) * (HD + 2) + HD + 1] = l1; }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * HD; e += NW * 32) {
    const int h = e / HD, d = e % HD;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) top = fmaxf(top, park[w * PER_WARP + h * (HD + 2) + HD]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float* pw = park + w * PER_WARP + h * (HD + 2);
      if (pw[HD] == -INFINITY) continue;           // a warp without pages
      const float f = exp2f(pw[HD] - top);
      den += f * pw[HD + 1];
      num += f * pw[d];
    }
    const int hq = kvh * G + h;
    if (a.splits == 1) {
      const __nv_bfloat16 v = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
      a.out[(size_t)seq * a.out_stride + (size_t)hq * HD + d] = *reinterpret_cast<const uint16_t*>(&v);
    } else {
      const size_t ix = ((size_t)seq * Hq + hq) * a.splits + split;
      a.part_o[ix * HD + d] = num;
      if (d == 0) { a.part_ml[ix * 2] = top; a.part_ml[ix * 2 + 1] = den; }
    }
  }
}

// One warp per (sequence, query head): weighs the split partials by exp2(m_j - max m) and normalises.
__global__ void __launch_bounds__(128) kv_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                       uint16_t* __restrict__ out, long long out_stride, int Hq,
                                                       int splits, long long rows) {
  pdl_wait();
  pdl_launch_dependents();
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* ml = part_ml + (size_t)row * splits * 2;
  float top = -INFINITY;
  for (int j = lane; j < splits; j += 32) top = fmaxf(top, ml[2 * j]);
#pragma unroll
  for (int o = 16; o; o >>= 1) top = fmaxf(top, __shfl_xor_sync(FULL, top, o));
  float den = 0.f;
  float4 num = make_float4(0.f, 0.f, 0.f, 0.f);    // this lane's four dims
  for (int j = 0; j < splits; ++j) {
    const float mj = ml[2 * j];
    if (mj == -INFINITY) continue;                  // a split without tokens
    const float f = exp2f(mj - top);
    den += f * ml[2 * j + 1];
    const float4 o = *reinterpret_cast<const float4*>(part_o + ((size_t)row * splits + j) * HD + 4 * lane);
    num.x += f * o.x; num.y += f * o.y; num.z += f * o.z; num.w += f * o.w;
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  uint2 packed;
  packed.x = pack_bf16(num.x * inv, num.y * inv);
  packed.y = pack_bf16(num.z * inv, num.w * inv);
  *reinterpret_cast<uint2*>(out + (size_t)(row / Hq) * out_stride + (size_t)(row % Hq) * HD + 4 * lane) = packed;
}

template <int NW, int STG>
int attn_launch(const AttnLaunch& a, int B, cudaStream_t st) {
  const int smem = NW * STG * PAGE_BYTES + NW * STG * 8;
  static bool set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set[dev]) {
    if (int e = st::cuda_fail(cudaFuncSetAttribute(kv_attn_kernel<NW, STG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   smem), "st_kv_attn: shared memory attribute"))
      return e;
    set[dev] = true;
  }
  return st::launch("st_kv_attn launch", kv_attn_kernel<NW, STG>, dim3((unsigned)(B * a.kv_heads * a.splits)),
                    dim3(NW * 32), (size_t)smem, st, a);
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
  ST_REQUIRE(Hq / Hkv <= 8, "st_kv_attn: at most 8 query heads per KV head (got %lld)", (long long)(Hq / Hkv));
  ST_REQUIRE(S >= 1 && S <= 1024, "st_kv_attn: splits must be in [1, 1024]");
  if (B == 0) return 0;
  ST_REQUIRE(q && kv && pool && bt && lens && out, "st_kv_attn: null pointer");
  ST_REQUIRE(S == 1 || (wo && wml), "st_kv_attn: split workspace (wo, wml) missing");
  ST_REQUIRE(nblocks > 0, "st_kv_attn: empty cache");
  ST_REQUIRE(((uintptr_t)q & 3u) == 0 && qs % 2 == 0 && st::aligned16(kv), "st_kv_attn: alignment");
  ST_REQUIRE(S == 1 || (((uintptr_t)wo & 15u) == 0 && ((uintptr_t)out & 7u) == 0 && os % 4 == 0),
             "st_kv_attn: wo must be 16-byte aligned, out 8-byte aligned with a row stride that is a multiple of 4");
  ST_REQUIRE(B * Hkv * S < (1ll << 31), "st_kv_attn: grid too large");
  AttnLaunch a;
  a.q = (const uint16_t*)q; a.q_stride = qs; a.pages = (const uint8_t*)kv; a.n_pages = nblocks;
  a.pool = pool; a.pool_blocks = (int)P; a.table = bt; a.table_stride = bts; a.seq_len = lens; a.seq_start = starts;
  a.out = (uint16_t*)out; a.out_stride = os; a.part_o = wo; a.part_ml = wml;
  a.scale_log2 = (float)(scale * 1.4426950408889634);
  a.kv_heads = (int)Hkv; a.group = (int)(Hq / Hkv); a.splits = (int)S; a.min_pages = (int)(minpps < 1 ? 1 : minpps);
  a.status = st::status_ptr();
  ST_REQUIRE(a.status != nullptr, "st_kv_attn: no device status word");
  cudaStream_t st_ = (cudaStream_t)stream;
  // four warps with two pages in flight each (51 KB): several CTAs share an SM and hide each other's latencies
  if (int e = attn_launch<4, 2>(a, (int)B, st_)) return e;
  if (S > 1) {
    const long long rows = B * Hq;
    return st::launch("st_kv_attn merge launch", kv_merge_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, st_,
                      (const float*)wo, (const float*)wml, (uint16_t*)out, (long long)os, (int)Hq, (int)S, rows);
  }
  return 0;
}
