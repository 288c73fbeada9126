// Small-batch fused tree-decode GEMV for sm_100a: Y[B, M] = X[B, N] W[M, N]^T, B <= 32, W stored as state-tree records.
//
// The record stream is consumed in MEMORY ORDER.  Work unit = up to 8 consecutive records of one 16-row tile
// (12 416 B); the U units of the (virtual) matrix are cut into one contiguous range per CTA, so every CTA streams one
// contiguous span of HBM.  A producer warp moves each unit into a ring of shared-memory stages with 1-D bulk copies
// (TMA, mbarrier byte counting, L2 evict-first): the records, the unit's 64-byte escape block, and the matching
// 512-column slice of every activation row.  Eight consumer warps each take one record of the unit: three 128-bit
// shared loads per lane give the lane's fragment of the record, five integer ops per four weights decode it into the
// mma.m16n8k16 A fragment, escapes are patched in registers, and the activations come in as B fragments by ldmatrix.
// Accumulators stay in registers across the units of a tile; at the end of a tile a reducer warp sums the eight warps
// in warp order in shared memory.  A tile whose units span several CTAs is finished through exchange slots in the
// workspace (see the reducer warp): its parts are added in one fixed order, so results are bit-identical from run to
// run, and the CTA that arrives second pays a single round trip.
//
// The same kernel serves the mixture-of-experts products: MODE 1 makes every (token, expert) slot its own problem
// with one activation row; MODE 2 makes every block of 8 slots of one expert (moe_align_block_size layout) a problem.
// MODE 3 multiplies one activation batch by a short LIST of matrices with the same number of columns (q / k / v, or
// gate / up, stored as separate trees) in one launch: their tiles are concatenated into one virtual matrix, so the list
// pays the launch, ring fill and tail of a single kernel, and each member writes its own output.
// MODE 4 is the row-parallel product of a tensor-parallel group: every rank multiplies its column shard, and the
// reducer warp, instead of storing a finished tile, writes its fp32 sums into the receive area of every rank's
// communication buffer over NVLink (plain peer stores, one self-validating word per value) and later adds the ranks'
// words from its OWN buffer in rank order: the all-reduce costs no second launch and no flag round trip.
// MODE 5 takes the activations as the decode step has them before a projection: the residual stream x, the previous
// block's output delta and the RMSNorm weights.  Every CTA forms x + delta, normalises it and scales it into its own
// shared-memory copy of the activations (a few KB per row, read from L2), so the add + norm launch in front of the
// q / k / v and gate / up projections disappears; CTA 0 also writes the new residual stream.
#include "../../include/statetree_b200.h"
#include "st_comm.cuh"
#include "st_common.cuh"
#include <stdlib.h>

#include <mutex>

#include "st_host.h"


namespace {
using namespace st;

constexpr int CW = 8;                     // consumer warps = records per unit
constexpr int UNIT_BYTES = CW * REC;      // 12416
constexpr int SIDE_BYTES = 64;            // escape block of a unit
constexpr int XROW = CW * 128 + 16;       // bytes per staged activation row (512 columns + pad: conflict-free ldmatrix)
constexpr int MODE_DENSE = 0, MODE_SLOT = 1, MODE_GROUP = 2, MODE_LIST = 3, MODE_AR = 4, MODE_NORM = 5;
constexpr int FIN_CAP = 32;               // MODE_AR: tiles a CTA may have delivered and not yet summed over the ranks
__host__ __device__ constexpr bool one_matrix(int mode) {
  return mode == MODE_DENSE || mode == MODE_LIST || mode == MODE_AR || mode == MODE_NORM;
}
constexpr int MAXL = 4;                   // matrices in one MODE_LIST launch
constexpr uint32_t EMPTY_SLOT = 0xFFFFFFFFu;  // what every word of the workspace holds between launches

struct ListTab {                          // MODE_LIST: the members of the list, by value in the kernel arguments
  const uint8_t* tree[MAXL]; const int* eo[MAXL]; const uint32_t* eb[MAXL]; const uint32_t* el[MAXL];
  uint16_t* Y[MAXL]; float* Yf[MAXL];
  int M[MAXL];                            // rows of each member
  int tend[MAXL];                         // first tile after each member in the concatenation
  int n;
};

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
  int nprob, maxcover, stages, fill, stage_bytes, nxrows, xwhole, xw_stride, xw_bytes;
  int act;                                // dense mode: rows are gate / up tiles in turn, the reducer stores silu(gate) * up
  ListTab lt;
  const uint16_t* delta; const uint16_t* nw; uint16_t* xout; float eps;   // MODE_NORM: X = RMSNorm(X + delta) * nw
  uint8_t* peer[MAX_RANKS];               // MODE_AR: communication buffer of every rank (peer[rank] is the own one)
  int rank, world;
  long long wait_ns;                      // bound of the wait for the other ranks' sums
};

struct Prob {                             // what a unit's problem resolves to
  const uint8_t* tree; const int* eo; const uint32_t* eb; const uint32_t* el;
  bool skip;
};

struct Member {                           // MODE_LIST: the list member a tile of the concatenation belongs to
  const uint8_t* tree; const int* eo; const uint32_t* eb; const uint32_t* el;
  uint16_t* Y; float* Yf; long long M;
  int tile;                               // the tile's index inside the member
  int end;                                // first tile (of the concatenation) after the member
};
__device__ __forceinline__ Member member_of(const GemvArgs& a, int tile) {
  int m = 0;
  while (m + 1 < a.lt.n && tile >= a.lt.tend[m]) ++m;
  Member r;
  r.tree = a.lt.tree[m]; r.eo = a.lt.eo[m]; r.eb = a.lt.eb[m]; r.el = a.lt.el[m];
  r.Y = a.lt.Y[m]; r.Yf = a.lt.Yf[m]; r.M = a.lt.M[m];
  r.tile = tile - (m ? a.lt.tend[m - 1] : 0);
  r.end = a.lt.tend[m];
  return r;
}

template <int MODE>
__device__ __forceinline__ Prob resolve(const GemvArgs& a, int p) {
  Prob r;
  r.skip = false;
  if (one_matrix(MODE)) {                                      // (a list resolves per tile: UnitCursor::retile)
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
  if (one_matrix(MODE)) return n < a.B ? n : -1;
  if (MODE == MODE_SLOT) return n == 0 ? p : -1;
  const int s = a.sorted[p * 8 + n];
  return (n < 8 && s >= 0 && s < a.B) ? s : -1;
}

__device__ __forceinline__ int cta_of_unit(long long u, long long U, int C) { return (int)(((u + 1) * C - 1) / U); }

// Walks a CTA's units without divisions: problem p, tile, unit c inside the tile.  The CTA's range [u0, u1) is
// visited as two segments: first the units of the trailing tile it shares with the next CTA, then the rest.  Both
// tiles that a CTA shares with its neighbours are thus finished in its first microsecond, and the cross-CTA
// hand-over (fence, semaphore, re-read of partial sums) overlaps the streaming instead of forming the kernel's tail.
template <int MODE>
struct UnitCursor {
  int u, end, p, tile, c;
  int seg, b0, e0, b1, e1;
  Prob pr;
  Member mb;                                                           // MODE_LIST only
  __device__ __forceinline__ void retile(const GemvArgs& a) { if (MODE == MODE_LIST && u < end) mb = member_of(a, tile); }
  __device__ __forceinline__ void next_tile(const GemvArgs& a) {     // tile was just incremented
    if (MODE != MODE_LIST) return;
    if (tile < mb.end) ++mb.tile;
    else retile(a);
  }
  __device__ __forceinline__ int ltile() const { return MODE == MODE_LIST ? mb.tile : tile; }
  __device__ __forceinline__ const uint8_t* tree() const { return MODE == MODE_LIST ? mb.tree : pr.tree; }
  __device__ __forceinline__ const int* eo() const { return MODE == MODE_LIST ? mb.eo : pr.eo; }
  __device__ __forceinline__ const uint32_t* eb() const { return MODE == MODE_LIST ? mb.eb : pr.eb; }
  __device__ __forceinline__ const uint32_t* el() const { return MODE == MODE_LIST ? mb.el : pr.el; }
  __device__ __forceinline__ void seek(const GemvArgs& a, int ub, int ue) {
    u = ub; end = ue;
    if (u >= end) return;
    const int upp = a.T * a.CPT;
    p = u / upp;
    const int ul = u - p * upp;
    tile = ul / a.CPT; c = ul - tile * a.CPT;
    enter(a);
    retile(a);
  }
  __device__ __forceinline__ void enter(const GemvArgs& a) {          // (p, tile, c) just changed problem
    while (u < end) {
      pr = resolve<MODE>(a, p);
      if (MODE != MODE_GROUP || !pr.skip) return;
      u += a.T * a.CPT - (tile * a.CPT + c);                         // jump over a skipped problem
      ++p; tile = 0; c = 0;
    }
  }
  __device__ __forceinline__ void init(const GemvArgs& a, int u0, int u1) {
    const int ts = u1 - u1 % a.CPT;                                   // first unit of the tile that holds u1
    if (ts > u0 && ts < u1) { b0 = ts; e0 = u1; b1 = u0; e1 = ts; }
    else { b0 = u0; e0 = u1; b1 = u1; e1 = u1; }
    seg = 0;
    seek(a, b0, e0);
    if (u >= end) { seg = 1; seek(a, b1, e1); }
  }
  __device__ __forceinline__ bool valid() const { return u < end; }
  __device__ __forceinline__ int nrec(const GemvArgs& a) const { return c == a.CPT - 1 ? a.NG - c * CW : CW; }
  __device__ __forceinline__ bool tile_end(const GemvArgs& a) const { return c == a.CPT - 1 || u + 1 == end; }
  // a run = the units of one tile that lie in the current segment, starting at the cursor
  __device__ __forceinline__ int run_len(const GemvArgs& a) const { return min(a.CPT - c, end - u); }
  __device__ __forceinline__ void advance(const GemvArgs& a, int len) {
    u += len; c += len;
    if (c == a.CPT) {
      c = 0;
      if (++tile == a.T) { tile = 0; ++p; enter(a); }
      next_tile(a);
    }
    if (u >= end && seg == 0) { seg = 1; seek(a, b1, e1); }
  }
  __device__ __forceinline__ void next(const GemvArgs& a) {
    ++u;
    if (++c == a.CPT) {
      c = 0;
      if (++tile == a.T) { tile = 0; ++p; enter(a); }
      next_tile(a);
    }
    if (u >= end && seg == 0) { seg = 1; seek(a, b1, e1); }
  }
};

// Eight consumer warps (warp r takes record r of every unit), then one producer warp and one reducer warp.
template <int NT, int MODE>
__global__ void __launch_bounds__((CW + 2) * 32, NT <= 2 ? 2 : 1) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int NB = 8 * NT;                                   // activation columns of the mma
  constexpr int EL = 16 * NB;                                  // outputs of one tile
  constexpr int NRED = NT == 1 ? 4 : 2;                        // tile results in flight between consumers and reducer
  const int S = a.stages, STAGE = a.stage_bytes, NX = a.nxrows;
  uint8_t* ring = smem;
  uint8_t* zrow = smem + (size_t)S * STAGE;                                 // one all-zero activation row
  uint8_t* xw = zrow + XROW;                                                // whole activation rows (xwhole mode)
  float* red = reinterpret_cast<float*>(xw + a.xw_bytes);                   // [NRED][CW][EL]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + NRED * CW * EL);
  uint64_t* empty = full + S;
  uint64_t* done = empty + S;                                               // [NRED] partials of a tile are in red[buf]
  uint64_t* freeb = done + NRED;                                            // [NRED] red[buf] may be overwritten
  uint64_t* xbar = freeb + NRED;                                            // whole activation rows have landed
  int* fin_tile = reinterpret_cast<int*>(xbar + 1);                         // MODE_AR: [FIN_CAP] delivered tiles
  uint16_t* fin_mask = reinterpret_cast<uint16_t*>(fin_tile + FIN_CAP);     // MODE_AR: [FIN_CAP][32] values per lane

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = gridDim.x;
  int u0 = (int)((long long)blockIdx.x * a.U / C), u1 = (int)((long long)(blockIdx.x + 1) * a.U / C);

  if (tid < S) {                                               // one thread per ring stage sets its barriers up
    mbar_init(full + tid, 1);
    mbar_init(empty + tid, CW);
    fence_barrier_init();
  } else if (tid == 32) {
    for (int b = 0; b < NRED; ++b) { mbar_init(done + b, CW); mbar_init(freeb + b, 1); }
    mbar_init(xbar, 1);
    fence_barrier_init();
  }
  if (tid >= 64 && tid < 64 + XROW / 16) reinterpret_cast<uint4*>(zrow)[tid - 64] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  pdl_launch_dependents();                 // the next kernel in the stream may start its own weight prefetch
  if (MODE == MODE_SLOT || MODE == MODE_GROUP) pdl_wait();   // expert ids / slot tables come from earlier kernels
  if (MODE == MODE_GROUP) {
    // The block table is sized for the worst case on the host; how many blocks the routing filled is known only here.
    // The CTAs share the tiles of the blocks in use, whole tiles each, so no CTA idles over the unused tail and no
    // tile is shared (no hand-over of partial sums at all).
    const int used = min(a.nprob, (a.npost[0] + 7) >> 3);
    const long long tiles = (long long)used * a.T;
    u0 = (int)(blockIdx.x * tiles / C) * a.CPT;
    u1 = (int)((blockIdx.x + 1) * tiles / C) * a.CPT;
  }

  UnitCursor<MODE> cur;
  cur.init(a, u0, u1);

  if (warp == CW) {
    // ------------------------------------------------------------------ producer warp.  Lane 0 moves the records,
    // lane 1 the escape block, lane n activation row n.  Weights never depend on the previous kernel, so the first
    // ring fill is issued before griddepcontrol.wait; activations (and everything the reducer touches) after it.
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    int lastp = -1;
    const uint16_t* xrow = nullptr;                           // this lane's activation row of the current problem
    unsigned nx = 0;
    auto row_of = [&](const UnitCursor<MODE>& k) {
      if (k.p != lastp) {
        lastp = k.p;
        const long long r = lane < NX ? out_row<MODE>(a, k.p, lane) : -1;
        xrow = r < 0 ? nullptr : a.X + (one_matrix(MODE) ? r : r / a.xdiv) * a.N;
        nx = a.xwhole ? 0u : __popc(__ballot_sync(FULL, xrow != nullptr));
      }
    };
    auto weights = [&](const UnitCursor<MODE>& k, int s) {
      const int nrec = k.nrec(a);
      uint8_t* st = ring + (size_t)s * STAGE;
      if (lane == 0) {
        mbar_expect_tx(full + s, (uint32_t)(nrec * REC + SIDE_BYTES) + nx * (uint32_t)(nrec * 128));
        bulk_g2s(st, k.tree() + ((size_t)k.ltile() * a.NG + (size_t)k.c * CW) * REC, (uint32_t)(nrec * REC), full + s, pol_w);
      }
      __syncwarp();
      if (lane == 1)
        bulk_g2s(st + UNIT_BYTES, k.eb() + ((size_t)k.ltile() * a.CPT + k.c) * 16, SIDE_BYTES, full + s, pol_w);
    };
    auto acts = [&](const UnitCursor<MODE>& k, int s) {
      if (!a.xwhole && xrow != nullptr)
        bulk_g2s(ring + (size_t)s * STAGE + UNIT_BYTES + SIDE_BYTES + lane * XROW, xrow + (size_t)k.c * CW * 64,
                 (uint32_t)(k.nrec(a) * 128), full + s, pol_x);
    };
    UnitCursor<MODE> mine = cur;                               // lane i looks at unit i of this CTA
    for (int i = 0; i < lane && mine.valid(); ++i) mine.next(a);
    // first ring fill: weights, then wait for the previous kernel, then the activations
    UnitCursor<MODE> pre = cur;
    int filled = 0;
    if (one_matrix(MODE)) {                                    // lane i fills stage i
      const bool on = lane < a.fill && mine.valid();
      if (on) {
        const int nrec = mine.nrec(a);
        uint8_t* st = ring + (size_t)lane * STAGE;
        mbar_expect_tx(full + lane, (uint32_t)(nrec * REC + SIDE_BYTES) + (a.xwhole ? 0u : (uint32_t)(NX * nrec * 128)));
        bulk_g2s(st, mine.tree() + ((size_t)mine.ltile() * a.NG + (size_t)mine.c * CW) * REC, (uint32_t)(nrec * REC),
                 full + lane, pol_w);
        bulk_g2s(st + UNIT_BYTES, mine.eb() + ((size_t)mine.ltile() * a.CPT + mine.c) * 16, SIDE_BYTES, full + lane, pol_w);
      }
      filled = __popc(__ballot_sync(FULL, on));
    } else {
      for (; pre.valid() && filled < a.fill; pre.next(a), ++filled) { row_of(pre); weights(pre, filled); }
    }
    pdl_wait();
    if (a.xwhole && MODE != MODE_NORM) {                       // every activation row once, whole
      if (lane == 0) mbar_expect_tx(xbar, (uint32_t)(NX * a.N * 2));
      __syncwarp();
      if (lane < NX) bulk_g2s(xw + (size_t)lane * a.xw_stride, a.X + (size_t)lane * a.N, (uint32_t)(a.N * 2), xbar, pol_x);
    }
    lastp = -1;
    int s = 0;
    for (int i = 0; i < filled; ++i, cur.next(a)) {
      row_of(cur);
      acts(cur, s);
      ++s;
    }
    // the stages beyond the first fill are taken without a wait on their first use
    int fresh = S - filled;
    s = fresh > 0 ? filled : 0;
    uint32_t ph = fresh > 0 ? 1u : 0u;                         // flips to 0 at the first wrap
    for (; cur.valid(); cur.next(a)) {
      row_of(cur);
      if (fresh > 0) {
        --fresh;
      } else if (!mbar_wait(empty + s, ph)) {
        if (lane == 0) atomicExch(a.status, ERR_WAIT_EMPTY);
        break;
      }
      weights(cur, s);
      acts(cur, s);
      if (++s == S) { s = 0; ph ^= 1u; }
    }
    return;
  }

  if (warp == CW + 1) {
    // ------------------------------------------------------------------ reducer warp: finishes tiles behind the
    // consumers (sums the consumer warps in order, then stores or meets the other CTAs of the tile), so the consumers
    // never wait.
    //
    // A tile cut by CTA boundaries is finished without semaphores, word by word, through exchange slots in `ws` that
    // hold a sentinel (all ones, a NaN pattern no arithmetic produces) between launches.  For a tile in n parts the
    // sums are folded left to right, ((p0 + p1) + p2) + ...: slot level L is where the fold of parts < L meets part L.
    // Each of the two parties swaps its value into the slot (atomicExch); the one that finds the sentinel is done, the
    // one that finds the other's value adds it (fp32 addition is commutative, so who came second does not matter),
    // restores the sentinel and either stores the result (last level) or carries the fold to the next level.  The
    // result has one fixed summation order, and the usual two-part tile costs its second arriver a single round trip.
    pdl_wait();                                                // ws and Y may still be in use by the previous kernel
    int nf = 0;
    float gate[EL / 32];                                       // act mode: the gate tile, until its up tile is done
#pragma unroll
    for (int k = 0; k < EL / 32; ++k) gate[k] = 0.f;
    // MODE_AR.  A value this warp finishes (its tile, or its word of a cut tile) goes to every rank's receive area,
    // word idx of (call parity, this rank); `mask` collects the lane's finished values of the current tile.  The sum
    // over the ranks is taken later (settle), when the peers' words have had time to arrive.
    uint8_t* const own = MODE == MODE_AR ? a.peer[a.rank] : nullptr;
    uint32_t calls = 0;
    if (MODE == MODE_AR) {
      // Every CTA reads the call counter, then counts itself in; the last one to do so advances the counter for the next
      // call (whose kernel reads it only after this grid has completed).  Done here, not at the end, so that it costs
      // the tail of the launch nothing.
      uint32_t* g = reinterpret_cast<uint32_t*>(own + OFF_GEMV);
      calls = ld_relaxed_sys(g);
      calls = __shfl_sync(FULL, calls, 0);
      __threadfence();                                         // the read is ordered before the count
      if (lane == 0 && atomicAdd(g + 1, 1u) == gridDim.x - 1) {
        g[1] = 0u;
        g[0] = calls + 1u;
      }
    }
    const int half = (int)(calls & 1u);
    int nfin = 0;
    unsigned mask = 0;
    long long deadline = 0;                                    // set at the first word that is not here yet
    auto deliver = [&](int tile, int k, float v) {
      uint32_t bits = __float_as_uint(v);
      if (bits == RECV_EMPTY) bits = 0x7FFFFFFFu;              // never the "not here yet" pattern
      const long long idx = (long long)tile * EL + lane + 32 * k;
      for (int p = 0; p < a.world; ++p) st_relaxed_sys(recv_word(a.peer[p], half, a.rank, idx), bits);
      mask |= 1u << k;
    };
    // adds the ranks' words of this lane's values of `tile` in rank order, stores the result, empties the words.
    // The words of up to four values are requested together (a local load at system scope costs a trip to L2), then
    // whatever has not arrived yet is polled.
    auto settle = [&](int tile, unsigned m) {
      constexpr int KC = EL / 32 < 4 ? EL / 32 : 4;
#pragma unroll
      for (int k0 = 0; k0 < EL / 32; k0 += KC) {
        if (!((m >> k0) & ((1u << KC) - 1u))) continue;
        uint32_t bits[KC][MAX_RANKS];
#pragma unroll
        for (int kk = 0; kk < KC; ++kk)
#pragma unroll
          for (int p = 0; p < MAX_RANKS; ++p)
            bits[kk][p] = (p < a.world && ((m >> (k0 + kk)) & 1u))
                              ? ld_relaxed_sys(recv_word(own, half, p, (long long)tile * EL + lane + 32 * (k0 + kk)))
                              : 0u;
#pragma unroll
        for (int kk = 0; kk < KC; ++kk) {
          const int k = k0 + kk;
          if (!((m >> k) & 1u)) continue;
          const long long idx = (long long)tile * EL + lane + 32 * k;
          float v = 0.f;
          bool ok = true;
#pragma unroll
          for (int p = 0; p < MAX_RANKS; ++p) {
            if (p >= a.world || !ok) continue;
            uint32_t b = bits[kk][p];
            while (b == RECV_EMPTY) {                           // bounded by wall time, once for the whole CTA
              const long long now = now_ns();
              if (deadline == 0) deadline = now + a.wait_ns;
              if (now > deadline) { ok = false; break; }
              b = ld_relaxed_sys(recv_word(own, half, p, idx));
            }
            v += __uint_as_float(b);
          }
          if (!ok) {                                            // a rank never delivered: leave the output unwritten
            atomicExch(a.status, ERR_WAIT_PEER);
            continue;
          }
          for (int p = 0; p < a.world; ++p) *recv_word(own, half, p, idx) = RECV_EMPTY;
          const int n = (lane + 32 * k) >> 4, r = (lane + 32 * k) & 15;
          const __nv_bfloat16 hv = __float2bfloat16_rn(v);
          a.Y[(size_t)n * a.M + (size_t)tile * 16 + r] = *reinterpret_cast<const uint16_t*>(&hv);
          if (a.Yf) a.Yf[(size_t)n * a.M + (size_t)tile * 16 + r] = v;
        }
      }
    };
    for (; cur.valid(); cur.advance(a, cur.run_len(a))) {      // one hand-over per run of units of a tile
      const int buf = nf % NRED;
      if (!mbar_wait(done + buf, (uint32_t)(nf / NRED) & 1u)) {
        if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
        return;
      }
      ++nf;
      float sum[EL / 32];
      const float* rb = red + buf * CW * EL;
#pragma unroll
      for (int k = 0; k < EL / 32; ++k) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) v += rb[w * EL + lane + 32 * k];
        sum[k] = v;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(freeb + buf);
      const int tbase = cur.u - cur.c;                          // first unit of the tile
      const bool owned = tbase >= u0 && tbase + a.CPT <= u1;
      uint16_t* const Yp = MODE == MODE_LIST ? cur.mb.Y : a.Y;  // where this tile's results go
      float* const Yfp = MODE == MODE_LIST ? cur.mb.Yf : a.Yf;
      const long long Mp = MODE == MODE_LIST ? cur.mb.M : a.M;
      const size_t row0 = (size_t)cur.ltile() * 16;
      long long orow[EL / 32];                                  // output row of each of this lane's values, -1 = none
#pragma unroll
      for (int k = 0; k < EL / 32; ++k) orow[k] = out_row<MODE>(a, cur.p, (lane + 32 * k) >> 4);
      mask = 0;
      if (!owned) {
        const long long tg = (long long)cur.p * a.T + cur.tile;
        const int cfirst = cta_of_unit(tbase, a.U, C), clast = cta_of_unit(tbase + a.CPT - 1, a.U, C);
        const int last_level = clast - cfirst;                  // parts - 1
        const int part = blockIdx.x - cfirst;
        uint32_t* slots = reinterpret_cast<uint32_t*>(a.ws) + (size_t)tg * a.maxcover * EL;
        const int level0 = part > 0 ? part : 1;
        uint32_t old[EL / 32];
#pragma unroll
        for (int k = 0; k < EL / 32; ++k)                       // all swaps of the first level in flight together
          old[k] = orow[k] >= 0 ? atomicExch(slots + (size_t)(level0 - 1) * EL + lane + 32 * k, __float_as_uint(sum[k]))
                                : EMPTY_SLOT;
#pragma unroll
        for (int k = 0; k < EL / 32; ++k) {
          uint32_t o = old[k];
          int level = level0;
          float v = sum[k];
          while (o != EMPTY_SLOT) {                             // met the other party of this level
            slots[(size_t)(level - 1) * EL + lane + 32 * k] = EMPTY_SLOT;
            v += __uint_as_float(o);
            if (level == last_level) {
              if (MODE == MODE_AR) {
                deliver(cur.tile, k, v);
              } else {
                const int r = (lane + 32 * k) & 15;
                const __nv_bfloat16 hv = __float2bfloat16_rn(v);
                Yp[orow[k] * Mp + row0 + r] = *reinterpret_cast<const uint16_t*>(&hv);
                if (Yfp) Yfp[orow[k] * Mp + row0 + r] = v;
              }
              break;
            }
            ++level;
            o = atomicExch(slots + (size_t)(level - 1) * EL + lane + 32 * k, __float_as_uint(v));
          }
        }
      } else if (MODE == MODE_AR) {
#pragma unroll
        for (int k = 0; k < EL / 32; ++k)
          if (orow[k] >= 0) deliver(cur.tile, k, sum[k]);
      } else if ((MODE == MODE_DENSE || MODE == MODE_NORM) && a.act) {
        // SwiGLU epilogue: tiles 2j and 2j + 1 hold rows 16j .. 16j + 15 of the gate and of the up projection; the host
        // only allows this when every CTA owns whole tiles in pairs, so the gate tile is always the one just before.
        // Rounding as the separate kernels: both outputs to BF16, silu in fp32 to BF16, BF16 product.
        if ((cur.tile & 1) == 0) {
#pragma unroll
          for (int k = 0; k < EL / 32; ++k) gate[k] = sum[k];
        } else {
#pragma unroll
          for (int k = 0; k < EL / 32; ++k) {
            const int r = (lane + 32 * k) & 15;
            if (orow[k] >= 0) {
              const float gte = __bfloat162float(__float2bfloat16_rn(gate[k]));
              const __nv_bfloat16 hv = __hmul(__float2bfloat16_rn(gte / (1.f + __expf(-gte))), __float2bfloat16_rn(sum[k]));
              a.Y[orow[k] * (a.M >> 1) + (size_t)(cur.tile >> 1) * 16 + r] = *reinterpret_cast<const uint16_t*>(&hv);
            }
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < EL / 32; ++k) {
          const int r = (lane + 32 * k) & 15;
          if (orow[k] >= 0) {
            const __nv_bfloat16 hv = __float2bfloat16_rn(sum[k]);
            Yp[orow[k] * Mp + row0 + r] = *reinterpret_cast<const uint16_t*>(&hv);
            if (Yfp) Yfp[orow[k] * Mp + row0 + r] = sum[k];
          }
        }
      }
      if (MODE == MODE_AR && __any_sync(FULL, mask != 0u)) {
        if (nfin < FIN_CAP) {                                   // the peers' words need a while: sum them later
          if (lane == 0) fin_tile[nfin] = cur.tile;
          fin_mask[nfin * 32 + lane] = (uint16_t)mask;
          ++nfin;
        } else {
          settle(cur.tile, mask);
        }
      }
    }
    if (MODE == MODE_AR) {
      __syncwarp();
      for (int e = 0; e < nfin; ++e) settle(fin_tile[e], fin_mask[e * 32 + lane]);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers.  To them a list is one dense
  // matrix (the concatenation): they walk it with the dense cursor and look a member up only for a crowded record.
  UnitCursor<one_matrix(MODE) ? MODE_DENSE : MODE> cc;
  cc.init(a, u0, u1);
  const int g = lane >> 2, rec = warp;
  constexpr int NCH = 2;                                     // independent accumulator chains per column tile
  float acc[NT][NCH][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int h = 0; h < NCH; ++h) acc[nt][h][0] = acc[nt][h][1] = acc[nt][h][2] = acc[nt][h][3] = 0.f;
  int s = 0, nf = 0;
  uint32_t ph = 0;
  // ldmatrix row addresses of this lane: activation row nt * 8 + (lane & 7), or the zero row beyond the batch
  const uint32_t colo = (uint32_t)(rec * 128 + (lane >> 3) * 16);
  const uint32_t zaddr = smem_addr(zrow) + colo;
  uint32_t xo[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + (lane & 7);
    if (n >= NX) xo[nt] = 0u;
    else if (a.xwhole) xo[nt] = smem_addr(xw) + (uint32_t)(n * a.xw_stride) + colo;
    else xo[nt] = (uint32_t)(UNIT_BYTES + SIDE_BYTES + n * XROW) + colo;
  }
  bool xready = !a.xwhole;
  if (MODE == MODE_NORM) {
    // x + delta -> new residual stream (BF16), its RMSNorm times the norm weights -> this CTA's activation rows.  The
    // eight consumer warps share the work: 16-byte vectors, thread t takes vectors t, t + 256, ...
    pdl_wait();
    const int ct = warp * 32 + lane, nvec = (int)(a.N / 8);
    float* part = red;                                         // [rows][CW] partial sums of squares (red is still idle)
    for (int b = 0; b < a.B; ++b) {
      float ss = 0.f;
      for (int v = ct; v < nvec; v += CW * 32) {
        uint4 xv = *reinterpret_cast<const uint4*>(a.X + (size_t)b * a.N + (size_t)v * 8);
        if (a.delta != nullptr) {
          const uint4 dv = *reinterpret_cast<const uint4*>(a.delta + (size_t)b * a.N + (size_t)v * 8);
          const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ds[4] = {dv.x, dv.y, dv.z, dv.w};
          uint32_t so[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)                           // the residual stream stays BF16
            so[q] = pack_bf16(__uint_as_float(xs[q] << 16) + __uint_as_float(ds[q] << 16),
                              __uint_as_float(xs[q] & 0xFFFF0000u) + __uint_as_float(ds[q] & 0xFFFF0000u));
          xv = make_uint4(so[0], so[1], so[2], so[3]);
        }
        if (blockIdx.x == 0 && a.xout != nullptr) *reinterpret_cast<uint4*>(a.xout + (size_t)b * a.N + (size_t)v * 8) = xv;
        *reinterpret_cast<uint4*>(xw + (size_t)b * a.xw_stride + (size_t)v * 16) = xv;
        const uint32_t ws_[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float lo = __uint_as_float(ws_[q] << 16), hi = __uint_as_float(ws_[q] & 0xFFFF0000u);
          ss += lo * lo + hi * hi;
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(FULL, ss, o);
      if (lane == 0) part[b * CW + warp] = ss;
    }
    asm volatile("bar.sync 2, %0;" :: "n"(CW * 32) : "memory");
    for (int b = 0; b < a.B; ++b) {
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < CW; ++i) tot += part[b * CW + i];
      const float r = rsqrtf(tot / (float)a.N + a.eps);
      for (int v = ct; v < nvec; v += CW * 32) {
        uint4* slot = reinterpret_cast<uint4*>(xw + (size_t)b * a.xw_stride + (size_t)v * 16);
        const uint4 xv = *slot;
        const uint4 gv = *reinterpret_cast<const uint4*>(a.nw + (size_t)v * 8);
        const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, gs[4] = {gv.x, gv.y, gv.z, gv.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {                           // normalised value rounded, then scaled
          const uint32_t n = pack_bf16(__uint_as_float(xs[q] << 16) * r, __uint_as_float(xs[q] & 0xFFFF0000u) * r);
          o[q] = pack_bf16(__uint_as_float(n << 16) * __uint_as_float(gs[q] << 16),
                           __uint_as_float(n & 0xFFFF0000u) * __uint_as_float(gs[q] & 0xFFFF0000u));
        }
        *slot = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    asm volatile("bar.sync 2, %0;" :: "n"(CW * 32) : "memory");
    xready = true;
  }
  const int last_nrec = a.NG - (a.CPT - 1) * CW;
  // escapes of this warp's record: word 0 of the unit's escape block = escapes in the unit | (mask of the unit's records
  // that have any) << 16, so seven warps in eight are done after one broadcast load
  auto patch_unit = [&](uint32_t (&A)[4][4], const uint32_t sw0, const uint32_t sw, const int c) {
    if ((sw0 >> (16 + rec)) & 1u) {
      const uint32_t ne = sw0 & 0xFFFFu;
      if (ne <= 14u) {                                       // lanes 2..15 hold the inline entries: one vote
        const bool hit = lane >= 2 && lane < 16 && (uint32_t)(lane - 2) < ne && ((sw >> 10) & 7u) == (uint32_t)rec;
        unsigned m = __ballot_sync(FULL, hit);
        while (m) {
          const int src = __ffs(m) - 1;
          m &= m - 1;
          patch_entry(A, __shfl_sync(FULL, sw, src), lane);
        }
      } else {                                               // crowded unit: this record's own list
        // (a list looks its member up here, on the rare path, so the consumers carry no member state in their loop)
        const int* eo_ = cc.pr.eo;
        const uint32_t* el_ = cc.pr.el;
        int lt = cc.tile;
        if (MODE == MODE_LIST) {
            const Member mm = member_of(a, cc.tile);
            eo_ = mm.eo; el_ = mm.el; lt = mm.tile;
        }
        const size_t r = (size_t)lt * a.NG + (size_t)c * CW + rec;
        const int lo = __ldg(eo_ + r), hi = __ldg(eo_ + r + 1);
        for (int base = lo; base < hi; base += 32) {
          const int n = min(32, hi - base);
          const uint32_t ent = (lane < n) ? __ldg(el_ + base + lane) : 0u;
          for (int i = 0; i < n; ++i) patch_entry(A, __shfl_sync(FULL, ent, i), lane);
        }
      }
    }
  };
  while (cc.valid()) {
    const int len = cc.run_len(a), cbeg = cc.c;
    for (int j = 0; j < len; ++j) {
      const int c = cbeg + j;
      if (!xready) {                                          // whole activation rows: waited for once
        if (!mbar_wait(xbar, 0u)) {
          if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
          return;
        }
        xready = true;
      }
      const int nrec = c == a.CPT - 1 ? last_nrec : CW;
      if (!mbar_wait(full + s, ph)) {
        if (lane == 0) atomicExch(a.status, ERR_WAIT_FULL);
        return;
      }
      const uint8_t* st = ring + (size_t)s * STAGE;
      if (rec < nrec) {
        // activations first: their shared-memory latency hides behind the decode
        uint32_t b[NT][8];
        const uint32_t sb = a.xwhole ? (uint32_t)(c * (CW * 128)) : smem_addr(st);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t xa = xo[nt] ? sb + xo[nt] : zaddr;
          ldmatrix_x4(xa, b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
          ldmatrix_x4(xa + 64, b[nt][4], b[nt][5], b[nt][6], b[nt][7]);
        }
        const uint32_t sw0 = *reinterpret_cast<const uint32_t*>(st + UNIT_BYTES);            // escape block, word 0
        const uint32_t sw = reinterpret_cast<const uint32_t*>(st + UNIT_BYTES)[lane & 15];   // inline entries
        const RecRegs raw = load_rec_shared(st + rec * REC, lane);
        // everything this warp needs from the stage is in registers: hand the slot back before the arithmetic
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        uint32_t A[4][4];
        decode_frag(raw, A);
        patch_unit(A, sw0, sw, c);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) mma_bf16(acc[nt][ks % NCH], A[ks], b[nt][2 * ks], b[nt][2 * ks + 1]);
      } else {                                                // no record of this unit for the warp: release only
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
      }
      if (++s == S) { s = 0; ph ^= 1u; }
    }
    // ---- end of this CTA's share of the tile: hand the warp's partial sums to the reducer
    const int buf = nf % NRED;
    if (nf >= NRED && !mbar_wait(freeb + buf, (uint32_t)(nf / NRED - 1) & 1u)) {
      if (lane == 0) atomicExch(a.status, ERR_WAIT_ACC);
      return;
    }
    ++nf;
    float* mine = red + (buf * CW + warp) * EL;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int n0 = nt * 8 + 2 * (lane & 3);
      float t4[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        t4[q] = acc[nt][0][q] + acc[nt][1][q];
      }
      mine[n0 * 16 + g] = t4[0];
      mine[(n0 + 1) * 16 + g] = t4[1];
      mine[n0 * 16 + g + 8] = t4[2];
      mine[(n0 + 1) * 16 + g + 8] = t4[3];
#pragma unroll
      for (int h = 0; h < NCH; ++h) acc[nt][h][0] = acc[nt][h][1] = acc[nt][h][2] = acc[nt][h][3] = 0.f;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(done + buf);
    cc.advance(a, len);
  }
}

struct Plan {
  int C, stages, fill, maxcover, stage_bytes, nxrows, xwhole, xw_stride, xw_bytes;
  size_t smem;
  long long U;
  int CPT, T, NG, nprob;
};

// development builds (-DST_TUNE) read a few planning constants from the environment; the shipped library does not
static int tune(const char* name, int dflt) {
#ifdef ST_TUNE
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
#else
  (void)name;
  return dflt;
#endif
}

// nx = activation rows staged per unit (the batch for a dense matrix, 1 per slot, 8 per block of slots).
template <int NT>
Plan make_plan(long long M, long long N, int nprob, int nx, bool dense, bool act = false, bool ar = false) {
  Plan p;
  p.NG = (int)(N / 64);
  p.CPT = (p.NG + CW - 1) / CW;
  p.T = (int)(M / 16);
  p.nprob = nprob;
  p.U = (long long)nprob * p.T * p.CPT;
  p.nxrows = nx;
  // Whole activation rows stay resident in shared memory when they fit in 66 KB (8 rows of 4096 columns), which leaves
  // at least three ring stages; beyond that every stage carries the matching 512-column slice of each row.
  static const int xw_kb = tune("STATETREE_GEMV_XWHOLE_KB", 66);
  p.xwhole = (dense && (long long)nx * (N * 2 + 16) <= (long long)xw_kb * 1024) ? 1 : 0;
  p.xw_stride = p.xwhole ? (int)(N * 2 + 16) : 0;
  p.xw_bytes = p.xwhole ? nx * p.xw_stride : 0;
  p.stage_bytes = UNIT_BYTES + SIDE_BYTES + (p.xwhole ? 0 : nx * XROW);
  constexpr int EL = 16 * 8 * NT;
  const size_t fixed = XROW + p.xw_bytes + (size_t)(NT == 1 ? 4 : 2) * CW * EL * 4 + (2 * 16 + 9) * 8 + 16 +
                       (ar ? (size_t)FIN_CAP * (4 + 32 * 2) : 0);
  // Two CTAs per SM, each with the deepest ring (at most 8 stages) that fits half of the SM's shared memory; one CTA
  // when even two stages do not fit twice (32 activation rows).
  static const int want_per_sm = tune("STATETREE_GEMV_CTAS_PER_SM", 2), max_stages = tune("STATETREE_GEMV_STAGES", 8),
                   align = tune("STATETREE_GEMV_ALIGN", 1), min_units = tune("STATETREE_GEMV_MIN_UNITS", 2);
  int per_sm = want_per_sm < 1 ? 1 : (want_per_sm > 2 ? 2 : want_per_sm);
  int stages = 0;
  for (; per_sm >= 1; --per_sm) {
    // shared memory of an SM with 1 KB per CTA reserved; a single CTA is capped at the 200 KB the kernel opts in to
    const long long budget = per_sm == 1 ? 200 * 1024 : 233472 / per_sm - 1024;
    stages = (int)((budget - (long long)fixed) / p.stage_bytes);
    if (stages >= 2 || per_sm == 1) break;
  }
  if (stages > max_stages) stages = max_stages;
  if (stages > 16) stages = 16;
  p.stages = stages;
  p.smem = (size_t)stages * p.stage_bytes + fixed;
  const long long slots = (long long)st::sm_count() * per_sm;
  long long want = p.U / (min_units < 1 ? 1 : min_units);     // small matrices: no CTA with less than min_units units
  if (want < 1) want = 1;
  p.C = (int)(want < slots ? want : slots);
  // Grid.  Cutting tiles at arbitrary unit boundaries fills every slot with the same amount of work, but the CTA that
  // meets its neighbour last on a cut tile pays an exchange round trip at its tail: worth about three units of work.
  // A grid whose boundaries fall on tile boundaries (or that cuts every tile into equal parts) pays nothing, but leaves
  // slots empty and quantises the work.  Take the largest such grid with at least half the slots, and choose between
  // the two by the units of the longest CTA (12288 x 4096 on 296 slots: cut, 20.8 + 3 units against 24 on 256 whole-
  // tile CTAs; 4096 x 4096: whole tiles, 8 against 6.9 + 3).
  static const int cut_cost = tune("STATETREE_GEMV_CUT_COST", 3), align_pct = tune("STATETREE_GEMV_ALIGN_PCT", 50);
  if (act) {                                                   // SwiGLU epilogue: every CTA owns whole gate / up tile pairs
    const long long pairs = (long long)nprob * p.T / 2;
    for (long long c = p.C; c >= 1; --c)
      if (pairs % c == 0) { p.C = (int)c; break; }
  } else if (align) {
    const long long tiles = (long long)nprob * p.T;
    for (long long c = p.C; c * 100 >= (long long)p.C * align_pct && c >= 1; --c) {
      const bool whole = tiles % c == 0;
      const bool even = c % tiles == 0 && p.CPT % (c / tiles) == 0;
      if (whole || even) {
        if (p.U / c <= p.U / p.C + cut_cost) p.C = (int)c;
        break;
      }
    }
  }
  const long long per = p.U / p.C;
  // First ring fill.  A CTA with a short range starts sooner when it asks for three stages at first and for the others
  // as it goes (the copies of a fill share the SM's load path, so the first one lands later the more there are); a CTA
  // with a long range gains more from the deeper start.
  static const int fill = tune("STATETREE_GEMV_FILL", 0), fill_units = tune("STATETREE_GEMV_FILL_UNITS", 16);
  p.fill = fill > 0 ? fill : (per <= fill_units ? 3 : p.stages);
  if (p.fill > p.stages) p.fill = p.stages;
  long long mc = (p.CPT + per - 1) / per + 1;
  if (mc > p.CPT) mc = p.CPT;
  p.maxcover = (int)(mc < 1 ? 1 : mc);
  return p;
}

template <int NT, int MODE>
int launch(GemvArgs& a, int nprob, int nx, long long ws_bytes, cudaStream_t stream, const char* who) {
  const Plan p = make_plan<NT>(a.M, a.N, nprob, nx, one_matrix(MODE), a.act != 0, MODE == MODE_AR);
  a.NG = p.NG; a.CPT = p.CPT; a.T = p.T; a.U = p.U; a.nprob = nprob; a.maxcover = p.maxcover; a.stages = p.stages; a.fill = p.fill;
  a.stage_bytes = p.stage_bytes; a.nxrows = p.nxrows; a.xwhole = p.xwhole; a.xw_stride = p.xw_stride;
  a.xw_bytes = p.xw_bytes;
  const long long need = (long long)nprob * p.T * p.maxcover * 16 * 8 * NT * 4;
  ST_REQUIRE(p.maxcover == 1 || (a.ws && ws_bytes >= need), "%s: workspace of %lld bytes needed, %lld given", who, need,
             ws_bytes);
  ST_REQUIRE(p.stages >= 2, "%s: internal: ring does not fit", who);
  ST_REQUIRE(!a.act || (p.U % p.C == 0 && (p.U / p.C) % (2 * p.CPT) == 0),
             "%s: the SwiGLU epilogue needs a grid in which every CTA owns whole tiles in pairs (%lld units on %d CTAs)", who,
             (long long)p.U, p.C);
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
  return st::launch(who, gemv_kernel<NT, MODE>, dim3((unsigned)p.C), dim3((CW + 2) * 32), p.smem, stream, a);
}

template <int NT>
long long ws_need(long long M, long long N, int nprob, int nx, bool dense = true) {
  const Plan p = make_plan<NT>(M, N, nprob, nx, dense);
  return p.maxcover == 1 ? 0 : (long long)nprob * p.T * p.maxcover * 16 * 8 * NT * 4;
}

int shape_checks(const char* who, int64_t M, int64_t N, int64_t B) {
  ST_REQUIRE(M > 0 && N > 0 && M % 16 == 0 && N % 64 == 0, "%s: M %% 16 and N %% 64 must be 0 (got %lld x %lld)", who,
             (long long)M, (long long)N);
  ST_REQUIRE(B >= 1 && B <= 32, "%s: batch must be in [1, 32] (got %lld)", who, (long long)B);
  ST_REQUIRE((M / 16) * ((N / 64 + 7) / 8) < (1ll << 31), "%s: too many units", who);
  return 0;
}

int dense_gemv(const char* who, const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el,
               const void* X, void* Y, float* Yf32, int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes,
               int32_t* cnt, int act, cudaStream_t s) {
  if (int e = shape_checks(who, M, N, B)) return e;
  ST_REQUIRE(!act || (M % 32 == 0 && B <= 8 && Yf32 == nullptr),
             "%s: the SwiGLU epilogue needs M %% 32 == 0, batch <= 8 and no fp32 output", who);
  ST_REQUIRE(tree && eo && eb && el && X && Y && cnt, "%s: null pointer", who);
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(eb) && st::aligned16(X), "%s: tree, eb and X must be 16-byte aligned", who);
  GemvArgs a = {};
  a.tree = (const uint8_t*)tree; a.eo = eo; a.eb = eb; a.el = el;
  a.X = (const uint16_t*)X; a.Y = (uint16_t*)Y; a.Yf = Yf32; a.ws = (float*)ws; a.cnt = cnt;
  a.M = M; a.N = N; a.B = (int)B; a.E = 1; a.xdiv = 1; a.act = act ? 1 : 0;
  if (B <= 8) return launch<1, MODE_DENSE>(a, 1, (int)B, ws_bytes, s, who);
  if (B <= 16) return launch<2, MODE_DENSE>(a, 1, (int)B, ws_bytes, s, who);
  return launch<4, MODE_DENSE>(a, 1, (int)B, ws_bytes, s, who);
}
}  // namespace

extern "C" int64_t st_gemv_workspace_bytes(int64_t M, int64_t N, int64_t B) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || B < 1 || B > 32) return -1;
  return B <= 8 ? ws_need<1>(M, N, 1, (int)B) : (B <= 16 ? ws_need<2>(M, N, 1, (int)B) : ws_need<4>(M, N, 1, (int)B));
}

extern "C" int st_gemv(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X,
                       void* Y, float* Yf32, int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt,
                       void* stream) {
  return dense_gemv("st_gemv", tree, eo, eb, el, X, Y, Yf32, B, M, N, ws, ws_bytes, cnt, 0, (cudaStream_t)stream);
}

extern "C" int st_gemv_swiglu_supported(int64_t M, int64_t N, int64_t B) {
  if (M <= 0 || N <= 0 || M % 32 || N % 64 || B < 1 || B > 8) return 0;
  const Plan p = make_plan<1>(M, N, 1, (int)B, true, true);
  return (p.stages >= 2 && p.C * 2 >= st::sm_count() && p.U % p.C == 0 && (p.U / p.C) % (2 * p.CPT) == 0) ? 1 : 0;
}

extern "C" int st_gemv_swiglu(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X,
                              void* act, int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt,
                              void* stream) {
  return dense_gemv("st_gemv_swiglu", tree, eo, eb, el, X, act, nullptr, B, M, N, ws, ws_bytes, cnt, 1,
                    (cudaStream_t)stream);
}

extern "C" int64_t st_gemv_list_workspace_bytes(int64_t n, const int64_t* M, int64_t N, int64_t B) {
  if (n < 1 || n > MAXL || !M || N <= 0 || N % 64 || B < 1 || B > 32) return -1;
  int64_t total = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (M[i] <= 0 || M[i] % 16) return -1;
    total += M[i];
  }
  return B <= 8 ? ws_need<1>(total, N, 1, (int)B) : (B <= 16 ? ws_need<2>(total, N, 1, (int)B) : ws_need<4>(total, N, 1, (int)B));
}

extern "C" int st_gemv_list(int64_t n, const void* const* trees, const int32_t* const* eo, const uint32_t* const* eb,
                            const uint32_t* const* el, const void* X, void* const* Y, float* const* Yf32, int64_t B,
                            const int64_t* M, int64_t N, void* ws, int64_t ws_bytes, void* stream) {
  const char* who = "st_gemv_list";
  ST_REQUIRE(n >= 1 && n <= MAXL, "%s: 1 to %d matrices per call (got %lld)", who, MAXL, (long long)n);
  ST_REQUIRE(trees && eo && eb && el && X && Y && M, "%s: null pointer", who);
  ST_REQUIRE(st::aligned16(X), "%s: X must be 16-byte aligned", who);
  GemvArgs a = {};
  long long total = 0;
  for (int i = 0; i < (int)n; ++i) {
    ST_REQUIRE(trees[i] && eo[i] && eb[i] && el[i] && Y[i], "%s: null pointer in member %d", who, i);
    ST_REQUIRE(st::aligned16(trees[i]) && st::aligned16(eb[i]), "%s: tree and eb of member %d must be 16-byte aligned", who, i);
    ST_REQUIRE(M[i] > 0 && M[i] % 16 == 0 && M[i] < (1ll << 31), "%s: rows of member %d must be a positive multiple of 16", who, i);
    a.lt.tree[i] = (const uint8_t*)trees[i]; a.lt.eo[i] = eo[i]; a.lt.eb[i] = eb[i]; a.lt.el[i] = el[i];
    a.lt.Y[i] = (uint16_t*)Y[i]; a.lt.Yf[i] = Yf32 ? Yf32[i] : nullptr;
    a.lt.M[i] = (int)M[i];
    total += M[i];
    a.lt.tend[i] = (int)(total / 16);
  }
  a.lt.n = (int)n;
  if (int e = shape_checks(who, total, N, B)) return e;
  a.tree = a.lt.tree[0]; a.eo = a.lt.eo[0]; a.eb = a.lt.eb[0]; a.el = a.lt.el[0];
  a.X = (const uint16_t*)X; a.Y = a.lt.Y[0]; a.ws = (float*)ws;
  a.M = total; a.N = N; a.B = (int)B; a.E = 1; a.xdiv = 1;
  cudaStream_t s = (cudaStream_t)stream;
  if (B <= 8) return launch<1, MODE_LIST>(a, 1, (int)B, ws_bytes, s, who);
  if (B <= 16) return launch<2, MODE_LIST>(a, 1, (int)B, ws_bytes, s, who);
  return launch<4, MODE_LIST>(a, 1, (int)B, ws_bytes, s, who);
}

// ---------------------------------------------------------------------------------------------- st_gemv_prenorm
extern "C" int st_gemv_prenorm_supported(int64_t M, int64_t N, int64_t B, int act) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || N % 8 || B < 1 || B > 8) return 0;
  if (act && !st_gemv_swiglu_supported(M, N, B)) return 0;
  const Plan p = make_plan<1>(M, N, 1, (int)B, true, act != 0);
  return (p.xwhole && p.stages >= 2) ? 1 : 0;
}

extern "C" int st_gemv_prenorm(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* x,
                               const void* delta, const void* norm_w, double eps, void* x_out, void* Y, int64_t B,
                               int64_t M, int64_t N, int act, void* ws, int64_t ws_bytes, void* stream) {
  const char* who = "st_gemv_prenorm";
  if (int e = shape_checks(who, M, N, B)) return e;
  ST_REQUIRE(st_gemv_prenorm_supported(M, N, B, act), "%s: shape not supported (batch <= 8, the activation rows must fit in "
             "shared memory%s)", who, act ? "; the SwiGLU epilogue needs whole gate / up tile pairs per CTA" : "");
  ST_REQUIRE(tree && eo && eb && el && x && norm_w && Y, "%s: null pointer", who);
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(eb) && st::aligned16(x) && st::aligned16(norm_w) &&
             (!delta || st::aligned16(delta)) && (!x_out || st::aligned16(x_out)), "%s: 16-byte alignment", who);
  ST_REQUIRE(x_out == nullptr || (x_out != x && x_out != delta), "%s: x_out must not alias x or delta (every CTA reads them)", who);
  GemvArgs a = {};
  a.tree = (const uint8_t*)tree; a.eo = eo; a.eb = eb; a.el = el;
  a.X = (const uint16_t*)x; a.delta = (const uint16_t*)delta; a.nw = (const uint16_t*)norm_w; a.xout = (uint16_t*)x_out;
  a.eps = (float)eps;
  a.Y = (uint16_t*)Y; a.ws = (float*)ws;
  a.M = M; a.N = N; a.B = (int)B; a.E = 1; a.xdiv = 1; a.act = act ? 1 : 0;
  return launch<1, MODE_NORM>(a, 1, (int)B, ws_bytes, (cudaStream_t)stream, who);
}

// ---------------------------------------------------------------------------------------------- st_gemv_allreduce
extern "C" int st_gemv_allreduce(void* const* bufs, int rank, int world, const void* tree, const int32_t* eo,
                                 const uint32_t* eb, const uint32_t* el, const void* X, void* Y, float* Yf32, int64_t B,
                                 int64_t M, int64_t N, void* ws, int64_t ws_bytes, void* stream) {
  const char* who = "st_gemv_allreduce";
  ST_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "%s: rank %d of %d (2..%d ranks)", who, rank,
             world, MAX_RANKS);
  ST_REQUIRE(bufs != nullptr, "%s: null buffer table", who);
  if (int e = shape_checks(who, M, N, B)) return e;
  ST_REQUIRE(tree && eo && eb && el && X && Y, "%s: null pointer", who);
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(eb) && st::aligned16(X), "%s: tree, eb and X must be 16-byte aligned", who);
  const int nt = B <= 8 ? 1 : (B <= 16 ? 2 : 4);
  ST_REQUIRE((M / 16) * (long long)(128 * nt) <= RECV_VALUES,
             "%s: %lld rows at batch %lld exceed the receive area (%lld padded values per call)", who, (long long)M,
             (long long)B, (long long)RECV_VALUES);
  GemvArgs a = {};
  for (int p = 0; p < world; ++p) {
    ST_REQUIRE(bufs[p] != nullptr, "%s: buffer of rank %d missing", who, p);
    a.peer[p] = (uint8_t*)bufs[p];
  }
  a.rank = rank; a.world = world; a.wait_ns = st::comm_wait_ns();
  a.tree = (const uint8_t*)tree; a.eo = eo; a.eb = eb; a.el = el;
  a.X = (const uint16_t*)X; a.Y = (uint16_t*)Y; a.Yf = Yf32; a.ws = (float*)ws;
  a.M = M; a.N = N; a.B = (int)B; a.E = 1; a.xdiv = 1;
  cudaStream_t s = (cudaStream_t)stream;
  if (nt == 1) return launch<1, MODE_AR>(a, 1, (int)B, ws_bytes, s, who);
  if (nt == 2) return launch<2, MODE_AR>(a, 1, (int)B, ws_bytes, s, who);
  return launch<4, MODE_AR>(a, 1, (int)B, ws_bytes, s, who);
}

// ---------------------------------------------------------------------------------------------- st_gemv_static
// The same GEMV for callers that cannot hand over a workspace because they cannot allocate device memory at all: a
// plugin running inside a serving process whose memory pool is owned (and fully reserved) by the host framework, or
// code that runs where cudaMalloc is forbidden.  The exchange slots of its cut tiles live in the file-scope array
// below instead of a caller buffer.  Every GPU that loads the library carries the array (4.06 MiB) until exit.
namespace {
constexpr long long STATIC_WS_BYTES = 4ll << 20;        // fp32 exchange slots of tiles cut between CTAs
constexpr long long STATIC_TILES = 16384;               // tiles a shape may have (M <= 262144); the tail of the array is spare
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_WS_BYTES + STATIC_TILES * 4];
unsigned char* g_static_addr[64];                       // device address of the array, per device
std::mutex g_static_mu;
}  // namespace

extern "C" int st_gemv_static(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X,
                              void* Y, int64_t B, int64_t M, int64_t N, void* stream) {
  ST_REQUIRE(M > 0 && N > 0 && M % 16 == 0 && N % 64 == 0,
             "st_gemv_static: M %% 16 and N %% 64 must be 0 (got %lld x %lld)", (long long)M, (long long)N);
  ST_REQUIRE(B >= 1 && B <= 32, "st_gemv_static: batch must be in [1, 32] (got %lld)", (long long)B);
  ST_REQUIRE(tree && eo && eb && el && X && Y, "st_gemv_static: null pointer");
  ST_REQUIRE(st::aligned16(tree) && st::aligned16(eb) && st::aligned16(X),
             "st_gemv_static: tree, eb and X must be 16-byte aligned");
  ST_REQUIRE((M / 16) * ((N / 64 + 7) / 8) < (1ll << 31), "st_gemv_static: too many units");
  const long long need = B <= 8 ? ws_need<1>(M, N, 1, (int)B) : (B <= 16 ? ws_need<2>(M, N, 1, (int)B)
                                                                         : ws_need<4>(M, N, 1, (int)B));
  ST_REQUIRE(need <= STATIC_WS_BYTES && M / 16 <= STATIC_TILES,
             "st_gemv_static: this shape needs %lld bytes of exchange slots and has %lld tiles; the built-in scratch "
             "holds %lld bytes and allows %lld tiles (use st_gemv with a caller workspace)",
             need, (long long)(M / 16), STATIC_WS_BYTES, STATIC_TILES);
  int dev = 0;
  if (int e = st::cuda_fail(cudaGetDevice(&dev), "st_gemv_static: cudaGetDevice")) return e;
  ST_REQUIRE(dev >= 0 && dev < 64, "st_gemv_static: device index out of range");
  unsigned char* base = nullptr;
  {
    // set-up, once per device, with that device current: the array's name is only a host-side handle here, the
    // kernel needs its device address
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_addr[dev] == nullptr) {
      void* p = nullptr;
      if (int e = st::cuda_fail(cudaGetSymbolAddress(&p, g_static_scratch), "st_gemv_static: cudaGetSymbolAddress"))
        return e;
      ST_REQUIRE(p != nullptr, "st_gemv_static: no device address for the scratch array");
      g_static_addr[dev] = static_cast<unsigned char*>(p);
    }
    base = g_static_addr[dev];
  }
  cudaStream_t s = (cudaStream_t)stream;
  int* cnt = reinterpret_cast<int*>(base + STATIC_WS_BYTES);
  // the array keeps whatever the last call left: the exchange slots this shape uses must hold the sentinel (all ones)
  if (need > 0)
    if (int e = st::cuda_fail(cudaMemsetAsync(base, 0xFF, (size_t)need, s), "st_gemv_static: resetting exchange slots"))
      return e;
  GemvArgs a = {};
  a.tree = (const uint8_t*)tree; a.eo = eo; a.eb = eb; a.el = el;
  a.X = (const uint16_t*)X; a.Y = (uint16_t*)Y; a.Yf = nullptr; a.ws = reinterpret_cast<float*>(base); a.cnt = cnt;
  a.M = M; a.N = N; a.B = (int)B; a.E = 1; a.xdiv = 1;
  if (B <= 8) return launch<1, MODE_DENSE>(a, 1, (int)B, STATIC_WS_BYTES, s, "st_gemv_static");
  if (B <= 16) return launch<2, MODE_DENSE>(a, 1, (int)B, STATIC_WS_BYTES, s, "st_gemv_static");
  return launch<4, MODE_DENSE>(a, 1, (int)B, STATIC_WS_BYTES, s, "st_gemv_static");
}

extern "C" int64_t st_moe_gemv_workspace_bytes(int64_t S, int64_t M, int64_t N) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || S < 1) return -1;
  return ws_need<1>(M, N, (int)S, 1, false);
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
  return launch<1, MODE_SLOT>(a, (int)S, 1, ws_bytes, (cudaStream_t)stream, "st_moe_gemv");
}

extern "C" int64_t st_moe_group_workspace_bytes(int64_t nblk, int64_t M, int64_t N) {
  if (M <= 0 || N <= 0 || M % 16 || N % 64 || nblk < 1) return -1;
  return ws_need<1>(M, N, (int)nblk, 8, false);
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
  return launch<1, MODE_GROUP>(a, (int)nblk, 8, ws_bytes, (cudaStream_t)stream, "st_moe_group_gemv");
}
