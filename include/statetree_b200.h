/* statetree_b200: C ABI of the sm_100a (B200) kernels for the state-tree decode hot path.
 *
 * This library takes the place of the reference project's two pybind extension modules, `statetree._C`
 * (statetree/csrc/bindings.cpp:47-76) and `statetree._kv` (statetree/csrc/kvcache.cu:588-599).  Every entry point
 * takes plain device pointers, sizes and a CUDA stream handle (a `cudaStream_t` passed as `void*`; NULL = the legacy
 * default stream), launches on that stream without synchronising, allocates nothing per call and returns 0 on
 * success.  A non-zero return means the arguments were rejected before any launch (or the launch itself failed);
 * st_last_error() then holds the message, as the reference raised a RuntimeError from TORCH_CHECK.  The caller owns
 * every buffer (outputs, fp32 workspaces, semaphores, KV pool), as in the reference.  Semaphore arrays must be zero
 * on entry and are left zero by the kernels, so CUDA-graph replays need no memset.  The current CUDA device must be
 * the one that owns the pointers.
 *
 * Data formats (frozen by the reference):
 *   tree      uint8 [M/16, N/64, 1552]      weight records (statetree/format.py:9-12)
 *   eo, el    escape side table: eo int32 [M/16 * N/64 + 1] offsets per record into el; el uint32 entries
 *             bits << 16 | (record % 8) << 10 | row << 6 | col   (row, col inside the 16 x 64 record)
 *   eb        uint32 [U, 16] per unit of up to 8 consecutive records of one 16-row tile (U = M/16 * ceil(N/512)):
 *             word 0 = escapes in the unit | (bit r set if record r of the unit has any) << 16, word 1 = offset of the
 *             unit's first entry in el, words 2..15 = the first 14 entries inline (the rest are read from el)
 *   kv        uint8 [blocks, H, 2, 2, 1600] KV pages; pool uint32 [P, 16]; pool_cnt int32 [2]
 *             (statetree/csrc/kvcache.cu:1-14)
 *   X, Y      BF16 row-major, 16-byte aligned; Y[B, M] = X[B, N] * W[M, N]^T
 */
#ifndef STATETREE_B200_H
#define STATETREE_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ST_ABI_VERSION 2

/* replaces the `ABI` attribute check of statetree/ops.py:12 */
int st_abi_version(void);
/* message of the last failed call on this thread */
const char* st_last_error(void);
/* Reads (and clears) the device-side status word of the current device: 0 = no kernel gave up on a bounded wait.
 * Synchronises the device.  No counterpart in the reference (its device-side waits are unbounded). */
int st_device_status(void);

/* ---- weights ---------------------------------------------------------------------------------------------------- */
/* tree -> dense BF16 W [M, N].  Replaces `_C.dec(T, EO, EL, W)` (statetree/csrc/kernels.cu:1540-1582). */
int st_dec(const void* tree, const int32_t* eo, const uint32_t* el, int64_t M, int64_t N, void* W, void* stream);
/* out[i, :] = W[ids[i], :] (embedding lookup); ids int64.  Replaces `_C.rows` (statetree/csrc/kernels.cu:1587-1630). */
int st_rows(const void* tree, const int32_t* eo, const uint32_t* el, int64_t M, int64_t N, const int64_t* ids,
            int64_t n, void* out, void* stream);

/* Small-batch fused decode + GEMV, 1 <= B <= 32.  Replaces the reference's mv / mvs / mvh / mvc / mvt entry points
 * (statetree/csrc/kernels.cu:243-254, 370-400, 548-599, 771-808; statetree/csrc/hop.cu:993-1019).
 * ws: workspace of st_gemv_workspace_bytes() bytes whose 32-bit words all hold 0xFFFFFFFF on entry and are left so
 * (fill it once after allocating it; the kernels use the words as exchange slots for tiles shared between CTAs and put
 * the all-ones sentinel back).  cnt: int32 [M/16] (MoE: [problems * M/16], problems = S slots or nblk blocks), zero
 * on entry and on exit; kept in the signature for callers of the reference's layout, the GEMV no longer touches it.
 * Yf32 (optional, may be NULL): the fp32 accumulators [B, M] before BF16 rounding, for verification. */
int64_t st_gemv_workspace_bytes(int64_t M, int64_t N, int64_t B);
int st_gemv(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X, void* Y,
            float* Yf32, int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream);

/* One activation batch X [B, N] times a LIST of 1 to 4 matrices that share N (the q / k / v or gate / up projections of
 * a checkpoint that stores them as separate trees), in one launch: Y[i] [B, M[i]] = X W[i]^T.  The members' tiles are
 * concatenated into one virtual matrix, so the list pays one launch, one ring fill and one tail.  trees / eo / eb / el /
 * Y / Yf32 / M are HOST arrays of n entries (Yf32 or any of its entries may be NULL); ws as for st_gemv, sized by
 * st_gemv_list_workspace_bytes.  Results are bit-identical from run to run; they equal st_gemv on each member wherever
 * both cut the member's tiles alike.  The reference reaches the same end by fusing the trees at conversion time
 * (statetree/model.py:22-24 DEFAULT_FUSE); this entry gives unfused checkpoints the same launch count. */
int64_t st_gemv_list_workspace_bytes(int64_t n, const int64_t* M, int64_t N, int64_t B);
int st_gemv_list(int64_t n, const void* const* trees, const int32_t* const* eo, const uint32_t* const* eb,
                 const uint32_t* const* el, const void* X, void* const* Y, float* const* Yf32, int64_t B,
                 const int64_t* M, int64_t N, void* ws, int64_t ws_bytes, void* stream);

/* st_gemv (or, with act != 0, st_gemv_swiglu) whose activations are formed inside the kernel from what a decode step
 * holds in front of a projection: X = RMSNorm(x + delta) * norm_w, the sum rounded to BF16 as the residual stream is
 * (delta may be NULL: X = RMSNorm(x) * norm_w).  Every CTA computes its own copy in shared memory; CTA 0 also writes
 * the new residual stream x + delta to x_out (may be NULL; must not alias x or delta).  It replaces the
 * st_add_rmsnorm launch in front of the q / k / v and the gate / up projection.  1 <= B <= 8; ask
 * st_gemv_prenorm_supported first.  ws as for st_gemv.  No counterpart in the reference. */
int st_gemv_prenorm_supported(int64_t M, int64_t N, int64_t B, int act);
int st_gemv_prenorm(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* x,
                    const void* delta, const void* norm_w, double eps, void* x_out, void* Y, int64_t B, int64_t M,
                    int64_t N, int act, void* ws, int64_t ws_bytes, void* stream);

/* st_gemv for callers that cannot allocate device memory and so have no workspace to pass: code running inside a
 * host framework that owns the whole device pool, or anywhere cudaMalloc is off limits.  The exchange slots of tiles
 * shared between CTAs live in a 4.06 MiB array built into the library (present on every GPU that loads it, until exit),
 * so the call takes only inputs and outputs and calls no allocator.  Limits: the shape's partial sums must fit
 * 4 MiB and M <= 262144, otherwise the call is rejected with a message and nothing is launched.  The first call on
 * a device looks up the array's device address; make that first call before any stream capture.  All calls on a
 * device share the array (the slots a shape uses are reset on the stream at every call), so two calls that overlap on the
 * GPU - different streams, or different threads - race: serialise them.  No counterpart in the reference. */
int st_gemv_static(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X, void* Y,
                   int64_t B, int64_t M, int64_t N, void* stream);

/* Large-batch fused decode + tcgen05 GEMM, B >= 1 (meant for B > 32), M % 128 == 0.  Replaces `_C.tm`, `_C.th`,
 * `_C.tt` (statetree/csrc/kernels.cu:1892-1924, statetree/csrc/hop.cu:864-925, statetree/csrc/tt.cu:508-556).
 * ws: scratch of st_gemm_workspace_bytes() bytes (possibly 0) for the partial tiles of k ranges split between CTAs;
 * its contents do not matter on entry and are undefined on exit, so it must not be the buffer the GEMV entry points
 * use for their exchange slots (or must be refilled with 0xFF before they see it again).  cnt: int32
 * [M/128 * ceil(B/256)], zero on entry and on exit. */
int64_t st_gemm_workspace_bytes(int64_t M, int64_t N, int64_t B);
int st_gemm(const void* tree, const int32_t* eo, const uint32_t* el, const void* X, void* Y, float* Yf32, int64_t B,
            int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream);

/* st_gemm for a LIST of 1 to 4 matrices that share N and the activations (q / k / v, gate / up kept as separate
 * trees), in one launch: Y[i] [B, M[i]] = X W[i]^T, M[i] % 128 == 0.  The members' 128-row blocks form one grid, so
 * the list pays one launch, one pipeline fill and one epilogue.  trees / eo / el / Y / Yf32 / M are HOST arrays of n
 * entries (Yf32 or any of its entries may be NULL).  Same results as st_gemm on each member wherever both split the k
 * range alike.  The reference reaches the same end by fusing the trees at conversion time (statetree/model.py:22-24). */
int st_gemm_list(int64_t n, const void* const* trees, const int32_t* const* eo, const uint32_t* const* el, const void* X,
                 void* const* Y, float* const* Yf32, int64_t B, const int64_t* M, int64_t N, int32_t* cnt, void* stream);

/* ---- mixture of experts ----------------------------------------------------------------------------------------- */
/* y[s] = W[ids[s]] x[s / xdiv] for S (token, expert) slots; tp / eop / ebp / elp: int64 [E] device addresses of each
 * expert's tree, eo, eb and el tables (all experts M x N); ids int32 (ids64 = 0) or int64 (ids64 = 1), clamped to [0, E).
 * Replaces `_C.mvx` / `_C.mvwx` (statetree/csrc/kernels.cu:883-926, 1218-1246). */
int64_t st_moe_gemv_workspace_bytes(int64_t S, int64_t M, int64_t N);
int st_moe_gemv(const int64_t* tp, const int64_t* eop, const int64_t* ebp, const int64_t* elp, int64_t E, const void* X,
                const void* ids, int ids64, void* Y, int64_t S, int64_t M, int64_t N, int64_t xdiv, void* ws,
                int64_t ws_bytes, int32_t* cnt, void* stream);
/* The same product for slots grouped by expert in the moe_align_block_size layout with block size 8: sorted int32
 * [nblk * 8] slot ids padded with values >= S, bexp int32 [nblk] expert of each block (negative: skipped, another
 * rank's expert), npost int32 [1] number of used entries of sorted.  Rows of skipped blocks are not written.
 * Replaces `_C.mvg` / `_C.mvwg` / `_C.gtt` (statetree/csrc/kernels.cu:1043-1086, 1249-1279; statetree/csrc/gtt.cu:322-368). */
int64_t st_moe_group_workspace_bytes(int64_t nblk, int64_t M, int64_t N);
int st_moe_group_gemv(const int64_t* tp, const int64_t* eop, const int64_t* ebp, const int64_t* elp, int64_t E,
                      const void* X, const int32_t* sorted, const int32_t* bexp, const int32_t* npost, int64_t nblk,
                      void* Y, int64_t S, int64_t M, int64_t N, int64_t xdiv, void* ws, int64_t ws_bytes, int32_t* cnt,
                      void* stream);
/* Pairs grouped by expert in blocks of bs (8 for st_moe_group_gemv, 64 or 128 for st_moe_group_gemm): sorted int32
 * [nblk * bs] (pair indices, expert-major, original order inside an expert, runs padded to a multiple of bs with the
 * value S), bexp int32 [nblk], npost int32 [1] = entries of the first used_bins experts (used_bins = E, or E - 1 when
 * the last id collects the pairs of other ranks' experts, whose blocks the grouped kernels then never visit); ids
 * int64 (ids64 = 1) or int32 [S], clamped to [0, E); nblk >= S / bs + min(S, E); E <= 1024.  The reference takes
 * this layout from vLLM's moe_align_block_size (statetree/experts.py:52-120). */
int st_moe_align(const void* ids, int ids64, int64_t S, int64_t E, int64_t used_bins, int64_t bs, int32_t* sorted,
                 int32_t* bexp, int32_t* npost, int64_t nblk, void* stream);

/* Grouped fused decode + tcgen05 GEMM over per-expert trees, for many pairs per expert (prefill-sized calls):
 * y[pair] = W[expert of pair] x[pair / xdiv].  Replaces `_C.gtt` (statetree/csrc/gtt.cu:80-299, 322-368).
 *   st_moe_tensor_maps  writes one weight tensor map (st_moe_tensor_map_bytes() bytes each, 64-byte aligned) per
 *                       expert tree into maps_dev; trees_host is a HOST array of E device addresses.  Once per
 *                       expert set, outside graph capture.
 *   st_moe_gather       Xg[i, :] = X[sorted[i] / xdiv, :] for the used entries of sorted (rows = nblk * bs)
 *   st_moe_group_gemm   one CTA per (block of bs pairs, 128 rows of M): Y[sorted[i], :] = W[bexp[block]] Xg[i, :];
 *                       rows of padding entries and of blocks with a negative expert are not written; eop / elp as
 *                       for st_moe_gemv; M % 128 == 0, bs = 64 or 128.  Yf32 optional as for st_gemv. */
int64_t st_moe_tensor_map_bytes(void);
int st_moe_tensor_maps(const int64_t* trees_host, int64_t E, int64_t M, int64_t N, void* maps_dev, void* stream);
int st_moe_gather(const void* X, const int32_t* sorted, const int32_t* npost, int64_t rows, int64_t S, int64_t xdiv,
                  int64_t N, void* Xg, void* stream);
int st_moe_group_gemm(const void* maps, const int64_t* eop, const int64_t* elp, int64_t E, const void* Xg,
                      const int32_t* sorted, const int32_t* bexp, const int32_t* npost, int64_t nblk, int64_t bs,
                      void* Y, float* Yf32, int64_t S, int64_t M, int64_t N, void* stream);
/* Router of a mixture-of-experts layer in one launch: softmax over the E <= 1024 expert logits of each of T tokens
 * (BF16, or float32 with logits_f32 = 1), the K <= 32 largest probabilities in descending order (ties: the lower
 * expert first) -> ids int32 [T, K], w float32 [T, K]; renorm != 0 divides the K weights by their sum.  expert_map
 * (optional, int32 [E]: global id -> local id or -1) returns local ids; pairs of other ranks' experts get id 0 and
 * weight 0.  No counterpart in the reference (the model's own PyTorch code routes). */
int st_moe_route(const void* logits, int logits_f32, int64_t T, int64_t E, int64_t K, int renorm,
                 const int32_t* expert_map, int32_t* ids, float* w, void* stream);
/* out[t] = sum_j w[t, j] * Y[t * K + j] in fp32, expert order, BF16 out; w float32 (w_bf16 = 0) or BF16 (1).
 * Replaces `_C.wsum` (statetree/csrc/kernels.cu:1489-1535). */
int st_wsum(const void* Y, const void* w, int w_bf16, void* out, int64_t T, int64_t K, int64_t H, void* stream);
/* act[s, i] = silu(gu[s, i]) * gu[s, I + i]: silu in fp32, rounded to BF16, then multiplied (the rounding points of
 * statetree/csrc/kernels.cu:1327-1333). */
int st_silu_mul(const void* gu, void* act, int64_t S, int64_t I, void* stream);

/* ---- glue kernels of the decode step (no counterpart in the reference, which leaves them to PyTorch) --------------- */
/* x[r, :] += delta[r, :] (delta may be NULL), out[r, :] = RMSNorm(x[r, :]) * w; BF16, fp32 arithmetic. */
int st_add_rmsnorm(void* x, const void* delta, const void* w, void* out, int64_t rows, int64_t cols, double eps,
                   void* stream);
/* Per-head RMSNorm (weights wq / wk [128]) + rotary embedding (interleaved pairs; cos_t / sin_t float [max_pos, 64];
 * the position is the device scalar pos[0]) of the q and k heads of fused qkv rows [B, (hq + 2 hkv) * 128] with row
 * stride row_stride (elements) -> q_out [B, hq, 128], k_out [B, hkv, 128]. */
int st_qk_norm_rope(const void* qkv, int64_t row_stride, const void* wq, const void* wk, const float* cos_t,
                    const float* sin_t, const int64_t* pos, int64_t max_pos, void* q_out, void* k_out, int64_t B,
                    int64_t hq, int64_t hkv, double eps, void* stream);

/* ---- KV pages --------------------------------------------------------------------------------------------------- */
/* 6400 * H.  Replaces `_kv.page_bytes` (statetree/csrc/kvcache.cu:295). */
int64_t st_kv_page_bytes(int64_t H);
/* Append N tokens: K, V BF16 [N, H, 128] with token strides ks / vs (elements, heads contiguous); slot int64 [N]
 * (block * 16 + row, negative = skipped).  Replaces `_kv.append` (statetree/csrc/kvcache.cu:297-324). */
int st_kv_append(const void* K, const void* V, int64_t ks, int64_t vs, const int64_t* slot, int64_t N, int64_t H,
                 void* kv, int64_t nblocks, uint32_t* pool, int64_t P, int32_t* pool_cnt, int reuse, void* stream);
/* All pages -> dense BF16 Kd, Vd [nblocks, 16, H, 128].  Replaces `_kv.dequant` (statetree/csrc/kvcache.cu:326-336). */
int st_kv_dequant(const void* kv, int64_t nblocks, int64_t H, const uint32_t* pool, int64_t P, void* Kd, void* Vd,
                  void* stream);
/* Listed pages -> dense BF16 [n, 16, H, 128]; ids outside [0, nblocks) give zeros.  Replaces `_kv.dequant_blocks`
 * (statetree/csrc/kvcache.cu:338-354). */
int st_kv_dequant_blocks(const void* kv, int64_t nblocks, int64_t H, const uint32_t* pool, int64_t P,
                         const int32_t* blocks, int64_t n, void* Kd, void* Vd, void* stream);
/* Decode attention, one query token per sequence: q, out BF16 [B, Hq, 128] with token strides qs / os; bt int32
 * [B, bts] block table; lens int32 [B]; starts int32 [B] or NULL; S splits with >= minpps pages each; wo float
 * [B, Hq, S, 128] and wml float [B, Hq, S, 2] hold the split partials (unnormalised O; max and sum in the exp2
 * domain) when S > 1.  Replaces `_kv.attn` (statetree/csrc/kvcache.cu:536-585). */
int st_kv_attn(const void* q, int64_t qs, int64_t B, int64_t Hq, const void* kv, int64_t nblocks, int64_t Hkv,
               const uint32_t* pool, int64_t P, const int32_t* bt, int64_t bts, const int32_t* lens,
               const int32_t* starts, void* out, int64_t os, float* wo, float* wml, double scale, int64_t S,
               int64_t minpps, void* stream);

/* st_gemv (1 <= B <= 8) of a fused gate/up projection with the SwiGLU gate in the epilogue: the M = 2 I rows of the tree
 * are the gate and up projections interleaved in 16-row tiles (tile 2j = gate rows 16j .. 16j + 15, tile 2j + 1 = the
 * same rows of up); act BF16 [B, I] = silu(gate) * up with the rounding points of st_silu_mul (both products to BF16,
 * silu in fp32 to BF16, BF16 multiply).  Shapes whose work does not divide into whole tile pairs per CTA are rejected
 * (the caller then runs st_gemv + st_silu_mul).  The reference fuses the same step into its expert kernels only
 * (`mvwx` / `mvwg`, statetree/csrc/kernels.cu:1159-1279). */
int st_gemv_swiglu_supported(int64_t M, int64_t N, int64_t B);   /* 1 when st_gemv_swiglu takes the shape on this GPU */
int st_gemv_swiglu(const void* tree, const int32_t* eo, const uint32_t* eb, const uint32_t* el, const void* X, void* act,
                   int64_t B, int64_t M, int64_t N, void* ws, int64_t ws_bytes, int32_t* cnt, void* stream);

/* Decode step, one new token per sequence: st_qk_norm_rope for the query heads and st_kv_append of the step's K
 * (normalised and rotated by the appending warps themselves) and V rows, in one launch.  qkv BF16 [B, (hq + 2 hkv) *
 * 128] with row stride row_stride; slot int64 [B] (negative or outside the cache = no write); the pages are
 * bit-identical to st_qk_norm_rope followed by st_kv_append.  No single counterpart in the reference (its harness
 * leaves norm and rotary embedding to PyTorch and then calls `_kv.append`, statetree/csrc/kvcache.cu:297-324). */
int st_rope_kv_append(const void* qkv, int64_t row_stride, const void* wq, const void* wk, const float* cos_t,
                      const float* sin_t, const int64_t* pos, int64_t max_pos, void* q_out, int64_t B, int64_t hq,
                      int64_t hkv, double eps, const int64_t* slot, void* kv, int64_t nblocks, uint32_t* pool, int64_t P,
                      int32_t* pool_cnt, void* stream);

/* ---- tensor-parallel exchange over NVLink peer memory -------------------------------------------------------------- *
 * No counterpart in the reference: it has no communication code (under vLLM each rank runs the reference's kernels on
 * its shard and vLLM all-reduces the outputs of the row-parallel o / down projections with NCCL).  These entry points
 * do that all-reduce for the small decode-step tensors with plain peer loads and stores.
 * Set-up, once per process: st_comm_alloc gives this rank's communication buffer (st_comm_bytes() of device memory,
 * cleared); st_comm_export writes its 64-byte CUDA IPC handle, which the host code sends to the other ranks of the
 * node (any channel); st_comm_import maps a peer's handle and returns a device pointer valid in this process.  The
 * calls then take `bufs`, a host array of `world` device pointers indexed by rank (bufs[rank] = the own buffer).
 * Every rank must make the same sequence of calls with the same sizes.  Waits on peers are bounded by wall time
 * (st_comm_set_timeout_ms; 20 s unless set, long enough for a peer held up by a lazy module load or a graph capture);
 * a call that gives up leaves its output unwritten and sets the device status word: the step's result is then
 * invalid, so check st_device_status() at the step's sync point and redo the step (or fall back to NCCL). */
int64_t st_comm_bytes(void);
int st_comm_set_timeout_ms(int64_t ms);
int st_comm_alloc(void** buf);
int st_comm_free(void* buf);
int st_comm_export(void* buf, void* handle64);
int st_comm_import(const void* handle64, void** buf);
int st_comm_close(void* buf);
/* out[i] = sum over ranks of in[i], BF16, fp32 accumulation in rank order (the same bits on every rank); n a multiple
 * of 8, at most 524288 values; in / out 16-byte aligned, may be the same buffer. */
int st_allreduce(void* const* bufs, int rank, int world, const void* in, void* out, int64_t n, void* stream);
/* st_allreduce of delta [rows, cols] fused with st_add_rmsnorm: x += sum over ranks of delta; out = RMSNorm(x) * w.
 * rows <= 64, cols <= 8192 and a multiple of 8. */
int st_allreduce_add_rmsnorm(void* const* bufs, int rank, int world, void* x, const void* delta, const void* w,
                             void* out, int64_t rows, int64_t cols, double eps, void* stream);

/* The row-parallel product of a tensor-parallel group in ONE launch per rank: Y [B, M] (BF16, the same bits on every
 * rank) = sum over ranks of X_r [B, N_r] W_r [M, N_r]^T, where this rank passes its column shard (tree, eo, eb, el of
 * W_r) and its slice X_r of the activations.  The GEMV's reducer warp writes every finished fp32 tile sum into the
 * receive area of every rank's communication buffer (plain stores over NVLink, one self-validating word per value)
 * and then adds the ranks' words from its own buffer in rank order, so no second kernel and no flag round trip follow
 * the product, and the partial sums are added in fp32 (st_gemv + st_allreduce rounds them to BF16 first).
 * bufs / rank / world as for st_allreduce; ws as for st_gemv (st_gemv_workspace_bytes(M, N, B)); 1 <= B <= 32 and
 * (M / 16) * 128 * ceil(B / 8 rounded up to 1, 2 or 4) <= 131072 (M = 4096 at any B, M = 16384 at B <= 8).  Every rank
 * makes the same calls in the same order; the wait for the peers' sums is bounded (st_comm_set_timeout_ms), a rank
 * that never delivers leaves ERR_WAIT_PEER (5) in the status word and the affected outputs unwritten.  No counterpart
 * in the reference (vLLM all-reduces the outputs of its RowParallelLinear with NCCL). */
int st_gemv_allreduce(void* const* bufs, int rank, int world, const void* tree, const int32_t* eo, const uint32_t* eb,
                      const uint32_t* el, const void* X, void* Y, float* Yf32, int64_t B, int64_t M, int64_t N, void* ws,
                      int64_t ws_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif
