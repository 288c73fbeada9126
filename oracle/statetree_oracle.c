/* CPU oracle for the state-tree decode hot path.  TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA kernels
 * (parity tests, the smoke check) and the timed CPU baseline of the benchmark.  Nothing in the shipped library calls,
 * links or loads this file; the product path has no CPU fallback.
 *
 * It restates, in plain C, the algorithm of the reference implementation (paths relative to the reference project):
 *   - weight format encode / decode ............ statetree/format.py:43-83, 101-121 (record layout: format.py:9-12,
 *                                                 closed-form offsets: statetree/csrc/kvcache.cu:31-38)
 *   - 4-weight decode identity ................. statetree/csrc/kernels.cu:45-50
 *   - KV page append (slots, extension chain) .. statetree/csrc/kvcache.cu:62-192
 *   - KV record decode + patches ............... statetree/csrc/kvcache.cu:197-238
 *   - dequant / dequant_blocks ................. statetree/csrc/kvcache.cu:241-293
 *   - decode attention semantics ............... statetree/csrc/kvcache.cu:399-527 (computed here in fp64)
 *   - linear y = x W^T ......................... statetree/linear.py:883-886 (decode + matmul), fp64 and fp32 variants
 * Parity pin: the weight format functions are checked byte for byte against fixtures produced by importing the
 * reference's format.py (tests/golden/make_golden.py).  The KV record bytes are pinned the same way (a record is the
 * format.py encoding of a 16-token x 64-dim block); the escape-pool chain has no CPU implementation in the reference
 * and is pinned only through losslessness (decode(append(x)) == x).
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC statetree_oracle.c -o liboracle.so   (see oracle/build.py)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define REC 1552
#define RKV 1600
#define PAGE 16
#define HD 128
#define NSLOT 11
#define XSLOT 15

/* ---- record geometry (statetree/format.py:9-12; statetree/csrc/kvcache.cu:31-38) ---------------------------------
 * element (r in 0..15, c in 0..63) of a 16 x 64 block; l = c / 2 is its bf16 pair */
static inline int leaf_pos(int r, int c) {
  const int l = c >> 1, s = l >> 3, t = l & 3, hi = (l >> 2) & 1;
  return (s >> 1) * 512 + ((r & 7) * 4 + t) * 16 + ((s & 1) * 2 + (r >> 3)) * 4 + 2 * hi + (c & 1);
}
static inline int state_pos(int r, int c) {
  const int l = c >> 1, s = l >> 3, t = l & 3, hi = (l >> 2) & 1;
  return 1024 + ((r & 7) * 4 + t) * 16 + s * 4 + 2 * hi + (c & 1);
}
static inline int node_pos(int r) { return 1536 + 2 * (r & 7) + (r >> 3); }

/* encode one row (64 bf16 bit patterns) into row r of a record; returns the number of escapes and lists their
 * columns in esc_c (ascending).  statetree/format.py:46-59 */
static int encode_row(const uint16_t* w, int r, uint8_t* rec, int* esc_c) {
  int E = 0, n = 0;
  for (int c = 0; c < 64; ++c) {
    const int e = (w[c] >> 7) & 0xFF;
    if (e > E) E = e;
  }
  int D[64], X[64];
  for (int c = 0; c < 64; ++c) {
    D[c] = E - ((w[c] >> 7) & 0xFF);
    X[c] = D[c] > 14;
    if (X[c]) esc_c[n++] = c;
  }
  for (int c = 0; c < 64; ++c) {
    const int p = c ^ 1;
    const unsigned mant = X[c] ? 0u : (w[c] & 0x7Fu);
    const unsigned psign = X[p] ? 0u : (unsigned)(w[p] >> 15);
    rec[leaf_pos(r, c)] = (uint8_t)((mant << 1) | psign);
    const unsigned d = X[c] ? 15u : (unsigned)D[c];
    uint8_t* st = rec + state_pos(r, c);
    *st = (r < 8) ? (uint8_t)((*st & 0xF0u) | d) : (uint8_t)((*st & 0x0Fu) | (d << 4));
  }
  rec[node_pos(r)] = (uint8_t)E;
  return n;
}

/* decode element (r, c) of a record, ignoring escapes.  statetree/format.py:106-118, kernels.cu:45-50 */
static inline uint16_t decode_elem(const uint8_t* rec, int r, int c) {
  const unsigned leaf = rec[leaf_pos(r, c)], pleaf = rec[leaf_pos(r, c ^ 1)];
  const unsigned sb = rec[state_pos(r, c)];
  const int d = (r < 8) ? (int)(sb & 15u) : (int)(sb >> 4);
  int ex = (int)rec[node_pos(r)] - d;
  if (ex < 0) ex = 0;
  return (uint16_t)(((pleaf & 1u) << 15) | ((unsigned)ex << 7) | (leaf >> 1));
}

/* ---- weights ---------------------------------------------------------------------------------------------------- */
/* W [M, N] bf16 bits -> tree [M/16, N/64, 1552]; escapes in (row, col) ascending order.  Returns the escape count
 * (also when it exceeds cap: then only the first cap are stored).  statetree/format.py:66-83 */
int64_t st_ref_encode(const uint16_t* W, int64_t M, int64_t N, uint8_t* tree, int32_t* esc_rows, int32_t* esc_cols,
                      int16_t* esc_bits, int64_t cap) {
  const int64_t T = M / 16, NG = N / 64;
  int64_t* cnt = (int64_t*)calloc((size_t)T + 1, sizeof(int64_t));
  /* pass 1: records + per-tile escape counts */
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    int64_t k = 0;
    int ec[64];
    for (int64_t g = 0; g < NG; ++g) {
      uint8_t* rec = tree + (t * NG + g) * REC;
      memset(rec, 0, REC);
      for (int r = 0; r < 16; ++r) k += encode_row(W + (t * 16 + r) * N + g * 64, r, rec, ec);
    }
    cnt[t + 1] = k;
  }
  for (int64_t t = 0; t < T; ++t) cnt[t + 1] += cnt[t];
  const int64_t total = cnt[T];
  /* pass 2: escape list in (row, col) order */
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    int64_t k = cnt[t];
    for (int r = 0; r < 16; ++r) {
      const uint16_t* row = W + (t * 16 + r) * N;
      for (int64_t g = 0; g < NG; ++g) {
        int E = 0;
        for (int c = 0; c < 64; ++c) {
          const int e = (row[g * 64 + c] >> 7) & 0xFF;
          if (e > E) E = e;
        }
        for (int c = 0; c < 64; ++c)
          if (E - ((row[g * 64 + c] >> 7) & 0xFF) > 14) {
            if (k < cap) {
              esc_rows[k] = (int32_t)(t * 16 + r);
              esc_cols[k] = (int32_t)(g * 64 + c);
              esc_bits[k] = (int16_t)row[g * 64 + c];
            }
            ++k;
          }
      }
    }
  }
  free(cnt);
  return total;
}

/* statetree/format.py:87-97 */
int64_t st_ref_escape_count(const uint16_t* W, int64_t rows, int64_t N) {
  int64_t n = 0;
#pragma omp parallel for reduction(+ : n) schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t g = 0; g < N / 64; ++g) {
      int E = 0;
      for (int c = 0; c < 64; ++c) {
        const int e = (W[r * N + g * 64 + c] >> 7) & 0xFF;
        if (e > E) E = e;
      }
      for (int c = 0; c < 64; ++c) n += (E - ((W[r * N + g * 64 + c] >> 7) & 0xFF)) > 14;
    }
  return n;
}

/* tree -> W [M, N] bf16 bits, escapes scattered over.  statetree/format.py:101-121 */
void st_ref_decode(const uint8_t* tree, int64_t M, int64_t N, const int32_t* esc_rows, const int32_t* esc_cols,
                   const int16_t* esc_bits, int64_t n_esc, uint16_t* W) {
  const int64_t T = M / 16, NG = N / 64;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t)
    for (int64_t g = 0; g < NG; ++g) {
      const uint8_t* rec = tree + (t * NG + g) * REC;
      for (int r = 0; r < 16; ++r)
        for (int c = 0; c < 64; ++c) W[(t * 16 + r) * N + g * 64 + c] = decode_elem(rec, r, c);
    }
  for (int64_t i = 0; i < n_esc; ++i) W[(int64_t)esc_rows[i] * N + esc_cols[i]] = (uint16_t)esc_bits[i];
}

static inline float bf2f(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f2bf(float f) { /* round to nearest even, as __float2bfloat16_rn for finite values */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u) return (uint16_t)((u >> 16) | ((u & 0xFFFFu) ? 0x40u : 0u));
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* Y[B, M] (fp64) = X[B, N] W[M, N]^T over bf16 bit patterns: the exact product the parity tolerance is stated on */
void st_ref_linear_f64(const uint16_t* W, const uint16_t* X, int64_t B, int64_t M, int64_t N, double* Y) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t b = 0; b < B; ++b) {
      double s = 0.0;
      for (int64_t n = 0; n < N; ++n) s += (double)bf2f(W[m * N + n]) * (double)bf2f(X[b * N + n]);
      Y[b * M + m] = s;
    }
}

/* the reference's CPU path for a linear: decode the tree, then a BF16 matmul with fp32 accumulation and BF16
 * round-to-nearest output (statetree/linear.py:883-886 run on the host).  scratch: M * N bf16. */
void st_ref_linear_cpu(const uint8_t* tree, int64_t M, int64_t N, const int32_t* esc_rows, const int32_t* esc_cols,
                       const int16_t* esc_bits, int64_t n_esc, const uint16_t* X, int64_t B, uint16_t* scratch,
                       uint16_t* Y) {
  st_ref_decode(tree, M, N, esc_rows, esc_cols, esc_bits, n_esc, scratch);
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t b = 0; b < B; ++b) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      const uint16_t* w = scratch + m * N;
      const uint16_t* x = X + b * N;
      for (int64_t n = 0; n < N; n += 8)
        for (int j = 0; j < 8; ++j) acc[j] += bf2f(w[n + j]) * bf2f(x[n + j]);
      Y[b * M + m] = f2bf(((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7])));
    }
}

/* ---- KV pages --------------------------------------------------------------------------------------------------- */
static inline uint8_t* kv_record(uint8_t* kv, int64_t blk, int H, int h, int kvi, int half) {
  return kv + ((((size_t)blk * H + h) * 2 + kvi) * 2 + half) * RKV;
}

typedef struct {
  uint32_t* pool;
  int32_t* pool_cnt;
  int P;
  int cnt, xh, xt, xc;
  uint32_t* slots;
} put_state;

/* append one escape entry: the 11 in-record slots first, then the extension chain.  kvcache.cu:104-141 */
static void put_entry(put_state* s, uint32_t e) {
  if (s->cnt < NSLOT) {
    s->slots[s->cnt++] = e;
    return;
  }
  if (s->xh >= 0 && s->xt < 0) { /* continue an existing chain at its first non-full block */
    s->xt = s->xh;
    for (int hops = 0; hops < 4096; ++hops) {
      const uint32_t w0 = s->pool[(size_t)s->xt * 16];
      const int nx = (int)(w0 >> 8) - 1;
      s->xc = (int)(w0 & 0xFF);
      if (s->xc < XSLOT || nx < 0 || nx >= s->P) break;
      s->xt = nx;
    }
  }
  if (s->xt >= 0 && s->xc == XSLOT) { /* full: a recycled block further down the chain, if any */
    const int nx = (int)(s->pool[(size_t)s->xt * 16] >> 8) - 1;
    if (nx >= 0 && nx < s->P) {
      s->xt = nx;
      s->xc = (int)(s->pool[(size_t)s->xt * 16] & 0xFF);
    }
  }
  if (s->xt < 0 || s->xc == XSLOT) {
    const int nb = s->pool_cnt[0]++;
    if (nb >= s->P) {
      s->pool_cnt[1] = 1; /* pool exhausted: flagged, never silently lossy */
      return;
    }
    s->pool[(size_t)nb * 16] = 0;
    if (s->xt < 0) s->xh = nb;
    else s->pool[(size_t)s->xt * 16] = (s->pool[(size_t)s->xt * 16] & 0xFFu) | ((uint32_t)(nb + 1) << 8);
    s->xt = nb;
    s->xc = 0;
  }
  s->pool[(size_t)s->xt * 16 + 1 + s->xc] = e;
  ++s->xc;
  s->pool[(size_t)s->xt * 16] = (s->pool[(size_t)s->xt * 16] & ~0xFFu) | (uint32_t)s->xc;
}

/* K, V [N, H, 128] bf16 bits with token strides ks / vs (elements); slot[n] = block * 16 + row, -1 = skip.
 * kv: uint8 [blocks, H, 2, 2, 1600]; pool: uint32 [P, 16]; pool_cnt: int32 [2].  kvcache.cu:62-192 */
void st_ref_kv_append(const uint16_t* K, const uint16_t* V, int64_t ks, int64_t vs, const int64_t* slot, int64_t N,
                      int H, uint8_t* kv, uint32_t* pool, int P, int32_t* pool_cnt, int reuse) {
  for (int64_t n = 0; n < N; ++n) {
    const int64_t s0 = slot[n];
    if (s0 < 0) continue;
    const int64_t blk = s0 / PAGE;
    if (n > 0) {
      const int64_t sp = slot[n - 1];
      if (sp >= 0 && sp + 1 == s0 && sp / PAGE == blk) continue; /* not the start of a segment */
    }
    for (int q = 0; q < H * 4; ++q) {
      const int h = q >> 2, kvi = (q >> 1) & 1, half = q & 1;
      uint8_t* rec = kv_record(kv, blk, H, h, kvi, half);
      uint32_t* hdr = (uint32_t*)(rec + REC);
      uint32_t head;
      if (s0 % PAGE == 0) { /* fresh page */
        int keep = -1;
        if (reuse) {
          const uint32_t oh = *hdr;
          if ((oh & 16u) && (int)(oh >> 8) < P) keep = (int)(oh >> 8);
        }
        memset(rec, 0, RKV);
        if (keep >= 0) {
          int hops = 0;
          for (int b = keep; b >= 0 && b < P && hops < 4096; ++hops) {
            const uint32_t w0 = pool[(size_t)b * 16];
            pool[(size_t)b * 16] = w0 & ~0xFFu;
            b = (int)(w0 >> 8) - 1;
          }
        }
        head = keep >= 0 ? (16u | ((uint32_t)keep << 8)) : 0u;
      } else {
        head = *hdr;
      }
      put_state st;
      st.pool = pool; st.pool_cnt = pool_cnt; st.P = P;
      st.cnt = (int)(head & 15u);
      st.xh = (head & 16u) ? (int)(head >> 8) : -1;
      st.xt = -1; st.xc = 0;
      st.slots = hdr + 1;
      for (int64_t m = n; m < N; ++m) {
        const int64_t sm = slot[m];
        if (m > n && !(sm >= 0 && sm == slot[m - 1] + 1 && sm / PAGE == blk)) break;
        const int r = (int)(sm % PAGE);
        const uint16_t* src = (kvi ? V + m * vs : K + m * ks) + h * HD + half * 64;
        int ec[64];
        const int ne = encode_row(src, r, rec, ec);
        for (int i = 0; i < ne; ++i)
          put_entry(&st, ((uint32_t)src[ec[i]] << 16) | ((uint32_t)r << 6) | (uint32_t)ec[i]);
      }
      *hdr = (uint32_t)st.cnt | (st.xh >= 0 ? 16u | ((uint32_t)st.xh << 8) : 0u);
    }
  }
}

/* one record (+ slots + chain) -> 16 x 64 bf16 bits, out[r * ostride + c].  kvcache.cu:197-238 */
static void kv_decode_record(const uint8_t* rec, const uint32_t* pool, int P, uint16_t* out, int64_t ostride) {
  for (int r = 0; r < 16; ++r)
    for (int c = 0; c < 64; ++c) out[r * ostride + c] = decode_elem(rec, r, c);
  uint32_t head;
  memcpy(&head, rec + REC, 4);
  int cnt = (int)(head & 15u);
  if (cnt > NSLOT) cnt = NSLOT;
  const uint32_t* sl = (const uint32_t*)(rec + REC + 4);
  for (int i = 0; i < cnt; ++i) out[((sl[i] >> 6) & 15u) * ostride + (sl[i] & 63u)] = (uint16_t)(sl[i] >> 16);
  if (head & 16u) {
    int hops = 0;
    for (int b = (int)(head >> 8); b >= 0 && b < P && hops < 4096; ++hops) {
      const uint32_t w0 = pool[(size_t)b * 16];
      int xc = (int)(w0 & 0xFF);
      if (xc > XSLOT) xc = XSLOT;
      for (int i = 0; i < xc; ++i) {
        const uint32_t e = pool[(size_t)b * 16 + 1 + i];
        out[((e >> 6) & 15u) * ostride + (e & 63u)] = (uint16_t)(e >> 16);
      }
      b = (int)(w0 >> 8) - 1;
    }
  }
}

/* listed pages -> dense Kd, Vd [n, 16, H, 128]; a block id outside [0, nblocks) gives zeros.  kvcache.cu:263-293.
 * blocks == NULL: every page in order (kvcache.cu:241-261). */
void st_ref_kv_dequant_blocks(const uint8_t* kv, int64_t nblocks, int H, const uint32_t* pool, int P,
                              const int32_t* blocks, int64_t n, uint16_t* Kd, uint16_t* Vd) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const int64_t blk = blocks ? blocks[i] : i;
    for (int h = 0; h < H; ++h)
      for (int kvi = 0; kvi < 2; ++kvi)
        for (int half = 0; half < 2; ++half) {
          uint16_t* out = (kvi ? Vd : Kd) + ((size_t)i * PAGE * H + h) * HD + half * 64;
          if (blk >= 0 && blk < nblocks)
            kv_decode_record(kv_record((uint8_t*)kv, blk, H, h, kvi, half), pool, P, out, (int64_t)H * HD);
          else
            for (int r = 0; r < 16; ++r) memset(out + (size_t)r * H * HD, 0, 64 * 2);
        }
  }
}

/* decode attention over the pages, fp64: out[b, hq, :] = softmax(q K^T scale) V over tokens [starts[b], lens[b]);
 * lens[b] == 0 -> zeros.  q [B, Hq, 128] bf16 bits; bt int32 [B, bts].  kvcache.cu:399-527 */
void st_ref_kv_attn_f64(const uint16_t* q, int64_t B, int Hq, const uint8_t* kv, int64_t nblocks, int Hkv,
                        const uint32_t* pool, int P, const int32_t* bt, int64_t bts, const int32_t* lens,
                        const int32_t* starts, double scale, double* out) {
  const int G = Hq / Hkv;
#pragma omp parallel for schedule(dynamic)
  for (int64_t bh = 0; bh < B * Hkv; ++bh) {
    const int64_t b = bh / Hkv;
    const int h = (int)(bh % Hkv);
    const int len = lens[b], st0 = starts ? starts[b] : 0;
    const int ntok = len > st0 ? len : 0;
    double* o = out + ((size_t)b * Hq + (size_t)h * G) * HD;
    for (int i = 0; i < G * HD; ++i) o[i] = 0.0;
    if (ntok <= 0) continue;
    const int npg = (len + PAGE - 1) / PAGE;
    uint16_t* Kd = (uint16_t*)malloc((size_t)npg * PAGE * HD * 2 * sizeof(uint16_t));
    uint16_t* Vd = Kd + (size_t)npg * PAGE * HD;
    for (int p = st0 / PAGE; p < npg; ++p) {
      const int64_t blk = bt[b * bts + p];
      for (int half = 0; half < 2; ++half) {
        kv_decode_record(kv_record((uint8_t*)kv, blk, Hkv, h, 0, half), pool, P, Kd + (size_t)p * PAGE * HD + half * 64, HD);
        kv_decode_record(kv_record((uint8_t*)kv, blk, Hkv, h, 1, half), pool, P, Vd + (size_t)p * PAGE * HD + half * 64, HD);
      }
    }
    double* sc = (double*)malloc((size_t)len * sizeof(double));
    for (int g = 0; g < G; ++g) {
      const uint16_t* qp = q + ((size_t)b * Hq + (size_t)h * G + g) * HD;
      double mx = -INFINITY;
      for (int t = st0; t < len; ++t) {
        double s = 0.0;
        for (int d = 0; d < HD; ++d) s += (double)bf2f(qp[d]) * (double)bf2f(Kd[(size_t)t * HD + d]);
        sc[t] = s * scale;
        if (sc[t] > mx) mx = sc[t];
      }
      double l = 0.0;
      for (int t = st0; t < len; ++t) {
        sc[t] = exp(sc[t] - mx);
        l += sc[t];
      }
      for (int t = st0; t < len; ++t) {
        const double p = sc[t] / l;
        for (int d = 0; d < HD; ++d) o[g * HD + d] += p * (double)bf2f(Vd[(size_t)t * HD + d]);
      }
    }
    free(sc);
    free(Kd);
  }
}

/* launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks for the cores it is allowed to use */
void st_ref_set_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int st_ref_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}
