"""CPU oracle for the state-tree decode hot path: numpy front end of oracle/statetree_oracle.c.

TEST INFRASTRUCTURE ONLY.  Importable from tests/, the smoke check and the benchmark's CPU-baseline legs; the shipped
package never imports it (there is no CPU fallback on the product path).  All arrays are numpy; BF16 values travel as
uint16 bit patterns.  Each function names the reference code it restates in statetree_oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "liboracle.so")
_SRC = os.path.join(_DIR, "statetree_oracle.c")
_LIB = None

RECORD_BYTES = 1552
RKV = 1600
PAGE = 16


def build(force=False):
    """gcc -O3 -fopenmp -shared: compiles the C restatement next to its source (git-ignored)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", _SRC, "-o", _SO, "-lm"])
    return _SO


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(_SO):
            build()
        _LIB = ctypes.CDLL(_SO)
        _LIB.st_ref_encode.restype = ctypes.c_int64
        _LIB.st_ref_escape_count.restype = ctypes.c_int64
    return _LIB


def _p(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _i64(v):
    return ctypes.c_int64(int(v))


# ------------------------------------------------------------------------------------------------ bf16 helpers
def f32_to_bf16_bits(x):
    """round-to-nearest-even float32 -> bf16 bit patterns (uint16)"""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------------------------------------ weights
def encode(W):
    """W [M, N] uint16 (bf16 bits) -> dict(tree uint8 [M/16, N/64, 1552], esc_rows/esc_cols int32, esc_bits int16).
    Restates statetree/format.py:66-83."""
    W = np.ascontiguousarray(W, dtype=np.uint16)
    M, N = W.shape
    assert M % 16 == 0 and N % 64 == 0
    tree = np.empty((M // 16, N // 64, RECORD_BYTES), dtype=np.uint8)
    n = lib().st_ref_escape_count(_p(W), _i64(M), _i64(N))
    er, ec, eb = np.empty(n, np.int32), np.empty(n, np.int32), np.empty(n, np.int16)
    got = lib().st_ref_encode(_p(W), _i64(M), _i64(N), _p(tree), _p(er), _p(ec), _p(eb), _i64(n))
    assert got == n
    return dict(tree=tree, esc_rows=er, esc_cols=ec, esc_bits=eb)


def escape_count(W):
    W = np.ascontiguousarray(W, dtype=np.uint16)
    W2 = W.reshape(-1, W.shape[-1])
    return int(lib().st_ref_escape_count(_p(W2), _i64(W2.shape[0]), _i64(W2.shape[1])))


def decode(tree, esc_rows, esc_cols, esc_bits):
    """exact inverse of encode -> uint16 [M, N].  Restates statetree/format.py:101-121."""
    tree = np.ascontiguousarray(tree, dtype=np.uint8)
    T, NG, _ = tree.shape
    M, N = T * 16, NG * 64
    er = np.ascontiguousarray(esc_rows, dtype=np.int32)
    ec = np.ascontiguousarray(esc_cols, dtype=np.int32)
    eb = np.ascontiguousarray(esc_bits, dtype=np.int16)
    W = np.empty((M, N), dtype=np.uint16)
    lib().st_ref_decode(_p(tree), _i64(M), _i64(N), _p(er), _p(ec), _p(eb), _i64(er.size), _p(W))
    return W


def linear_f64(W, X):
    """fp64 product X W^T over bf16 bit patterns (the quantity the output tolerance is stated on)"""
    W = np.ascontiguousarray(W, dtype=np.uint16)
    X = np.ascontiguousarray(X, dtype=np.uint16)
    B, N = X.shape
    M = W.shape[0]
    Y = np.empty((B, M), dtype=np.float64)
    lib().st_ref_linear_f64(_p(W), _p(X), _i64(B), _i64(M), _i64(N), _p(Y))
    return Y


def linear_cpu(enc, X, scratch=None):
    """The reference's CPU path for one linear (decode_reference + a BF16 matmul, statetree/linear.py:883-886):
    returns uint16 [B, M]."""
    tree = np.ascontiguousarray(enc["tree"], dtype=np.uint8)
    T, NG, _ = tree.shape
    M, N = T * 16, NG * 64
    X = np.ascontiguousarray(X, dtype=np.uint16)
    B = X.shape[0]
    if scratch is None:
        scratch = np.empty((M, N), dtype=np.uint16)
    Y = np.empty((B, M), dtype=np.uint16)
    er, ec, eb = (np.ascontiguousarray(enc[k]) for k in ("esc_rows", "esc_cols", "esc_bits"))
    lib().st_ref_linear_cpu(_p(tree), _i64(M), _i64(N), _p(er), _p(ec), _p(eb), _i64(er.size), _p(X), _i64(B),
                            _p(scratch), _p(Y))
    return Y


def threads():
    return int(lib().st_ref_threads())


def set_threads(n):
    """OpenMP threads of the C restatement (launchers export OMP_NUM_THREADS=1; the timed baseline uses the host's cores)"""
    lib().st_ref_set_threads(int(n))


# ------------------------------------------------------------------------------------------------ KV pages
def kv_append(K, V, slots, kv, pool, pool_cnt, reuse=False):
    """K, V uint16 [N, H, 128]; slots int64 [N] (-1 = skip); kv uint8 [blocks, H, 2, 2, 1600] (in place); pool uint32
    [P, 16]; pool_cnt int32 [2].  Restates statetree/csrc/kvcache.cu:62-192 (single-threaded, token order)."""
    K = np.ascontiguousarray(K, dtype=np.uint16)
    V = np.ascontiguousarray(V, dtype=np.uint16)
    slots = np.ascontiguousarray(slots, dtype=np.int64)
    N, H, D = K.shape
    assert D == 128 and kv.dtype == np.uint8 and kv.flags.c_contiguous and kv.shape[1:] == (H, 2, 2, RKV)
    assert pool.dtype == np.uint32 and pool.flags.c_contiguous and pool_cnt.dtype == np.int32
    lib().st_ref_kv_append(_p(K), _p(V), _i64(H * D), _i64(H * D), _p(slots), _i64(N), ctypes.c_int(H), _p(kv),
                           _p(pool), ctypes.c_int(pool.shape[0]), _p(pool_cnt), ctypes.c_int(1 if reuse else 0))


def kv_dequant_blocks(kv, pool, blocks=None):
    """listed pages (or all) -> Kd, Vd uint16 [n, 16, H, 128].  Restates statetree/csrc/kvcache.cu:241-293."""
    nb, H = kv.shape[0], kv.shape[1]
    if blocks is not None:
        blocks = np.ascontiguousarray(blocks, dtype=np.int32)
    n = nb if blocks is None else blocks.size
    Kd = np.empty((n, PAGE, H, 128), dtype=np.uint16)
    Vd = np.empty_like(Kd)
    lib().st_ref_kv_dequant_blocks(_p(kv), _i64(nb), ctypes.c_int(H), _p(pool), ctypes.c_int(pool.shape[0]),
                                   _p(blocks), _i64(n), _p(Kd), _p(Vd))
    return Kd, Vd


def kv_attn_f64(q, kv, pool, bt, lens, scale, starts=None):
    """fp64 decode attention over the pages -> float64 [B, Hq, 128].  Semantics of statetree/csrc/kvcache.cu:399-527."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    B, Hq, D = q.shape
    bt = np.ascontiguousarray(bt, dtype=np.int32)
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    if starts is not None:
        starts = np.ascontiguousarray(starts, dtype=np.int32)
    out = np.empty((B, Hq, D), dtype=np.float64)
    lib().st_ref_kv_attn_f64(_p(q), _i64(B), ctypes.c_int(Hq), _p(kv), _i64(kv.shape[0]), ctypes.c_int(kv.shape[1]),
                             _p(pool), ctypes.c_int(pool.shape[0]), _p(bt), _i64(bt.shape[1]), _p(lens), _p(starts),
                             ctypes.c_double(scale), _p(out))
    return out


# ------------------------------------------------------------------------------------------------ tiny pure-Python
def encode_record_py(block):
    """One 16 x 64 block (uint16) -> (1552 record bytes, [(row, col, bits)]) with plain Python loops: an independent
    second statement of statetree/format.py:9-12, 43-62 used to cross-check the C code on small cases."""
    rec = np.zeros(RECORD_BYTES, dtype=np.uint8)
    esc = []
    b = np.asarray(block, dtype=np.uint16)
    for r in range(16):
        e = (b[r] >> 7) & 0xFF
        E = int(e.max())
        D = E - e.astype(np.int64)
        x = D > 14
        for c in range(64):
            p = c ^ 1
            l, s_, t, hi = c // 2, (c // 2) >> 3, (c // 2) & 3, ((c // 2) >> 2) & 1
            lo = (s_ >> 1) * 512 + ((r & 7) * 4 + t) * 16 + ((s_ & 1) * 2 + (r >> 3)) * 4 + 2 * hi + (c & 1)
            so = 1024 + ((r & 7) * 4 + t) * 16 + s_ * 4 + 2 * hi + (c & 1)
            mant = 0 if x[c] else int(b[r, c]) & 0x7F
            ps = 0 if x[p] else int(b[r, p]) >> 15
            rec[lo] = (mant << 1) | ps
            d = 15 if x[c] else int(D[c])
            rec[so] |= d if r < 8 else d << 4
            if x[c]:
                esc.append((r, c, int(b[r, c])))
        rec[1536 + 2 * (r & 7) + (r >> 3)] = E
    return rec, esc
