"""Loads the C-ABI kernel library (libstatetree_b200.so) and exposes it as two objects with the call shapes of the
reference's extension modules: ext() stands where `statetree._C` stood and kv_ext() where `statetree._kv` stood
(reference: statetree/ops.py:7-27, 85-103).  Tensors are passed as device pointers plus sizes; the launch goes to
torch's current stream of the tensors' device.  There is no fallback: a missing library or a non-CUDA tensor raises.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# STATETREE_B200_LIB names another build of the same library (the reference accepts a prebuilt extension the same way,
# statetree/ops.py:7-27); the ABI version is checked either way
LIB_PATH = os.environ.get("STATETREE_B200_LIB") or os.path.join(_HERE, "libstatetree_b200.so")
ABI = 2
_LIB = None

_i64, _int, _vp, _dbl = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_double

_SIGNATURES = {
    "st_abi_version": (_int, []),
    "st_last_error": (ctypes.c_char_p, []),
    "st_device_status": (_int, []),
    "st_dec": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "st_rows": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _i64, _vp, _vp]),
    "st_gemv_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "st_gemv": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "st_gemv_static": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "st_gemv_allreduce": (_int, [_vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "st_gemv_prenorm_supported": (_int, [_i64, _i64, _i64, _int]),
    "st_gemv_prenorm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_double, _vp, _vp, _i64, _i64, _i64, _int, _vp,
                               _i64, _vp]),
    "st_moe_route": (_int, [_vp, _int, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "st_gemm_list": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp]),
    "st_gemv_list_workspace_bytes": (_i64, [_i64, _vp, _i64, _i64]),
    "st_gemv_list": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "st_gemm_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "st_gemm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "st_moe_gemv_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "st_moe_gemv": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "st_moe_group_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "st_moe_group_gemv": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp,
                                 _i64, _vp, _vp]),
    "st_wsum": (_int, [_vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "st_silu_mul": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "st_add_rmsnorm": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _dbl, _vp]),
    "st_qk_norm_rope": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _dbl, _vp]),
    "st_kv_page_bytes": (_i64, [_i64]),
    "st_kv_append": (_int, [_vp, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _int, _vp]),
    "st_kv_dequant": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp]),
    "st_kv_dequant_blocks": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp]),
    "st_gemv_swiglu_supported": (_int, [_i64, _i64, _i64]),
    "st_gemv_swiglu": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "st_rope_kv_append": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _dbl, _vp, _vp, _i64,
                                 _vp, _i64, _vp, _vp]),
    "st_moe_align": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "st_moe_tensor_map_bytes": (_i64, []),
    "st_moe_tensor_maps": (_int, [_vp, _i64, _i64, _i64, _vp, _vp]),
    "st_moe_gather": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "st_moe_group_gemm": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _i64, _i64, _vp]),
    "st_comm_bytes": (_i64, []),
    "st_comm_set_timeout_ms": (_int, [_i64]),
    "st_comm_alloc": (_int, [ctypes.POINTER(ctypes.c_void_p)]),
    "st_comm_free": (_int, [_vp]),
    "st_comm_export": (_int, [_vp, _vp]),
    "st_comm_import": (_int, [_vp, ctypes.POINTER(ctypes.c_void_p)]),
    "st_comm_close": (_int, [_vp]),
    "st_allreduce": (_int, [ctypes.POINTER(ctypes.c_void_p), _int, _int, _vp, _vp, _i64, _vp]),
    "st_allreduce_add_rmsnorm": (_int, [ctypes.POINTER(ctypes.c_void_p), _int, _int, _vp, _vp, _vp, _vp, _i64, _i64,
                                        ctypes.c_double, _vp]),
    "st_kv_attn": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp,
                          _dbl, _i64, _i64, _vp]),
}


def exported_symbols():
    """names the header include/statetree_b200.h declares (used by the load test)"""
    return sorted(_SIGNATURES)


def lib():
    """the ctypes handle; raises when the library has not been built (python statetree-representation_b200/build.py)"""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"statetree_b200: {LIB_PATH} is missing; build it with "
                               "`python statetree-representation_b200/build.py` (there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)                       # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        if L.st_abi_version() != ABI:
            raise RuntimeError(f"statetree_b200: library ABI {L.st_abi_version()} != {ABI}; rebuild it")
        _LIB = L
    return _LIB


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("statetree_b200: the kernels take CUDA tensors only (no CPU path)")
    return t.data_ptr()


def _ctx(t):
    if not t.is_cuda:
        raise RuntimeError("statetree_b200: the kernels take CUDA tensors only (no CPU path)")
    return torch.cuda.device(t.device)


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(rc):
    if rc != 0:
        raise RuntimeError(lib().st_last_error().decode())


def device_status():
    """0 unless a kernel gave up on one of its bounded waits since the last call (synchronises)"""
    return int(lib().st_device_status())


class _Weights:
    """call shapes of the reference's `statetree._C` entry points that this library keeps"""
    ABI = ABI

    @staticmethod
    def dec(T, EO, EL, W):
        M, N = W.shape
        with _ctx(T):
            _check(lib().st_dec(_ptr(T), _ptr(EO), _ptr(EL), M, N, _ptr(W), _stream(T)))

    @staticmethod
    def rows(T, EO, EL, ids, out):
        M, N = T.shape[0] * 16, T.shape[1] * 64
        with _ctx(T):
            _check(lib().st_rows(_ptr(T), _ptr(EO), _ptr(EL), M, N, _ptr(ids), ids.numel(), _ptr(out), _stream(T)))

    @staticmethod
    def gemv_workspace_bytes(M, N, B):
        return int(lib().st_gemv_workspace_bytes(M, N, B))

    @staticmethod
    def gemv(T, EO, EB, EL, X, Y, WS, CNT, Yf32=None):
        B, N = X.shape
        M = Y.shape[1]
        with _ctx(T):
            _check(lib().st_gemv(_ptr(T), _ptr(EO), _ptr(EB), _ptr(EL), _ptr(X), _ptr(Y), _ptr(Yf32), B, M, N, _ptr(WS),
                                 WS.numel() * WS.element_size(), _ptr(CNT), _stream(T)))

    @staticmethod
    def gemv_static(T, EO, EB, EL, X, Y):
        """the GEMV without caller workspaces (for callers that cannot allocate): scratch built into the library"""
        B, N = X.shape
        M = Y.shape[1]
        with _ctx(T):
            _check(lib().st_gemv_static(_ptr(T), _ptr(EO), _ptr(EB), _ptr(EL), _ptr(X), _ptr(Y), B, M, N, _stream(T)))

    @staticmethod
    def gemv_list_workspace_bytes(Ms, N, B):
        arr = (ctypes.c_int64 * len(Ms))(*Ms)
        return int(lib().st_gemv_list_workspace_bytes(len(Ms), arr, N, B))

    @staticmethod
    def gemv_list_args(tabs, Ys, Yf32s=None):
        """host pointer arrays of a list call: tabs = [(T, EO, EB, EL), ...] (1 to 4 matrices that share their column
        count), Ys = their outputs [B, M_i].  Build once for fixed buffers, pass to gemv_list on every call."""
        n = len(tabs)
        VP = ctypes.c_void_p * n
        cols = [VP(*[_ptr(t[k]) for t in tabs]) for k in range(4)]
        ys = VP(*[_ptr(y) for y in Ys])
        yf = VP(*[_ptr(y) for y in Yf32s]) if Yf32s is not None else None
        Ms = (ctypes.c_int64 * n)(*[t[0].shape[0] * 16 for t in tabs])
        return (n, cols[0], cols[1], cols[2], cols[3], ys, yf, Ms, tabs[0][0].shape[1] * 64, tabs[0][0].device)

    @staticmethod
    def gemv_list(args, X, WS):
        """Y_i = X W_i^T for every member of the list, in one launch"""
        n, t, eo, eb, el, ys, yf, Ms, N, dev = args
        B = X.shape[0]
        if X.shape[1] != N or not X.is_contiguous():
            raise RuntimeError(f"gemv_list: X must be contiguous [B, {N}]")
        with torch.cuda.device(dev):
            _check(lib().st_gemv_list(n, t, eo, eb, el, _ptr(X), ys, yf, B, Ms, N, _ptr(WS),
                                      WS.numel() * WS.element_size(), torch.cuda.current_stream(dev).cuda_stream))

    @staticmethod
    def gemm_list(args, X, CNT):
        """the same list (gemv_list_args; the eb column is not used) through the tcgen05 GEMM: any batch, rows % 128 == 0"""
        n, t, eo, eb, el, ys, yf, Ms, N, dev = args
        B = X.shape[0]
        if X.shape[1] != N or not X.is_contiguous():
            raise RuntimeError(f"gemm_list: X must be contiguous [B, {N}]")
        with torch.cuda.device(dev):
            _check(lib().st_gemm_list(n, t, eo, el, _ptr(X), ys, yf, B, Ms, N, _ptr(CNT),
                                      torch.cuda.current_stream(dev).cuda_stream))

    @staticmethod
    def gemv_prenorm_supported(M, N, B, act=False):
        return bool(lib().st_gemv_prenorm_supported(M, N, B, 1 if act else 0))

    @staticmethod
    def gemv_prenorm(T, EO, EB, EL, x, delta, norm_w, eps, x_out, Y, WS, act=False):
        """Y = RMSNorm(x + delta) * norm_w times W^T (act: the SwiGLU of a gate / up tree), x_out = x + delta"""
        B, N = x.shape
        M = T.shape[0] * 16
        with _ctx(T):
            _check(lib().st_gemv_prenorm(_ptr(T), _ptr(EO), _ptr(EB), _ptr(EL), _ptr(x), _ptr(delta), _ptr(norm_w),
                                         float(eps), _ptr(x_out), _ptr(Y), B, M, N, 1 if act else 0, _ptr(WS),
                                         WS.numel() * WS.element_size(), _stream(T)))

    @staticmethod
    def moe_route(logits, K, renorm=True, expert_map=None):
        """(ids int32 [T, K], w float32 [T, K]): softmax + top-K (+ renormalisation) of router logits [T, E] in one launch"""
        T, E = logits.shape
        if logits.dtype not in (torch.bfloat16, torch.float32) or not logits.is_contiguous():
            raise RuntimeError("moe_route: contiguous BF16 or float32 logits")
        ids = torch.empty(T, K, dtype=torch.int32, device=logits.device)
        w = torch.empty(T, K, dtype=torch.float32, device=logits.device)
        with _ctx(logits):
            _check(lib().st_moe_route(_ptr(logits), 1 if logits.dtype == torch.float32 else 0, T, E, K, 1 if renorm else 0,
                                      _ptr(expert_map), _ptr(ids), _ptr(w), _stream(logits)))
        return ids, w

    @staticmethod
    def gemm_workspace_bytes(M, N, B):
        return int(lib().st_gemm_workspace_bytes(M, N, B))

    @staticmethod
    def gemm(T, EO, EL, X, Y, WS, CNT, Yf32=None):
        B, N = X.shape
        M = Y.shape[1]
        with _ctx(T):
            _check(lib().st_gemm(_ptr(T), _ptr(EO), _ptr(EL), _ptr(X), _ptr(Y), _ptr(Yf32), B, M, N, _ptr(WS),
                                 WS.numel() * WS.element_size(), _ptr(CNT), _stream(T)))

    @staticmethod
    def moe_gemv_workspace_bytes(S, M, N):
        return int(lib().st_moe_gemv_workspace_bytes(S, M, N))

    @staticmethod
    def mvx(TP, EOP, EBP, ELP, X, ids, Y, WS, CNT, xdiv):
        S, M = Y.shape
        N = X.shape[1]
        with _ctx(X):
            _check(lib().st_moe_gemv(_ptr(TP), _ptr(EOP), _ptr(EBP), _ptr(ELP), TP.numel(), _ptr(X), _ptr(ids),
                                     1 if ids.dtype == torch.int64 else 0, _ptr(Y), S, M, N, xdiv, _ptr(WS),
                                     WS.numel() * WS.element_size(), _ptr(CNT), _stream(X)))

    @staticmethod
    def moe_group_workspace_bytes(nblk, M, N):
        return int(lib().st_moe_group_workspace_bytes(nblk, M, N))

    @staticmethod
    def mvg(TP, EOP, EBP, ELP, X, sorted_ids, bexp, npost, Y, WS, CNT, xdiv):
        S, M = Y.shape
        N = X.shape[1]
        with _ctx(X):
            _check(lib().st_moe_group_gemv(_ptr(TP), _ptr(EOP), _ptr(EBP), _ptr(ELP), TP.numel(), _ptr(X),
                                           _ptr(sorted_ids), _ptr(bexp), _ptr(npost), bexp.numel(), _ptr(Y), S, M, N,
                                           xdiv, _ptr(WS), WS.numel() * WS.element_size(), _ptr(CNT), _stream(X)))

    @staticmethod
    def gemv_swiglu(T, EO, EB, EL, X, act, WS, CNT):
        """act [B, I] = silu(gate) * up for a tree whose 2 I rows interleave gate and up in 16-row tiles (B <= 8)"""
        B, N = X.shape
        M = T.shape[0] * 16
        with _ctx(T):
            _check(lib().st_gemv_swiglu(_ptr(T), _ptr(EO), _ptr(EB), _ptr(EL), _ptr(X), _ptr(act), B, M, N, _ptr(WS),
                                        WS.numel() * WS.element_size(), _ptr(CNT), _stream(T)))

    @staticmethod
    def moe_align(ids, E, used_bins, sorted_ids, bexp, npost, bs=8):
        with _ctx(ids):
            _check(lib().st_moe_align(_ptr(ids), 1 if ids.dtype == torch.int64 else 0, ids.numel(), E, used_bins, bs,
                                      _ptr(sorted_ids), _ptr(bexp), _ptr(npost), bexp.numel(), _stream(ids)))

    @staticmethod
    def moe_tensor_maps(trees, M, N):
        """uint8 device buffer holding one weight tensor map per expert tree (built on the host, copied once)"""
        E = len(trees)
        nb = int(lib().st_moe_tensor_map_bytes())
        dev = trees[0].device
        maps = torch.empty(E * nb + 64, dtype=torch.uint8, device=dev)
        maps = maps[(-maps.data_ptr()) % 64:][:E * nb]                       # 64-byte aligned view
        host = (ctypes.c_int64 * E)(*[t.data_ptr() for t in trees])
        with _ctx(trees[0]):
            _check(lib().st_moe_tensor_maps(host, E, M, N, _ptr(maps), _stream(trees[0])))
        return maps

    @staticmethod
    def moe_gather(X, sorted_ids, npost, S, xdiv, Xg):
        with _ctx(X):
            _check(lib().st_moe_gather(_ptr(X), _ptr(sorted_ids), _ptr(npost), Xg.shape[0], S, xdiv, X.shape[1], _ptr(Xg),
                                       _stream(X)))

    @staticmethod
    def gtt(maps, EOP, ELP, Xg, sorted_ids, bexp, npost, bs, Y, Yf32=None):
        """grouped fused decode + tcgen05 GEMM (the place of the reference's `_C.gtt`)"""
        S, M = Y.shape
        with _ctx(Xg):
            _check(lib().st_moe_group_gemm(_ptr(maps), _ptr(EOP), _ptr(ELP), EOP.numel(), _ptr(Xg), _ptr(sorted_ids),
                                           _ptr(bexp), _ptr(npost), bexp.numel(), bs, _ptr(Y), _ptr(Yf32), S, M,
                                           Xg.shape[1], _stream(Xg)))

    @staticmethod
    def wsum(Y, W, out):
        T, K = W.shape
        with _ctx(Y):
            _check(lib().st_wsum(_ptr(Y), _ptr(W), 1 if W.dtype == torch.bfloat16 else 0, _ptr(out), T, K, Y.shape[1],
                                 _stream(Y)))

    @staticmethod
    def add_rmsnorm(x, delta, w, out, eps):
        """x += delta (in place, delta may be None); out = RMSNorm(x) * w"""
        rows, cols = x.shape
        with _ctx(x):
            _check(lib().st_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(w), _ptr(out), rows, cols, float(eps), _stream(x)))

    @staticmethod
    def qk_norm_rope(qkv, wq, wk, cos_t, sin_t, pos, q_out, k_out, eps):
        B, hq, hkv = q_out.shape[0], q_out.shape[1], k_out.shape[1]
        with _ctx(qkv):
            _check(lib().st_qk_norm_rope(_ptr(qkv), qkv.stride(0), _ptr(wq), _ptr(wk), _ptr(cos_t), _ptr(sin_t), _ptr(pos),
                                         cos_t.shape[0], _ptr(q_out), _ptr(k_out), B, hq, hkv, float(eps), _stream(qkv)))

    @staticmethod
    def silu_mul(gu, act):
        S, I2 = gu.shape
        with _ctx(gu):
            _check(lib().st_silu_mul(_ptr(gu), _ptr(act), S, I2 // 2, _stream(gu)))


class _KV:
    """call shapes of the reference's `statetree._kv` module (statetree/csrc/kvcache.cu:588-599)"""

    @staticmethod
    def rope_append(qkv, wq, wk, cos_t, sin_t, pos, q_out, hq, hkv, eps, slot, kv, pool, pool_cnt):
        """decode step: q heads of qkv [B, (hq + 2 hkv) * 128] normalised + rotated into q_out, K (normalised + rotated)
        and V rows appended to the pages at slot [B]"""
        B = qkv.shape[0]
        with _ctx(qkv):
            _check(lib().st_rope_kv_append(_ptr(qkv), qkv.stride(0), _ptr(wq), _ptr(wk), _ptr(cos_t), _ptr(sin_t),
                                           _ptr(pos), cos_t.shape[0], _ptr(q_out), B, hq, hkv, float(eps), _ptr(slot),
                                           _ptr(kv), kv.size(0), _ptr(pool), pool.size(0), _ptr(pool_cnt), _stream(qkv)))

    @staticmethod
    def version():
        return 2

    @staticmethod
    def page_bytes(H):
        return int(lib().st_kv_page_bytes(H))

    @staticmethod
    def append(K, V, slot, kv, pool, pool_cnt, reuse=False):
        if not (K.dtype == V.dtype == torch.bfloat16 and K.dim() == 3 and V.dim() == 3):
            raise RuntimeError("kv_append: K/V")
        if not (K.size(2) == 128 and V.size(2) == 128 and K.stride(2) == 1 and V.stride(2) == 1 and
                K.stride(1) == 128 and V.stride(1) == 128):
            raise RuntimeError("kv_append: [N, H, 128] with heads contiguous")
        if not (slot.dtype == torch.int64 and slot.is_contiguous() and slot.numel() == K.size(0)):
            raise RuntimeError("kv_append: slots")
        if not (kv.dtype == torch.uint8 and kv.is_contiguous() and kv.dim() == 5 and kv.size(1) == K.size(1) and
                kv.size(4) == 1600):
            raise RuntimeError("kv_append: cache [blocks, H, 2, 2, 1600]")
        if not (pool.dtype == torch.int32 and pool.dim() == 2 and pool.size(1) == 16):
            raise RuntimeError("kv_append: pool [P, 16]")
        with _ctx(K):
            _check(lib().st_kv_append(_ptr(K), _ptr(V), K.stride(0), V.stride(0), _ptr(slot), K.size(0), K.size(1),
                                      _ptr(kv), kv.size(0), _ptr(pool), pool.size(0), _ptr(pool_cnt),
                                      1 if reuse else 0, _stream(K)))

    @staticmethod
    def dequant(kv, pool, Kd, Vd):
        nb, H = kv.size(0), kv.size(1)
        if not (Kd.is_contiguous() and Vd.is_contiguous() and Kd.numel() == nb * 16 * H * 128 and
                Vd.numel() == Kd.numel()):
            raise RuntimeError("kv_dequant: outputs")
        with _ctx(kv):
            _check(lib().st_kv_dequant(_ptr(kv), nb, H, _ptr(pool), pool.size(0), _ptr(Kd), _ptr(Vd), _stream(kv)))

    @staticmethod
    def dequant_blocks(kv, pool, blocks, Kd, Vd):
        if not (kv.dtype == torch.uint8 and kv.is_contiguous() and kv.dim() == 5 and kv.size(4) == 1600):
            raise RuntimeError("kv_dequant_blocks: cache [blocks, H, 2, 2, 1600]")
        if not (blocks.dtype == torch.int32 and blocks.is_contiguous() and blocks.dim() == 1):
            raise RuntimeError("kv_dequant_blocks: blocks int32 [n]")
        n, H = blocks.numel(), kv.size(1)
        if not (Kd.dtype == Vd.dtype == torch.bfloat16 and Kd.is_contiguous() and Vd.is_contiguous() and
                Kd.numel() >= n * 16 * H * 128 and Vd.numel() >= n * 16 * H * 128):
            raise RuntimeError("kv_dequant_blocks: outputs [n, 16, H, 128]")
        with _ctx(kv):
            _check(lib().st_kv_dequant_blocks(_ptr(kv), kv.size(0), H, _ptr(pool), pool.size(0), _ptr(blocks), n,
                                              _ptr(Kd), _ptr(Vd), _stream(kv)))

    @staticmethod
    def attn(q, kv, pool, bt, lens, out, wo, wml, scale, S, starts=None, minpps=1):
        if not (q.dtype == torch.bfloat16 and q.dim() == 3 and q.size(2) == 128 and q.stride(2) == 1 and
                q.stride(1) == 128):
            raise RuntimeError("kv_attn: q [B, Hq, 128]")
        if not (out.dtype == torch.bfloat16 and out.dim() == 3 and out.size(1) == q.size(1) and out.stride(2) == 1 and
                out.stride(1) == 128):
            raise RuntimeError("kv_attn: out [B, Hq, 128]")
        if not (kv.dtype == torch.uint8 and kv.dim() == 5 and kv.size(4) == 1600):
            raise RuntimeError("kv_attn: cache")
        if not (bt.dtype == torch.int32 and bt.dim() == 2 and bt.stride(1) == 1 and lens.dtype == torch.int32):
            raise RuntimeError("kv_attn: block table / lens int32")
        B, Hq, Hkv = q.size(0), q.size(1), kv.size(1)
        if Hq % Hkv or S < 1:
            raise RuntimeError("kv_attn: heads / splits")
        if S > 1 and not (wo.numel() >= B * Hq * S * 128 and wml.numel() >= B * Hq * S * 2):
            raise RuntimeError("kv_attn: workspace")
        if starts is not None and not (starts.dtype == torch.int32 and starts.numel() >= B):
            raise RuntimeError("kv_attn: starts int32 [B]")
        with _ctx(q):
            _check(lib().st_kv_attn(_ptr(q), q.stride(0), B, Hq, _ptr(kv), kv.size(0), Hkv, _ptr(pool), pool.size(0),
                                    _ptr(bt), bt.stride(0), _ptr(lens), _ptr(starts), _ptr(out), out.stride(0),
                                    _ptr(wo), _ptr(wml), float(scale), int(S), int(minpps), _stream(q)))


def ext():
    lib()
    return _Weights


def kv_ext():
    lib()
    return _KV
