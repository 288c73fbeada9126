"""TreeLinear / TreeSlice / TreeEmbedding: drop-in modules over the sm_100a kernels, with the buffers and call
surface of the reference's statetree/linear.py (TreeLinear 595-1018, TreeSlice / TreeEmbedding below it).

Dispatch is one kernel per regime (no tuner, no multi-kernel ladder): batch <= GEMV_MAX rows run the memory-order
fused decode GEMV, larger batches the fused decode + tcgen05 GEMM.  Workspaces (fp32 split partials and zeroed
semaphores) are kept per (device, stream) because callers may run layers on side streams concurrently (the reason
given at statetree/linear.py:457-466); they are sized once per shape, so steady-state calls allocate only the output.
"""
import os

import torch
import torch.nn as nn

from . import format as F
from .ops import ext

GEMV_MAX = int(os.environ.get("STATETREE_GEMV_MAX", "10"))     # rows up to which the GEMV kernel runs (<= 32);
# measured on B200 (Qwen3-8B shapes, ms per step of 252 linears): GEMV 3.39 at 8 rows, 4.22 at 9, 4.54 at 12, 4.95 at
# 16; tcgen05 GEMM 4.41-4.44 at 9-16 and 4.32 at 32
_STATES = {}


class EscapeHeavy(RuntimeError):
    """more weights escape than the caller allows (the layer is better left in BF16)"""


class _DevState:
    """per (device, stream): the fp32 workspace of the small-batch kernels and the semaphore array.  The kernels expect
    every workspace word to hold 0xFFFFFFFF between launches (their exchange-slot sentinel) and every semaphore to be
    zero, and leave them so.  Buffers only ever grow, and a buffer that was handed out is never freed: a CUDA graph
    captured earlier keeps replaying into the old one."""

    def __init__(self, device):
        self.device = device
        self._retired = []
        self.ws = self._new_ws(1 << 20)
        self.cnt = torch.zeros(1 << 16, dtype=torch.int32, device=device)

    def _new_ws(self, words):
        return torch.full((words,), -1, dtype=torch.int32, device=self.device).view(torch.float32)

    def get_ws(self, nbytes):
        if self.ws.numel() * 4 < nbytes:
            self._retired.append(self.ws)
            self.ws = self._new_ws((nbytes + 3) // 4)
        return self.ws

    def get_cnt(self, n):
        if self.cnt.numel() < n:
            self._retired.append(self.cnt)
            self.cnt = torch.zeros(n, dtype=torch.int32, device=self.device)
        return self.cnt


def _state(device):
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    st = _STATES.get(key)
    if st is None:
        st = _STATES[key] = _DevState(device)
    return st


class TreeLinear(nn.Module):
    """y = x W^T (+ b) with W [out, in] BF16 stored as a lossless state tree (~12.1 bits/weight).

    Buffers (state dict): tree uint8 [out/16, in/64, 1552], esc_rows / esc_cols int32, esc_bits int16 (exact bits of
    the weights the tree cannot hold), bias (optional, bf16)."""

    def __init__(self, in_features, out_features, bias=False, device=None, n_esc=0):
        super().__init__()
        assert out_features % 16 == 0 and in_features % 64 == 0, "TreeLinear needs out % 16 == 0 and in % 64 == 0"
        self.in_features, self.out_features = in_features, out_features
        dev = torch.device(device) if device is not None else None
        self.register_buffer("tree", torch.empty(out_features // 16, in_features // 64, F.RECORD_BYTES,
                                                 dtype=torch.uint8, device=dev))
        self.register_buffer("esc_rows", torch.empty(n_esc, dtype=torch.int32, device=dev))
        self.register_buffer("esc_cols", torch.empty(n_esc, dtype=torch.int32, device=dev))
        self.register_buffer("esc_bits", torch.empty(n_esc, dtype=torch.int16, device=dev))
        if bias:
            self.register_buffer("bias", torch.empty(out_features, dtype=torch.bfloat16, device=dev))
        else:
            self.bias = None
        self._reset_runtime()

    # ---------------------------------------------------------------- construction / state dict
    @classmethod
    def from_linear(cls, lin, verify=True, max_escape_fraction=None):
        return cls.from_weight(lin.weight, lin.bias, verify=verify, max_escape_fraction=max_escape_fraction)

    @classmethod
    @torch.no_grad()
    def from_weight(cls, W, bias=None, verify=True, max_escape_fraction=None):
        """W [out, in] bf16.  max_escape_fraction: raise EscapeHeavy when more weights escape."""
        W = W.detach()
        assert W.dtype == torch.bfloat16, f"TreeLinear: weight dtype {W.dtype}, expected bfloat16"
        if max_escape_fraction is not None:
            k = F.escape_count(W)
            if k > max_escape_fraction * W.numel():
                raise EscapeHeavy(f"{k / W.numel():.2%} of the weights escape")
        enc = F.encode(W)
        self = cls(W.shape[1], W.shape[0], bias=bias is not None, device="meta", n_esc=int(enc["esc_rows"].numel()))
        for name in ("tree", "esc_rows", "esc_cols", "esc_bits"):
            self._buffers[name] = enc[name]
        if bias is not None:
            self._buffers["bias"] = bias.detach().to(device=W.device, dtype=torch.bfloat16).clone()
        self._reset_runtime()
        if verify:
            got = self.dequantize() if self.tree.is_cuda else F.decode_reference(self.tree, self.esc_rows,
                                                                                  self.esc_cols, self.esc_bits)
            if not torch.equal(got.view(torch.int16), W.view(torch.int16)):
                raise RuntimeError("TreeLinear: decoded weights differ from the original (format bug)")
        return self

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        for name in ("esc_rows", "esc_cols", "esc_bits"):        # data-dependent sizes: adopt the stored size
            v = state_dict.get(prefix + name)
            if v is not None and v.shape != self._buffers[name].shape:
                self._buffers[name] = torch.empty(v.shape, dtype=v.dtype, device=self._buffers[name].device)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)
        self._reset_runtime()

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        self._reset_runtime()
        return out

    def _reset_runtime(self):
        self._tables = None                             # (eo, el, eb) on the tree's device

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"escapes={self.esc_rows.numel()}, bits_per_weight={self.bits_per_weight:.3f}")

    @property
    def bits_per_weight(self):
        return F.bits_per_weight(self.out_features, self.in_features, self.esc_rows.numel())

    def storage_bytes(self):
        return sum(b.numel() * b.element_size() for b in (self.tree, self.esc_rows, self.esc_cols, self.esc_bits))

    def record_bytes(self):
        return self.tree.numel()

    def tables(self):
        """(eo, el, eb) escape side tables, built on first use (outside any graph capture)"""
        if self._tables is None or self._tables[0].device != self.tree.device:
            self._tables = F.escape_tables(self.out_features, self.in_features, self.esc_rows, self.esc_cols,
                                           self.esc_bits)
        return self._tables

    def dequantize(self):
        """The exact BF16 weight [out, in] (decoded by the CUDA kernel)."""
        W = torch.empty(self.out_features, self.in_features, dtype=torch.bfloat16, device=self.tree.device)
        eo, el, _ = self.tables()
        ext().dec(self.tree, eo, el, W)
        return W

    @torch.no_grad()
    def rows(self, ids):
        """W[ids] (exact BF16 rows), decoded on the fly: the embedding lookup of a tree-stored table."""
        dev = self.tree.device
        flat = ids.reshape(-1)
        if flat.dtype != torch.int64 or not flat.is_contiguous() or flat.device != dev:
            flat = flat.to(device=dev, dtype=torch.int64).contiguous()
        out = torch.empty(flat.numel(), self.in_features, dtype=torch.bfloat16, device=dev)
        eo, el, _ = self.tables()
        ext().rows(self.tree, eo, el, flat, out)
        return out.view(*ids.shape, self.in_features)

    # ---------------------------------------------------------------- forward
    def _run(self, x, y, yf32=None):
        """x [B, in] bf16 contiguous 16-byte aligned -> y [B, out] (one launch per GEMV_MAX rows or one GEMM)"""
        E = ext()
        B = x.shape[0]
        M, N = self.out_features, self.in_features
        eo, el, eb = self.tables()
        st = _state(x.device)
        if B <= min(GEMV_MAX, 32):
            ws = st.get_ws(E.gemv_workspace_bytes(M, N, B))
            E.gemv(self.tree, eo, eb, el, x, y, ws, st.get_cnt(M // 16), yf32)
        elif M % 128 == 0:
            ws = st.get_ws(E.gemm_workspace_bytes(M, N, B))
            E.gemm(self.tree, eo, el, x, y, ws, st.get_cnt((M // 128) * ((B + 255) // 256)), yf32)
        else:                                           # rows not a multiple of 128: GEMV kernel in row chunks
            step = min(32, max(GEMV_MAX, 16))
            ws = st.get_ws(E.gemv_workspace_bytes(M, N, step))
            for b0 in range(0, B, step):
                E.gemv(self.tree, eo, eb, el, x[b0:b0 + step], y[b0:b0 + step], ws, st.get_cnt(M // 16),
                       None if yf32 is None else yf32[b0:b0 + step])

    def forward(self, x):
        return self._forward(x)

    def _forward(self, x, yf32=None):
        dev, src = self.tree.device, x.device
        if src != dev:
            x = x.to(dev)
        shp = x.shape
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if not x2.is_contiguous() or x2.data_ptr() % 16:
            x2 = x2.clone(memory_format=torch.contiguous_format)
        B = x2.shape[0]
        y = torch.empty(B, self.out_features, dtype=torch.bfloat16, device=x2.device)
        if B:
            self._run(x2, y, yf32)
        if self.bias is not None:
            y += self.bias
        y = y.view(*shp[:-1], self.out_features)
        y = y if x.dtype == torch.bfloat16 else y.to(x.dtype)
        return y if src == dev else y.to(src)


def interleave_gate_up(gate, up):
    """[2 I, in] weight whose 16-row tiles alternate between the gate and the up projection (tile 2j = gate rows
    16j .. 16j + 15, tile 2j + 1 = the same rows of up): the layout TreeLinear.swiglu expects"""
    I, N = gate.shape
    assert up.shape == gate.shape and I % 16 == 0
    return torch.stack([gate.view(I // 16, 16, N), up.view(I // 16, 16, N)], 1).reshape(2 * I, N).contiguous()


def swiglu(self, x):
    """x [B, in] BF16, B <= 8 -> silu(gate x) * (up x) [B, I] in one launch, for a TreeLinear built from
    interleave_gate_up(gate, up); raises RuntimeError for shapes the fused epilogue does not take"""
    B = x.shape[0]
    eo, el, eb = self.tables()
    E, st = ext(), _state(x.device)
    act = torch.empty(B, self.out_features // 2, dtype=torch.bfloat16, device=x.device)
    ws = st.get_ws(E.gemv_workspace_bytes(self.out_features, self.in_features, B))
    E.gemv_swiglu(self.tree, eo, eb, el, x, act, ws, st.get_cnt(self.out_features // 16))
    return act


class TreeSlice(nn.Module):
    """Rows [start, start + size) of a fused TreeLinear (q / k / v of a fused qkv, gate / up of a fused gate_up):
    parts called with the same input object share one product (reference: statetree/linear.py TreeSlice)."""

    def __init__(self, parent, start, size, nparts):
        super().__init__()
        self.__dict__["_parent"] = parent               # not a submodule: the parent is registered once elsewhere
        self.start, self.size, self.nparts = start, size, nparts
        self.in_features, self.out_features = parent.in_features, size

    def forward(self, x):
        p = self._parent
        c = getattr(p, "_fcache", None)
        if c is None or c[0] is not x:
            c = p._fcache = [x, p(x), 0]
        out = c[1].narrow(-1, self.start, self.size)
        c[2] += 1
        if c[2] >= self.nparts:
            p._fcache = None
        return out


class TreeEmbedding(nn.Module):
    """Embedding lookup from a tree-stored table (optionally shared with a tied lm_head TreeLinear)."""

    def __init__(self, table):
        super().__init__()
        self.table = table
        self.num_embeddings, self.embedding_dim = table.out_features, table.in_features

    @classmethod
    def from_embedding(cls, emb, verify=True):
        return cls(TreeLinear.from_weight(emb.weight, verify=verify))

    def forward(self, ids):
        return self.table.rows(ids)


TreeLinear.swiglu = swiglu
