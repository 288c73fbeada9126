"""TreeLinear / TreeSlice / TreeEmbedding: drop-in modules over the sm_100a kernels, with the buffers and call
surface of the reference's statetree/linear.py (TreeLinear 595-1018, TreeSlice 1021-1036, TreeEmbedding 1039-1067,
torch.compile custom ops 1070-1095).

Dispatch is one kernel per regime (no tuner, no multi-kernel ladder): up to GEMV_MAX activation rows run the
memory-order fused decode GEMV, more rows the fused decode + tcgen05 GEMM, more than PREFILL_MIN rows the decode kernel
into a BF16 scratch matrix + cuBLAS (the reference's prefill path).  Workspaces (exchange slots and zeroed
semaphores) are kept per (device, stream) because callers may run layers on side streams concurrently (the reason
given at statetree/linear.py:457-466); they are sized once per shape, so steady-state calls allocate only the output.
"""
import os
import weakref

import torch
import torch.nn as nn

from . import format as F
from .ops import ext

GEMV_MAX = int(os.environ.get("STATETREE_GEMV_MAX", "12"))     # activation rows up to which the GEMV kernel runs (<= 32)
# more activation rows than this (prefill): the tree is decoded once into a BF16 scratch matrix and cuBLAS multiplies by
# it, the reference's path above 1024 rows (statetree/linear.py:37, 879-886), here from the size at which it overtakes the
# tcgen05 kernel; 0 turns it off
PREFILL_MIN = int(os.environ.get("STATETREE_PREFILL_MIN", "512"))
DENSE_MAX = 1 << 28                 # weights: larger matrices (vocabulary-sized tables) never get a dense scratch copy
_STATES = {}
_BUFFERS = ("tree", "esc_rows", "esc_cols", "esc_bits")


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
        self.scratch = torch.empty(1 << 20, dtype=torch.float32, device=device)   # the GEMM's partial tiles (no contract)
        self.cnt = torch.zeros(1 << 16, dtype=torch.int32, device=device)

    def _new_ws(self, words):
        return torch.full((words,), -1, dtype=torch.int32, device=self.device).view(torch.float32)

    def get_ws(self, nbytes):
        if self.ws.numel() * 4 < nbytes:
            self._retired.append(self.ws)
            self.ws = self._new_ws((nbytes + 3) // 4)
        return self.ws

    def get_scratch(self, nbytes):
        if self.scratch.numel() * 4 < nbytes:
            self._retired.append(self.scratch)
            self.scratch = torch.empty((nbytes + 3) // 4, dtype=torch.float32, device=self.device)
        return self.scratch

    def dense_stage(self):
        if self.__dict__.get("_dense") is None:
            self._dense = _DenseStage(self.device)
        return self._dense

    def get_cnt(self, n):
        if self.cnt.numel() < n:
            self._retired.append(self.cnt)
            self.cnt = torch.zeros(n, dtype=torch.int32, device=self.device)
        return self.cnt


class _DenseStage:
    """Prefill-size batches: decode once, multiply with cuBLAS (statetree/linear.py:286-368 is the reference's form).
    Two BF16 scratch matrices per (device, stream).  While the GEMM reads one, a side stream decodes the layer linked
    as `_next` (by model.prepare, in module order) into the other: the decode is HBM-bound, the GEMM tensor-bound, so
    from the second layer of a pass on the decode hides under the GEMM.  A wrong guess of the next layer costs one
    wasted decode, never a wrong result: a scratch matrix is used only if it holds exactly the asked tree."""

    def __init__(self, device):
        self.device = device
        self.side = torch.cuda.Stream(device)                # (a high-priority stream measured slower: 17.2 against 14.8 ms at 1024 rows)
        self.mat = [None, None]                              # flat BF16 scratch
        self.holds = [None, None]                            # identity of the tree decoded into each
        self.decoded = [None, None]                          # event: that decode has finished
        self.read = [None, None]                             # event: the last GEMM that read it has finished
        self.turn = 0

    @staticmethod
    def _ident(layer):
        return (id(layer), layer.tree.data_ptr(), layer.tree._version)

    def _matrix(self, slot, layer):
        need = layer.out_features * layer.in_features
        if self.mat[slot] is None or self.mat[slot].numel() < need:
            if self.mat[slot] is not None:
                self.mat[slot].record_stream(self.side)       # a decode on the side stream may still be writing it
            self.mat[slot] = torch.empty(need, dtype=torch.bfloat16, device=self.device)
            self.mat[slot].record_stream(self.side)
            self.holds[slot] = None
        return self.mat[slot][:need].view(layer.out_features, layer.in_features)

    def run(self, layer, x, y):
        cur = torch.cuda.current_stream(self.device)
        me = self._ident(layer)
        if me in self.holds:
            slot = self.holds.index(me)
            cur.wait_event(self.decoded[slot])
            W = self._matrix(slot, layer)
        else:
            slot = self.turn
            if self.decoded[slot] is not None:
                cur.wait_event(self.decoded[slot])           # a prefetch of some other layer into this slot
            W = self._matrix(slot, layer)
            eo, el, _ = layer.tables()
            ext().dec(layer.tree, eo, el, W)
            self.holds[slot] = me
            self.decoded[slot] = cur.record_event()
        other = 1 - slot
        nxt = layer._next() if layer._next is not None else None
        fork = None
        if (nxt is not None and nxt.dense_ok() and nxt.tree.device == layer.tree.device
                and self.holds[other] != self._ident(nxt)):
            nxt.tables()                                     # built on the caller's stream, before the fork
            Wn = self._matrix(other, nxt)
            fork = cur.record_event()
        torch.matmul(x, W.t(), out=y)
        self.read[slot] = cur.record_event()
        self.turn = other
        if fork is not None:
            self.side.wait_event(fork)
            if self.read[other] is not None:
                self.side.wait_event(self.read[other])       # the GEMM that last read the other matrix
            with torch.cuda.stream(self.side):
                eo, el, _ = nxt.tables()
                ext().dec(nxt.tree, eo, el, Wn)
                self.decoded[other] = self.side.record_event()
            self.holds[other] = self._ident(nxt)


def _state(device):
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    st = _STATES.get(key)
    if st is None:
        st = _STATES[key] = _DevState(device)
    return st


def _rows_2d(x, width):
    """x [..., width] of any float dtype / layout -> BF16 [rows, width], contiguous and 16-byte aligned"""
    flat = x.reshape(-1, width)
    if flat.dtype != torch.bfloat16:
        flat = flat.to(torch.bfloat16)
    if flat.data_ptr() % 16 or not flat.is_contiguous():
        flat = flat.clone(memory_format=torch.contiguous_format)
    return flat


# layers reachable from the custom ops by a string handle (torch.compile passes plain strings, not modules)
_BY_HANDLE = weakref.WeakValueDictionary()


def _tracing():
    comp = getattr(torch, "compiler", None)
    return comp is not None and hasattr(comp, "is_compiling") and comp.is_compiling()


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
        self._handle = f"tl{id(self):x}"
        _BY_HANDLE[self._handle] = self
        self._reset_runtime()

    def set_handle(self, name):
        """The string under which the torch.compile custom ops find this layer; a stable name (the module path) keeps a
        compiled graph valid in another process (statetree/linear.py:621-625)."""
        self._handle = str(name)
        _BY_HANDLE[self._handle] = self

    def prepare(self, batch_sizes=(1,)):
        """Side tables and workspaces for these batch sizes now, so that a later call (or a CUDA-graph capture)
        allocates nothing (statetree/linear.py:1014-1018; there is no plan to pick here: one kernel per regime)."""
        if not self.tree.is_cuda:
            raise RuntimeError("TreeLinear.prepare: the layer must be on a GPU")
        E, st = ext(), _state(self.tree.device)
        self.tables()
        M, N = self.out_features, self.in_features
        for B in batch_sizes:
            if B <= min(GEMV_MAX, 32) or M % 128:
                st.get_ws(E.gemv_workspace_bytes(M, N, min(B, 32)))
                st.get_cnt(M // 16)
            else:
                st.get_scratch(E.gemm_workspace_bytes(M, N, B))
                st.get_cnt((M // 128) * ((B + 255) // 256))
        return self

    # ---------------------------------------------------------------- construction / state dict
    @classmethod
    def from_linear(cls, lin, verify=True, max_escape_fraction=None):
        return cls.from_weight(lin.weight, lin.bias, verify=verify, max_escape_fraction=max_escape_fraction)

    @classmethod
    @torch.no_grad()
    def from_weight(cls, W, bias=None, verify=True, max_escape_fraction=None):
        """W [out, in] bf16.  max_escape_fraction: raise EscapeHeavy when more weights escape."""
        W = W.detach()
        if W.dtype != torch.bfloat16:
            raise TypeError(f"TreeLinear.from_weight: expected a bfloat16 weight, got {W.dtype}")
        if max_escape_fraction is not None:
            escapes = F.escape_count(W)
            if escapes > max_escape_fraction * W.numel():
                raise EscapeHeavy(f"{escapes / W.numel():.2%} of the weights escape")
        enc = F.encode(W)
        out_features, in_features = W.shape
        layer = cls(in_features, out_features, bias=bias is not None, device="meta", n_esc=int(enc["esc_rows"].numel()))
        layer._buffers.update({name: enc[name] for name in _BUFFERS})
        if bias is not None:
            layer._buffers["bias"] = bias.detach().to(device=W.device, dtype=torch.bfloat16).clone()
        layer._reset_runtime()
        if verify:
            back = layer.dequantize() if layer.tree.is_cuda else F.decode_reference(*(layer._buffers[n] for n in _BUFFERS))
            if not torch.equal(back.view(torch.int16), W.view(torch.int16)):
                raise RuntimeError("TreeLinear: the tree does not decode to the weights it was built from")
        return layer

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        # how many weights escape depends on the data: make room for whatever the checkpoint holds
        for name in _BUFFERS[1:]:
            stored = state_dict.get(prefix + name)
            mine = self._buffers[name]
            if stored is not None and stored.shape != mine.shape:
                self._buffers[name] = torch.empty(stored.shape, dtype=stored.dtype, device=mine.device)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)
        self._reset_runtime()

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        self._reset_runtime()
        return out

    def _reset_runtime(self):
        self._tables = None                             # (eo, el, eb) on the tree's device
        self.__dict__["_shared"] = None                 # product shared by the TreeSlice views of this layer
        self.__dict__.setdefault("_next", None)         # weak reference to the layer that runs after this one
        self.__dict__.setdefault("allow_dec", True)     # False: never a dense scratch copy (the reference's flag for
                                                        # vocabulary-sized tables, statetree/linear.py:808-810)

    def __getstate__(self):
        state = self.__dict__.copy()
        state["_next"] = None                           # (a weak reference cannot be pickled; prepare() links again)
        return state

    def dense_ok(self):
        """may this layer be decoded into a BF16 scratch matrix for prefill-size batches"""
        return self.allow_dec and self.tree.is_cuda and self.out_features * self.in_features <= DENSE_MAX

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"escapes={self.esc_rows.numel()}, bits_per_weight={self.bits_per_weight:.3f}")

    @property
    def bits_per_weight(self):
        return F.bits_per_weight(self.out_features, self.in_features, self.esc_rows.numel())

    def storage_bytes(self):
        return sum(self._buffers[n].numel() * self._buffers[n].element_size() for n in _BUFFERS)

    def record_bytes(self):
        return self.tree.numel()

    def tables(self):
        """(eo, el, eb) escape side tables, built on first use (outside any graph capture).  The kernels read them
        before they wait for the preceding kernel of the stream (programmatic dependent launch), so the tables must be
        complete before that kernel starts: the stream is synchronised once after building them."""
        if self._tables is None or self._tables[0].device != self.tree.device:
            self._tables = F.escape_tables(self.out_features, self.in_features, self.esc_rows, self.esc_cols,
                                           self.esc_bits)
            if self.tree.is_cuda and not torch.cuda.is_current_stream_capturing():
                torch.cuda.current_stream(self.tree.device).synchronize()
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
        where = self.tree.device
        index = ids.reshape(-1).to(device=where, dtype=torch.int64).contiguous()
        gathered = torch.empty(index.numel(), self.in_features, dtype=torch.bfloat16, device=where)
        eo, el, _ = self.tables()
        ext().rows(self.tree, eo, el, index, gathered)
        return gathered.view(*ids.shape, self.in_features)

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
        elif 0 < PREFILL_MIN < B and yf32 is None and self.dense_ok() and not torch.cuda.is_current_stream_capturing():
            st.dense_stage().run(self, x, y)                # decode once + cuBLAS, the next layer decoded meanwhile
        elif M % 128 == 0:
            ws = st.get_scratch(E.gemm_workspace_bytes(M, N, B))
            E.gemm(self.tree, eo, el, x, y, ws, st.get_cnt((M // 128) * ((B + 255) // 256)), yf32)
        else:                                           # rows not a multiple of 128: GEMV kernel in row chunks
            step = min(32, max(GEMV_MAX, 16))
            ws = st.get_ws(E.gemv_workspace_bytes(M, N, step))
            for b0 in range(0, B, step):
                E.gemv(self.tree, eo, eb, el, x[b0:b0 + step], y[b0:b0 + step], ws, st.get_cnt(M // 16),
                       None if yf32 is None else yf32[b0:b0 + step])

    def forward(self, x):
        if _tracing() and _OPS_READY:
            return torch.ops.statetree.linear(x, self.tree, self._handle)
        return self._forward(x)

    def _forward(self, x, yf32=None):
        """any leading shape, any float dtype, any device: the product runs where the tree lives, in BF16, and comes
        back in the caller's dtype on the caller's device"""
        home, asked_dtype, asked_device = self.tree.device, x.dtype, x.device
        if home.type != "cuda":
            raise RuntimeError("statetree_b200: the kernels take CUDA tensors only (no CPU path); move the layer to a GPU")
        lead = x.shape[:-1]
        acts = _rows_2d(x if asked_device == home else x.to(home), self.in_features)
        result = torch.empty(acts.shape[0], self.out_features, dtype=torch.bfloat16, device=home)
        if acts.shape[0] > 0:
            with torch.cuda.device(home):
                self._run(acts, result, yf32)
        if self.bias is not None:
            result += self.bias
        result = result.view(*lead, self.out_features)
        if asked_dtype != torch.bfloat16:
            result = result.to(asked_dtype)
        return result if asked_device == home else result.to(asked_device)

    def _fused_part(self, x, start, size, nparts):
        """rows [start, start + size) of the product for a TreeSlice: the first part called with an input computes the
        whole fused output, the others reuse it; after the last part the shared result is dropped"""
        shared = self.__dict__.get("_shared")
        if shared is None or shared[0] is not x:
            shared = self.__dict__["_shared"] = [x, self(x), 0]
        shared[2] += 1
        if shared[2] >= nparts:
            self.__dict__["_shared"] = None
        return shared[1].narrow(-1, start, size)


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


TreeLinear.swiglu = swiglu


@torch.no_grad()
def forward_list(layers, x):
    """[layer(x) for layer in layers] for TreeLinear layers that read the same input (q / k / v or gate / up of a
    checkpoint that keeps them as separate trees): up to four layers run as ONE launch over the concatenation of their
    tiles (the GEMV up to GEMV_MAX rows, the tcgen05 GEMM beyond, if every layer has a multiple of 128 rows); anything
    else falls back to one call per layer."""
    first = layers[0]
    home = first.tree.device
    same = all(l.in_features == first.in_features and l.tree.device == home for l in layers)
    lead = x.shape[:-1]
    acts = _rows_2d(x if x.device == home else x.to(home), first.in_features) if same and home.type == "cuda" else None
    if acts is None or acts.shape[0] < 1 or not 2 <= len(layers) <= 4:
        return [l(x) for l in layers]
    use_gemm = acts.shape[0] > min(GEMV_MAX, 32)
    if use_gemm and any(l.out_features % 128 for l in layers):
        return [l(x) for l in layers]
    E, B = ext(), acts.shape[0]
    widths = [l.out_features for l in layers]
    flat = torch.empty(B * sum(widths), dtype=torch.bfloat16, device=home)
    outs, at = [], 0
    for w in widths:
        outs.append(flat[at:at + B * w].view(B, w))
        at += B * w
    tabs = []
    for l in layers:
        eo, el, eb = l.tables()
        tabs.append((l.tree, eo, eb, el))
    with torch.cuda.device(home):
        if use_gemm:
            E.gemm_list(E.gemv_list_args(tabs, outs), acts, _state(home).get_cnt((sum(widths) // 128) * ((B + 255) // 256)))
        else:
            ws = _state(home).get_ws(E.gemv_list_workspace_bytes(widths, first.in_features, B))
            E.gemv_list(E.gemv_list_args(tabs, outs), acts, ws)
    res = []
    for l, y in zip(layers, outs):
        if l.bias is not None:
            y += l.bias
        y = y.view(*lead, l.out_features)
        if x.dtype != torch.bfloat16:
            y = y.to(x.dtype)
        res.append(y if x.device == home else y.to(x.device))
    return res


class TreeSlice(nn.Module):
    """One of several linear layers that read the same input (q / k / v, gate / up), stored together as one TreeLinear
    on the parent module: rows [start, start + size) of that layer's output.  `fused` is the shared layer; it is not
    registered as a submodule here, its buffers belong to the parent (reference: statetree/linear.py:1021-1036)."""

    def __init__(self, fused, start, size, nparts):
        super().__init__()
        object.__setattr__(self, "fused", fused)
        self.in_features, self.out_features = fused.in_features, size
        self.start, self.nparts = start, nparts

    def forward(self, x):
        return self.fused._fused_part(x, self.start, self.out_features, self.nparts)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, rows from {self.start} of the fused layer"


class TreeEmbedding(nn.Module):
    """Embedding lookup from a tree-stored table: rows are decoded exactly on lookup.  The table is either owned
    (`table`, a registered TreeLinear) or, for tied input / output embeddings, the output layer's TreeLinear
    (`source`, not registered here) (reference: statetree/linear.py:1039-1067)."""

    def __init__(self, num_embeddings, embedding_dim, table=None, source=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.table = table
        object.__setattr__(self, "source", source)

    @classmethod
    def from_embedding(cls, emb, verify=True):
        return cls(emb.num_embeddings, emb.embedding_dim, table=TreeLinear.from_weight(emb.weight, verify=verify))

    def _rows_from(self):
        return self.table if self.table is not None else self.source

    def forward(self, ids):
        src = self._rows_from()
        if _tracing() and _OPS_READY:
            return torch.ops.statetree.rows(ids, src.tree, src._handle)
        return src.rows(ids)

    def extra_repr(self):
        return f"{self.num_embeddings}, {self.embedding_dim}, " + ("own table" if self.table is not None else "tied to the output layer")


# ---------------------------------------------------------------------------------------------- torch.compile
# Under torch.compile the layers appear in the traced graph as two opaque custom ops with shape-only fake kernels, so
# Dynamo neither traces into the ctypes shim nor specialises on it (reference: statetree/linear.py:1070-1095).
_OPS_READY = False


def _register_ops():
    global _OPS_READY
    library = getattr(torch, "library", None)
    if library is None or not hasattr(library, "custom_op"):
        return

    @library.custom_op("statetree::linear", mutates_args=())
    def linear_op(x: torch.Tensor, tree: torch.Tensor, handle: str) -> torch.Tensor:
        return _BY_HANDLE[handle]._forward(x)

    @linear_op.register_fake
    def _(x, tree, handle):
        return x.new_empty(*x.shape[:-1], tree.shape[0] * 16)

    @library.custom_op("statetree::rows", mutates_args=())
    def rows_op(ids: torch.Tensor, tree: torch.Tensor, handle: str) -> torch.Tensor:
        return _BY_HANDLE[handle].rows(ids)

    @rows_op.register_fake
    def _(ids, tree, handle):
        return tree.new_empty(*ids.shape, tree.shape[1] * 64, dtype=torch.bfloat16)

    _OPS_READY = True


try:
    _register_ops()
except Exception:                                       # noqa: BLE001  (a torch without torch.library.custom_op,
    _OPS_READY = False                                  # or the ops already registered by another copy of the package)
