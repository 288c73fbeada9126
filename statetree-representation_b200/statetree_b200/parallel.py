"""Tensor- and expert-parallel wiring of the tree-stored layers: one process per GPU, torch.distributed (NCCL on
GPUs; the host logic is backend-agnostic and tested with gloo).

The reference has no communication code: under vLLM each rank encodes its own weight shard
(statetree/_vllm.py:218-238) and vLLM adds the collectives.  The same partition is used here:
  column-parallel (q, k, v, gate, up): output rows split in whole 16-row tiles; no collective, the consumer of the
      activations is sharded the same way
  row-parallel (o, down): input columns split in whole 64-column groups; the partial [B, out] sums are all-reduced
  experts: contiguous blocks of experts per rank; every rank sees all tokens, pairs routed to another rank's experts
      contribute zero, partial outputs are all-reduced
Because a group's exponent node covers 64 columns of one row, a shard's records are byte-identical to the same tiles /
groups of the unsharded encode.
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from .linear import TreeLinear


def shard_bounds(n, unit, rank, world):
    """[lo, hi) of dimension n for this rank, in whole multiples of `unit`"""
    assert n % (unit * world) == 0, f"dimension {n} does not split into {world} parts of whole {unit}-element units"
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weight(W, kind, rank, world):
    """this rank's part of W [out, in]: kind 'col' = rows (column-parallel), 'row' = columns (row-parallel)"""
    if kind == "col":
        lo, hi = shard_bounds(W.shape[0], 16, rank, world)
        return W[lo:hi].contiguous()
    if kind == "row":
        lo, hi = shard_bounds(W.shape[1], 64, rank, world)
        return W[:, lo:hi].contiguous()
    raise ValueError(kind)


def shard_tree(tree, kind, rank, world):
    """the same partition applied to an already encoded tree uint8 [out/16, in/64, 1552] (records are shard-invariant)"""
    dim = 0 if kind == "col" else 1
    lo, hi = shard_bounds(tree.shape[dim], 1, rank, world)
    return tree.narrow(dim, lo, hi - lo).contiguous()


class PeerComm:
    """Peer-memory exchange between the ranks of one node (one process per GPU): every rank allocates a communication
    buffer in the kernel library, the 64-byte CUDA IPC handles travel through torch.distributed, and the all-reduce of
    the small decode-step tensors then runs as one kernel of peer loads and stores per rank (csrc/st_comm.cu) instead of
    an NCCL call.  Capturable in CUDA graphs (the call sequence must be the same on every rank, as with NCCL).
    STATETREE_PEER_COMM=0 keeps NCCL."""

    MAX_VALUES = 524288

    def __init__(self, group=None, device=None):
        import ctypes
        from . import ops
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if not 2 <= self.world <= 8:
            raise RuntimeError("PeerComm: 2 to 8 ranks of one node")
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        L = ops.lib()
        with torch.cuda.device(self.device):
            own = ctypes.c_void_p()
            ops._check(L.st_comm_alloc(ctypes.byref(own)))
            handle = ctypes.create_string_buffer(64)
            ops._check(L.st_comm_export(own, handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(own.value)
                else:
                    peer = ctypes.c_void_p()
                    ops._check(L.st_comm_import(ctypes.create_string_buffer(h, 64), ctypes.byref(peer)))
                    ptrs.append(peer.value)
        self._own = own
        self._bufs = (ctypes.c_void_p * self.world)(*ptrs)
        self._lib = L
        dist.barrier(group=group)                              # every buffer is mapped before the first call

    def all_reduce(self, y):
        """y (BF16, contiguous, a multiple of 8 values) <- sum over ranks, in place"""
        from . import ops
        assert y.dtype == torch.bfloat16 and y.is_contiguous() and y.numel() % 8 == 0 and y.numel() <= self.MAX_VALUES
        with torch.cuda.device(y.device):
            ops._check(self._lib.st_allreduce(self._bufs, self.rank, self.world, ops._ptr(y), ops._ptr(y), y.numel(),
                                              ops._stream(y)))
        return y

    GEMV_AR_VALUES = 128 << 10                                     # padded output values one fused call may deliver

    def gemv_allreduce_fits(self, M, B):
        nt = 1 if B <= 8 else (2 if B <= 16 else 4)
        return 1 <= B <= 32 and (M // 16) * 128 * nt <= self.GEMV_AR_VALUES

    def gemv_allreduce(self, tree, eo, eb, el, x, y, ws, yf32=None):
        """y [B, M] <- sum over ranks of x_r [B, N_r] W_r^T: the row-parallel product and its all-reduce as one launch"""
        from . import ops
        B, N = x.shape
        M = y.shape[1]
        with torch.cuda.device(y.device):
            ops._check(self._lib.st_gemv_allreduce(self._bufs, self.rank, self.world, ops._ptr(tree), ops._ptr(eo),
                                                   ops._ptr(eb), ops._ptr(el), ops._ptr(x), ops._ptr(y), ops._ptr(yf32),
                                                   B, M, N, ops._ptr(ws), ws.numel() * ws.element_size(), ops._stream(y)))
        return y

    def all_reduce_add_rmsnorm(self, x, delta, w, out, eps):
        """x += sum over ranks of delta; out = RMSNorm(x) * w  (x, delta, out BF16 [rows, cols])"""
        from . import ops
        rows, cols = x.shape
        with torch.cuda.device(x.device):
            ops._check(self._lib.st_allreduce_add_rmsnorm(self._bufs, self.rank, self.world, ops._ptr(x), ops._ptr(delta),
                                                          ops._ptr(w), ops._ptr(out), rows, cols, float(eps),
                                                          ops._stream(x)))
        return out


_COMMS = {}
PEER_COMM_DEFAULT = "1"


def peer_comm(group=None):
    """the PeerComm of a process group (created on first use), or None when it is switched off or does not apply"""
    import os
    if os.environ.get("STATETREE_PEER_COMM", PEER_COMM_DEFAULT) == "0" or not torch.cuda.is_available():
        return None
    if not (dist.is_available() and dist.is_initialized()) or not 2 <= dist.get_world_size(group) <= 8:
        return None
    if dist.get_backend(group) != "nccl":
        return None
    key = id(group)
    if key not in _COMMS:
        _COMMS[key] = PeerComm(group)
    return _COMMS[key]


def reduce_partials(y, group=None):
    """sum the row-parallel partial outputs over the tensor-parallel group, in place: the peer-memory kernel for the
    small BF16 tensors of a decode step, NCCL otherwise (and on CPU / gloo)"""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        comm = peer_comm(group) if y.is_cuda else None
        if (comm is not None and y.dtype == torch.bfloat16 and y.is_contiguous() and y.numel() % 8 == 0
                and y.numel() <= PeerComm.MAX_VALUES):
            return comm.all_reduce(y)
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


class ColumnParallelTreeLinear(nn.Module):
    """rows [rank * out / world, ...) of a linear; the output stays sharded"""

    def __init__(self, W, rank, world, bias=None, verify=True):
        super().__init__()
        b = None if bias is None else bias[slice(*shard_bounds(W.shape[0], 16, rank, world))]
        self.inner = TreeLinear.from_weight(shard_weight(W, "col", rank, world), b, verify=verify)

    def forward(self, x):
        return self.inner(x)


class RowParallelTreeLinear(nn.Module):
    """columns [rank * in / world, ...) of a linear; takes the sharded activation, returns the all-reduced output"""

    def __init__(self, W, rank, world, group=None, verify=True):
        super().__init__()
        self.inner = TreeLinear.from_weight(shard_weight(W, "row", rank, world), verify=verify)
        self.group = group

    def forward(self, x_local):
        from .linear import GEMV_MAX, _rows_2d, _state
        tl = self.inner
        comm = peer_comm(self.group) if tl.tree.is_cuda else None
        rows = x_local.numel() // tl.in_features
        if comm is None or tl.bias is not None or not (1 <= rows <= min(GEMV_MAX, 32)) \
                or not comm.gemv_allreduce_fits(tl.out_features, rows):
            return reduce_partials(tl(x_local), self.group)
        from . import ops
        acts = _rows_2d(x_local, tl.in_features)
        y = torch.empty(rows, tl.out_features, dtype=torch.bfloat16, device=tl.tree.device)
        eo, el, eb = tl.tables()
        ws = _state(tl.tree.device).get_ws(ops.ext().gemv_workspace_bytes(tl.out_features, tl.in_features, rows))
        comm.gemv_allreduce(tl.tree, eo, eb, el, acts, y, ws)
        y = y.view(*x_local.shape[:-1], tl.out_features)
        return y if x_local.dtype == torch.bfloat16 else y.to(x_local.dtype)


def expert_partition(num_experts, rank, world, device=None):
    """(lo, hi, expert_map): this rank owns experts [lo, hi); expert_map int32 [E] maps a global id to the local id
    or -1 (the convention of the grouped kernel: blocks with a negative expert are skipped)"""
    assert num_experts % world == 0
    per = num_experts // world
    lo, hi = rank * per, (rank + 1) * per
    ids = torch.arange(num_experts, device=device)
    emap = torch.where((ids >= lo) & (ids < hi), ids - lo, torch.full_like(ids, -1)).to(torch.int32)
    return lo, hi, emap
