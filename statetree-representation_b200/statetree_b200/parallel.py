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


def reduce_partials(y, group=None):
    """sum the row-parallel partial outputs over the tensor-parallel group, in place"""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
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
        return reduce_partials(self.inner(x_local), self.group)


def expert_partition(num_experts, rank, world, device=None):
    """(lo, hi, expert_map): this rank owns experts [lo, hi); expert_map int32 [E] maps a global id to the local id
    or -1 (the convention of the grouped kernel: blocks with a negative expert are skipped)"""
    assert num_experts % world == 0
    per = num_experts // world
    lo, hi = rank * per, (rank + 1) * per
    ids = torch.arange(num_experts, device=device)
    emap = torch.where((ids >= lo) & (ids < hi), ids - lo, torch.full_like(ids, -1)).to(torch.int32)
    return lo, hi, emap
