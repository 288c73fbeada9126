"""Host-side logic of the multi-GPU path with two gloo ranks on CPU: shard-invariant records, the row-parallel
all-reduce, the expert partition, moe_align and the split heuristic."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import gen_inputs as G
from util import bits_to_torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    for p in (os.path.dirname(here), os.path.join(os.path.dirname(here), "statetree-representation_b200"),
              os.path.join(here, "golden"), here):
        if p not in sys.path:
            sys.path.insert(0, p)
    from statetree_b200 import format as F
    from statetree_b200 import parallel as P
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        W = bits_to_torch(G.weights(64, 256, 3, "mixed"))
        full = F.encode(W)
        x = torch.randn(3, 256, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
        ref = x.double() @ W.double().t()
        ok = True
        # column parallel: rows; records of the shard are the same tiles of the full tree
        enc = F.encode(P.shard_weight(W, "col", rank, world))
        ok &= torch.equal(enc["tree"], P.shard_tree(full["tree"], "col", rank, world))
        dec = F.decode_reference(**enc)
        y_col = (x.double() @ dec.double().t())
        gathered = [torch.empty_like(y_col) for _ in range(world)]
        dist.all_gather(gathered, y_col)
        ok &= torch.allclose(torch.cat(gathered, 1), ref)
        # row parallel: columns; partial sums all-reduced
        enc = F.encode(P.shard_weight(W, "row", rank, world))
        ok &= torch.equal(enc["tree"], P.shard_tree(full["tree"], "row", rank, world))
        dec = F.decode_reference(**enc)
        lo, hi = P.shard_bounds(256, 64, rank, world)
        part = (x[:, lo:hi].double() @ dec.double().t()).float()
        y = P.reduce_partials(part)
        ok &= torch.allclose(y.double(), ref, rtol=1e-5, atol=1e-6)
        # experts: the local maps of all ranks partition the experts
        lo, hi, emap = P.expert_partition(8, rank, world)
        owned = (emap >= 0).int()
        dist.all_reduce(owned)
        ok &= bool((owned == 1).all()) and int(emap[lo]) == 0 and int(emap[hi - 1]) == hi - lo - 1
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_reduction():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]


def test_shard_bounds_reject_ragged_splits():
    from statetree_b200 import parallel as P
    with pytest.raises(AssertionError):
        P.shard_bounds(48, 16, 0, 2)            # 24 rows per rank is not a whole number of tiles
    assert P.shard_bounds(4096, 64, 3, 8) == (1536, 2048)


def test_moe_align_layout():
    from statetree_b200.experts import moe_align
    for S, E in ((1, 4), (37, 5), (300, 16), (8, 128)):
        ids = torch.randint(0, E, (S,), generator=torch.Generator().manual_seed(S))
        sorted_ids, bexp, npost = moe_align(ids, E, 8)
        n = int(npost)
        assert n % 8 == 0 and sorted_ids.numel() == bexp.numel() * 8
        used = sorted_ids[:n].view(-1, 8)
        for b in range(n // 8):
            real = used[b][used[b] < S]
            assert real.numel() > 0 and bool((ids[real.long()] == int(bexp[b])).all())
        assert bool((sorted_ids[n:] == S).all())
        real = sorted_ids[sorted_ids < S]
        assert torch.equal(real.sort().values, torch.arange(S, dtype=torch.int32))


def test_decode_split_heuristic():
    from statetree_b200.kvcache import decode_splits
    # long single sequences: about sqrt(pages) splits; large batches: what fills the GPU, two at least
    assert decode_splits(1, 8, 1024) == 32 and decode_splits(1, 8, 256) == 16 and decode_splits(1, 8, 64) == 8
    assert decode_splits(8, 8, 256) == 7 and decode_splits(16, 8, 1024) == 4 and decode_splits(64, 8, 1024) == 2
    assert decode_splits(8, 8, 8) == 2 and decode_splits(8, 8, 3) == 1
    for B in (1, 8, 32, 64):
        for pages in (3, 64, 256, 1024):
            s = decode_splits(B, 8, pages)
            assert 1 <= s <= 64 and (s == 1 or pages // s >= 4)


def test_peer_comm_is_not_used_off_gpu():
    """the peer-memory all-reduce needs NCCL ranks with CUDA devices; everywhere else reduce_partials stays on the
    process group's own all-reduce (the gloo ranks above exercise that path)"""
    from statetree_b200 import parallel
    assert parallel.peer_comm(None) is None                      # no process group here
    assert parallel.PeerComm.MAX_VALUES == 524288
