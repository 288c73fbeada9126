"""Worker of tests/test_gpu_peer_comm.py: one process per GPU (torchrun), checks the peer-memory all-reduce against an
all-gather + fp32 sum in rank order (bit-exact), eagerly, back to back and inside a replayed CUDA graph."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "statetree-representation_b200"))

from statetree_b200 import ops  # noqa: E402
from statetree_b200.parallel import PeerComm  # noqa: E402


def expected(y, world):
    parts = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(parts, y)
    acc = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
    for p in parts:                                     # rank order, fp32, one rounding at the end
        acc += p.float()
    return acc.to(torch.bfloat16)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = PeerComm()
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    for n in (8, 4096, 8 * 4096, 64 * 4096, 524288):
        for it in range(6):                             # consecutive calls: both halves of the double buffer, many epochs
            y = torch.randn(n, device=dev, generator=gen).to(torch.bfloat16)
            want = expected(y, world)
            comm.all_reduce(y)
            assert torch.equal(y, want), (n, it, (y.float() - want.float()).abs().max().item())
    # a captured sequence of calls of different sizes, replayed
    ys = [torch.randn(n, device=dev, generator=gen).to(torch.bfloat16) for n in (4096, 8 * 4096, 4096, 16 * 4096)]
    wants = [expected(y, world) for y in ys]
    src = [y.clone() for y in ys]
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for y in ys:
            comm.all_reduce(y)
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for y in ys:
            comm.all_reduce(y)
    for _ in range(20):
        for y, s in zip(ys, src):
            y.copy_(s)
        g.replay()
        torch.cuda.synchronize()
        for y, w in zip(ys, wants):
            assert torch.equal(y, w)
    # fused with the residual add and RMSNorm
    E = ops.ext()
    for rows, cols in ((1, 4096), (8, 4096), (3, 2048), (64, 8192)):
        x0 = torch.randn(rows, cols, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).to(torch.bfloat16)
        w = torch.randn(cols, device=dev, generator=torch.Generator(device=dev).manual_seed(8)).to(torch.bfloat16)
        delta = torch.randn(rows, cols, device=dev, generator=gen).to(torch.bfloat16)
        xa, ha = x0.clone(), torch.empty_like(x0)
        E.add_rmsnorm(xa, expected(delta, world), w, ha, 1e-6)
        xb, hb = x0.clone(), torch.empty_like(x0)
        comm.all_reduce_add_rmsnorm(xb, delta, w, hb, 1e-6)
        assert torch.equal(xa, xb), (rows, cols)
        assert (ha.float() - hb.float()).abs().max().item() <= 2e-2 * ha.float().abs().max().item(), (rows, cols)
    # the row-parallel GEMV that adds the ranks' sums itself: against the plain GEMV's fp32 accumulators gathered and
    # added in rank order; eagerly (both call parities) and in a replayed graph; the same bits on every rank
    from statetree_b200 import TreeLinear
    from statetree_b200.linear import _state
    for (M, N, B) in ((4096, 4096, 1), (4096, 12288, 1), (4096, 4096, 8), (1024, 2048, 12), (2048, 4096, 20)):
        Nr = N // world // 64 * 64
        if Nr == 0:
            continue
        Wr = (torch.randn(M, Nr, device=dev, generator=gen) * 0.05).to(torch.bfloat16)
        tl = TreeLinear.from_weight(Wr, verify=False)
        eo, el, eb = tl.tables()
        torch.cuda.synchronize()
        ws = _state(dev).get_ws(E.gemv_workspace_bytes(M, Nr, B))
        for it in range(5):
            x = torch.randn(B, Nr, device=dev, generator=gen).to(torch.bfloat16)
            yf = torch.empty(B, M, dtype=torch.float32, device=dev)
            E.gemv(tl.tree, eo, eb, el, x, torch.empty(B, M, dtype=torch.bfloat16, device=dev), ws,
                   _state(dev).get_cnt(M // 16), yf)              # the plain GEMV's fp32 accumulators of this shard
            parts = [torch.empty_like(yf) for _ in range(world)]
            dist.all_gather(parts, yf)
            acc = torch.zeros_like(yf)
            for p_ in parts:
                acc += p_
            y = torch.empty(B, M, dtype=torch.bfloat16, device=dev)
            got32 = torch.empty(B, M, dtype=torch.float32, device=dev)
            comm.gemv_allreduce(tl.tree, eo, eb, el, x, y, ws, got32)
            torch.cuda.synchronize()
            assert torch.equal(got32, acc), (M, N, B, it, (got32 - acc).abs().max().item())
            assert torch.equal(y, acc.to(torch.bfloat16)), (M, N, B, it)
        if B == 1:
            x = torch.randn(B, Nr, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(B, M, dtype=torch.bfloat16, device=dev)
            comm.gemv_allreduce(tl.tree, eo, eb, el, x, y, ws)
            want = y.clone()
            side.wait_stream(torch.cuda.current_stream(dev))
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=side):
                for _ in range(7):                              # an odd count: replays start on alternating parities
                    comm.gemv_allreduce(tl.tree, eo, eb, el, x, y, ws)
            for _ in range(10):
                y.zero_()
                g2.replay()
                torch.cuda.synchronize()
                assert torch.equal(y, want), (M, N)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    dist.barrier()
    if rank == 0:
        print("PEER_COMM_OK")
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
