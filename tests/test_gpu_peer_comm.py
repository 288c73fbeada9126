"""Peer-memory all-reduce (csrc/st_comm.cu) on two GPUs of one node; skipped where fewer are visible.  The CPU-side
rules of the partition it serves are covered by tests/test_parallel_cpu.py."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_peer_allreduce_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "peer_comm_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "PEER_COMM_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.gpu
def test_wait_on_absent_peer_runs_out_and_reports():
    """One GPU, a second buffer standing in for a rank that never arrives: the kernel's bounded wait (set to 300 ms
    here) runs out, the output stays unwritten, the status word says so and the context remains usable."""
    import ctypes
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "statetree-representation_b200"))
    from statetree_b200 import ops
    L = ops.lib()
    torch.cuda.set_device(0)
    assert ops.device_status() == 0
    ops._check(L.st_comm_set_timeout_ms(300))
    own, absent = ctypes.c_void_p(), ctypes.c_void_p()
    ops._check(L.st_comm_alloc(ctypes.byref(own)))
    ops._check(L.st_comm_alloc(ctypes.byref(absent)))
    try:
        bufs = (ctypes.c_void_p * 2)(own.value, absent.value)
        y = torch.ones(4096, dtype=torch.bfloat16, device="cuda")
        out = torch.full((4096,), 7.0, dtype=torch.bfloat16, device="cuda")
        ops._check(L.st_allreduce(bufs, 0, 2, y.data_ptr(), out.data_ptr(), y.numel(),
                                  torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert ops.device_status() == 5                              # ERR_WAIT_PEER
        assert bool((out == 7.0).all())                             # nothing was written
        assert ops.device_status() == 0                              # read-and-clear; the context still works
        assert float((y + y).float().sum()) == 2 * 4096
    finally:
        ops._check(L.st_comm_set_timeout_ms(20000))
        ops._check(L.st_comm_free(own))
        ops._check(L.st_comm_free(absent))


@pytest.mark.gpu
def test_gemv_that_sums_over_ranks_on_one_gpu():
    """The row-parallel GEMV that adds the ranks' sums itself (st_gemv_allreduce), two "ranks" on ONE GPU with a buffer
    each.  Kernels that wait on one another cannot run together on one GPU, so the ranks run in turn: rank 1 first,
    with a 300 ms limit; it delivers its sums to both buffers, finds rank 0's missing, gives up (status 5, its output
    unwritten).  Rank 0 then finds rank 1's words waiting and completes: its output must equal the fp32 sum of both
    shards' accumulators rounded to BF16, and the fp64 product over the whole matrix within the usual bars; its
    receive words and exchange slots are left empty."""
    import ctypes
    import numpy as np
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "statetree-representation_b200"))
    sys.path.insert(0, HERE)
    import gen_inputs as G
    import oracle
    from statetree_b200 import ops
    from util import bits_to_torch, layer_from_oracle, rel_fro
    L, E = ops.lib(), ops.ext()
    torch.cuda.set_device(0)
    assert ops.device_status() == 0
    ops._check(L.st_comm_set_timeout_ms(300))
    try:
        for (M, N, B) in ((256, 1024, 1), (512, 2048, 5), (4096, 1024, 1), (1024, 512, 12), (192, 256, 20)):
            b0, b1 = ctypes.c_void_p(), ctypes.c_void_p()
            ops._check(L.st_comm_alloc(ctypes.byref(b0)))
            ops._check(L.st_comm_alloc(ctypes.byref(b1)))
            bufs = (ctypes.c_void_p * 2)(b0.value, b1.value)
            W = G.weights(M, N, M + N + B, "mixed")
            X = G.to_bf16_bits(np.random.RandomState(B).standard_normal((B, N)))
            half = N // 2
            parts, accs = [], []
            for r in range(2):
                tl, _ = layer_from_oracle(np.ascontiguousarray(W[:, r * half:(r + 1) * half]))
                eo, el, eb = tl.tables()
                xr = bits_to_torch(np.ascontiguousarray(X[:, r * half:(r + 1) * half]), "cuda")
                yf = torch.empty(B, M, dtype=torch.float32, device="cuda")
                E.gemv(tl.tree, eo, eb, el, xr, torch.empty(B, M, dtype=torch.bfloat16, device="cuda"),
                       torch.full((max(E.gemv_workspace_bytes(M, half, B) // 4, 1),), -1, dtype=torch.int32,
                                  device="cuda").view(torch.float32),
                       torch.zeros(M // 16, dtype=torch.int32, device="cuda"), yf)   # the plain GEMV's fp32 accumulators
                parts.append((tl, eo, el, eb, xr))
                accs.append(yf)
            nbytes = E.gemv_workspace_bytes(M, half, B)
            ws = torch.full((max(nbytes // 4, 1),), -1, dtype=torch.int32, device="cuda")
            ys = [torch.full((B, M), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
            yf0 = torch.empty(B, M, dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            for r in (1, 0):
                tl, eo, el, eb, xr = parts[r]
                ops._check(L.st_gemv_allreduce(bufs, r, 2, tl.tree.data_ptr(), eo.data_ptr(), eb.data_ptr(), el.data_ptr(),
                                               xr.data_ptr(), ys[r].data_ptr(), yf0.data_ptr() if r == 0 else None, B, M,
                                               half, ws.data_ptr(), ws.numel() * 4,
                                               torch.cuda.current_stream().cuda_stream))
                torch.cuda.synchronize()
                if r == 1:
                    assert ops.device_status() == 5                      # rank 0 never delivered: the wait ran out
                    assert bool((ys[1] == 7.0).all())
                else:
                    assert ops.device_status() == 0
            want32 = accs[0] + accs[1]                                    # rank order, fp32
            assert torch.equal(yf0, want32), (M, N, B)
            assert torch.equal(ys[0], want32.to(torch.bfloat16)), (M, N, B)
            ref = oracle.linear_f64(W, X)
            assert rel_fro(yf0.cpu().numpy(), ref) < 1e-3
            assert bool((ws == -1).all())
            ops._check(L.st_comm_free(b0))
            ops._check(L.st_comm_free(b1))
    finally:
        ops._check(L.st_comm_set_timeout_ms(20000))
