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
