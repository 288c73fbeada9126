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
