"""st_gemv_static, the GEMV entry point for callers that cannot allocate device memory (its scratch is an array built
into the library): called through the C ABI twice in a row and compared with st_gemv, which takes caller workspaces.
Both run the same kernel with the same split, so the outputs must be identical bit for bit.  This file sorts last so
that a failure here cannot hide the result of any other test."""
import numpy as np
import pytest
import torch

import gen_inputs as G
from util import bits_to_torch, layer_from_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("M,N,B", [(2048, 4096, 1), (512, 1024, 8), (1024, 768, 12), (256, 2048, 32)])
def test_static_scratch_entry_matches_workspace_entry(M, N, B):
    from statetree_b200 import ops
    W = G.weights(M, N, M + N + B, "mixed")
    tl, _ = layer_from_oracle(W)
    eo, el, eb = tl.tables()
    E = ops.ext()
    x = bits_to_torch(G.to_bf16_bits(np.random.RandomState(B).standard_normal((B, N))), DEV)
    want = torch.empty(B, M, dtype=torch.bfloat16, device=DEV)
    ws = torch.full((max(1, E.gemv_workspace_bytes(M, N, B) // 4),), -1, dtype=torch.int32, device=DEV).view(torch.float32)
    cnt = torch.zeros(M // 16, dtype=torch.int32, device=DEV)
    E.gemv(tl.tree, eo, eb, el, x, want, ws, cnt)
    for call in range(2):                                   # the second call reuses what the first left in the scratch
        got = torch.full((B, M), 7.0, dtype=torch.bfloat16, device=DEV)
        E.gemv_static(tl.tree, eo, eb, el, x, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (M, N, B, call, (got.float() - want.float()).abs().max().item())
    assert ops.device_status() == 0


def test_static_scratch_entry_rejects_what_does_not_fit():
    from statetree_b200 import ops
    L = ops.lib()
    one = torch.zeros(16, dtype=torch.uint8, device=DEV)
    p = one.data_ptr()
    # more 16-row tiles than the built-in array has semaphores for: refused before any launch
    rc = L.st_gemv_static(p, p, p, p, p, p, 1, 16 * 16385, 64, None)
    assert rc != 0 and b"built-in scratch" in L.st_last_error()
    rc = L.st_gemv_static(p, p, p, p, p, p, 40, 64, 64, None)
    assert rc != 0 and b"batch" in L.st_last_error()
