"""The package's torch encoder / decoder / side tables on CPU against the golden fixtures and the oracle."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import gen_inputs as G
import oracle
from statetree_b200 import format as F
from util import bits_to_torch, torch_to_bits

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", ["mixed", "heavy", "each", "llm"])
def test_encode_decode_match_reference_bytes(name):
    g = np.load(os.path.join(GOLD, "weights_small.npz"))
    W = bits_to_torch(g[f"{name}_W"])
    enc = F.encode(W, chunk_rows=32)                     # several row chunks
    assert np.array_equal(enc["tree"].numpy(), g[f"{name}_tree"])
    for k in ("esc_rows", "esc_cols", "esc_bits"):
        assert np.array_equal(enc[k].numpy(), g[f"{name}_{k}"]), k
    back = F.decode_reference(torch.from_numpy(g[f"{name}_tree"]), enc["esc_rows"], enc["esc_cols"], enc["esc_bits"])
    assert np.array_equal(torch_to_bits(back), g[f"{name}_W"])
    assert F.escape_count(W) == g[f"{name}_esc_rows"].size


def test_digests_of_larger_cases():
    with open(os.path.join(GOLD, "weights_digests.json")) as f:
        dig = json.load(f)
    for key, d in dig.items():
        enc = F.encode(bits_to_torch(G.weights(d["M"], d["N"], d["seed"], d["regime"])))
        assert sha(enc["tree"].numpy()) == d["tree"], key
        assert sha(enc["esc_bits"].numpy()) == d["esc_bits"], key
        assert abs(F.bits_per_weight(d["M"], d["N"], d["n_esc"]) - d["bits_per_weight"]) < 1e-12


def test_reference_side_tables_and_leaf_migration():
    """escape_lists / escape_chunks / escape_blocks, PERM and the leaf-format migration give the reference's bits
    (digests of statetree/format.py:141-216, 16-40 run on the same seeded matrices)"""
    with open(os.path.join(GOLD, "weights_digests.json")) as f:
        dig = json.load(f)
    for key, d in dig.items():
        M, N = d["M"], d["N"]
        enc = F.encode(bits_to_torch(G.weights(M, N, d["seed"], d["regime"])))
        esc = (enc["esc_rows"], enc["esc_cols"], enc["esc_bits"])
        got = {"lists": F.escape_lists(M, N, *esc), "chunks": F.escape_chunks(M, N, *esc),
               "blocks1": F.escape_blocks(M, N, 1, *esc), "blocks2": F.escape_blocks(M, N, 2, *esc)}
        for tag, tensors in got.items():
            assert [sha(t.numpy()) for t in tensors] == d["side_tables"][tag], (key, tag)
        v1 = F.leaves_v2_to_v1(enc["tree"])
        assert sha(v1[..., :1024].numpy()) == d["leaves_v1"], key
        assert torch.equal(F.leaves_v1_to_v2(v1), enc["tree"]), key
        assert F.PERM == d["PERM"]


def test_side_tables_are_consistent():
    g = np.load(os.path.join(GOLD, "weights_small.npz"))
    for name in ("mixed", "heavy", "each"):
        W = g[f"{name}_W"]
        M, N = W.shape
        er, ec, eb = (torch.from_numpy(g[f"{name}_{k}"]) for k in ("esc_rows", "esc_cols", "esc_bits"))
        eo, el, blk = F.escape_tables(M, N, er, ec, eb)
        assert np.array_equal(eo.numpy(), g[f"{name}_eo"])          # same per-record offsets as the reference's lists
        el_u = el.numpy().view(np.uint32)
        NG, cpt = N // 64, F.units_per_tile(N)
        # every entry patches the decoded-without-escapes matrix into the exact one
        plain = oracle.decode(g[f"{name}_tree"], er[:0].numpy(), ec[:0].numpy(), eb[:0].numpy())
        for r in range((M // 16) * NG):
            t, gcol = divmod(r, NG)
            for e in el_u[eo[r]:eo[r + 1]]:
                assert (e >> 10) & 7 == gcol % 8
                plain[t * 16 + ((e >> 6) & 15), gcol * 64 + (e & 63)] = e >> 16
        assert np.array_equal(plain, W)
        blk_u = blk.numpy().view(np.uint32)
        for u in range(blk_u.shape[0]):
            t, c = divmod(u, cpt)
            first = t * NG + c * 8
            last = min(first + 8, (t + 1) * NG)
            assert (blk_u[u, 0] & 0xFFFF) == eo[last] - eo[first] and blk_u[u, 1] == eo[first]
            for r in range(first, last):                              # bit 16 + r: record r of the unit has escapes
                assert bool((blk_u[u, 0] >> (16 + r - first)) & 1) == bool(eo[r + 1] > eo[r])
            n = min(14, int(blk_u[u, 0] & 0xFFFF))
            assert np.array_equal(blk_u[u, 2:2 + n], el_u[eo[first]:eo[first] + n])


def test_shape_checks():
    with pytest.raises(AssertionError):
        F.encode(torch.zeros(8, 64, dtype=torch.bfloat16))
    with pytest.raises(AssertionError):
        F.encode(torch.zeros(16, 64))


def test_interleave_gate_up_layout():
    """tile 2j of the fused weight = rows 16j .. 16j + 15 of gate, tile 2j + 1 = the same rows of up"""
    import torch
    from statetree_b200.linear import interleave_gate_up
    I, N = 64, 8
    g = torch.arange(I * N, dtype=torch.float32).view(I, N)
    u = -g
    w = interleave_gate_up(g, u)
    assert w.shape == (2 * I, N)
    for j in range(I // 16):
        assert torch.equal(w[32 * j:32 * j + 16], g[16 * j:16 * j + 16])
        assert torch.equal(w[32 * j + 16:32 * j + 32], u[16 * j:16 * j + 16])
