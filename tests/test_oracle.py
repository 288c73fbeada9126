"""The CPU oracle against the golden fixtures made from the reference's format.py (tests/golden/make_golden.py)."""
import hashlib
import json
import os

import numpy as np
import pytest

import gen_inputs as G
import oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def small():
    return np.load(os.path.join(GOLD, "weights_small.npz"))


@pytest.mark.parametrize("name", ["mixed", "heavy", "each", "llm"])
def test_encode_matches_reference_bytes(small, name):
    W = small[f"{name}_W"]
    enc = oracle.encode(W)
    assert np.array_equal(enc["tree"], small[f"{name}_tree"])
    for k in ("esc_rows", "esc_cols", "esc_bits"):
        assert np.array_equal(enc[k], small[f"{name}_{k}"]), k
    back = oracle.decode(small[f"{name}_tree"], small[f"{name}_esc_rows"], small[f"{name}_esc_cols"],
                         small[f"{name}_esc_bits"])
    assert np.array_equal(back, W)
    assert oracle.escape_count(W) == small[f"{name}_esc_rows"].size


def test_large_cases_match_reference_digests():
    with open(os.path.join(GOLD, "weights_digests.json")) as f:
        dig = json.load(f)
    for key, d in dig.items():
        W = G.weights(d["M"], d["N"], d["seed"], d["regime"])
        assert sha(W) == d["W"], key                       # the seeded generator reproduced the input
        enc = oracle.encode(W)
        assert enc["esc_rows"].size == d["n_esc"], key
        assert sha(enc["tree"]) == d["tree"], key
        for k in ("esc_rows", "esc_cols", "esc_bits"):
            assert sha(enc[k]) == d[k], (key, k)
        assert np.array_equal(oracle.decode(**enc), W), key


def test_pure_python_record_agrees_with_c(small):
    W = small["mixed_W"]
    enc = oracle.encode(W)
    for t, g in ((0, 0), (1, 1), (6, 0), (2, 2)):
        rec, esc = oracle.encode_record_py(W[t * 16:(t + 1) * 16, g * 64:(g + 1) * 64])
        assert np.array_equal(rec, enc["tree"][t, g])
        want = [(int(r) - t * 16, int(c) - g * 64, int(b) & 0xFFFF) for r, c, b in
                zip(enc["esc_rows"], enc["esc_cols"], enc["esc_bits"]) if r // 16 == t and c // 64 == g]
        assert esc == want


def _fresh(nb, H, P=4096):
    return (np.zeros((nb, H, 2, 2, oracle.RKV), dtype=np.uint8), np.zeros((P, 16), dtype=np.uint32),
            np.zeros(2, dtype=np.int32))


@pytest.mark.parametrize("name", ["tiny", "chan"])
def test_kv_records_match_reference_bytes(name):
    g = np.load(os.path.join(GOLD, "kv_records.npz"))
    K, V = g[f"{name}_K"], g[f"{name}_V"]
    n, H, _ = K.shape
    kv, pool, cnt = _fresh(n // 16, H)
    # append in two calls that split a page, then check bytes, headers and slots
    cut = 21
    slots = np.arange(n, dtype=np.int64)
    oracle.kv_append(K[:cut], V[:cut], slots[:cut], kv, pool, cnt)
    oracle.kv_append(K[cut:], V[cut:], slots[cut:], kv, pool, cnt)
    i = 0
    for kvi in range(2):
        for p in range(n // 16):
            for h in range(H):
                for half in range(2):
                    rec = kv[p, h, kvi, half]
                    assert np.array_equal(rec[:1552], g[f"{name}_records"][i]), (kvi, p, h, half)
                    head = int(rec[1552:1556].view(np.uint32)[0])
                    c = int(g[f"{name}_counts"][i])
                    assert (head & 15) == min(c, 11)
                    assert bool(head & 16) == (c > 11)
                    assert np.array_equal(rec[1556:1600].view(np.uint32)[:min(c, 11)],
                                          g[f"{name}_slots"][i][:min(c, 11)])
                    i += 1
    Kd, Vd = oracle.kv_dequant_blocks(kv, pool)
    assert np.array_equal(Kd.reshape(n, H, 128), K) and np.array_equal(Vd.reshape(n, H, 128), V)
    assert cnt[1] == 0


def test_kv_pool_chains_recycle_and_stay_lossless():
    H, nb = 2, 12
    kv, pool, cnt = _fresh(nb, H, P=8192)
    rs = np.random.RandomState(0)
    used = []
    for rnd, tiny in enumerate((0.3, 0.5, 0.1, 0.5)):
        K, V = G.kv_tokens(nb * 16 - 5, H, seed=20 + rnd, tiny=tiny)
        perm = rs.permutation(nb)
        pos = np.arange(K.shape[0])
        slots = (perm[pos // 16] * 16 + pos % 16).astype(np.int64)
        for a, b in ((0, 37), (37, 38), (38, K.shape[0])):
            oracle.kv_append(K[a:b], V[a:b], slots[a:b], kv, pool, cnt, reuse=True)
        Kd, Vd = oracle.kv_dequant_blocks(kv, pool, perm.astype(np.int32))
        assert np.array_equal(Kd.reshape(-1, H, 128)[:K.shape[0]], K)
        assert np.array_equal(Vd.reshape(-1, H, 128)[:K.shape[0]], V)
        assert cnt[1] == 0
        used.append(int(cnt[0]))
    assert used[0] > 0 and used[-1] < 1.6 * used[1], used
    # out-of-range block ids decode to zeros
    Kd, Vd = oracle.kv_dequant_blocks(kv, pool, np.array([-1, nb, 3], dtype=np.int32))
    assert not Kd[:2].any() and not Vd[:2].any()
    # an undersized pool raises the error flag instead of dropping escapes silently
    kv2, pool2, cnt2 = _fresh(2, H, P=1)
    K, V = G.kv_tokens(32, H, seed=5, tiny=0.6)
    oracle.kv_append(K, V, np.arange(32, dtype=np.int64), kv2, pool2, cnt2)
    assert cnt2[1] == 1


def test_attention_oracle_against_dense_numpy():
    H, Hq, n = 2, 8, 75
    K, V = G.kv_tokens(n, H, seed=3, tiny=0.02)
    kv, pool, cnt = _fresh(8, H)
    bt = np.array([[5, 2, 7, 0, 1, 3, 4, 6]], dtype=np.int32)
    pos = np.arange(n)
    oracle.kv_append(K, V, (bt[0][pos // 16] * 16 + pos % 16).astype(np.int64), kv, pool, cnt)
    q = G.to_bf16_bits(np.random.RandomState(4).standard_normal((1, Hq, 128)))
    for start in (0, 19):
        got = oracle.kv_attn_f64(q, kv, pool, bt, np.array([n], np.int32), 128 ** -0.5,
                                 None if start == 0 else np.array([start], np.int32))
        kf = G.bits_to_f32(K).astype(np.float64)[start:].repeat(Hq // H, axis=1)
        vf = G.bits_to_f32(V).astype(np.float64)[start:].repeat(Hq // H, axis=1)
        qf = G.bits_to_f32(q).astype(np.float64)[0]
        s = np.einsum("hd,lhd->hl", qf, kf) * 128 ** -0.5
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        want = np.einsum("hl,lhd->hd", p, vf)
        assert np.abs(got[0] - want).max() < 1e-12
    z = oracle.kv_attn_f64(q, kv, pool, bt, np.array([0], np.int32), 1.0)
    assert not z.any()


def test_linear_cpu_path():
    W = G.weights(64, 256, 9, "mixed")
    enc = oracle.encode(W)
    X = G.to_bf16_bits(np.random.RandomState(1).standard_normal((3, 256)))
    y = G.bits_to_f32(oracle.linear_cpu(enc, X)).astype(np.float64)
    ref = oracle.linear_f64(W, X)
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 5e-3
    # one-hot activations read columns of W back bit for bit
    X1 = np.zeros((2, 256), dtype=np.uint16)
    X1[0, 70] = 0x3F80
    X1[1, 5] = 0x3F80
    y1 = oracle.linear_cpu(enc, X1)
    assert np.array_equal(y1[0] & 0x7FFF, W[:, 70] & 0x7FFF) and np.array_equal(y1[1] & 0x7FFF, W[:, 5] & 0x7FFF)
