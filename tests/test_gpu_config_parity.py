"""GPU parity at the benchmark's own sizes, through the module API (TreeLinear, PageStore).

Linears: the four Qwen3-8B shapes (4096x4096, 1024x4096, 12288x4096, 4096x12288), N(0, 0.02) weights with 1% of the
columns scaled x8, seeds 0-4 at one activation row and one seed at 8 / 32 / 64 / 256 rows, so the GEMV (up to 10 rows)
and the tcgen05 GEMM (beyond) both run their full-size grids.  Bars as in the reference's kernel tests
(tests/test_kernels.py:47-72, 75-115): fp32 accumulators within 1e-3 relative Frobenius error of the oracle's fp64
product, BF16 output == rounded accumulator, one-hot activations read escape columns back bit for bit, reruns
bit-identical, semaphores left at zero.

Attention: K = N(0,1) x per-channel LogNormal(0,1), V, q = N(0,1); contexts 1K / 4K / 16K x batch 1 / 8 / 64 with the
split count decode_splits picks and at least 4 pages per split: pages exact through dequant_blocks, fp32 split
partials merged in fp64 within 1e-3 of the oracle's fp64 attention over the same pages (the bar of
tests/test_kv_cache.py:108-132 is 1e-2 max-abs on the BF16 output; it is asserted too).
"""
import math

import numpy as np
import pytest
import torch

import gen_inputs as G
import oracle
from util import bits_to_torch, layer_from_oracle, rel_fro, torch_to_bits

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-3
SHAPES = [(4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288)]


def _forward_checked(tl, W, X, what):
    from statetree_b200.linear import _state
    B = X.shape[0]
    x = bits_to_torch(X, DEV)
    yf = torch.empty(B, W.shape[0], dtype=torch.float32, device=DEV)
    y = tl._forward(x, yf)
    torch.cuda.synchronize()
    ref = oracle.linear_f64(W, X)
    e32 = rel_fro(yf.cpu().numpy(), ref)
    assert e32 < TOL, (what, e32)
    assert torch.equal(y, yf.to(torch.bfloat16)), (what, "BF16 output is not the rounded accumulator")
    assert rel_fro(y.float().cpu().numpy(), ref) < 5e-3, what
    assert torch.equal(tl(x), y), (what, "rerun differs")
    assert int(_state(torch.device(DEV)).cnt.abs().sum()) == 0, (what, "semaphores not reset")


@pytest.mark.parametrize("M,N", SHAPES)
def test_benchmark_linears_match_fp64(M, N):
    for seed in range(5):
        W = G.weights(M, N, seed, "llm")
        tl, enc = layer_from_oracle(W)
        assert 0 < enc["esc_rows"].size < 0.001 * W.size
        rs = np.random.RandomState(1000 + seed)
        _forward_checked(tl, W, G.to_bf16_bits(rs.standard_normal((1, N))), (M, N, seed, 1))
        if seed == 0:
            for B in (8, 32, 64, 256):
                _forward_checked(tl, W, G.to_bf16_bits(rs.standard_normal((B, N))), (M, N, seed, B))
            # one-hot activations on the columns that hold escapes: exact weights come back, GEMV and GEMM
            cols = sorted(set(enc["esc_cols"].tolist()))[:24] + [0, N - 1]
            for B in (1, 8, 64):
                x = torch.zeros(B, N, dtype=torch.bfloat16, device=DEV)
                for b in range(B):
                    x[b, cols[b % len(cols)]] = 1.0
                want = bits_to_torch(np.stack([W[:, cols[b % len(cols)]] for b in range(B)]), DEV)
                assert torch.equal(tl(x), want), (M, N, B)
        del tl
    from statetree_b200 import ops
    assert ops.device_status() == 0


def _merge64(wo, wml, B, Hq, S, D=128):
    wo = wo.cpu().numpy().astype(np.float64).reshape(B, Hq, S, D)
    ml = wml.cpu().numpy().astype(np.float64).reshape(B, Hq, S, 2)
    m, l = ml[..., 0], ml[..., 1]
    M = m.max(-1, keepdims=True)
    f = np.where(np.isfinite(m), np.exp2(m - np.where(np.isfinite(M), M, 0.0)), 0.0)
    L = (f * l).sum(-1)
    O = (f[..., None] * wo).sum(-2)
    return np.where(L[..., None] > 0, O / np.where(L[..., None] > 0, L[..., None], 1.0), 0.0)


@pytest.mark.parametrize("ctx,B", [(1024, 1), (1024, 8), (1024, 64), (4096, 1), (4096, 8), (4096, 64), (16384, 1),
                                   (16384, 8), (16384, 64)])
def test_benchmark_attention_matches_fp64(ctx, B):
    from statetree_b200.kvcache import PageStore, decode_splits
    Hq, Hkv, D = 32, 8, 128
    npg = ctx // 16
    gen = torch.Generator(device=DEV).manual_seed(ctx * 131 + B)
    layer = PageStore(B * npg, Hkv, DEV, pool_blocks=1 << 14)
    bt = torch.randperm(B * npg, device=DEV, generator=gen).view(B, npg).to(torch.int32)
    chan = torch.exp(torch.randn(Hkv, D, device=DEV, generator=gen))
    pos = torch.arange(ctx, device=DEV)
    lens_l = [ctx - (7 * b) % 23 for b in range(B)]               # ragged ends inside the last pages
    Ks, Vs = [], []
    for b in range(B):
        K = (torch.randn(ctx, Hkv, D, device=DEV, generator=gen) * chan).to(torch.bfloat16)
        V = torch.randn(ctx, Hkv, D, device=DEV, generator=gen).to(torch.bfloat16)
        slots = bt[b].long()[pos // 16] * 16 + pos % 16
        layer.append(K[:lens_l[b]], V[:lens_l[b]], slots[:lens_l[b]])
        Ks.append(K)
        Vs.append(V)
    layer.check()
    # pages exact: every stored value comes back bit for bit
    for b in range(B):
        Kd, Vd = layer.dense(bt[b])
        L = lens_l[b]
        assert torch.equal(Kd.view(-1, Hkv, D)[:L].view(torch.int16), Ks[b][:L].view(torch.int16)), b
        assert torch.equal(Vd.view(-1, Hkv, D)[:L].view(torch.int16), Vs[b][:L].view(torch.int16)), b
    q = torch.randn(B, Hq, D, device=DEV, generator=gen).to(torch.bfloat16)
    lens = torch.tensor(lens_l, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    S = decode_splits(B, Hkv, npg)
    assert S >= 2
    out = layer.attention(q, bt, lens, scale, splits=S, min_pages=4)
    torch.cuda.synchronize()
    wo, wml = layer._wo[:B * Hq * S * D], layer._wml[:B * Hq * S * 2]
    merged = _merge64(wo, wml, B, Hq, S)
    # fp64 reference: the oracle over the same pages for a bounded number of sequences (CPU time), and fp64 attention
    # over the exactly decoded values on the GPU for every sequence
    nb_or = min(B, 2 if ctx >= 16384 else 4)
    pages_h = layer.pages.cpu().numpy()
    pool_h = layer.pool.cpu().numpy().view(np.uint32)
    ref_or = oracle.kv_attn_f64(torch_to_bits(q[:nb_or]), pages_h, pool_h, bt[:nb_or].cpu().numpy(),
                                np.array(lens_l[:nb_or], np.int32), scale)
    e = rel_fro(merged[:nb_or], ref_or)
    assert e < TOL, ("oracle", ctx, B, S, e)
    ref = torch.empty(B, Hq, D, dtype=torch.float64, device=DEV)
    for b in range(B):
        L = lens_l[b]
        k = Ks[b][:L].double().permute(1, 0, 2).repeat_interleave(Hq // Hkv, 0)      # [Hq, L, D]
        v = Vs[b][:L].double().permute(1, 0, 2).repeat_interleave(Hq // Hkv, 0)
        p = torch.softmax(torch.einsum("hd,hld->hl", q[b].double(), k) * scale, -1)
        ref[b] = torch.einsum("hl,hld->hd", p, v)
    ref = ref.cpu().numpy()
    assert rel_fro(ref[:nb_or], ref_or) < 1e-9                  # the two fp64 references agree
    e = rel_fro(merged, ref)
    assert e < TOL, ("fp64", ctx, B, S, e)
    got = out.float().cpu().numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-2
    assert rel_fro(got, ref) < 5e-3
    out2 = layer.attention(q, bt, lens, scale, splits=S, min_pages=4)
    assert torch.equal(out, out2)
    from statetree_b200 import ops
    assert ops.device_status() == 0
