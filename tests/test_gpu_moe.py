"""GPU parity of the mixture-of-experts kernels: slot and grouped products, routing-weighted sum, SwiGLU gate."""
import numpy as np
import pytest
import torch

import gen_inputs as G
from util import bits_to_torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _experts(E, M, N, seed, heavy=None):
    from statetree_b200 import TreeLinear
    Ws = []
    for e in range(E):
        Ws.append(G.weights(M, N, seed * 1000 + e, "heavy" if e == heavy else "mixed"))
    mods = [TreeLinear.from_weight(bits_to_torch(W, DEV)) for W in Ws]
    return Ws, mods


def test_slot_and_grouped_products_match_fp64():
    from statetree_b200.experts import expert_tables, moe_align, moe_gemv, moe_group_gemv, moe_wsum, silu_mul
    E, M, N = 32, 256, 512
    Ws, mods = _experts(E, M, N, 1)
    tabs = expert_tables(mods)
    Wall = torch.stack([bits_to_torch(W, DEV) for W in Ws]).double()
    g = torch.Generator(DEV).manual_seed(0)
    for S, K in ((1, 1), (8, 4), (64, 8), (300, 4)):
        ids = torch.randint(0, E, (S,), device=DEV, generator=g)
        x = torch.randn(S // K, N, device=DEV, generator=g).to(torch.bfloat16)
        ref = torch.einsum("sn,smn->sm", x.repeat_interleave(K, 0).double(), Wall[ids])
        outs = {"slot": moe_gemv(tabs, x, ids, M, K), "slot_i32": moe_gemv(tabs, x, ids.int(), M, K)}
        al = moe_align(ids, E, 8)
        sid = al[0][al[0] < S]
        assert torch.equal(sid.sort().values, torch.arange(S, device=DEV, dtype=torch.int32))   # every pair once
        outs["group"] = moe_group_gemv(tabs, x, al, S, M, K)
        for k, y in outs.items():
            rel = float((y.double() - ref).norm() / ref.norm())
            assert rel < 4e-3, (S, k, rel)
        assert torch.equal(outs["slot"], outs["slot_i32"])
        bad = ids.int().clone()                          # ids outside [0, E) are clamped in the kernel
        bad[0] = E + 5
        if S > 1:
            bad[-1] = -2
        assert torch.equal(moe_gemv(tabs, x, bad, M, K), moe_gemv(tabs, x, bad.clamp(0, E - 1), M, K)), S
        # another rank's experts: negative block ids are skipped and their rows stay untouched
        bexp = al[1].clone()
        bexp[bexp % 2 == 1] = -1
        y = torch.full((S, M), 7.0, dtype=torch.bfloat16, device=DEV)
        from statetree_b200.linear import _state
        from statetree_b200.ops import ext
        st = _state(torch.device(DEV))
        ws = st.get_ws(ext().moe_group_workspace_bytes(bexp.numel(), M, N))
        ext().mvg(*tabs, x, al[0], bexp, al[2], y, ws, st.get_cnt(bexp.numel() * (M // 16)), K)
        odd = (ids % 2 == 1)
        assert bool((y[odd] == 7.0).all()) and torch.equal(y[~odd], outs["group"][~odd])
    T, K, Hd = 5, 3, 64
    y = torch.randn(T * K, Hd, device=DEV, generator=g).to(torch.bfloat16)
    for w in (torch.rand(T, K, device=DEV, generator=g), torch.rand(T, K, device=DEV, generator=g).to(torch.bfloat16)):
        got = moe_wsum(y, w).float()
        want = (y.view(T, K, Hd).float() * w.float().unsqueeze(-1)).sum(1)
        assert bool(((got - want).abs() <= want.abs() * 2.0 ** -8 + 1e-6).all())          # one BF16 rounding
    gu = torch.randn(7, 2 * 96, device=DEV, generator=g).to(torch.bfloat16)
    want = (torch.nn.functional.silu(gu[:, :96].float()).to(torch.bfloat16) * gu[:, 96:])
    assert (silu_mul(gu).float() - want.float()).abs().max().item() < 2e-2
    from statetree_b200 import ops
    assert ops.device_status() == 0


def test_one_hot_inputs_read_expert_columns_exactly():
    from statetree_b200.experts import expert_tables, moe_align, moe_gemv, moe_group_gemv
    E, M = 12, 256
    for N in (256, 768):
        Ws, mods = _experts(E, M, N, 2 + N, heavy=3)
        assert mods[3].esc_rows.numel() > 0.15 * M * N
        tabs = expert_tables(mods)
        g = torch.Generator(DEV).manual_seed(N)
        for S in (1, 8, 37, 200):
            ids = torch.randint(0, E, (S,), device=DEV, generator=g)
            ids[: S // 3] = 3                                              # the escape-heavy expert
            cols = torch.randint(0, N, (S,), device=DEV, generator=g)
            x = torch.zeros(S, N, device=DEV, dtype=torch.bfloat16)
            x[torch.arange(S, device=DEV), cols] = 1.0
            want = torch.stack([bits_to_torch(Ws[int(e)][:, int(c)], DEV) for e, c in zip(ids.tolist(), cols.tolist())])
            outs = {"slot": moe_gemv(tabs, x, ids, M, 1),
                    "group": moe_group_gemv(tabs, x, moe_align(ids, E, 8), S, M, 1)}
            for k, y in outs.items():
                assert torch.equal(y, want), (N, S, k, (y.float() - want.float()).abs().max().item())


def test_tree_experts_block_matches_dense():
    from statetree_b200.experts import TreeExperts
    E, Hd, I, K = 16, 256, 128, 4
    g = torch.Generator(DEV).manual_seed(3)
    gate_up = (torch.randn(E, 2 * I, Hd, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    down = (torch.randn(E, Hd, I, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    te = TreeExperts.from_weights(gate_up, down)
    for T in (1, 4, 8, 40):
        x = torch.randn(T, Hd, device=DEV, generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, device=DEV, generator=g)
        w, ids = torch.softmax(logits, -1).topk(K, -1)
        got = te(x, ids, w).double()
        ref = torch.zeros(T, Hd, dtype=torch.float64, device=DEV)
        for t in range(T):
            for j in range(K):
                e = int(ids[t, j])
                gu = gate_up[e].double() @ x[t].double()
                act = torch.nn.functional.silu(gu[:I]) * gu[I:]
                ref[t] += float(w[t, j]) * (down[e].double() @ act)
        assert float((got - ref).norm() / ref.norm()) < 2e-2, T
        if T <= 8:
            # the reference's functional names for the same block and its small-K products
            from statetree_b200 import experts as X
            t13, t2 = X.expert_tables(list(te.w13)), X.expert_tables(list(te.w2))
            fused = X.moe_fused_decode(t13, t2, x, ids.reshape(-1), w, I)
            assert float((fused.double() - ref).norm() / ref.norm()) < 2e-2, T
            flat = ids.reshape(-1)
            assert torch.equal(X.moe_gemv_w(t13, x, flat, 2 * I, K), X.moe_gemv(t13, x, flat, 2 * I, K))
        # expert parallelism: experts split over two ranks, partial outputs add up
        emap0 = torch.where(torch.arange(E, device=DEV) < E // 2, torch.arange(E, device=DEV), -1).int()
        emap1 = torch.where(torch.arange(E, device=DEV) >= E // 2, torch.arange(E, device=DEV) - E // 2, -1).int()
        te0 = TreeExperts(list(te.w13)[:E // 2], list(te.w2)[:E // 2])
        te1 = TreeExperts(list(te.w13)[E // 2:], list(te.w2)[E // 2:])
        part = te0(x, ids, w, emap0).double() + te1(x, ids, w, emap1).double()
        assert float((part - ref).norm() / ref.norm()) < 2e-2, T


@pytest.mark.gpu
def test_moe_align_kernel_matches_torch_formulation():
    from statetree_b200.experts import _moe_align_torch, moe_align
    gen = torch.Generator(device="cuda").manual_seed(3)
    for S, E, dt in ((1, 8, torch.int64), (8, 128, torch.int64), (64, 128, torch.int32), (512, 128, torch.int64),
                     (513, 129, torch.int64), (4096, 60, torch.int32), (20000, 1024, torch.int64), (300, 1, torch.int64)):
        ids = torch.randint(0, E, (S,), device="cuda", generator=gen).to(dt)
        if S >= 64:
            ids[: S // 3] = ids[0]                                  # a crowded expert
        for used in (None, max(1, E - 1)):
            got = moe_align(ids, E, 8, used)
            want = _moe_align_torch(ids, E, 8, used)
            for g, w, name in zip(got, want, ("sorted_ids", "bexp", "npost")):
                assert g.dtype == w.dtype and torch.equal(g, w), (S, E, used, name)


@pytest.mark.parametrize("bs", [64, 128])
def test_grouped_tcgen05_gemm_matches_fp64(bs):
    """the grouped fused decode + tcgen05 GEMM against fp64, after the reference's gtt test (tests/test_moe.py:282-315):
    escapes (one expert with a fifth of its weights escaping), an expert without pairs, experts with several blocks,
    padded blocks, one row per token (xdiv = k) and one row per pair, one-hot rows read exact weights back, other
    ranks' blocks skipped, repeat runs bit-identical"""
    from statetree_b200.experts import expert_tables, moe_align, moe_group_gemm, moe_group_gemv
    from statetree_b200.ops import ext
    E, M, N = 12, 256, 320
    Ws, mods = _experts(E, M, N, 5, heavy=3)
    tabs = expert_tables(mods)
    maps = ext().moe_tensor_maps([m.tree for m in mods], M, N)
    Wall = torch.stack([bits_to_torch(W, DEV) for W in Ws]).double()
    g = torch.Generator(DEV).manual_seed(bs)
    for S, K in ((5, 1), (96, 4), (1000, 4), (777, 1)):
        ids = torch.randint(0, E - 1, (S,), device=DEV, generator=g)       # expert E - 1 gets no pairs
        ids[:S // 3] = 7                                                    # one expert with several blocks
        ids[S // 3:S // 3 + min(S, 50)] = 3                                 # the escape-heavy one
        x = torch.randn(-(-S // K), N, device=DEV, generator=g).to(torch.bfloat16)
        ref = torch.einsum("sn,smn->sm", x.repeat_interleave(K, 0)[:S].double(), Wall[ids])
        al = moe_align(ids, E, bs)
        yf = torch.zeros(S, M, dtype=torch.float32, device=DEV)
        y = moe_group_gemm(tabs, maps, x, al, bs, S, M, K, yf32=yf)
        assert float((yf.double() - ref).norm() / ref.norm()) < 1e-3, (S, K)           # fp32 accumulators
        assert torch.equal(y, yf.to(torch.bfloat16)), (S, K)
        assert float((y.double() - ref).norm() / ref.norm()) < 5e-3, (S, K)
        assert torch.equal(moe_group_gemm(tabs, maps, x, al, bs, S, M, K), y), (S, K)  # deterministic
        # other ranks' experts: blocks with a negative expert are skipped, their rows stay as they were
        bexp = al[1].clone()
        bexp[bexp % 2 == 1] = -1
        part = moe_group_gemm(tabs, maps, x, (al[0], bexp, al[2]), bs, S, M, K, zero=True)
        odd = ids % 2 == 1
        assert int((part[odd] != 0).sum()) == 0 and torch.equal(part[~odd], y[~odd])
    # one-hot rows: the exact weights come back, escapes included
    S = 300
    ids = torch.randint(0, E, (S,), device=DEV, generator=g)
    ids[:100] = 3
    cols = torch.randint(0, N, (S,), device=DEV, generator=g)
    x = torch.zeros(S, N, device=DEV, dtype=torch.bfloat16)
    x[torch.arange(S, device=DEV), cols] = 1.0
    want = torch.stack([bits_to_torch(Ws[int(e)][:, int(c)], DEV) for e, c in zip(ids.tolist(), cols.tolist())])
    got = moe_group_gemm(tabs, maps, x, moe_align(ids, E, bs), bs, S, M, 1)
    assert torch.equal(got, want)
    assert torch.equal(got, moe_group_gemv(tabs, x, moe_align(ids, E, 8), S, M, 1))
    from statetree_b200 import ops
    assert ops.device_status() == 0


def test_tree_experts_prefill_sized_call_uses_the_grouped_gemm():
    from statetree_b200 import experts as X
    E, Hd, I, K = 8, 256, 128, 2
    g = torch.Generator(DEV).manual_seed(9)
    gate_up = (torch.randn(E, 2 * I, Hd, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    down = (torch.randn(E, Hd, I, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    te = X.TreeExperts.from_weights(gate_up, down)
    T = 300                                                                # 600 pairs on 8 experts: the GEMM regime
    assert T * K >= X.GEMM_PAIRS_PER_EXPERT * E and te.tensor_maps() is not None
    x = torch.randn(T, Hd, device=DEV, generator=g).to(torch.bfloat16)
    w, ids = torch.softmax(torch.randn(T, E, device=DEV, generator=g), -1).topk(K, -1)
    got = te(x, ids, w).double()
    gu = torch.einsum("tkmh,th->tkm", gate_up[ids].double(), x.double())
    act = torch.nn.functional.silu(gu[..., :I]) * gu[..., I:]
    ref = (torch.einsum("tkhi,tki->tkh", down[ids].double(), act) * w.double().unsqueeze(-1)).sum(1)
    assert float((got - ref).norm() / ref.norm()) < 2e-2


def test_moe_route_matches_torch():
    """softmax + top-k + renormalisation in one launch against the PyTorch formulation it replaces; the expert-map form
    returns local ids and zero weights for other ranks' experts"""
    from statetree_b200 import ops
    E_ = ops.ext()
    gen = torch.Generator(device=DEV).manual_seed(5)
    for (T, E, K, dt) in ((1, 128, 8, torch.bfloat16), (7, 128, 8, torch.float32), (64, 60, 4, torch.bfloat16),
                          (3, 1024, 32, torch.float32), (5, 8, 2, torch.bfloat16), (2, 1, 1, torch.float32)):
        logits = (torch.randn(T, E, device=DEV, generator=gen) * 3).to(dt)
        probs = torch.softmax(logits.float(), -1)
        w_ref, i_ref = probs.topk(K, -1)
        w_ref = w_ref / w_ref.sum(-1, keepdim=True)
        ids, w = E_.moe_route(logits, K, True)
        torch.cuda.synchronize()
        # ties in BF16 logits may be ordered differently by topk: compare the picked probabilities, and the ids where
        # the picked values are distinct
        assert torch.allclose(w, w_ref, rtol=2e-5, atol=1e-7), (T, E, K)
        picked = torch.gather(probs, 1, ids.long())
        assert torch.allclose(picked / picked.sum(-1, keepdim=True), w_ref, rtol=2e-5, atol=1e-7)
        distinct = torch.ones_like(ids, dtype=torch.bool)
        srt = torch.sort(logits.float(), -1, descending=True).values[:, :K + 1] if E > K else None
        if srt is not None:
            distinct = (srt[:, :-1] != srt[:, 1:]) & torch.cat([torch.ones(T, 1, dtype=torch.bool, device=DEV),
                                                                 srt[:, :-2] != srt[:, 1:-1]], 1)
        assert torch.equal(ids[distinct], i_ref.to(torch.int32)[distinct]), (T, E, K)
        ids2, w2 = E_.moe_route(logits, K, False)
        assert torch.allclose(w2, probs.topk(K, -1).values, rtol=2e-5, atol=1e-7)
        if E >= 4:
            emap = torch.where(torch.arange(E, device=DEV) % 2 == 0, torch.arange(E, device=DEV) // 2,
                               torch.full((E,), -1, device=DEV)).to(torch.int32)
            ids3, w3 = E_.moe_route(logits, K, True, emap)
            local = emap[ids.long()]
            assert torch.equal(ids3, local.clamp(min=0))
            assert torch.equal(w3, torch.where(local >= 0, w, torch.zeros_like(w)))
    _ = ops.device_status()
    assert _ == 0


def test_tree_experts_replaces_a_transformers_experts_module():
    """TreeExperts.from_experts on a Transformers 5 experts module (3-D gate_up_proj / down_proj): same call, same
    result as the BF16 module within BF16 rounding, for few pairs (slot kernel), many pairs (grouped kernels) and ids
    beyond the experts (another rank's pairs contribute nothing); a module with biases takes the expert-by-expert path"""
    transformers = pytest.importorskip("transformers")
    from transformers import Qwen3MoeConfig
    from transformers.models.qwen3_moe.modeling_qwen3_moe import Qwen3MoeExperts
    from statetree_b200.experts import TreeExperts, expert_layout
    cfg = Qwen3MoeConfig(hidden_size=128, moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2)
    torch.manual_seed(7)
    src = Qwen3MoeExperts(cfg).to(torch.bfloat16).to(DEV)
    with torch.no_grad():
        for prm in src.parameters():
            prm.copy_((torch.randn(prm.shape, device=DEV) * 0.05).to(torch.bfloat16))
    import copy
    ref = copy.deepcopy(src)
    te = TreeExperts.from_experts(src, verify=True)
    assert expert_layout(src) is None and te._fast_ok()          # the source's 3-D tensors are gone
    gen = torch.Generator(device=DEV).manual_seed(3)
    for T in (1, 4, 64, 700):
        x = torch.randn(T, 128, device=DEV, generator=gen).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(8, device=DEV, generator=gen)[:2] for _ in range(T)])
        w = torch.rand(T, 2, device=DEV, generator=gen).to(torch.bfloat16)
        want = ref(x, ids, w).float()
        got = te(x, ids, w).float()
        assert got.shape == want.shape
        assert (got - want).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-3, T
        # pairs of another rank's experts (ids >= E) contribute nothing
        ids2 = ids.clone()
        ids2[:, 1] = 8
        only_first = te(x, ids2, w).float()
        w0 = w.clone()
        w0[:, 1] = 0
        assert torch.allclose(only_first, te(x, ids, w0).float(), atol=1e-6)
    # biases: the generic path through the layers
    class Biased(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.is_transposed, self.has_bias, self.has_gate, self.num_experts = True, True, True, 4
            mk = lambda *sh: torch.nn.Parameter((torch.randn(*sh, device=DEV) * 0.05).to(torch.bfloat16))   # noqa: E731
            self.gate_up_proj, self.gate_up_proj_bias = mk(4, 128, 128), mk(4, 128)
            self.down_proj, self.down_proj_bias = mk(4, 64, 128), mk(4, 128)
            self.act_fn = torch.nn.SiLU()
    b = Biased()
    Wu, bu, Wd, bd = (t.detach().clone() for t in (b.gate_up_proj, b.gate_up_proj_bias, b.down_proj, b.down_proj_bias))
    tb = TreeExperts.from_experts(b, verify=True)
    assert not tb._fast_ok() and tb.has_bias
    x = torch.randn(6, 128, device=DEV, generator=gen).to(torch.bfloat16)
    ids = torch.randint(0, 4, (6, 2), device=DEV, generator=gen)
    w = torch.rand(6, 2, device=DEV, generator=gen)
    got = tb(x, ids, w).float()
    want = torch.zeros(6, 128, device=DEV)
    for t in range(6):
        for j in range(2):
            e = int(ids[t, j])
            h = (x[t].float() @ Wu[e].float() + bu[e].float()).to(torch.bfloat16)
            g, u = h.chunk(2)
            a = torch.nn.functional.silu(g) * u
            want[t] += w[t, j] * (a.float() @ Wd[e].float() + bd[e].float()).to(torch.bfloat16).float()
    assert (got - want).abs().max().item() <= 0.03 * want.abs().max().item() + 1e-3
