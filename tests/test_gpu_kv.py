"""GPU parity of the KV page kernels against the CPU oracle: page bytes and decoded values bit-exact, decode attention
within 1e-3 relative Frobenius error of fp64 on its fp32 split partials."""
import math
import os

import numpy as np
import pytest
import torch

import gen_inputs as G
import oracle
from util import bits_to_torch, rel_fro, torch_to_bits

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
H, HQ, PAGE, D = 8, 32, 16, 128


def _kx():
    from statetree_b200.ops import kv_ext
    return kv_ext()


def _fresh(nb, h=H, P=1 << 15):
    return (torch.zeros(nb, h, 2, 2, 1600, dtype=torch.uint8, device=DEV),
            torch.zeros(P, 16, dtype=torch.int32, device=DEV), torch.zeros(2, dtype=torch.int32, device=DEV))


def test_page_size():
    assert _kx().page_bytes(1) == 6400 and _kx().version() == 2


@pytest.mark.parametrize("name", ["tiny", "chan"])
def test_records_match_reference_bytes(name):
    g = np.load(os.path.join(GOLD, "kv_records.npz"))
    K, V = g[f"{name}_K"], g[f"{name}_V"]
    n, h, _ = K.shape
    cache, pool, cnt = _fresh(n // 16, h, 1024)
    slots = torch.arange(n, device=DEV)
    Kt, Vt = bits_to_torch(K, DEV), bits_to_torch(V, DEV)
    for a, b in ((0, 21), (21, n)):                                        # a call boundary inside a page
        _kx().append(Kt[a:b], Vt[a:b], slots[a:b], cache, pool, cnt)
    got = cache.cpu().numpy()
    i = 0
    for kvi in range(2):
        for p in range(n // 16):
            for hh in range(h):
                for half in range(2):
                    rec = got[p, hh, kvi, half]
                    assert np.array_equal(rec[:1552], g[f"{name}_records"][i])
                    c = int(g[f"{name}_counts"][i])
                    head = int(rec[1552:1556].view(np.uint32)[0])
                    assert (head & 15) == min(c, 11) and bool(head & 16) == (c > 11)
                    assert np.array_equal(rec[1556:1600].view(np.uint32)[:min(c, 11)], g[f"{name}_slots"][i][:min(c, 11)])
                    i += 1


def _write(cache, pool, cnt, lens, pre, maxp, seed, tiny, reuse=True, o_state=None):
    """chunked prefill (pages split across calls) then batched decode steps with a padding slot -1; the same calls go
    to the oracle's pages when o_state = (kv, pool, cnt) numpy arrays is given"""
    rs = np.random.RandomState(seed)
    nb = cache.shape[0]
    bt = rs.permutation(nb)[:len(lens) * maxp].reshape(len(lens), maxp).astype(np.int32)
    data = [G.kv_tokens(L, H, seed=seed * 100 + i, tiny=tiny) for i, L in enumerate(lens)]

    def slots(s, pos):
        pos = np.asarray(pos)
        return (bt[s][pos // PAGE].astype(np.int64) * PAGE + pos % PAGE)

    def app(K, V, sl):
        _kx().append(bits_to_torch(K, DEV), bits_to_torch(V, DEV), torch.from_numpy(sl).to(DEV), cache, pool, cnt, reuse)
        if o_state is not None:
            oracle.kv_append(K, V, sl, *o_state, reuse=reuse)

    for s, p0 in enumerate(pre):
        c = min(p0, (p0 * 3) // 5 + 3)
        for a, b in ((0, c), (c, p0)):
            if b > a:
                app(data[s][0][a:b], data[s][1][a:b], slots(s, np.arange(a, b)))
    pos = list(pre)
    while any(p < L for p, L in zip(pos, lens)):
        ks, vs, sl = [], [], []
        for s, L in enumerate(lens):
            if pos[s] < L:
                ks.append(data[s][0][pos[s]:pos[s] + 1])
                vs.append(data[s][1][pos[s]:pos[s] + 1])
                sl.append(slots(s, [pos[s]]))
                pos[s] += 1
        ks.append(np.zeros((1, H, D), np.uint16))
        vs.append(np.zeros((1, H, D), np.uint16))
        sl.append(np.array([-1], np.int64))
        app(np.concatenate(ks), np.concatenate(vs), np.concatenate(sl))
    return bt, data


def _wrong(cache, pool, bt, data, lens):
    n = 0
    for s, L in enumerate(lens):
        npg = (L + PAGE - 1) // PAGE
        Kd = torch.empty(npg, PAGE, H, D, dtype=torch.bfloat16, device=DEV)
        Vd = torch.empty_like(Kd)
        _kx().dequant_blocks(cache, pool, torch.from_numpy(bt[s][:npg].copy()).to(DEV), Kd, Vd)
        n += int((torch_to_bits(Kd).reshape(-1, H, D)[:L] != data[s][0]).sum())
        n += int((torch_to_bits(Vd).reshape(-1, H, D)[:L] != data[s][1]).sum())
    return n


LENS, PRE, MAXP = [600, 333, 17, 513], [400, 333, 5, 500], 40
NB = len(LENS) * MAXP + 5


def test_pages_exact_with_recycling():
    cache, pool, cnt = _fresh(NB, H, 1 << 17)
    used = []
    for rnd, tiny in enumerate((0.05, 0.12, 0.02, 0.12)):                  # 5-13 % escapes: chains needed
        bt, data = _write(cache, pool, cnt, LENS, PRE, MAXP, rnd, tiny)
        assert _wrong(cache, pool, bt, data, LENS) == 0
        assert int(cnt[1]) == 0
        used.append(int(cnt[0]))
    assert used[0] > 0
    assert used[-1] < 1.6 * used[1], used                                 # chains are recycled, no leak


def test_pages_equal_the_oracle_bytes():
    lens, pre, maxp = [70, 33, 17], [40, 33, 5], 6
    nb = len(lens) * maxp + 2
    cache, pool, cnt = _fresh(nb, H, 4096)
    o = (np.zeros((nb, H, 2, 2, 1600), np.uint8), np.zeros((4096, 16), np.uint32), np.zeros(2, np.int32))
    bt, data = _write(cache, pool, cnt, lens, pre, maxp, 7, 0.01, reuse=False, o_state=o)
    got = cache.cpu().numpy()
    # units without extension chains are byte-identical (chain block numbers depend on allocation order)
    heads = got[..., 1552:1556].copy().view(np.uint32)[..., 0]
    plain = (heads & 16) == 0
    assert plain.mean() > 0.5
    assert np.array_equal(got[plain], o[0][plain])
    assert np.array_equal(got[..., :1552], o[0][..., :1552])
    Kd, Vd = oracle.kv_dequant_blocks(o[0], o[1])
    Kg = torch.empty(nb, PAGE, H, D, dtype=torch.bfloat16, device=DEV)
    Vg = torch.empty_like(Kg)
    _kx().dequant(cache, pool, Kg, Vg)
    assert np.array_equal(torch_to_bits(Kg), Kd) and np.array_equal(torch_to_bits(Vg), Vd)


def test_long_append_call_matches_oracle():
    """one call with thousands of tokens (the grouped mapping of long calls): three sequences back to back, a padding
    token between them, ragged starts inside pages"""
    nb, P = 200, 1 << 16
    cache, pool, cnt = _fresh(nb, H, P)
    o = (np.zeros((nb, H, 2, 2, 1600), np.uint8), np.zeros((P, 16), np.uint32), np.zeros(2, np.int32))
    rs = np.random.RandomState(3)
    perm = rs.permutation(nb)
    lens = [1203, 517, 899]
    Ks, Vs, sl, used = [], [], [], 0
    # a short first call leaves sequence 0 mid-page, so the long call starts inside a page
    K0, V0 = G.kv_tokens(5, H, seed=90, tiny=0.05)
    s0 = (perm[0] * 16 + np.arange(5)).astype(np.int64)
    _kx().append(bits_to_torch(K0, DEV), bits_to_torch(V0, DEV), torch.from_numpy(s0).to(DEV), cache, pool, cnt)
    oracle.kv_append(K0, V0, s0, *o)
    for i, L in enumerate(lens):
        K, V = G.kv_tokens(L, H, seed=91 + i, tiny=0.05)
        pos = np.arange(L) + (5 if i == 0 else 0)
        pages = perm[used:used + (pos[-1] // 16 + 1)]
        used += len(pages)
        Ks += [K, np.zeros((1, H, D), np.uint16)]
        Vs += [V, np.zeros((1, H, D), np.uint16)]
        sl += [(pages[pos // 16] * 16 + pos % 16).astype(np.int64), np.array([-1], np.int64)]
    K, V, slots = np.concatenate(Ks), np.concatenate(Vs), np.concatenate(sl)
    assert K.shape[0] >= 1024
    _kx().append(bits_to_torch(K, DEV), bits_to_torch(V, DEV), torch.from_numpy(slots).to(DEV), cache, pool, cnt)
    oracle.kv_append(K, V, slots, *o)
    got = cache.cpu().numpy()
    assert np.array_equal(got[..., :1552], o[0][..., :1552])
    Kd, Vd = oracle.kv_dequant_blocks(o[0], o[1])
    Kg = torch.empty(nb, PAGE, H, D, dtype=torch.bfloat16, device=DEV)
    Vg = torch.empty_like(Kg)
    _kx().dequant(cache, pool, Kg, Vg)
    assert np.array_equal(torch_to_bits(Kg), Kd) and np.array_equal(torch_to_bits(Vg), Vd)
    assert int(cnt[1]) == 0


def test_dequant_blocks_out_of_range_is_zero():
    cache, pool, cnt = _fresh(NB)
    _write(cache, pool, cnt, LENS, PRE, MAXP, 1, 0.01)
    blocks = torch.tensor([-1, NB, 5], dtype=torch.int32, device=DEV)
    Kd = torch.full((3, PAGE, H, D), 7.0, dtype=torch.bfloat16, device=DEV)
    Vd = torch.full_like(Kd, 7.0)
    _kx().dequant_blocks(cache, pool, blocks, Kd, Vd)
    assert int((Kd[:2] != 0).sum()) == 0 and int((Vd[:2] != 0).sum()) == 0
    K5, V5 = torch.empty_like(Kd[:1]), torch.empty_like(Vd[:1])
    _kx().dequant_blocks(cache, pool, blocks[2:].contiguous(), K5, V5)
    assert torch.equal(Kd[2:], K5) and torch.equal(Vd[2:], V5)


def test_pool_exhaustion_is_flagged():
    cache, pool, cnt = _fresh(2, H, 1)
    K, V = G.kv_tokens(32, H, seed=5, tiny=0.6)
    _kx().append(bits_to_torch(K, DEV), bits_to_torch(V, DEV), torch.arange(32, device=DEV), cache, pool, cnt)
    assert int(cnt[1]) == 1


def _merge64(wo, wml, B, S):
    wo = wo.cpu().numpy().astype(np.float64).reshape(B, HQ, S, D)
    ml = wml.cpu().numpy().astype(np.float64).reshape(B, HQ, S, 2)
    m, l = ml[..., 0], ml[..., 1]
    M = m.max(-1, keepdims=True)
    f = np.where(np.isfinite(m), np.exp2(m - np.where(np.isfinite(M), M, 0.0)), 0.0)
    L = (f * l).sum(-1)
    O = (f[..., None] * wo).sum(-2)
    return np.where(L[..., None] > 0, O / np.where(L[..., None] > 0, L[..., None], 1.0), 0.0)


@pytest.mark.parametrize("tiny,left_pad", [(0.02, False), (0.0, True)])
def test_decode_attention_matches_fp64(tiny, left_pad):
    cache, pool, cnt = _fresh(NB)
    o = (np.zeros((NB, H, 2, 2, 1600), np.uint8), np.zeros((1 << 15, 16), np.uint32), np.zeros(2, np.int32))
    bt, data = _write(cache, pool, cnt, LENS, PRE, MAXP, 2, tiny, reuse=False, o_state=o)
    lens_l = LENS + [0]                                                    # an empty sequence
    B = len(lens_l)
    bt = np.concatenate([bt, bt[:1]])
    starts = np.array([37, 0, 3, 500, 0], np.int32) if left_pad else None
    q = G.to_bf16_bits(np.random.RandomState(9).standard_normal((B, HQ, D)))
    scale = 1.0 / math.sqrt(D)
    ref = oracle.kv_attn_f64(q, o[0], o[1], bt, np.array(lens_l, np.int32), scale, starts)
    qt, btt = bits_to_torch(q, DEV), torch.from_numpy(bt).to(DEV)
    lens = torch.tensor(lens_l, dtype=torch.int32, device=DEV)
    st_t = None if starts is None else torch.from_numpy(starts).to(DEV)
    for S, minpps in ((1, 1), (2, 1), (8, 4), (32, 4)):
        out = torch.full((B, HQ, D), 7.0, dtype=torch.bfloat16, device=DEV)
        wo = torch.zeros(B * HQ * S * D, dtype=torch.float32, device=DEV)
        wml = torch.zeros(B * HQ * S * 2, dtype=torch.float32, device=DEV)
        _kx().attn(qt, cache, pool, btt, lens, out, wo, wml, scale, S, st_t, minpps)
        got = out.float().cpu().numpy()
        assert np.abs(got[:-1] - ref[:-1]).max() / np.abs(ref[:-1]).max() < 1e-2, S   # the reference's own bar
        assert rel_fro(got[:-1], ref[:-1]) < 5e-3, (S, rel_fro(got[:-1], ref[:-1]))   # BF16 output rounding floor
        assert not got[-1].any()                                                      # length 0 -> zeros
        if S > 1:                                                                     # fp32 partials, merged in fp64
            e = rel_fro(_merge64(wo, wml, B, S)[:-1], ref[:-1])
            assert e < 1e-3, (S, e)
        out2 = torch.empty_like(out)
        _kx().attn(qt, cache, pool, btt, lens, out2, wo, wml, scale, S, st_t, minpps)
        assert torch.equal(out, out2)
    from statetree_b200 import ops
    assert ops.device_status() == 0


@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 4), (16, 2), (6, 2)])
def test_decode_attention_other_group_sizes(hq, hkv):
    """1, 2, 8 and 3 query heads per KV head (the kernel puts up to 8 heads on the N side of the tensor-core shape)"""
    from statetree_b200.kvcache import PageStore
    B, ctx = 3, 333
    npg = (ctx + 15) // 16
    gen = torch.Generator(device=DEV).manual_seed(hq * 10 + hkv)
    layer = PageStore(B * npg, hkv, DEV, pool_blocks=1 << 12)
    bt = torch.randperm(B * npg, device=DEV, generator=gen).view(B, npg).to(torch.int32)
    pos = torch.arange(ctx, device=DEV)
    Ks, Vs = [], []
    for b in range(B):
        K = torch.randn(ctx, hkv, D, device=DEV, generator=gen).to(torch.bfloat16)
        V = torch.randn(ctx, hkv, D, device=DEV, generator=gen).to(torch.bfloat16)
        layer.append(K, V, bt[b].long()[pos // 16] * 16 + pos % 16)
        Ks.append(K)
        Vs.append(V)
    q = torch.randn(B, hq, D, device=DEV, generator=gen).to(torch.bfloat16)
    lens = torch.tensor([ctx, ctx - 17, 5], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    for S in (1, 3):
        out = layer.attention(q, bt, lens, scale, splits=S, min_pages=2)
        for b in range(B):
            L = int(lens[b])
            k = Ks[b][:L].double().permute(1, 0, 2).repeat_interleave(hq // hkv, 0)
            v = Vs[b][:L].double().permute(1, 0, 2).repeat_interleave(hq // hkv, 0)
            p = torch.softmax(torch.einsum("hd,hld->hl", q[b].double(), k) * scale, -1)
            ref = torch.einsum("hl,hld->hd", p, v)
            assert float((out[b].double() - ref).norm() / ref.norm()) < 5e-3, (hq, hkv, S, b)
    from statetree_b200 import ops
    assert ops.device_status() == 0


def test_cache_object_decode_steps():
    """PagedKVCache: prefill + decode steps through update() / attention() against dense fp64 attention"""
    from statetree_b200.kvcache import PagedKVCache
    B, T0, steps = 3, 37, 5
    cache = PagedKVCache(1, B, 64, H, DEV, pool_blocks=4096)
    rs = np.random.RandomState(0)
    Kall = G.to_bf16_bits(rs.standard_normal((B, H, T0 + steps, D)))
    Vall = G.to_bf16_bits(rs.standard_normal((B, H, T0 + steps, D)))
    Kt, Vt = bits_to_torch(Kall, DEV), bits_to_torch(Vall, DEV)
    cache.update(0, Kt[:, :, :T0], Vt[:, :, :T0])
    for s in range(steps):
        t = T0 + s
        cache.update(0, Kt[:, :, t:t + 1], Vt[:, :, t:t + 1])
        q = torch.randn(B, HQ, D, device=DEV, generator=torch.Generator(DEV).manual_seed(s)).to(torch.bfloat16)
        out = cache.attention(0, q, 1.0 / math.sqrt(D))
        k = Kt[:, :, :t + 1].double().repeat_interleave(HQ // H, dim=1)
        v = Vt[:, :, :t + 1].double().repeat_interleave(HQ // H, dim=1)
        p = torch.softmax(torch.einsum("bhd,bhld->bhl", q.double(), k) / math.sqrt(D), -1)
        ref = torch.einsum("bhl,bhld->bhd", p, v)
        assert float((out.double() - ref).norm() / ref.norm()) < 5e-3
    cache.check()


@pytest.mark.gpu
def test_fused_rope_append_matches_rope_then_append():
    """q/k norm + rotary embedding + append in one launch leaves the same q and the same page bytes as the two kernels
    it replaces (several steps, so rows other than 0 and the page change at row 16 are covered)"""
    from statetree_b200.kvcache import PageStore
    from statetree_b200.ops import ext, kv_ext
    dev = torch.device("cuda")
    B, hq, hkv, D, max_pos = 3, 8, 2, 128, 64
    gen = torch.Generator(device=dev).manual_seed(11)
    wq = (1 + 0.1 * torch.randn(D, device=dev, generator=gen)).to(torch.bfloat16)
    wk = (1 + 0.1 * torch.randn(D, device=dev, generator=gen)).to(torch.bfloat16)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    ang = torch.arange(max_pos, device=dev, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    la, lb = PageStore(8, hkv, dev, pool_blocks=256), PageStore(8, hkv, dev, pool_blocks=256)
    bt = torch.tensor([[0, 3], [1, 4], [2, 5]], device=dev)
    pos = torch.zeros(1, dtype=torch.long, device=dev)
    for step in range(20):
        y = torch.randn(B, (hq + 2 * hkv) * D, device=dev, generator=gen)
        y[:, (hq + 1) * D + 5] *= 1e5                                # a channel that escapes
        y = y.to(torch.bfloat16)
        slots = bt[:, step // 16] * 16 + step % 16
        pos.fill_(step)
        qa, ka = torch.empty(B, hq, D, dtype=torch.bfloat16, device=dev), torch.empty(B, hkv, D, dtype=torch.bfloat16, device=dev)
        ext().qk_norm_rope(y, wq, wk, cos, sin, pos, qa, ka, 1e-6)
        la.append(ka, y[:, (hq + hkv) * D:].view(B, hkv, D), slots)
        qb = torch.empty_like(qa)
        kv_ext().rope_append(y, wq, wk, cos, sin, pos, qb, hq, hkv, 1e-6, slots, lb.pages, lb.pool, lb.pcnt)
        assert torch.equal(qa, qb), step
        # record bytes (leaves, states, nodes) and the in-record slot count are the same; a unit's header also names its
        # first pool block, and which block a warp draws from the pool depends on the order the warps get there
        assert torch.equal(la.pages[..., :1552], lb.pages[..., :1552]), step
        assert torch.equal(la.pages[..., 1552] & 31, lb.pages[..., 1552] & 31), step
        assert torch.equal(la.pages[..., 1556:], lb.pages[..., 1556:]), step      # the 11 in-record slots
    assert torch.equal(la.pcnt, lb.pcnt) and int(la.pcnt[0]) > 0     # the escaping channel reached the pool
    Ka, Va = la.dense()
    Kb, Vb = lb.dense()
    assert torch.equal(Ka, Kb) and torch.equal(Va, Vb)               # every stored value, escapes included


def test_vllm_page_backend_data_path():
    """PageBackend (the data path of the vLLM backend): writes at a slot mapping into a vLLM-shaped layer cache, decode
    attention against fp64, exact decode of cached pages, and blocks recycled by later requests do not leak pool blocks"""
    from statetree_b200.vllm_kv import PageBackend, SharedPool, decode_splits, prefill_page_tables
    nb, ctx, B = 64, 150, 3
    sh = SharedPool(DEV, HQ, H, pool_mb=2)
    be = PageBackend(HQ, H, 1.0 / math.sqrt(D), sh)
    cache = torch.zeros(nb, H, 16, 400, dtype=torch.uint8, device=DEV)        # vLLM's layout: 400 B per token per head
    rs = np.random.RandomState(4)
    used = []
    for rnd in range(3):                                                       # three rounds of requests over the same blocks
        bt = torch.from_numpy(rs.permutation(B * 10).reshape(B, 10).astype(np.int32)).to(DEV)   # the same 30 blocks, reshuffled
        Ks, Vs = [], []
        for b in range(B):
            Kb, Vb = G.kv_tokens(ctx, H, seed=rnd * 10 + b, tiny=0.08)
            K, V = bits_to_torch(Kb, DEV), bits_to_torch(Vb, DEV)
            pos = torch.arange(ctx, device=DEV)
            be.write(K.view(ctx, H * D), V.view(ctx, H * D), cache, bt[b].long()[pos // 16] * 16 + pos % 16)
            Ks.append(K)
            Vs.append(V)
        assert sh.poll() is None or True
        used.append(sh.usage()[0])
        q = torch.randn(B, HQ * D, device=DEV, generator=torch.Generator(DEV).manual_seed(rnd)).to(torch.bfloat16)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
        out = torch.empty(B, HQ * D, dtype=torch.bfloat16, device=DEV)
        be.decode(q, cache, bt, lens, out, splits=decode_splits(B, H))
        for b in range(B):
            k = Ks[b].double().permute(1, 0, 2).repeat_interleave(HQ // H, 0)
            v = Vs[b].double().permute(1, 0, 2).repeat_interleave(HQ // H, 0)
            p = torch.softmax(torch.einsum("hd,hld->hl", q[b].view(HQ, D).double(), k) / math.sqrt(D), -1)
            ref = torch.einsum("hl,hld->hd", p, v)
            assert float((out[b].view(HQ, D).double() - ref).norm() / ref.norm()) < 5e-3, (rnd, b)
        blocks, table = prefill_page_tables(torch.tensor([ctx] * B), bt)
        Kd, Vd = be.cached_pages(cache, blocks)
        for b in range(B):
            got = Kd[table[b].long()[:10]].reshape(-1, H, D)[:ctx]
            assert torch.equal(got.view(torch.int16), Ks[b].view(torch.int16)), (rnd, b)
    assert used[0] > 0 and used[-1] < 1.7 * used[0], used                      # recycled chains, no leak
    assert sh.usage()[2] is False
