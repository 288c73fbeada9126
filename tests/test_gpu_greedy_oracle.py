"""Greedy token streams of the compressed decoder against an fp64 oracle decoder that rounds to BF16 at the same points
(oracle/decoder.py), on a tiny random model.  Random weights give nearly flat logits, so the comparison follows the
reference's practice for such models (tests/test_vllm_moe.py:213-227): the GPU's tokens are fed to the oracle
(teacher forcing), the logits of every step must agree within a measured bound, and the GPU's token must be the
oracle's arg-max wherever the oracle's top-2 margin exceeds twice that bound."""
import numpy as np
import pytest
import torch

import oracle
from oracle.decoder import OracleDecoder

pytestmark = pytest.mark.gpu


def _dense(tl):
    """the exact BF16 values of a TreeLinear, decoded by the CPU oracle (not by the GPU kernel under test)"""
    bits = oracle.decode(tl.tree.cpu().numpy(), tl.esc_rows.cpu().numpy(), tl.esc_cols.cpu().numpy(), tl.esc_bits.cpu().numpy())
    return oracle.bf16_bits_to_f32(bits).astype(np.float64)


@pytest.mark.parametrize("batch", [1, 3])
def test_greedy_stream_follows_the_fp64_oracle(batch):
    from statetree_b200 import ops
    from statetree_b200.decoder import DecoderConfig, TreeDecoder
    cfg = DecoderConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, inter=1024, vocab=2048)
    P, Gn = 10, 14
    m = TreeDecoder(cfg, "cuda", batch, P + Gn + 8, compressed=True, seed=5)
    m.capture()
    layers = []
    D, hq, hkv = cfg.head_dim, cfg.heads, cfg.kv_heads
    for qkv, o, gu, d in m.blocks:
        Wqkv, Wgu = _dense(qkv), _dense(gu)
        if m.fused_act:                                   # gate / up stored as alternating 16-row tiles
            t = Wgu.reshape(-1, 2, 16, cfg.hidden)
            gate, up = t[:, 0].reshape(-1, cfg.hidden), t[:, 1].reshape(-1, cfg.hidden)
        else:
            gate, up = Wgu[:cfg.inter], Wgu[cfg.inter:]
        layers.append(dict(q=Wqkv[:hq * D], k=Wqkv[hq * D:(hq + hkv) * D], v=Wqkv[(hq + hkv) * D:], o=_dense(o),
                           gate=gate, up=up, down=_dense(d)))
    ref = OracleDecoder(dict(embed=_dense(m.embed), lm_head=_dense(m.lm_head), layers=layers), hq, hkv, cfg.eps,
                        m.cos.cpu().numpy(), m.sin.cpu().numpy())
    prompt = torch.randint(0, cfg.vocab, (batch, P), generator=torch.Generator().manual_seed(2)).cuda()
    gpu_logits, fed = [], []
    for t in range(P + Gn):
        tok = prompt[:, t] if t < P else m.next_tok.clone()
        m.tokens.copy_(tok)
        m.graph.replay()
        fed.append(tok.cpu().numpy())
        gpu_logits.append(m.logits.float().cpu().numpy().astype(np.float64))
    m.cache.check()
    worst, flips, checked, first_div = 0.0, 0, 0, None
    for t in range(P + Gn):
        want = ref.step(fed[t])
        got = gpu_logits[t]
        worst = max(worst, float(np.abs(got - want).max()))
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        assert rel < 2e-2, (t, rel)                       # same function; BF16 roundings may fall differently
    # second pass with the bound known
    ref2 = OracleDecoder(ref.w, hq, hkv, cfg.eps, ref.cos, ref.sin)
    for t in range(P + Gn):
        want = ref2.step(fed[t])
        top2 = np.sort(want, -1)[:, -2:]
        margin = top2[:, 1] - top2[:, 0]
        same = gpu_logits[t].argmax(-1) == want.argmax(-1)
        clear = margin > 2 * worst
        checked += int(clear.sum())
        assert bool(same[clear].all()), (t, margin, worst)       # a clear winner is never missed
        flips += int((~same).sum())
        if first_div is None and not same.all():
            first_div = (t, float(margin[~same].max()))
    assert checked > 0
    # where the streams part at all, the oracle itself had a near-tie there (margin within the error bound)
    assert first_div is None or first_div[1] <= 2 * worst, (first_div, worst)
    assert ops.device_status() == 0
