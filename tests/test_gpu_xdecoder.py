"""The minimal Qwen3-architecture decoder on a tiny random model: the compressed model (tree-stored weights, compressed
KV pages, fused glue kernels, CUDA-graph replay) must follow the BF16 control built from the same seeds."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tiny_decoder_follows_bf16_control():
    from statetree_b200 import ops
    from statetree_b200.decoder import DecoderConfig, TreeDecoder
    cfg = DecoderConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, inter=1024, vocab=2048)
    B, P, Gn = 3, 40, 8
    prompt = torch.randint(0, cfg.vocab, (B, P), generator=torch.Generator().manual_seed(0)).cuda()
    preds, logits = {}, {}
    for name, compressed in (("tree", True), ("bf16", False)):
        m = TreeDecoder(cfg, "cuda", B, P + Gn + 8, compressed=compressed, seed=3)
        m.capture()
        got = []
        first = m.run(prompt, Gn, collect=got).cpu()
        preds[name] = torch.stack(got, 1).cpu()                 # teacher-forced predictions after every prompt token
        logits[name] = []
        m.reset()
        for t in range(P):                                      # same tokens again: logits of every step
            m.tokens.copy_(prompt[:, t])
            m.graph.replay()
            logits[name].append(m.logits.float().cpu().clone())
        if compressed:
            m.cache.check()
            m.reset()
            assert torch.equal(m.run(prompt, Gn).cpu(), first)   # bit-identical from run to run
        del m
    a, b = torch.stack(logits["tree"]), torch.stack(logits["bf16"])
    rel = float((a - b).norm() / b.norm())
    assert rel < 2e-2, rel                                       # same function up to BF16 rounding of intermediate sums
    agree = (preds["tree"] == preds["bf16"]).float().mean().item()
    assert agree > 0.85, agree                                   # near-ties of a flat random model may flip
    assert ops.device_status() == 0


def test_glue_kernels_match_torch():
    from statetree_b200.ops import ext
    E = ext()
    g = torch.Generator("cuda").manual_seed(0)
    x = torch.randn(5, 512, device="cuda", generator=g).to(torch.bfloat16)
    d = torch.randn(5, 512, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(512, device="cuda", generator=g)).to(torch.bfloat16)
    out = torch.empty_like(x)
    x2 = x.clone()
    E.add_rmsnorm(x2, d, w, out, 1e-6)
    xs = (x.float() + d.float()).to(torch.bfloat16)
    assert torch.equal(x2, xs)
    ref = (xs.float() * torch.rsqrt(xs.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16).float() * w.float()
    assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item()
    hq, hkv, B = 4, 2, 3
    qkv = torch.randn(B, (hq + 2 * hkv) * 128, device="cuda", generator=g).to(torch.bfloat16)
    wq = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    ang = torch.arange(16, device="cuda", dtype=torch.float32)[:, None] * (1.0 / (1e6 ** (torch.arange(0, 128, 2, device="cuda") / 128.0)))[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([7], device="cuda")
    q = torch.empty(B, hq, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.empty(B, hkv, 128, dtype=torch.bfloat16, device="cuda")
    E.qk_norm_rope(qkv, wq, wq, cos, sin, pos, q, k, 1e-6)
    heads = qkv[:, :(hq + hkv) * 128].view(B, hq + hkv, 128).float()
    n = (heads * torch.rsqrt(heads.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16).float()
    x1, x2_ = n[..., 0::2], n[..., 1::2]
    ref = torch.stack([x1 * cos[7] - x2_ * sin[7], x1 * sin[7] + x2_ * cos[7]], -1).flatten(-2)
    got = torch.cat([q, k], 1).float()
    assert (got - ref).abs().max().item() < 0.03
