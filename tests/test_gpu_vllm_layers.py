"""The layer methods of the vLLM integration (statetree_b200/vllm_layers.py) on plain modules that carry what vLLM's
layers carry: after `process_weights_after_loading` the BF16 weights are gone and `apply` gives the BF16 layer's
result within rounding; what the format cannot (or should not) hold stays BF16."""
import pytest
import torch
import torch.nn.functional as Fn

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _Layer(torch.nn.Module):
    def __init__(self, **tensors):
        super().__init__()
        for k, v in tensors.items():
            setattr(self, k, torch.nn.Parameter(v, requires_grad=False))


def _bf16(*shape, seed=0, scale=0.05):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


def test_linear_method():
    from statetree_b200.linear import TreeLinear
    from statetree_b200.vllm_layers import StateTreeLinearMethod, install, min_params
    assert install()[0] is False and "0.32" in install()[1]
    W = _bf16(2048, 1024, seed=1)
    assert W.numel() >= min_params()
    layer, m = _Layer(weight=W.clone()), StateTreeLinearMethod("model.layers.0.mlp.down_proj", batches=(1, 8, 64))
    m.process_weights_after_loading(layer)
    assert isinstance(layer.statetree, TreeLinear) and layer.weight.numel() == 0
    assert "statetree.tree" in layer.state_dict()
    bias = _bf16(2048, seed=2)
    for B in (1, 7, 64, 200):
        x = _bf16(B, 1024, seed=10 + B, scale=1.0)
        want = Fn.linear(x, W, bias).float()
        got = m.apply(layer, x, bias).float()
        assert (got - want).abs().max().item() <= 0.02 * want.abs().max().item()
    small = _Layer(weight=_bf16(64, 128, seed=3))                       # below min_params: stays BF16
    m.process_weights_after_loading(small)
    assert small.statetree is None and small.weight.numel() == 64 * 128
    x = _bf16(3, 128, seed=4, scale=1.0)
    assert torch.equal(m.apply(small, x), Fn.linear(x, small.weight))
    odd = _Layer(weight=_bf16(2050, 1024, seed=5))                      # rows not a multiple of 16
    m.process_weights_after_loading(odd)
    assert odd.statetree is None


def test_embedding_method():
    from statetree_b200.vllm_layers import StateTreeEmbeddingMethod
    table = _bf16(512, 256, seed=6, scale=1.0)
    layer, m = _Layer(weight=table.clone()), StateTreeEmbeddingMethod("model.embed_tokens")
    m.process_weights_after_loading(layer)
    assert layer.statetree is not None and layer.weight.numel() == 0
    ids = torch.tensor([[0, 511, 17], [5, 5, 300]], device=DEV)
    assert torch.equal(m.embedding(layer, ids).view(torch.int16), table[ids].view(torch.int16))      # exact rows
    head, hm = _Layer(weight=table.clone()), StateTreeEmbeddingMethod("lm_head", lm_head=True, batches=(1, 4))
    hm.process_weights_after_loading(head)
    x = _bf16(4, 256, seed=7, scale=1.0)
    want = Fn.linear(x, table).float()
    assert (hm.apply(head, x).float() - want).abs().max().item() <= 0.02 * want.abs().max().item()


def test_moe_method():
    from statetree_b200.experts import TreeExperts
    from statetree_b200.vllm_layers import StateTreeMoEMethod
    E, H, I, K = 8, 256, 128, 2
    w13, w2 = _bf16(E, 2 * I, H, seed=8), _bf16(E, H, I, seed=9)
    layer, m = _Layer(w13_weight=w13.clone(), w2_weight=w2.clone()), StateTreeMoEMethod("model.layers.0.mlp.experts")
    m.process_weights_after_loading(layer)
    assert isinstance(layer.statetree, TreeExperts) and layer.w13_weight.numel() == 0 and layer.w2_weight.numel() == 0
    g = torch.Generator(device=DEV).manual_seed(12)
    for T in (1, 5, 90):
        x = _bf16(T, H, seed=20 + T, scale=1.0)
        ids = torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(T)])
        ids[0, 1] = -1                                                  # a pair of another rank's expert
        w = torch.rand(T, K, device=DEV, generator=g)
        got = m.apply(layer, x, w, ids).float()
        want = torch.zeros(T, H, device=DEV)
        for t in range(T):
            for j in range(K):
                e = int(ids[t, j])
                if e < 0:
                    continue
                h = Fn.linear(x[t], w13[e])
                a = Fn.silu(h[:I].float()).to(torch.bfloat16) * h[I:]
                want[t] += w[t, j] * Fn.linear(a, w2[e]).float()
        assert (got - want).abs().max().item() <= 0.03 * want.abs().max().item() + 1e-3, T
