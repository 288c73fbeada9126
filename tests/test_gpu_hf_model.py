"""The user path of the reference on a GPU: convert a Hugging Face model in place (linear layers, fused groups,
embeddings, 3-D experts), run it, save it, load it back.  The converted model computes with bit-identical weights, so
its logits differ from the BF16 model's only by summation order and BF16 rounding points; the loaded model must
reproduce the converted one (exactly for a single token, where attention has nothing to reorder)."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")
pytest.importorskip("safetensors")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))


def _logits(model, ids):
    with torch.no_grad():
        return model(input_ids=ids).logits.float()


@pytest.mark.parametrize("kind", ["dense_tied", "dense", "moe"])
def test_converted_model_runs_saves_and_loads(kind, tmp_path):
    import copy
    from make_model_golden import tiny_model, tiny_moe_model
    from statetree_b200 import model as M
    from statetree_b200 import ops
    from statetree_b200.experts import TreeExperts
    from statetree_b200.linear import TreeLinear
    src = (tiny_moe_model() if kind == "moe" else tiny_model(kind == "dense_tied")).cuda()
    ref = copy.deepcopy(src)
    gen = torch.Generator(device="cuda").manual_seed(11)
    short = torch.randint(0, 256, (1, 1), device="cuda", generator=gen)        # one token: the GEMV kernels
    longer = torch.randint(0, 256, (3, 40), device="cuda", generator=gen)      # 120 rows: the tcgen05 GEMM
    want = [_logits(ref, short), _logits(ref, longer)]
    model = M.convert(src, verify=True, verbose=False)
    assert any(isinstance(m, TreeLinear) for m in model.modules())
    if kind == "moe":
        assert isinstance(model.model.layers[0].mlp.experts, TreeExperts)
    M.prepare(model, batch_sizes=(1, 8))
    got = [_logits(model, short), _logits(model, longer)]
    for g, w in zip(got, want):
        rel = float((g - w).norm() / w.norm())
        assert rel < 3e-2, (kind, rel)
    if kind == "dense":
        # a prefill-size batch (640 rows > PREFILL_MIN): decode once + cuBLAS, the next layer decoded meanwhile, against
        # the same batch through the tcgen05 kernel
        import statetree_b200.linear as L
        layers = [m for _, m in M.tree_modules(model)]
        assert all(m._next is not None and isinstance(m._next(), TreeLinear) for m in layers)
        wide = torch.randint(0, 256, (16, 40), device="cuda", generator=gen)
        dense_way = _logits(model, wide)
        stage = L._state(torch.device("cuda", torch.cuda.current_device())).dense_stage()
        assert any(h is not None for h in stage.holds)
        keep, L.PREFILL_MIN = L.PREFILL_MIN, 0
        try:
            kernel_way = _logits(model, wide)
        finally:
            L.PREFILL_MIN = keep
        rel = float((dense_way - kernel_way).norm() / kernel_way.norm())
        assert rel < 1e-2, rel
        assert float((dense_way - _logits(ref, wide)).norm() / kernel_way.norm()) < 3e-2
    rep = M.size_report(model)
    assert rep["bits_per_weight"] < 12.7 and rep["total_bytes"] < sum(t.numel() * 2 for t in ref.parameters())
    M.save_pretrained(model, str(tmp_path))
    loaded = M.load_pretrained(str(tmp_path), device="cuda")
    again = [_logits(loaded, short), _logits(loaded, longer)]
    assert torch.equal(got[0], again[0]), kind                  # same trees, same kernels, same bits
    rel = float((got[1] - again[1]).norm() / got[1].norm())     # (the rebuilt model may pick another attention backend)
    assert rel < 1e-2, (kind, rel)
    assert ops.device_status() == 0
