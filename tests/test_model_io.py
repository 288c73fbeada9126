"""convert / save_pretrained / load_pretrained against the reference's on-disk format (CPU).

tests/golden/model_checkpoint.json was written by the reference's own convert + save_pretrained on two tiny seeded
models (make_model_golden.py): the checkpoint this package writes for the same models must have the same safetensors
keys, the same statetree.json and byte-identical tensors, and must load back into a model whose trees decode to the
original weights.  A version-2 file (older leaf format) is migrated on load."""
import json
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

transformers = pytest.importorskip("transformers")
pytest.importorskip("safetensors")


def _golden():
    with open(os.path.join(HERE, "golden", "model_checkpoint.json")) as fh:
        return json.load(fh)


@pytest.mark.parametrize("tied", [False, True])
def test_checkpoint_equals_the_reference_format(tied, tmp_path):
    from make_model_golden import digest, tiny_model
    from statetree_b200 import format as F
    from statetree_b200 import model as M
    from statetree_b200.linear import TreeEmbedding, TreeLinear, TreeSlice
    src = tiny_model(tied)
    original = {k: v.clone() for k, v in src.state_dict().items()}
    model = M.convert(src, verify=True, verbose=False)
    layer0 = model.model.layers[0]
    assert isinstance(layer0.self_attn.qkv_proj, TreeLinear) and isinstance(layer0.self_attn.q_proj, TreeSlice)
    assert isinstance(layer0.mlp.gate_up_proj, TreeLinear) and isinstance(layer0.mlp.down_proj, TreeLinear)
    assert isinstance(model.model.embed_tokens, TreeEmbedding) and isinstance(model.lm_head, TreeLinear)
    assert (model.model.embed_tokens.table is None) == tied                  # tied: the head's tree serves both
    rep = M.size_report(model)
    assert rep["tree_layers"] == (2 * 4 + 1 + (0 if tied else 1)) and 12.0 < rep["bits_per_weight"] < 12.6
    assert rep["escape_fraction"] > 0
    M.save_pretrained(model, str(tmp_path))
    got, want = digest(str(tmp_path)), _golden()["tied" if tied else "untied"]
    assert sorted(got["tensors"]) == sorted(want["tensors"])
    assert got["info"] == want["info"]
    for key in want["tensors"]:
        assert got["tensors"][key] == want["tensors"][key], key
    # and back: nothing on the meta device, every tree decodes to the weights the model started from
    loaded = M.load_pretrained(str(tmp_path), device="cpu")
    qkv = loaded.model.layers[1].self_attn.qkv_proj
    W = F.decode_reference(qkv.tree, qkv.esc_rows, qkv.esc_cols, qkv.esc_bits)
    want_w = torch.cat([original[f"model.layers.1.self_attn.{p}_proj.weight"] for p in "qkv"])
    assert torch.equal(W.view(torch.int16), want_w.view(torch.int16))
    head = loaded.lm_head
    Wh = F.decode_reference(head.tree, head.esc_rows, head.esc_cols, head.esc_bits)
    assert torch.equal(Wh.view(torch.int16), original["lm_head.weight"].view(torch.int16))
    emb = loaded.model.embed_tokens
    assert (emb.source is loaded.lm_head) if tied else (emb.table is not None)
    assert torch.equal(loaded.model.norm.weight, original["model.norm.weight"])
    assert isinstance(loaded.model.layers[0].mlp.up_proj, TreeSlice)
    assert loaded.model.layers[0].mlp.up_proj.fused is loaded.model.layers[0].mlp.gate_up_proj


def test_moe_checkpoint_equals_the_reference_format(tmp_path):
    """experts held as 3-D parameters become a TreeExperts whose state dict, statetree.json entry and tensor bytes are
    the reference's; the checkpoint loads back into empty TreeExperts skeletons"""
    from make_model_golden import digest, tiny_moe_model
    from statetree_b200 import format as F
    from statetree_b200 import model as M
    from statetree_b200.experts import TreeExperts, expert_layout
    src = tiny_moe_model()
    experts0 = src.model.layers[0].mlp.experts
    assert expert_layout(experts0) == ("gate_up_proj", False, False)
    original = {k: v.clone() for k, v in src.state_dict().items()}
    model = M.convert(src, verify=True, verbose=False)
    te = model.model.layers[0].mlp.experts
    assert isinstance(te, TreeExperts) and te.num_experts == 4 and te.up_name == "gate_up_proj"
    assert expert_layout(te) is None
    M.save_pretrained(model, str(tmp_path))
    got, want = digest(str(tmp_path)), _golden()["moe"]
    assert sorted(got["tensors"]) == sorted(want["tensors"])
    assert got["info"] == want["info"]
    for key in want["tensors"]:
        assert got["tensors"][key] == want["tensors"][key], key
    loaded = M.load_pretrained(str(tmp_path), device="cpu")
    le = loaded.model.layers[1].mlp.experts
    assert isinstance(le, TreeExperts)
    for e in range(4):
        up, down = le.gate_up_proj[e], le.down_proj[e]
        Wu = F.decode_reference(up.tree, up.esc_rows, up.esc_cols, up.esc_bits)
        Wd = F.decode_reference(down.tree, down.esc_rows, down.esc_cols, down.esc_bits)
        assert torch.equal(Wu.view(torch.int16), original["model.layers.1.mlp.experts.gate_up_proj"][e].view(torch.int16))
        assert torch.equal(Wd.view(torch.int16), original["model.layers.1.mlp.experts.down_proj"][e].view(torch.int16))
    assert M.convert(tiny_moe_model(), experts=False, verify=False, verbose=False).model.layers[0].mlp.experts.__class__ \
        is not TreeExperts


def test_version_2_checkpoint_is_migrated(tmp_path):
    from safetensors.torch import load_file, save_file
    from make_model_golden import tiny_model
    from statetree_b200 import format as F
    from statetree_b200 import model as M
    model = M.convert(tiny_model(False), verify=False, verbose=False)
    M.save_pretrained(model, str(tmp_path))
    sd = load_file(os.path.join(str(tmp_path), M.WEIGHTS_NAME))
    old = {k: (F.leaves_v2_to_v1(v) if k.endswith("tree") else v) for k, v in sd.items()}
    save_file(old, os.path.join(str(tmp_path), M.WEIGHTS_NAME), metadata={"format": "pt", "statetree": "2"})
    info_path = os.path.join(str(tmp_path), M.INFO_NAME)
    with open(info_path) as fh:
        info = json.load(fh)
    info["version"] = 2
    with open(info_path, "w") as fh:
        json.dump(info, fh)
    loaded = M.load_pretrained(str(tmp_path), device="cpu")
    assert torch.equal(loaded.lm_head.tree, model.lm_head.tree)


def test_convert_options_and_errors(tmp_path):
    from make_model_golden import tiny_model
    from statetree_b200 import model as M
    from statetree_b200.linear import TreeLinear, TreeSlice
    m = M.convert(tiny_model(False), fuse=None, exclude=("lm_head",), embeddings=False, verbose=False)
    assert isinstance(m.model.layers[0].self_attn.q_proj, TreeLinear)          # not fused: each layer its own tree
    assert isinstance(m.lm_head, torch.nn.Linear) and isinstance(m.model.embed_tokens, torch.nn.Embedding)
    m2 = M.convert(tiny_model(False), include=("*.mlp.*",), verbose=False)
    assert isinstance(m2.model.layers[0].mlp.gate_proj, TreeSlice)
    assert isinstance(m2.model.layers[0].self_attn.q_proj, torch.nn.Linear)
    m3 = M.convert(tiny_model(False), max_escape_fraction=0.0, embeddings=False, verbose=False)   # anything that escapes stays BF16
    assert isinstance(m3.model.layers[0].mlp.down_proj, torch.nn.Linear)
    with open(os.path.join(str(tmp_path), "statetree.json"), "w") as fh:
        json.dump({"format": "something else"}, fh)
    with pytest.raises(ValueError, match="not a statetree checkpoint"):
        M.load_pretrained(str(tmp_path), device="cpu")
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        m.model.layers[0].self_attn.q_proj(torch.zeros(1, 128, dtype=torch.bfloat16))     # no CPU path
