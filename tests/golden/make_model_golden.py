"""Generates tests/golden/model_checkpoint.json by running the REFERENCE's convert + save_pretrained on tiny seeded
Hugging Face models (CPU): the safetensors key names, the statetree.json structure and a SHA-256 of every stored tensor.
The test (tests/test_model_io.py) rebuilds the same models, converts and saves them with this package and compares.

    python tests/golden/make_model_golden.py /path/to/reference-checkout
"""
import hashlib
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def tiny_model(tied):
    """a two-layer Qwen3-architecture model with BF16 weights from a fixed seed (shapes fit the format: out % 16, in % 64)"""
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, max_position_embeddings=64, tie_word_embeddings=tied)
    torch.manual_seed(1234 + int(tied))
    model = Qwen3ForCausalLM(cfg).to(torch.bfloat16)
    with torch.no_grad():
        model.model.layers[0].mlp.down_proj.weight[3, 5] = 0.0          # a value the tree cannot hold: an escape
        model.model.layers[1].self_attn.o_proj.weight[7, 70:80] = 1e-12
    return model.eval()


def tiny_moe_model():
    """a two-layer Qwen3-MoE-architecture model (4 experts held as 3-D parameters, top-2) with BF16 weights from a seed"""
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
    cfg = Qwen3MoeConfig(vocab_size=256, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                         max_position_embeddings=64, num_experts=4, num_experts_per_tok=2, decoder_sparse_step=1,
                         mlp_only_layers=[], tie_word_embeddings=False)
    torch.manual_seed(4321)
    model = Qwen3MoeForCausalLM(cfg).to(torch.bfloat16)
    with torch.no_grad():
        model.model.layers[0].mlp.experts.down_proj[2, 3, 5] = 0.0      # an escape inside an expert
    return model.eval()


def digest(path):
    from safetensors.torch import load_file
    sd = load_file(os.path.join(path, "model.safetensors"))
    tensors = {k: [str(v.dtype), list(v.shape), hashlib.sha256(v.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()]
               for k, v in sorted(sd.items())}
    with open(os.path.join(path, "statetree.json")) as fh:
        info = json.load(fh)
    return {"tensors": tensors, "info": info}


def main():
    if len(sys.argv) != 2 or not os.path.isdir(os.path.join(sys.argv[1], "statetree")):
        sys.exit("usage: make_model_golden.py /path/to/reference-checkout")
    sys.path.insert(0, sys.argv[1])
    import statetree.model as R
    out = {}
    for tied in (False, True):
        model = R.convert(tiny_model(tied), verify=True, verbose=False)
        with tempfile.TemporaryDirectory() as d:
            R.save_pretrained(model, d)
            out["tied" if tied else "untied"] = digest(d)
    model = R.convert(tiny_moe_model(), verify=True, verbose=False)
    with tempfile.TemporaryDirectory() as d:
        R.save_pretrained(model, d)
        out["moe"] = digest(d)
    with open(os.path.join(HERE, "model_checkpoint.json"), "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)
    print("wrote", os.path.join(HERE, "model_checkpoint.json"))


if __name__ == "__main__":
    main()
