"""The transformers glue of the compressed KV cache (StateTreeKVCache + the 'statetree' attention implementation) on a
tiny Qwen3-architecture model: prefill + decode steps with left padding must reproduce a cache-free forward pass over
the whole sequence (the check of the reference's tests/test_kv_cache.py for its Hugging Face path)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def test_generate_steps_match_full_forward():
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from statetree_b200.kvcache import StateTreeKVCache, enable
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = Qwen3ForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    B, P, steps = 2, 21, 6
    ids = torch.randint(0, cfg.vocab_size, (B, P + steps), device="cuda")
    mask = torch.ones(B, P + steps, dtype=torch.long, device="cuda")
    mask[1, :5] = 0                                                    # left padding on the second sequence
    with torch.no_grad():
        full = model(input_ids=ids, attention_mask=mask).logits.float()          # no cache: the reference
        enable(model)
        cache = StateTreeKVCache(model.config, batch_size=B, max_cache_len=P + steps + 8)
        out = model(input_ids=ids[:, :P], attention_mask=mask[:, :P], past_key_values=cache, use_cache=True)
        got = [out.logits[:, -1].float()]
        for t in range(steps - 1):
            out = model(input_ids=ids[:, P + t:P + t + 1], attention_mask=mask[:, :P + t + 1], past_key_values=cache,
                        use_cache=True)
            got.append(out.logits[:, -1].float())
    cache.check()
    assert cache.storage_bytes() > 0 and int(cache.layers[0].get_seq_length()) == P + steps - 1
    for t, g in enumerate(got):
        want = full[:, P - 1 + t]
        rel = float((g - want).norm() / want.norm())
        assert rel < 3e-2, (t, rel)                                    # BF16 model: roundings fall differently
        assert bool((g.argmax(-1) == want.argmax(-1)).all()) or rel < 1e-2
    # the pages hold exactly what the model produced: stored keys of layer 0 decode to BF16 values without loss
    k0, v0 = cache.layers[0].dense(P)
    assert k0.shape == (B, 2, P, 128) and torch.isfinite(k0.float()).all()
