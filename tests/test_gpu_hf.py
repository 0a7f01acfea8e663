"""Hugging Face generate() with the paged cache and the registered attention function: the
drop-in for the reference's HF path (its model classes inherit generate() from transformers).
Tiny random-init Qwen2 / Llama models (the shapes of the reference's own test factory,
test/_helpers/model_factory.py:50-67, with head_dim 64)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny(kind, dtype):
    import transformers
    common = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                  num_key_value_heads=1, max_position_embeddings=256, rope_theta=10000.0, tie_word_embeddings=False)
    torch.manual_seed(3)
    if kind == "qwen2":
        m = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**common))
    else:
        m = transformers.LlamaForCausalLM(transformers.LlamaConfig(**common))
    return m.to(dtype).cuda().eval()


def run_generate(model, ids, new, cache=None):
    return model.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=new, min_new_tokens=new, do_sample=False,
                          pad_token_id=0, eos_token_id=None, past_key_values=cache, return_dict_in_generate=True,
                          output_logits=True)


@pytest.mark.parametrize("kind", ["qwen2", "llama"])
def test_generate_fp32_pages_same_tokens(cuda, kind):
    """Unquantized fp32 pages: greedy tokens identical to the stock cache for 32 steps, logits
    within fp32 summation-order noise."""
    from transformer_surgeon_b200 import hf_cache
    model = tiny(kind, torch.float32)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (3, 19), generator=g).cuda()
    ref = run_generate(model, ids, 32)
    model.config._attn_implementation = hf_cache.ATTN_NAME
    cache = hf_cache.PagedQuantCache(model.config, batch=3, max_len=64, kv_format="fp32")
    out = run_generate(model, ids, 32, cache)
    assert torch.equal(out.sequences, ref.sequences)
    for a, b in zip(out.logits, ref.logits):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-4)
    assert cache.get_seq_length() == 19 + 31          # the last sampled token is never fed back


@pytest.mark.parametrize("fmt", ["int8", "fp8", "nvfp4"])
def test_generate_quantized_pages_close(cuda, fmt):
    """Quantized pages: every step's logits stay close to the dense-cache run when both are driven
    with the same tokens (teacher forcing removes the divergence a flipped argmax would cause)."""
    from transformer_surgeon_b200 import hf_cache
    model = tiny("llama", torch.float32)
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, 512, (2, 40), generator=g).cuda()
    with torch.no_grad():
        ref = model(ids).logits                                   # dense causal attention over all 40 tokens
        model.config._attn_implementation = hf_cache.ATTN_NAME
        cache = hf_cache.PagedQuantCache(model.config, batch=2, max_len=48, kv_format=fmt)
        out = [model(ids[:, :24], past_key_values=cache).logits]   # prefill reads dequantized pages
        for t in range(24, 40):                                    # decode steps on the paged kernel
            out.append(model(ids[:, t:t + 1], past_key_values=cache).logits)
    out = torch.cat(out, dim=1)
    err = (out - ref).abs().max().item() / ref.abs().max().item()
    assert err < {"int8": 2e-2, "fp8": 8e-2, "nvfp4": 2.5e-1}[fmt], err
    assert cache.get_seq_length() == 40


def test_cache_requires_registered_attention(cuda):
    from transformer_surgeon_b200 import hf_cache
    model = tiny("llama", torch.float32)
    with pytest.raises(ValueError):
        hf_cache.PagedQuantCache(model.config, batch=1, max_len=32)
