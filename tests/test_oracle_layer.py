"""Pins oracle/decoder_layer.py (the one-layer decoder restatement used by the config-width GPU tests) against the
reference's own one-layer `LlamaForCausalLMCompress` / `Qwen2ForCausalLMCompress` run on the host (oracle/_ref),
with LRD + fake-quantized weights as `manager.apply` leaves them and a dense cache."""
import pytest
import torch

from oracle import decoder_layer as odl


def weights_of(model, dtype=torch.float32):
    sd = {k: v.float() for k, v in model.state_dict().items()}
    g = lambda p: (sd[p + ".weight"], sd.get(p + ".linear_V.weight"), sd.get(p + ".bias"))
    L = "model.layers.0."
    W = {n: g(L + p) for n, p in (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                                  ("o", "self_attn.o_proj"), ("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"),
                                  ("down", "mlp.down_proj"))}
    W.update(embed=sd["model.embed_tokens.weight"], ln1=sd[L + "input_layernorm.weight"],
             ln2=sd[L + "post_attention_layernorm.weight"], norm=sd["model.norm.weight"], lm_head=g("lm_head"))
    return W


@pytest.mark.parametrize("family", ["llama", "qwen2"])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1e-2)])
def test_one_layer_oracle_matches_reference_model(reference, family, dtype, tol):
    T = reference
    torch.manual_seed(41)
    kw = dict(vocab_size=300, hidden_size=128, intermediate_size=320, num_hidden_layers=1, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=64, tie_word_embeddings=False)
    if family == "llama":
        model = T.LlamaForCausalLMCompress(T.LlamaConfigCompress(**kw)); mgr = T.LlamaCompressionSchemesManager(model)
    else:
        model = T.Qwen2ForCausalLMCompress(T.Qwen2ConfigCompress(**kw)); mgr = T.Qwen2CompressionSchemesManager(model)
    model = model.to(dtype).eval()
    mgr.set("lrd", "rank", 24, criteria=["mlp"])
    mgr.set("quantization", "precision", 4, criteria=["self_attn", "mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    mgr.apply(hard=False)
    g = torch.Generator().manual_seed(42)
    ids = torch.randint(0, 300, (3, 11), generator=g)
    nxt = torch.randint(0, 300, (3,), generator=g)
    with torch.no_grad():
        ref0 = model(input_ids=ids).logits[:, -1].float()
        ref1 = model(input_ids=torch.cat([ids, nxt[:, None]], dim=1)).logits[:, -1].float()
    cfg = model.config
    theta = getattr(cfg, "rope_theta", None) or cfg.rope_parameters["rope_theta"]
    l0, l1 = odl.one_layer_logits(weights_of(model), ids, nxt, 4, 2, 32, float(theta), float(cfg.rms_norm_eps), None, act=dtype)
    for a, b in ((l0, ref0), (l1, ref1)):
        assert ((a - b).abs().max() / b.abs().max()).item() < tol
