"""Generate the golden fixtures in this directory by running the REFERENCE itself.

Run where the reference checkout is importable:
    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py
The fixtures are small .npz files; bf16 tensors are stored as uint16 bit patterns under
a key ending in "__bf16".  Nothing in the test-suite needs the reference at run time.

Reference entry points exercised (paths inside the reference project):
  transformersurgeon/compression/quantization_methods/vanilla.py:40  quantize_vanilla
  transformersurgeon/compression/lrd_methods/svd.py:5                 low_rank_svd
  transformersurgeon/blocks/linear_compressed.py:81                    LinearCompressed.forward
  transformersurgeon/blocks/mha.py:9                                   attention
  transformersurgeon/blocks/rope.py:45,64,140                          RoPE tables / rotation
  transformersurgeon/blocks/norm.py:8                                  RMSNorm.forward
  transformersurgeon/blocks/mlp.py:171                                 MLPGated.forward
  transformersurgeon/models/{qwen2_c,llama_c}                          *ForCausalLMCompress + manager
"""
import os
import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def put(d, key, t):
    if isinstance(t, torch.Tensor):
        if t.dtype == torch.bfloat16:
            d[key + "__bf16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
        else:
            d[key] = t.detach().contiguous().numpy()
    else:
        d[key] = np.asarray(t)


def gen_weight_quant():
    from transformersurgeon.compression.quantization_methods.vanilla import quantize_vanilla
    out = {}
    g = torch.Generator().manual_seed(11)
    for dt, name in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
        w = (torch.randn(96, 200, generator=g) * 0.02).to(dt)
        w[3] = 0          # an all-zero (pruned) row -> scale 0, codes 0
        w[5, 7] = 0
        put(out, f"w_{name}", w)
        for p in (8, 4, 2, "binary"):
            for gran in ("per_channel", "per_tensor"):
                q, s, deq = quantize_vanilla(w, p, 1e-6, gran)
                tag = f"{name}_{p}_{gran}"
                put(out, f"q_{tag}", q)
                put(out, f"s_{tag}", s.reshape(-1))
                put(out, f"deq_{tag}", deq(q, s).to(dt))
    np.savez_compressed(os.path.join(HERE, "weight_quant.npz"), **out)


def gen_linear():
    from transformersurgeon.blocks import LinearCompressed
    from transformersurgeon.compression.lrd_methods.svd import low_rank_svd
    from transformersurgeon.compression.quantization_methods.vanilla import quantize_vanilla
    out = {}
    g = torch.Generator().manual_seed(12)
    W = torch.randn(192, 256, generator=g) * 0.05
    bias = torch.randn(192, generator=g) * 0.1
    put(out, "W", W)
    put(out, "bias", bias)
    for dt, name in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
        x = torch.randn(2, 5, 256, generator=g).to(dt)
        put(out, f"x_{name}", x)
        # full rank, with bias
        m = LinearCompressed(256, 192, bias=True, dtype=dt)
        with torch.no_grad():
            m.weight.copy_(W.to(dt)); m.bias.copy_(bias.to(dt))
            put(out, f"y_full_{name}", m(x))
        # rank 64 via the reference's SVD, no bias
        US, V = low_rank_svd(W.to(dt), 64)
        put(out, f"US_{name}", US); put(out, f"V_{name}", V)
        m = LinearCompressed(256, 192, bias=False, rank=64, dtype=dt)
        with torch.no_grad():
            m.weight.copy_(US); m.linear_V.weight.copy_(V)
            put(out, f"y_lrd_{name}", m(x))
            # fake-quantized factors (per-channel) exactly as Quantizer.apply stores them
            for p in (8, 4, "binary"):
                qu, su, f = quantize_vanilla(US, p, 1e-6, "per_channel")
                qv, sv, _ = quantize_vanilla(V, p, 1e-6, "per_channel")
                m.weight.copy_(f(qu, su)); m.linear_V.weight.copy_(f(qv, sv))
                put(out, f"y_lrd_q{p}_{name}", m(x))
                put(out, f"qu_{p}_{name}", qu); put(out, f"su_{p}_{name}", su.reshape(-1))
                put(out, f"qv_{p}_{name}", qv); put(out, f"sv_{p}_{name}", sv.reshape(-1))
    np.savez_compressed(os.path.join(HERE, "linear.npz"), **out)


def gen_blocks():
    from transformersurgeon.blocks.mha import attention
    from transformersurgeon.blocks.rope import (precompute_rope_inv_freqs,
                                                precompute_rope_cos_sin_half,
                                                apply_rope_multihead)
    from transformersurgeon.blocks.norm import RMSNorm
    from transformersurgeon.blocks.mlp import MLPGated
    out = {}
    g = torch.Generator().manual_seed(13)
    # attention: one query token over L cached tokens, GQA 8/2 and 14/2, d 64
    for tag, (H, Hkv, d, L) in {"a": (8, 2, 64, 37), "b": (14, 2, 64, 50), "c": (4, 4, 128, 16)}.items():
        q = torch.randn(1, H, d, generator=g); k = torch.randn(L, Hkv, d, generator=g)
        v = torch.randn(L, Hkv, d, generator=g)
        put(out, f"att_{tag}_q", q); put(out, f"att_{tag}_k", k); put(out, f"att_{tag}_v", v)
        put(out, f"att_{tag}_o", attention(q, k, v))
        mask = torch.where(torch.arange(L) > L // 2, -1e4, 0.0).view(1, 1, L)
        put(out, f"att_{tag}_mask", mask)
        put(out, f"att_{tag}_om", attention(q, k, v, mask))
    # RoPE
    inv = precompute_rope_inv_freqs(64, 1e6)
    cos, sin = precompute_rope_cos_sin_half(inv, 40, 0)
    put(out, "rope_cos", cos[:, 0]); put(out, "rope_sin", sin[:, 0])
    for dt, name in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
        x = torch.randn(40, 3, 64, generator=g).to(dt)
        put(out, f"rope_x_{name}", x)
        put(out, f"rope_y_{name}", apply_rope_multihead(x, cos.to(dt), sin.to(dt)))
        n = RMSNorm(96, dtype=dt)
        with torch.no_grad():
            n.weight.copy_((1 + 0.1 * torch.randn(96, generator=g)).to(dt))
            xn = (torch.randn(7, 96, generator=g) * 3).to(dt)
            put(out, f"norm_w_{name}", n.weight); put(out, f"norm_x_{name}", xn)
            put(out, f"norm_y_{name}", n(xn))
    # SwiGLU through MLPGated (fp32)
    torch.manual_seed(14)
    mlp = MLPGated(64, 160, activation="silu") if _mlp_accepts_activation() else MLPGated(64, 160)
    with torch.no_grad():
        x = torch.randn(6, 64, generator=g)
        put(out, "mlp_x", x)
        for nme in ("gate_proj", "up_proj", "down_proj"):
            lin = getattr(mlp, nme)
            put(out, f"mlp_{nme}_w", lin.weight)
            if lin.bias is not None:
                put(out, f"mlp_{nme}_b", lin.bias)
        put(out, "mlp_y", mlp(x))
    np.savez_compressed(os.path.join(HERE, "blocks.npz"), **out)


def _mlp_accepts_activation():
    import inspect
    from transformersurgeon.blocks.mlp import MLPGated
    return "activation" in inspect.signature(MLPGated.__init__).parameters


def gen_model(family):
    import transformersurgeon as T
    torch.manual_seed(21 if family == "qwen2" else 22)
    # head_dim = 128 / 2 = 64 (the smallest head size the kernels support), GQA group of 2
    kw = dict(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
              num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=128,
              tie_word_embeddings=False)
    if family == "qwen2":
        cfg = T.Qwen2ConfigCompress(**kw); model = T.Qwen2ForCausalLMCompress(cfg)
        mgr = T.Qwen2CompressionSchemesManager(model)
    else:
        cfg = T.LlamaConfigCompress(**kw); model = T.LlamaForCausalLMCompress(cfg)
        mgr = T.LlamaCompressionSchemesManager(model)
    model.eval()
    mgr.set("lrd", "rank", 16, criteria=["mlp"])
    mgr.set("lrd", "rank", 32, criteria=["self_attn.q_proj"])
    mgr.set("quantization", "precision", 8, criteria=["self_attn", "mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    mgr.apply(hard=False, verbose=False) if "verbose" in mgr.apply.__code__.co_varnames else mgr.apply(hard=False)
    out = {}
    for k, v in model.state_dict().items():
        put(out, "sd::" + k, v)
    g = torch.Generator().manual_seed(23)
    ids = torch.randint(0, 256, (2, 12), generator=g)
    with torch.no_grad():
        logits = model(input_ids=ids).logits
        toks = model.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=32,
                              do_sample=False, pad_token_id=0, eos_token_id=None)
    put(out, "ids", ids); put(out, "logits", logits); put(out, "tokens", toks)
    out["rope_theta"] = np.float64(getattr(cfg, "rope_theta", None) or cfg.rope_parameters["rope_theta"])
    out["rms_norm_eps"] = np.float64(cfg.rms_norm_eps)
    np.savez_compressed(os.path.join(HERE, f"model_{family}.npz"), **out)


if __name__ == "__main__":
    with torch.no_grad():
        gen_weight_quant(); gen_linear(); gen_blocks()
    gen_model("qwen2"); gen_model("llama")
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
