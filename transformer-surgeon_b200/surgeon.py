"""Drop-in glue between transformer-surgeon models and the B200 kernels.

pack_model(model)   after `manager.apply()`: attaches a PackedLinear to every LinearCompressed
                    instance and rebinds `forward` ON THE INSTANCE, so `type(m) is LinearCompressed`
                    stays true (the reference tests type identity with `is`: utils/scheme.py:316-320,
                    utils/manager.py:1064-1066, utils/modeling.py:57).  unpack_model() detaches,
                    e.g. before `manager.restore()` rewrites the weights (utils/scheme.py:572-579).
decoder_from_state_dict / decoder_from_model
                    build the CUDA decode engine (decoder.CompressedDecoder) for a Qwen2 / Llama
                    `*ForCausalLMCompress` model.

Codes and scales are re-derived on the GPU from the stored (fake-quantized) factors with the
reference's arithmetic (compression/quantization_methods/vanilla.py:10-37).  For fixed-point
precisions this reproduces the codes the reference computed before it discarded them
(re-quantizing q*scale gives q back); precision / granularity / eps come from
`model.config.compression_config[path]["quantization"]` (utils/configuration.py:54-73).
"""
import types

import torch

from . import ops
from .decoder import CompressedDecoder, DecoderConfig, LayerWeights, fuse_rows

BLOCK_LINEARS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                 "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")


def _quant_of(compression_config, path):
    """(precision, granularity, eps) for a module path, or None when it is not quantized."""
    if not compression_config:
        return None
    q = (compression_config.get(path) or {}).get("quantization") or {}
    prec = q.get("precision", "full")
    if prec in ("full", None):
        return None
    return prec, q.get("granularity", "per_tensor"), float(q.get("eps", 1e-6))


def pack_linear(weight, v_weight=None, bias=None, quant=None, dtype=None, device="cuda"):
    """weight [out, r|in], v_weight [r, in] or None -> ops.PackedLinear."""
    dtype = dtype or weight.dtype
    w = weight.detach().to(device=device, dtype=dtype).contiguous()
    v = None if v_weight is None else v_weight.detach().to(device=device, dtype=dtype).contiguous()
    if quant is None:
        fu, fv = ops.Factor.dense(w), (None if v is None else ops.Factor.dense(v))
    else:
        prec, gran, eps = quant
        fu = ops.Factor.quantize(w, prec, gran, eps)
        fv = None if v is None else ops.Factor.quantize(v, prec, gran, eps)
    b = None if bias is None else bias.detach().to(device=device, dtype=dtype).contiguous()
    return ops.PackedLinear(fu, fv, b, dtype)


def decoder_from_state_dict(sd, cfg, compression_config=None, batch=1, max_seq_len=256, device="cuda",
                            prefix="model.", fuse_qkv=True, tp_group=None):
    """sd: state dict of a Qwen2/Llama `*ForCausalLMCompress` (keys `model.layers.N.<linear>.weight`,
    `.linear_V.weight`, `.bias`, norms, `model.embed_tokens.weight`, `lm_head.weight`)."""
    dt = cfg.dtype
    dev = torch.device(device)

    def lin(path):
        w = sd[path + ".weight"]
        return pack_linear(w, sd.get(path + ".linear_V.weight"), sd.get(path + ".bias"),
                           _quant_of(compression_config, path), dt, dev)

    layers = []
    for i in range(cfg.num_layers):
        base = f"{prefix}layers.{i}."
        L = {name: lin(base + name) for name in BLOCK_LINEARS}
        q, k, v = L["self_attn.q_proj"], L["self_attn.k_proj"], L["self_attn.v_proj"]
        qkv = None
        if fuse_qkv and cfg.tp_world == 1 and not (q.rank or k.rank or v.rank):
            qkv = fuse_rows([q.u, k.u, v.u], [q.bias, k.bias, v.bias], dt)
        ln1 = sd[base + "input_layernorm.weight"].to(device=dev, dtype=dt).contiguous()
        ln2 = sd[base + "post_attention_layernorm.weight"].to(device=dev, dtype=dt).contiguous()
        layers.append(LayerWeights(ln1, ln2, L["self_attn.o_proj"], L["mlp.gate_proj"], L["mlp.up_proj"],
                                   L["mlp.down_proj"], qkv=qkv, q=None if qkv else q, k=None if qkv else k,
                                   v=None if qkv else v))
    embed = sd[prefix + "embed_tokens.weight"].to(device=dev, dtype=dt).contiguous()
    head_key = "lm_head.weight" if "lm_head.weight" in sd else prefix + "embed_tokens.weight"
    lm_head = pack_linear(sd[head_key], sd.get("lm_head.linear_V.weight"), sd.get("lm_head.bias"),
                          _quant_of(compression_config, "lm_head"), dt, dev)
    norm = sd[prefix + "norm.weight"].to(device=dev, dtype=dt).contiguous()
    return CompressedDecoder(cfg, embed, layers, norm, lm_head, batch, max_seq_len, dev, tp_group=tp_group)


def decoder_config_from_hf(config, kv_format="fp8", dtype=None, max_positions=None):
    theta = getattr(config, "rope_theta", None)
    if theta is None:
        theta = (getattr(config, "rope_parameters", None) or {}).get("rope_theta", 10000.0)
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    return DecoderConfig(config.num_hidden_layers, config.hidden_size, config.num_attention_heads,
                         config.num_key_value_heads, head_dim, config.intermediate_size, config.vocab_size,
                         float(theta), float(config.rms_norm_eps), 0, dtype or torch.bfloat16, kv_format,
                         max_positions or config.max_position_embeddings)


def decoder_from_model(model, batch, max_seq_len, kv_format="fp8", device="cuda"):
    """Build the decode engine from a live `Qwen2ForCausalLMCompress` / `LlamaForCausalLMCompress`."""
    dtype = next(model.parameters()).dtype
    cfg = decoder_config_from_hf(model.config, kv_format, dtype, max(max_seq_len, 16))
    return decoder_from_state_dict(model.state_dict(), cfg, getattr(model.config, "compression_config", None),
                                   batch, max_seq_len, device)


# ------------------------------------------------------------------------ per-module rebinding
def _is_linear_compressed(m):
    return type(m).__name__ == "LinearCompressed" and hasattr(m, "linear_V") and hasattr(m, "rank")


def _packed_forward(self, input):
    # LinearCompressed.forward contract (blocks/linear_compressed.py:81-105): skip -> identity,
    # any leading shape, result in the input dtype.
    if getattr(self, "skip", False):
        return input
    return self._tsb200(input)


def pack_model(model, device="cuda"):
    """Attach kernels to every LinearCompressed instance of `model` (moved to `device` by the caller)."""
    cc = getattr(getattr(model, "config", None), "compression_config", None)
    n = 0
    for path, m in model.named_modules():
        if not _is_linear_compressed(m) or getattr(m, "skip", False):
            continue
        v = m.linear_V.weight if (isinstance(m.rank, int) and m.linear_V is not None) else None
        m._tsb200 = pack_linear(m.weight, v, m.bias, _quant_of(cc, path), m.weight.dtype, device)
        m.forward = types.MethodType(_packed_forward, m)      # instance attribute: the class is untouched
        n += 1
    return n


PACKED_KEY = "._tsb200."


def packed_state_dict(model):
    """Packed codes, scales and biases of every packed LinearCompressed of `model` as a flat dict of
    CPU tensors keyed `<module path>._tsb200.<field>` - extra entries for a checkpoint, so that
    loading does not need the pack step (the reference re-creates factorised modules from
    `config.compression_config` on load, utils/modeling.py:65-77, but discards quantization codes)."""
    sd = {}
    for path, m in model.named_modules():
        if hasattr(m, "_tsb200"):
            for k, t in m._tsb200.state(path + PACKED_KEY).items():
                sd[k] = t.detach().cpu()
    return sd


def load_packed_state_dict(model, sd, device="cuda"):
    """Attach kernels from `packed_state_dict` output; the modules' float weights are not read.
    Returns the number of modules attached; a LinearCompressed without an entry is left alone."""
    n = 0
    for path, m in model.named_modules():
        if not _is_linear_compressed(m) or (path + PACKED_KEY + "u.meta") not in sd:
            continue
        p = ops.PackedLinear.from_state(sd, path + PACKED_KEY, device)
        if p.out_features != m.weight.shape[0] or p.in_features != (m.linear_V.weight.shape[1] if p.v is not None else m.weight.shape[1]):
            raise ValueError(f"{path}: packed entry is {p.out_features}x{p.in_features}, module differs")
        m._tsb200 = p
        m.forward = types.MethodType(_packed_forward, m)
        n += 1
    return n


def unpack_model(model):
    for _, m in model.named_modules():
        if hasattr(m, "_tsb200"):
            del m._tsb200
            if "forward" in m.__dict__:
                del m.__dict__["forward"]
