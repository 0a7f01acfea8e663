"""Drop-in glue between transformer-surgeon models and the B200 kernels.

capture_quantization(model)
                    context manager for `manager.apply()`: records the integer codes and scales every
                    quantization method returns (compression/quantization.py:108) before the reference
                    overwrites the parameter with the dequantized floats and drops them (:112, :126).
pack_model(model)   after `manager.apply()`: attaches a PackedLinear to every LinearCompressed
                    instance and rebinds `forward` ON THE INSTANCE, so `type(m) is LinearCompressed`
                    stays true (the reference tests type identity with `is`: utils/scheme.py:316-320,
                    utils/manager.py:1064-1066, utils/modeling.py:57).  unpack_model() detaches,
                    e.g. before `manager.restore()` rewrites the weights (utils/scheme.py:572-579).
decoder_from_state_dict / decoder_from_model
                    build the CUDA decode engine (decoder.CompressedDecoder) for a Qwen2 / Llama /
                    Qwen2.5-VL-text `*Compress` model.

Where the codes come from, in order of preference: (1) codes captured at apply time (exact for every
method, GPTQ included); (2) persisted packed entries (`packed_state_dict`); (3) re-derivation on the GPU
from the stored fake-quantized factors with the reference's arithmetic
(compression/quantization_methods/vanilla.py:10-37; binary: sign and the common magnitude, which the
stored row holds exactly).  Re-derivation reproduces the codes for fp32 parameters with eps far below
scale/qmax; it can differ otherwise (a bf16-stored q*scale, a scale near eps).  Whatever the source, a
packed factor is kept only if it reconstructs the stored weights BIT FOR BIT; otherwise the factor stays
dense, so a packed model never computes with other weights than the reference's.
Precision / granularity / eps come from `model.config.compression_config[path]["quantization"]`
(utils/configuration.py:54-73).
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


def _factor(w, quant, codes=None):
    """One factor in kernel form.  `codes` = (int8 codes, scales) captured from the reference; without
    them the codes are re-derived from the stored floats.  Falls back to the dense matrix whenever the
    packed factor would not reconstruct `w` bit for bit."""
    if quant is None:
        return ops.Factor.dense(w)
    prec, gran, eps = quant
    if codes is not None:
        f = ops.Factor.from_codes(codes[0].to(w.device), codes[1], prec)
    elif prec == "binary":
        # stored row = sign * scale: every non-zero entry has the scale's magnitude, no mean to re-derive
        q = torch.sign(w).to(torch.int8)
        sc = w.abs().amax(dim=1).float() if gran == "per_channel" else w.abs().max().float().reshape(1)
        f = ops.Factor.from_codes(q, sc, prec)
    else:
        f = ops.Factor.quantize(w, prec, gran, eps)
    if not torch.equal(f.reconstruct(w.dtype), w):
        return ops.Factor.dense(w)
    return f


def pack_linear(weight, v_weight=None, bias=None, quant=None, dtype=None, device="cuda", codes=None, v_codes=None):
    """weight [out, r|in], v_weight [r, in] or None -> ops.PackedLinear.  `codes` / `v_codes`: optional
    (int8 codes, scales) of the two factors as the reference's quantization method returned them."""
    dtype = dtype or weight.dtype
    w = weight.detach().to(device=device, dtype=dtype).contiguous()
    v = None if v_weight is None else v_weight.detach().to(device=device, dtype=dtype).contiguous()
    fu = _factor(w, quant, codes)
    fv = None if v is None else _factor(v, quant, v_codes)
    b = None if bias is None else bias.detach().to(device=device, dtype=dtype).contiguous()
    return ops.PackedLinear(fu, fv, b, dtype)


class capture_quantization:
    """`with capture_quantization(model) as cap: manager.apply()` keeps what the reference throws away.

    Quantizer.apply calls `METHOD_FUNCTIONS[method](param.data, precision, eps, granularity, ...)`
    (compression/quantization.py:108) and writes `dequantize(q, scale)` back into the parameter (:112, :126).
    Inside the context every entry of that table is wrapped so that (q, scale, precision) is recorded under
    the parameter's storage address; on exit the addresses are resolved to `<module path>.<param name>`
    (so call it BEFORE moving the model to another device) and the result is attached to the model as
    `model._tsb200_codes`, where pack_model and decoder_from_model find it.  A record whose dequantized
    values do not equal the stored parameter (e.g. a sparsity mask mixed the original weights back in)
    is dropped."""

    def __init__(self, model):
        self.model, self.codes, self._by_ptr, self._saved = model, {}, {}, None

    def __enter__(self):
        from transformersurgeon.compression import quantization as refq
        self._table = refq.METHOD_FUNCTIONS
        self._saved = dict(self._table)
        for name, fn in self._saved.items():
            self._table[name] = self._wrap(fn)
        return self

    def _wrap(self, fn):
        def wrapped(weight, precision, *args, **kwargs):
            q, scale, deq = fn(weight, precision, *args, **kwargs)
            self._by_ptr[weight.data_ptr()] = (q.detach().clone(), scale.detach().clone(), precision, deq)
            return q, scale, deq
        return wrapped

    def __exit__(self, *exc):
        self._table.update(self._saved)
        for path, m in self.model.named_modules():
            if not _is_linear_compressed(m):
                continue
            for pname, prm in (("weight", m.weight), ("linear_V.weight", getattr(m.linear_V, "weight", None))):
                rec = None if prm is None else self._by_ptr.get(prm.data_ptr())
                if rec is None:
                    continue
                q, scale, precision, deq = rec
                if q.shape == prm.shape and torch.equal(deq(q, scale).to(prm.dtype), prm.data):
                    self.codes[f"{path}.{pname}"] = (q.to(torch.int8).cpu(), scale.detach().float().reshape(-1).cpu(), precision)
        self._by_ptr.clear()
        self.model._tsb200_codes = self.codes
        return False


def _captured(codes, path, pname):
    rec = (codes or {}).get(f"{path}.{pname}")
    return None if rec is None else (rec[0], rec[1])


def decoder_from_state_dict(sd, cfg, compression_config=None, batch=1, max_seq_len=256, device="cuda",
                            prefix="model.", fuse_qkv=True, tp_group=None, codes=None):
    """sd: state dict of a Qwen2/Llama `*ForCausalLMCompress` (keys `model.layers.N.<linear>.weight`,
    `.linear_V.weight`, `.bias`, norms, `model.embed_tokens.weight`, `lm_head.weight`)."""
    dt = cfg.dtype
    dev = torch.device(device)

    def lin(path):
        w = sd[path + ".weight"]
        return pack_linear(w, sd.get(path + ".linear_V.weight"), sd.get(path + ".bias"),
                           _quant_of(compression_config, path), dt, dev,
                           _captured(codes, path, "weight"), _captured(codes, path, "linear_V.weight"))

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
    head_key = "lm_head.weight" if "lm_head.weight" in sd else prefix + "embed_tokens.weight"     # tied embeddings
    lm_head = pack_linear(sd[head_key], sd.get("lm_head.linear_V.weight"), sd.get("lm_head.bias"),
                          _quant_of(compression_config, "lm_head"), dt, dev,
                          _captured(codes, "lm_head", "weight"), _captured(codes, "lm_head", "linear_V.weight"))
    norm = sd[prefix + "norm.weight"].to(device=dev, dtype=dt).contiguous()
    return CompressedDecoder(cfg, embed, layers, norm, lm_head, batch, max_seq_len, dev, tp_group=tp_group)


def decoder_config_from_hf(config, kv_format="fp8", dtype=None, max_positions=None):
    """DecoderConfig of a Qwen2 / Llama config, or of the text tower of a Qwen2.5-VL config."""
    config = config.get_text_config() if hasattr(config, "get_text_config") else config
    theta = getattr(config, "rope_theta", None)
    if theta is None:
        theta = (getattr(config, "rope_parameters", None) or {}).get("rope_theta", 10000.0)
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    return DecoderConfig(config.num_hidden_layers, config.hidden_size, config.num_attention_heads,
                         config.num_key_value_heads, head_dim, config.intermediate_size, config.vocab_size,
                         float(theta), float(config.rms_norm_eps), 0, dtype or torch.bfloat16, kv_format,
                         max_positions or config.max_position_embeddings)


def decoder_from_model(model, batch=1, max_seq_len=None, kv_format=None, device="cuda", options=None, **kw):
    """Build the decode engine from a live `Qwen2ForCausalLMCompress` / `LlamaForCausalLMCompress` /
    `Qwen2_5_VLForConditionalGenerationCompress` (text tower; text-only prompts, for which the three mrope
    position rows coincide and the rotary embedding is the plain 1-D one).

    options: the dict `convert_for_export` takes (utils/convert.py:304-308): `max_cache_len` (default 2048)
    bounds the context, `cache_impl` picks the cache format among blocks_path.CACHE_IMPLS (`paged_int8`,
    `paged_fp8`, `paged_nvfp4`, `paged_bf16`, `paged_fp32`); `use_sdpa` has no meaning here.  Explicit
    `max_seq_len` / `kv_format` arguments win over the options.  The layer math is the HF model's (what
    `generate()` runs); for the reference's blocks-path variant of the math use `convert_for_export`."""
    from . import blocks_path
    options = dict(options or {})
    if kv_format is None:
        kv_format = blocks_path.kv_format_of(options["cache_impl"]) if "cache_impl" in options else "fp8"
    if max_seq_len is None:
        max_seq_len = int(options.get("max_cache_len", 2048))
    dtype = next(model.parameters()).dtype
    cfg = decoder_config_from_hf(model.config, kv_format, dtype, max(max_seq_len, 16))
    text = model.config.get_text_config() if hasattr(model.config, "get_text_config") else model.config
    cc = getattr(text, "compression_config", None) or getattr(model.config, "compression_config", None)
    sd = model.state_dict()
    prefix = "model.language_model." if "model.language_model.embed_tokens.weight" in sd else "model."
    return decoder_from_state_dict(sd, cfg, cc, batch, max_seq_len, device, prefix=prefix,
                                   codes=getattr(model, "_tsb200_codes", None), **kw)


def convert_for_export(model, options=None, batch=1, device="cuda", verbose=False):
    """`convert_for_export` (utils/convert.py:266) with the paged cache implementations added to `cache_impl`.

    For the reference's own values (`mutable`, `io_scatter`, `io_concat`) the call is handed to the reference
    unchanged.  For `paged_int8 | paged_fp8 | paged_nvfp4 | paged_bf16 | paged_fp32` the reference still does
    the conversion (indexing, layer matching, bias flags, extra layers - none of that is re-implemented) in one
    of its own modes, and every converted `TransformerDecoder` is then packed into a
    blocks_path.PagedTransformerDecoder that runs on the kernels.  Returns the same {component: decoder} dict."""
    from transformersurgeon.utils.convert import convert_for_export as reference_convert
    from . import blocks_path
    options = dict(options or {})
    impl = options.get("cache_impl", "mutable")
    if impl not in blocks_path.CACHE_IMPLS:
        return reference_convert(model, options=options, verbose=verbose)       # the reference validates the value
    options["cache_impl"] = "io_scatter"
    converted = reference_convert(model, options=options, verbose=verbose)
    out = {}
    for name, dec in converted.items():
        if type(dec).__name__ == "TransformerDecoder":
            out[name] = blocks_path.PagedTransformerDecoder.from_converted(dec, impl, batch=batch, device=device)
        else:
            out[name] = dec
    return out


# ------------------------------------------------------------------------ per-module rebinding
def _is_linear_compressed(m):
    return type(m).__name__ == "LinearCompressed" and hasattr(m, "linear_V") and hasattr(m, "rank")


def _packed_forward(self, input):
    # LinearCompressed.forward contract (blocks/linear_compressed.py:81-105): skip -> identity,
    # any leading shape, result in the input dtype.
    if getattr(self, "skip", False):
        return input
    return self._tsb200(input)


def pack_model(model, device="cuda", codes=None):
    """Attach kernels to every LinearCompressed instance of `model` (moved to `device` by the caller).
    `codes`: what `capture_quantization` recorded (default: `model._tsb200_codes` when present)."""
    cc = getattr(getattr(model, "config", None), "compression_config", None)
    codes = codes if codes is not None else getattr(model, "_tsb200_codes", None)
    n = 0
    for path, m in model.named_modules():
        if not _is_linear_compressed(m) or getattr(m, "skip", False):
            continue
        v = m.linear_V.weight if (isinstance(m.rank, int) and m.linear_V is not None) else None
        m._tsb200 = pack_linear(m.weight, v, m.bias, _quant_of(cc, path), m.weight.dtype, device,
                                _captured(codes, path, "weight"), _captured(codes, path, "linear_V.weight"))
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


BUFFER_PREFIX = "_tsb200_"


def register_packed_buffers(model):
    """Make the packed codes part of the checkpoint: every tensor of a packed LinearCompressed's state
    (`PackedLinear.state`) becomes a persistent buffer `_tsb200_<field>` of that module, so it is in
    `model.state_dict()`, is left alone by `manager.prepare_for_save()` (utils/manager.py:843-894 strips only
    the Quantizer's own attributes, compression/quantization.py:198-230) and is written by `save_pretrained` /
    `export_to_hf` (hf/hf_export.py:42-51).  Loading the checkpoint into a freshly built model reports the
    entries as unexpected keys and ignores them; `load_packed_checkpoint` attaches them.  Returns the number
    of modules."""
    n = 0
    for _, m in model.named_modules():
        if hasattr(m, "_tsb200"):
            for k, t in m._tsb200.state("").items():
                m.register_buffer(BUFFER_PREFIX + k.replace(".", "_"), t.detach().clone(), persistent=True)
            n += 1
    return n


def remove_packed_buffers(model):
    for _, m in model.named_modules():
        for name in [b for b in m._buffers if b.startswith(BUFFER_PREFIX)]:
            del m._buffers[name]


def packed_buffers_to_state(sd):
    """`<path>._tsb200_u_data`-style keys of a state dict -> the `<path>._tsb200.u.data` keys that
    `load_packed_state_dict` reads."""
    out = {}
    for k, t in sd.items():
        path, _, name = k.rpartition(".")
        if not name.startswith(BUFFER_PREFIX):
            continue
        field = name[len(BUFFER_PREFIX):]
        for head in ("u_", "v_"):
            if field.startswith(head):
                field = head[0] + "." + field[2:]
        out[path + PACKED_KEY + field] = t
    return out


def load_packed_checkpoint(model, directory, device="cuda"):
    """Attach kernels to `model` (built by `from_pretrained(directory)`) from the packed buffers stored in the
    checkpoint's safetensors files: no pack step, no re-quantization.  Returns the number of modules attached."""
    import glob
    import os
    from safetensors.torch import load_file
    sd = {}
    for f in sorted(glob.glob(os.path.join(directory, "*.safetensors"))):
        sd.update({k: t for k, t in load_file(f).items() if ("." + BUFFER_PREFIX) in k})
    return load_packed_state_dict(model, packed_buffers_to_state(sd), device)


def unpack_model(model):
    remove_packed_buffers(model)
    for _, m in model.named_modules():
        if hasattr(m, "_tsb200"):
            del m._tsb200
            if "forward" in m.__dict__:
                del m.__dict__["forward"]
