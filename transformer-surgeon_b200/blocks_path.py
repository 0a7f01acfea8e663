"""The reference's BLOCKS path (single-token decode contract) on the B200 kernels.

The reference converts a `*ForCausalLMCompress` model with `convert_for_export(model, options)`
(utils/convert.py:266-406) into a `TransformerDecoder` (blocks/decoder.py:152-250), wraps it as
`LLMWrapper(embedding, decoder, final_layer)` (export/common.py:141-176) and drives it one token at a
time: `logits, key_caches, value_caches = wrapper(token, pos_id, key_caches, value_caches)`
(examples/04_cache_impl_export_interface.py:115-139).  `cache_impl` selects how the KV cache is
written; the reference knows `mutable | io_scatter | io_concat` (blocks/mha.py:438), all dense.

This module adds the quantized, paged implementations under the same vocabulary and call shape:

    converted = surgeon.convert_for_export(model, options={"cache_impl": "paged_fp8", "max_cache_len": 2048})
    wrapper   = LLMWrapper(model.get_input_embeddings(), converted["text"], model.lm_head)
    caches    = build_paged_caches(wrapper.decoder)                  # the caller owns the caches (io_* contract)
    logits, caches = wrapper(token_id, pos_id, caches)               # cache in -> cache out

As on the reference's path the decoder uses the blocks RMSNorm (x / max(1, |x|_inf), eps 1e-5,
blocks/norm.py:8-23), a RoPE base fixed at 1e6 (blocks/decoder.py:184-187) and writes the new K/V at
`clamp(pos_id, 0, max_cache_len - 1)` (blocks/mha.py:583); attention covers positions 0..pos_id, which is
what the reference's -1e4 penalty on later positions (blocks/mha.py:592-593) amounts to in fp32.

Beyond the reference: `batch` sequences may share one wrapper (input_ids [B], one pos_id for all), and
`LLMWrapper.prefill` feeds a whole prompt in one pass (needed for `paged_fp8`, whose per-sequence scales
are taken over the prompt).
"""
import torch

from . import ops
from .decoder import CompressedDecoder, DecoderConfig, LayerWeights, fuse_rows

# cache_impl values served here (the reference's own three stay with the reference)
CACHE_IMPLS = ("paged_int8", "paged_fp8", "paged_nvfp4", "paged_bf16", "paged_fp32")
_BLOCK_LINEARS = ("attn.q_proj", "attn.k_proj", "attn.v_proj", "attn.out_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")


def kv_format_of(cache_impl):
    if cache_impl not in CACHE_IMPLS:
        raise ValueError(f"Unsupported cache_impl {cache_impl!r}; expected one of {CACHE_IMPLS}")
    return cache_impl[len("paged_"):]


class PagedCaches:
    """What the caller threads through every call instead of (key_caches, value_caches): one ops.PagedKV per
    block (pools, and scales for FP8) plus the block table and the per-sequence lengths they share."""

    def __init__(self, kv, block_table, seq_lens, cache_impl):
        self.kv, self.block_table, self.seq_lens, self.cache_impl = kv, block_table, seq_lens, cache_impl

    @property
    def key_caches(self):
        return [x.k_pool for x in self.kv]

    @property
    def value_caches(self):
        return [x.v_pool for x in self.kv]

    def reset(self):
        self.seq_lens.zero_()


class PagedTransformerDecoder:
    """Counterpart of blocks/decoder.py:152 `TransformerDecoder` for the paged cache implementations: the
    packed block weights and the final norm.  The decode engine is completed by `LLMWrapper`, which brings the
    embedding and the final layer, as in the reference."""

    def __init__(self, cfg, layers, final_norm, cache_impl, max_cache_len, batch, device):
        self.cfg, self.layers, self.final_norm = cfg, layers, final_norm
        self.cache_impl, self.max_cache_len, self.batch, self.device = cache_impl, int(max_cache_len), batch, device
        self.depth = cfg.num_layers
        self.engine = None

    @staticmethod
    def from_converted(ref_decoder, cache_impl, batch=1, device="cuda", fuse_qkv=True):
        """ref_decoder: the reference's converted `TransformerDecoder` (any of its cache_impl values; only its
        config and weights are read)."""
        from . import surgeon
        fmt = kv_format_of(cache_impl)
        c = ref_decoder.config
        dev = torch.device(device)
        sd = ref_decoder.state_dict()
        dt = sd["norm.weight"].dtype                      # the converted config may leave `dtype` unset
        hkv = getattr(c, "num_key_value_heads", None) or c.num_attention_heads
        max_len = int(c.max_cache_len)
        cfg = DecoderConfig(num_layers=c.num_hidden_layers, hidden=c.hidden_size, num_heads=c.num_attention_heads,
                            num_kv_heads=hkv, head_dim=c.hidden_size // c.num_attention_heads,
                            intermediate=c.intermediate_size, vocab=0, rope_theta=1e6, rms_eps=1e-5, norm_variant=1,
                            dtype=dt, kv_format=fmt, max_positions=max_len)
        if getattr(c, "hidden_act", "silu") != "silu" or getattr(c, "mlp_type", "mlp_gated") != "mlp_gated":
            raise ValueError("the kernels implement the SiLU-gated MLP (Qwen2 / Llama)")
        cc = getattr(c, "compression_config", None) or {}

        def lin(path):
            return surgeon.pack_linear(sd[path + ".weight"], sd.get(path + ".linear_V.weight"), sd.get(path + ".bias"),
                                       surgeon._quant_of(cc, path), dt, dev)

        layers = []
        for i in range(cfg.num_layers):
            base = f"blocks.{i}."
            L = {n: lin(base + n) for n in _BLOCK_LINEARS}
            q, k, v = L["attn.q_proj"], L["attn.k_proj"], L["attn.v_proj"]
            qkv = fuse_rows([q.u, k.u, v.u], [q.bias, k.bias, v.bias], dt) if fuse_qkv and not (q.rank or k.rank or v.rank) else None
            ln1 = sd[base + "norm_in.weight"].to(device=dev, dtype=dt).contiguous()
            ln2 = sd[base + "norm_out.weight"].to(device=dev, dtype=dt).contiguous()
            layers.append(LayerWeights(ln1, ln2, L["attn.out_proj"], L["mlp.gate_proj"], L["mlp.up_proj"], L["mlp.down_proj"],
                                       qkv=qkv, q=None if qkv else q, k=None if qkv else k, v=None if qkv else v))
        norm = sd["norm.weight"].to(device=dev, dtype=dt).contiguous()
        return PagedTransformerDecoder(cfg, layers, norm, cache_impl, max_len, batch, dev)

    def attach(self, embedding, final_layer):
        """Complete the engine with the embedding module and the final layer (a LinearCompressed / nn.Linear)."""
        from . import surgeon
        c, dev = self.cfg, self.device
        with torch.no_grad():
            vocab = embedding.num_embeddings if hasattr(embedding, "num_embeddings") else embedding.weight.shape[0]
            table = embedding(torch.arange(vocab, device=next(embedding.parameters()).device))     # any embedding module
            embed = table.to(device=dev, dtype=c.dtype).contiguous()
            v = final_layer.linear_V.weight if isinstance(getattr(final_layer, "rank", "full"), int) and \
                getattr(final_layer, "linear_V", None) is not None else None
            prec = getattr(final_layer, "_soft_quant_precision", None)
            head = None
            for gran in ("per_channel", "per_tensor"):      # the module carries its precision tag, not its granularity:
                if prec in (None, "full"):                  # take the one that reconstructs the stored weights exactly
                    break
                cand = surgeon.pack_linear(final_layer.weight, v, final_layer.bias, (prec, gran, 1e-6), c.dtype, dev)
                if cand.u.bits < 16:
                    head = cand
                    break
            if head is None:
                head = surgeon.pack_linear(final_layer.weight, v, final_layer.bias, None, c.dtype, dev)
        cfg = DecoderConfig(**{**c.__dict__, "vocab": vocab})
        self.cfg = cfg
        self.engine = CompressedDecoder(cfg, embed, self.layers, self.final_norm, head, self.batch, self.max_cache_len, dev,
                                        own_caches=False)
        return self.engine


def build_paged_caches(decoder, fp8_scales=None):
    """Caller-owned caches for `decoder` (counterpart of export/common.py:120 `build_zero_caches`): zero-filled
    pools of ceil(max_cache_len / 16) pages per sequence, pages handed out in ascending order sequence by
    sequence.  fp8_scales: optional (k_scale, v_scale) floats or [B, hkv] tensors for `paged_fp8` when the
    prompt will be fed token by token (otherwise use LLMWrapper.prefill, which measures them)."""
    c, B, dev = decoder.cfg, decoder.batch, decoder.device
    pages = (decoder.max_cache_len + ops.PAGE - 1) // ops.PAGE
    block_table = torch.arange(B * pages, dtype=torch.int32, device=dev).reshape(B, pages)
    seq_lens = torch.zeros(B, dtype=torch.int32, device=dev)
    kv = [ops.PagedKV(c.kv_format, B * pages, c.num_kv_heads, c.head_dim, block_table, seq_lens, dev) for _ in range(c.num_layers)]
    if fp8_scales is not None:
        for x in kv:
            x.fill_fp8_scales(*fp8_scales)
    return PagedCaches(kv, block_table, seq_lens, decoder.cache_impl)


class LLMWrapper:
    """export/common.py:141 `LLMWrapper` for the paged cache implementations:
        forward(input_ids, pos_id_tensor, caches) -> (logits, caches)
    input_ids: LongTensor [1] (or [B] for a batch-B decoder), pos_id_tensor: LongTensor [1] = absolute position of
    the token = where its K/V is written.  logits: [vocab] ([B, vocab] for B > 1), a view of a buffer the next
    call overwrites."""

    def __init__(self, embedding, decoder, final_layer):
        if not isinstance(decoder, PagedTransformerDecoder):
            raise TypeError("decoder must come from surgeon.convert_for_export with a paged cache_impl")
        self.decoder = decoder
        self.cache_impl = decoder.cache_impl
        self.engine = decoder.attach(embedding, final_layer)
        self._bound = None

    def eval(self):
        return self

    def _bind(self, caches):
        if caches is None:
            raise ValueError(f"cache_impl {self.cache_impl!r}: the caller owns the caches - pass build_paged_caches(decoder)")
        if caches is not self._bound:
            if caches.cache_impl != self.cache_impl:
                raise ValueError(f"caches were built for {caches.cache_impl!r}, decoder runs {self.cache_impl!r}")
            self.engine.bind_caches(caches.kv, caches.block_table, caches.seq_lens)
            self._bound = caches

    @torch.no_grad()
    def forward(self, input_ids, pos_id_tensor, caches=None):
        eng = self.engine
        self._bind(caches)
        if eng.cfg.kv_format == "fp8" and not all(x.fp8_scales_set for x in caches.kv):
            raise ValueError("paged_fp8: scales are unset - feed the prompt with LLMWrapper.prefill, or pass "
                             "fp8_scales to build_paged_caches")
        pos = torch.clamp(pos_id_tensor.reshape(-1).to(eng.device), 0, self.decoder.max_cache_len - 1).to(torch.int32)
        caches.seq_lens.copy_(pos.expand_as(caches.seq_lens))        # the step appends at seq_lens, then attends over seq_lens + 1
        logits = eng.step(input_ids.reshape(-1).to(eng.device))
        return (logits[0] if eng.B == 1 else logits), caches

    __call__ = forward

    @torch.no_grad()
    def prefill(self, prompt_ids, caches):
        """All prompt tokens in one pass (positions 0..T-1); returns the last token's logits like `forward`.
        prompt_ids: [T] or [B, T]."""
        eng = self.engine
        self._bind(caches)
        ids = prompt_ids.reshape(eng.B, -1)
        logits = eng.prefill(ids)
        return (logits[0] if eng.B == 1 else logits), caches
