"""Hugging Face drop-in for the KV-cache boundary of the reference's HF path.

The reference's model classes inherit `generate()` from `transformers`
(models/qwen2_c/define_qwen2_c.py:22-27, models/llama_c/define_llama_c.py:24-30): every attention
layer calls `past_key_values.update(key, value, layer_idx)` and hands what comes back to the
attention function selected by `config._attn_implementation`.  This module supplies both halves:

  * `PagedQuantCache` - a `transformers.Cache` whose layers quantize-and-append into the paged pools
    (`tsb200_kv_append`) instead of concatenating tensors;
  * the attention function registered as `"tsb200_paged"`: one query token per sequence goes to the
    paged decode kernel (`tsb200_paged_decode_attn`); a prompt chunk (T > 1) attends causally over the
    cache's DEQUANTIZED contents with the prefill kernel (`tsb200_kv_gather_heads` + `tsb200_prefill_attn`
    on tcgen05 for bf16 models; fp32 models go through the paged decode kernel, one query token at a time).

Usage (generate() itself is untouched):

    model.config._attn_implementation = "tsb200_paged"      # or attn_implementation= at load time
    cache = PagedQuantCache(model.config, batch, max_len, kv_format="int8")
    model.generate(ids, past_key_values=cache, do_sample=False, ...)

Limits: every sequence of the batch has the same length and the mask is the plain causal one (a padded
batch is refused when first met); no beam reordering, cropping or sliding windows.
"""
import torch
from transformers import AttentionInterface
from transformers.cache_utils import Cache, CacheLayerMixin
from transformers.masking_utils import AttentionMaskInterface, sdpa_mask

from . import ops

ATTN_NAME = "tsb200_paged"
# Hand-over from `PagedCacheLayer.update` to the attention function of the same decoder layer, which runs right
# after it: keyed by layer index (the attention module carries `layer_idx`), taken out when used.
_PENDING = {}


class PagedCacheLayer(CacheLayerMixin):
    """One layer's paged pools.  Sequence b owns pages [b * P, (b + 1) * P) in logical order."""

    def __init__(self, kv_format, batch, max_len, hkv, head_dim, device, layer_idx=0):
        super().__init__()
        self.kv_format, self.batch, self.max_len, self.layer_idx = kv_format, batch, int(max_len), layer_idx
        self.mask_checked = False
        pages = (self.max_len + 15) // 16
        self.block_table = torch.arange(batch * pages, dtype=torch.int32, device=device).reshape(batch, pages)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=device)
        self.kv = ops.PagedKV(kv_format, batch * pages, hkv, head_dim, self.block_table, self.seq_lens, device)
        self.cumulative_length = 0
        self.is_initialized = True
        self.device = device

    def lazy_initialization(self, key_states, value_states):
        pass                                    # pools are allocated up front

    def update(self, key_states, value_states, *args, **kwargs):
        """key_states, value_states [B, hkv, T, d] (keys after RoPE).  Quantizes and appends, and hands this
        layer over to the attention function of the same decoder layer; the returned tensors are the inputs."""
        B, hkv, T, d = key_states.shape
        if B != self.batch:
            raise ValueError(f"cache was built for batch {self.batch}, got {B}")
        if self.cumulative_length + T > self.max_len:
            raise ValueError(f"cache holds {self.max_len} positions, {self.cumulative_length + T} requested")
        k = key_states.transpose(1, 2).contiguous()
        v = value_states.transpose(1, 2).contiguous()
        if self.kv.k_scale is not None and self.cumulative_length == 0:
            self.kv.set_fp8_scales(k, v)        # amax/448 over the prompt, frozen for decode
        self.kv.append(k, v)
        self.seq_lens += T
        self.cumulative_length += T
        _PENDING[self.layer_idx] = self         # the attention function reads the pages, not these tensors
        return key_states, value_states

    def get_mask_sizes(self, query_length):
        return self.cumulative_length + query_length, 0

    def get_seq_length(self):
        return self.cumulative_length

    def get_max_cache_shape(self):
        return self.max_len

    def reset(self):
        self.seq_lens.zero_()
        self.cumulative_length = 0
        self.mask_checked = False


class PagedQuantCache(Cache):
    """`past_key_values` object backed by quantized paged pools, one `PagedCacheLayer` per decoder layer."""

    def __init__(self, config, batch, max_len, kv_format="int8", device="cuda"):
        if getattr(config, "_attn_implementation", None) != ATTN_NAME:
            raise ValueError(f'set config._attn_implementation = "{ATTN_NAME}": other attention functions would '
                             "see only the newest token on a decode step")
        text = config.get_text_config() if hasattr(config, "get_text_config") else config
        hkv = getattr(text, "num_key_value_heads", None) or text.num_attention_heads
        head_dim = getattr(text, "head_dim", None) or text.hidden_size // text.num_attention_heads
        device = torch.device(device)
        layers = [PagedCacheLayer(kv_format, batch, max_len, hkv, head_dim, device, i) for i in range(text.num_hidden_layers)]
        super().__init__(layers=layers)


def _check_plain_causal(layer, attention_mask, T, L):
    """Once per generate(): the kernels implement the plain causal mask over equal-length sequences."""
    if layer.mask_checked:
        return
    if attention_mask is not None:
        m = attention_mask if attention_mask.dtype == torch.bool else (attention_mask == 0)
        m = m[..., -T:, :L]
        q = torch.arange(L - T, L, device=m.device)[:, None]
        k = torch.arange(L, device=m.device)[None, :]
        if not bool((m == (k <= q)).all()):
            raise NotImplementedError("PagedQuantCache: only the plain causal mask over equal-length sequences is "
                                      "supported (a padded batch would attend over its padding)")
    layer.mask_checked = True


def paged_attention_forward(module, query, key, value, attention_mask, dropout=0.0, scaling=None, **kwargs):
    """Attention function for `ALL_ATTENTION_FUNCTIONS`: query [B, H, T, d] -> ([B, T, H, d], None)."""
    layer = _PENDING.pop(getattr(module, "layer_idx", None), None)
    if layer is None:
        raise RuntimeError(f'attention "{ATTN_NAME}" needs past_key_values=PagedQuantCache(...) (the cache layer of this '
                           "decoder layer did not announce itself)")
    T, L = query.shape[2], layer.cumulative_length
    _check_plain_causal(layer, attention_mask, T, L)
    if T == 1:
        q = query[:, :, 0, :].contiguous()
        out = ops.paged_decode_attention(layer.kv, q, max_seq_len=layer.max_len, sm_scale=scaling)
        return out[:, None], None
    out = ops.prefill_attention(layer.kv, query.transpose(1, 2).contiguous(), L, sm_scale=scaling)
    return out, None


AttentionInterface.register(ATTN_NAME, paged_attention_forward)
AttentionMaskInterface.register(ATTN_NAME, sdpa_mask)
