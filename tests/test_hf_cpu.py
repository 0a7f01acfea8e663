"""Host-side checks of the Hugging Face adapter that need no GPU."""
import pytest


def test_attention_function_and_mask_are_registered():
    from transformers import AttentionInterface
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
    from transformer_surgeon_b200 import hf_cache
    assert hf_cache.ATTN_NAME in AttentionInterface._global_mapping or hf_cache.ATTN_NAME in AttentionInterface().valid_keys()
    assert hf_cache.ATTN_NAME in ALL_MASK_ATTENTION_FUNCTIONS.valid_keys()


def test_cache_refuses_other_attention_functions():
    import transformers
    from transformer_surgeon_b200 import hf_cache
    cfg = transformers.LlamaConfig(vocab_size=64, hidden_size=128, intermediate_size=128, num_hidden_layers=1,
                                   num_attention_heads=2, num_key_value_heads=1)
    with pytest.raises(ValueError):
        hf_cache.PagedQuantCache(cfg, batch=1, max_len=32, device="cpu")
