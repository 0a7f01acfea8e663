"""Prompt (prefill) attention: tsb200_kv_gather_heads + tsb200_prefill_attn (tcgen05, bf16) and the fp32 route
through the paged decode kernel, against the oracle's attention() (oracle/attention.py, pinned to the reference's
blocks/mha.py:9-103 by tests/test_oracle_golden.py) over the dequantized cache with the causal mask the reference's
models apply.  KV formats are this project's definitions (parity unpinned for them); unquantized bf16 / fp32 pages
hold the appended values themselves."""
import numpy as np
import pytest
import torch

from oracle import attention as oatt

pytestmark = pytest.mark.gpu


def reference(q, K, V, L):
    """q [T, H, d], K, V [L, hkv, d] fp32 -> (out, out_abs) [T, H, d]: attention() with the causal penalty the
    reference adds (query i at position L - T + i), and the same weights applied to |V| (error scale)."""
    T = q.shape[0]
    pos = torch.arange(L - T, L)[:, None]
    mask = torch.where(torch.arange(L)[None, :] > pos, float("-inf"), 0.0)[None]          # [1, T, L]
    out = oatt.attention(q, K, V, mask).transpose(0, 1)
    out_abs = oatt.attention(q, K, V.abs(), mask).transpose(0, 1)
    return out, out_abs


def setup(cuda, fmt, B, L, H, Hkv, d, dtype, seed):
    from transformer_surgeon_b200 import ops
    g = torch.Generator(device=cuda).manual_seed(seed)
    pages = (L + 15) // 16 + 1
    bt = torch.randperm(B * pages, generator=g, device=cuda).to(torch.int32).reshape(B, pages)
    seq = torch.zeros(B, dtype=torch.int32, device=cuda)
    kv = ops.PagedKV(fmt, B * pages, Hkv, d, bt, seq, cuda)
    k = torch.randn((B, L, Hkv, d), generator=g, device=cuda).to(dtype)
    v = torch.randn((B, L, Hkv, d), generator=g, device=cuda).to(dtype)
    v[:, :, :, 3] *= 20                                  # an outlier channel
    if fmt == "fp8":
        kv.set_fp8_scales(k, v)
    kv.append(k, v)
    seq += L
    return ops, kv, g


@pytest.mark.parametrize("T,L", [(17, 17), (128, 128), (300, 300), (2048, 2048), (100, 356), (129, 1000)])
@pytest.mark.parametrize("H,Hkv,d", [(8, 2, 128), (7, 1, 128), (4, 2, 64)])
def test_prefill_attention_bf16_against_oracle(cuda, T, L, H, Hkv, d):
    """Whole prompts (L == T) and later chunks (L > T), GQA groups of 4 / 7 / 2, head sizes 128 / 64; bf16 pages."""
    B = 2
    ops, kv, g = setup(cuda, "bf16", B, L, H, Hkv, d, torch.bfloat16, 50 + T)
    q = torch.randn((B, T, H, d), generator=g, device=cuda).bfloat16()
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    out = ops.prefill_attention(kv, q, L, status=st).float().cpu()
    assert int(st.item()) == 0
    kd, vd = ops.kv_gather(kv, L, dtype=torch.float32)
    for b in range(B):
        ref, ref_abs = reference(q[b].float().cpu(), kd[b].cpu(), vd[b].cpu(), L)
        tol = 1e-2 * ref_abs + 4e-3 * ref.abs() + 1e-5         # P and the output are rounded to bf16
        assert torch.all((out[b] - ref).abs() <= tol), ((out[b] - ref).abs() / tol).max()


@pytest.mark.parametrize("fmt", ["int8", "fp8", "nvfp4"])
def test_prefill_attention_reads_dequantized_pages(cuda, fmt):
    """Quantized pages: the kernel attends over exactly the values the dequantizing gather returns."""
    B, T, L, H, Hkv, d = 2, 200, 264, 8, 2, 128
    ops, kv, g = setup(cuda, fmt, B, L, H, Hkv, d, torch.bfloat16, 71)
    q = torch.randn((B, T, H, d), generator=g, device=cuda).bfloat16()
    out = ops.prefill_attention(kv, q, L).float().cpu()
    kd, vd = ops.kv_gather(kv, L, dtype=torch.float32)
    for b in range(B):
        ref, ref_abs = reference(q[b].float().cpu(), kd[b].bfloat16().float().cpu(), vd[b].bfloat16().float().cpu(), L)
        tol = 1e-2 * ref_abs + 4e-3 * ref.abs() + 1e-5
        assert torch.all((out[b] - ref).abs() <= tol), ((out[b] - ref).abs() / tol).max()


def test_prefill_attention_fp32_route(cuda):
    """fp32 activations: every query token runs as a one-token sequence of the paged decode kernel (fp32 math)."""
    B, T, L, H, Hkv, d = 2, 37, 53, 4, 2, 64
    ops, kv, g = setup(cuda, "fp32", B, L, H, Hkv, d, torch.float32, 72)
    q = torch.randn((B, T, H, d), generator=g, device=cuda)
    out = ops.prefill_attention(kv, q, L).cpu()
    kd, vd = ops.kv_gather(kv, L, dtype=torch.float32)
    for b in range(B):
        ref, ref_abs = reference(q[b].cpu(), kd[b].cpu(), vd[b].cpu(), L)
        assert torch.all((out[b] - ref).abs() <= 2e-4 * ref_abs + 1e-5 * ref.abs() + 1e-6)


def test_prefill_attention_strided_q_and_argument_errors(cuda):
    from transformer_surgeon_b200 import Tsb200Error
    B, T, L, H, Hkv, d = 1, 64, 64, 4, 2, 128
    ops, kv, g = setup(cuda, "bf16", B, L, H, Hkv, d, torch.bfloat16, 73)
    qkv = torch.randn((B, T, (H + 2 * Hkv) * d), generator=g, device=cuda).bfloat16()
    q = qkv[:, :, :H * d].unflatten(2, (H, d))                   # a column slice of a fused projection output
    out = ops.prefill_attention(kv, q, L)
    assert torch.equal(out, ops.prefill_attention(kv, q.contiguous(), L))
    with pytest.raises(Tsb200Error):
        ops.prefill_attention(kv, q.contiguous(), L - 1)         # fewer cached positions than query tokens
