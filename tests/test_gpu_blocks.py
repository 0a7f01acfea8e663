"""RoPE, RMSNorm (+ residual add) and SwiGLU kernels against the reference fixtures / oracle."""
import pytest
import torch

from oracle import attention as oatt

pytestmark = pytest.mark.gpu
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}


@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_rope_matches_reference(cuda, golden, name):
    from transformer_surgeon_b200 import ops
    g = golden("blocks.npz")
    x = g[f"rope_x_{name}"].to(cuda).unsqueeze(0).contiguous()      # [1, 40, 3, 64]
    cos, sin = g["rope_cos"].to(cuda), g["rope_sin"].to(cuda)
    y = ops.rope_(x.clone(), cos, sin)
    assert torch.equal(y[0].cpu(), g[f"rope_y_{name}"])             # bit-exact: same rounding points
    # per-sequence start positions: decode-style [B, 1, heads, d]
    xb = g[f"rope_x_{name}"][:8].to(cuda).reshape(8, 1, 3, 64).contiguous()
    pos0 = torch.arange(8, dtype=torch.int32, device=cuda)
    y = ops.rope_(xb.clone(), cos, sin, pos0)
    assert torch.equal(y.reshape(8, 3, 64).cpu(), g[f"rope_y_{name}"][:8])


@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_rmsnorm_variants(cuda, golden, name):
    from transformer_surgeon_b200 import ops
    g = golden("blocks.npz")
    x, w = g[f"norm_x_{name}"], g[f"norm_w_{name}"]
    y = ops.add_rmsnorm(x.to(cuda).clone(), None, w.to(cuda), variant=1)
    tol = dict(rtol=2e-2, atol=2e-2) if name == "bf16" else dict(rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(y.cpu(), g[f"norm_y_{name}"], **tol)
    # Hugging Face variant with a residual add
    gen = torch.Generator().manual_seed(3)
    d = torch.randn(x.shape, generator=gen).to(x.dtype)
    res = x.to(cuda).clone()
    y = ops.add_rmsnorm(res, d.to(cuda), w.to(cuda), eps=1e-6, variant=0)
    s = x + d
    assert torch.equal(res.cpu(), s)
    torch.testing.assert_close(y.cpu(), oatt.rmsnorm_hf(s, w, 1e-6), **tol)


@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_swiglu(cuda, name):
    from transformer_surgeon_b200 import ops
    gen = torch.Generator().manual_seed(4)
    gu = (torch.randn(9, 2 * 160, generator=gen) * 2).to(DT[name])
    y = ops.swiglu(gu.to(cuda)[:, :160], gu.to(cuda)[:, 160:])
    ref = oatt.swiglu(gu[:, :160], gu[:, 160:])
    tol = dict(rtol=1e-2, atol=1e-2) if name == "bf16" else dict(rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(y.cpu(), ref, **tol)


def test_swiglu_prompt_sized_equals_elementwise_form(cuda):
    """Prompt-sized bf16 calls take the 16-byte form of the kernel: the same bits as the element-wise form (reached
    through rows that are not 16-byte aligned), column slices of one [M, 2n] buffer included."""
    from transformer_surgeon_b200 import ops
    gen = torch.Generator().manual_seed(5)
    M, n = 300, 2048
    gu = (torch.randn(M, 2 * n, generator=gen) * 3).bfloat16().to(cuda)
    y = ops.swiglu(gu[:, :n], gu[:, n:])                                  # aligned rows: 16-byte form
    wide = torch.zeros((M, 2 * n + 2), dtype=torch.bfloat16, device=cuda)  # row starts 4 bytes off: element-wise form
    wide[:, 1:2 * n + 1] = gu
    y_ref = ops.swiglu(wide[:, 1:n + 1], wide[:, n + 1:2 * n + 1])
    assert torch.equal(y, y_ref)
    ref = oatt.swiglu(gu[:, :n].cpu(), gu[:, n:].cpu())
    torch.testing.assert_close(y.cpu(), ref, rtol=1e-2, atol=1e-2)
