"""GPU weight quantize / pack / unpack / reconstruct: bit-exact against the oracle and the
reference's own outputs (tests/golden/weight_quant.npz)."""
import numpy as np
import pytest
import torch

from oracle import weight_quant as wq

pytestmark = pytest.mark.gpu
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}


@pytest.mark.parametrize("name", ["fp32", "bf16"])
@pytest.mark.parametrize("p", [8, 4, 2, "binary"])
@pytest.mark.parametrize("gran", ["per_channel", "per_tensor"])
def test_quantize_matches_reference_fixture(cuda, golden, name, p, gran):
    from transformer_surgeon_b200 import ops
    g = golden("weight_quant.npz")
    w = g[f"w_{name}"].to(cuda)
    tag = f"{name}_{p}_{gran}"
    codes, scales = ops.quantize_weight(w, p, gran, 1e-6)
    assert torch.equal(codes.cpu(), g[f"q_{tag}"])
    s_ref = g[f"s_{tag}"].float().reshape(-1)
    s_ref = s_ref.expand(w.shape[0]) if s_ref.numel() == 1 else s_ref
    if p == "binary" and name == "fp32":
        torch.testing.assert_close(scales.cpu(), s_ref, rtol=2e-7, atol=0)
    else:
        assert torch.equal(scales.cpu(), s_ref)
    # pack -> unpack -> reconstruct
    f = ops.Factor.from_codes(codes, scales, p)
    assert f.bits == wq.container_bits(p, g[f"q_{tag}"].numpy())
    assert torch.equal(f.codes().cpu(), g[f"q_{tag}"])
    packed_ref = wq.pack_codes(g[f"q_{tag}"].numpy(), f.bits)
    assert np.array_equal(f.data.cpu().numpy(), packed_ref)
    if not (p == "binary" and name == "fp32"):
        assert torch.equal(f.reconstruct(DT[name]).cpu(), g[f"deq_{tag}"])


@pytest.mark.parametrize("name", ["fp32", "bf16"])
@pytest.mark.parametrize("p", [8, 4, 3, 2])
def test_quantize_large_matrix_against_oracle(cuda, name, p):
    """Config-2 sized factor (4096 x 1024): codes and scales bit-exact against the oracle."""
    from transformer_surgeon_b200 import ops
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(4096, 1024, generator=g) * 0.02).to(DT[name])
    w[17] = 0
    codes, scales = ops.quantize_weight(w.to(cuda), p, "per_channel")
    q, s = wq.quantize_vanilla(w.float().numpy(), p, 1e-6, "per_channel", name)
    assert np.array_equal(codes.cpu().numpy(), q)
    assert np.array_equal(scales.cpu().numpy(), s[:, 0])
    f = ops.Factor.from_codes(codes, scales, p)
    assert np.array_equal(f.reconstruct(DT[name]).float().cpu().numpy(), wq.dequantize(q, s, name))


def test_ragged_columns_and_empty(cuda):
    from transformer_surgeon_b200 import ops
    w = torch.randn(7, 100).to(cuda)                       # 100 columns -> padded to 128
    for p, bits in ((8, 8), (4, 4), (2, 2)):
        codes, scales = ops.quantize_weight(w, p)
        q, s = wq.quantize_vanilla(w.cpu().numpy(), p, 1e-6, "per_channel", "fp32")
        assert np.array_equal(codes.cpu().numpy(), q)
        packed, _ = ops.pack_codes(codes, bits)
        assert np.array_equal(packed.cpu().numpy(), wq.pack_codes(q, bits))
        assert torch.equal(ops.unpack_codes(packed, 7, 100, bits), codes)
    e = torch.empty((0, 64), device=cuda)
    codes, scales = ops.quantize_weight(e, 8)
    assert codes.shape == (0, 64)


def test_bad_arguments_are_rejected(cuda):
    from transformer_surgeon_b200 import ops, Tsb200Error
    w = torch.randn(4, 64, device=cuda)
    with pytest.raises(ValueError):
        ops.quantize_weight(w, 9)
    with pytest.raises(ValueError):
        ops.quantize_weight(w.cpu(), 8)
    with pytest.raises(Tsb200Error):
        ops.pack_codes(torch.zeros((4, 64), dtype=torch.int8, device=cuda), 3)
