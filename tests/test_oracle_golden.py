"""The oracle against the fixtures produced by the reference itself (tests/golden/)."""
import numpy as np
import pytest
import torch

from oracle import weight_quant as wq
from oracle import linear as olin
from oracle import attention as oatt

DT = {"fp32": torch.float32, "bf16": torch.bfloat16}


@pytest.mark.parametrize("name", ["fp32", "bf16"])
@pytest.mark.parametrize("p", [8, 4, 2, "binary"])
@pytest.mark.parametrize("gran", ["per_channel", "per_tensor"])
def test_weight_quant_bit_exact(golden, name, p, gran):
    g = golden("weight_quant.npz")
    w = g[f"w_{name}"].float().numpy()
    tag = f"{name}_{p}_{gran}"
    q, s = wq.quantize_vanilla(w, p, 1e-6, gran, name)
    assert np.array_equal(q, g[f"q_{tag}"].numpy())
    s_ref = g[f"s_{tag}"].float().numpy().reshape(-1)
    s_mine = np.broadcast_to(s.reshape(-1), s_ref.shape) if s.size == 1 else s.reshape(-1)
    if p == "binary" and name == "fp32":
        # torch's fp32 cascade sum vs a correctly rounded mean: at most 1 ulp apart
        assert np.allclose(s_mine, s_ref, rtol=2e-7, atol=0)
    else:
        assert np.array_equal(s_mine, s_ref)
        assert np.array_equal(wq.dequantize(q, s, name), g[f"deq_{tag}"].float().numpy())
    bits = wq.container_bits(p, q)
    assert np.array_equal(wq.unpack_codes(wq.pack_codes(q, bits), bits, q.shape[1]), q)


def test_binary_with_zero_needs_two_bits(golden):
    g = golden("weight_quant.npz")
    q = g["q_fp32_binary_per_channel"].numpy()
    assert (q == 0).any() and wq.container_bits("binary", q) == 2
    assert wq.container_bits("binary", np.ones((2, 2), np.int8)) == 1


@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_linear_forward(golden, name):
    g = golden("linear.npz")
    dt = DT[name]
    x = g[f"x_{name}"]
    y = olin.linear_compressed_forward(x, g["W"].to(dt), g["bias"].to(dt))
    assert torch.equal(y, g[f"y_full_{name}"])
    y = olin.linear_compressed_forward(x, g[f"US_{name}"], None, g[f"V_{name}"])
    assert torch.equal(y, g[f"y_lrd_{name}"])
    for p in (8, 4, "binary"):
        U = torch.from_numpy(wq.dequantize(g[f"qu_{p}_{name}"].numpy(), g[f"su_{p}_{name}"].float().numpy()[:, None], name)).to(dt)
        V = torch.from_numpy(wq.dequantize(g[f"qv_{p}_{name}"].numpy(), g[f"sv_{p}_{name}"].float().numpy()[:, None], name)).to(dt)
        y = olin.linear_compressed_forward(x, U, None, V)
        assert torch.equal(y, g[f"y_lrd_q{p}_{name}"])
        # codes captured by the reference are reproduced from its pre-quant factors
        q2, s2 = wq.quantize_vanilla(g[f"US_{name}"].float().numpy(), p, 1e-6, "per_channel", name)
        assert np.array_equal(q2, g[f"qu_{p}_{name}"].numpy())


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_attention(golden, tag):
    g = golden("blocks.npz")
    q, k, v = g[f"att_{tag}_q"], g[f"att_{tag}_k"], g[f"att_{tag}_v"]
    torch.testing.assert_close(oatt.attention(q, k, v), g[f"att_{tag}_o"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(oatt.attention(q, k, v, g[f"att_{tag}_mask"]), g[f"att_{tag}_om"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_rope_and_norm(golden, name):
    g = golden("blocks.npz")
    cos, sin = oatt.rope_tables(64, 1e6, torch.arange(40))
    assert torch.equal(cos, g["rope_cos"]) and torch.equal(sin, g["rope_sin"])
    y = oatt.apply_rope(g[f"rope_x_{name}"], cos, sin)
    assert torch.equal(y, g[f"rope_y_{name}"])
    y = oatt.rmsnorm_blocks(g[f"norm_x_{name}"], g[f"norm_w_{name}"])
    assert torch.equal(y, g[f"norm_y_{name}"])


def test_mlp_gated(golden):
    g = golden("blocks.npz")
    x = g["mlp_x"]
    lin = lambda n, t: olin.linear_compressed_forward(t, g[f"mlp_{n}_w"], g.get(f"mlp_{n}_b"))
    y = lin("down_proj", oatt.swiglu(lin("gate_proj", x), lin("up_proj", x)))
    torch.testing.assert_close(y, g["mlp_y"], rtol=1e-6, atol=1e-6)
