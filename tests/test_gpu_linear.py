"""LinearCompressed.forward on the GPU against the oracle and the reference's outputs."""
import numpy as np
import pytest
import torch

from oracle import linear as olin
from oracle import weight_quant as wq

pytestmark = pytest.mark.gpu
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}
# stated tolerance: bf16 max-rel-err <= 1e-2 (relative to the largest |y|); fp32 1e-4
TOL = {"fp32": 1e-4, "bf16": 1e-2}


def rel_err(y, ref):
    return ((y.float() - ref.float()).abs().max() / ref.float().abs().max()).item()


@pytest.mark.parametrize("name", ["fp32", "bf16"])
@pytest.mark.parametrize("simt", [True, False])
def test_reference_fixture(cuda, golden, name, simt):
    from transformer_surgeon_b200 import ops
    g = golden("linear.npz")
    dt = DT[name]
    x = g[f"x_{name}"].to(cuda)
    lin = ops.PackedLinear(ops.Factor.dense(g["W"].to(dt).to(cuda)), None, g["bias"].to(dt).to(cuda), dt)
    lin.force_simt = simt
    y = lin(x)
    assert y.shape == (2, 5, 192)
    assert rel_err(y.cpu(), g[f"y_full_{name}"]) < TOL[name]
    lin = ops.PackedLinear(ops.Factor.dense(g[f"US_{name}"].to(cuda)), ops.Factor.dense(g[f"V_{name}"].to(cuda)), None, dt)
    lin.force_simt = simt
    assert rel_err(lin(x).cpu(), g[f"y_lrd_{name}"]) < TOL[name]
    for p in (8, 4, "binary"):
        fu = ops.Factor.from_codes(g[f"qu_{p}_{name}"].to(cuda), g[f"su_{p}_{name}"].to(cuda), p)
        fv = ops.Factor.from_codes(g[f"qv_{p}_{name}"].to(cuda), g[f"sv_{p}_{name}"].to(cuda), p)
        lin = ops.PackedLinear(fu, fv, None, dt)
        lin.force_simt = simt
        assert rel_err(lin(x).cpu(), g[f"y_lrd_q{p}_{name}"]) < TOL[name], (p, name)


def _case(M, K, N, r, p, name, seed=0):
    g = torch.Generator().manual_seed(seed)
    dt = DT[name]
    x = torch.randn(M, K, generator=g).to(dt)
    if r:
        U = (torch.randn(N, r, generator=g) * 0.05).to(dt)
        V = (torch.randn(r, K, generator=g) * 0.05).to(dt)
    else:
        U = (torch.randn(N, K, generator=g) * 0.05).to(dt)
        V = None
    b = (torch.randn(N, generator=g) * 0.1).to(dt)
    return x, U, V, b


@pytest.mark.parametrize("name", ["bf16", "fp32"])
@pytest.mark.parametrize("p", [8, 4, 2, "binary", None])
@pytest.mark.parametrize("M,K,N,r", [(1, 256, 192, 64), (5, 896, 128, 0), (16, 512, 320, 128), (33, 1024, 256, 0),
                                     (128, 1024, 512, 256), (200, 320, 72, 64)])
def test_against_oracle(cuda, name, p, M, K, N, r):
    from transformer_surgeon_b200 import ops
    dt = DT[name]
    x, U, V, b = _case(M, K, N, r, p, name)
    if p is None:
        fu, fv = ops.Factor.dense(U.to(cuda)), (ops.Factor.dense(V.to(cuda)) if r else None)
        Ud, Vd = U, V
    else:
        fu = ops.Factor.quantize(U.to(cuda), p)
        fv = ops.Factor.quantize(V.to(cuda), p) if r else None
        qu, su = wq.quantize_vanilla(U.float().numpy(), p, 1e-6, "per_channel", name)
        assert np.array_equal(fu.codes().cpu().numpy(), qu)
        Ud = torch.from_numpy(wq.dequantize(qu, su, name)).to(dt)
        Vd = None
        if r:
            qv, sv = wq.quantize_vanilla(V.float().numpy(), p, 1e-6, "per_channel", name)
            Vd = torch.from_numpy(wq.dequantize(qv, sv, name)).to(dt)
    ref32 = olin.linear_compressed_fp32(x, Ud, b, Vd)
    for simt in (True, False):
        lin = ops.PackedLinear(fu, fv, b.to(cuda), dt)
        lin.force_simt = simt
        y = lin(x.to(cuda)).cpu()
        assert rel_err(y, ref32) < TOL[name], (simt, rel_err(y, ref32))


@pytest.mark.parametrize("p", [4, 8, "binary"])
@pytest.mark.parametrize("M,K,N,r", [(300, 2048, 1000, 0),      # two 256-token tiles (one ragged), 8-way split-K, ragged row tile
                                     (700, 1024, 2052, 256),    # N not a multiple of 8: outputs leave as single elements
                                     (257, 4096, 136, 1024),    # one token past a tile, 18-way split-K then 4-way
                                     (1024, 512, 4096, 0),      # no split-K, several items per CTA
                                     (129, 832, 264, 0)])       # K not a multiple of the k-block pair
def test_prompt_sized_token_counts(cuda, p, M, K, N, r):
    """More than 128 tokens: the 256-token tile with its transposed 16-byte output stores, every split-K batch
    shape, ragged tiles in both directions; bf16, max-rel-err <= 1e-2 against the fp32 result on the dequantized
    factors, and a second identical call returns the same bits."""
    from transformer_surgeon_b200 import ops
    x, U, V, b = _case(M, K, N, r, p, "bf16", seed=5)
    fu = ops.Factor.quantize(U.to(cuda), p)
    fv = ops.Factor.quantize(V.to(cuda), p) if r else None
    Ud = fu.reconstruct(torch.bfloat16).cpu()
    Vd = fv.reconstruct(torch.bfloat16).cpu() if r else None
    ref32 = olin.linear_compressed_fp32(x, Ud, b, Vd)
    lin = ops.PackedLinear(fu, fv, b.to(cuda), torch.bfloat16)
    y = lin(x.to(cuda))
    assert rel_err(y.cpu(), ref32) < TOL["bf16"], rel_err(y.cpu(), ref32)
    # element-wise: no output may be missing or misplaced (a max-error bound alone would let a zero row through)
    err = (y.cpu().float() - ref32.float()).abs()
    assert (err <= 2e-2 * ref32.float().abs() + 1e-2 * ref32.float().abs().max()).all()
    assert torch.equal(lin(x.to(cuda)), y)


def test_config2_shape_sweep(cuda):
    """x [M, 4096], W 4096x4096 factored at r in {256, 1024}, 8/4-bit + binary factors, bf16:
    compared with the dequantized fp32 result (max-rel-err <= 1e-2)."""
    from transformer_surgeon_b200 import ops
    g = torch.Generator().manual_seed(2)
    for r in (256, 1024):
        U = (torch.randn(4096, r, generator=g) * 0.02).bfloat16().to(cuda)
        V = (torch.randn(r, 4096, generator=g) * 0.02).bfloat16().to(cuda)
        for p in (8, 4, "binary"):
            fu, fv = ops.Factor.quantize(U, p), ops.Factor.quantize(V, p)
            Ud, Vd = fu.reconstruct(torch.bfloat16).float(), fv.reconstruct(torch.bfloat16).float()
            lin = ops.PackedLinear(fu, fv, None, torch.bfloat16)
            for M in (1, 16, 128, 2048):
                x = torch.randn(M, 4096, generator=g).bfloat16().to(cuda)
                ref = (x.float() @ Vd.T) @ Ud.T
                y = lin(x)
                assert rel_err(y, ref) < 1e-2, (r, p, M, rel_err(y, ref))


def test_linearity_and_leading_shape(cuda):
    from transformer_surgeon_b200 import ops
    x, U, V, b = _case(6, 512, 128, 64, 4, "fp32")
    lin = ops.PackedLinear(ops.Factor.quantize(U.to(cuda), 4), ops.Factor.quantize(V.to(cuda), 4), None, torch.float32)
    xa = x.to(cuda)
    y1 = lin(xa)
    y2 = lin((2.0 * xa).reshape(2, 3, 512)).reshape(6, 128)
    torch.testing.assert_close(2.0 * y1, y2, rtol=1e-5, atol=1e-5)
    assert lin(xa[:0]).shape == (0, 128)


@pytest.mark.parametrize("name", ["bf16", "fp32"])
@pytest.mark.parametrize("p", [8, 4, None])
@pytest.mark.parametrize("M,K,I,r,N", [(32, 512, 7168, 256, 512), (12, 512, 7168, 0, 384), (32, 256, 640, 64, 256), (5, 256, 640, 64, 256)])
def test_gated_mlp_block(cuda, name, p, M, K, I, r, N):
    """MLPGated.forward (blocks/mlp.py:171-185): fused one-launch path (wide intermediate, bf16, 9<=M<=64)
    and the composed path, against the oracle's silu(gate)*up -> down in fp32 from the dequantized factors."""
    from transformer_surgeon_b200 import ops
    from oracle import attention as oatt
    dt = DT[name]
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, K, generator=g).to(dt)

    def layer(out, inn, rank, bias):
        U = (torch.randn(out, rank or inn, generator=g) * (0.5 / (rank or inn) ** 0.5)).to(dt)
        V = (torch.randn(rank, inn, generator=g) * (1.0 / inn ** 0.5)).to(dt) if rank else None
        b = (torch.randn(out, generator=g) * 0.1).to(dt) if bias else None
        if p is None:
            fu, fv = ops.Factor.dense(U.to(cuda)), (ops.Factor.dense(V.to(cuda)) if rank else None)
        else:
            fu, fv = ops.Factor.quantize(U.to(cuda), p), (ops.Factor.quantize(V.to(cuda), p) if rank else None)
        lin = ops.PackedLinear(fu, fv, None if b is None else b.to(cuda), dt)
        Ud = fu.reconstruct(dt).float().cpu()
        Vd = fv.reconstruct(dt).float().cpu() if rank else None
        return lin, (Ud, Vd, None if b is None else b.float())

    gate, gw = layer(I, K, r, True)
    up, uw = layer(I, K, r, False)
    down, dw = layer(N, I, r, True)

    def ref_lin(t, w):
        U, V, b = w
        h = t @ V.T if V is not None else t
        y = h @ U.T
        return y + b if b is not None else y

    ref = ref_lin(oatt.swiglu(ref_lin(x.float(), gw), ref_lin(x.float(), uw)), dw)
    mlp = ops.GatedMLP(gate, up, down)
    y = mlp(x.to(cuda))
    y2 = mlp(x.to(cuda))
    if p is None:       # dense factors: the bf16 kernel adds its K splits with fp32 atomics (order varies)
        assert rel_err(y, y2) < 1e-2
    else:               # packed factors: deterministic split-K, workspace left clean
        assert torch.equal(y, y2)
    assert rel_err(y.cpu(), ref) < (2e-2 if name == "bf16" else 1e-4), rel_err(y.cpu(), ref)
    # identical to composing the public pieces
    yc = down(ops.swiglu(gate(x.to(cuda)), up(x.to(cuda))))
    assert rel_err(y, yc) < (1e-2 if name == "bf16" else 1e-5)
    assert ops.PackedLinear.device_status(ws=ops.workspace(cuda, 1, "mlp")) == 0


@pytest.mark.parametrize("p", [4, 8, 2, "binary"])
@pytest.mark.parametrize("M,K,N,r", [(32, 4096, 4096, 0),        # o_proj
                                     (32, 4096, 6144, 0),        # q|k|v
                                     (7, 3584, 4608, 0),         # config-5 q|k|v
                                     (16, 4096, 14336, 1024),    # low-rank pair
                                     (32, 14336, 4096, 1024),    # down_proj: long K
                                     (32, 1792, 200, 0),         # rows not a multiple of 16 / 8
                                     (3, 896, 72, 64)])          # K tail, tiny N
def test_few_tokens_at_model_widths(cuda, p, M, K, N, r):
    """Packed linears at decode token counts and the widths of the benchmark models (split-K over many CTAs, odd
    row counts, K tails): against the fp32 oracle on the dequantized factors (bf16: max-rel-err <= 1e-2); the
    result must not change from run to run (fixed summation order)."""
    from transformer_surgeon_b200 import ops
    g = torch.Generator(device=cuda).manual_seed(31)
    rnd = lambda a, b, s: (torch.randn((a, b), generator=g, device=cuda) * s).bfloat16()
    if r:
        fu, fv = ops.Factor.quantize(rnd(N, r, 0.05), p), ops.Factor.quantize(rnd(r, K, 0.05), p)
    else:
        fu, fv = ops.Factor.quantize(rnd(N, K, 0.05), p), None
    bias = rnd(1, N, 0.1)[0].contiguous()
    lin = ops.PackedLinear(fu, fv, bias, torch.bfloat16)
    x = rnd(M, K, 1.0)
    Ud = fu.reconstruct(torch.bfloat16).float()
    h = x.float() @ fv.reconstruct(torch.bfloat16).float().T if r else x.float()
    ref = h @ Ud.T + bias.float()
    y = lin(x)
    y2 = lin(x)
    assert torch.equal(y, y2)
    assert rel_err(y, ref) < 1e-2, rel_err(y, ref)
    assert ops.PackedLinear.device_status(device=cuda) == 0


@pytest.mark.parametrize("M,K,N", [(1, 512, 1000), (32, 1024, 50257), (100, 256, 4099)])
def test_greedy_head_equals_argmax_of_logits(cuda, M, K, N):
    """tsb200_linear_argmax on a dense bf16 head (reduction in the GEMM epilogue, logits never stored) picks the token
    torch.argmax picks from tsb200_linear's logits - including ties, which go to the first maximum."""
    from transformer_surgeon_b200 import ops
    g = torch.Generator(device=cuda).manual_seed(41)
    W = (torch.randn((N, K), generator=g, device=cuda) * 0.05).bfloat16()
    W[N - 3] = W[7]                                      # duplicated rows: their logits tie exactly
    W[N // 2] = W[7]
    b = (torch.randn(N, generator=g, device=cuda) * 0.1).bfloat16()
    b[N - 3] = b[7]
    b[N // 2] = b[7]
    x = torch.randn((M, K), generator=g, device=cuda).bfloat16()
    x[0] = W[7].float().sign().bfloat16()                # make row 7 (and its copies) the winner for token 0
    lin = ops.PackedLinear(ops.Factor.dense(W), None, b, torch.bfloat16)
    logits = lin(x)
    toks = lin.argmax(x)
    assert torch.equal(toks, torch.argmax(logits, dim=-1))
    assert int(toks[0]) == 7
    assert torch.equal(lin.argmax(x), toks)


def test_greedy_head_general_route(cuda):
    """A packed low-rank head and an fp32 head: logits into the workspace, then the library's own argmax kernel."""
    from transformer_surgeon_b200 import ops
    g = torch.Generator(device=cuda).manual_seed(42)
    U = (torch.randn((3000, 64), generator=g, device=cuda) * 0.05).bfloat16()
    V = (torch.randn((64, 256), generator=g, device=cuda) * 0.05).bfloat16()
    lin = ops.PackedLinear(ops.Factor.quantize(U, 4), ops.Factor.quantize(V, 4), None, torch.bfloat16)
    x = torch.randn((9, 256), generator=g, device=cuda).bfloat16()
    assert torch.equal(lin.argmax(x), torch.argmax(lin(x), dim=-1))
    W = torch.randn((777, 96), generator=g, device=cuda)
    lin32 = ops.PackedLinear(ops.Factor.dense(W), None, None, torch.float32)
    x32 = torch.randn((5, 96), generator=g, device=cuda)
    assert torch.equal(lin32.argmax(x32), torch.argmax(lin32(x32), dim=-1))


def test_split_k_launches_repeat_bit_for_bit(cuda):
    """The split-K exchange (slices in global memory, one fence by the signalling thread, acquire polling, wrap-around
    tile counters) and the grid barriers of the fused MLP under programmatic dependent launch: 600 back-to-back
    launches per shape on cycling weights give the same bits every time, and no bounded wait runs out."""
    from transformer_surgeon_b200 import ops
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(13)

    def lin(out, inn, rank):
        U = (torch.randn(out, rank or inn, generator=g) * 0.05).to(dt).to(cuda)
        V = (torch.randn(rank, inn, generator=g) * 0.05).to(dt).to(cuda) if rank else None
        return ops.PackedLinear(ops.Factor.quantize(U, 4), ops.Factor.quantize(V, 4) if rank else None, None, dt)

    x = torch.randn(32, 4096, generator=g).to(dt).to(cuda)
    qkv = [lin(6144, 4096, 0) for _ in range(3)]                       # 48 tiles x 3 splits
    o = [lin(4096, 4096, 0) for _ in range(3)]                         # 32 tiles x 4 splits
    mlp = [ops.GatedMLP(lin(7168, 4096, 512), lin(7168, 4096, 512), lin(4096, 7168, 512)) for _ in range(2)]   # four phases
    old = ops.set_pdl(True)
    try:
        for layers in (qkv, o, mlp):
            refs = [L(x) for L in layers]
            outs = [torch.empty_like(r) for r in refs]
            bad = torch.zeros((), dtype=torch.int64, device=cuda)
            for it in range(600 // len(layers)):
                for L, out in zip(layers, outs):
                    L(x, out=out)
                if it % 4 == 3:
                    for out, r in zip(outs, refs):
                        bad += (out != r).any()
            torch.cuda.synchronize()
            assert int(bad.item()) == 0
    finally:
        ops.set_pdl(old)
    assert ops.PackedLinear.device_status(device=x.device) == 0
