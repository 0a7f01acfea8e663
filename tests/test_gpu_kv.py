"""Quantized paged KV cache on the GPU: append is bit-exact against the oracle (codes,
scales, page placement); decode attention is within tolerance of the oracle's fp32
attention over the dequantized cache; full-size cases are covered by properties."""
import numpy as np
import pytest
import torch

from oracle import kv_cache as kc
from oracle import attention as oatt

pytestmark = pytest.mark.gpu
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}
FMTS = ["int8", "fp8", "nvfp4"]
# Decode-attention tolerance, per output element e of head h:
#     |out - oracle| <= C_P * sum_t p_t |V_t,e|  +  C_OUT * |oracle|
# The first term is the element's own error scale (softmax weights applied to |V|, from the oracle): an
# outlier channel (values x20) gets a 20x larger allowance than a normal channel, and no element borrows the
# allowance of another.  C_P covers the relative error of the softmax weights: q and P pass through f16
# (2^-11) or three e4m3 terms (2^-12) in the tensor-core kernels, and the score error of a d=128 dot
# product with outlier channels reaches ~1e-2 before the exponential.  The CUDA-core kernel computes in
# fp32 on the dequantized values.  C_OUT is the rounding of the stored output (bf16: 2^-9).
C_P_TC, C_P_SIMT = 2e-2, 2e-4
C_OUT = {"fp32": 1e-5, "bf16": 4e-3}


def attn_tol(ref, ref_abs, name, simt):
    return (C_P_SIMT if simt else C_P_TC) * ref_abs + C_OUT[name] * np.abs(ref) + 1e-6


def outlier_kv(rng, B, T, Hkv, d, dtype):
    """N(0,1) with 4 outlier channels per head scaled x20 (the config-3 distribution)."""
    k = rng.standard_normal((B, T, Hkv, d)).astype(np.float32)
    v = rng.standard_normal((B, T, Hkv, d)).astype(np.float32)
    for h in range(Hkv):
        ch = rng.choice(d, 4, replace=False)
        k[:, :, h, ch] *= 20
        v[:, :, h, ch] *= 20
    kt, vt = torch.from_numpy(k).to(dtype), torch.from_numpy(v).to(dtype)
    return kt, vt


def make_pair(fmt, B, pages_per_seq, Hkv, d, dev, rng, extra_pages=3):
    npg = B * pages_per_seq + extra_pages
    bt = rng.permutation(npg)[:B * pages_per_seq].reshape(B, pages_per_seq).astype(np.int32)
    from transformer_surgeon_b200 import ops
    o = kc.PagedKV(kc.FMT_NAMES[fmt], npg, Hkv, d, bt, B)
    seq = torch.zeros(B, dtype=torch.int32, device=dev)
    g = ops.PagedKV(fmt, npg, Hkv, d, torch.from_numpy(bt).to(dev), seq, dev)
    return o, g


def sync_scales(o, g, k, v, rope=None):
    if o.fmt == kc.FMT_FP8:
        g.set_fp8_scales(k.to(g.k_pool.device), v.to(g.k_pool.device), rope=rope, pos0=g.seq_lens if rope else None)
        o.k_scale[:] = g.k_scale.cpu().numpy()
        o.v_scale[:] = g.v_scale.cpu().numpy()


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("name", ["fp32", "bf16"])
@pytest.mark.parametrize("d", [64, 128])
def test_append_bit_exact(cuda, fmt, name, d):
    rng = np.random.default_rng(10)
    B, T, Hkv = 3, 37, 2
    o, g = make_pair(fmt, B, 4, Hkv, d, cuda, rng)
    k, v = outlier_kv(rng, B, T, Hkv, d, DT[name])
    sync_scales(o, g, k, v)
    if fmt == "fp8":   # scale kernel: amax/448 exactly
        ref = kc.fp8_scale_from_amax(k.float().abs().amax(dim=(1, 3)).numpy())
        assert np.array_equal(o.k_scale, ref)
    # prompt in one bulk append, then 5 single-token decode appends
    g.append(k.to(cuda), v.to(cuda))
    g.seq_lens += T
    kc.append_vectorized(o, k.float().numpy(), v.float().numpy())
    for step in range(5):
        k1, v1 = outlier_kv(rng, B, 1, Hkv, d, DT[name])
        g.append(k1.to(cuda), v1.to(cuda))
        g.seq_lens += 1
        o.append(k1.float().numpy(), v1.float().numpy())
    assert np.array_equal(g.k_pool.cpu().numpy(), o.k_pool)
    assert np.array_equal(g.v_pool.cpu().numpy(), o.v_pool)
    assert g.seq_lens.cpu().tolist() == o.seq_lens.tolist()


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_append_with_fused_rope_and_ragged_lengths(cuda, fmt, name):
    rng = np.random.default_rng(11)
    B, T, Hkv, d = 4, 21, 2, 128
    o, g = make_pair(fmt, B, 3, Hkv, d, cuda, rng)
    cos, sin = oatt.rope_tables(d, 5e5, torch.arange(64))
    k, v = outlier_kv(rng, B, T, Hkv, d, DT[name])
    new_lens = np.array([21, 0, 7, 16], dtype=np.int32)
    start = np.array([3, 0, 16, 5], dtype=np.int32)          # sequences already hold some tokens
    o.seq_lens[:] = start
    g.seq_lens.copy_(torch.from_numpy(start))
    rope = (cos.to(cuda), sin.to(cuda))
    sync_scales(o, g, k, v, rope=rope)
    g.append(k.to(cuda), v.to(cuda), new_lens=torch.from_numpy(new_lens).to(cuda), rope=rope)
    # oracle: rotate with the same rounding points, then append
    pos = torch.from_numpy(start.astype(np.int64))[:, None] + torch.arange(T)[None, :]
    kr = torch.stack([oatt.apply_rope(k[b], cos[pos[b]], sin[pos[b]]) for b in range(B)])
    if fmt == "fp8":
        ref = kc.fp8_scale_from_amax(kr.float().abs().amax(dim=(1, 3)).numpy())
        assert np.array_equal(o.k_scale, ref)
    o.append(kr.float().numpy(), v.float().numpy(), new_lens=new_lens)
    assert np.array_equal(g.k_pool.cpu().numpy(), o.k_pool)
    assert np.array_equal(g.v_pool.cpu().numpy(), o.v_pool)


def test_append_empty_and_overflow(cuda):
    from transformer_surgeon_b200 import ops
    rng = np.random.default_rng(12)
    o, g = make_pair("int8", 2, 1, 2, 64, cuda, rng)
    e = torch.empty((2, 0, 2, 64), device=cuda)
    g.append(e, e)                                             # T == 0: no-op
    k, v = outlier_kv(rng, 2, 20, 2, 64, torch.float32)        # 20 tokens but only one page each
    g.append(k.to(cuda), v.to(cuda))
    o.append(k[:, :16].numpy(), v[:, :16].numpy())             # positions >= 16 are skipped
    assert np.array_equal(g.k_pool.cpu().numpy(), o.k_pool)


@pytest.mark.parametrize("fmt", FMTS + ["fp32", "bf16"])
@pytest.mark.parametrize("d", [64, 128])
def test_gather_dequantizes_bit_exact(cuda, fmt, d):
    """tsb200_kv_gather == the oracle's dequantized cache, element for element (fp32 output), with
    ragged lengths, an empty sequence and zeros beyond each length."""
    from transformer_surgeon_b200 import ops
    rng = np.random.default_rng(21)
    B, Hkv = 4, 2
    lens = np.array([37, 16, 0, 1], dtype=np.int32)
    T = int(lens.max())
    src = torch.bfloat16 if fmt == "bf16" else torch.float32
    if fmt in FMTS:
        o, g = make_pair(fmt, B, 3, Hkv, d, cuda, rng)
        k, v = outlier_kv(rng, B, T, Hkv, d, src)
        sync_scales(o, g, k, v)
        o.append(k.float().numpy(), v.float().numpy(), new_lens=lens)
    else:                                           # unquantized pages: no oracle object needed
        bt = torch.from_numpy(rng.permutation(B * 3 + 2)[:B * 3].reshape(B, 3).astype(np.int32)).to(cuda)
        g = ops.PagedKV(fmt, B * 3 + 2, Hkv, d, bt, torch.zeros(B, dtype=torch.int32, device=cuda), cuda)
        k, v = outlier_kv(rng, B, T, Hkv, d, src)
    nl = torch.from_numpy(lens).to(cuda)
    g.append(k.to(cuda), v.to(cuda), new_lens=nl)
    g.seq_lens.copy_(nl)
    L = 40
    kd, vd = ops.kv_gather(g, L, dtype=torch.float32)
    kd, vd = kd.cpu().numpy(), vd.cpu().numpy()
    for b in range(B):
        if fmt in FMTS:
            Kr, Vr = o.gather(b)
        else:                                       # unquantized pages hold the appended values themselves
            Kr, Vr = k[b, :lens[b]].float().numpy(), v[b, :lens[b]].float().numpy()
        assert np.array_equal(kd[b, :lens[b]], Kr) and np.array_equal(vd[b, :lens[b]], Vr)
        assert not kd[b, lens[b]:].any() and not vd[b, lens[b]:].any()


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("name", ["fp32", "bf16"])
@pytest.mark.parametrize("H,Hkv,d", [(8, 2, 128), (14, 2, 64), (4, 4, 128), (32, 8, 128)])
@pytest.mark.parametrize("simt", [True, False])
def test_decode_attention_against_oracle(cuda, fmt, name, H, Hkv, d, simt):
    from transformer_surgeon_b200 import ops
    rng = np.random.default_rng(13)
    B = 5
    lens = np.array([1, 16, 17, 130, 0], dtype=np.int32)       # single token, exact page, ragged, multi-split, empty
    o, g = make_pair(fmt, B, 9, Hkv, d, cuda, rng)
    T = int(lens.max())
    k, v = outlier_kv(rng, B, T, Hkv, d, DT[name])
    sync_scales(o, g, k, v)
    nl = torch.from_numpy(lens).to(cuda)
    g.append(k.to(cuda), v.to(cuda), new_lens=nl)
    g.seq_lens.copy_(nl)
    o.append(k.float().numpy(), v.float().numpy(), new_lens=lens)
    assert np.array_equal(g.k_pool.cpu().numpy(), o.k_pool)
    q = torch.from_numpy(rng.standard_normal((B, H, d)).astype(np.float32)).to(DT[name])
    ref, ref_abs = oatt.paged_decode_attention(o, q.float().numpy(), with_abs=True)
    out = ops.paged_decode_attention(g, q.to(cuda), max_seq_len=144, simt=simt).float().cpu().numpy()
    assert np.all(out[4] == 0)
    tol = attn_tol(ref, ref_abs, name, simt)
    assert np.all(np.abs(out - ref) <= tol), (np.abs(out - ref) / tol).max()


@pytest.mark.parametrize("fmt", FMTS)
def test_decode_attention_config3_shape(cuda, fmt):
    """Llama-3-8B layout (32 q heads / 8 kv heads / d 128), batch 8, context 4096, seeded random
    block table: kernel vs oracle on every sequence, and tensor-core vs CUDA-core kernel."""
    from transformer_surgeon_b200 import ops
    rng = np.random.default_rng(14)
    B, L, H, Hkv, d = 8, 4096, 32, 8, 128
    o, g = make_pair(fmt, B, L // 16, Hkv, d, cuda, rng, extra_pages=5)
    k, v = outlier_kv(rng, B, L, Hkv, d, torch.bfloat16)
    sync_scales(o, g, k, v)
    g.append(k.to(cuda), v.to(cuda))
    g.seq_lens += L
    kc.append_vectorized(o, k.float().numpy(), v.float().numpy())
    assert np.array_equal(g.k_pool.cpu().numpy(), o.k_pool)
    assert np.array_equal(g.v_pool.cpu().numpy(), o.v_pool)
    q = torch.from_numpy(rng.standard_normal((B, H, d)).astype(np.float32)).bfloat16()
    ref, ref_abs = oatt.paged_decode_attention(o, q.float().numpy(), with_abs=True)
    out = ops.paged_decode_attention(g, q.to(cuda), max_seq_len=L).float().cpu().numpy()
    out_simt = ops.paged_decode_attention(g, q.to(cuda), max_seq_len=L, simt=True).float().cpu().numpy()
    tol, tol_simt = attn_tol(ref, ref_abs, "bf16", False), attn_tol(ref, ref_abs, "bf16", True)
    assert np.all(np.abs(out - ref) <= tol), (np.abs(out - ref) / tol).max()
    assert np.all(np.abs(out_simt - ref) <= tol_simt), (np.abs(out_simt - ref) / tol_simt).max()


@pytest.mark.parametrize("fmt", FMTS)
def test_full_size_properties(cuda, fmt):
    """Batch 64, context 32768 (the largest config-3 case, ~4.3 GB of pages), checked through
    size-independent properties:
      * V == 1 everywhere -> softmax weights sum to 1 -> output == 1 (exactly representable codes);
      * K == 0 -> uniform weights -> output == mean of V over the context;
      * run-to-run determinism of the split reduction."""
    from transformer_surgeon_b200 import ops
    B, L, H, Hkv, d = 64, 32768, 32, 8, 128
    npg = B * L // 16
    gen = torch.Generator(device=cuda).manual_seed(15)
    bt = torch.randperm(npg, generator=gen, device=cuda).to(torch.int32).reshape(B, L // 16)
    seq = torch.zeros(B, dtype=torch.int32, device=cuda)
    g = ops.PagedKV(fmt, npg, Hkv, d, bt, seq, cuda)
    chunk = 2048
    vmean = torch.zeros((B, Hkv, d), dtype=torch.float64, device=cuda)
    for t0 in range(0, L, chunk):
        k = torch.zeros((B, chunk, Hkv, d), dtype=torch.bfloat16, device=cuda)
        v = (2 * torch.randint(-1, 2, (B, chunk, Hkv, d), generator=gen, device=cuda)).to(torch.bfloat16)
        if fmt == "fp8" and t0 == 0:
            g.k_scale.fill_(1.0); g.v_scale.fill_(1.0 / 64)
        g.append(k, v)
        seq += chunk
        vmean += v.double().sum(dim=1)
    vmean /= L
    q = torch.randn((B, H, d), generator=gen, device=cuda).bfloat16()
    out = ops.paged_decode_attention(g, q, max_seq_len=L)
    out2 = ops.paged_decode_attention(g, q, max_seq_len=L)
    assert torch.equal(out, out2)
    # values in {-2, 0, 2}: int8 and fp8 (scale 1/64) store them exactly; nvfp4 stores 2 as
    # e2m1(2 / e4m3(2/6)) * e4m3(2/6) = 6 * 0.34375 = 2.0625 in every block that holds a 2
    gain = 1.03125 if fmt == "nvfp4" else 1.0
    ref = gain * vmean.float().repeat_interleave(H // Hkv, dim=1)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-3)
    # V == 1: overwrite the pools through a second append pass at position 0
    seq.zero_()
    for t0 in range(0, L, chunk):
        k = torch.randn((B, chunk, Hkv, d), generator=gen, device=cuda).bfloat16()
        v = torch.ones((B, chunk, Hkv, d), dtype=torch.bfloat16, device=cuda)
        if fmt == "fp8" and t0 == 0:
            g.k_scale.fill_(6.0 / 448); g.v_scale.fill_(1.0 / 64)
        g.append(k, v)
        seq += chunk
    out = ops.paged_decode_attention(g, q, max_seq_len=L).float()
    one = 1.03125 if fmt == "nvfp4" else 1.0          # 1 -> 6 * e4m3(1/6) = 6 * 0.171875
    torch.testing.assert_close(out, torch.full_like(out, one), rtol=1e-2, atol=1e-2)


def test_argument_errors(cuda):
    from transformer_surgeon_b200 import ops, Tsb200Error
    rng = np.random.default_rng(16)
    o, g = make_pair("int8", 2, 2, 2, 64, cuda, rng)
    q = torch.zeros((2, 5, 64), device=cuda)                    # 5 q heads not divisible by 2 kv heads
    with pytest.raises(Tsb200Error):
        ops.paged_decode_attention(g, q, max_seq_len=32)
    with pytest.raises(ValueError):
        ops.PagedKV("int8", 4, 2, 48, g.block_table, g.seq_lens, cuda)      # head_dim 48 unsupported
    small = torch.empty(16, dtype=torch.uint8, device=cuda)
    with pytest.raises(Tsb200Error):
        ops.paged_decode_attention(g, torch.zeros((2, 4, 64), device=cuda), max_seq_len=32, ws=small)
    # max_seq_len beyond what the block table covers (2 pages = 32 tokens): refused, nothing is launched
    with pytest.raises(Tsb200Error) as ei:
        ops.paged_decode_attention(g, torch.zeros((2, 4, 64), device=cuda), max_seq_len=33)
    assert ei.value.status == -1
    empty = ops.PagedKV("int8", 4, 2, 64, g.block_table, g.seq_lens, cuda)
    empty.num_pages = 0                                         # a descriptor with no pages is refused too
    with pytest.raises(Tsb200Error):
        ops.paged_decode_attention(empty, torch.zeros((2, 4, 64), device=cuda), max_seq_len=32)


@pytest.mark.parametrize("name", ["fp32", "bf16"])
def test_rope_append_fused_equals_separate_calls(cuda, name):
    """tsb200_rope_append on column slices of one fused [B, (H+2Hkv)d] projection buffer gives the
    same q and the same pages as tsb200_rope + tsb200_kv_append on dense copies."""
    from transformer_surgeon_b200 import ops
    rng = np.random.default_rng(17)
    B, H, Hkv, d = 6, 8, 2, 128
    _, g1 = make_pair("int8", B, 2, Hkv, d, cuda, rng)
    rng = np.random.default_rng(17)
    _, g2 = make_pair("int8", B, 2, Hkv, d, cuda, rng)
    start = torch.tensor([0, 3, 15, 16, 20, 31], dtype=torch.int32, device=cuda)
    g1.seq_lens.copy_(start); g2.seq_lens.copy_(start)
    cos, sin = oatt.rope_tables(d, 1e6, torch.arange(64))
    rope = (cos.to(cuda), sin.to(cuda))
    qkv = torch.randn((B, (H + 2 * Hkv) * d), generator=torch.Generator().manual_seed(3)).to(DT[name]).to(cuda)
    q_ref = qkv[:, :H * d].reshape(B, 1, H, d).clone()
    k_ref = qkv[:, H * d:(H + Hkv) * d].reshape(B, 1, Hkv, d).clone()
    v_ref = qkv[:, (H + Hkv) * d:].reshape(B, 1, Hkv, d).clone()
    ops.rope_(q_ref, rope[0], rope[1], start)
    g1.append(k_ref, v_ref, rope=rope)
    q4 = qkv[:, :H * d].unflatten(1, (H, d)).unsqueeze(1)
    k4 = qkv[:, H * d:(H + Hkv) * d].unflatten(1, (Hkv, d)).unsqueeze(1)
    v4 = qkv[:, (H + Hkv) * d:].unflatten(1, (Hkv, d)).unsqueeze(1)
    g2.rope_append(q4, k4, v4, rope)
    assert torch.equal(q4, q_ref)
    assert torch.equal(g1.k_pool, g2.k_pool) and torch.equal(g1.v_pool, g2.v_pool)


def test_fp8_attention_after_append_under_dependent_launch(cuda):
    """One decode step's append -> attention pair with programmatic dependent launch on: the attention may fetch pages
    older than the newest token before the append has finished.  Lengths sit on, before and after page boundaries and
    around the page count at which that early fetch starts; the result equals, bit for bit, the one with the setting
    off, and the oracle's within the attention tolerance."""
    from transformer_surgeon_b200 import ops
    rng = np.random.default_rng(29)
    B, H, Hkv, d = 32, 16, 4, 128                            # 128 (sequence, kv head) pairs: one split
    lens = np.array([0, 1, 15, 16, 17, 31, 32, 33, 95, 96, 97, 111, 112, 113, 127, 128, 129, 191, 192, 193, 207, 208, 209,
                     223, 224, 225, 239, 240, 241, 300, 400, 430], dtype=np.int32)
    o, g = make_pair("fp8", B, 28, Hkv, d, cuda, rng)
    T = int(lens.max())
    k, v = outlier_kv(rng, B, T + 1, Hkv, d, torch.bfloat16)
    sync_scales(o, g, k, v)
    nl = torch.from_numpy(lens).to(cuda)
    g.append(k[:, :T].to(cuda), v[:, :T].to(cuda), new_lens=nl)
    o.append(k[:, :T].float().numpy(), v[:, :T].float().numpy(), new_lens=lens)
    k_new = torch.stack([k[b, lens[b]] for b in range(B)]).unsqueeze(1).to(cuda)      # token at position lens[b]
    v_new = torch.stack([v[b, lens[b]] for b in range(B)]).unsqueeze(1).to(cuda)
    q = torch.from_numpy(rng.standard_normal((B, H, d)).astype(np.float32)).bfloat16().to(cuda)
    write_pos, after = nl.clone(), nl + 1
    outs = []
    for pdl in (False, True):
        old = ops.set_pdl(pdl)
        try:
            for _ in range(3):                               # the same token into the same slot every time
                g.append(k_new, v_new, seq_lens=write_pos)
                out = ops.paged_decode_attention(g, q, max_seq_len=448, seq_lens=after)
            torch.cuda.synchronize()
        finally:
            ops.set_pdl(old)
        outs.append(out.clone())
    assert torch.equal(outs[0], outs[1])
    o.seq_lens[:] = lens
    o.append(k_new.float().cpu().numpy(), v_new.float().cpu().numpy())
    o.seq_lens[:] = lens + 1
    ref, ref_abs = oatt.paged_decode_attention(o, q.float().cpu().numpy(), with_abs=True)
    tol = attn_tol(ref, ref_abs, "bf16", False)
    assert np.all(np.abs(outs[1].float().cpu().numpy() - ref) <= tol)
