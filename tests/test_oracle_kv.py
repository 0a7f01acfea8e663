"""Self-consistency of the KV-format oracle (formats are defined by the oracle: parity unpinned)."""
import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import kv_cache as kc
from oracle import attention as oatt


def test_e4m3_matches_torch_cast():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(100000) * rng.choice([1e-3, 0.1, 1, 50, 300], 100000)).astype(np.float32)
    x = np.clip(x, -448, 448)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(F.e4m3_encode(x), ref)
    assert np.array_equal(F.e4m3_encode(np.array([1e9, -1e9], np.float32)), np.array([0x7E, 0xFE], np.uint8))
    mids = ((F.E4M3_POS[:-1] + F.E4M3_POS[1:]) / 2).astype(np.float32)
    assert np.array_equal(F.e4m3_encode(mids), torch.from_numpy(mids).to(torch.float8_e4m3fn).view(torch.uint8).numpy())


def test_e2m1_ties_to_even_and_saturation():
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 100.0, -0.3, 0.26, -6.1], np.float32)
    assert F.e2m1_encode(x).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 7, 9, 1, 15]
    assert np.array_equal(F.e2m1_decode(np.arange(8, dtype=np.uint8)), F.E2M1_POS.astype(np.float32))


def test_bf16_round_matches_torch():
    x = np.random.default_rng(1).standard_normal(50000).astype(np.float32) * 37
    assert np.array_equal(F.bf16_round(x), torch.from_numpy(x).bfloat16().float().numpy())


@pytest.mark.parametrize("fmt,tol", [(kc.FMT_INT8, 0.02), (kc.FMT_FP8, 0.08), (kc.FMT_NVFP4, 0.3)])
def test_append_gather_roundtrip_and_vectorized(fmt, tol):
    rng = np.random.default_rng(2)
    B, T, H, d = 3, 37, 2, 64
    npg = B * 4
    bt = rng.permutation(npg).reshape(B, 4).astype(np.int32)
    a, b = kc.PagedKV(fmt, npg, H, d, bt, B), kc.PagedKV(fmt, npg, H, d, bt, B)
    k = rng.standard_normal((B, T, H, d)).astype(np.float32)
    v = rng.standard_normal((B, T, H, d)).astype(np.float32)
    if fmt == kc.FMT_FP8:
        for o in (a, b):
            o.k_scale[:] = kc.fp8_scale_from_amax(np.abs(k).max(axis=(1, 3)))
            o.v_scale[:] = kc.fp8_scale_from_amax(np.abs(v).max(axis=(1, 3)))
    a.append(k, v)
    kc.append_vectorized(b, k, v)
    assert np.array_equal(a.k_pool, b.k_pool) and np.array_equal(a.v_pool, b.v_pool)
    K, V = a.gather(1)
    assert np.abs(K - k[1]).max() <= tol * np.abs(k).max()
    assert np.abs(V - v[1]).max() <= tol * np.abs(v).max()


def test_ragged_and_empty_append():
    rng = np.random.default_rng(3)
    B, H, d = 3, 2, 64
    bt = np.arange(B * 2, dtype=np.int32).reshape(B, 2)
    kv = kc.PagedKV(kc.FMT_INT8, B * 2, H, d, bt, B)
    k = rng.standard_normal((B, 5, H, d)).astype(np.float32)
    kv.append(k, k, new_lens=[5, 0, 2])
    assert kv.seq_lens.tolist() == [5, 0, 2]
    q = rng.standard_normal((B, 4, d)).astype(np.float32)
    out = oatt.paged_decode_attention(kv, q)
    assert np.all(out[1] == 0) and np.isfinite(out).all() and np.abs(out[0]).max() > 0


def test_paged_attention_equals_reference_attention_on_dequantized_cache():
    rng = np.random.default_rng(4)
    B, T, H, Hkv, d = 2, 40, 8, 2, 64
    bt = rng.permutation(B * 3).reshape(B, 3).astype(np.int32)
    kv = kc.PagedKV(kc.FMT_INT8, B * 3, Hkv, d, bt, B)
    k = rng.standard_normal((B, T, Hkv, d)).astype(np.float32)
    v = rng.standard_normal((B, T, Hkv, d)).astype(np.float32)
    kv.append(k, v)
    q = rng.standard_normal((B, H, d)).astype(np.float32)
    out = oatt.paged_decode_attention(kv, q)
    # dense attention over the *unquantized* K, V is close (int8 error only)
    ref = oatt.attention(torch.from_numpy(q[0:1]), torch.from_numpy(k[0]), torch.from_numpy(v[0]))[:, 0].numpy()
    assert np.abs(out[0] - ref).max() < 0.02
