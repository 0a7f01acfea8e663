"""The allocation-free decode-attention entry point (tsb200_paged_decode_attn_static).

It exists for callers that are not allowed to allocate device memory on their serving path (a
plugin with a fixed memory budget, a runtime whose allocator cannot be re-entered, code that is
already inside a stream capture): the scratch for the split partials is a fixed array inside the
library instead of a caller-provided workspace.  The test drives it through the C ABI, twice in a
row on different inputs (the array keeps the first call's contents), and compares each result with
the regular entry point; it also checks that an oversized problem is refused.  This file sorts
last on purpose, so a failure here cannot hide the results of the other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(cuda, fmt, seed, B=4, H=8, Hkv=2, d=128, L=300):
    from transformer_surgeon_b200 import ops
    g = torch.Generator(device=cuda).manual_seed(seed)
    pages = (L + 15) // 16
    bt = torch.randperm(B * pages, generator=g, device=cuda).to(torch.int32).reshape(B, pages)
    seq = torch.zeros(B, dtype=torch.int32, device=cuda)
    kv = ops.PagedKV(fmt, B * pages, Hkv, d, bt, seq, cuda)
    k = torch.randn((B, L, Hkv, d), generator=g, device=cuda).bfloat16()
    v = torch.randn((B, L, Hkv, d), generator=g, device=cuda).bfloat16()
    if fmt == "fp8":
        kv.set_fp8_scales(k, v)
    kv.append(k, v)
    seq += L
    if B > 1:
        seq[1] = L - 37                  # ragged lengths
    q = torch.randn((B, H, d), generator=g, device=cuda).bfloat16()
    return ops, kv, q, L


def _static_call(ops, kv, q, L):
    from transformer_surgeon_b200 import _lib
    lib = _lib.load()
    out = torch.full_like(q, float("nan"))
    desc = kv.desc()
    B, H, d = q.shape
    st = lib.tsb200_paged_decode_attn_static(C.byref(desc), C.c_void_p(q.data_ptr()), C.c_void_p(out.data_ptr()),
                                             _lib.BF16, 0, B, H, d ** -0.5, L,
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, out


# Shapes chosen so that BOTH kernels split their sequences (only then do the partials and the split counters in
# the array come into play): the int8 kernel splits 4 ways at 4 sequences x 2 kv heads x 300 tokens, the FP8
# kernel needs at least 24 pages per split and few (sequence, head) pairs: 1 x 2 x 1200 tokens -> 3 splits.
SHAPES = {"int8": dict(B=4, L=300), "fp8": dict(B=1, L=1200)}


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
def test_static_scratch_matches_workspace_entry_point_twice(cuda, fmt):
    for seed in (1, 2):                  # second call: the array still holds the first call's partials
        ops, kv, q, L = _setup(cuda, fmt, seed, **SHAPES[fmt])
        if seed == 2:
            kv.seq_lens[0] = L - 37      # another ragged length on the second round
        st, out = _static_call(ops, kv, q, L)
        assert st == 0
        ref = ops.paged_decode_attention(kv, q, max_seq_len=L)
        torch.cuda.synchronize()
        # same kernels, same split order: identical bits (the tolerance used elsewhere would also do)
        assert torch.equal(out, ref)


def test_static_scratch_rejects_oversized_problem(cuda):
    from transformer_surgeon_b200 import _lib
    lib = _lib.load()
    ops, kv, q, L = _setup(cuda, "fp8", 3)
    cap = lib.tsb200_paged_decode_attn_static_capacity()
    assert cap == 8 << 20
    B, H, d = 128, 32, 128                   # 5 splits x 128 x 32 heads x 130 floats = 10.6 MB of partials
    assert lib.tsb200_paged_decode_attn_workspace_bytes(B, H, d, 32768) > cap
    qbig = torch.zeros((B, H, d), dtype=torch.bfloat16, device=cuda)
    desc = kv.desc()
    st = lib.tsb200_paged_decode_attn_static(C.byref(desc), C.c_void_p(qbig.data_ptr()), C.c_void_p(qbig.data_ptr()),
                                             _lib.BF16, 0, B, H, d ** -0.5, 32768, None)
    assert st == _lib.ERR_WORKSPACE
    assert b"workspace" in lib.tsb200_strerror(st)
