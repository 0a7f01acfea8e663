"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tsb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as ge
    ge.build()
    from transformer_surgeon_b200 import _lib
    lib = _lib.load()
    syms = declared_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/tsb200.h but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(syms)


def test_status_strings_and_sizes():
    from transformer_surgeon_b200 import _lib
    lib = _lib.load()
    assert lib.tsb200_version() >= 100
    assert lib.tsb200_strerror(0) == b"ok"
    for st in range(-6, 0):
        assert lib.tsb200_strerror(st) not in (b"ok", b"unknown status")
    assert lib.tsb200_packed_row_bytes(100, 4) == 64       # padded to 128 columns
    assert lib.tsb200_packed_row_bytes(4096, 8) == 4096
    assert lib.tsb200_packed_row_bytes(64, 1) == 8
    assert lib.tsb200_packed_row_bytes(64, 3) == 0
    assert lib.tsb200_kv_record_bytes(_lib.KV_INT8, 128) == 2112
    assert lib.tsb200_kv_record_bytes(_lib.KV_FP8, 128) == 2048
    assert lib.tsb200_kv_record_bytes(_lib.KV_NVFP4, 128) == 1152
    assert lib.tsb200_kv_record_bytes(_lib.KV_NVFP4, 64) == 576
    assert lib.tsb200_paged_decode_attn_workspace_bytes(64, 32, 128, 32768) == 16384 + 64 * 32 * 64 * 130 * 4


def test_record_sizes_match_oracle():
    from transformer_surgeon_b200 import _lib
    from oracle import kv_cache as kc
    lib = _lib.load()
    for fmt in (0, 1, 2):
        for d in (64, 128):
            assert lib.tsb200_kv_record_bytes(fmt, d) == kc.record_bytes(fmt, d)


def test_no_gpu_means_loud_failure():
    """Without a usable sm_100 device a compute entry point must fail, not fall back."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from transformer_surgeon_b200 import _lib
    lib = _lib.load()
    assert lib.tsb200_check_device() != 0
    assert lib.tsb200_swiglu(None, None, None, 0, 1, 1, 1, 1, 1, None) != 0
