"""Oracle: weight quantization, bit packing and reconstruction.  Test infrastructure only.

Restates transformersurgeon/compression/quantization_methods/vanilla.py:5-49
(`_dequantize_symmetric`, `_quantize_maxabs`, `_quantize_binarize`, `quantize_vanilla`)
with every rounding step written out, so a CUDA kernel can follow it bit for bit:

* the reference does its arithmetic in the PARAMETER dtype.  For bf16 parameters every
  torch op (amax/qmax, scale+eps, w/(scale+eps)) computes in fp32 and rounds the result
  to bf16 before the next op; `torch.round` is round-half-even.
* the fake-quantized weight the reference stores back is RN_dtype(float(q) * scale)
  (transformersurgeon/compression/quantization.py:112,126).

Packed container layouts (defined by this build; the reference keeps no codes):
  bits=8 : one two's-complement byte per code, natural column order
  bits<8 : little-endian 32-bit words of per = 32/bits fields; a word covers `per`
           consecutive columns, "pair-interleaved": field i < per/2 holds column 2i of
           the group, field i >= per/2 holds column 2(i - per/2) + 1.  (Masking the word
           with a 16-bit-periodic mask then yields columns (2j, 2j+1) in the two halves
           of a register: the order a bf16x2 tensor-core operand wants.)
           bits=4 / 2: two's-complement fields; bits=1: 1 -> +1, 0 -> -1 (no zero code).
Rows are padded with zero bytes to a multiple of 64 columns.
"""
import numpy as np
from .formats import bf16_round

EPS_DEFAULT = 1e-6   # transformersurgeon/compression/registry.py default `eps`


def _rnd(x, dtype):
    return bf16_round(x) if dtype == "bf16" else np.asarray(x, dtype=np.float32)


def quantize_maxabs(w, precision, eps=EPS_DEFAULT, per_channel=True, dtype="fp32"):
    """vanilla.py:10-24.  w: fp32 array holding exact values of `dtype`, shape [rows, cols].
    Returns (codes int8 [rows, cols], scale fp32 [rows, 1] (or [1,1]) holding `dtype` values)."""
    w = np.asarray(w, dtype=np.float32)
    qmax = np.float32(2 ** (precision - 1) - 1)
    if per_channel:
        amax = np.abs(w).max(axis=1, keepdims=True)
    else:
        amax = np.abs(w).max().reshape(1, 1)
    scale = _rnd(amax / qmax, dtype)
    denom = _rnd(scale + np.float32(eps), dtype)
    with np.errstate(divide="ignore", invalid="ignore"):
        quo = _rnd(w / denom, dtype)
    q = np.clip(np.rint(quo), -qmax, qmax).astype(np.int8)
    return q, scale


def quantize_binarize(w, per_channel=True, dtype="fp32"):
    """vanilla.py:27-37.  sign(w) in {-1,0,1}; scale = mean|w| (fp32 accumulation, rounded
    to `dtype`).  torch's CPU sum order is an implementation detail: the mean is taken
    here in fp64 and rounded once, which can differ from torch's fp32 cascade sum by an
    ulp for fp32 parameters (never observed for bf16)."""
    w = np.asarray(w, dtype=np.float32)
    s = np.sign(w).astype(np.int8)
    if per_channel:
        m = np.abs(w).astype(np.float64).mean(axis=1, keepdims=True)
    else:
        m = np.abs(w).astype(np.float64).mean().reshape(1, 1)
    return s, _rnd(m.astype(np.float32), dtype)


def quantize_vanilla(w, precision, eps=EPS_DEFAULT, granularity="per_tensor", dtype="fp32"):
    """vanilla.py:40-49."""
    pc = granularity == "per_channel"
    if precision == "binary":
        return quantize_binarize(w, pc, dtype)
    return quantize_maxabs(w, int(precision), eps, pc, dtype)


def dequantize(q, scale, dtype="fp32"):
    """vanilla.py:5-7 followed by the copy into the parameter (quantization.py:126)."""
    return _rnd(q.astype(np.float32) * np.asarray(scale, dtype=np.float32), dtype)


def container_bits(precision, codes=None):
    """Storage width for a precision: 8->8, 3..4->4, 2->2, binary->1 (2 when zeros occur)."""
    if precision == "binary":
        if codes is not None and (np.asarray(codes) == 0).any():
            return 2
        return 1
    p = int(precision)
    if p > 4:
        return 8
    if p > 2:
        return 4
    return 2


def _field_of_column(per):
    """Position (field index inside its word) of each of the `per` columns of a group."""
    c = np.arange(per)
    return (c >> 1) + (c & 1) * (per // 2)


def pack_codes(q, bits):
    """int8 codes [rows, cols] -> uint8 [rows, ceil64(cols)*bits/8]."""
    q = np.asarray(q, dtype=np.int8)
    rows, cols = q.shape
    cpad = (cols + 63) // 64 * 64
    qq = np.zeros((rows, cpad), dtype=np.int8)
    qq[:, :cols] = q
    if bits == 8:
        return qq.view(np.uint8).copy()
    per = 32 // bits
    mask = (1 << bits) - 1
    if bits == 1:
        u = np.zeros((rows, cpad), dtype=np.uint32)
        u[:, :cols] = (q > 0)
    else:
        u = qq.view(np.uint8).astype(np.uint32) & mask
    u = u.reshape(rows, cpad // per, per)
    words = np.zeros((rows, cpad // per), dtype=np.uint32)
    pos = _field_of_column(per)
    for c in range(per):
        words |= u[:, :, c] << np.uint32(bits * int(pos[c]))
    return words.view(np.uint8).reshape(rows, -1).copy()


def unpack_codes(p, bits, cols):
    p = np.ascontiguousarray(p, dtype=np.uint8)
    rows = p.shape[0]
    if bits == 8:
        return p.view(np.int8)[:, :cols].copy()
    per = 32 // bits
    mask = (1 << bits) - 1
    words = p.view(np.uint32)                                    # [rows, groups]
    pos = _field_of_column(per)
    out = np.zeros((rows, words.shape[1], per), dtype=np.int16)
    for c in range(per):
        f = ((words >> np.uint32(bits * int(pos[c]))) & mask).astype(np.int16)
        if bits == 1:
            out[:, :, c] = f * 2 - 1
        else:
            out[:, :, c] = np.where(f >= (1 << (bits - 1)), f - (1 << bits), f)
    return out.reshape(rows, -1)[:, :cols].astype(np.int8)
