"""Bit-level number formats used by the oracle (numpy, CPU).  Test infrastructure only.

e4m3 (OCP FP8 E4M3FN: bias 7, no inf, max 448, 0x7f = NaN) and e2m1 (OCP FP4: values
0, .5, 1, 1.5, 2, 3, 4, 6) encoders round to nearest, ties to the even code, and
saturate to the largest finite value.  bf16 rounding is round-to-nearest-even on the
upper 16 bits of the fp32 pattern.
"""
import numpy as np

# ---- bf16 -----------------------------------------------------------------
def bf16_round(x):
    """Round fp32 array to the nearest bf16 value (ties to even); returns fp32."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32).reshape(a.shape)
    nan = np.isnan(a)
    if nan.any():
        out = np.where(nan, np.float32(np.nan), out)
    return out


def bf16_bits(x):
    """fp32 array holding exact bf16 values -> uint16 bit patterns."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    return (a.view(np.uint32) >> 16).astype(np.uint16).reshape(a.shape)


def bf16_from_bits(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- e4m3 -----------------------------------------------------------------
def _e4m3_table():
    v = np.zeros(127, dtype=np.float64)
    for c in range(127):
        e, m = c >> 3, c & 7
        v[c] = (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
    return v

E4M3_POS = _e4m3_table()              # code 0..126 -> value (0 .. 448)
_E4M3_MID = (E4M3_POS[:-1] + E4M3_POS[1:]) / 2.0


def e4m3_encode(x):
    """fp32 -> uint8 e4m3 codes, round-nearest-even, saturate-to-finite (|x|>448 -> 448)."""
    a = np.asarray(x, dtype=np.float32)
    mag = np.abs(a).astype(np.float64)
    idx = np.searchsorted(_E4M3_MID, mag, side="left")       # mag <= mid[i] -> i
    # exact ties: mag == mid[i] lands on i (lower); choose the even code of (i, i+1)
    tie = (idx < 126) & (mag == _E4M3_MID[np.minimum(idx, 125)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    idx = np.minimum(idx, 126)
    idx = np.where(np.isnan(a), 0x7F, idx)
    sign = (np.signbit(a)).astype(np.uint8) << 7
    return (idx.astype(np.uint8) | sign).astype(np.uint8)


def e4m3_decode(c):
    c = np.asarray(c, dtype=np.uint8)
    mag = np.concatenate([E4M3_POS, [np.nan]])[c & 0x7F]
    return np.where(c & 0x80, -mag, mag).astype(np.float32)


# ---- e2m1 -----------------------------------------------------------------
E2M1_POS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_E2M1_MID = (E2M1_POS[:-1] + E2M1_POS[1:]) / 2.0


def e2m1_encode(x):
    """fp32 -> 4-bit e2m1 codes (uint8 0..15), round-nearest-even-code, saturating."""
    a = np.asarray(x, dtype=np.float32)
    mag = np.abs(a).astype(np.float64)
    idx = np.searchsorted(_E2M1_MID, mag, side="left")
    tie = (idx < 7) & (mag == _E2M1_MID[np.minimum(idx, 6)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    idx = np.minimum(idx, 7)
    sign = (np.signbit(a)).astype(np.uint8) << 3
    return (idx.astype(np.uint8) | sign).astype(np.uint8)


def e2m1_decode(c):
    c = np.asarray(c, dtype=np.uint8)
    mag = E2M1_POS[c & 7]
    return np.where(c & 8, -mag, mag).astype(np.float32)
