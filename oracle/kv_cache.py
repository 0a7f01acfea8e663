"""Oracle: quantized paged KV cache (int8 / FP8-e4m3 / NVFP4).  Test infrastructure only.

PARITY UNPINNED: the reference has no quantized or paged KV cache (its `cache_impl`
values are "mutable" | "io_scatter" | "io_concat", transformersurgeon/blocks/mha.py:438,
all dense fixed-size rows written at clamp(pos_id), mha.py:514-535,583).  The formats
below are DEFINED here, following the reference's own weight-quantization conventions
(symmetric max-abs, q = clamp(round(x/(scale+eps))), eps 1e-6, dequant q*scale:
transformersurgeon/compression/quantization_methods/vanilla.py:5-24).  All arithmetic
is IEEE fp32 with round-to-nearest-even, written so a CUDA kernel reproduces it bit for
bit.

Formats (per token, per kv head, vector of d elements)
  int8  : s = amax/127 ; code = clip(rint(x/(s+1e-6)), +-127) ; one fp32 scale s.
  fp8   : code = e4m3_sat(x / S) with S an fp32 scale per (sequence, kv head) chosen by
          the caller (fp8_scale_from_amax: amax/448 over the prompt, 1.0 if amax == 0).
  nvfp4 : blocks of 16 consecutive elements; sb = e4m3_sat(amax_blk/6) stored as a byte,
          code = e2m1_sat(x / decode(sb)) (0 when decode(sb) == 0); two codes per byte,
          low nibble = even element.

Page record (page = 16 tokens) for one (page, kv head); K and V live in separate pools
of shape [num_pages, Hkv, record_bytes]:
  K int8  : codes [16 tok][d]      then scales fp32 [16 tok]
  K fp8   : codes [16 tok][d]
  K nvfp4 : codes [16 tok][d/2]    then block scales [16 tok][d/16]
  V int8  : codes [d][16 tok]      then scales fp32 [16 tok]        (token-minor: V^T)
  V fp8   : codes [d][16 tok]
  V nvfp4 : codes [d/2][16 tok] (byte = elements 2i (low nibble), 2i+1 of one token)
            then block scales [d/16][16 tok]
Token p of sequence b lives in page block_table[b, p // 16], slot p % 16.
"""
import numpy as np
from .formats import e4m3_encode, e4m3_decode, e2m1_encode, e2m1_decode

PAGE = 16
FMT_INT8, FMT_FP8, FMT_NVFP4 = 0, 1, 2
FMT_NAMES = {"int8": FMT_INT8, "fp8": FMT_FP8, "nvfp4": FMT_NVFP4}
_EPS = np.float32(1e-6)


def record_bytes(fmt, d):
    if fmt == FMT_INT8:
        return PAGE * d + PAGE * 4
    if fmt == FMT_FP8:
        return PAGE * d
    return PAGE * d // 2 + PAGE * d // 16


# ---- per-vector encoders (x: fp32 [..., d]) ------------------------------------
def int8_encode(x):
    x = np.asarray(x, dtype=np.float32)
    amax = np.abs(x).max(axis=-1, keepdims=True)
    s = (amax / np.float32(127.0)).astype(np.float32)
    q = np.clip(np.rint(x / (s + _EPS)), -127, 127).astype(np.int8)
    return q, s[..., 0]


def int8_decode(q, s):
    return q.astype(np.float32) * np.asarray(s, dtype=np.float32)[..., None]


def fp8_scale_from_amax(amax):
    amax = np.asarray(amax, dtype=np.float32)
    return np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)


def fp8_encode(x, scale):
    """scale broadcastable to x[..., 0]."""
    x = np.asarray(x, dtype=np.float32)
    return e4m3_encode(x / np.asarray(scale, dtype=np.float32)[..., None])


def fp8_decode(c, scale):
    return e4m3_decode(c) * np.asarray(scale, dtype=np.float32)[..., None]


def nvfp4_encode(x):
    """-> (codes uint8 [..., d] values 0..15, block scale bytes uint8 [..., d/16])."""
    x = np.asarray(x, dtype=np.float32)
    d = x.shape[-1]
    xb = x.reshape(*x.shape[:-1], d // 16, 16)
    amax = np.abs(xb).max(axis=-1)
    sb = e4m3_encode(amax / np.float32(6.0))
    sd = e4m3_decode(sb)
    with np.errstate(divide="ignore", invalid="ignore"):
        y = xb / sd[..., None]
    y = np.where(sd[..., None] > 0, y, np.float32(0.0)).astype(np.float32)
    return e2m1_encode(y).reshape(x.shape), sb


def nvfp4_decode(codes, sb):
    d = codes.shape[-1]
    v = e2m1_decode(codes).reshape(*codes.shape[:-1], d // 16, 16)
    return (v * e4m3_decode(sb)[..., None]).reshape(codes.shape).astype(np.float32)


# ---- paged pools ------------------------------------------------------------------
class PagedKV:
    """K and V pools for ONE layer plus the block table; numpy mirror of the device layout."""

    def __init__(self, fmt, num_pages, hkv, d, block_table, batch):
        self.fmt, self.hkv, self.d = fmt, hkv, d
        self.rec = record_bytes(fmt, d)
        self.k_pool = np.zeros((num_pages, hkv, self.rec), dtype=np.uint8)
        self.v_pool = np.zeros((num_pages, hkv, self.rec), dtype=np.uint8)
        self.block_table = np.asarray(block_table, dtype=np.int32)
        self.seq_lens = np.zeros(batch, dtype=np.int32)
        self.k_scale = np.ones((batch, hkv), dtype=np.float32)   # fp8 only
        self.v_scale = np.ones((batch, hkv), dtype=np.float32)

    # views into one record
    def _k_views(self, page, h):
        d, r = self.d, self.k_pool[page, h]
        if self.fmt == FMT_INT8:
            return r[:PAGE * d].reshape(PAGE, d), r[PAGE * d:].view(np.float32)
        if self.fmt == FMT_FP8:
            return r.reshape(PAGE, d), None
        return r[:PAGE * d // 2].reshape(PAGE, d // 2), r[PAGE * d // 2:].reshape(PAGE, d // 16)

    def _v_views(self, page, h):
        d, r = self.d, self.v_pool[page, h]
        if self.fmt == FMT_INT8:
            return r[:PAGE * d].reshape(d, PAGE), r[PAGE * d:].view(np.float32)
        if self.fmt == FMT_FP8:
            return r.reshape(d, PAGE), None
        return r[:PAGE * d // 2].reshape(d // 2, PAGE), r[PAGE * d // 2:].reshape(d // 16, PAGE)

    def append(self, k, v, new_lens=None):
        """k, v: fp32 [B, T, Hkv, d] (already rotated).  Appends new_lens[b] (default T)
        tokens of sequence b at positions seq_lens[b]...; then advances seq_lens."""
        B, T = k.shape[:2]
        new_lens = np.full(B, T, dtype=np.int32) if new_lens is None else np.asarray(new_lens)
        for b in range(B):
            for j in range(int(new_lens[b])):
                p = int(self.seq_lens[b]) + j
                page, slot = int(self.block_table[b, p // PAGE]), p % PAGE
                for h in range(self.hkv):
                    self._write(page, h, slot, b, k[b, j, h], v[b, j, h])
            self.seq_lens[b] += new_lens[b]

    def _write(self, page, h, slot, b, kx, vx):
        kc, ks = self._k_views(page, h)
        vc, vs = self._v_views(page, h)
        if self.fmt == FMT_INT8:
            q, s = int8_encode(kx); kc[slot] = q.view(np.uint8); ks[slot] = s
            q, s = int8_encode(vx); vc[:, slot] = q.view(np.uint8); vs[slot] = s
        elif self.fmt == FMT_FP8:
            kc[slot] = fp8_encode(kx, self.k_scale[b, h])
            vc[:, slot] = fp8_encode(vx, self.v_scale[b, h])
        else:
            c, sb = nvfp4_encode(kx); kc[slot] = c[0::2] | (c[1::2] << 4); ks[slot] = sb
            c, sb = nvfp4_encode(vx); vc[:, slot] = c[0::2] | (c[1::2] << 4); vs[:, slot] = sb

    def gather(self, b):
        """Dequantized K, V of sequence b: fp32 [L, Hkv, d] each."""
        L = int(self.seq_lens[b])
        K = np.zeros((L, self.hkv, self.d), dtype=np.float32)
        V = np.zeros_like(K)
        for p in range(L):
            page, slot = int(self.block_table[b, p // PAGE]), p % PAGE
            for h in range(self.hkv):
                kc, ks = self._k_views(page, h)
                vc, vs = self._v_views(page, h)
                if self.fmt == FMT_INT8:
                    K[p, h] = int8_decode(kc[slot].view(np.int8), ks[slot])
                    V[p, h] = int8_decode(vc[:, slot].view(np.int8), vs[slot])
                elif self.fmt == FMT_FP8:
                    K[p, h] = fp8_decode(kc[slot], self.k_scale[b, h])
                    V[p, h] = fp8_decode(vc[:, slot], self.v_scale[b, h])
                else:
                    c = np.empty(self.d, dtype=np.uint8)
                    c[0::2], c[1::2] = kc[slot] & 15, kc[slot] >> 4
                    K[p, h] = nvfp4_decode(c, ks[slot])
                    c[0::2], c[1::2] = vc[:, slot] & 15, vc[:, slot] >> 4
                    V[p, h] = nvfp4_decode(c, vs[:, slot])
        return K, V


def append_vectorized(kv, k, v):
    """Same result as PagedKV.append for uniform T, written with array ops so that
    full-size cases finish in seconds.  k, v: fp32 [B, T, Hkv, d]."""
    B, T, H, d = k.shape
    pos = kv.seq_lens[:, None].astype(np.int64) + np.arange(T)[None, :]          # [B,T]
    pages = np.take_along_axis(kv.block_table.astype(np.int64), pos // PAGE, axis=1)
    slots = pos % PAGE
    pg = np.repeat(pages[:, :, None], H, axis=2)                                   # [B,T,H]
    sl = np.repeat(slots[:, :, None], H, axis=2)
    hh = np.broadcast_to(np.arange(H)[None, None, :], (B, T, H))
    kr = kv.k_pool
    vr = kv.v_pool
    if kv.fmt == FMT_INT8:
        qk, sk = int8_encode(k); qv, sv = int8_encode(v)
        kc = kr[:, :, :PAGE * d].reshape(-1, H, PAGE, d)
        kc[pg, hh, sl] = qk.view(np.uint8)
        kr[:, :, PAGE * d:].view(np.float32)[pg, hh, sl] = sk
        vc = vr[:, :, :PAGE * d].reshape(-1, H, d, PAGE)
        vc[pg, hh, :, sl] = qv.view(np.uint8)
        vr[:, :, PAGE * d:].view(np.float32)[pg, hh, sl] = sv
    elif kv.fmt == FMT_FP8:
        ck = fp8_encode(k, kv.k_scale[:, None, :]); cv = fp8_encode(v, kv.v_scale[:, None, :])
        kr.reshape(-1, H, PAGE, d)[pg, hh, sl] = ck
        vr.reshape(-1, H, d, PAGE)[pg, hh, :, sl] = cv
    else:
        ck, sbk = nvfp4_encode(k); cv, sbv = nvfp4_encode(v)
        bk = ck[..., 0::2] | (ck[..., 1::2] << 4); bv = cv[..., 0::2] | (cv[..., 1::2] << 4)
        n = PAGE * d // 2
        kr[:, :, :n].reshape(-1, H, PAGE, d // 2)[pg, hh, sl] = bk
        kr[:, :, n:].reshape(-1, H, PAGE, d // 16)[pg, hh, sl] = sbk
        vr[:, :, :n].reshape(-1, H, d // 2, PAGE)[pg, hh, :, sl] = bv
        vr[:, :, n:].reshape(-1, H, d // 16, PAGE)[pg, hh, :, sl] = sbv
    kv.seq_lens += T


def dequant_pools(kv, batch_of_page=None):
    """Vectorised dequantisation of whole pools -> K, V fp32 [num_pages, Hkv, 16, d].
    fp8 needs the owning sequence of every page: batch_of_page int [num_pages] (-1 = free)."""
    P, H, d = kv.k_pool.shape[0], kv.hkv, kv.d
    if kv.fmt == FMT_INT8:
        n = PAGE * d
        K = kv.k_pool[:, :, :n].reshape(P, H, PAGE, d).view(np.int8).astype(np.float32)
        K *= np.ascontiguousarray(kv.k_pool[:, :, n:]).view(np.float32).reshape(P, H, PAGE, 1)
        V = kv.v_pool[:, :, :n].reshape(P, H, d, PAGE).view(np.int8).astype(np.float32).transpose(0, 1, 3, 2)
        V = V * np.ascontiguousarray(kv.v_pool[:, :, n:]).view(np.float32).reshape(P, H, PAGE, 1)
        return K, V
    if kv.fmt == FMT_FP8:
        bop = np.asarray(batch_of_page)
        ks = np.where(bop[:, None] >= 0, kv.k_scale[np.maximum(bop, 0)], 0).astype(np.float32)   # [P, H]
        vs = np.where(bop[:, None] >= 0, kv.v_scale[np.maximum(bop, 0)], 0).astype(np.float32)
        K = e4m3_decode(kv.k_pool.reshape(P, H, PAGE, d)) * ks[:, :, None, None]
        V = e4m3_decode(kv.v_pool.reshape(P, H, d, PAGE)).transpose(0, 1, 3, 2) * vs[:, :, None, None]
        return np.nan_to_num(K), np.nan_to_num(V)
    n = PAGE * d // 2
    kb = kv.k_pool[:, :, :n].reshape(P, H, PAGE, d // 2)
    kcodes = np.stack([kb & 15, kb >> 4], axis=-1).reshape(P, H, PAGE, d)
    K = nvfp4_decode(kcodes, kv.k_pool[:, :, n:].reshape(P, H, PAGE, d // 16))
    vb = kv.v_pool[:, :, :n].reshape(P, H, d // 2, PAGE).transpose(0, 1, 3, 2)          # [P,H,16,d/2]
    vcodes = np.stack([vb & 15, vb >> 4], axis=-1).reshape(P, H, PAGE, d)
    V = nvfp4_decode(vcodes, kv.v_pool[:, :, n:].reshape(P, H, d // 16, PAGE).transpose(0, 1, 3, 2))
    return np.nan_to_num(K), np.nan_to_num(V)


def batch_of_page(kv):
    bop = np.full(kv.k_pool.shape[0], -1, dtype=np.int64)
    for b in range(kv.block_table.shape[0]):
        npg = (int(kv.seq_lens[b]) + PAGE - 1) // PAGE
        bop[kv.block_table[b, :npg]] = b
    return bop


def gather_all(kv):
    """Dequantised caches of every sequence: lists K[b], V[b] of fp32 [L_b, Hkv, d]."""
    Kp, Vp = dequant_pools(kv, batch_of_page(kv) if kv.fmt == FMT_FP8 else None)
    Ks, Vs = [], []
    for b in range(kv.block_table.shape[0]):
        L = int(kv.seq_lens[b])
        npg = (L + PAGE - 1) // PAGE
        pg = kv.block_table[b, :npg]
        Ks.append(Kp[pg].transpose(0, 2, 1, 3).reshape(npg * PAGE, kv.hkv, kv.d)[:L])
        Vs.append(Vp[pg].transpose(0, 2, 1, 3).reshape(npg * PAGE, kv.hkv, kv.d)[:L])
    return Ks, Vs
