"""Oracle: attention and the small decoder ops on CPU torch.  Test infrastructure only.

attention()      restates transformersurgeon/blocks/mha.py:9-103 (GQA by expanding K/V,
                 scores = (q*scale) @ k^T, + mask, softmax, @ v), computed in fp32.
paged_decode_attention()  one query token per sequence over the dequantized pages.
apply_rope()     restates transformersurgeon/blocks/rope.py:140-173 (half-split rotation)
                 with each product and the sum rounded to the activation dtype, which is
                 what both the reference and Hugging Face's rotate-half form do in bf16.
rope_tables()    restates rope.py:45-62 and 64-94 (inv_freq, cos/sin of t*inv_freq).
rmsnorm_blocks() restates transformersurgeon/blocks/norm.py:8-23 (max-abs prescale, eps 1e-5).
rmsnorm_hf()     Hugging Face Qwen2/Llama RMSNorm: fp32 x*rsqrt(mean(x^2)+eps), cast, *w.
swiglu()         restates transformersurgeon/blocks/mlp.py:181-183: silu(gate)*up.
"""
import math
import numpy as np
import torch


def attention(query, key, value, attn_mask=None):
    """query [T,H,d], key/value [L,Hkv,d] -> [H,T,d] (the layout mha.py:56,103 returns);
    fp32 math (mha.py:9-103)."""
    q, k, v = query.float(), key.float(), value.float()
    T, H, dq = q.shape
    L, Hkv, _ = k.shape
    g = H // Hkv
    scale = 1.0 / math.sqrt(dq)
    k = k.unsqueeze(2).expand(-1, -1, g, -1).reshape(L, H, -1).transpose(0, 1)
    v = v.unsqueeze(2).expand(-1, -1, g, -1).reshape(L, H, -1).transpose(0, 1)
    scores = torch.matmul(q.transpose(0, 1) * scale, k.transpose(-2, -1))
    if attn_mask is not None:
        scores = scores + attn_mask
    p = torch.softmax(scores, dim=-1)
    return torch.matmul(p, v)


def paged_decode_attention(kv, q, with_abs=False):
    """kv: oracle.kv_cache.PagedKV, q: fp32 array [B,H,d] -> fp32 [B,H,d].
    A sequence of length 0 yields zeros.  with_abs: also return sum_t p_t |V_t,e| per output element (the
    same softmax weights applied to |V|) - the natural scale of an element's rounding error, which the
    tests use as the error bound instead of a global max |V|."""
    from .kv_cache import gather_all
    B, H, d = q.shape
    out = np.zeros((B, H, d), dtype=np.float32)
    out_abs = np.zeros((B, H, d), dtype=np.float32)
    Ks, Vs = gather_all(kv)
    for b in range(B):
        if kv.seq_lens[b] == 0:
            continue
        K, V = Ks[b], Vs[b]
        qb = torch.from_numpy(q[b:b + 1])
        out[b] = attention(qb, torch.from_numpy(K), torch.from_numpy(V))[:, 0].numpy()
        if with_abs:
            out_abs[b] = attention(qb, torch.from_numpy(K), torch.from_numpy(np.abs(V)))[:, 0].numpy()
    return (out, out_abs) if with_abs else out


def rope_tables(head_dim, base, positions):
    """fp32 cos, sin of shape [len(positions), head_dim/2] (rope.py:45-94)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = torch.as_tensor(positions).float().unsqueeze(-1) * inv_freq.unsqueeze(0)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x, cos, sin):
    """x [..., T, heads, d] in its own dtype; cos/sin [T, d/2] fp32 (cast to x.dtype first)."""
    cos = cos.to(x.dtype).unsqueeze(-2)
    sin = sin.to(x.dtype).unsqueeze(-2)
    xr, xi = torch.chunk(x, 2, dim=-1)
    return torch.cat((xr * cos - xi * sin, xr * sin + xi * cos), dim=-1)


def rmsnorm_blocks(x, w):
    mx = torch.clamp(x.abs().amax(dim=-1, keepdim=True), min=1.0)
    x = x / mx
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return w * (x * torch.rsqrt(var + 1e-5))


def rmsnorm_hf(x, w, eps=1e-6):
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    return w * (xf * torch.rsqrt(var + eps)).to(x.dtype)


def swiglu(gate, up):
    return torch.nn.functional.silu(gate) * up
