"""Oracle: one Qwen2 / Llama decoder layer + final norm + lm_head on CPU torch, with a fake-quantized KV
cache.  TEST INFRASTRUCTURE ONLY (tests and the CPU legs of bench.py).

Layer math = the Hugging Face decoder layer that the reference's `Qwen2ForCausalLMCompress` /
`LlamaForCausalLMCompress` / Qwen2.5-VL text tower inherit (transformersurgeon/models/qwen2_c/define_qwen2_c.py:22-27,
models/llama_c/define_llama_c.py:24-30, models/qwen2_5_vl_c/define_qwen2_5_vl_c.py:44-50), with every linear a
`LinearCompressed.forward` (blocks/linear_compressed.py:81-105) on DEQUANTIZED factors:
    h = x + o_proj(attn(rope(q_proj(n1(x))), cache(rope(k_proj(n1(x))), v_proj(n1(x)))))
    y = h + down_proj(silu(gate_proj(n2(h))) * up_proj(n2(h)))
The KV cache formats are this project's own definitions (oracle/kv_cache.py: "parity unpinned"): K and V are
quantized when appended and every attention read sees the dequantized values.

`act` selects the rounding points: torch.bfloat16 rounds where a bf16 model rounds (each module output, each
elementwise op), with fp32 accumulation inside the matrix products; torch.float32 rounds nowhere.
With ONE layer the prompt's K and V depend on the embeddings only, so the logits of the last prompt token and of
one decode step need the full prompt only through K and V: cheap enough to run at the full width of the
benchmark configurations.
"""
import numpy as np
import torch
import torch.nn.functional as F

from . import attention as oatt
from . import kv_cache as kc


def _lin(x, w, act):
    """LinearCompressed.forward: w = (U, V or None, bias or None), fp32 tensors holding dequantized values."""
    U, V, b = w
    x = x.float()
    if V is not None:
        x = F.linear(x, V).to(act).float()            # the rank-r intermediate is a module output: rounded
    return F.linear(x, U, b).to(act)


def kv_fake_quant(x, fmt, scale=None):
    """x fp32 [B, T, hkv, d] -> the values an attention read sees after quantize-on-append.
    fmt: "int8" | "fp8" | "nvfp4" | None (dense).  fp8: scale [B, hkv]."""
    if fmt is None:
        return x
    a = x.numpy()
    if fmt == "int8":
        q, s = kc.int8_encode(a)
        out = kc.int8_decode(q, s)
    elif fmt == "fp8":
        sc = np.asarray(scale, dtype=np.float32)[:, None, :]
        out = kc.fp8_decode(kc.fp8_encode(a, sc), sc)
    else:
        codes, sb = kc.nvfp4_encode(a)
        out = kc.nvfp4_decode(codes, sb)
    return torch.from_numpy(np.ascontiguousarray(out, dtype=np.float32))


def one_layer_logits(W, ids, next_ids, heads, kv_heads, head_dim, theta, eps, kv_fmt, act=torch.bfloat16):
    """W: dict with `embed` [vocab, hidden], `ln1`, `ln2`, `norm` [hidden], and `q`, `k`, `v`, `o`, `gate`, `up`,
    `down`, `lm_head` = (U, V or None, bias or None); all fp32 CPU tensors (dequantized values).
    ids [B, T] prompt, next_ids [B] the token fed to one decode step.
    Returns (logits after the prompt's last token, logits after the decode step), fp32 [B, vocab]."""
    B, T = ids.shape
    H, Hkv, d = heads, kv_heads, head_dim
    cos, sin = oatt.rope_tables(d, theta, torch.arange(T + 1))
    r = lambda t: t.to(act)

    def norm(x, w):
        return oatt.rmsnorm_hf(r(x), r(w), eps)

    def mlp(x):
        g, u = _lin(x, W["gate"], act), _lin(x, W["up"], act)
        return _lin(r(F.silu(g)) * u, W["down"], act)

    def attend(q, K, V):                                # q [B, H, d]; K, V [B, L, Hkv, d] (fp32 dequantized)
        out = torch.stack([oatt.attention(q[b:b + 1].float(), K[b], V[b])[:, 0] for b in range(B)])
        return r(out).reshape(B, H * d)

    def tail(x_last, att):
        h = r(x_last) + _lin(att, W["o"], act)
        y = h + mlp(norm(h, W["ln2"]))
        return _lin(norm(y, W["norm"]), W["lm_head"], act).float()

    x = W["embed"][ids]                                                     # [B, T, hidden]
    xn = norm(x, W["ln1"])
    k = oatt.apply_rope(_lin(xn, W["k"], act).view(B, T, Hkv, d), cos[:T], sin[:T])
    v = _lin(xn, W["v"], act).view(B, T, Hkv, d)
    ks = vs = None
    if kv_fmt == "fp8":                                                     # amax / 448 over the prompt, then frozen
        ks = kc.fp8_scale_from_amax(k.float().abs().amax(dim=(1, 3)).numpy())
        vs = kc.fp8_scale_from_amax(v.float().abs().amax(dim=(1, 3)).numpy())
    K, V = kv_fake_quant(k.float(), kv_fmt, ks), kv_fake_quant(v.float(), kv_fmt, vs)
    q = oatt.apply_rope(_lin(xn[:, -1], W["q"], act).view(B, 1, H, d), cos[T - 1:T], sin[T - 1:T])[:, 0]
    logits0 = tail(x[:, -1], attend(q, K, V))
    # ---- one decode step at position T
    x1 = W["embed"][next_ids]                                               # [B, hidden]
    xn1 = norm(x1, W["ln1"])
    k1 = oatt.apply_rope(_lin(xn1, W["k"], act).view(B, 1, Hkv, d), cos[T:T + 1], sin[T:T + 1])
    v1 = _lin(xn1, W["v"], act).view(B, 1, Hkv, d)
    K = torch.cat([K, kv_fake_quant(k1.float(), kv_fmt, ks)], dim=1)
    V = torch.cat([V, kv_fake_quant(v1.float(), kv_fmt, vs)], dim=1)
    q1 = oatt.apply_rope(_lin(xn1, W["q"], act).view(B, 1, H, d), cos[T:T + 1], sin[T:T + 1])[:, 0]
    logits1 = tail(x1, attend(q1, K, V))
    return logits0, logits1
