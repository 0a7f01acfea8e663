"""CPU decode step of the benchmark workload, for the CPU legs of bench.py (TEST / BASELINE INFRASTRUCTURE).

`ReferenceDecode` runs the REFERENCE's own code from oracle/_ref (placed by oracle/make_ref.py): a
`LlamaForCausalLMCompress` (transformersurgeon/models/llama_c/define_llama_c.py:24-30) of ONE decoder layer at the
full width of the workload, its MLP linears factorised by `LinearCompressed.init_lrd`
(blocks/linear_compressed.py:36-62), driven the way `generate()` drives it for a decode step: embedding, the
decoder layer with a Hugging Face `DynamicCache` holding `context` tokens per sequence (torch.cat append, SDPA
read), final norm, lm_head, argmax.  A full-depth step calls that one layer `layers` times (the weights and the
cache of one layer are reused - 32 distinct layers of bf16 weights plus caches would need ~25 GB of host memory
and minutes of random initialisation; the arithmetic per layer is identical) and crops the cache back to
`context` after each call.  Weights are fake-quantized floats in the reference, so the weight precision does not
change the work; the reference has no quantized KV cache, so the cache is dense bf16.

`PortDecode` is the fallback when oracle/_ref is absent: the same step from this package's restatements
(oracle/linear.py, oracle/attention.py).
"""
import os
import time

import torch


class ReferenceDecode:
    kind = "reference"

    def __init__(self, hidden, heads, kv_heads, inter, vocab, rank, batch, context, theta=5e5, eps=1e-5, seed=0):
        from . import make_ref
        T = make_ref.import_reference()
        from transformers import DynamicCache
        torch.manual_seed(seed)
        cfg = T.LlamaConfigCompress(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=1,
                                    num_attention_heads=heads, num_key_value_heads=kv_heads,
                                    max_position_embeddings=context + 4096, rope_theta=theta, rms_norm_eps=eps,
                                    tie_word_embeddings=False, dtype=torch.bfloat16)
        model = T.LlamaForCausalLMCompress(cfg).to(torch.bfloat16).eval()
        layer = model.model.layers[0]
        for m in (layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            m.init_lrd(rank)
            with torch.no_grad():
                m.weight.normal_(0, 0.02)
                m.linear_V.weight.normal_(0, 0.02)
        model.to(torch.bfloat16)
        self.model, self.layer, self.B, self.ctx = model, layer, batch, context
        d = hidden // heads
        g = torch.Generator().manual_seed(seed + 1)
        self.cache = DynamicCache(config=cfg)
        k = torch.randn(batch, kv_heads, context, d, generator=g).to(torch.bfloat16)
        v = torch.randn(batch, kv_heads, context, d, generator=g).to(torch.bfloat16)
        self.cache.update(k, v, 0)
        self.tok = torch.randint(0, vocab, (batch, 1), generator=g)

    @torch.no_grad()
    def step(self, layers):
        m = self.model.model
        hidden = m.embed_tokens(self.tok)
        pos = torch.full((self.B, 1), self.ctx, dtype=torch.long)
        pe = m.rotary_emb(hidden, pos)
        for _ in range(layers):
            out = self.layer(hidden, attention_mask=None, position_ids=pos, past_key_values=self.cache, use_cache=True,
                             position_embeddings=pe)
            hidden = out[0] if isinstance(out, tuple) else out
            self.cache.crop(self.ctx)
        logits = self.model.lm_head(m.norm(hidden)[:, -1])
        self.tok = torch.argmax(logits, dim=-1, keepdim=True)
        return self.tok


class PortDecode:
    kind = "port"

    def __init__(self, hidden, heads, kv_heads, inter, vocab, rank, batch, context, theta=5e5, eps=1e-5, seed=0):
        from . import attention as oatt
        g = torch.Generator().manual_seed(seed)
        dt = torch.bfloat16
        d = hidden // heads
        rn = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dt)
        self.w = dict(q=rn(heads * d, hidden), k=rn(kv_heads * d, hidden), v=rn(kv_heads * d, hidden), o=rn(hidden, heads * d),
                      ug=rn(inter, rank), vg=rn(rank, hidden), uu=rn(inter, rank), vu=rn(rank, hidden), ud=rn(hidden, rank),
                      vd=rn(rank, inter), lm=rn(vocab, hidden), n=torch.ones(hidden, dtype=dt))
        self.kc = torch.randn(batch, context + 1, kv_heads, d, generator=g).to(dt)
        self.vc = torch.randn(batch, context + 1, kv_heads, d, generator=g).to(dt)
        self.cos, self.sin = oatt.rope_tables(d, theta, torch.arange(context, context + 1))
        self.x = torch.randn(batch, hidden, generator=g).to(dt)
        self.dims = (batch, context, heads, kv_heads, d, eps)

    @torch.no_grad()
    def step(self, layers):
        from . import attention as oatt, linear as olin
        B, L, H, Hkv, d, eps = self.dims
        w, x = self.w, self.x
        for _ in range(layers):
            xn = oatt.rmsnorm_hf(x, w["n"], eps)
            q = olin.linear_compressed_forward(xn, w["q"]).view(B, 1, H, d)
            k = olin.linear_compressed_forward(xn, w["k"]).view(B, 1, Hkv, d)
            v = olin.linear_compressed_forward(xn, w["v"]).view(B, 1, Hkv, d)
            q, k = oatt.apply_rope(q, self.cos, self.sin), oatt.apply_rope(k, self.cos, self.sin)
            self.kc[:, L] = k[:, 0]
            self.vc[:, L] = v[:, 0]
            att = torch.stack([oatt.attention(q[b], self.kc[b], self.vc[b])[:, 0] for b in range(B)]).to(x.dtype)
            h = x + olin.linear_compressed_forward(att.reshape(B, H * d), w["o"])
            hn = oatt.rmsnorm_hf(h, w["n"], eps)
            m = oatt.swiglu(olin.linear_compressed_forward(hn, w["ug"], None, w["vg"]),
                            olin.linear_compressed_forward(hn, w["uu"], None, w["vu"]))
            x = (h + olin.linear_compressed_forward(m, w["ud"], None, w["vd"])) * 0.5
        return torch.argmax(olin.linear_compressed_forward(oatt.rmsnorm_hf(x, w["n"], eps), w["lm"]), dim=-1)


def make_decode(**kw):
    """The reference's own code when oracle/_ref is installed, else the port."""
    from . import make_ref
    torch.set_num_threads(os.cpu_count() or 1)
    if make_ref.ref_path():
        try:
            return ReferenceDecode(**kw)
        except Exception as ex:              # an incompatible transformers version etc.: say so and fall back
            print(f"oracle/_ref unusable ({ex!r}); timing the port instead", flush=True)
    return PortDecode(**kw)


def time_steps(dec, steps, warmup, layers):
    for _ in range(warmup):
        dec.step(layers)
    t0 = time.perf_counter()
    for _ in range(steps):
        dec.step(layers)
    return (time.perf_counter() - t0) / max(steps, 1)
