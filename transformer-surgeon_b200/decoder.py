"""Qwen2 / Llama decoder built from the C-ABI kernels: the decode step that
`*ForCausalLMCompress.generate()` runs per token, with the attention and MLP modules rewired
onto PackedLinear, the quantized paged KV cache and the fused small ops.

Layer math follows Hugging Face's Qwen2/Llama decoder layer (what the reference's
`Qwen2ForCausalLMCompress` / `LlamaForCausalLMCompress` inherit, models/qwen2_c/define_qwen2_c.py:22-27,
models/llama_c/define_llama_c.py:24-30):
    h = x + o_proj(attn(rope(q_proj(n1(x))), cache(rope(k_proj(n1(x))), v_proj(n1(x)))))
    y = h + down_proj(silu(gate_proj(n2(h))) * up_proj(n2(h)))
The `variant=1` norm and rope base of the reference's own blocks path (blocks/decoder.py:100-149,
blocks/norm.py:8-23) are selectable through DecoderConfig.

There is no CPU path: every tensor lives on the GPU and every op is a libtsb200 kernel, except
the embedding gather, the final argmax and integer bookkeeping (torch).
"""
from dataclasses import dataclass

import torch

from . import ops


@dataclass
class DecoderConfig:
    num_layers: int
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    norm_variant: int = 0          # 0 = Hugging Face RMSNorm, 1 = blocks/norm.py RMSNorm
    dtype: torch.dtype = torch.bfloat16
    kv_format: str = "fp8"         # int8 | fp8 | nvfp4 | fp32 | bf16
    max_positions: int = 4096
    tp_world: int = 1              # tensor-parallel group size (1 = none); num_heads / num_kv_heads are GLOBAL
    tp_rank: int = 0


class LayerWeights:
    """Kernel-side weights of one decoder layer.  `qkv` is one PackedLinear producing
    [q | k | v] when the three projections could be fused (same container, full rank),
    otherwise q, k, v are separate."""

    def __init__(self, ln1, ln2, o, gate, up, down, qkv=None, q=None, k=None, v=None):
        self.ln1, self.ln2, self.o, self.gate, self.up, self.down = ln1, ln2, o, gate, up, down
        self.qkv, self.q, self.k, self.v = qkv, q, k, v
        self.mlp = ops.GatedMLP(gate, up, down)


def fuse_rows(factors, biases, act_dtype):
    """Stack full-rank factors with identical containers row-wise into one PackedLinear
    (per-row scales make this exact).  Returns None when they cannot be fused."""
    f0 = factors[0]
    if any(f.bits != f0.bits or f.cols != f0.cols for f in factors):
        return None
    data = torch.cat([f.data for f in factors], dim=0).contiguous()
    scales = None if f0.scales is None else torch.cat([f.scales for f in factors]).contiguous()
    rows = sum(f.rows for f in factors)
    bias = None
    if any(b is not None for b in biases):
        bias = torch.cat([b if b is not None else torch.zeros(f.rows, dtype=act_dtype, device=data.device)
                          for f, b in zip(factors, biases)]).contiguous()
    return ops.PackedLinear(ops.Factor(data, scales, f0.bits, rows, f0.cols), None, bias, act_dtype)


def rope_tables(head_dim, theta, max_positions, device):
    """fp32 cos/sin [max_positions, head_dim/2]: inv_freq = theta^(-2i/d), angle = pos * inv_freq
    (blocks/rope.py:45-94; identical to Hugging Face's default rotary embedding)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    ang = torch.arange(max_positions, dtype=torch.float32).unsqueeze(-1) * inv.unsqueeze(0)
    return torch.cos(ang).to(device).contiguous(), torch.sin(ang).to(device).contiguous()


class CompressedDecoder:
    def __init__(self, cfg, embed, layers, final_norm, lm_head, batch, max_seq_len, device, tp_group=None, own_caches=True):
        self.cfg, self.embed, self.layers, self.final_norm, self.lm_head = cfg, embed, layers, final_norm, lm_head
        self.B, self.max_seq_len, self.device = batch, max_seq_len, device
        self.tp_group = tp_group
        c = cfg
        if c.tp_world > 1:
            if c.num_heads % c.tp_world or c.num_kv_heads % c.tp_world:
                raise ValueError("heads must split evenly over the tensor-parallel ranks")
            layers = self.layers = [self._shard_layer(L, c) for L in layers]
        self.H_local, self.Hkv_local = c.num_heads // c.tp_world, c.num_kv_heads // c.tp_world
        self.pages_per_seq = (max_seq_len + ops.PAGE - 1) // ops.PAGE
        num_pages = batch * self.pages_per_seq
        # sequence-major ascending page allocation: reproducible block tables
        self.block_table = torch.arange(num_pages, dtype=torch.int32, device=device).reshape(batch, self.pages_per_seq)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=device)    # tokens in cache (after this step's append)
        self.write_pos = torch.zeros(batch, dtype=torch.int32, device=device)   # position of the token being appended
        # own_caches=False: the caller brings the caches (bind_caches) before the first step
        self.kv = [ops.PagedKV(c.kv_format, num_pages, self.Hkv_local, c.head_dim, self.block_table, self.seq_lens, device)
                   for _ in range(c.num_layers)] if own_caches else []
        self.cos, self.sin = rope_tables(c.head_dim, c.rope_theta, c.max_positions, device)
        H, Hkv, d = self.H_local, self.Hkv_local, c.head_dim
        dt = c.dtype
        B = batch
        # persistent activation buffers (stable addresses -> the step can be captured in a CUDA graph)
        self.tokens = torch.zeros(B, dtype=torch.int64, device=device)
        self.resid = torch.zeros((B, c.hidden), dtype=dt, device=device)
        self.xn = torch.empty((B, c.hidden), dtype=dt, device=device)
        self.qkv = torch.empty((B, (H + 2 * Hkv) * d), dtype=dt, device=device)
        self.qb = torch.empty((B, H * d), dtype=dt, device=device)
        self.kb = torch.empty((B, Hkv * d), dtype=dt, device=device)
        self.vb = torch.empty((B, Hkv * d), dtype=dt, device=device)
        self.attn = torch.empty((B, H * d), dtype=dt, device=device)
        self.delta = torch.empty((B, c.hidden), dtype=dt, device=device)
        self.logits = torch.empty((B, c.vocab), dtype=dt, device=device)
        self.next_tokens = torch.zeros(B, dtype=torch.int64, device=device)
        lin_ws = 256
        for L in layers:
            for lin in (L.qkv, L.q, L.k, L.v, L.o, L.gate, L.up, L.down):
                if lin is not None:
                    lin_ws = max(lin_ws, lin.workspace_bytes(B))
        lin_ws = max(lin_ws, lm_head.workspace_bytes(B))
        self.lin_ws = torch.zeros(lin_ws, dtype=torch.uint8, device=device)
        self.mlp_ws = torch.zeros(max(L.mlp.workspace_bytes(B) for L in layers), dtype=torch.uint8, device=device)
        self.attn_ws = torch.zeros(ops.decode_attn_workspace_bytes(B, H, d, max_seq_len), dtype=torch.uint8, device=device)
        self.graph = None
        self.kernel_launches_per_step = 0
        self.peer = None                    # tensor_parallel.PeerBuffers once enable_peer_allreduce() ran
        # greedy_head: the step ends in tsb200_linear_argmax (no logits in memory; `step` then returns None and only
        # `next_tokens` is updated) instead of lm_head -> logits -> argmax.  Set before capture().
        self.greedy_head = False
        self.head_ws = None

    def enable_peer_allreduce(self):
        """Tensor parallel: sum the row-parallel partial outputs with the library's own kernel over NVLink
        peer memory, fused with the residual add and RMSNorm that follow (`tsb200_peer_allreduce_add_rmsnorm`),
        instead of an NCCL all-reduce plus a separate normalisation launch.  Call on every rank, before
        `capture()`.  Returns False (and changes nothing) when the configuration is outside what the kernel takes."""
        c = self.cfg
        if c.tp_world < 2 or c.dtype != torch.bfloat16 or c.norm_variant != 0 or c.hidden % 8 or c.hidden > 8192 or self.B > 1024:
            return False
        from .tensor_parallel import PeerBuffers
        self.peer = PeerBuffers(self.B, c.hidden, self.device, self.tp_group)
        self.graph = None
        return True

    @staticmethod
    def _shard_layer(L, c):
        """Tensor-parallel shard of one layer: q/k/v/gate/up column-parallel, o/down row-parallel."""
        from . import tensor_parallel as tp
        w, r, d = c.tp_world, c.tp_rank, c.head_dim
        if L.qkv is not None:
            raise ValueError("build tensor-parallel engines with separate q/k/v projections (fuse_qkv=False)")
        q, k, v = (tp.column_parallel(x, w, r, d) for x in (L.q, L.k, L.v))
        qkv = None
        if not (q.rank or k.rank or v.rank):
            qkv = fuse_rows([q.u, k.u, v.u], [q.bias, k.bias, v.bias], c.dtype)
        return LayerWeights(L.ln1, L.ln2, tp.row_parallel(L.o, w, r, d), tp.column_parallel(L.gate, w, r),
                            tp.column_parallel(L.up, w, r), tp.row_parallel(L.down, w, r), qkv=qkv,
                            q=None if qkv else q, k=None if qkv else k, v=None if qkv else v)

    # ------------------------------------------------------------------ one decode step
    def _step_kernels(self):
        c = self.cfg
        B, H, Hkv, d = self.B, self.H_local, self.Hkv_local, c.head_dim
        tp_on = c.tp_world > 1
        if tp_on:
            from .tensor_parallel import all_reduce_sum
        n = 0
        torch.index_select(self.embed, 0, self.tokens, out=self.resid)
        self.write_pos.copy_(self.seq_lens)
        self.seq_lens.add_(1)
        delta = None
        rope = (self.cos, self.sin)
        peer = self.peer if tp_on else None
        for li, L in enumerate(self.layers):
            if peer is not None and li > 0:      # the previous layer's down_proj partials: summed, added, normalised
                peer.allreduce_add_rmsnorm(1, self.resid, L.ln1, c.rms_eps, out=self.xn); n += 1
            else:
                ops.add_rmsnorm(self.resid, delta, L.ln1, c.rms_eps, c.norm_variant, out=self.xn); n += 1
            if L.qkv is not None:
                L.qkv(self.xn, out=self.qkv, ws=self.lin_ws); n += 1
                q4 = self.qkv[:, :H * d].unflatten(1, (H, d)).unsqueeze(1)                   # [B,1,H,d] views
                k4 = self.qkv[:, H * d:(H + Hkv) * d].unflatten(1, (Hkv, d)).unsqueeze(1)
                v4 = self.qkv[:, (H + Hkv) * d:].unflatten(1, (Hkv, d)).unsqueeze(1)
            else:
                L.q(self.xn, out=self.qb, ws=self.lin_ws)
                L.k(self.xn, out=self.kb, ws=self.lin_ws)
                L.v(self.xn, out=self.vb, ws=self.lin_ws)
                n += sum(2 if l.rank else 1 for l in (L.q, L.k, L.v))
                q4, k4, v4 = self.qb.view(B, 1, H, d), self.kb.view(B, 1, Hkv, d), self.vb.view(B, 1, Hkv, d)
            self.kv[li].rope_append(q4, k4, v4, rope, seq_lens=self.write_pos); n += 1
            ops.paged_decode_attention(self.kv[li], q4[:, 0], self.max_seq_len, out=self.attn.view(B, H, d),
                                       ws=self.attn_ws, seq_lens=self.seq_lens); n += 2
            if peer is not None:
                L.o(self.attn, out=peer.partial(0), ws=self.lin_ws); n += 1
                peer.allreduce_add_rmsnorm(0, self.resid, L.ln2, c.rms_eps, out=self.xn); n += 1
                L.mlp(self.xn, out=peer.partial(1), ws=self.mlp_ws); n += 1
                continue
            L.o(self.attn, out=self.delta, ws=self.lin_ws); n += 1
            if tp_on:
                all_reduce_sum(self.delta, self.tp_group)       # row-parallel o_proj: sum of the partial outputs
            ops.add_rmsnorm(self.resid, self.delta, L.ln2, c.rms_eps, c.norm_variant, out=self.xn); n += 1
            L.mlp(self.xn, out=self.delta, ws=self.mlp_ws); n += 1
            if tp_on:
                all_reduce_sum(self.delta, self.tp_group)       # row-parallel down_proj
            delta = self.delta
        if peer is not None:
            peer.allreduce_add_rmsnorm(1, self.resid, self.final_norm, c.rms_eps, out=self.xn); n += 1
        else:
            ops.add_rmsnorm(self.resid, delta, self.final_norm, c.rms_eps, c.norm_variant, out=self.xn); n += 1
        if self.greedy_head:
            if self.head_ws is None:
                self.head_ws = torch.zeros(self.lm_head.argmax_workspace_bytes(B), dtype=torch.uint8, device=self.device)
            self.lm_head.argmax(self.xn, out=self.next_tokens, ws=self.head_ws); n += 2
            self.kernel_launches_per_step = n
            return None
        self.lm_head(self.xn, out=self.logits, ws=self.lin_ws); n += 1
        torch.argmax(self.logits, dim=-1, out=self.next_tokens)
        self.kernel_launches_per_step = n
        return self.logits

    def capture(self, pdl=True):
        """Capture one decode step in a CUDA graph (the per-token Python loop of Hugging Face's
        `_sample` and ~15 launches per layer collapse into one graph launch).  With `pdl` the
        kernels are captured with programmatic dependent launch edges: each kernel's prologue and
        weight prefetch overlap the tail of its predecessor."""
        old_pdl = ops.set_pdl(pdl)
        try:
            self._capture()
        finally:
            ops.set_pdl(old_pdl)

    def _capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        saved = self.seq_lens.clone()
        with torch.cuda.stream(s):
            self._step_kernels()            # warm-up outside capture (sets function attributes)
            self.seq_lens.copy_(saved)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step_kernels()
        self.seq_lens.copy_(saved)
        self.graph = g

    def step(self, tokens=None):
        """Append one token per sequence and return logits [B, vocab] (a persistent buffer)."""
        if tokens is not None:
            self.tokens.copy_(tokens, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
            return None if self.greedy_head else self.logits
        return self._step_kernels()

    def reset(self):
        self.seq_lens.zero_()

    def bind_caches(self, kv, block_table, seq_lens):
        """Run on caller-owned caches (the blocks-path contract: the caller owns the caches and threads them
        through every call, blocks/mha.py:608-612).  `kv`: one ops.PagedKV per layer sharing `block_table`
        [B, pages] and `seq_lens` [B].  A captured graph holds the old addresses and is dropped."""
        c = self.cfg
        if len(kv) != c.num_layers or block_table.shape[0] != self.B or seq_lens.shape[0] != self.B:
            raise ValueError("caches do not match the engine (layers / batch)")
        fmt = ops.KV_FORMATS[c.kv_format]
        for x in kv:
            if x.fmt != fmt or x.hkv != self.Hkv_local or x.head_dim != c.head_dim:
                raise ValueError("cache format / geometry differs from the engine's")
            if x.block_table is not block_table or x.seq_lens is not seq_lens:
                raise ValueError("all layers must share one block table and one seq_lens tensor")
        self.kv, self.block_table, self.seq_lens = list(kv), block_table, seq_lens
        self.pages_per_seq = block_table.shape[1]
        self.max_seq_len = min(self.max_seq_len, self.pages_per_seq * ops.PAGE)
        self.graph = None

    def check_status(self):
        """Raise if any bounded device-side wait of the step's kernels ran out since the last check
        (the kernels then return early and the results of that step are not to be trusted).  Synchronises;
        generate() calls it once at the end, long-running callers every so many steps."""
        words = {"linear": self.lin_ws[:4], "mlp": self.mlp_ws[:4], "attention": self.attn_ws[ops.ATTN_STATUS_OFFSET:ops.ATTN_STATUS_OFFSET + 4]}
        if self.head_ws is not None:
            words["head"] = self.head_ws[:4]
        bad = {k: int(v.view(torch.int32).item()) for k, v in words.items()}
        if self.peer is not None:
            bad["peer all-reduce"] = int(self.peer.status())
        bad = {k: v for k, v in bad.items() if v}
        if bad:
            for v in words.values():
                v.zero_()
            if self.peer is not None:
                self.peer.clear_status()
            raise ops.Tsb200Error(ops._lib.ERR_TIMEOUT, "a bounded device-side wait ran out: " +
                                  ", ".join(f"{k} status {v}" for k, v in bad.items()))

    @torch.no_grad()
    def prefill(self, input_ids):
        """Batched prompt pass (single GPU): all T prompt tokens of every sequence go through the packed
        linears at once (M = B * T rows), K and V are rotated, quantized and appended for the whole chunk
        (FP8: the per-sequence scales are taken over the prompt first, amax / 448, and then frozen), and the
        causal attention of the chunk reads the DEQUANTIZED cache: bf16 engines on the tcgen05 prefill kernel
        (`tsb200_kv_gather_heads` + `tsb200_prefill_attn`), fp32 engines on the paged decode kernel with one
        one-token "sequence" per query.  Leaves the engine in the state the token-by-token prompt loop leaves it
        in: logits / next_tokens of the last prompt token, seq_lens == T.  Starts from an empty cache."""
        c = self.cfg
        if c.tp_world > 1:
            raise NotImplementedError("batched prefill is single-GPU; tensor-parallel engines feed the prompt stepwise")
        ids = input_ids.to(self.device)
        B, T = ids.shape
        if B != self.B or T < 1 or T > self.max_seq_len:
            raise ValueError("prompt does not fit the engine")
        H, Hkv, d = self.H_local, self.Hkv_local, c.head_dim
        self.reset()
        zeros = torch.zeros_like(self.seq_lens)
        rope = (self.cos, self.sin)
        resid = self.embed[ids.reshape(-1)].contiguous()                # [B*T, hidden]
        delta = None
        for li, L in enumerate(self.layers):
            xn = ops.add_rmsnorm(resid, delta, L.ln1, c.rms_eps, c.norm_variant)
            if L.qkv is not None:
                qkv = L.qkv(xn)
                q4 = qkv[:, :H * d].unflatten(1, (H, d)).unflatten(0, (B, T))
                k4 = qkv[:, H * d:(H + Hkv) * d].unflatten(1, (Hkv, d)).unflatten(0, (B, T))
                v4 = qkv[:, (H + Hkv) * d:].unflatten(1, (Hkv, d)).unflatten(0, (B, T))
            else:
                q4, k4, v4 = L.q(xn).view(B, T, H, d), L.k(xn).view(B, T, Hkv, d), L.v(xn).view(B, T, Hkv, d)
            q4, k4, v4 = q4.contiguous(), k4.contiguous(), v4.contiguous()
            kv = self.kv[li]
            if kv.k_scale is not None:
                kv.set_fp8_scales(k4, v4, rope=rope, pos0=zeros)
            kv.rope_append(q4, k4, v4, rope, seq_lens=zeros)            # q4 rotated in place
            self.seq_lens.fill_(T)
            # causal attention of the chunk over the DEQUANTIZED cache (what every attention read sees)
            att = ops.prefill_attention(kv, q4, T, status=self.attn_ws[ops.ATTN_STATUS_OFFSET:ops.ATTN_STATUS_OFFSET + 4])
            delta = L.o(att.view(B * T, H * d))
            xn = ops.add_rmsnorm(resid, delta, L.ln2, c.rms_eps, c.norm_variant)
            delta = L.mlp(xn)
        last = resid.view(B, T, -1)[:, -1].contiguous()
        dl = delta.view(B, T, -1)[:, -1].contiguous()
        self.resid.copy_(last)
        ops.add_rmsnorm(self.resid, dl, self.final_norm, c.rms_eps, c.norm_variant, out=self.xn)
        self.lm_head(self.xn, out=self.logits, ws=self.lin_ws)
        torch.argmax(self.logits, dim=-1, out=self.next_tokens)
        self.seq_lens.fill_(T)
        return self.logits

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens, batched_prefill=None):
        """Greedy decoding.  The prompt is fed one token at a time through the decode step (as the
        reference's blocks path does, examples/04_cache_impl_export_interface.py:128-139) or, with
        `batched_prefill=True`, in one pass by `prefill()`.  Default: stepwise, except for FP8 pages, whose
        per-sequence scales are DEFINED as amax / 448 over the prompt - only the one-pass prefill can take
        them layer by layer, so it is the default there.  Stepwise FP8 is refused unless the scales were set
        beforehand (PagedKV.fill_fp8_scales / set_fp8_scales)."""
        ids = input_ids.to(self.device)
        B, T = ids.shape
        if B != self.B:
            raise ValueError(f"engine was built for batch {self.B}, got {B}")
        fp8 = self.cfg.kv_format == "fp8"
        if batched_prefill is None:
            batched_prefill = fp8 and self.cfg.tp_world == 1 and not all(kv.fp8_scales_set for kv in self.kv)
        if batched_prefill:
            self.prefill(ids)
        else:
            if fp8 and not all(kv.fp8_scales_set for kv in self.kv):
                raise ValueError("FP8 pages: the per-sequence scales are unset (placeholders 1.0); use "
                                 "batched_prefill=True or set them with PagedKV.fill_fp8_scales")
            self.reset()
            for t in range(T):
                self.step(ids[:, t])
        prefill_logits = self.logits.clone()
        out = [ids]
        for _ in range(max_new_tokens):
            nxt = self.next_tokens.clone()
            out.append(nxt[:, None])
            self.step(nxt)
        self.check_status()
        return torch.cat(out, dim=1), prefill_logits
