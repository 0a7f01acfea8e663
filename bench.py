"""Benchmark of the compressed decode hot path.

Workload (BASELINE.json configs[3]): Llama-3-8B architecture (32 layers, hidden 4096, 32 query /
8 KV heads, head_dim 128, MLP 14336, vocab 128256), bf16 activations; every MLP linear low-rank
at 25% of full rank (r = 1024); every block linear 4-bit per-channel fixed point; lm_head dense
bf16; FP8-e4m3 paged KV cache (page 16).  Batch 32 sequences PER GPU with a 2048-token context,
greedy decode.  One "step" = one decode step of the whole batch (32 new tokens per GPU).
Weights are seeded random factors and the prompt KV is seeded random data of that shape
(`data: synthetic`): there is no checkpoint or dataset in this environment.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Multi-GPU (torchrun, one rank per GPU): independent replicas, sequences sharded by rank, no
data-path collective (weak scaling); time = max over ranks of the CUDA-event time.
`--impl reference` times the reference's CPU path (PyTorch CPU ops restated in oracle/) on a
bounded sample of the same workload on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA3_8B = dict(num_layers=32, hidden=4096, num_heads=32, num_kv_heads=8, head_dim=128, intermediate=14336,
                 vocab=128256, rope_theta=5e5, rms_eps=1e-5)
# Kernel that serves each KV format, and dram__bytes_read.sum + dram__bytes_write.sum per algorithmic
# byte from an ncu capture of that kernel (profiles/decode_attn_fp8_mma_b32_ctx4096.md: 269.84 MB +
# 5.07 MB against 268.4 MB algorithmic; profiles/decode_attn_mma_f16widen_fp8_b32_ctx4096.md for the
# f16-widening kernel).  The traffic of these kernels grows in proportion to the KV bytes.
ATTN_KERNEL = {"fp8": "decode_attn_fp8_kernel (split merge fused)", "int8": "decode_attn_mma_kernel (split merge fused)"}
NCU_DRAM_PER_ALG_BYTE = {"fp8": (269.84 + 5.07) / 268.4}
METRIC = "decode tokens/s (Llama-3-8B LRD+W4+FP8-KV)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=32, help="sequences per GPU")
    ap.add_argument("--context", type=int, default=2048, help="prompt tokens already in the cache")
    ap.add_argument("--layers", type=int, default=LLAMA3_8B["num_layers"])
    ap.add_argument("--rank", type=int, default=1024, help="LRD rank of the MLP linears")
    ap.add_argument("--wbits", type=int, default=4)
    ap.add_argument("--kv", default="fp8")
    ap.add_argument("--parallel", default="replica", choices=["replica", "tp"],
                    help="N > 1: independent replicas (sequences sharded, no collective; the default the scaling run uses) "
                         "or tensor-parallel linears with an NCCL all-reduce (one batch shared by all ranks)")
    ap.add_argument("--tp-allreduce", default="peer", choices=["peer", "nccl"],
                    help="tensor parallel: the library's fused all-reduce + add + RMSNorm over NVLink peer memory, or NCCL")
    ap.add_argument("--sweep", default=None, choices=["linear", "attention"],
                    help="op-level sweeps (BASELINE.json configs[1] / configs[2]) instead of the decode step; "
                         "prints one JSON line per case")
    ap.add_argument("--sweep-m", default="1,16,128,2048", help="token counts of the linear sweep")
    ap.add_argument("--sweep-ctx", default="4096,16384,32768", help="contexts of the attention sweep")
    ap.add_argument("--sweep-batch", type=int, default=64)
    return ap.parse_args()


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


# ------------------------------------------------------------------------------ model
def algorithmic_bytes(a, context):
    """Bytes one decode step must move per GPU: packed weights + scales + lm_head + KV pages."""
    c = LLAMA3_8B
    H, Hkv, d, hid, inter = c["num_heads"], c["num_kv_heads"], c["head_dim"], c["hidden"], c["intermediate"]
    wb = a.wbits / 8.0
    attn_w = ((H + 2 * Hkv) * d * hid + hid * H * d) * wb + ((H + 2 * Hkv) * d + hid) * 4
    mlp_w = (2 * (inter * a.rank + a.rank * hid) + (hid * a.rank + a.rank * inter)) * wb + (2 * (inter + a.rank) + hid + a.rank) * 4
    kv_elem = {"fp8": 1.0, "int8": 1.0 + 4.0 / d, "nvfp4": 0.5625, "bf16": 2.0}[a.kv]
    kv = a.batch * context * 2 * Hkv * d * kv_elem
    lm = c["vocab"] * hid * 2
    return a.layers * (attn_w + mlp_w + kv) + lm, a.batch * context * 2 * Hkv * d * kv_elem


def build_engine(a, device, seed, tp_world=1, tp_rank=0):
    import torch
    from transformer_surgeon_b200 import ops
    from transformer_surgeon_b200.decoder import CompressedDecoder, DecoderConfig, LayerWeights, fuse_rows
    c = dict(LLAMA3_8B)
    c["num_layers"] = a.layers
    max_seq = a.context + a.steps + a.warmup + 16
    cfg = DecoderConfig(dtype=torch.bfloat16, kv_format=a.kv, max_positions=max_seq + 16, tp_world=tp_world, tp_rank=tp_rank, **c)
    g = torch.Generator(device=device).manual_seed(seed)
    dt = torch.bfloat16
    H, Hkv, d, hid, inter = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden, cfg.intermediate

    def rnd(rows, cols, std):
        return (torch.randn((rows, cols), generator=g, device=device) * std).to(dt)

    def qfactor(rows, cols, std):
        return ops.Factor.quantize(rnd(rows, cols, std), a.wbits, "per_channel")

    def lrd(out, inn):      # U [out, r], V [r, in]: product has the scale of a N(0, 0.02^2) dense weight
        return ops.PackedLinear(qfactor(out, a.rank, 0.02 * (inn / a.rank) ** 0.5 / 4), qfactor(a.rank, inn, 0.25 / inn ** 0.5 * 4), None, dt)

    layers = []
    for _ in range(a.layers):
        fq, fk, fv = qfactor(H * d, hid, 0.02), qfactor(Hkv * d, hid, 0.02), qfactor(Hkv * d, hid, 0.02)
        o = ops.PackedLinear(qfactor(hid, H * d, 0.02), None, None, dt)
        ones = torch.ones(hid, dtype=dt, device=device)
        if tp_world > 1:     # the engine shards q/k/v/o/gate/up/down itself (and fuses the local q|k|v again)
            mk = lambda f: ops.PackedLinear(f, None, None, dt)
            layers.append(LayerWeights(ones, ones.clone(), o, lrd(inter, hid), lrd(inter, hid), lrd(hid, inter),
                                       q=mk(fq), k=mk(fk), v=mk(fv)))
        else:
            layers.append(LayerWeights(ones, ones.clone(), o, lrd(inter, hid), lrd(inter, hid), lrd(hid, inter),
                                       qkv=fuse_rows([fq, fk, fv], [None] * 3, dt)))
    embed = rnd(cfg.vocab, hid, 0.02)
    lm_head = ops.PackedLinear(ops.Factor.dense(rnd(cfg.vocab, hid, 0.02)), None, None, dt)
    dec = CompressedDecoder(cfg, embed, layers, torch.ones(hid, dtype=dt, device=device), lm_head, a.batch, max_seq, device)
    # synthetic prompt KV of the benchmark's shape: N(0,1) with 4 outlier channels per head (x20)
    B = a.batch
    chunk = 512
    Hkv = dec.Hkv_local
    outl = torch.ones((Hkv, d), device=device)
    for h in range(Hkv):
        outl[h, torch.randperm(d, generator=g, device=device)[:4]] = 20.0
    for kv in dec.kv:
        if a.kv == "fp8":
            kv.k_scale.fill_(20.0 * 5.5 / 448.0)
            kv.v_scale.fill_(20.0 * 5.5 / 448.0)
        dec.seq_lens.zero_()
        for t0 in range(0, a.context, chunk):
            n = min(chunk, a.context - t0)
            k = (torch.randn((B, n, Hkv, d), generator=g, device=device) * outl).to(dt)
            v = (torch.randn((B, n, Hkv, d), generator=g, device=device) * outl).to(dt)
            kv.append(k, v)
            dec.seq_lens.add_(n)
    torch.cuda.synchronize()
    return dec


def time_attention_kernel(dec, a, reps=5):
    """CUDA-event time of one decode-attention call (split kernel + reducer).  The calls for all
    layers are captured in one CUDA graph (so the host launch rate does not limit the measurement)
    and cycle through the layers' caches, so no launch finds its pages in L2 (one layer's cache is
    larger than L2)."""
    import torch
    from transformer_surgeon_b200 import ops
    c = dec.cfg
    q = torch.randn((dec.B, dec.H_local, c.head_dim), device=dec.device).to(c.dtype)
    out = torch.empty_like(q)
    for kv in dec.kv[:2]:
        ops.paged_decode_attention(kv, q, dec.max_seq_len, out=out, ws=dec.attn_ws)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for kv in dec.kv:
            ops.paged_decode_attention(kv, q, dec.max_seq_len, out=out, ws=dec.attn_ws)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * len(dec.kv))


def time_mlp_kernel(dec, reps=5):
    """CUDA-event time of one fused gated-MLP launch (linear_tcq_kernel, four phases), cycling through the
    layers' weights inside one CUDA graph so that no launch finds its weights in L2 when the model is deep."""
    import torch
    x = torch.randn((dec.B, dec.cfg.hidden), device=dec.device).to(dec.cfg.dtype)
    out = torch.empty_like(x)
    for L in dec.layers[:2]:
        L.mlp(x, out=out, ws=dec.mlp_ws)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for L in dec.layers:
            L.mlp(x, out=out, ws=dec.mlp_ws)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * len(dec.layers))


# ------------------------------------------------------------------------------ CPU reference arm
def cpu_reference_sample(a, steps, warmup):
    """One decoder layer of the workload at full width on the host cores, the way the reference runs
    it: LinearCompressed.forward on dequantized bf16 factors (blocks/linear_compressed.py:81-105),
    attention() over a dense cache per sequence (blocks/mha.py:9-103), RMSNorm, SwiGLU, plus the
    lm_head; per-layer time is scaled to the full depth.  Returns (tokens/s, sample description)."""
    import torch
    from oracle import linear as olin, attention as oatt
    torch.set_num_threads(os.cpu_count() or 1)
    c = LLAMA3_8B
    H, Hkv, d, hid, inter = c["num_heads"], c["num_kv_heads"], c["head_dim"], c["hidden"], c["intermediate"]
    B, L, r = a.batch, a.context, a.rank
    g = torch.Generator().manual_seed(0)
    dt = torch.bfloat16
    rn = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dt)
    wq, wk, wv, wo = rn(H * d, hid), rn(Hkv * d, hid), rn(Hkv * d, hid), rn(hid, H * d)
    ug, vg, uu, vu, ud, vd = rn(inter, r), rn(r, hid), rn(inter, r), rn(r, hid), rn(hid, r), rn(r, inter)
    lm = rn(c["vocab"], hid)
    w1 = torch.ones(hid, dtype=dt)
    kc = torch.randn(B, L + 1, Hkv, d, generator=g).to(dt)
    vc = torch.randn(B, L + 1, Hkv, d, generator=g).to(dt)
    cos, sin = oatt.rope_tables(d, c["rope_theta"], torch.arange(L, L + 1))
    x = torch.randn(B, hid, generator=g).to(dt)

    def layer(x):
        xn = oatt.rmsnorm_hf(x, w1, c["rms_eps"])
        q = olin.linear_compressed_forward(xn, wq).view(B, 1, H, d)
        k = olin.linear_compressed_forward(xn, wk).view(B, 1, Hkv, d)
        v = olin.linear_compressed_forward(xn, wv).view(B, 1, Hkv, d)
        q, k = oatt.apply_rope(q, cos, sin), oatt.apply_rope(k, cos, sin)
        kc[:, L] = k[:, 0]
        vc[:, L] = v[:, 0]
        att = torch.stack([oatt.attention(q[b], kc[b], vc[b])[:, 0] for b in range(B)]).to(dt)
        h = x + olin.linear_compressed_forward(att.reshape(B, H * d), wo)
        hn = oatt.rmsnorm_hf(h, w1, c["rms_eps"])
        m = oatt.swiglu(olin.linear_compressed_forward(hn, ug, None, vg), olin.linear_compressed_forward(hn, uu, None, vu))
        return h + olin.linear_compressed_forward(m, ud, None, vd)

    def head(x):
        return torch.argmax(olin.linear_compressed_forward(oatt.rmsnorm_hf(x, w1, c["rms_eps"]), lm), dim=-1)

    with torch.no_grad():
        for _ in range(warmup):
            layer(x); head(x)
        t0 = time.perf_counter()
        for _ in range(steps):
            layer(x)
        t_layer = (time.perf_counter() - t0) / steps
        t0 = time.perf_counter()
        for _ in range(steps):
            head(x)
        t_head = (time.perf_counter() - t0) / steps
    step_s = a.layers * t_layer + t_head
    sample = (f"1 decoder layer (batch {B}, context {L}, dense bf16 KV, dequantized bf16 factors) x{steps} "
              f"+ lm_head, scaled to {a.layers} layers; torch CPU, {os.cpu_count()} threads")
    return B / step_s, step_s * 1e3, sample


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = min(a.steps, 3), min(a.warmup, 1)
    tps, ms, sample = cpu_reference_sample(a, steps, max(warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama3-8b-arch decode, MLP LRD r=%d, W%d, batch %d, context %d (CPU: dense bf16 KV)" % (a.rank, a.wbits, a.batch, a.context)},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------ GPU arm
def run_ours(a):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))
    import __graft_entry__ as ge
    if not os.path.exists(os.path.join(ROOT, "transformer-surgeon_b200", "libtsb200.so")):
        ge.build()
    tp = a.parallel == "tp" and world > 1
    dec = build_engine(a, device, seed=1 if tp else 1 + rank, tp_world=world if tp else 1, tp_rank=rank if tp else 0)
    peer_ar = False
    if tp and a.tp_allreduce == "peer":
        try:
            peer_ar = dec.enable_peer_allreduce()
        except RuntimeError as ex:           # raised on every rank alike: all of them stay on NCCL
            if rank == 0:
                print("peer all-reduce unavailable, using NCCL: %s" % ex, file=sys.stderr)
    dec.capture()
    B = a.batch
    tgen = torch.Generator().manual_seed(7 if tp else 7 + rank)     # tensor parallel: every rank feeds the same tokens
    tok_host = torch.randint(0, dec.cfg.vocab, (B,), generator=tgen, dtype=torch.int64).pin_memory()
    out_host = torch.empty(B, dtype=torch.int64).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident steps (inputs already in HBM): `value`
    dec.tokens.copy_(tok_host)
    for _ in range(a.warmup):
        dec.step()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = int(dec.seq_lens[0].item())
    e0.record()
    for _ in range(a.steps):
        dec.step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    # ---- end to end through the public call: host tokens in, host tokens out, every step
    saved = dec.seq_lens.clone()
    dec.seq_lens.fill_(a.context)          # rewind: same contexts as the device-timed steps
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(a.steps):
        dec.step(tok_host)                                  # H2D of the step's input tokens
        out_host.copy_(dec.next_tokens, non_blocking=True)  # D2H of the step's result
        torch.cuda.current_stream().synchronize()
        tok_host.copy_(out_host)                            # greedy feedback on the host
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    dec.seq_lens.copy_(saved)
    # per-kernel timing captures a second CUDA graph; kept out of the tensor-parallel mode, whose ranks
    # must stay in lockstep on the NCCL communicator
    t_attn = time_attention_kernel(dec, a) if not tp else None   # tensor parallel: the kernel is not timed alone
    t_mlp = time_mlp_kernel(dec) if not tp else None
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        peak, which = peaks()
        ctx_mid = ctx0 + a.steps // 2
        step_bytes, attn_bytes = algorithmic_bytes(a, ctx_mid)
        attn_alg = algorithmic_bytes(a, int(dec.seq_lens[0].item()))[1]
        achieved = attn_alg / (t_attn * 1e-3) / 1e9 if t_attn else None
        seqs = B if tp else world * B                  # tensor parallel: one batch shared by all ranks
        tps = seqs * a.steps / (ms * 1e-3)
        line = {"metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "llama3-8b-arch decode: %d layers, MLP LRD r=%d, W%d per-channel, %s paged KV, "
                           "batch %d/GPU, context %d->%d" % (a.layers, a.rank, a.wbits, a.kv, B, ctx0, ctx0 + a.steps),
                           "sharding": ("tensor parallel x%d: heads / MLP columns split, 2 all-reduces per layer (%s), batch %d shared"
                                        % (world, "fused with add + RMSNorm over NVLink peer loads" if peer_ar else "NCCL", B))
                           if tp else "replicas, %d sequences per GPU, no collective" % B,
                           "l2": "inputs larger than L2 (%.1f GB read per step)" % (step_bytes / 1e9),
                           "cuda_graph": True},
                "e2e": {"value": seqs * a.steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
                "gpu_launches": dec.kernel_launches_per_step * a.steps,
                "clocks": clocks,
                "roofline": {"kernel": ATTN_KERNEL.get(a.kv, "decode_attn_simt_kernel"), "bound": "hbm", "achieved": achieved,
                             "peak": peak, "unit": "GB/s", "frac": achieved / peak if achieved else None, "peak_source": which,
                             "traffic": (attn_alg * NCU_DRAM_PER_ALG_BYTE[a.kv]) if a.kv in NCU_DRAM_PER_ALG_BYTE else None,
                             "traffic_source": "dram bytes of one ncu capture (batch 32 x context 4096) scaled by algorithmic bytes",
                             "ms_per_launch": t_attn,
                             "step_achieved": step_bytes / (ms / a.steps * 1e-3) / 1e9,
                             "step_frac": step_bytes / (ms / a.steps * 1e-3) / 1e9 / peak}}
        if t_mlp:
            # the other large kernel of the step, for the record: the fused gated MLP moves its packed weights once
            # per launch and is bound by dependent latencies (phases, split-K rendezvous), not by HBM
            c = LLAMA3_8B
            mlp_bytes = 3 * (c["intermediate"] * a.rank + a.rank * c["hidden"]) * a.wbits / 8.0
            line["roofline_mlp"] = {"kernel": "linear_tcq_kernel (gated MLP: 4 GEMM phases in one launch)", "bound": "hbm",
                                    "achieved": mlp_bytes / (t_mlp * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                    "frac": mlp_bytes / (t_mlp * 1e-3) / 1e9 / peak, "ms_per_launch": t_mlp}
        try:
            cpu_tps, _, sample = cpu_reference_sample(a, 2, 1) if world == 1 else (None, None, None)
            if cpu_tps is not None:
                line["cpu_baseline"] = {"value": cpu_tps, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                        "sample": sample}
        except Exception as ex:  # the CPU leg must not hide the GPU result
            line["cpu_baseline"] = {"value": None, "error": repr(ex)}
        print(json.dumps(line))
    if world > 1:
        if tp:
            # the captured step holds NCCL work: drop the graph and leave without tearing the communicator
            # down (destroying the group with a live graph has been seen to block at exit)
            dec.graph = None
            torch.cuda.synchronize()
            sys.stdout.flush()
            os._exit(0)
        dist.destroy_process_group()


def _graph_time_us(fn, copies, reps=5):
    """Average time of fn(i), i = 0..copies-1, replayed from one CUDA graph (CUDA events)."""
    import torch
    for i in range(min(2, copies)):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(copies):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / (reps * copies)


def sweep_linear(a):
    """configs[1]: x [M, 4096] bf16, W 4096x4096 factored at r in {256, 1024}, factors at 8 / 4 bits and
    binary; time of LinearCompressed.forward per call, TFLOP/s and GB/s against the measured peaks."""
    import torch
    from transformer_surgeon_b200 import ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2)
    peak_bw, _ = peaks()
    for r in (256, 1024):
        for p in (8, 4, "binary"):
            n_copies = 8          # distinct weight copies: 8 x (r x 8192 codes) > L2 only for the larger cases; stated per line
            lins = []
            for _ in range(n_copies):
                U = (torch.randn((4096, r), generator=g, device=dev) * 0.02).bfloat16()
                V = (torch.randn((r, 4096), generator=g, device=dev) * 0.02).bfloat16()
                lins.append(ops.PackedLinear(ops.Factor.quantize(U, p), ops.Factor.quantize(V, p), None, torch.bfloat16))
            bits = lins[0].u.bits
            for M in [int(v) for v in a.sweep_m.split(",")]:
                x = torch.randn((M, 4096), generator=g, device=dev).bfloat16()
                y = torch.empty((M, 4096), dtype=torch.bfloat16, device=dev)
                ws = torch.zeros(lins[0].workspace_bytes(M), dtype=torch.uint8, device=dev)
                us = _graph_time_us(lambda i: lins[i](x, out=y, ws=ws), n_copies)
                flops = 2.0 * M * r * 8192
                byts = r * 8192 * bits / 8 + (4096 + r) * 4 + 2 * M * 4096 * 2
                print(json.dumps({"sweep": "linear", "M": M, "rank": r, "precision": p, "container_bits": bits,
                                  "us_per_call": us, "tflops": flops / us / 1e6, "gbs": byts / us / 1e3,
                                  "frac_hbm": byts / us / 1e3 / peak_bw, "frac_tensor_burst": flops / us / 1e6 / 1671.9,
                                  "weights_mb_cycled": n_copies * r * 8192 * bits / 8 / 1e6}))


def sweep_attention(a):
    """configs[2]: 32 q heads / 8 kv heads / d 128, batch 64, page 16, seeded random block table, K/V
    N(0,1) with 4 outlier channels per head (x20); decode attention and single-token append per format."""
    import torch
    from transformer_surgeon_b200 import ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    peak_bw, _ = peaks()
    B, H, Hkv, d = a.sweep_batch, 32, 8, 128
    outl = torch.ones((Hkv, d), device=dev)
    for h in range(Hkv):
        outl[h, torch.randperm(d, generator=g, device=dev)[:4]] = 20.0
    for L in [int(v) for v in a.sweep_ctx.split(",")]:
        for fmt in ("int8", "fp8", "nvfp4"):
            pages = L // 16 + 1
            rec = ops.kv_record_bytes(ops.KV_FORMATS[fmt], d)
            layers = max(1, min(4, int(3e9 // (B * pages * Hkv * rec * 2))))     # a few GB on the device at most
            kvs = []
            seq = torch.zeros(B, dtype=torch.int32, device=dev)
            bt = torch.randperm(B * pages, generator=g, device=dev).to(torch.int32).reshape(B, pages)
            for _ in range(layers):
                kv = ops.PagedKV(fmt, B * pages, Hkv, d, bt, seq, dev)
                if fmt == "fp8":
                    kv.k_scale.fill_(110.0 / 448)
                    kv.v_scale.fill_(110.0 / 448)
                seq.zero_()
                for t0 in range(0, L, 1024):
                    n = min(1024, L - t0)
                    k = (torch.randn((B, n, Hkv, d), generator=g, device=dev) * outl).bfloat16()
                    v = (torch.randn((B, n, Hkv, d), generator=g, device=dev) * outl).bfloat16()
                    kv.append(k, v)
                    seq += n
                kvs.append(kv)
            q = torch.randn((B, H, d), generator=g, device=dev).bfloat16()
            out = torch.empty_like(q)
            ws = torch.zeros(ops.decode_attn_workspace_bytes(B, H, d, L + 16), dtype=torch.uint8, device=dev)
            us = _graph_time_us(lambda i: ops.paged_decode_attention(kvs[i], q, L + 16, out=out, ws=ws), layers, reps=4)
            byts = B * (L // 16) * Hkv * rec * 2 + B * (L // 16) * 4 + 2 * B * H * d * 2
            k1 = torch.randn((B, 1, Hkv, d), generator=g, device=dev).bfloat16()
            us_app = _graph_time_us(lambda i: kvs[i].append(k1, k1), layers, reps=4)
            app_bytes = B * 2 * Hkv * d * (2 + rec / (16.0 * d))
            print(json.dumps({"sweep": "attention", "format": fmt, "batch": B, "context": L, "decode_us": us,
                              "decode_gbs": byts / us / 1e3, "decode_frac_hbm": byts / us / 1e3 / peak_bw,
                              "pages_mb": byts / 1e6, "append_us": us_app, "append_gbs": app_bytes / us_app / 1e3,
                              "layers_cycled": layers}))
            del kvs


if __name__ == "__main__":
    args = parse()
    if args.sweep:
        import torch
        torch.cuda.set_device(0)
        (sweep_linear if args.sweep == "linear" else sweep_attention)(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
