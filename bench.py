"""Benchmark of the compressed decode hot path.

Workload (BASELINE.json configs[3]): Llama-3-8B architecture (32 layers, hidden 4096, 32 query /
8 KV heads, head_dim 128, MLP 14336, vocab 128256), bf16 activations; every MLP linear low-rank
at 25% of full rank (r = 1024); every block linear 4-bit per-channel fixed point; lm_head dense
bf16 (it is a separate `final_layer` scheme in the reference, utils/manager.py:1021-1046, which the
configuration's "all linears" does not reach); FP8-e4m3 paged KV cache (page 16).  Batch 32 sequences
PER GPU with a 2048-token context, greedy decode.  One "step" = one decode step of the whole batch
(32 new tokens per GPU).  Weights are seeded random factors and the prompts are seeded random token ids
(`data: synthetic`): there is no checkpoint or dataset in this environment.  The 2048-token prompts go through the
engine's own batched prefill before the timed decode steps (`prefill` record: its time and throughput;
`--prompt synthetic` appends random K/V of the config-3 distribution instead, as the tensor-parallel leg does).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

JSON line of the GPU arm: `value` = device-resident graph-replayed steps, `e2e` = the same through
`CompressedDecoder.step(host tokens)` with the copies inside the timed region; `roofline` = the kernel with
the largest share of the step (the packed-weight GEMM kernel: its three launches per layer timed one by one),
`roofline_attention` = the decode-attention launch; fractions against the measured copy bandwidth
(`frac`) and against the 8 TB/s nominal figure (`frac_nominal`); `sweeps` = op-level cases of
configs[1] / configs[2] (N = 1 only); `cpu_baseline` = a bounded sample of the reference's CPU path.
Multi-GPU (torchrun, one rank per GPU): independent replicas, sequences sharded by rank, no
data-path collective (weak scaling); time = max over ranks of the CUDA-event time; for N > 1 a `tp`
record follows from a second, tensor-parallel engine over the same ranks (one batch of 32 shared:
strong scaling).
`--impl reference` times the reference's own CPU code (oracle/_ref; oracle/ref_decode.py) on the host
cores: `--steps` full-depth decode steps of the same workload.
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
# Kernel that serves each KV format, and DRAM bytes (read + write) per algorithmic byte from one ncu capture
# of that kernel on a smaller case (batch 32 x context 4096: 274.9 MB against 268.4 MB algorithmic; packed
# GEMMs of one layer: 50.5 MB against 49.3 MB).  The traffic of these kernels grows in proportion to the bytes.
ATTN_KERNEL = {"fp8": "decode_attn_fp8_kernel (split merge fused)", "int8": "decode_attn_mma_kernel (split merge fused)"}
NCU_DRAM_PER_ALG_BYTE = {"fp8": (269.84 + 5.07) / 268.4}
NCU_DRAM_PER_ALG_BYTE_LINEAR = (12.940 + 8.738 + 28.788) / (12.58 + 8.39 + 28.31)
HBM_NOMINAL_GBS = 8000.0
METRIC = "decode tokens/s (Llama-3-8B LRD+W4+FP8-KV)"


_RESULT_OUT = None


def divert_stdout():
    """Whatever a library writes to stdout during the run (NCCL prints its version there) goes to stderr; the result
    line alone reaches the real stdout through emit()."""
    global _RESULT_OUT
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(text):
    out = _RESULT_OUT or sys.stdout
    out.write(text + "\n")
    out.flush()


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
    ap.add_argument("--sweep", default=None, choices=["linear", "attention", "prefill"],
                    help="op-level sweeps (BASELINE.json configs[1] / configs[2]) instead of the decode step; "
                         "prints one JSON line per case")
    ap.add_argument("--sweep-m", default="1,16,128,2048", help="token counts of the linear sweep")
    ap.add_argument("--sweep-ranks", default="256,1024", help="ranks of the linear sweep")
    ap.add_argument("--sweep-precisions", default="8,4,binary", help="factor precisions of the linear sweep")
    ap.add_argument("--sweep-ctx", default="4096,16384,32768", help="contexts of the attention sweep")
    ap.add_argument("--sweep-batch", type=int, default=64)
    ap.add_argument("--prompt", default="real", choices=["synthetic", "real"],
                    help="real: the cache is filled by the engine's own batched prefill of random prompt tokens "
                         "(timed, reported as `prefill`), not by appending synthetic K/V")
    ap.add_argument("--no-sweeps", action="store_true", help="N = 1: leave the op-level `sweeps` records out of the line")
    ap.add_argument("--config", default="c4", choices=["c4", "c5"],
                    help="c4 (default, the headline): Llama-3-8B architecture; c5: Qwen2.5-VL-7B text tower with per-layer "
                         "precisions / ranks and an NVFP4 cache (one GPU, decode steps only; BASELINE.json configs[4])")
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
        self.index, self.rows, self.proc, self.t_begin = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")] + [time.monotonic()])

    def wait_first(self, limit_s=3.0):
        """Blocks until the first sample has arrived (the tool needs a moment to start), at most limit_s."""
        t0 = time.monotonic()
        while self.proc is not None and not self.rows and time.monotonic() - t0 < limit_s:
            time.sleep(0.01)

    def mark_begin(self):
        """Start of the timed region: only samples that arrive from here on are reported (the sampler itself is
        started ahead of the warm-up steps, so that it is already streaming by then)."""
        self.t_begin = time.monotonic()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        rows = [r for r in self.rows if self.t_begin is None or r[-1] >= self.t_begin]
        mhz = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 2 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[2 + i] == "Active" for r in rows)]
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
    dec.greedy_head = True                # greedy decode: the step ends in the fused lm_head + argmax (no logits in memory)
    # synthetic prompt KV of the benchmark's shape: N(0,1) with 4 outlier channels per head (x20)
    B = a.batch
    chunk = 512
    Hkv = dec.Hkv_local
    outl = torch.ones((Hkv, d), device=device)
    for h in range(Hkv):
        outl[h, torch.randperm(d, generator=g, device=device)[:4]] = 20.0
    for kv in dec.kv:
        if a.kv == "fp8":
            kv.fill_fp8_scales(20.0 * 5.5 / 448.0, 20.0 * 5.5 / 448.0)
        dec.seq_lens.zero_()
        for t0 in range(0, a.context, chunk):
            n = min(chunk, a.context - t0)
            k = (torch.randn((B, n, Hkv, d), generator=g, device=device) * outl).to(dt)
            v = (torch.randn((B, n, Hkv, d), generator=g, device=device) * outl).to(dt)
            kv.append(k, v)
            dec.seq_lens.add_(n)
    torch.cuda.synchronize()
    return dec


def _graph_time_us(fn, copies, reps=5, pdl=True):
    """Average time (us) of fn(i), i = 0..copies-1, replayed from one CUDA graph, CUDA events on the replay stream.
    The calls are captured with programmatic dependent launch, as the decode step captures them."""
    import torch
    from transformer_surgeon_b200 import ops
    for i in range(min(2, copies)):
        fn(i)
    torch.cuda.synchronize()
    old = ops.set_pdl(pdl)
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(copies):
                fn(i)
    finally:
        ops.set_pdl(old)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / (reps * copies)


def time_layer_kernels(dec, a):
    """CUDA-event time per launch of the four large kernels of a decoder layer, each replayed from a CUDA graph that
    cycles through ALL layers' weights / caches, so that no launch finds its operands in L2 (one layer's cache and
    the weights of a few layers exceed it): the three packed-weight GEMM launches (q|k|v, o_proj, the gated MLP) and
    the decode attention.  Returns microseconds."""
    import torch
    c = dec.cfg
    B, H, d = dec.B, dec.H_local, c.head_dim
    x = torch.randn((B, c.hidden), device=dec.device).to(c.dtype)
    att = torch.randn((B, H * d), device=dec.device).to(c.dtype)
    q = torch.randn((B, H, d), device=dec.device).to(c.dtype)
    out = torch.empty_like(q)
    n = len(dec.layers)
    from transformer_surgeon_b200 import ops
    t = {}
    if dec.layers[0].qkv is not None:
        t["qkv"] = _graph_time_us(lambda i: dec.layers[i].qkv(x, out=dec.qkv, ws=dec.lin_ws), n)
    t["o_proj"] = _graph_time_us(lambda i: dec.layers[i].o(att, out=dec.delta, ws=dec.lin_ws), n)
    t["mlp"] = _graph_time_us(lambda i: dec.layers[i].mlp(x, out=dec.delta, ws=dec.mlp_ws), n)
    t["attention"] = _graph_time_us(lambda i: ops.paged_decode_attention(dec.kv[i], q, dec.max_seq_len, out=out, ws=dec.attn_ws), n)
    return t


# ------------------------------------------------------------------------------ CPU reference arm
def cpu_decode(a):
    """The workload's decode step on the host cores (oracle/ref_decode.py: the reference's own classes from
    oracle/_ref when installed, else the port)."""
    from oracle import ref_decode
    c = LLAMA3_8B
    return ref_decode, ref_decode.make_decode(hidden=c["hidden"], heads=c["num_heads"], kv_heads=c["num_kv_heads"],
                                              inter=c["intermediate"], vocab=c["vocab"], rank=a.rank, batch=a.batch,
                                              context=a.context, theta=c["rope_theta"], eps=c["rms_eps"])


def cpu_baseline_sample(a):
    """Bounded sample for the GPU arm's line: 2 steps of 4 layers + lm_head, the per-layer share scaled to full depth."""
    rd, dec = cpu_decode(a)
    t_head = rd.time_steps(dec, 2, 1, 0)
    t_4 = rd.time_steps(dec, 2, 1, 4)
    step_s = (t_4 - t_head) / 4 * a.layers + t_head
    return {"value": a.batch / step_s, "unit": "tokens/s", "cores": os.cpu_count(), "kind": dec.kind,
            "sample": "2 decode steps of 4 decoder layers + lm_head (batch %d, context %d, dense bf16 KV, bf16 fake-quantized "
                      "factors), per-layer time scaled to %d layers; %d threads" % (a.batch, a.context, a.layers, os.cpu_count())}


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rd, dec = cpu_decode(a)
    step_s = rd.time_steps(dec, a.steps, a.warmup, a.layers)          # every step at full depth, as many as asked for
    tps = a.batch / step_s
    sample = ("%d full-depth decode steps (%d layer calls each, one layer's weights and cache reused; batch %d, context %d, "
              "dense bf16 KV); %d threads" % (a.steps, a.layers, a.batch, a.context, os.cpu_count()))
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama3-8b-arch decode: %d layers, MLP LRD r=%d, W%d fake-quantized factors, lm_head bf16, batch %d, "
                                   "context %d (the reference has no quantized KV cache: dense bf16 KV)"
                                   % (a.layers, a.rank, a.wbits, a.batch, a.context)},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": os.cpu_count(), "kind": dec.kind, "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(json.dumps(line))


# ------------------------------------------------------------------------------ GPU arm
def layer_weight_bytes(a):
    """Algorithmic bytes of the three packed-weight GEMM launches of a layer: codes + fp32 row scales + bf16 in/out."""
    c = LLAMA3_8B
    H, Hkv, d, hid, inter, r, B = c["num_heads"], c["num_kv_heads"], c["head_dim"], c["hidden"], c["intermediate"], a.rank, a.batch
    wb = a.wbits / 8.0
    act = lambda k, n: 2.0 * B * (k + n)
    qkv_n = (H + 2 * Hkv) * d
    return {"qkv": qkv_n * hid * wb + 4 * qkv_n + act(hid, qkv_n),
            "o_proj": hid * H * d * wb + 4 * hid + act(H * d, hid),
            "mlp": 3 * (inter * r + r * hid) * wb + 4 * (2 * (inter + r) + hid + r) + act(hid, hid)}


def timed_steps(dec, a, tok_host, out_host, barrier, sampler=None):
    """(ms of K device-resident steps, ms of K end-to-end steps, context at the start)."""
    import torch
    dec.tokens.copy_(tok_host)
    if sampler is not None:
        sampler.start()
        sampler.wait_first()
    for _ in range(a.warmup):
        dec.step()
    barrier()
    if sampler is not None:
        sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = int(dec.seq_lens[0].item())
    e0.record()
    for _ in range(a.steps):
        dec.step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # ---- end to end through the public call: host tokens in, host tokens out, every step
    saved = dec.seq_lens.clone()
    dec.seq_lens.fill_(ctx0)               # rewind: same contexts as the device-timed steps
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
    return ms, ms_e2e, ctx0


def tp_leg(a, device, world, rank, barrier):
    """Tensor-parallel engine over the same ranks (one batch of `a.batch` sequences shared: strong scaling).
    Returns the record for the JSON line (rank 0) - time = max over ranks of the CUDA-event time."""
    import torch
    import torch.distributed as dist
    dec = build_engine(a, device, seed=1, tp_world=world, tp_rank=rank)
    mode = "nccl"
    if a.tp_allreduce == "peer":
        try:
            if dec.enable_peer_allreduce():
                mode = "peer"
        except RuntimeError as ex:           # raised on every rank alike: all of them stay on NCCL
            if rank == 0:
                print("peer all-reduce unavailable, using NCCL: %s" % ex, file=sys.stderr)
    dec.capture()
    tgen = torch.Generator().manual_seed(7)                 # every rank feeds the same tokens
    tok_host = torch.randint(0, dec.cfg.vocab, (a.batch,), generator=tgen, dtype=torch.int64).pin_memory()
    out_host = torch.empty(a.batch, dtype=torch.int64).pin_memory()
    ms, ms_e2e, ctx0 = timed_steps(dec, a, tok_host, out_host, barrier)
    status = dec.peer.status() if dec.peer is not None else 0
    t = torch.tensor([ms, ms_e2e, float(status)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    rec = {"ranks": world, "batch_total": a.batch, "scaling": "strong", "ms_per_step": float(t[0]) / a.steps,
           "tokens_per_s": a.batch * a.steps / (float(t[0]) * 1e-3), "e2e_tokens_per_s": a.batch * a.steps / (float(t[1]) * 1e-3),
           "allreduce": ("tsb200_peer_allreduce_add_rmsnorm: all-reduce + residual add + RMSNorm in one kernel over NVLink peer loads"
                         if mode == "peer" else "NCCL all-reduce (captured in the step graph)"),
           "collectives_per_step": 2 * a.layers, "allreduce_bytes": a.batch * LLAMA3_8B["hidden"] * 2,
           "peer_status": int(t[2]), "context": ctx0}
    # Teardown order matters: a captured graph that holds NCCL kernels keeps the communicator referenced, and tearing
    # the process group down while such a graph is alive blocks.  So: drop the graph, collect, synchronise, and only
    # then let the caller destroy the group.
    dec.graph = None
    del dec
    import gc
    gc.collect()
    torch.cuda.synchronize()
    return rec


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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if a.parallel == "tp" and world > 1:                     # tensor parallel only (development runs)
        rec = tp_leg(a, device, world, rank, barrier)
        if rank == 0:
            emit(json.dumps({"metric": METRIC, "value": rec["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
                             "warmup": a.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                             "tp": rec}))
        barrier()
        dist.destroy_process_group()
        return
    dec = build_engine(a, device, seed=1 + rank)
    prefill_rec = None
    if a.prompt == "real":
        # the prompt goes through the library: packed GEMMs at M = batch x context rows, bulk quantize-and-append, causal
        # attention on tcgen05 over the dequantized cache; the decode steps then run on the cache this leaves
        pg = torch.Generator().manual_seed(11 + rank)
        ids = torch.randint(0, dec.cfg.vocab, (a.batch, a.context), generator=pg, dtype=torch.int64).to(device)
        dec.prefill(ids[:, :min(a.context, 128)])             # warm-up of every kernel on a short prompt
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        dec.prefill(ids)
        p1.record()
        torch.cuda.synchronize()
        dec.check_status()
        pms = p0.elapsed_time(p1)
        c = LLAMA3_8B
        macs = a.layers * (c["hidden"] * (c["num_heads"] + 2 * c["num_kv_heads"]) * c["head_dim"] + c["num_heads"] * c["head_dim"] * c["hidden"]
                           + 3 * (c["hidden"] * a.rank + a.rank * c["intermediate"]))
        flops = 2.0 * macs * a.batch * a.context + a.layers * 2.0 * a.batch * c["num_heads"] * c["head_dim"] * a.context * a.context
        prefill_rec = {"prompt_tokens": a.batch * a.context, "ms": pms, "prompt_tokens_per_s": a.batch * a.context / (pms * 1e-3),
                       "tflops": flops / (pms * 1e-3) / 1e12, "frac_tensor_burst": flops / (pms * 1e-3) / 1e12 / 1671.9,
                       "what": "one batched pass of all prompt tokens through every layer (packed GEMMs, bulk append, causal "
                               "attention on tcgen05), outside the timed decode region"}
    dec.capture()
    B = a.batch
    tgen = torch.Generator().manual_seed(7 + rank)
    tok_host = torch.randint(0, dec.cfg.vocab, (B,), generator=tgen, dtype=torch.int64).pin_memory()
    out_host = torch.empty(B, dtype=torch.int64).pin_memory()
    sampler = ClockSampler(local) if rank == 0 else None
    ms, ms_e2e, ctx0 = timed_steps(dec, a, tok_host, out_host, barrier, sampler)
    t_k = time_layer_kernels(dec, a)                          # still under the clock sampler: more samples under load
    clocks = sampler.stop() if rank == 0 else None
    dec.check_status()
    launches = dec.kernel_launches_per_step
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    line, rec, done = None, None, threading.Event()
    if rank == 0:
        peak, which = peaks()
        ctx_mid = ctx0 + a.steps // 2
        step_bytes, _ = algorithmic_bytes(a, ctx_mid)
        attn_alg = algorithmic_bytes(a, int(dec.seq_lens[0].item()))[1]
        tps = world * B * a.steps / (ms * 1e-3)
        wbytes = layer_weight_bytes(a)
        lin_names = [k for k in ("qkv", "o_proj", "mlp") if k in t_k]
        lin_us = sum(t_k[k] for k in lin_names)
        lin_bytes = sum(wbytes[k] for k in lin_names)
        step_us = ms / a.steps * 1e3

        def hbm(bytes_, us):
            gbs = bytes_ / us / 1e3
            return {"achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_source": which,
                    "frac_nominal": gbs / HBM_NOMINAL_GBS, "peak_nominal": HBM_NOMINAL_GBS}

        lin_rec = {"kernel": "linear_tcq_kernel (packed-weight GEMM; 3 launches per layer: q|k|v, o_proj, gated MLP)", "bound": "hbm",
                   **hbm(lin_bytes, lin_us), "traffic": lin_bytes * NCU_DRAM_PER_ALG_BYTE_LINEAR / len(lin_names),
                   "traffic_source": "dram bytes of one ncu capture of the three launches (4-layer case), per launch, scaled by algorithmic bytes",
                   "algorithmic_bytes_per_launch": lin_bytes / len(lin_names), "ms_per_launch": lin_us / len(lin_names) * 1e-3,
                   "share_of_step": a.layers * lin_us / step_us,
                   "launches": {k: {"us": t_k[k], "bytes": wbytes[k], **hbm(wbytes[k], t_k[k])} for k in lin_names},
                   "step_achieved": step_bytes / (step_us * 1e-6) / 1e9, "step_frac": step_bytes / (step_us * 1e-6) / 1e9 / peak}
        att_rec = {"kernel": ATTN_KERNEL.get(a.kv, "decode_attn_simt_kernel"), "bound": "hbm", **hbm(attn_alg, t_k["attention"]),
                   "traffic": (attn_alg * NCU_DRAM_PER_ALG_BYTE[a.kv]) if a.kv in NCU_DRAM_PER_ALG_BYTE else None,
                   "traffic_source": "dram bytes of one ncu capture (batch 32 x context 4096) scaled by algorithmic bytes",
                   "ms_per_launch": t_k["attention"] * 1e-3, "share_of_step": a.layers * t_k["attention"] / step_us,
                   "parity": "KV formats are this project's definitions: parity unpinned"}
        dominant_linear = lin_us >= t_k["attention"]
        line = {"metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "llama3-8b-arch decode: %d layers, MLP LRD r=%d, W%d per-channel block linears, lm_head bf16, "
                           "%s paged KV, batch %d/GPU, context %d->%d" % (a.layers, a.rank, a.wbits, a.kv, B, ctx0, ctx0 + a.steps),
                           "sharding": "replicas, %d sequences per GPU, no collective" % B,
                           "l2": "inputs larger than L2 (%.1f GB read per step)" % (step_bytes / 1e9),
                           "cuda_graph": True},
                "e2e": {"value": world * B * a.steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
                "gpu_launches": launches * a.steps,
                "clocks": clocks,
                "roofline": lin_rec if dominant_linear else att_rec,
                ("roofline_attention" if dominant_linear else "roofline_linear"): att_rec if dominant_linear else lin_rec}
        if prefill_rec is not None:
            line["prefill"] = prefill_rec
            line["config"]["prompt"] = "cache filled by the engine's batched prefill of %d random tokens per sequence" % a.context
    if world == 1 and rank == 0:
        del dec
        torch.cuda.empty_cache()
        if not a.no_sweeps:
            try:
                line["sweeps"] = {"linear": sweep_linear(a, ranks=(1024,), precisions=(4,), ms=(1, 128, 2048), copies=4),
                                  "attention": sweep_attention(a, contexts=(4096,)),
                                  "prefill": sweep_prefill(a, cases=[(8, 2048)])}
            except Exception as ex:          # a sweep must not hide the headline
                line["sweeps"] = {"error": repr(ex)}
        try:
            line["cpu_baseline"] = cpu_baseline_sample(a)
        except Exception as ex:              # the CPU leg must not hide the GPU result
            line["cpu_baseline"] = {"value": None, "error": repr(ex)}
    elif world > 1:
        # second engine over the same ranks: tensor parallel, one shared batch.  A watchdog bounds the leg so that the
        # replica result is printed whatever happens to it.
        del dec
        torch.cuda.empty_cache()

        def watchdog():
            if not done.wait(240.0):
                if rank == 0:
                    line["tp"] = {"error": "tensor-parallel leg did not finish within 240 s"}
                    emit(json.dumps(line))
                os._exit(0)
        threading.Thread(target=watchdog, daemon=True).start()
        try:
            rec = tp_leg(a, device, world, rank, barrier)
        except Exception as ex:
            rec = {"error": repr(ex)}
        if rank == 0:
            line["tp"] = rec
    if rank == 0:
        emit(json.dumps(line))
    if world > 1:
        if rec is not None and "error" in rec:
            os._exit(0)                      # a failed leg may have left collectives unmatched: leave without a teardown
        barrier()
        dist.destroy_process_group()
        done.set()


QWEN25VL_7B_TEXT = dict(num_layers=28, hidden=3584, num_heads=28, num_kv_heads=4, head_dim=128, intermediate=18944,
                        vocab=152064, rope_theta=1e6, rms_eps=1e-6)


def run_c5(a):
    """BASELINE.json configs[4] on one GPU: Qwen2.5-VL-7B language-tower shapes, bf16, per-layer weight precision drawn
    with seed 2 from {2, 4, 8} (first and last layer 8) and per-layer MLP rank from {25%, 50%, 100%} of hidden, q/k/v
    biases, NVFP4 paged KV, batch 8, synthetic cache of `--context` tokens (default 32768), greedy decode steps."""
    import random
    import torch
    from transformer_surgeon_b200 import ops
    from transformer_surgeon_b200.decoder import CompressedDecoder, DecoderConfig, LayerWeights, fuse_rows
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    c = dict(QWEN25VL_7B_TEXT)
    nl = a.layers if a.layers != LLAMA3_8B["num_layers"] else c["num_layers"]
    c["num_layers"] = nl
    B = a.batch if a.batch != 32 else 8
    context = a.context if a.context != 2048 else 32768
    rnd_ = random.Random(2)
    bits = [8 if i in (0, nl - 1) else rnd_.choice([2, 4, 8]) for i in range(nl)]
    ranks = [rnd_.choice([c["hidden"] // 4, c["hidden"] // 2, 0]) for _ in range(nl)]
    max_seq = context + a.steps + a.warmup + 16
    cfg = DecoderConfig(dtype=torch.bfloat16, kv_format="nvfp4", max_positions=max_seq + 16, **c)
    g = torch.Generator(device=device).manual_seed(2)
    dt = torch.bfloat16
    H, Hkv, d, hid, inter = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden, cfg.intermediate
    rnd = lambda rows, cols, std: (torch.randn((rows, cols), generator=g, device=device) * std).to(dt)
    wbytes = 0
    layers = []
    for i in range(nl):
        qf = lambda rows, cols, std: ops.Factor.quantize(rnd(rows, cols, std), bits[i], "per_channel")

        def lin(out, inn):
            r = ranks[i]
            if r:
                return ops.PackedLinear(qf(out, r, 0.02 * (inn / r) ** 0.5 / 4), qf(r, inn, 0.25 / inn ** 0.5 * 4), None, dt)
            return ops.PackedLinear(qf(out, inn, 0.02), None, None, dt)
        fq, fk, fv = qf(H * d, hid, 0.02), qf(Hkv * d, hid, 0.02), qf(Hkv * d, hid, 0.02)
        bias = [(torch.randn(n, generator=g, device=device) * 0.1).to(dt) for n in (H * d, Hkv * d, Hkv * d)]
        ones = torch.ones(hid, dtype=dt, device=device)
        L = LayerWeights(ones, ones.clone(), ops.PackedLinear(qf(hid, H * d, 0.02), None, None, dt), lin(inter, hid), lin(inter, hid),
                         lin(hid, inter), qkv=fuse_rows([fq, fk, fv], bias, dt))
        layers.append(L)
        for pl in (L.qkv, L.o, L.gate, L.up, L.down):
            for f in (pl.u, pl.v):
                if f is not None:
                    wbytes += f.data.numel() + 4 * f.rows
    embed = rnd(cfg.vocab, hid, 0.02)
    lm_head = ops.PackedLinear(ops.Factor.dense(rnd(cfg.vocab, hid, 0.02)), None, None, dt)
    dec = CompressedDecoder(cfg, embed, layers, torch.ones(hid, dtype=dt, device=device), lm_head, B, max_seq, device)
    dec.greedy_head = True
    outl = torch.ones((Hkv, d), device=device)
    for h in range(Hkv):
        outl[h, torch.randperm(d, generator=g, device=device)[:4]] = 20.0
    for kv in dec.kv:
        dec.seq_lens.zero_()
        for t0 in range(0, context, 2048):
            n = min(2048, context - t0)
            k = (torch.randn((B, n, Hkv, d), generator=g, device=device) * outl).to(dt)
            v = (torch.randn((B, n, Hkv, d), generator=g, device=device) * outl).to(dt)
            kv.append(k, v)
            dec.seq_lens.add_(n)
    torch.cuda.synchronize()
    dec.capture()
    tok_host = torch.randint(0, cfg.vocab, (B,), dtype=torch.int64).pin_memory()
    out_host = torch.empty(B, dtype=torch.int64).pin_memory()
    sampler = ClockSampler(0)
    ms, ms_e2e, ctx0 = timed_steps(dec, a, tok_host, out_host, torch.cuda.synchronize, sampler)
    q = torch.randn((B, H, d), device=device).to(dt)
    o = torch.empty_like(q)
    t_attn = _graph_time_us(lambda i: ops.paged_decode_attention(dec.kv[i], q, dec.max_seq_len, out=o, ws=dec.attn_ws), nl)
    clocks = sampler.stop()
    dec.check_status()
    peak, which = peaks()
    kv_bytes = B * ctx0 * 2 * Hkv * d * 0.5625
    step_bytes = wbytes + cfg.vocab * hid * 2 + nl * kv_bytes
    step_us = ms / a.steps * 1e3
    line = {"metric": "decode tokens/s (Qwen2.5-VL-7B text tower, per-layer LRD + W2/4/8 + NVFP4-KV)", "value": B * a.steps / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "qwen2.5-vl-7b text-tower decode: %d layers, weight bits per layer %s, MLP rank per layer %s (0 = full), "
                                   "lm_head bf16, nvfp4 paged KV, batch %d, context %d->%d" % (nl, bits, ranks, B, ctx0, ctx0 + a.steps),
                       "l2": "inputs larger than L2 (%.1f GB read per step)" % (step_bytes / 1e9), "cuda_graph": True},
            "e2e": {"value": B * a.steps / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
            "gpu_launches": dec.kernel_launches_per_step * a.steps, "clocks": clocks,
            "roofline": {"kernel": "decode_attn_mma_kernel (NVFP4 pages, group of 7 query heads; split merge fused)", "bound": "hbm",
                         "achieved": kv_bytes / t_attn / 1e3, "peak": peak, "unit": "GB/s", "frac": kv_bytes / t_attn / 1e3 / peak,
                         "peak_source": which, "frac_nominal": kv_bytes / t_attn / 1e3 / HBM_NOMINAL_GBS, "traffic": None,
                         "ms_per_launch": t_attn * 1e-3, "share_of_step": nl * t_attn / step_us,
                         "parity": "KV formats are this project's definitions: parity unpinned",
                         "step_achieved": step_bytes / (step_us * 1e-6) / 1e9, "step_frac": step_bytes / (step_us * 1e-6) / 1e9 / peak}}
    emit(json.dumps(line))


def sweep_linear(a, ranks=(256, 1024), precisions=(8, 4, "binary"), ms=None, copies=8):
    """configs[1]: x [M, 4096] bf16, W 4096x4096 factored at rank r, factors at 8 / 4 bits and binary; time of
    LinearCompressed.forward per call, TFLOP/s and GB/s against the measured peaks.  Returns a list of records."""
    import torch
    from transformer_surgeon_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(2)
    peak_bw, _ = peaks()
    ms = ms or [int(v) for v in a.sweep_m.split(",")]
    if ranks == (256, 1024) and getattr(a, "sweep_ranks", None):
        ranks = tuple(int(v) for v in a.sweep_ranks.split(","))
    if precisions == (8, 4, "binary") and getattr(a, "sweep_precisions", None):
        precisions = tuple(v if v == "binary" else int(v) for v in a.sweep_precisions.split(","))
    out = []
    for r in ranks:
        for p in precisions:
            lins = []
            for _ in range(copies):       # distinct weight copies cycled by the graph; their total size is stated per record
                U = (torch.randn((4096, r), generator=g, device=dev) * 0.02).bfloat16()
                V = (torch.randn((r, 4096), generator=g, device=dev) * 0.02).bfloat16()
                lins.append(ops.PackedLinear(ops.Factor.quantize(U, p), ops.Factor.quantize(V, p), None, torch.bfloat16))
            bits = lins[0].u.bits
            for M in ms:
                x = torch.randn((M, 4096), generator=g, device=dev).bfloat16()
                y = torch.empty((M, 4096), dtype=torch.bfloat16, device=dev)
                ws = torch.zeros(lins[0].workspace_bytes(M), dtype=torch.uint8, device=dev)
                us = _graph_time_us(lambda i: lins[i](x, out=y, ws=ws), copies)
                flops = 2.0 * M * r * 8192
                byts = r * 8192 * bits / 8 + (4096 + r) * 4 + 2 * M * 4096 * 2
                out.append({"sweep": "linear", "M": M, "rank": r, "precision": p, "container_bits": bits,
                            "us_per_call": us, "tflops": flops / us / 1e6, "gbs": byts / us / 1e3,
                            "frac_hbm": byts / us / 1e3 / peak_bw, "frac_tensor_burst": flops / us / 1e6 / 1671.9,
                            "weights_mb_cycled": copies * r * 8192 * bits / 8 / 1e6})
    return out


def sweep_attention(a, contexts=None, formats=("int8", "fp8", "nvfp4")):
    """configs[2]: 32 q heads / 8 kv heads / d 128, batch 64, page 16, seeded random block table, K/V N(0,1) with 4
    outlier channels per head (x20); per format: decode attention, single-token append, bulk append of 2048 tokens per
    sequence.  KV formats are this project's definitions (parity unpinned).  Returns a list of records."""
    import torch
    from transformer_surgeon_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(3)
    peak_bw, _ = peaks()
    B, H, Hkv, d = a.sweep_batch, 32, 8, 128
    outl = torch.ones((Hkv, d), device=dev)
    for h in range(Hkv):
        outl[h, torch.randperm(d, generator=g, device=dev)[:4]] = 20.0
    out = []
    contexts = contexts or [int(v) for v in a.sweep_ctx.split(",")]
    for L in contexts:
        for fmt in formats:
            pages = L // 16 + 1
            rec = ops.kv_record_bytes(ops.KV_FORMATS[fmt], d)
            layers = max(1, min(4, int(3e9 // (B * pages * Hkv * rec * 2))))     # a few GB on the device at most
            kvs = []
            seq = torch.zeros(B, dtype=torch.int32, device=dev)
            bt = torch.randperm(B * pages, generator=g, device=dev).to(torch.int32).reshape(B, pages)
            bulk_us = []
            for _ in range(layers):
                kv = ops.PagedKV(fmt, B * pages, Hkv, d, bt, seq, dev)
                if fmt == "fp8":
                    kv.fill_fp8_scales(110.0 / 448, 110.0 / 448)
                seq.zero_()
                for t0 in range(0, L, 2048):
                    n = min(2048, L - t0)
                    k = (torch.randn((B, n, Hkv, d), generator=g, device=dev) * outl).bfloat16()
                    v = (torch.randn((B, n, Hkv, d), generator=g, device=dev) * outl).bfloat16()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    kv.append(k, v)
                    e1.record()
                    torch.cuda.synchronize()
                    if n == 2048 and len(kvs) + t0 > 0:          # skip the very first call (module load, cold caches)
                        bulk_us.append(e0.elapsed_time(e1) * 1e3)
                    seq += n
                kvs.append(kv)
            q = torch.randn((B, H, d), generator=g, device=dev).bfloat16()
            o = torch.empty_like(q)
            ws = torch.zeros(ops.decode_attn_workspace_bytes(B, H, d, L + 16), dtype=torch.uint8, device=dev)
            us = _graph_time_us(lambda i: ops.paged_decode_attention(kvs[i], q, L + 16, out=o, ws=ws), layers, reps=4)
            byts = B * (L // 16) * Hkv * rec * 2 + B * (L // 16) * 4 + 2 * B * H * d * 2
            k1 = torch.randn((B, 1, Hkv, d), generator=g, device=dev).bfloat16()
            us_app = _graph_time_us(lambda i: kvs[i].append(k1, k1), layers, reps=4)
            app_bytes = B * 2 * Hkv * d * (2 + rec / (16.0 * d))
            r = {"sweep": "attention", "format": fmt, "batch": B, "context": L, "decode_us": us,
                 "decode_gbs": byts / us / 1e3, "decode_frac_hbm": byts / us / 1e3 / peak_bw,
                 "decode_frac_nominal": byts / us / 1e3 / HBM_NOMINAL_GBS, "pages_mb": byts / 1e6,
                 "append_us": us_app, "append_gbs": app_bytes / us_app / 1e3, "layers_cycled": layers}
            if bulk_us:
                bu = sorted(bulk_us)[len(bulk_us) // 2]
                bulk_bytes = B * 2048 * 2 * Hkv * d * (2 + rec / (16.0 * d))
                r.update(bulk_append_tokens=2048, bulk_append_us=bu, bulk_append_gbs=bulk_bytes / bu / 1e3,
                         bulk_append_frac_hbm=bulk_bytes / bu / 1e3 / peak_bw)
            out.append(r)
            del kvs
    return out


def sweep_prefill(a, cases=None):
    """Prompt attention (tsb200_kv_gather_heads + tsb200_prefill_attn) at the Llama-3-8B layout: 32 query / 8 KV heads,
    d 128, FP8 pages, whole prompts of T tokens; causal flops 4 B H d T^2 / 2 against the measured bf16 peak."""
    import torch
    from transformer_surgeon_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(4)
    H, Hkv, d = 32, 8, 128
    out = []
    for B, T in cases or [(a.sweep_batch if a.sweep_batch != 64 else 8, 2048)]:
        pages = T // 16
        bt = torch.randperm(B * pages, generator=g, device=dev).to(torch.int32).reshape(B, pages)
        seq = torch.full((B,), T, dtype=torch.int32, device=dev)
        kv = ops.PagedKV("fp8", B * pages, Hkv, d, bt, seq, dev)
        kv.fill_fp8_scales(0.02, 0.02)
        kv.k_pool.random_(0, 120)
        kv.v_pool.random_(0, 120)
        q = torch.randn((B, T, H, d), generator=g, device=dev).bfloat16()
        o = torch.empty_like(q)
        ops.prefill_attention(kv, q, T, out=o)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            ops.prefill_attention(kv, q, T, out=o)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 5
        flops = 4.0 * B * H * d * T * T / 2
        out.append({"sweep": "prefill_attention", "batch": B, "tokens": T, "ms": ms, "prompt_tokens_per_s": B * T / (ms * 1e-3),
                    "tflops": flops / ms / 1e9, "frac_tensor_burst": flops / ms / 1e9 / 1671.9,
                    "includes": "dequantizing head-major gather + causal attention on tcgen05"})
    return out


if __name__ == "__main__":
    args = parse()
    divert_stdout()
    if args.sweep:
        import torch
        torch.cuda.set_device(0)
        for rec in {"linear": sweep_linear, "attention": sweep_attention, "prefill": sweep_prefill}[args.sweep](args):
            emit(json.dumps(rec))
    elif args.impl == "reference":
        run_reference(args)
    elif args.config == "c5":
        run_c5(args)
    else:
        run_ours(args)
