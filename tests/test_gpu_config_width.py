"""Parity at the FULL WIDTH of the benchmark configurations (one decoder layer + final norm + lm_head):

  config 4  Llama-3-8B layout: hidden 4096, 32 / 8 heads, d 128, MLP 14336 low-rank at r = 1024, every block
            linear 4-bit per-channel, bf16, FP8 paged KV, batch 32 - the shape the headline number is quoted on;
  config 5  Qwen2.5-VL-7B text layout: hidden 3584, 28 / 4 heads (group of 7), MLP 18944 at r = 1792, 2-bit
            per-channel weights, q/k/v biases, NVFP4 paged KV, batch 8.

Weights are seeded random factors quantized by the library; the oracle (oracle/decoder_layer.py, pinned against
the reference's own one-layer model in tests/test_oracle_layer.py) runs the same layer on the host from the
DEQUANTIZED factors.  Checked: weight codes and scales bit-exact against the oracle's quantize_vanilla, and the
logits after a 256-token prompt and after one decode step within max-rel-err 1e-2 (the tolerance stated for bf16
logits), against the oracle rounding where a bf16 model rounds; 2e-2 against the oracle that never rounds.
KV formats are this project's definitions (parity unpinned for them)."""
import numpy as np
import pytest
import torch

from oracle import decoder_layer as odl
from oracle import weight_quant as wq

pytestmark = pytest.mark.gpu

CONFIGS = {
    "config4_llama8b_w4_fp8": dict(hidden=4096, heads=32, kv_heads=8, inter=14336, vocab=128256, rank=1024, bits=4,
                                   kv="fp8", batch=32, theta=5e5, eps=1e-5, bias=False, seed=1),
    "config5_qwen25vl7b_w2_nvfp4": dict(hidden=3584, heads=28, kv_heads=4, inter=18944, vocab=152064, rank=1792, bits=2,
                                        kv="nvfp4", batch=8, theta=1e6, eps=1e-6, bias=True, seed=2),
}


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_one_layer_at_config_width(cuda, name):
    from transformer_surgeon_b200 import ops
    from transformer_surgeon_b200.decoder import CompressedDecoder, DecoderConfig, LayerWeights, fuse_rows
    c = CONFIGS[name]
    hid, H, Hkv, d, inter, r, bits = c["hidden"], c["heads"], c["kv_heads"], 128, c["inter"], c["rank"], c["bits"]
    dt = torch.bfloat16
    g = torch.Generator(device=cuda).manual_seed(c["seed"])
    T = 256

    def rnd(rows, cols, std):
        return (torch.randn((rows, cols), generator=g, device=cuda) * std).to(dt)

    W = {}          # oracle side: fp32 dequantized values on the host

    def qfac(rows, cols, std):
        f = ops.Factor.quantize(rnd(rows, cols, std), bits, "per_channel")
        return f, f.reconstruct(dt).float().cpu()

    def full(name_, out, inn, bias):
        f, deq = qfac(out, inn, 0.02)
        b = (torch.randn(out, generator=g, device=cuda) * 0.1).to(dt) if bias else None
        W[name_] = (deq, None, None if b is None else b.float().cpu())
        return f, b

    def lrd(name_, out, inn):
        raw = rnd(out, r, 0.02 * (inn / r) ** 0.5 / 4)
        fu = ops.Factor.quantize(raw, bits, "per_channel")
        fv, dv = qfac(r, inn, 0.25 / inn ** 0.5 * 4)
        W[name_] = (fu.reconstruct(dt).float().cpu(), dv, None)
        return ops.PackedLinear(fu, fv, None, dt), raw, fu

    (fq, bq), (fk, bk), (fv_, bv) = full("q", H * d, hid, c["bias"]), full("k", Hkv * d, hid, c["bias"]), full("v", Hkv * d, hid, c["bias"])
    fo, _ = full("o", hid, H * d, False)
    gate, gate_raw, gate_u = lrd("gate", inter, hid)
    up, _, _ = lrd("up", inter, hid)
    down, _, _ = lrd("down", hid, inter)
    # weight codes / scales: bit-exact against the oracle's restatement of quantize_vanilla (bf16 parameter arithmetic)
    qo, so = wq.quantize_vanilla(gate_raw.float().cpu().numpy(), bits, 1e-6, "per_channel", "bf16")
    assert np.array_equal(gate_u.codes().cpu().numpy(), qo) and np.array_equal(gate_u.scales.cpu().numpy(), so[:, 0])
    ln1 = (1 + 0.1 * torch.randn(hid, generator=g, device=cuda)).to(dt)
    ln2 = (1 + 0.1 * torch.randn(hid, generator=g, device=cuda)).to(dt)
    nrm = (1 + 0.1 * torch.randn(hid, generator=g, device=cuda)).to(dt)
    embed, head = rnd(c["vocab"], hid, 1.0), rnd(c["vocab"], hid, 0.02)
    W.update(ln1=ln1.float().cpu(), ln2=ln2.float().cpu(), norm=nrm.float().cpu(), embed=embed.float().cpu(),
             lm_head=(head.float().cpu(), None, None))
    layer = LayerWeights(ln1, ln2, ops.PackedLinear(fo, None, None, dt), gate, up, down,
                         qkv=fuse_rows([fq, fk, fv_], [bq, bk, bv], dt))
    cfg = DecoderConfig(num_layers=1, hidden=hid, num_heads=H, num_kv_heads=Hkv, head_dim=d, intermediate=inter,
                        vocab=c["vocab"], rope_theta=c["theta"], rms_eps=c["eps"], dtype=dt, kv_format=c["kv"], max_positions=T + 16)
    dec = CompressedDecoder(cfg, embed, [layer], nrm, ops.PackedLinear(ops.Factor.dense(head), None, None, dt), c["batch"], T + 16, cuda)
    gen = torch.Generator().manual_seed(c["seed"] + 100)
    ids = torch.randint(0, c["vocab"], (c["batch"], T), generator=gen)
    nxt = torch.randint(0, c["vocab"], (c["batch"],), generator=gen)
    out0 = dec.prefill(ids).float().cpu()                      # prompt in one pass (FP8: scales = amax / 448 over it)
    out1 = dec.step(nxt.to(cuda)).float().cpu()                # one decode step on the paged kernels
    dec.check_status()
    ref0, ref1 = odl.one_layer_logits(W, ids, nxt, H, Hkv, d, c["theta"], c["eps"], c["kv"], act=dt)
    f0, f1 = odl.one_layer_logits(W, ids, nxt, H, Hkv, d, c["theta"], c["eps"], c["kv"], act=torch.float32)
    assert rel(out0, ref0) < 1e-2 and rel(out1, ref1) < 1e-2, (rel(out0, ref0), rel(out1, ref1))
    assert rel(out0, f0) < 2e-2 and rel(out1, f1) < 2e-2, (rel(out0, f0), rel(out1, f1))
