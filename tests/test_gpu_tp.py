"""Tensor-parallel sharding: layer-level identities on one GPU and a 2-rank NCCL engine run."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lin(ops, out, inn, rank, p, bias, g, cuda, dt=torch.float32):
    U = (torch.randn(out, rank or inn, generator=g) * 0.05).to(dt).to(cuda)
    V = (torch.randn(rank, inn, generator=g) * 0.05).to(dt).to(cuda) if rank else None
    b = (torch.randn(out, generator=g) * 0.1).to(dt).to(cuda) if bias else None
    if p is None:
        return ops.PackedLinear(ops.Factor.dense(U), ops.Factor.dense(V) if rank else None, b, dt)
    return ops.PackedLinear(ops.Factor.quantize(U, p), ops.Factor.quantize(V, p) if rank else None, b, dt)


@pytest.mark.parametrize("p", [None, 8, 4])
@pytest.mark.parametrize("rank", [0, 64])
def test_column_and_row_parallel_reproduce_the_full_layer(cuda, p, rank):
    from transformer_surgeon_b200 import ops, tensor_parallel as tp
    g = torch.Generator().manual_seed(31)
    lin = _lin(ops, 256, 512, rank, p, True, g, cuda)
    x = torch.randn(6, 512, generator=g).to(cuda)
    full = lin(x)
    world = 4
    cols = torch.cat([tp.column_parallel(lin, world, r, 64)(x) for r in range(world)], dim=1)
    torch.testing.assert_close(cols, full, rtol=1e-5, atol=1e-5)
    parts = sum(tp.row_parallel(lin, world, r, 64)(x[:, r * 128:(r + 1) * 128].contiguous()) for r in range(world))
    torch.testing.assert_close(parts, full, rtol=1e-4, atol=1e-4)
    # sharded codes are slices of the original codes, scales are untouched
    if p is not None and rank:
        sh = tp.row_parallel(lin, world, 1, 64)
        assert torch.equal(sh.v.codes(), lin.v.codes()[:, 128:256])
        assert torch.equal(sh.v.scales, lin.v.scales)
    with pytest.raises(ValueError):
        tp.shard_range(100, 3, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _state_dict(g, hidden=256, inter=512, H=4, Hkv=2, d=64, vocab=128, layers=2):
    sd = {"model.embed_tokens.weight": torch.randn(vocab, hidden, generator=g) * 0.5,
          "lm_head.weight": torch.randn(vocab, hidden, generator=g) * 0.1, "model.norm.weight": torch.ones(hidden)}
    for i in range(layers):
        b = f"model.layers.{i}."
        sd[b + "self_attn.q_proj.weight"] = torch.randn(H * d, hidden, generator=g) * 0.05
        sd[b + "self_attn.k_proj.weight"] = torch.randn(Hkv * d, hidden, generator=g) * 0.05
        sd[b + "self_attn.v_proj.weight"] = torch.randn(Hkv * d, hidden, generator=g) * 0.05
        sd[b + "self_attn.q_proj.bias"] = torch.randn(H * d, generator=g) * 0.1
        sd[b + "self_attn.o_proj.weight"] = torch.randn(hidden, H * d, generator=g) * 0.05
        for n, (o, k) in {"gate_proj": (inter, hidden), "up_proj": (inter, hidden), "down_proj": (hidden, inter)}.items():
            sd[b + f"mlp.{n}.weight"] = torch.randn(o, 32, generator=g) * 0.1           # rank-32 factors
            sd[b + f"mlp.{n}.linear_V.weight"] = torch.randn(32, k, generator=g) * 0.1
        sd[b + "input_layernorm.weight"] = torch.ones(hidden)
        sd[b + "post_attention_layernorm.weight"] = torch.ones(hidden)
    return sd


def _tp_worker(rank, world, port, out_path):
    import torch.distributed as dist
    from transformer_surgeon_b200 import surgeon
    from transformer_surgeon_b200.decoder import DecoderConfig
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(32)
        sd = _state_dict(g)
        ids = torch.randint(0, 128, (3, 10), generator=g)
        cc = {k[:-7]: {"quantization": {"precision": 8, "granularity": "per_channel"}} for k in sd if "proj.weight" in k}
        from transformer_surgeon_b200 import ops
        for k in list(sd):          # store what the reference's soft quantization stores: the dequantized 8-bit codes
            if "proj." in k and k.endswith("weight"):
                sd[k] = ops.Factor.quantize(sd[k].to(dev).contiguous(), 8, "per_channel").reconstruct(torch.float32).cpu()
        outs = {}
        for tp_world in (1, world):
            cfg = DecoderConfig(num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate=512,
                                vocab=128, dtype=torch.float32, kv_format="int8", max_positions=64,
                                tp_world=tp_world, tp_rank=rank if tp_world > 1 else 0)
            dec = surgeon.decoder_from_state_dict(sd, cfg, cc, batch=3, max_seq_len=32, device=dev)
            assert dec.layers[0].o.u.bits == 8 and dec.layers[0].gate.v.bits == 8       # packed, not the dense fallback
            toks, logits = dec.generate(ids, max_new_tokens=4)
            outs[tp_world] = (toks.cpu(), logits.float().cpu())
        if rank == 0:
            torch.save(outs, out_path)
    finally:
        dist.destroy_process_group()


def test_two_rank_engine_matches_single_gpu(tmp_path):
    """TP=2 over NCCL (NVLS off, plain all-reduce) gives the logits / greedy tokens of the unsharded engine."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "tp.pt")
    mp.spawn(_tp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    outs = torch.load(out)
    torch.testing.assert_close(outs[2][1], outs[1][1], rtol=2e-4, atol=2e-4)
    assert torch.equal(outs[2][0], outs[1][0])


def _peer_worker(rank, world, port, out_path):
    import torch.distributed as dist
    from transformer_surgeon_b200 import ops, surgeon, tensor_parallel as tp
    from transformer_surgeon_b200.decoder import DecoderConfig
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    try:
        # ---- kernel level: fused all-reduce + add + RMSNorm against NCCL all-reduce + tsb200_add_rmsnorm
        M, hidden = 32, 512
        pb = tp.PeerBuffers(M, hidden, dev)
        g = torch.Generator().manual_seed(40)                      # same stream of numbers on every rank
        w = (1.0 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().to(dev)
        resid_a = torch.randn(M, hidden, generator=g).bfloat16().to(dev)
        resid_b = resid_a.clone()
        out_a, out_b = torch.empty_like(resid_a), torch.empty_like(resid_a)
        same = True
        for it in range(6):
            parts = [torch.randn(M, hidden, generator=g).bfloat16() for _ in range(world)]
            pb.partial(it % 2).copy_(parts[rank])
            pb.allreduce_add_rmsnorm(it % 2, resid_a, w, 1e-6, out_a)
            ref = parts[rank].to(dev)
            dist.all_reduce(ref)
            ops.add_rmsnorm(resid_b, ref, w, 1e-6, 0, out=out_b)
            same = same and torch.equal(out_a, out_b) and torch.equal(resid_a, resid_b)
        # replayed from a CUDA graph: the epoch advances on the device
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                pb.allreduce_add_rmsnorm(0, resid_a, w, 1e-6, out_a)
                pb.allreduce_add_rmsnorm(1, resid_a, w, 1e-6, out_a)
            for _ in range(3):
                gr.replay()
        torch.cuda.synchronize()
        for _ in range(3):
            for i in (0, 1):
                ref = pb.partial(i).clone()
                dist.all_reduce(ref)
                ops.add_rmsnorm(resid_b, ref, w, 1e-6, 0, out=out_b)
        res["kernel_same"] = bool(same and torch.equal(out_a, out_b) and torch.equal(resid_a, resid_b))
        res["status"] = pb.status()
        # ---- engine level: bf16 TP engine with the fused kernel against the same engine over NCCL
        g = torch.Generator().manual_seed(32)
        sd = _state_dict(g)
        ids = torch.randint(0, 128, (3, 10), generator=g)
        cc = {k[:-7]: {"quantization": {"precision": 4, "granularity": "per_channel"}} for k in sd if "proj.weight" in k}
        for k in list(sd):          # what the reference's soft quantization stores in a bf16 model: dequantized 4-bit codes
            if "proj." in k and k.endswith("weight"):
                sd[k] = ops.Factor.quantize(sd[k].to(dev).bfloat16().contiguous(), 4, "per_channel").reconstruct(torch.bfloat16).cpu()
        outs = {}
        for mode in ("nccl", "peer"):
            cfg = DecoderConfig(num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate=512,
                                vocab=128, dtype=torch.bfloat16, kv_format="int8", max_positions=64, tp_world=world, tp_rank=rank)
            dec = surgeon.decoder_from_state_dict(sd, cfg, cc, batch=3, max_seq_len=32, device=dev)
            assert dec.layers[0].o.u.bits == 4 and dec.layers[0].gate.v.bits == 4       # packed, not the dense fallback
            if mode == "peer":
                assert dec.enable_peer_allreduce()
            toks, logits = dec.generate(ids, max_new_tokens=4)
            outs[mode] = (toks.cpu(), logits.float().cpu())
            if mode == "peer":
                res["engine_status"] = dec.peer.status()
        res["outs"] = outs
        if rank == 0:
            torch.save(res, out_path)
    finally:
        dist.destroy_process_group()


def test_peer_allreduce_matches_nccl(tmp_path):
    """The fused all-reduce + residual add + RMSNorm over NVLink peer loads gives the bits of an NCCL
    all-reduce followed by tsb200_add_rmsnorm (2 ranks), eagerly and replayed from a CUDA graph, and the
    tensor-parallel engine produces the same tokens and logits with either."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "peer.pt")
    mp.spawn(_peer_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["status"] == 0 and res["engine_status"] == 0
    assert res["kernel_same"]
    assert torch.equal(res["outs"]["peer"][0], res["outs"]["nccl"][0])
    torch.testing.assert_close(res["outs"]["peer"][1], res["outs"]["nccl"][1], rtol=0, atol=0)
