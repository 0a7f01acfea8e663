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
        outs = {}
        for tp_world in (1, world):
            cfg = DecoderConfig(num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate=512,
                                vocab=128, dtype=torch.float32, kv_format="int8", max_positions=64,
                                tp_world=tp_world, tp_rank=rank if tp_world > 1 else 0)
            dec = surgeon.decoder_from_state_dict(sd, cfg, cc, batch=3, max_seq_len=32, device=dev)
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
