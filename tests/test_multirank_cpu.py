"""World-size-2 (gloo, CPU) test of the replica-sharding host logic used for N > 1 GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from transformer_surgeon_b200 import sharding
        b, e = sharding.shard_range(total, world, rank)
        # every rank "decodes" its own sequences: token = 1000 * sequence index + step
        local = torch.stack([torch.arange(4) + 1000 * i for i in range(b, e)]) if e > b else torch.zeros((0, 4), dtype=torch.int64)
        allt = sharding.gather_tokens(local, total)
        assert allt.shape == (total, 4)
        assert torch.equal(allt[:, 0], 1000 * torch.arange(total))
        # the job's time is the slowest rank's
        assert sharding.max_over_ranks(10.0 + rank) == 10.0 + world - 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [32, 33, 1])
def test_shard_gather_and_max_over_two_ranks(total):
    mp.spawn(_worker, args=(2, _free_port(), total), nprocs=2, join=True)


def test_shard_range_partitions_exactly():
    from transformer_surgeon_b200 import sharding
    for total in (0, 1, 7, 32, 65):
        for world in (1, 2, 3, 8):
            cover = []
            for r in range(world):
                b, e = sharding.shard_range(total, world, r)
                cover += list(range(b, e))
            assert cover == list(range(total))
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)
