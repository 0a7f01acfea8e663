"""Replica sharding of independent sequences across GPUs (one process per GPU).

The decode path has no cross-sequence dependency (per-sequence KV pages and block-table rows), so
N GPUs run N independent engines over disjoint slices of the batch and no collective is needed on
the data path; torch.distributed is used only to agree on timings and to gather results.
"""
import torch
import torch.distributed as dist


def shard_range(total, world, rank):
    """Contiguous slice [begin, end) of `total` sequences owned by `rank`; sizes differ by at most 1."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def max_over_ranks(value, device="cpu"):
    """Maximum of a scalar over all ranks (the job's time is the slowest rank's)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def gather_tokens(local_tokens, total, device="cpu"):
    """All-gather per-rank token tensors [n_local, T] (ragged over ranks) into [total, T] on every rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local_tokens
    world, rank = dist.get_world_size(), dist.get_rank()
    sizes = [shard_range(total, world, r) for r in range(world)]
    width = local_tokens.shape[1]
    cap = max(e - b for b, e in sizes)
    pad = torch.zeros((cap, width), dtype=local_tokens.dtype, device=device)
    pad[:local_tokens.shape[0]] = local_tokens.to(device)
    outs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(outs, pad)
    return torch.cat([o[:e - b] for o, (b, e) in zip(outs, sizes)], dim=0)
