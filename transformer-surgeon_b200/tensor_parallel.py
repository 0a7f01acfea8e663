"""Tensor-parallel sharding of the decoder's LinearCompressed layers (one process per GPU).

Column-parallel (q, k, v, gate, up): the OUTPUT features are split; for a low-rank layer the rows of
U are split and V is replicated.  Row-parallel (o, down): the INPUT features are split; for a
low-rank layer the columns of V are split, U is replicated, and the partial outputs are summed over
ranks with one all-reduce of [M, hidden] per layer (NCCL over NVLink).  KV heads follow the q/k/v
split, so every rank owns the pages of its own heads and attention needs no exchange.

Per-row quantization scales are unaffected by either split: a row of U keeps its scale, and a
column slice of V keeps the scale of the full row it was quantized with (the codes are sliced, not
re-derived), so the sharded layers reconstruct exactly the same weights as the unsharded ones.
The reference has no multi-GPU path (no torch.distributed import in the package).
"""
import torch
import torch.distributed as dist

from . import ops


def _slice_factor_rows(f, begin, end):
    """Rows [begin, end) of a Factor (packed containers are row-major: a plain slice)."""
    data = f.data[begin:end].contiguous()
    scales = None if f.scales is None else f.scales[begin:end].contiguous()
    return ops.Factor(data, scales, f.bits, end - begin, f.cols)


def _slice_factor_cols(f, begin, end):
    """Columns [begin, end) of a Factor; packed codes are unpacked, sliced and packed again."""
    if f.bits >= 16:
        return ops.Factor(f.data[:, begin:end].contiguous(), None, f.bits, f.rows, end - begin)
    codes = f.codes()[:, begin:end].contiguous()
    packed, _ = ops.pack_codes(codes, f.bits)
    return ops.Factor(packed, f.scales, f.bits, f.rows, end - begin)


def shard_range(n, world, rank, multiple=1):
    """[begin, end) of `n` features for `rank`; n must split evenly in units of `multiple`."""
    if n % (world * multiple):
        raise ValueError(f"{n} features do not split over {world} ranks in units of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def column_parallel(lin, world, rank, multiple=1):
    """Shard the output features of a PackedLinear."""
    b, e = shard_range(lin.out_features, world, rank, multiple)
    bias = None if lin.bias is None else lin.bias[b:e].contiguous()
    return ops.PackedLinear(_slice_factor_rows(lin.u, b, e), lin.v, bias, lin.act_dtype)


def row_parallel(lin, world, rank, multiple=1):
    """Shard the input features of a PackedLinear; the bias is kept on rank 0 only (it is added once)."""
    b, e = shard_range(lin.in_features, world, rank, multiple)
    bias = lin.bias if rank == 0 else None
    if lin.v is not None:
        return ops.PackedLinear(lin.u, _slice_factor_cols(lin.v, b, e), bias, lin.act_dtype)
    return ops.PackedLinear(_slice_factor_cols(lin.u, b, e), None, bias, lin.act_dtype)


def all_reduce_sum(t, group=None):
    """Sum of the row-parallel partial outputs over the tensor-parallel group (in place)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
