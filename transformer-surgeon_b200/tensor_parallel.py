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
import ctypes as C

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import check


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


# ---------------------------------------------------------------- all-reduce over peer memory
# An exported allocator block can be imported once per process: several PeerBuffers whose tensors
# share a block reuse the mapping, which then lives until the process exits.
_ipc_bases = {}


class PeerBuffers:
    """Two [M, hidden] bf16 partial-output buffers per rank plus the flag blocks of
    `tsb200_peer_allreduce_add_rmsnorm`, each mapped into every rank of the group.

    The row-parallel projections write their partial outputs straight into `partial(i)`; the fused
    kernel then reads every rank's copy over NVLink.  The buffer is a PyTorch allocation; its CUDA IPC
    handle (`tsb200_ipc_export`) travels through the process group and every rank imports it on ITS OWN
    device (`tsb200_ipc_open`; one process per GPU on one node, every process seeing all GPUs)."""

    def __init__(self, M, hidden, device, group=None):
        lib = _lib.load()
        self.group, self.M, self.hidden, self.device = group, M, hidden, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise ValueError("peer all-reduce serves 2..8 ranks")
        part = (M * hidden * 2 + 255) // 256 * 256
        flag = int(lib.tsb200_peer_flag_bytes())
        self._off = {"p0": 0, "p1": part, "flags": 2 * part}
        # one allocation per rank: [partial 0 | partial 1 | flags], zero-filled (flags must start at 0)
        self.local = torch.zeros(2 * part + flag, dtype=torch.uint8, device=self.device)
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)     # [epoch, finished CTAs, status, -]
        # A failure on one rank (export or import) is turned into the same RuntimeError on EVERY rank, after the
        # collectives have been matched, so that callers can fall back together.
        hbuf, off = C.create_string_buffer(64), C.c_uint64()
        with torch.cuda.device(self.device):
            st = lib.tsb200_ipc_export(self.local.data_ptr(), hbuf, C.byref(off))
        meta = (hbuf.raw, int(off.value)) if st == 0 else None
        metas = [None] * self.world
        dist.all_gather_object(metas, meta, group=group)
        bases, ok = [], all(m is not None for m in metas)
        if ok:
            with torch.cuda.device(self.device):
                for s, (handle, offset) in enumerate(metas):
                    if s == self.rank:
                        bases.append(self.local.data_ptr())
                        continue
                    key = (self.device.index, handle)
                    if key not in _ipc_bases:
                        base = C.c_void_p()
                        if lib.tsb200_ipc_open(handle, C.byref(base)) != 0:
                            ok = False
                            break
                        _ipc_bases[key] = base.value
                    bases.append(_ipc_bases[key] + offset)
        oks = [None] * self.world
        dist.all_gather_object(oks, ok, group=group)
        if not all(oks):
            raise RuntimeError("peer buffers could not be exported / imported on ranks %s (CUDA IPC needs one node, "
                               "every process seeing all GPUs, and a cudaMalloc-backed allocator)"
                               % [i for i, o in enumerate(oks) if not o])
        self._desc = []
        for i in range(2):
            d = _lib.PeerDesc()
            d.world, d.rank = self.world, self.rank
            for s in range(self.world):
                d.partial[s] = bases[s] + self._off["p%d" % i]
                d.flags[s] = bases[s] + self._off["flags"]
            d.epoch = self.state.data_ptr()
            d.status = self.state.data_ptr() + 8
            self._desc.append(d)
        dist.barrier(group=group)          # every rank has mapped every buffer before anyone signals

    def partial(self, i):
        """This rank's partial-output buffer i (0 / 1) as a [M, hidden] bf16 tensor."""
        off = self._off["p%d" % i]
        return self.local[off:off + self.M * self.hidden * 2].view(torch.bfloat16).view(self.M, self.hidden)

    def allreduce_add_rmsnorm(self, i, residual, weight, eps, out):
        """residual += sum over ranks of partial(i); out = RMSNorm(residual) * weight."""
        lib = _lib.load()
        check(lib.tsb200_peer_allreduce_add_rmsnorm(C.byref(self._desc[i]), residual.data_ptr(), weight.data_ptr(),
                                                    out.data_ptr(), ops.BF16, residual.shape[0], self.hidden, float(eps),
                                                    ops._stream()), "tsb200_peer_allreduce_add_rmsnorm")
        return out

    def status(self):
        """0, or the code recorded when a peer did not show up within the bounded wait (synchronises)."""
        return int(self.state[2].item())

    def clear_status(self):
        self.state[2:3].zero_()
