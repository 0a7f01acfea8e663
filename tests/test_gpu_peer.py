"""Single-GPU checks of the peer all-reduce kernel's bounded wait: a rank whose peer never signals
gives up after a fraction of a second, records a status code, sums what it has, and leaves the
context usable.  (The two-rank exchange itself is covered in test_gpu_tp.py.)"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_missing_peer_times_out_with_status(cuda):
    from transformer_surgeon_b200 import _lib, ops
    lib = _lib.load()
    M, hidden = 4, 256
    g = torch.Generator().manual_seed(50)
    part = torch.randn(M, hidden, generator=g).bfloat16().to(cuda)
    ghost = torch.randn(M, hidden, generator=g).bfloat16().to(cuda)      # the absent rank's buffer: must not be read
    flags = torch.zeros(int(lib.tsb200_peer_flag_bytes()), dtype=torch.uint8, device=cuda)
    state = torch.zeros(4, dtype=torch.int32, device=cuda)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().to(cuda)
    resid = torch.randn(M, hidden, generator=g).bfloat16().to(cuda)
    ref_resid, out, ref_out = resid.clone(), torch.empty_like(resid), torch.empty_like(resid)
    d = _lib.PeerDesc()
    d.world, d.rank = 2, 0
    d.partial[0], d.partial[1] = part.data_ptr(), ghost.data_ptr()
    d.flags[0] = d.flags[1] = flags.data_ptr()        # rank 0 signals slot [0][row]; it polls slot [1][row], which nothing sets
    d.epoch, d.status = state.data_ptr(), state.data_ptr() + 8
    st = lib.tsb200_peer_allreduce_add_rmsnorm(C.byref(d), resid.data_ptr(), w.data_ptr(), out.data_ptr(), ops.BF16, M, hidden,
                                               1e-6, ops._stream())
    assert st == 0
    torch.cuda.synchronize()                                              # returns: the wait was bounded
    assert int(state[2].item()) == 21                                     # "a peer did not show up"
    assert int(state[0].item()) == 1 and int(state[1].item()) == 0        # epoch advanced, CTA counter reset
    ops.add_rmsnorm(ref_resid, part, w, 1e-6, 0, out=ref_out)             # the sum holds this rank's partial only
    assert torch.equal(out, ref_out) and torch.equal(resid, ref_resid)
    assert torch.equal(part + 0, part)                                    # the context still runs kernels


def test_argument_checks(cuda):
    from transformer_surgeon_b200 import _lib, ops
    lib = _lib.load()
    d = _lib.PeerDesc()
    d.world, d.rank = 1, 0
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda)
    args = (x.data_ptr(), x.data_ptr(), x.data_ptr(), ops.BF16, 2, 64, 1e-6, ops._stream())
    assert lib.tsb200_peer_allreduce_add_rmsnorm(C.byref(d), *args) == _lib.ERR_ARG        # fewer than two ranks
    d.world = 2
    assert lib.tsb200_peer_allreduce_add_rmsnorm(C.byref(d), *args) == _lib.ERR_ARG        # null buffers
