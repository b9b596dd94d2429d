"""Failure detection without a GPU fault: a bounded device-side wait that runs out.

The flag barrier of the sharded path (``qlin_peer_barrier``) waits for every rank's slot of its flag array to
show the current epoch.  Here one GPU plays rank 0 of a world of two whose second rank never signals: both
flag arrays live on this GPU and nothing ever writes slot 1.  With a 50 ms limit the kernel must return by
itself, leave ``QLIN_ERR_TIMEOUT`` in the status word, and leave the context usable: a barrier on fresh flags
passes and a GEMM still gives the right answer afterwards.  Nothing here traps, asserts or reads a bad address.
"""

import ctypes as C
import time

import pytest
import torch

from fms_model_optimizer_b200 import _lib as L
from fms_model_optimizer_b200 import ops

pytestmark = pytest.mark.gpu


def _barrier_args(flags_mine, flags_peer, epoch, status, rank, world, timeout_ns):
    ptrs = [flags_mine.data_ptr() if r == rank else flags_peer.data_ptr() for r in range(world)] + [None] * (8 - world)
    return L.PeerBarrierArgs(local_flags=flags_mine.data_ptr(), peer_flags=(C.c_void_p * 8)(*ptrs), epoch=epoch.data_ptr(),
                             status=status.data_ptr(), rank=rank, world=world, timeout_ns=timeout_ns)


def test_barrier_wait_runs_out_and_the_context_survives(cuda_dev):
    lib = L.load()
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    mine = torch.zeros(64, dtype=torch.int32, device=cuda_dev)
    absent_peer = torch.zeros(64, dtype=torch.int32, device=cuda_dev)  # the rank that never arrives
    epoch = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    L.check(lib.qlin_peer_barrier(C.byref(_barrier_args(mine, absent_peer, epoch, status, 0, 2, 50_000_000)), stream), "barrier")
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(status.item()) == L.ERR_TIMEOUT
    assert 0.04 < waited < 5.0, waited  # gave up after about 50 ms, not after the 10 s default
    # rank 0 did announce itself to both flag arrays before it started waiting
    assert int(mine[0].item()) == 1 and int(absent_peer[0].item()) == 1 and int(mine[1].item()) == 0

    # the context is intact: a one-rank barrier on fresh flags passes with a clean status word ...
    status.zero_()
    fresh, e2 = torch.zeros(64, dtype=torch.int32, device=cuda_dev), torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    L.check(lib.qlin_peer_barrier(C.byref(_barrier_args(fresh, fresh, e2, status, 0, 1, 50_000_000)), stream), "barrier")
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(fresh[0].item()) == 1
    # ... the two-rank barrier passes once the missing rank's slot carries the epoch ...
    mine[1] = 2
    L.check(lib.qlin_peer_barrier(C.byref(_barrier_args(mine, absent_peer, epoch, status, 0, 2, 50_000_000)), stream), "barrier")
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(epoch.item()) == 2
    # ... and so does the next kernel
    a = torch.randint(-127, 128, (128, 256), dtype=torch.int8, device=cuda_dev)
    b = torch.randint(-127, 128, (64, 256), dtype=torch.int8, device=cuda_dev)
    assert torch.equal(ops.gemm(a, b).cpu(), a.cpu().int() @ b.cpu().int().t())
    ops.check_status(cuda_dev)


def test_barrier_rejects_a_negative_limit(cuda_dev):
    lib = L.load()
    f = torch.zeros(64, dtype=torch.int32, device=cuda_dev)
    e = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    assert lib.qlin_peer_barrier(C.byref(_barrier_args(f, f, e, e, 0, 1, -1)), None) == L.ERR_BAD_SHAPE
