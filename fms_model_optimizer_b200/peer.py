"""Buffers that the other GPUs of the node write into, and the barrier between the phases of a layer.

One process drives one GPU.  Every rank allocates one arena of the same size, exports it through a CUDA IPC
handle (``qlin_ipc_export``), gathers the handles of all ranks over ``torch.distributed`` and maps the peers'
arenas (``qlin_ipc_open``).  Sub-buffers are carved out of the arena at the same offsets on every rank, so
"the address of buffer X on rank p" is ``base[p] + offset``.  The kernels that take such addresses store to
them directly (GEMM epilogue with row-block scatter, replicated outputs of the fused quantiser); nothing here
moves data itself.  The reference has no multi-GPU code of its own for this path: its int8 Linear only
registers sharding tables for the serving stack (fms_mo/aiu_addons/i8i8/i8i8_aiu_linear.py:304-389).
"""

from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops


class PeerArena:
    def __init__(self, nbytes: int, dev: torch.device, group=None):
        self.dev = dev
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        # one allocation of its own: the handle names the whole cudaMalloc block
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=dev)
        self.used = 0
        lib = L.load()
        handle = (C.c_ubyte * 64)()
        off = C.c_int64(0)
        with torch.cuda.device(dev):
            L.check(lib.qlin_ipc_export(C.c_void_p(self.buf.data_ptr()), handle, C.byref(off)), "qlin_ipc_export")
        mine = (bytes(handle), int(off.value), dev.index)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self._opened = []
        self.base: List[int] = []
        for r, (h, o, _) in enumerate(everyone):
            if r == self.rank:
                self.base.append(self.buf.data_ptr())
                continue
            raw = (C.c_ubyte * 64).from_buffer_copy(h)
            b, p = C.c_void_p(), C.c_void_p()
            with torch.cuda.device(dev):
                L.check(lib.qlin_ipc_open(raw, o, C.byref(b), C.byref(p)), "qlin_ipc_open")
            self._opened.append(b.value)
            self.base.append(p.value)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def alloc(self, nbytes: int) -> Tuple[int, torch.Tensor]:
        """Carves ``nbytes`` (rounded up to 256) out of the arena: returns (offset, local uint8 view).  Every rank
        must make the same sequence of calls."""
        n = (int(nbytes) + 255) // 256 * 256
        if self.used + n > self.nbytes:
            raise RuntimeError("peer arena exhausted")
        off = self.used
        self.used += n
        return off, self.buf[off : off + n]

    def addr(self, rank: int, offset: int) -> int:
        return self.base[rank] + offset

    def copy2d(self, dst_addr: int, dpitch: int, src_addr: int, spitch: int, width: int, height: int = 1) -> None:
        """Queues a copy-engine transfer on the current stream (``qlin_peer_copy2d``); addresses are raw device
        addresses, typically ``self.addr(peer, offset)`` on one side."""
        with torch.cuda.device(self.dev):
            L.check(L.load().qlin_peer_copy2d(C.c_void_p(dst_addr), dpitch, C.c_void_p(src_addr), spitch, width, height,
                                              ops._stream(self.dev)), "qlin_peer_copy2d")  # fmt: skip

    def close(self):
        lib = L.load()
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.dev):
            for b in self._opened:
                lib.qlin_ipc_close(C.c_void_p(b))
        self._opened = []


class SymmArena:
    """The same arena interface over PyTorch's symmetric memory (``torch.distributed._symmetric_memory``): one
    allocation per rank made with the driver's virtual-memory calls, exchanged between the processes and, where the
    node has an NVLink switch, also bound to one multicast object.  ``mc_base`` is then the multicast mapping of the
    arena: a ``multimem.st`` to ``mc_base + off`` lands at offset ``off`` of every rank's arena, and a
    ``multimem.ld_reduce`` from it returns the sum of all ranks' values there.  ``mc_base`` is 0 when the node offers
    no multicast.  PyTorch does the allocation and the handle exchange; the kernels of this library do every access."""

    def __init__(self, nbytes: int, dev: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.dev = dev
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=dev)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.buf.zero_()
        self.used = 0
        self.base: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        if self.base[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory: this rank's pointer differs from the tensor's address")
        self.mc_base = int(self.handle.multicast_ptr or 0)
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)

    alloc = PeerArena.alloc
    addr = PeerArena.addr

    def mc_addr(self, offset: int) -> int:
        if not self.mc_base:
            raise RuntimeError("this node offers no NVLink multicast")
        return self.mc_base + offset

    def close(self):
        """Every rank must have stopped issuing work that touches the arena: a rank must never leave while another
        still sends multicast traffic to the memory it had bound."""
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self.group)


def make_arena(nbytes: int, dev: torch.device, want_multicast: bool, group=None):
    """A SymmArena when ``want_multicast`` and the node provides it, otherwise the CUDA-IPC PeerArena.  All ranks take
    the same branch (the decision is reduced over the group)."""
    ok = 0
    arena = None
    if want_multicast:
        try:
            arena = SymmArena(nbytes, dev, group)
            ok = 1 if arena.mc_base else 0
        except Exception as e:  # noqa: BLE001 -- no symmetric memory on this node: every rank falls back together
            print(f"# symmetric memory unavailable ({type(e).__name__}: {e}); using the CUDA-IPC arena", flush=True)
            ok = 0
        t = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
        ok = int(t.item())
    if ok:
        return arena
    del arena
    return PeerArena(nbytes, dev, group)


class PeerBarrier:
    """``qlin_peer_barrier`` over flag words that live in a PeerArena.  Stream-ordered: work queued on the calling
    stream after ``wait()`` sees what the peers stored to this GPU before their ``wait()``."""

    def __init__(self, arena, timeout_s: float = 10.0):
        self.arena = arena
        self.off, flags = arena.alloc(256)
        self.flags = flags
        self.epoch = torch.zeros(1, dtype=torch.int32, device=arena.dev)
        self.args = L.PeerBarrierArgs(
            local_flags=arena.addr(arena.rank, self.off),
            peer_flags=(C.c_void_p * 8)(*([arena.addr(r, self.off) for r in range(arena.world)] + [None] * (8 - arena.world))),
            epoch=self.epoch.data_ptr(), status=ops.status_word(arena.dev).data_ptr(), rank=arena.rank, world=arena.world,
            timeout_ns=int(timeout_s * 1e9),
        )  # fmt: skip

    def wait(self):
        dev = self.arena.dev
        with torch.cuda.device(dev):
            L.check(ops._timed("barrier", 0.0, dev, lambda: L.load().qlin_peer_barrier(C.byref(self.args), ops._stream(dev))), "qlin_peer_barrier")
