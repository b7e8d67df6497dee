"""Optional gather of the per-rank output slabs over NCCL (``ember_gather_outputs``).

Forward and backward shard over (batch * head) with no exchange (``ember_b200.shard``); this module
is only for callers that want the whole result on every rank. ``Communicator`` does the host-side
rendezvous through any key/value store with ``set``/``get``/``wait`` (``torch.distributed``'s
TCPStore, FileStore, HashStore or the store of an initialised process group): rank 0 publishes the
NCCL id, every rank checks in, and only when ALL ranks have checked in within the time limit is the
communicator built. A rank that never arrives therefore ends as a ``TimeoutError`` on the host of
the others, naming the missing ranks, before anything was launched on a GPU.
"""
from __future__ import annotations

import ctypes
import datetime
import time

from . import _lib
from .shard import shard_range


def wait_for_ranks(store, world: int, timeout_s: float, prefix: str = "ember_comm") -> None:
    """Blocks until ranks 0..world-1 have all checked in under ``prefix``; raises TimeoutError with
    the ranks still missing."""
    keys = [f"{prefix}/rank{r}" for r in range(world)]
    deadline = time.monotonic() + timeout_s
    missing = list(range(world))
    while True:
        still = []
        for r in missing:
            try:
                store.wait([keys[r]], datetime.timedelta(milliseconds=50))
            except Exception:
                still.append(r)
        missing = still
        if not missing:
            return
        if time.monotonic() > deadline:
            raise TimeoutError(f"ranks {missing} of {world} did not check in within {timeout_s:.1f} s")


class Communicator:
    """One NCCL communicator over ``world`` ranks, built after a host-side check-in."""

    def __init__(self, rank: int, world: int, store, timeout_s: float = 60.0, prefix: str = "ember_comm"):
        if world <= 0 or not (0 <= rank < world):
            raise ValueError(f"bad rank/world: {rank}/{world}")
        self.rank, self.world, self._comm = rank, world, None
        L = _lib.lib()
        if rank == 0:
            buf = ctypes.create_string_buffer(128)
            _lib.check(L.ember_comm_unique_id(buf))
            store.set(f"{prefix}/id", buf.raw)
        store.set(f"{prefix}/rank{rank}", b"1")
        wait_for_ranks(store, world, timeout_s, prefix)
        uid = bytes(store.get(f"{prefix}/id"))
        comm = ctypes.c_void_p()
        _lib.check(L.ember_comm_init(ctypes.byref(comm), uid, rank, world, int(timeout_s * 1000)))
        self._comm = comm

    def slab(self, batch_heads: int) -> tuple[int, int]:
        """[begin, end) of the (batch*head) units this rank owns."""
        return shard_range(batch_heads, self.rank, self.world)

    def gather_into(self, out_full_ptr: int, slab_ptr: int, slab_bytes: int, stream=None) -> None:
        """Raw form: device addresses; every rank passes the same ``slab_bytes``."""
        _lib.check(_lib.lib().ember_gather_outputs(out_full_ptr, slab_ptr, slab_bytes, self._comm, stream))

    def gather(self, slab):
        """``slab``: an ``ember_b200.Tensor`` whose leading axis is this rank's share of the sharded
        axis (equal on all ranks). Returns the full tensor (leading axis times ``world``)."""
        from .tensor import Tensor

        full = Tensor.empty((slab.shape[0] * self.world,) + tuple(slab.shape[1:]), slab.dtype)
        es = 2 if slab.dtype == "bfloat16" else 4
        self.gather_into(full.ptr, slab.ptr, slab.size * es)
        return full

    def close(self) -> None:
        if self._comm is not None:
            _lib.check(_lib.lib().ember_comm_destroy(self._comm))
            self._comm = None
