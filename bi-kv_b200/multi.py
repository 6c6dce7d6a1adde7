"""Host-side helpers for one-process-per-GPU runs.  Nothing here touches the data path:
pages move by direct loads/stores through peer mappings, never by a collective."""
from __future__ import annotations

import datetime
import mmap
import os
import struct
import time
import uuid
from typing import Optional, Sequence

import torch
import torch.distributed as dist


def reduce_over_ranks(values: Sequence[float], op: str, group=None, device="cpu") -> list:
    """Element-wise max or sum of a few floats over the ranks of ``group``."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op], group=group)
    return t.tolist()


def host_barrier(group=None, timeout_s: float = 60.0) -> None:
    """Barrier on a gloo group that FAILS instead of hanging when a rank is gone: raises
    ``RuntimeError`` after ``timeout_s`` naming the missing ranks.  Used between a scatter
    phase and a gather phase that depends on it."""
    dist.monitored_barrier(group=group, timeout=datetime.timedelta(seconds=timeout_s), wait_all_ranks=True)


def worker_of_request(request_id: int, n_workers: int) -> int:
    """Request placement of the reference's scheduler (``Scheduler/LLMScheduler.py:296-297``)."""
    return request_id % n_workers


class ShmBarrier:
    """Barrier for the ranks of one host through a small POSIX shared-memory block.

    Phase alignment costs one barrier per copy phase, and a phase lasts a few milliseconds, so
    the barrier's own latency shows: a gloo barrier over loopback TCP takes a few hundred
    microseconds for 8 ranks, this one a few microseconds.  Each rank owns one 64-byte slot
    holding the number of the last barrier it has entered; a rank leaves barrier ``k`` when
    every slot holds at least ``k``.  Like :func:`host_barrier` it does not hang on a rank that
    is gone: after ``timeout_s`` it raises ``RuntimeError`` naming the ranks that did not
    arrive.  The block is created by the group's rank 0 and its name travels through the
    group once, at construction."""

    SLOT = 64

    def __init__(self, group=None, name: Optional[str] = None):
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if name is None:
            names = [f"bikv_barrier_{os.getpid()}_{uuid.uuid4().hex[:10]}" if self.rank == 0 else None]
            if self.rank == 0:
                self._create(names[0])
            dist.broadcast_object_list(names, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                       group=group)
            name = names[0]
        elif self.rank == 0:
            self._create(name)
        self.name = name
        self._open(name)
        self.count = 0
        dist.barrier(group=group)           # everyone has the block mapped before rank 0 may unlink it
        if self.rank == 0:
            os.unlink(self._path(name))     # the mappings keep it alive; nothing is left behind in /dev/shm

    @staticmethod
    def _path(name: str) -> str:
        return os.path.join("/dev/shm", name)

    def _create(self, name: str) -> None:
        fd = os.open(self._path(name), os.O_RDWR | os.O_CREAT | os.O_EXCL, 0o600)
        try:
            os.ftruncate(fd, self.SLOT * self.world)
        finally:
            os.close(fd)

    def _open(self, name: str) -> None:
        fd = os.open(self._path(name), os.O_RDWR)
        try:
            self.map = mmap.mmap(fd, self.SLOT * self.world)
        finally:
            os.close(fd)

    def wait(self, timeout_s: float = 60.0) -> None:
        self.count += 1
        k = self.count
        struct.pack_into("<q", self.map, self.SLOT * self.rank, k)
        slots = [self.SLOT * r for r in range(self.world) if r != self.rank]
        deadline = None
        spins = 0
        while True:
            slots = [at for at in slots if struct.unpack_from("<q", self.map, at)[0] < k]
            if not slots:
                return
            spins += 1
            if spins & 0x3FF == 0:
                now = time.monotonic()
                if deadline is None:
                    deadline = now + timeout_s
                elif now > deadline:
                    missing = [at // self.SLOT for at in slots]
                    raise RuntimeError(f"barrier {k}: ranks {missing} did not arrive within {timeout_s} s")
                if spins > (1 << 16):
                    time.sleep(0.0002)       # a long wait: stop burning the core

    def close(self) -> None:
        m, self.map = getattr(self, "map", None), None
        if m is not None:
            m.close()
