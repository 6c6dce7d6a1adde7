"""Host-side helpers for one-process-per-GPU runs.  Nothing here touches the data path:
pages move by direct loads/stores through peer mappings, never by a collective."""
from __future__ import annotations

import datetime
from typing import Sequence

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
