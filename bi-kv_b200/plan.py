"""Plans: the coordinator's page lists turned into page records.

A record says: pool page ``page_id`` holds ``valid_tokens`` tokens that belong
at ``token_offset`` of worker tensor ``request``.  The walk over items and
pages, the running offset and the short-last-page rule restate the index loops
of ``KVCache.shared_data_batch_pages`` (``DistributedStorage/kvcache.py:158-174``);
unlike there, units are explicit (tokens here, bytes inside the kernels) and the
walk runs in native code over flat arrays.
"""
from __future__ import annotations

import ctypes as C
import itertools
import threading
from typing import Iterable, Optional, Sequence

import numpy as np
import torch

from . import _native as N

REC_DTYPE = np.dtype([("page_id", "<i4"), ("valid_tokens", "<i4"), ("request", "<i4"),
                      ("token_offset", "<i4")])


class _PinnedRows:
    """Recycles pinned int32 [rows, 4] buffers: pinning host memory costs far more than
    building a plan, so buffers of dropped TRANSIENT plans are handed out again.  A buffer
    comes back only when its ``Plan`` is garbage-collected; ``PageMover`` keeps every plan
    it has launched alive until the stream has passed the upload."""

    def __init__(self):
        self._free: list = []
        self._lock = threading.Lock()

    def get(self, n_rows: int) -> torch.Tensor:
        n_rows = max(n_rows, 1)
        with self._lock:
            for i, t in enumerate(self._free):
                if t.shape[0] >= n_rows:
                    return self._free.pop(i)
        cap = 1 << max(8, (n_rows - 1).bit_length())
        t = torch.empty((cap, 4), dtype=torch.int32)
        return t.pin_memory() if torch.cuda.is_available() else t

    def put(self, t: torch.Tensor) -> None:
        with self._lock:
            if len(self._free) < 16:
                self._free.append(t)
                self._free.sort(key=lambda x: x.shape[0])


_pinned = _PinnedRows()


def _pinned_i32(n_rows: int, cols: int) -> torch.Tensor:
    assert cols == 4
    return _pinned.get(n_rows)


class Plan:
    """Page records in host memory (pinned when a GPU is present)."""

    def __init__(self, recs: torch.Tensor, n_pages: int, request_tokens: np.ndarray, transient: bool = False):
        self._store = recs                      # int32 [cap, 4], keeps the memory alive
        self.n_pages = int(n_pages)
        self.request_tokens = request_tokens    # int64 [n_requests]
        self.transient = transient              # see __del__

    def __del__(self):
        # Only a plan marked transient gives its pinned buffer back for reuse: its creator
        # promised that no ``table`` / ``recs`` view outlives it (numpy views do not keep the
        # plan alive, so recycling under a live view would change what the view shows).
        store = self.__dict__.pop("_store", None)
        if store is None or not self.__dict__.get("transient") or _pinned is None:
            return
        try:
            _pinned.put(store)
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass

    @property
    def n_requests(self) -> int:
        return len(self.request_tokens)

    @property
    def recs(self) -> np.ndarray:
        """Structured view, one row per page."""
        return self._store.numpy()[: self.n_pages].view(REC_DTYPE).reshape(-1)

    @property
    def table(self) -> np.ndarray:
        """int32 [n_pages, 4] view: page_id, valid_tokens, request, token_offset."""
        return self._store.numpy()[: self.n_pages]

    @property
    def host_ptr(self) -> int:
        return self._store.data_ptr()

    @property
    def total_tokens(self) -> int:
        return int(self.request_tokens.sum())

    @classmethod
    def from_table(cls, table: np.ndarray, n_requests: Optional[int] = None, transient: bool = False) -> "Plan":
        table = np.ascontiguousarray(table, dtype=np.int32).reshape(-1, 4)
        store = _pinned_i32(len(table), 4)
        store.numpy()[: len(table)] = table
        nreq = int(n_requests if n_requests is not None else (table[:, 2].max() + 1 if len(table) else 1))
        req_tokens = np.zeros(nreq, dtype=np.int64)
        ok = (table[:, 2] >= 0) & (table[:, 2] < nreq)   # bad rows are the validator's business
        if ok.any():
            np.maximum.at(req_tokens, table[ok, 2], (table[ok, 1] + table[ok, 3]).astype(np.int64))
        return cls(store, len(table), req_tokens, transient)


def flatten_page_lists(cache_pages_list: Iterable[Sequence[int]]):
    """``List[List[int]]`` (or protobuf ``PageList`` messages) -> (flat int32, begin int64)."""
    lists = [getattr(p, "cache_pages_list", p) for p in cache_pages_list]
    lens = np.fromiter((len(p) for p in lists), dtype=np.int64, count=len(lists))
    begin = np.zeros(len(lists) + 1, dtype=np.int64)
    np.cumsum(lens, out=begin[1:])
    total = int(begin[-1])
    if lists and all(isinstance(p, np.ndarray) for p in lists):
        flat = np.concatenate(lists).astype(np.int32, copy=False)   # ~40x faster than iterating
    else:
        flat = np.fromiter(itertools.chain.from_iterable(lists), dtype=np.int32, count=total)
    return flat, begin


def build_plan(cache_pages_list, item_tokens, page_tokens: int, *, item_request=None,
               n_requests: int = 1, item_shard=None, pages_per_shard: int = 0, transient: bool = False) -> Plan:
    """Builds the records for a batch of items.

    ``cache_pages_list[j]`` are the pool pages of item ``j`` and ``item_tokens[j]``
    its token count (the ``cache_pages_list`` / ``id_token_pair`` of a combined
    task, ``DistributedStorage/kvcache.py:386-413``).  ``item_request[j]`` names
    the worker tensor the item lands in (default: all in tensor 0, one packed
    buffer as in the reference); offsets run per tensor in item order.
    ``item_shard`` turns shard-local page numbers into global ids for
    ``SHARD_BLOCK`` pools.  ``transient=True``: the caller keeps no ``table`` / ``recs`` view
    beyond the plan's life, so its pinned buffer may be reused by later plans.
    """
    if isinstance(cache_pages_list, tuple) and len(cache_pages_list) == 2:
        flat, begin = cache_pages_list
        flat = np.ascontiguousarray(flat, dtype=np.int32)
        begin = np.ascontiguousarray(begin, dtype=np.int64)
    else:
        flat, begin = flatten_page_lists(cache_pages_list)
    n_items = len(begin) - 1
    tokens = np.ascontiguousarray(item_tokens, dtype=np.int32)
    if len(tokens) != n_items:
        raise ValueError("item_tokens and cache_pages_list differ in length")
    req = None if item_request is None else np.ascontiguousarray(item_request, dtype=np.int32)
    shard = None if item_shard is None else np.ascontiguousarray(item_shard, dtype=np.int32)
    n_pages = int(begin[-1])
    store = _pinned_i32(n_pages, 4)
    req_tokens = np.zeros(n_requests, dtype=np.int64)
    ptr = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
    got = N.lib().bikv_plan_build(ptr(flat), ptr(begin), ptr(tokens), ptr(req), ptr(shard),
                                  int(pages_per_shard), n_items, int(page_tokens), ptr(req_tokens),
                                  int(n_requests), C.c_void_p(store.data_ptr()), n_pages)
    if got < 0:
        raise N.BikvError(int(got), "bikv_plan_build")
    return Plan(store, int(got), req_tokens, transient)


def plan_from_combined_task(task, page_tokens: int, *, pages_per_shard: int = 0,
                            block_sharded: bool = False) -> Plan:
    """Plan for a combined task (dict as built by ``receive_task_info_batch_gprc`` or a
    ``CombindedTaskInfo`` message): all items go into one packed tensor, in order."""
    if isinstance(task, dict):
        pages, pairs, cache_worker = task["cache_pages_list"], task["id_token_pair"], task["cache_worker"]
        tokens = [p[1] for p in pairs]
    else:
        pages, cache_worker = task.cache_pages_list, task.cache_worker
        tokens = [p.token_num for p in task.id_token_pair]
    shard = [cache_worker] * len(tokens) if block_sharded else None
    return build_plan(pages, tokens, page_tokens, item_shard=shard, pages_per_shard=pages_per_shard, transient=True)


def build_block_plan(cache_pages_list, item_tokens, page_tokens: int, block_ids, *, item_shard=None,
                     pages_per_shard: int = 0) -> Plan:
    """Plan for a worker whose KV is PAGED with blocks of ``page_tokens`` tokens: the k-th
    page of the batch (items in order, pages in order) lands in worker block
    ``block_ids[k]``, i.e. at slot ``block_ids[k] * page_tokens``.  Short last pages keep the
    rule of :func:`build_plan`."""
    plan = build_plan(cache_pages_list, item_tokens, page_tokens, item_shard=item_shard,
                      pages_per_shard=pages_per_shard)
    blocks = np.ascontiguousarray(block_ids, dtype=np.int64)
    if len(blocks) != plan.n_pages:
        raise ValueError(f"{plan.n_pages} pages but {len(blocks)} block ids")
    if len(blocks) and (blocks.min() < 0 or blocks.max() * page_tokens > 0x7fffffff - page_tokens):
        raise ValueError("block id out of range")
    plan.table[:, 3] = (blocks * page_tokens).astype(np.int32)
    return plan
