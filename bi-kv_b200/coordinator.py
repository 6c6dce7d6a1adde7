"""Coordinator-driven prefix-reuse workload (benchmark configuration 4), host side.

Plays the coordinator's part for the data path: every request names a user; the user's
cached history prefix is looked up in a ``MultiPageManager`` (hit -> the pages are
GATHERED into the request's KV tensor; miss -> pages are allocated, LRU items evicted if
the pool is full, and the prefix is SCATTERED in), and the request's new tokens are always
written back as a fresh item.  The decisions follow the live branch of the reference's
coordinator loop (``DistributedStorage/CacheCoordinator.py:180-236``: CHECK -> hit/miss
through the page manager, SEND filled with ``cache_worker`` + ``cache_pages_list``, RECV ->
``load_item``) with the page managers of ``page_manager.py``.

Within one batch every gather is issued before any scatter, and every item a batch
touches is protected from eviction until the batch is planned (the reference has the
protection counters, ``PageManager.py:91-103``, and leaves the calls commented out,
``Worker/Worker.py:150,209-211``); together these guarantee that no page is read after it
has been recycled and no page is written twice in a batch.
"""
from __future__ import annotations

import ctypes as C
import random
from dataclasses import dataclass
from typing import Iterator, List, Optional, Tuple

import numpy as np

from . import _native as N
from .page_manager import MultiPageManager
from .plan import Plan, build_plan


@dataclass
class Request:
    request_id: int
    user: int
    prefix_tokens: int
    new_tokens: int
    worker: int

    @property
    def tokens(self) -> int:
        return self.prefix_tokens + self.new_tokens


class PrefixReuseWorkload:
    """Seeded request stream: users ~ Zipf(s) over ``n_users`` ranks (inverse CDF), one fixed
    prefix length per user ~ lognormal(median, sigma) clipped, new tokens ~ U[lo, hi]."""

    def __init__(self, seed: int = 0, n_users: int = 100_000, zipf_s: float = 1.1, prefix_median: int = 1024,
                 prefix_sigma: float = 0.8, prefix_clip: Tuple[int, int] = (128, 8192),
                 new_tokens: Tuple[int, int] = (32, 256), n_requests: int = 20_000, batch: int = 64,
                 n_workers: int = 4):
        rng = np.random.default_rng(seed)
        weights = np.arange(1, n_users + 1, dtype=np.float64) ** (-zipf_s)
        cdf = np.cumsum(weights)
        cdf /= cdf[-1]
        self.users = np.searchsorted(cdf, rng.random(n_requests)).astype(np.int64)
        plen = rng.lognormal(np.log(prefix_median), prefix_sigma, size=n_users)
        self.prefix_of_user = np.clip(np.rint(plen), *prefix_clip).astype(np.int64)
        self.new = rng.integers(new_tokens[0], new_tokens[1] + 1, size=n_requests).astype(np.int64)
        self.n_users, self.n_requests, self.batch, self.n_workers = n_users, n_requests, batch, n_workers

    def batches(self) -> Iterator[List[Request]]:
        for at in range(0, self.n_requests, self.batch):
            yield [Request(i, int(self.users[i]), int(self.prefix_of_user[self.users[i]]), int(self.new[i]),
                           i % self.n_workers)          # request_id % workers, Scheduler/LLMScheduler.py:296-297
                   for i in range(at, min(at + self.batch, self.n_requests))]


@dataclass
class BatchPlan:
    """What one worker executes for one batch: tensors of ``tokens[i]`` tokens per request,
    a gather plan (hits' prefixes) and a scatter plan (misses' prefixes + all new tokens)."""
    requests: List[Request]
    gather: Plan
    scatter: Plan
    hit: List[bool]
    evicted: int = 0

    @property
    def tokens(self) -> List[int]:
        return [r.tokens for r in self.requests]


class PrefixCacheCoordinator:
    def __init__(self, n_shards: int, pages_per_shard: int, page_tokens: int, order: str = "reference",
                 seed: int = 0, rng=None):
        self.n_shards, self.pages_per_shard, self.page_tokens = n_shards, pages_per_shard, page_tokens
        self.pm = MultiPageManager(pages_per_shard * page_tokens, page_tokens, n_shards,
                                   rng=rng if rng is not None else random.Random(seed), order=order)
        self.hits = self.misses = 0
        self._next_new_item = 1 << 40      # ids of written-back new-token items, never user ids
        self._stored_tokens = {}           # item id -> tokens it holds

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def _protect(self, shard: int, item) -> None:
        self.pm.page_managers[shard].set_protected(item)

    def plan_batch(self, requests: List[Request]) -> BatchPlan:
        """Plans one worker's share of a batch.  Records are in request order; request ``i``
        of the list uses worker tensor ``i``."""
        g_pages, g_tokens, g_req, g_shard = [], [], [], []
        s_pages, s_tokens, s_req, s_shard, s_off = [], [], [], [], []
        hit, touched = [], []
        stored_now = set()     # users whose prefix is being stored by THIS batch
        for i, r in enumerate(requests):
            shard, pages = self.pm.access_item(r.user)
            if r.user in stored_now:
                # Missed earlier in this batch: the pages exist but are filled only by this
                # batch's scatter, which runs after its gathers.  The request computes its
                # prefix like the first one did; nothing to read, nothing more to store.
                self.misses += 1
                hit.append(False)
            elif shard is not None and self._stored_tokens.get(r.user) == r.prefix_tokens:
                self.hits += 1
                hit.append(True)
                g_pages.append(pages), g_tokens.append(r.prefix_tokens), g_req.append(i), g_shard.append(shard)
            else:
                self.misses += 1
                hit.append(False)
                shard, pages = self.pm.load_item(r.user, r.prefix_tokens)
                self._stored_tokens[r.user] = r.prefix_tokens
                stored_now.add(r.user)
                s_pages.append(pages), s_tokens.append(r.prefix_tokens), s_req.append(i)
                s_shard.append(shard), s_off.append(0)
            self._protect(shard, r.user)
            touched.append((shard, r.user))
            item = self._next_new_item
            self._next_new_item += 1
            shard, pages = self.pm.load_item(item, r.new_tokens)
            self._stored_tokens[item] = r.new_tokens
            self._protect(shard, item)
            touched.append((shard, item))
            s_pages.append(pages), s_tokens.append(r.new_tokens), s_req.append(i)
            s_shard.append(shard), s_off.append(r.prefix_tokens)
        for shard, item in touched:
            self.pm.page_managers[shard].remove_protected(item)
        # forget bookkeeping of evicted items
        live = set().union(*self.pm.cached_ids)
        if len(self._stored_tokens) > 2 * len(live) + 1024:
            self._stored_tokens = {k: v for k, v in self._stored_tokens.items() if k in live}
        n = len(requests)
        gather = build_plan(g_pages, g_tokens, self.page_tokens, item_request=g_req, n_requests=n,
                            item_shard=g_shard, pages_per_shard=self.pages_per_shard)
        scatter = build_plan(s_pages, s_tokens, self.page_tokens, item_request=s_req, n_requests=n,
                             item_shard=s_shard, pages_per_shard=self.pages_per_shard)
        # A request's new tokens sit behind its prefix in the worker tensor; on a miss both
        # its items are scattered and build_plan's running offset already places them so.
        # When the prefix is not scattered (a hit, or a repeat of a user this batch already
        # stores) the request's only scattered item must start at prefix_tokens.
        table = scatter.table
        with_prefix = set(s_req[k] for k in range(len(s_req)) if s_off[k] == 0)
        for i in range(n):
            if i not in with_prefix:
                rows = table[:, 2] == i
                table[rows, 3] += requests[i].prefix_tokens
        return BatchPlan(requests, gather, scatter, hit)


class NativePrefixCacheCoordinator:
    """Same planner on the native page directory: one ``bikv_pm_plan_prefix_batch`` call per
    batch instead of a Python loop over requests (LRU policy, smallest-free-page allocation:
    the decisions of ``PrefixCacheCoordinator(order="fast", rng=XorShiftChoice(seed))``)."""

    def __init__(self, n_shards: int, pages_per_shard: int, page_tokens: int, seed: int = 0,
                 transient_plans: bool = False):
        """``transient_plans``: the plans of a batch hand their pinned buffers back when the batch
        plan is dropped (a caller that keeps ``table`` views beyond that must leave it off)."""
        from .page_directory import PageDirectory

        self.transient_plans = bool(transient_plans)

        self.n_shards, self.pages_per_shard, self.page_tokens = n_shards, pages_per_shard, page_tokens
        self.pm = PageDirectory(pages_per_shard * page_tokens, page_tokens, n_shards, policy="lru", seed=seed)
        self.hits = self.misses = 0
        self._next_item = C.c_int64(1 << 40)

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def plan_batch(self, requests: List[Request]) -> BatchPlan:
        from .plan import _pinned_i32

        n = len(requests)
        users = np.fromiter((r.user for r in requests), dtype=np.int64, count=n)
        prefix = np.fromiter((r.prefix_tokens for r in requests), dtype=np.int32, count=n)
        fresh = np.fromiter((r.new_tokens for r in requests), dtype=np.int32, count=n)
        P = self.page_tokens
        g_cap = int(((prefix + P - 1) // P).sum())
        s_cap = g_cap + int(((fresh + P - 1) // P).sum())
        g_store, s_store = _pinned_i32(g_cap, 4), _pinned_i32(s_cap, 4)
        hit = np.zeros(max(n, 1), dtype=np.uint8)
        n_g, n_s = C.c_int64(), C.c_int64()
        ptr = lambda a: a.ctypes.data_as(C.c_void_p)
        rc = N.lib().bikv_pm_plan_prefix_batch(self.pm.handle, ptr(users), ptr(prefix), ptr(fresh), n,
                                               C.byref(self._next_item), C.c_void_p(g_store.data_ptr()), g_cap,
                                               C.byref(n_g), C.c_void_p(s_store.data_ptr()), s_cap, C.byref(n_s),
                                               ptr(hit))
        N.check(rc, "bikv_pm_plan_prefix_batch")
        hits = hit[:n].astype(bool).tolist()
        self.hits += sum(hits)
        self.misses += n - sum(hits)
        tokens = np.array([r.tokens for r in requests], dtype=np.int64)
        tr = self.transient_plans
        return BatchPlan(requests, Plan(g_store, n_g.value, tokens.copy(), tr), Plan(s_store, n_s.value, tokens.copy(), tr),
                         hits)


def split_by_worker(bp: BatchPlan, n_workers: int, gather_flags: Optional[np.ndarray] = None,
                    transient: bool = False):
    """One plan per worker out of a plan made for the WHOLE batch.  Planning the batch in one
    piece matters: a user that two requests of one batch name -- on different workers -- is
    stored by the first and, like a repeat on one worker, must not be read by the second,
    because every gather of a batch runs before (or while) its scatters do.  Planned share by
    share, the second request would see the entry the first one just made and count as a hit
    on pages nobody has written yet.  Request ``i`` of worker ``k``'s share is the ``i``-th
    request of the batch with ``worker == k``; rows keep their order within a worker.

    ``gather_flags`` (one value per row of ``bp.gather``) is split alongside: the call then
    returns ``(plans, flags_per_worker)``.  ``transient``: the plans hand their pinned buffers
    back for reuse when they are dropped, so no ``table`` view of them may be kept beyond that."""
    from .plan import _pinned_i32

    n = len(bp.requests)
    worker_of = np.fromiter((r.worker for r in bp.requests), dtype=np.int64, count=n)
    tokens = np.fromiter((r.tokens for r in bp.requests), dtype=np.int64, count=n)
    by_worker = np.argsort(worker_of, kind="stable")
    n_req = np.bincount(worker_of, minlength=n_workers)
    first_req = np.concatenate(([0], np.cumsum(n_req)))
    local = np.empty(n, dtype=np.int32)
    local[by_worker] = np.arange(n, dtype=np.int32) - np.repeat(first_req[:-1], n_req).astype(np.int32)

    def split(plan: Plan, flags=None):
        t = plan.table
        w_rows = worker_of[t[:, 2]] if len(t) else np.zeros(0, dtype=np.int64)
        order = np.argsort(w_rows, kind="stable")
        rows = t[order]
        if len(rows):
            rows[:, 2] = local[rows[:, 2]]
        first = np.concatenate(([0], np.cumsum(np.bincount(w_rows, minlength=n_workers))))
        plans = []
        for k in range(n_workers):
            part = rows[first[k]:first[k + 1]]
            store = _pinned_i32(len(part), 4)
            store.numpy()[:len(part)] = part
            req_tokens = tokens[by_worker[first_req[k]:first_req[k + 1]]]
            plans.append(Plan(store, len(part), req_tokens if len(req_tokens) else np.zeros(1, dtype=np.int64),
                              transient))
        if flags is None:
            return plans, None
        f = np.asarray(flags)[order]
        return plans, [f[first[k]:first[k + 1]] for k in range(n_workers)]

    gathers, flags = split(bp.gather, gather_flags)
    scatters, _ = split(bp.scatter)
    out = []
    for k in range(n_workers):
        idx = by_worker[first_req[k]:first_req[k + 1]]
        out.append(BatchPlan([bp.requests[i] for i in idx], gathers[k], scatters[k], [bp.hit[i] for i in idx]))
    return out if gather_flags is None else (out, flags)


def plan_stream(batches, coordinator, n_workers: int, total_pages: int, transient: bool = False):
    """For a pipeline that gathers batch k+1 while batch k is still being scattered: yields, per
    batch, ``(plans, late, any_late)`` -- one plan per worker (:func:`split_by_worker` of the
    batch planned in one piece), per worker a boolean array marking the gather rows that read a
    page the batch BEFORE writes (a prefix stored by batch k and asked for again in batch k+1;
    those rows must wait for that scatter), and whether any row is marked.  ``total_pages``:
    page ids are below it.  Decided over all workers' rows, so every rank that replays the
    same stream decides alike."""
    being_written = np.zeros(int(total_pages), dtype=bool)       # by the batch before
    prev_written = np.zeros(0, dtype=np.int32)
    for batch in batches:
        bp = coordinator.plan_batch(batch)
        late = being_written[bp.gather.table[:, 0]]
        being_written[prev_written] = False
        prev_written = bp.scatter.table[:, 0].copy()
        being_written[prev_written] = True
        plans, masks = split_by_worker(bp, n_workers, gather_flags=late, transient=transient)
        yield plans, masks, bool(late.any())
