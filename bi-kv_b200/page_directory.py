"""Python face of the native page directory (``include/bikv_pm.h``).

``PageDirectory`` offers the ``MultiPageManager`` methods (``load_item`` /
``access_item``; ``DistributedStorage/PageManager.py:136-161``, Go
``PageManager.go:306-356,404-417``) on top of the C++ implementation, with either
the Python coordinator's LRU policy or the Go coordinator's priority tiers.
``XorShiftChoice`` is the same generator as the native one, so a Python
``MultiPageManager(order="fast", rng=XorShiftChoice(seed))`` and a native LRU
directory with that seed make identical decisions.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import numpy as np

from . import _native as N

_MASK = (1 << 64) - 1


class XorShiftChoice:
    """xorshift64* as documented at ``bikv_pm_create``; ``choice`` picks like the native
    random shard choice."""

    def __init__(self, seed: int = 0):
        self.x = (seed or 0x9E3779B97F4A7C15) & _MASK

    def next(self) -> int:
        x = self.x
        x ^= x >> 12
        x ^= (x << 25) & _MASK
        x ^= x >> 27
        self.x = x
        return (x * 0x2545F4914F6CDD1D) & _MASK

    def choice(self, seq):
        return seq[(self.next() >> 33) % len(seq)]


class PageDirectory:
    def __init__(self, cache_size: int, page_size: int, kvcahe_num: int, policy: str = "lru", seed: int = 0,
                 ttl: Optional[int] = None, p1_max_pages: Optional[int] = None):
        self._lib = N.lib()
        self.policy = {"lru": N.PM_LRU, "tiered": N.PM_TIERED}[policy]
        self._h = self._lib.bikv_pm_create(cache_size, page_size, kvcahe_num, self.policy, seed)
        if not self._h:
            raise ValueError("bad page directory arguments")
        self.kvcahe_num = kvcahe_num
        self.page_size = page_size
        self.num_pages = cache_size // page_size
        self._pages = np.empty(max(self.num_pages, 1), dtype=np.int32)
        self._evicted = np.empty(4096, dtype=np.int64)
        if ttl is not None or p1_max_pages is not None:
            N.check(self._lib.bikv_pm_configure_tiers(self._h, ttl if ttl is not None else (1 << 62),
                                                      p1_max_pages if p1_max_pages is not None else self.num_pages // 4))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.bikv_pm_destroy(h)

    @property
    def handle(self):
        return self._h

    def load_item(self, item_id: int, list_length: int, weight: int = 0, item_type: str = "") -> Tuple[int, List[int]]:
        """(shard, pages); evicted ids of the call are in ``last_evicted``."""
        shard, cached, n_ev = C.c_int32(), C.c_int32(), C.c_int64()
        n = self._lib.bikv_pm_load_item(self._h, item_id, list_length, weight, int(item_type == "user cache"),
                                        C.byref(shard), self._pages.ctypes.data_as(C.c_void_p), len(self._pages),
                                        C.byref(cached), self._evicted.ctypes.data_as(C.c_void_p),
                                        len(self._evicted), C.byref(n_ev))
        if n == N.ERR_TOO_LARGE:
            raise ValueError("item too large for the pool")
        if n == N.PM_FULL:
            raise RuntimeError("Unable to free enough pages, even if all items are swapped out")
        if n < 0:
            raise N.BikvError(int(n), "bikv_pm_load_item")
        self.last_evicted = self._evicted[: min(n_ev.value, len(self._evicted))].tolist()
        self.last_was_cached = bool(cached.value)
        return shard.value, self._pages[:n].tolist()

    def access_item(self, item_id: int) -> Tuple[Optional[int], Optional[List[int]]]:
        shard = C.c_int32()
        n = self._lib.bikv_pm_access_item(self._h, item_id, C.byref(shard),
                                          self._pages.ctypes.data_as(C.c_void_p), len(self._pages))
        if n == N.PM_MISS:
            return None, None
        if n < 0:
            raise N.BikvError(int(n), "bikv_pm_access_item")
        return shard.value, self._pages[:n].tolist()

    def set_protected(self, item_id: int) -> None:
        if self._lib.bikv_pm_set_protected(self._h, item_id) != 0:
            raise KeyError(f"item {item_id} is not loaded")

    def remove_protected(self, item_id: int) -> None:
        if self._lib.bikv_pm_remove_protected(self._h, item_id) != 0:
            raise KeyError(f"item {item_id} is not loaded")

    def advance_clock(self, now: int) -> None:
        N.check(self._lib.bikv_pm_advance_clock(self._h, now), "bikv_pm_advance_clock")

    def set_clock(self, now: int) -> None:
        """Moves the clock forward without running the TTL pass (see ``bikv_pm_set_clock``)."""
        N.check(self._lib.bikv_pm_set_clock(self._h, now), "bikv_pm_set_clock")

    def free_pages(self, shard: int) -> int:
        return int(self._lib.bikv_pm_free_pages(self._h, shard))

    def item_count(self, shard: int) -> int:
        return int(self._lib.bikv_pm_item_count(self._h, shard))

    def priority(self, item_id: int) -> Optional[int]:
        p = self._lib.bikv_pm_item_priority(self._h, item_id)
        return None if p == N.PM_MISS else int(p)

    @property
    def evictions(self) -> int:
        return int(self._lib.bikv_pm_evictions(self._h))
