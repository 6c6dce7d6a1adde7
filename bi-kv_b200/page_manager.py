"""Page tables that produce the ``cache_pages_list`` of a plan.

``PageManager`` and ``MultiPageManager`` take the same arguments, return the same
values and make the same decisions as ``DistributedStorage/PageManager.py:8-161``
(page numbers, their order inside a list, who is evicted, which shard is
chosen), so a plan produced here is the plan the reference would have produced.
The bookkeeping differs: least-recently-used order is an ordered map touched
on access (the reference sorts the whole table at every eviction,
``PageManager.py:65-68``), and free pages sit in a binary heap.

Page numbers in the reference depend on CPython's ``set`` internals: free pages
live in a ``set``, the next page is ``next(iter(free_set))``, freed pages come
back through ``set.update`` (where a re-inserted number may land in a different
slot than before), and an item's pages are returned as ``list(set_of_pages)``
(``PageManager.py:105-115``).  No closed form describes that order, so the
default ``order="reference"`` performs the same operations on real ``set``
objects and is identical by construction on the same interpreter.
``order="fast"`` hands out the smallest free page from a heap instead: O(log n)
per page, deterministic on any interpreter, same eviction decisions, but page
numbers differ from the reference's once pages have been recycled.
"""
from __future__ import annotations

import heapq
import random as _random
from collections import OrderedDict
from typing import Dict, Hashable, List, Optional, Tuple


class _FreePages:
    """Free page numbers, smallest first."""

    def __init__(self, n: int):
        self._heap = list(range(n))  # already a valid heap
        self._members = bytearray(b"\x01") * n
        self._count = n

    def __len__(self) -> int:
        return self._count

    def __contains__(self, page: int) -> bool:
        return 0 <= page < len(self._members) and self._members[page] == 1

    def __iter__(self):
        return iter(sorted(self._heap))

    def pop_smallest(self) -> int:
        p = heapq.heappop(self._heap)
        self._members[p] = 0
        self._count -= 1
        return p

    def update(self, pages) -> None:
        for p in pages:
            if self._members[p]:
                continue
            self._members[p] = 1
            self._count += 1
            heapq.heappush(self._heap, p)


class PageManager:
    """One shard's page table: item id -> pages, LRU eviction, protection count."""

    def __init__(self, cache_size: int, page_size: int, pm_id: int = 0, order: str = "reference"):
        if order not in ("reference", "fast"):
            raise ValueError("order must be 'reference' or 'fast'")
        self.pm_id = pm_id
        self.page_size = page_size
        self.num_pages = cache_size // page_size
        self.order = order
        self.free_pages = set(range(self.num_pages)) if order == "reference" else _FreePages(self.num_pages)
        # Oldest access first.  Values keep the reference's keys.
        self.page_table: "OrderedDict[Hashable, Dict]" = OrderedDict()
        self._birth: Dict[Hashable, int] = {}   # load order, for get_loaded_lists
        self._births = 0
        self.current_time = 0

    def load_item(self, item_id, list_length: int) -> Tuple[List[int], list]:
        """Allocates pages for ``list_length`` tokens; evicts LRU items if needed.
        Returns ``(pages, evicted item ids)``; a known item is only touched."""
        if item_id in self.page_table:
            return self.access_item(item_id), []
        required = (list_length + self.page_size - 1) // self.page_size
        if required > self.num_pages:
            raise ValueError("item too large for the pool")
        freed_ids: list = []
        if len(self.free_pages) < required:
            freed_ids = self._perform_eviction(required)
        pages = self._allocate_pages(required)
        self.page_table[item_id] = {"pages": pages, "last_accessed": self.current_time, "protected": 0}
        self._birth[item_id] = self._births
        self._births += 1
        self.current_time += 1
        return pages, freed_ids

    def access_item(self, item_id) -> List[int]:
        entry = self.page_table.get(item_id)
        if entry is None:
            raise KeyError(f"item {item_id} is not loaded")
        entry["last_accessed"] = self.current_time
        self.current_time += 1
        self.page_table.move_to_end(item_id)
        return entry["pages"]

    def _perform_eviction(self, required: int) -> list:
        freed_ids = []
        for item_id in list(self.page_table.keys()):
            entry = self.page_table[item_id]
            if entry["protected"] != 0:
                continue
            del self.page_table[item_id]
            del self._birth[item_id]
            self.free_pages.update(entry["pages"])
            freed_ids.append(item_id)
            if len(self.free_pages) >= required:
                break
        if len(self.free_pages) < required:
            raise RuntimeError("Unable to free enough pages, even if all items are swapped out")
        return freed_ids

    def set_protected(self, item_id) -> None:
        if item_id not in self.page_table:
            raise KeyError(f"item {item_id} is not loaded")
        self.page_table[item_id]["protected"] += 1

    def remove_protected(self, item_id) -> None:
        if item_id not in self.page_table:
            raise KeyError(f"item {item_id} is not loaded")
        self.page_table[item_id]["protected"] -= 1

    def _allocate_pages(self, n: int) -> List[int]:
        if len(self.free_pages) < n:
            raise RuntimeError("internal error: not enough free pages")
        if self.order == "fast":
            return [self.free_pages.pop_smallest() for _ in range(n)]
        free, taken = self.free_pages, set()
        while len(taken) < n:
            page = next(iter(free))
            free.remove(page)
            taken.add(page)
        return list(taken)

    def _page_to_location(self, page: int) -> int:
        return page * self.page_size

    def get_loaded_lists(self) -> list:
        """Loaded item ids in the order they were first loaded (the reference's dict
        keeps insertion order; access does not reorder it)."""
        return sorted(self.page_table.keys(), key=self._birth.__getitem__)


class MultiPageManager:
    """Several shards.  A new item goes to the shard with most free pages while any
    shard has more than a tenth of its pages free, else to a random shard
    (``PageManager.py:136-154``; ``rng`` defaults to the module ``random`` the
    reference draws from)."""

    def __init__(self, cache_size: int, page_size: int, kvcahe_num: int, rng=None, order: str = "reference"):
        self.kvcahe_num = kvcahe_num
        self.page_managers = [PageManager(cache_size, page_size, pm_id=i, order=order) for i in range(kvcahe_num)]
        self.buffer_size = cache_size
        self.page_size = page_size
        self.num_pages = cache_size // page_size
        self.cached_ids = [set() for _ in range(kvcahe_num)]
        self._rng = rng if rng is not None else _random

    def load_item(self, item_id, list_length: int) -> Tuple[int, List[int]]:
        most_free = max(len(pm.free_pages) for pm in self.page_managers)
        if most_free > (self.num_pages / 10):
            target = max(self.page_managers, key=lambda pm: len(pm.free_pages))
        else:
            target = self._rng.choice(self.page_managers)
        pages, freed_ids = target.load_item(item_id, list_length)
        self.cached_ids[target.pm_id].add(item_id)
        for fid in freed_ids:
            self.cached_ids[target.pm_id].remove(fid)
        return target.pm_id, pages

    def access_item(self, item_id) -> Tuple[Optional[int], Optional[List[int]]]:
        for idx, ids in enumerate(self.cached_ids):
            if item_id in ids:
                return idx, self.page_managers[idx].access_item(item_id)
        return None, None
