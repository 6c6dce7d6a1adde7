"""Restatement of the Go coordinator's page manager.  TEST INFRASTRUCTURE ONLY.

Follows ``Go/CacheCoordinator/PageManager.go`` (LoadItem :101-141, performEviction
:157-195, MultiPageManager.LoadItem :306-356, AccessItem :404-417,
checkAndAdjustP1Pages / downgradeP1Items :420-486, downgradeP2Items :503-526) with three
substitutions that make it reproducible -- the Go code itself cannot be built here (no Go
toolchain) and is nondeterministic by construction (map iteration order in allocatePages,
``rand.Intn``, wall-clock timestamps), so **page-id parity with it is unpinned**; what this
restatement pins are the decisions:
  * time is a logical counter (one tick per load/access, or set by ``advance_clock``);
  * the free page handed out is the smallest one;
  * the random shard comes from the xorshift64* generator given as ``rng``.
Plain dicts, sorts and scans throughout, as in the Go source.
"""
from __future__ import annotations


class GoPageManagerOracle:
    def __init__(self, cache_size, page_size, n_shards, rng, ttl=1 << 62, p1_max_pages=None):
        self.page_size = page_size
        self.num_pages = cache_size // page_size
        self.n = n_shards
        self.free = [set(range(self.num_pages)) for _ in range(n_shards)]
        self.table = [dict() for _ in range(n_shards)]     # id -> dict(pages, last, protected, priority)
        self.cached = [set() for _ in range(n_shards)]
        self.p2_items = set()
        self.p1_max = self.num_pages // 4 if p1_max_pages is None else p1_max_pages
        self.ttl = ttl
        self.clock = 0
        self.rng = rng

    def _tick(self):
        self.clock += 1
        return self.clock

    def access_item(self, item_id):
        for idx in range(self.n):
            if item_id in self.cached[idx]:
                e = self.table[idx][item_id]
                e["last"] = self._tick()
                return idx, list(e["pages"])
        return None, None

    def _evict(self, idx, required):
        cands = [(e["priority"], e["last"], i) for i, e in self.table[idx].items()
                 if e["protected"] == 0 and e["priority"] != 2]
        cands.sort()
        freed = []
        for _, _, i in cands:
            if len(self.free[idx]) >= required:
                break
            e = self.table[idx].pop(i)
            self.free[idx].update(e["pages"])
            freed.append(i)
        if len(self.free[idx]) < required:
            # The Go process panics here; what it evicted on the way stays evicted.
            for f in freed:
                self.cached[idx].discard(f)
                self.p2_items.discard(f)
            raise RuntimeError("cannot free enough pages")
        return freed

    def load_item(self, item_id, length, weight=0, item_type=""):
        hit = self.access_item(item_id)
        if hit[0] is not None:
            return hit[0], hit[1], []
        most = max(len(f) for f in self.free)
        if most > self.num_pages // 10:
            idx = 0
            for i in range(self.n):
                if len(self.free[i]) == most:
                    idx = i                      # the Go loop keeps the LAST shard with the maximum
        else:
            idx = self.rng.choice(list(range(self.n)))
        required = (length + self.page_size - 1) // self.page_size
        if required > self.num_pages:
            raise ValueError("item too large")
        freed = self._evict(idx, required) if len(self.free[idx]) < required else []
        pages = sorted(self.free[idx])[:required]
        self.free[idx].difference_update(pages)
        self.table[idx][item_id] = {"pages": pages, "last": self._tick(), "protected": 0,
                                    "priority": 2 if weight != 0 else 0}
        if item_type == "user cache":
            self.p2_items.add(item_id)
        self.cached[idx].add(item_id)
        for f in freed:
            self.cached[idx].discard(f)
            self.p2_items.discard(f)
        self._check_p1()
        return idx, pages, freed

    def _check_p1(self):
        p1 = [(e["last"], i, idx) for idx in range(self.n) for i, e in self.table[idx].items() if e["priority"] == 1]
        total = sum(len(self.table[idx][i]["pages"]) for _, i, idx in p1)
        excess = total - self.p1_max
        if excess <= 0:
            return
        p1.sort()
        released = 0
        for _, i, idx in p1:
            if released >= excess:
                break
            self.table[idx][i]["priority"] = 0
            released += len(self.table[idx][i]["pages"])

    def advance_clock(self, now):
        self.clock = max(self.clock, now)
        for i in sorted(self.p2_items):
            for idx in range(self.n):
                e = self.table[idx].get(i)
                if e is not None and e["priority"] == 2 and self.clock - e["last"] >= self.ttl:
                    e["priority"] = 1
                    self.p2_items.discard(i)
        self._check_p1()

    def priority(self, item_id):
        for idx in range(self.n):
            if item_id in self.table[idx]:
                return self.table[idx][item_id]["priority"]
        return None

    def set_protected(self, item_id, delta=1):
        for idx in range(self.n):
            if item_id in self.table[idx]:
                self.table[idx][item_id]["protected"] += delta
                return
        raise KeyError(item_id)
