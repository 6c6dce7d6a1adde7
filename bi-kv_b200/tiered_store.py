"""Two-tier page store: a small pool in HBM backed by a larger pool in pinned host memory.

The reference keeps its whole pool in pinned host RAM and reads it from the GPU in place
(``DistributedStorage/kvcache.py:38-43,241-366``; ``zero_copy_page_kernel``,
``SharedMemory/CUDA_Shared/copy_kernel.cu:39-66``); the B200 design keeps the pool in HBM.
This module joins the two: items live in HBM while they are hot, an item that the HBM tier's
LRU evicts is DEMOTED -- its pages are copied to the host tier before anything overwrites
them -- and an item found only in the host tier is PROMOTED back on access.  Both moves are
flat page copies by the same kernel that serves the reference's zero-copy path
(``bikv_copy_pages_flat``: the host tier is read and written in place over PCIe / C2C), issued
on the caller's stream, so stream order alone keeps them ahead of the scatter or gather that
follows.

Each tier has its own page directory (``PageDirectory``, LRU).  The host tier is inclusive:
a promoted item keeps its host copy, so demoting it again later costs no copy as long as the
host tier has not evicted it (cached KV is immutable: an item id names one token sequence).

Page ids handed out are GLOBAL ids of a two-shard pool under the block rule: shard 0 is the
HBM tier, shard 1 the host tier (``pool`` below), so the ordinary gather/scatter entry points
work on them unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from . import _native as N
from .geometry import KVGeometry
from .mover import PageMover
from .page_directory import PageDirectory
from .pool import ShardedPool


@dataclass
class TierStats:
    hbm_hits: int = 0
    host_hits: int = 0
    misses: int = 0
    demotions: int = 0            # evictions from HBM that copied pages to the host tier
    clean_demotions: int = 0      # evictions whose host copy was still there: nothing copied
    promotions: int = 0
    dropped: int = 0              # evictions from HBM that the host tier could not take
    not_spilled: int = 0          # evictions of items the spill policy leaves out (see min_hits_to_spill)
    pages_demoted: int = 0
    pages_promoted: int = 0
    extra: dict = field(default_factory=dict)


class TieredPageStore:
    def __init__(self, geom: KVGeometry, hbm_pages: int, host_pages: int, device, mover: Optional[PageMover] = None,
                 seed: int = 0, copier=None, min_hits_to_spill: int = 0):
        """``min_hits_to_spill``: an item evicted from HBM is copied to the host tier only if it was
        fetched at least this often while it lived in HBM (0: every item is kept; 1: only items
        that have proved reusable -- host bandwidth is a fraction of HBM's, and most of what a
        prefix cache stores is never asked for again).  ``store(..., spill=False)`` excludes a
        single item.

        ``copier(src, dst, src_pages, dst_pages, stream)`` replaces the page-copy kernel; it
        exists so that the directory logic can be exercised on a machine without a GPU (with
        ``device="cpu"``).  Without it every move goes through ``PageMover.copy_pages_flat``,
        which needs the CUDA library and a CUDA device."""
        if geom.pool_layout != N.POOL_PAGED:
            raise ValueError("the tiered store keeps pages in the paged layout")
        self.geom = geom
        self.device = torch.device(device)
        self._copier = copier
        if copier is None:
            self.mover = mover if mover is not None else PageMover(self.device)
        self.hbm_pages, self.host_pages = int(hbm_pages), int(host_pages)
        self.hbm = torch.zeros(geom.pool_shape(self.hbm_pages), dtype=geom.dtype, device=self.device)
        self.host = torch.zeros(geom.pool_shape(self.host_pages), dtype=geom.dtype,
                                pin_memory=self.device.type == "cuda")
        self._per = max(self.hbm_pages, self.host_pages)      # id stride between the two tiers
        self.pool = ShardedPool([self.hbm.data_ptr(), self.host.data_ptr()], self._per, geom, rule=N.SHARD_BLOCK,
                                device=self.device, keepalive=[self.hbm, self.host])
        P = geom.page_tokens
        self.dir_hbm = PageDirectory(self.hbm_pages * P, P, 1, policy="lru", seed=seed)
        self.dir_host = PageDirectory(self.host_pages * P, P, 1, policy="lru", seed=seed + 1)
        self._hbm_items: Dict[int, list] = {}                     # item -> [HBM pages, tokens, hits, spill]
        self.min_hits_to_spill = int(min_hits_to_spill)
        self._host_tokens: Dict[int, int] = {}                    # items the host tier was given
        self.stats = TierStats()
        self._batch: Optional[dict] = None

    # -- ids -----------------------------------------------------------------
    def global_ids(self, pages: List[int], tier: int = 0) -> List[int]:
        return [tier * self._per + int(p) for p in pages]

    # -- batches ---------------------------------------------------------------
    def begin_batch(self) -> None:
        """Until :meth:`end_batch`, every item stored or fetched is protected from eviction and
        the page copies are collected instead of launched.  With nothing touched in the batch
        evictable, no demotion can read a page a promotion of the same batch writes, so
        ``end_batch`` may launch all demotions as ONE copy and then all promotions as one."""
        if self._batch is not None:
            raise RuntimeError("a batch is already open")
        self._batch = {"down": ([], []), "up": ([], []), "touched": []}

    def end_batch(self, stream=None) -> None:
        """Launches the batch's demotions, then its promotions, on ``stream`` and lifts the
        protections.  Gathers and scatters of the batch come after this call, on that stream."""
        b, self._batch = self._batch, None
        if b is None:
            raise RuntimeError("no batch is open")
        self._copy(self.hbm, self.host, b["down"][0], b["down"][1], stream)
        self._copy(self.host, self.hbm, b["up"][0], b["up"][1], stream)
        for item in b["touched"]:
            self.dir_hbm.remove_protected(item)

    def _touch(self, item: int) -> None:
        if self._batch is not None:
            self.dir_hbm.set_protected(item)
            self._batch["touched"].append(item)

    # -- moves between the tiers ---------------------------------------------
    def _copy(self, src: torch.Tensor, dst: torch.Tensor, src_pages: List[int], dst_pages: List[int], stream) -> None:
        if not src_pages:
            return
        if self._batch is not None:
            kind = "down" if src is self.hbm else "up"
            self._batch[kind][0].extend(src_pages)
            self._batch[kind][1].extend(dst_pages)
            return
        if self._copier is not None:
            self._copier(src, dst, src_pages, dst_pages, stream)
            return
        pe = self.geom.page_elems
        so = torch.tensor(src_pages, dtype=torch.int64).mul_(pe).to(self.device, non_blocking=False)
        do = torch.tensor(dst_pages, dtype=torch.int64).mul_(pe).to(self.device, non_blocking=False)
        self.mover.copy_pages_flat(src, dst, so, do, pe, stream=stream)
        # the offset arrays must outlive the launch; torch frees them in stream order of the
        # current stream, so hold them until the copy's stream has passed
        self._hold = getattr(self, "_hold", [])
        ev = torch.cuda.Event()
        ev.record(stream if stream is not None else torch.cuda.current_stream(self.device))
        self._hold = [(e, t) for e, t in self._hold if not e.query()] + [(ev, (so, do))]

    def _demote(self, evicted: List[int], stream) -> None:
        """Items the HBM directory has just evicted: their old pages are still intact (nothing
        has been launched since), copy them out now."""
        src, dst = [], []
        for item in evicted:
            pages, tokens, hits, spill = self._hbm_items.pop(int(item), (None, 0, 0, False))
            if pages is None:
                continue
            if not spill or hits < self.min_hits_to_spill:
                self.stats.not_spilled += 1
                continue
            shard, host_pages = self.dir_host.access_item(item)
            if shard is not None and self._host_tokens.get(item) == tokens:
                self.stats.clean_demotions += 1
                continue
            try:
                _, host_pages = self.dir_host.load_item(item, tokens)
            except (ValueError, RuntimeError):
                self.stats.dropped += 1          # larger than the host tier, or nothing evictable
                continue
            for gone in self.dir_host.last_evicted:
                self._host_tokens.pop(int(gone), None)
            self._host_tokens[int(item)] = tokens
            src += pages
            dst += host_pages
            self.stats.demotions += 1
        self.stats.pages_demoted += len(src)
        self._copy(self.hbm, self.host, src, dst, stream)

    # -- the store's interface -------------------------------------------------
    def store(self, item: int, tokens: int, stream=None, spill: bool = True) -> List[int]:
        """Pages (global ids, HBM tier) for a NEW item of ``tokens`` tokens; the caller scatters
        into them on ``stream`` afterwards.  Items the allocation evicts are demoted first.
        ``spill=False``: this item is simply dropped when HBM evicts it."""
        item = int(item)
        if item in self._hbm_items:
            raise ValueError(f"item {item} is already stored (cached KV is immutable)")
        self._host_tokens.pop(item, None)        # any host copy of a re-stored id is stale
        _, pages = self.dir_hbm.load_item(item, tokens)
        self._demote(self.dir_hbm.last_evicted, stream)
        self._hbm_items[item] = [pages, int(tokens), 0, bool(spill)]
        self._touch(item)
        return self.global_ids(pages, 0)

    def fetch(self, item: int, stream=None) -> Optional[List[int]]:
        """Pages (global ids, HBM tier) holding ``item``, promoting it from the host tier when it
        is only there; None on a miss.  The caller gathers from them on ``stream`` afterwards."""
        item = int(item)
        hit = self._hbm_items.get(item)
        if hit is not None:
            self.dir_hbm.access_item(item)
            hit[2] += 1
            self.stats.hbm_hits += 1
            self._touch(item)
            return self.global_ids(hit[0], 0)
        tokens = self._host_tokens.get(item)
        shard, host_pages = self.dir_host.access_item(item) if tokens is not None else (None, None)
        if shard is None:
            self._host_tokens.pop(item, None)
            self.stats.misses += 1
            return None
        _, pages = self.dir_hbm.load_item(item, tokens)
        self._demote(self.dir_hbm.last_evicted, stream)
        self._copy(self.host, self.hbm, host_pages, pages, stream)
        self._hbm_items[item] = [pages, tokens, 1, True]
        self.stats.host_hits += 1
        self.stats.promotions += 1
        self.stats.pages_promoted += len(pages)
        self._touch(item)
        return self.global_ids(pages, 0)

    def protect(self, item: int) -> None:
        """Keeps an item in HBM until :meth:`release` (while a batch that uses it is planned)."""
        self.dir_hbm.set_protected(int(item))

    def release(self, item: int) -> None:
        self.dir_hbm.remove_protected(int(item))

    def tokens_of(self, item: int) -> Optional[int]:
        hit = self._hbm_items.get(int(item))
        return hit[1] if hit is not None else self._host_tokens.get(int(item))

    def where(self, item: int) -> Optional[str]:
        if int(item) in self._hbm_items:
            return "hbm"
        if int(item) in self._host_tokens and self.dir_host.priority(int(item)) is not None:
            return "host"
        return None
