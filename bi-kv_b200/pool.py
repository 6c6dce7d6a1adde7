"""Sharded page pools as one worker GPU addresses them.

A pool is ``n_shards`` device allocations of ``pages_per_shard`` pages each.
The worker GPU holds one base pointer per shard: its own memory, a peer GPU's
memory mapped in-process, or another process's allocation opened through a
CUDA IPC handle (the role of ``consumer_init`` / ``producer_init`` in
``SharedMemory/CUDA_Shared/ipc_service.cpp:20-110``, minus the staging ring:
kernels read and write the shard memory itself).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _native as N
from .geometry import KVGeometry


def shard_of(page_id, n_shards: int, pages_per_shard: int, rule: int = N.SHARD_MOD):
    """(shard, local page) of a global page id; works on ints and arrays."""
    if rule == N.SHARD_MOD:
        return page_id % n_shards, page_id // n_shards
    return page_id // pages_per_shard, page_id % pages_per_shard


def global_page_id(shard, local, n_shards: int, pages_per_shard: int, rule: int = N.SHARD_MOD):
    if rule == N.SHARD_MOD:
        return local * n_shards + shard
    return shard * pages_per_shard + local


class ShardedPool:
    """Base pointers of every shard, valid on ``device``."""

    def __init__(self, bases: Sequence[int], pages_per_shard: int, geom: KVGeometry,
                 rule: int = N.SHARD_MOD, device: Optional[torch.device] = None,
                 keepalive: Optional[list] = None, imported: Optional[List[tuple]] = None):
        if not 1 <= len(bases) <= N.MAX_SHARDS:
            raise ValueError(f"1..{N.MAX_SHARDS} shards supported, got {len(bases)}")
        self.bases = [int(b) for b in bases]
        self.pages_per_shard = int(pages_per_shard)
        self.geom = geom
        self.rule = int(rule)
        self.device = device
        self._keepalive = keepalive or []
        self._imported = imported or []
        self.desc = N.PoolDesc()
        for i, b in enumerate(self.bases):
            self.desc.shard_base[i] = b
        self.desc.n_shards = len(self.bases)
        self.desc.shard_rule = self.rule
        self.desc.pages_per_shard = self.pages_per_shard

    @property
    def n_shards(self) -> int:
        return len(self.bases)

    @property
    def total_pages(self) -> int:
        return self.n_shards * self.pages_per_shard

    # -- constructors ------------------------------------------------------
    @staticmethod
    def allocate_shard(geom: KVGeometry, n_pages: int, device) -> torch.Tensor:
        """One shard's pool tensor in ``geom``'s pool layout (uninitialised)."""
        return torch.empty(geom.pool_shape(n_pages), dtype=geom.dtype, device=device)

    @classmethod
    def from_tensors(cls, shards: Sequence[torch.Tensor], geom: KVGeometry,
                     rule: int = N.SHARD_MOD, device=None) -> "ShardedPool":
        """In-process pool: one tensor per shard, possibly on different GPUs.  Peer
        access from ``device`` (default: shard 0's device) to every other shard's GPU
        is enabled here; failure raises."""
        shards = list(shards)
        dev = torch.device(device) if device is not None else shards[0].device
        per = {t.numel() * t.element_size() // geom.page_bytes for t in shards}
        if len(per) != 1:
            raise ValueError("all shards must hold the same number of pages")
        for t in shards:
            if not t.is_contiguous():
                raise ValueError("shard tensors must be contiguous")
            if t.device != dev:
                N.check(N.lib().bikv_enable_peer(dev.index or 0, t.device.index or 0), "bikv_enable_peer")
        return cls([t.data_ptr() for t in shards], per.pop(), geom, rule, dev, keepalive=shards)

    @classmethod
    def single(cls, shard: torch.Tensor, geom: KVGeometry) -> "ShardedPool":
        return cls.from_tensors([shard], geom)

    # -- cross-process -----------------------------------------------------
    @staticmethod
    def export_handle(shard: torch.Tensor) -> tuple:
        """(64-byte IPC handle, offset) for a shard tensor of this process."""
        h = C.create_string_buffer(64)
        off = C.c_int64(0)
        N.check(N.lib().bikv_pool_export(C.c_void_p(shard.data_ptr()), h, C.byref(off)), "bikv_pool_export")
        return bytes(h.raw), int(off.value)

    @classmethod
    def from_handles(cls, handles: Sequence[Optional[tuple]], own_rank: int, own_shard: torch.Tensor,
                     geom: KVGeometry, rule: int = N.SHARD_MOD, importer=None) -> "ShardedPool":
        """Pool whose shard ``own_rank`` is this process's tensor and whose other shards
        are opened from ``handles[r] = (handle bytes, offset)``.  ``importer`` replaces
        the CUDA IPC open (used by CPU tests)."""
        bases, imported = [], []
        for r, h in enumerate(handles):
            if r == own_rank:
                bases.append(own_shard.data_ptr())
                continue
            if importer is not None:
                bases.append(int(importer(r, h)))
                continue
            out = C.c_void_p()
            N.check(N.lib().bikv_pool_import(h[0], int(h[1]), C.byref(out)), "bikv_pool_import")
            bases.append(int(out.value))
            imported.append((int(out.value), int(h[1])))
        per = own_shard.numel() * own_shard.element_size() // geom.page_bytes
        return cls(bases, per, geom, rule, own_shard.device, keepalive=[own_shard], imported=imported)

    @classmethod
    def exchange(cls, own_shard: torch.Tensor, geom: KVGeometry, group=None,
                 rule: int = N.SHARD_MOD, exporter=None, importer=None) -> "ShardedPool":
        """One process per GPU: every rank exports its shard, the handles travel by
        ``torch.distributed.all_gather_object`` (host side, any backend), every rank
        opens the others'.  No data-path collective is involved."""
        import torch.distributed as dist

        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        mine = (exporter or cls.export_handle)(own_shard)
        handles: list = [None] * world
        dist.all_gather_object(handles, mine, group=group)
        return cls.from_handles(handles, rank, own_shard, geom, rule, importer=importer)

    def close(self) -> None:
        """Unmaps the shards opened from IPC handles (entries are (mapped pointer, offset))."""
        imported, self._imported = self._imported, []
        for ptr, offset in imported:
            N.check(N.lib().bikv_pool_close(C.c_void_p(ptr), offset), "bikv_pool_close")
