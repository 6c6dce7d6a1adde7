"""Seeded synthetic workloads with the shapes of the benchmark configurations.

No dataset is involved: request lengths and page ids are drawn from fixed-seed
generators, pool contents are N(0,1) cast to the configuration's dtype.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

import numpy as np
import torch

from . import _native as N
from .geometry import GEO_A, GEO_B, GEO_C, KVGeometry
from .plan import Plan, build_plan


@dataclass
class Workload:
    name: str
    geom: KVGeometry
    n_shards: int
    pages_per_shard: int
    request_tokens: np.ndarray            # int64 [n_requests]
    page_lists: List[np.ndarray]          # global page ids per request
    rule: int = N.SHARD_MOD
    notes: dict = field(default_factory=dict)

    @property
    def n_requests(self) -> int:
        return len(self.request_tokens)

    @property
    def n_pages(self) -> int:
        return int(sum(len(p) for p in self.page_lists))

    @property
    def total_tokens(self) -> int:
        return int(self.request_tokens.sum())

    @property
    def payload_bytes(self) -> int:
        """Bytes of valid tokens: what one gather (or one scatter) moves."""
        return self.total_tokens * self.geom.bytes_per_token

    def flat(self):
        lens = np.fromiter((len(p) for p in self.page_lists), dtype=np.int64, count=self.n_requests)
        begin = np.zeros(self.n_requests + 1, dtype=np.int64)
        np.cumsum(lens, out=begin[1:])
        flat = np.concatenate(self.page_lists).astype(np.int32) if self.n_requests else np.zeros(0, np.int32)
        return flat, begin

    def plan(self) -> Plan:
        """One worker tensor per request."""
        return build_plan(self.flat(), self.request_tokens.astype(np.int32), self.geom.page_tokens,
                          item_request=np.arange(self.n_requests, dtype=np.int32),
                          n_requests=self.n_requests)

    def remote_fraction(self, own_shard: int) -> float:
        ids = np.concatenate(self.page_lists)
        if self.rule == N.SHARD_MOD:
            shard = ids % self.n_shards
        else:
            shard = ids // self.pages_per_shard
        return float((shard != own_shard).mean())


def _pages_without_replacement(rng: np.random.Generator, total_pages: int, counts: np.ndarray):
    need = int(counts.sum())
    if need > total_pages:
        raise ValueError(f"workload needs {need} pages, pool has {total_pages}")
    perm = rng.permutation(total_pages)[:need].astype(np.int32)
    out, at = [], 0
    for c in counts:
        out.append(perm[at:at + int(c)])
        at += int(c)
    return out


def lognormal_lengths(rng, n, median, sigma, lo, hi) -> np.ndarray:
    x = rng.lognormal(mean=np.log(median), sigma=sigma, size=n)
    return np.clip(np.rint(x), lo, hi).astype(np.int64)


def config0(seed: int = 0, n_pages: int = 4096, n_requests: int = 32) -> Workload:
    """CPU-sized case: geometry A, 4096-page pool, 32 requests U[128,1024]."""
    rng = np.random.default_rng(seed)
    tokens = rng.integers(128, 1025, size=n_requests).astype(np.int64)
    counts = (tokens + GEO_A.page_tokens - 1) // GEO_A.page_tokens
    return Workload("config0", GEO_A, 1, n_pages, tokens, _pages_without_replacement(rng, n_pages, counts))


def config1(seed: int = 0, n_pages: int = 65536, n_requests: int = 64, geom: KVGeometry = GEO_B) -> Workload:
    """1 GPU: geometry B, 65,536-page pool, 64 requests lognormal(2048, 0.8) in [64, 8192]."""
    rng = np.random.default_rng(seed)
    tokens = lognormal_lengths(rng, n_requests, 2048, 0.8, 64, 8192)
    counts = (tokens + geom.page_tokens - 1) // geom.page_tokens
    return Workload("config1", geom, 1, n_pages, tokens, _pages_without_replacement(rng, n_pages, counts))


def config2(rank: int, world: int, seed: int = 0, pages_per_shard: int = 65536, n_requests: int = 64,
            geom: KVGeometry = GEO_B, pages_from: str = "all") -> Workload:
    """``world`` GPUs, pool striped by ``page_id mod world``; this rank's 64 requests draw
    pages uniformly over all shards.  Ranks draw from disjoint slices of one global
    permutation, so concurrent scatters never share a page."""
    rng = np.random.default_rng(seed)
    total = pages_per_shard * world
    perm = rng.permutation(total).astype(np.int32)
    share = total // world
    mine = perm[rank * share:(rank + 1) * share]
    if pages_from == "remote":      # side measurement: only pages of other shards
        mine = mine[mine % world != rank]
    elif pages_from == "local":
        mine = mine[mine % world == rank]
    share = len(mine)
    rrng = np.random.default_rng([seed, rank])
    tokens = lognormal_lengths(rrng, n_requests, 2048, 0.8, 64, 8192)
    counts = (tokens + geom.page_tokens - 1) // geom.page_tokens
    need = int(counts.sum())
    if need > share:
        raise ValueError("per-rank slice of the pool too small for this workload")
    lists, at = [], 0
    for c in counts:
        lists.append(mine[at:at + int(c)])
        at += int(c)
    return Workload(f"config2/{world}", geom, world, pages_per_shard, tokens, lists)


def config3(rank: int, world: int, seed: int = 0, pages_per_shard: int = 8192, n_requests: int = 16,
            geom: KVGeometry = GEO_C, lo: int = 16384, hi: int = 32768) -> List[Workload]:
    """Long context: geometry C, requests U[16k,32k] tokens.  One request is up to 2,048
    pages (10 GiB), so requests are STREAMED: the result is one single-request workload
    per request.  Page ids are unique inside a request; across requests of a rank they
    may repeat, and ranks use disjoint slices of the pool."""
    total = pages_per_shard * world
    share = total // world
    base = np.random.default_rng(seed).permutation(total).astype(np.int32)[rank * share:(rank + 1) * share]
    out = []
    for r in range(n_requests):
        rng = np.random.default_rng([seed, rank, r])
        tokens = rng.integers(lo, hi + 1, size=1).astype(np.int64)
        count = int((tokens[0] + geom.page_tokens - 1) // geom.page_tokens)
        if count > share:
            raise ValueError("request larger than this rank's slice of the pool")
        pages = rng.permutation(base)[:count]
        out.append(Workload(f"config3/{world}/r{r}", geom, world, pages_per_shard, tokens, [pages]))
    return out


def fill_normal_(t: torch.Tensor, seed: int, chunk_elems: int = 1 << 28) -> torch.Tensor:
    """Fills a (large) tensor with N(0,1) values chunk by chunk from a fixed seed, on the
    tensor's own device."""
    g = torch.Generator(device=t.device)
    g.manual_seed(seed)
    flat = t.view(-1)
    for at in range(0, flat.numel(), chunk_elems):
        part = flat[at:at + chunk_elems]
        part.copy_(torch.randn(part.numel(), generator=g, device=t.device, dtype=torch.float32))
    return t
