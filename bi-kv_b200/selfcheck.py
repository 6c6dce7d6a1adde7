"""Closed-form contents for page pools and worker tensors, and checks against them.

A copy path is easy to get subtly wrong in ways a checksum cannot see: the right bytes in
the wrong page, plane or token.  Here every 32-bit word of a pool page holds a hash of
(global page id, word index inside the page) and every word of a worker tensor a hash of
(rank, request, word index inside the tensor).  What a gathered worker tensor or a scattered
pool page must then hold follows from the plan alone -- page lists and token counts, as the
reference's plan loops define them (``DistributedStorage/kvcache.py:161-174``; per valid
token as ``SharedMemory/CUDA_Shared/copy_kernel.cu:26-35`` copies) -- so every rank of a
multi-GPU run can check every word it received without holding the other ranks' data.

Everything is plain torch arithmetic on the tensors' own device (CPU or GPU); the copy
kernels are not involved.  Paged pool layout only: a page is one contiguous run of
``[layer][kv][page_token][head][dim]`` (a worker tensor is ``[layer][kv][token][head][dim]``).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple

import numpy as np
import torch

from . import _native as N
from .geometry import KVGeometry

_M = 0xFFFFFFFF


def _mix(a: torch.Tensor, b: torch.Tensor, salt: int) -> torch.Tensor:
    """32-bit avalanche hash of two non-negative int64 tensors (broadcast), as int64 in
    [0, 2^32).  Products may wrap int64; the low 32 bits that are kept do not depend on it."""
    x = (a * 0x9E3779B1 + (b & _M) * 0x85EBCA77 + salt) & _M
    x = x ^ (x >> 15)
    x = (x * 0x2C1B3C6D) & _M
    x = x ^ (x >> 12)
    x = (x * 0x297A2D39) & _M
    return x ^ (x >> 15)


def _as_i32(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x >= (1 << 31), x - (1 << 32), x).to(torch.int32)


def _require_paged(geom: KVGeometry) -> None:
    if geom.pool_layout != N.POOL_PAGED:
        raise ValueError("closed-form checks cover the paged pool layout only")
    if geom.row_elems * geom.elt_bytes % 4:
        raise ValueError("rows must be a multiple of 4 bytes")


def _words(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1).view(torch.int32)


POOL_SALT, WORKER_SALT = 0x165667B1, 0x27D4EB2F


def page_words(geom: KVGeometry) -> int:
    return geom.page_bytes // 4


def global_ids_of_shard(shard_index: int, n_shards: int, pages_per_shard: int, rule: int = N.SHARD_MOD) -> np.ndarray:
    local = np.arange(pages_per_shard, dtype=np.int64)
    return local * n_shards + shard_index if rule == N.SHARD_MOD else shard_index * pages_per_shard + local


def fill_pool_(shard: torch.Tensor, geom: KVGeometry, global_ids: np.ndarray, chunk_pages: int = 0) -> None:
    """Word w of the page with global id g becomes mix(g, w)."""
    _require_paged(geom)
    pw = page_words(geom)
    view = _words(shard).view(-1, pw)
    chunk = chunk_pages or max(1, (1 << 25) // pw)
    w = torch.arange(pw, dtype=torch.int64, device=shard.device)[None, :]
    for at in range(0, view.shape[0], chunk):
        ids = torch.from_numpy(np.ascontiguousarray(global_ids[at:at + chunk])).to(shard.device)[:, None]
        view[at:at + chunk] = _as_i32(_mix(ids, w, POOL_SALT))


def token_map(page_list: Sequence[int], tokens: int, page_tokens: int) -> Tuple[np.ndarray, np.ndarray]:
    """(page id, token inside the page) of every token of a request whose pages are
    ``page_list`` in order -- the running-offset walk of the reference's plan loop with one
    item per request."""
    t = np.arange(int(tokens), dtype=np.int64)
    pages = np.asarray(page_list, dtype=np.int64)
    return pages[t // page_tokens], t % page_tokens


def expected_gathered(geom: KVGeometry, page_of_token: np.ndarray, token_in_page: np.ndarray, device) -> torch.Tensor:
    """int32 words ``[planes, tokens, row_words]`` of a worker tensor gathered out of a pool
    filled by :func:`fill_pool_`."""
    _require_paged(geom)
    rw = geom.row_elems * geom.elt_bytes // 4
    plane_words = rw * geom.page_tokens
    page = torch.from_numpy(page_of_token).to(device)[None, :, None]
    tip = torch.from_numpy(token_in_page).to(device)[None, :, None]
    plane = torch.arange(geom.planes, dtype=torch.int64, device=device)[:, None, None]
    roww = torch.arange(rw, dtype=torch.int64, device=device)[None, None, :]
    return _as_i32(_mix(page, plane * plane_words + tip * rw + roww, POOL_SALT))


def check_gathered(geom: KVGeometry, tensor: torch.Tensor, page_list: Sequence[int], tokens: int,
                   max_tokens_per_pass: int = 2048) -> bool:
    """Every word of ``tensor`` (``geom.worker_shape(tokens)``) equals what the plan says it
    must be, given a pool filled by :func:`fill_pool_`."""
    rw = geom.row_elems * geom.elt_bytes // 4
    got = _words(tensor).view(geom.planes, int(tokens), rw)
    page, tip = token_map(page_list, tokens, geom.page_tokens)
    for at in range(0, int(tokens), max_tokens_per_pass):
        want = expected_gathered(geom, page[at:at + max_tokens_per_pass], tip[at:at + max_tokens_per_pass], tensor.device)
        if not torch.equal(got[:, at:at + max_tokens_per_pass], want):
            return False
    return True


def worker_words(geom: KVGeometry, rank: int, request: int, tokens: int, token_at: int, n: int, device) -> torch.Tensor:
    """int32 words ``[planes, n, row_words]`` of tokens ``token_at .. token_at+n`` of the
    worker tensor (rank, request) under the second closed form."""
    rw = geom.row_elems * geom.elt_bytes // 4
    plane = torch.arange(geom.planes, dtype=torch.int64, device=device)[:, None, None]
    tok = torch.arange(token_at, token_at + n, dtype=torch.int64, device=device)[None, :, None]
    roww = torch.arange(rw, dtype=torch.int64, device=device)[None, None, :]
    key = torch.tensor((int(rank) << 20) | int(request), dtype=torch.int64, device=device)
    return _as_i32(_mix(key, (plane * int(tokens) + tok) * rw + roww, WORKER_SALT))


def fill_worker_(geom: KVGeometry, tensor: torch.Tensor, rank: int, request: int, max_tokens_per_pass: int = 2048) -> None:
    _require_paged(geom)
    tokens = tensor.shape[2]
    rw = geom.row_elems * geom.elt_bytes // 4
    view = _words(tensor).view(geom.planes, tokens, rw)
    for at in range(0, tokens, max_tokens_per_pass):
        n = min(max_tokens_per_pass, tokens - at)
        view[:, at:at + n] = worker_words(geom, rank, request, tokens, at, n, tensor.device)


def touched_pages(workloads: Iterable, shard_index: int, n_shards: int, pages_per_shard: int,
                  rule: int = N.SHARD_MOD) -> np.ndarray:
    """Rows (local page, rank, request, token offset, valid tokens, request tokens) for every
    page of ``workloads[rank]`` (objects with ``page_lists`` and ``request_tokens``, one item
    per request) that lives on shard ``shard_index``."""
    rows: List[np.ndarray] = []
    for rank, w in enumerate(workloads):
        pt = w.geom.page_tokens
        for req, (pages, tokens) in enumerate(zip(w.page_lists, w.request_tokens)):
            pages = np.asarray(pages, dtype=np.int64)
            k = np.arange(len(pages), dtype=np.int64)
            valid = np.minimum(pt, int(tokens) - k * pt)
            if rule == N.SHARD_MOD:
                shard, local = pages % n_shards, pages // n_shards
            else:
                shard, local = pages // pages_per_shard, pages % pages_per_shard
            m = shard == shard_index
            if m.any():
                n = int(m.sum())
                rows.append(np.stack([local[m], np.full(n, rank), np.full(n, req), k[m] * pt, valid[m],
                                      np.full(n, int(tokens))], axis=1))
    return np.concatenate(rows).astype(np.int64) if rows else np.zeros((0, 6), dtype=np.int64)


def check_scattered_pool(shard: torch.Tensor, geom: KVGeometry, global_ids: np.ndarray, touched: np.ndarray,
                         chunk_pages: int = 0) -> bool:
    """The shard was filled by :func:`fill_pool_`; then worker tensors filled by
    :func:`fill_worker_` were scattered into the pages of ``touched``
    (:func:`touched_pages`).  True when every word of the shard is what that implies: the
    valid tokens of touched pages hold the workers' words, everything else -- untouched pages
    and the rows past ``valid`` of a partial page -- still holds the first form."""
    _require_paged(geom)
    pw = page_words(geom)
    rw = geom.row_elems * geom.elt_bytes // 4
    pt = geom.page_tokens
    dev = shard.device
    view = _words(shard).view(-1, pw)
    chunk = chunk_pages or max(1, (1 << 25) // pw)
    order = np.argsort(touched[:, 0], kind="stable")
    touched = touched[order]
    if len(touched) and (np.diff(touched[:, 0]) == 0).any():
        raise ValueError("a pool page is scattered to twice")
    w = torch.arange(pw, dtype=torch.int64, device=dev)[None, :]
    plane = torch.arange(geom.planes, dtype=torch.int64, device=dev)[None, :, None, None]
    tip = torch.arange(pt, dtype=torch.int64, device=dev)[None, None, :, None]
    roww = torch.arange(rw, dtype=torch.int64, device=dev)[None, None, None, :]
    for at in range(0, view.shape[0], chunk):
        n = min(chunk, view.shape[0] - at)
        ids = torch.from_numpy(np.ascontiguousarray(global_ids[at:at + n])).to(dev)[:, None]
        want = _as_i32(_mix(ids, w, POOL_SALT)).view(n, geom.planes, pt, rw)
        lo, hi = np.searchsorted(touched[:, 0], [at, at + n])
        if hi > lo:
            rows = torch.from_numpy(np.ascontiguousarray(touched[lo:hi])).to(dev)
            col = lambda i: rows[:, i][:, None, None, None]      # noqa: E731
            key = (col(1) << 20) | col(2)
            idx = (plane * col(5) + col(3) + tip) * rw + roww
            form2 = _as_i32(_mix(key, idx, WORKER_SALT))
            keep = tip < col(4)
            sel = rows[:, 0] - at
            want[sel] = torch.where(keep, form2, want[sel])
        if not torch.equal(view[at:at + n].view(n, geom.planes, pt, rw), want):
            return False
    return True


def position_hash(t: torch.Tensor, chunk_words: int = 1 << 26) -> int:
    """64-bit hash of a tensor's bits in which every 32-bit word is weighted by an odd
    function of its position (wrapping int64 arithmetic), so words that move change it."""
    words = _words(t)
    total = torch.zeros((), dtype=torch.int64, device=t.device)
    for at in range(0, words.numel(), chunk_words):
        part = words[at:at + chunk_words].to(torch.int64) & _M
        pos = torch.arange(at, at + part.numel(), dtype=torch.int64, device=t.device)
        weight = _mix(pos & _M, pos >> 32, 0x51ED270B) | 1
        total += (part * weight + (part ^ weight)).sum()
    return int(total)
