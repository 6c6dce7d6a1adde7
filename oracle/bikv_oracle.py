"""CPU oracle for the KV-page gather/scatter path.  TEST INFRASTRUCTURE ONLY.

This file restates, with plain torch-CPU slicing and Python loops, what the
reference's path computes.  Only tests, the smoke check and the benchmark's
CPU-baseline leg may import it; nothing in the product imports it, and the
product has no CPU path of its own.

Parity status.  The reference holds no golden vectors for this path: its only
functional checks are "constant 7 in, constant 7 out, 5-D shape kept" on an
identity page map (``SharedMemory/CUDA_Shared/test_page_ipc.py:127-150``,
``test_zero_copy.py:86-103``).  Those two checks are reproduced in the test
suite.  Beyond them the oracle is pinned by
  * index arrays captured from the reference's own plan loop
    (``KVCache.shared_data_batch_pages``, run here with stubs; fixtures under
    ``tests/golden/``), which pin :func:`plan_records`;
  * the reference's CUDA kernel itself, compiled from its sources into
    ``oracle/_ref/`` and run on the GPU against :func:`copy_pages_flat`.
Layout conversion, partial last pages, scatter and multi-shard addressing do not
exist in the reference; for those, parity is pinned by this oracle alone.

One deliberate deviation: the reference's kernel always copies a whole page
while its plan advances the destination by the number of valid tokens, so the
tail of a short page overlaps the next item's first page and two thread blocks
race on it (``kvcache.py:165-174`` against ``copy_kernel.cu:26-35``).  The
layout-converting gather/scatter here move only the valid tokens of a page.
:func:`copy_pages_flat` keeps the kernel's whole-page semantics.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

POOL_PAGED = 0
POOL_TOKEN_MAJOR = 1
SHARD_MOD = 0
SHARD_BLOCK = 1

Rec = Tuple[int, int, int, int]  # page_id, valid_tokens, request, token_offset


# --------------------------------------------------------------------------
# Plan: follows DistributedStorage/kvcache.py:158-174 (page_indices /
# page_offsets loops), with the running offset kept per destination tensor.
# --------------------------------------------------------------------------
def plan_records(cache_pages_list: Sequence[Sequence[int]], item_tokens: Sequence[int], page_tokens: int,
                 item_request: Optional[Sequence[int]] = None, item_shard: Optional[Sequence[int]] = None,
                 pages_per_shard: int = 0) -> List[Rec]:
    recs: List[Rec] = []
    offsets: dict = {}
    for idx, page_list in enumerate(cache_pages_list):
        tokens = item_tokens[idx]
        req = 0 if item_request is None else item_request[idx]
        cur = offsets.get(req, 0)
        for page_idx, page in enumerate(page_list):
            # kvcache.py:169-170: only the item's last page is short, and only
            # when the token count is not a multiple of the page size.
            last = page_idx == len(page_list) - 1
            size = (tokens % page_tokens) if (last and tokens % page_tokens != 0) else page_tokens
            gid = page if item_shard is None else item_shard[idx] * pages_per_shard + page
            recs.append((gid, size, req, cur))
            cur += size
        offsets[req] = cur
    return recs


def reference_offsets(cache_pages_list, item_tokens, page_size):
    """The two arrays the reference uploads (kvcache.py:187-196): ``src_offsets`` =
    page * page_size and ``dest_offsets`` = running token offset, both in tokens."""
    recs = plan_records(cache_pages_list, item_tokens, page_size)
    return [r[0] * page_size for r in recs], [r[3] for r in recs]


# --------------------------------------------------------------------------
# Addressing
# --------------------------------------------------------------------------
def locate(page_id: int, n_shards: int, pages_per_shard: int, rule: int) -> Tuple[int, int]:
    if rule == SHARD_MOD:
        return page_id % n_shards, page_id // n_shards
    return page_id // pages_per_shard, page_id % pages_per_shard


def _page_view(shards, geom, page_id, rule):
    """The page as a [L, 2, P, H, D] view, whatever the pool layout."""
    L, H, D, P = geom.n_layers, geom.n_kv_heads, geom.head_dim, geom.page_tokens
    n_shards = len(shards)
    per = shards[0].numel() // (P * 2 * L * H * D)
    s, local = locate(page_id, n_shards, per, rule)
    if geom.pool_layout == POOL_PAGED:
        return shards[s].view(per, L, 2, P, H, D)[local]
    # token-major: [token, D, H, L, 2] (kvcache.py:38-43, qwen2.py:519-522)
    tok = shards[s].view(per * P, D, H, L, 2)[local * P:(local + 1) * P]
    return tok.permute(3, 4, 0, 2, 1)  # -> [L, 2, P, H, D]


# --------------------------------------------------------------------------
# Gather / scatter with layout conversion to [L, 2, T, H, D]
# (copy semantics of copy_kernel.cu:10-36 applied per valid token)
# --------------------------------------------------------------------------
def gather(shards: Sequence[torch.Tensor], geom, recs: Sequence[Rec], workers: Sequence[torch.Tensor],
           rule: int = SHARD_MOD) -> None:
    for page_id, valid, req, off in recs:
        page = _page_view(shards, geom, int(page_id), rule)
        workers[int(req)][:, :, off:off + valid] = page[:, :, :valid]


def scatter(shards: Sequence[torch.Tensor], geom, recs: Sequence[Rec], workers: Sequence[torch.Tensor],
            rule: int = SHARD_MOD) -> None:
    for page_id, valid, req, off in recs:
        page = _page_view(shards, geom, int(page_id), rule)
        page[:, :, :valid] = workers[int(req)][:, :, off:off + valid]


# --------------------------------------------------------------------------
# Paged worker KV: one [slot, kv, head, dim] tensor per layer (Worker.py:68-78).
# Record (page, valid, -, slot): token t of the page <-> slot + t of every layer.
# --------------------------------------------------------------------------
def gather_nhd(shards, geom, recs, layers, rule: int = SHARD_MOD) -> None:
    for page_id, valid, _, slot in recs:
        page = _page_view(shards, geom, int(page_id), rule)            # [L, 2, P, H, D]
        for l in range(geom.n_layers):
            layers[l][slot:slot + valid] = page[l, :, :valid].permute(1, 0, 2, 3)


def scatter_nhd(shards, geom, recs, layers, rule: int = SHARD_MOD) -> None:
    for page_id, valid, _, slot in recs:
        page = _page_view(shards, geom, int(page_id), rule)
        for l in range(geom.n_layers):
            page[l, :, :valid] = layers[l][slot:slot + valid].permute(1, 0, 2, 3)


# --------------------------------------------------------------------------
# Flat page copy: copy_kernel.cu:10-36 verbatim in meaning (element offsets,
# whole pages, pages applied in index order).
# --------------------------------------------------------------------------
def copy_pages_flat(src: torch.Tensor, dst: torch.Tensor, src_off: Sequence[int], dst_off: Sequence[int],
                    page_elems: int) -> None:
    s, d = src.reshape(-1), dst.reshape(-1)
    for so, do in zip(src_off, dst_off):
        d[do:do + page_elems] = s[so:so + page_elems]


# --------------------------------------------------------------------------
# The reference's CPU data path, as it would run with its commented lines live:
# pool and worker buffer are CPU tensors of token rows
# (kvcache.py:38-43, Worker.py:57-62) and the copy is torch advanced indexing
# over token indices (Worker.py:207: send_tensor[send_indices] =
# compute_buffer[buffer_indices]).  Used as the timed CPU baseline.
# --------------------------------------------------------------------------
def token_indices(recs: Sequence[Rec], page_tokens: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(pool token index, packed buffer token index) for every valid token; requests
    are packed one after another in request order."""
    recs = np.asarray(recs, dtype=np.int64).reshape(-1, 4)
    n_req = int(recs[:, 2].max()) + 1 if len(recs) else 0
    req_tokens = np.zeros(n_req, dtype=np.int64)
    np.maximum.at(req_tokens, recs[:, 2], recs[:, 1] + recs[:, 3])
    req_base = np.concatenate([[0], np.cumsum(req_tokens)[:-1]]) if n_req else np.zeros(0, np.int64)
    valid = recs[:, 1]
    within = np.arange(valid.sum()) - np.repeat(np.cumsum(valid) - valid, valid)
    src = np.repeat(recs[:, 0] * page_tokens, valid) + within
    dst = np.repeat(req_base[recs[:, 2]] + recs[:, 3], valid) + within
    return torch.from_numpy(src), torch.from_numpy(dst)


def cpu_gather_tokens(pool_tokens: torch.Tensor, buf: torch.Tensor, src_idx: torch.Tensor,
                      dst_idx: torch.Tensor) -> None:
    buf[dst_idx] = pool_tokens[src_idx]


def cpu_scatter_tokens(pool_tokens: torch.Tensor, buf: torch.Tensor, src_idx: torch.Tensor,
                       dst_idx: torch.Tensor) -> None:
    pool_tokens[src_idx] = buf[dst_idx]


def bits(t: torch.Tensor) -> torch.Tensor:
    """Integer view for bit-exact comparison (NaN-safe)."""
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[t.element_size()]
    return t.contiguous().view(view)
