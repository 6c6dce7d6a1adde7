"""Prefix-reuse workload (configuration 4): host-side invariants on CPU, and on a GPU the
gathered prefixes of sampled requests bit-exact against a shadow copy of what was stored."""
import numpy as np
import pytest
import torch

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200.coordinator import PrefixCacheCoordinator, PrefixReuseWorkload
from bikv_b200.geometry import KVGeometry

from helpers import equal_bits


def test_workload_is_seeded_and_shaped():
    a, b = PrefixReuseWorkload(seed=3, n_users=5000, n_requests=2000), PrefixReuseWorkload(seed=3, n_users=5000, n_requests=2000)
    assert (a.users == b.users).all() and (a.new == b.new).all()
    assert a.prefix_of_user.min() >= 128 and a.prefix_of_user.max() <= 8192
    assert a.new.min() >= 32 and a.new.max() <= 256
    counts = np.bincount(a.users, minlength=5000)
    assert counts[0] == counts.max() and counts[:10].sum() > counts[1000:1010].sum() * 5   # Zipf head
    batches = list(a.batches())
    assert len(batches) == 32 and len(batches[0]) == 64 and len(batches[-1]) == 2000 - 31 * 64
    assert [r.worker for r in batches[0][:5]] == [0, 1, 2, 3, 0]


@pytest.mark.parametrize("order", ["reference", "fast"])
def test_coordinator_invariants(native, order):
    wl = PrefixReuseWorkload(seed=1, n_users=400, n_requests=1500, batch=32, n_workers=1,
                             prefix_median=300, prefix_clip=(64, 1024))
    co = PrefixCacheCoordinator(n_shards=3, pages_per_shard=512, page_tokens=16, order=order, seed=0)
    stored = {}                       # global page id -> (user or new item) as of the last scatter
    for batch in wl.batches():
        bp = co.plan_batch(batch)
        assert N.lib().bikv_plan_validate is not None
        g, s = bp.gather.table, bp.scatter.table
        assert len(set(s[:, 0].tolist())) == len(s), "a page is written twice in one batch"
        assert (s[:, 0] < 3 * 512).all() and (g[:, 0] < 3 * 512).all()
        for i, r in enumerate(batch):
            gt = g[g[:, 2] == i]
            st = s[s[:, 2] == i]
            if bp.hit[i]:
                assert gt[:, 1].sum() == r.prefix_tokens and st[:, 1].sum() == r.new_tokens
                assert gt[0, 3] == 0 and st[0, 3] == r.prefix_tokens
                for page in gt[:, 0]:
                    assert stored[int(page)] == r.user, "hit reads a page that holds someone else's data"
            elif st[0, 3] == 0:
                assert len(gt) == 0 and st[:, 1].sum() == r.tokens
            else:       # same user missed earlier in this batch: prefix neither read nor stored twice
                assert len(gt) == 0 and st[:, 1].sum() == r.new_tokens and st[0, 3] == r.prefix_tokens
                assert any(q.user == r.user and not bp.hit[k] for k, q in enumerate(batch[:i]))
            ends = st[:, 3] + st[:, 1]
            assert ends.max() == r.tokens
        # gathers run before scatters, so bookkeeping of page owners updates afterwards
        for i, r in enumerate(batch):
            st = s[s[:, 2] == i]
            off = 0
            for page, valid, _, tok in st.tolist():
                stored[page] = r.user if tok < r.prefix_tokens and not bp.hit[i] else ("new", r.request_id)
    assert 0.2 < co.hit_rate < 0.95
    assert co.hits + co.misses == 1500


def test_reference_and_fast_order_agree_on_hits(native):
    wl = PrefixReuseWorkload(seed=2, n_users=300, n_requests=800, batch=16, n_workers=1,
                             prefix_median=200, prefix_clip=(64, 512))
    rates = []
    for order in ("reference", "fast"):
        co = PrefixCacheCoordinator(2, 1024, 16, order=order, seed=5)
        hits = [co.plan_batch(b).hit for b in wl.batches()]
        rates.append(hits)
    assert rates[0] == rates[1], "eviction decisions do not depend on page numbering"


@pytest.mark.gpu
def test_prefix_reuse_on_gpu_sampled_bit_exact(cuda):
    """4 shards and 2 workers on one GPU, small pool so that eviction is constant.  Every
    request's tensor is filled with seeded data; hits must gather back exactly the bits that
    the miss which stored them scattered."""
    geom = KVGeometry(2, 2, 64, 16, torch.bfloat16)
    n_shards, per = 4, 96
    shards = [torch.zeros(geom.pool_shape(per), dtype=geom.dtype, device=cuda) for _ in range(n_shards)]
    pool = B.ShardedPool.from_tensors(shards, geom, rule=N.SHARD_BLOCK)
    mover = B.PageMover(cuda)
    wl = PrefixReuseWorkload(seed=4, n_users=60, n_requests=600, batch=8, n_workers=1,
                             prefix_median=150, prefix_clip=(32, 400), new_tokens=(8, 40))
    co = PrefixCacheCoordinator(n_shards, per, 16, seed=1)
    shadow, checked = {}, 0

    def prefix_data(user, tokens):
        g = torch.Generator().manual_seed(1000 + user)
        return torch.randn(geom.worker_shape(tokens), generator=g).to(geom.dtype)

    for batch in wl.batches():
        bp = co.plan_batch(batch)
        tensors = []
        for i, r in enumerate(batch):
            t = torch.zeros(geom.worker_shape(r.tokens), dtype=geom.dtype, device=cuda)
            if not bp.hit[i]:
                shadow[r.user] = prefix_data(r.user, r.prefix_tokens)
                t[:, :, :r.prefix_tokens] = shadow[r.user].to(cuda)
            t[:, :, r.prefix_tokens:] = 1.0 + (r.request_id % 7)
            tensors.append(t)
        mover.gather(pool, bp.gather, tensors)           # all gathers before any scatter
        mover.scatter(pool, bp.scatter, tensors)
        torch.cuda.synchronize()
        for i, r in enumerate(batch):
            if bp.hit[i]:
                assert equal_bits(tensors[i][:, :, :r.prefix_tokens], shadow[r.user]), f"request {r.request_id}"
                checked += 1
    mover.check_status()
    assert checked > 100 and co.misses > 60, (checked, co.misses)     # evictions forced re-misses


@pytest.mark.parametrize("native_planner", [False, True])
def test_whole_batch_plan_split_by_worker(native, native_planner):
    """A batch planned in one piece and split by worker: the split plans together are the whole
    plan, and a user named by requests of two workers in ONE batch is stored once and not read
    by the other request (its pages are written only when the batch's scatters run)."""
    from bikv_b200.coordinator import NativePrefixCacheCoordinator, Request, split_by_worker
    co = (NativePrefixCacheCoordinator(2, 256, 16) if native_planner
          else PrefixCacheCoordinator(2, 256, 16, order="fast"))
    batch = [Request(0, 7, 100, 40, 0), Request(1, 9, 50, 33, 1), Request(2, 7, 100, 20, 1),     # user 7 twice
             Request(3, 5, 64, 32, 0), Request(4, 9, 50, 48, 0)]                                 # user 9 twice
    bp = co.plan_batch(batch)
    assert bp.hit == [False] * 5
    parts = split_by_worker(bp, 2)
    assert [len(p.requests) for p in parts] == [3, 2]
    assert [r.request_id for r in parts[0].requests] == [0, 3, 4] and [r.request_id for r in parts[1].requests] == [1, 2]
    assert sum(p.gather.n_pages for p in parts) == bp.gather.n_pages == 0
    assert sum(p.scatter.n_pages for p in parts) == bp.scatter.n_pages
    whole = sorted(map(tuple, bp.scatter.table[:, [0, 1, 3]].tolist()))
    assert sorted(t for p in parts for t in map(tuple, p.scatter.table[:, [0, 1, 3]].tolist())) == whole
    # worker 1's second request (user 7, stored by worker 0 in this batch) stores only its new tokens
    s1 = parts[1].scatter.table
    second = s1[s1[:, 2] == 1]
    assert second[:, 1].sum() == 20 and second[0, 3] == 100
    # the next batch finds both users: hits, gathered by whichever worker asks
    nxt = [Request(5, 7, 100, 10, 1), Request(6, 9, 50, 10, 0)]
    bp2 = co.plan_batch(nxt)
    assert bp2.hit == [True, True]
    parts2 = split_by_worker(bp2, 2)
    assert parts2[1].gather.table[:, 1].sum() == 100 and parts2[0].gather.table[:, 1].sum() == 50
    assert set(parts2[1].gather.table[:, 2].tolist()) == {0} and set(parts2[0].gather.table[:, 2].tolist()) == {0}


def test_split_by_worker_keeps_row_order_and_splits_row_flags(native):
    """Against a row-by-row restatement: rows of a worker keep the batch plan's order, requests
    are renumbered per worker, and a per-row flag array travels with its rows."""
    from bikv_b200.coordinator import NativePrefixCacheCoordinator, PrefixReuseWorkload, split_by_worker
    n_workers = 3
    co = NativePrefixCacheCoordinator(2, 4096, 16)
    wl = PrefixReuseWorkload(seed=3, n_users=50, n_workers=n_workers, n_requests=256, batch=64)
    for batch in wl.batches():
        bp = co.plan_batch(batch)
        flags = (bp.gather.table[:, 0] % 3 == 0)
        parts, part_flags = split_by_worker(bp, n_workers, gather_flags=flags)
        local, seen = {}, [0] * n_workers
        for i, r in enumerate(batch):
            local[i] = seen[r.worker]
            seen[r.worker] += 1
        for k in range(n_workers):
            assert [r.request_id for r in parts[k].requests] == [r.request_id for r in batch if r.worker == k]
            for plan, part in ((bp.gather, parts[k].gather), (bp.scatter, parts[k].scatter)):
                want = [[p, v, local[q], o] for p, v, q, o in plan.table.tolist() if batch[q].worker == k]
                assert part.table.tolist() == want
            want_flags = [bool(f) for f, row in zip(flags, bp.gather.table.tolist()) if batch[row[2]].worker == k]
            assert part_flags[k].tolist() == want_flags
        assert split_by_worker(bp, n_workers)[0].gather.table.tolist() == parts[0].gather.table.tolist()


def test_plan_stream_marks_gather_rows_that_read_what_the_batch_before_writes(native):
    """The late flags of batch k+1 are exactly the gather rows whose page batch k scatters into,
    for the striped (one directory) and the item-per-shard placement alike."""
    from bikv_b200.coordinator import NativePrefixCacheCoordinator, PrefixReuseWorkload, plan_stream
    for dirs, pages in ((1, 65536), (2, 32768)):
        co = NativePrefixCacheCoordinator(dirs, pages, 16, transient_plans=True)
        wl = PrefixReuseWorkload(seed=5, n_users=40, n_workers=2, n_requests=640, batch=64)
        prev_pages, n_late, n_steps = set(), 0, 0
        for plans, late, any_late in plan_stream(wl.batches(), co, 2, dirs * pages, transient=True):
            want_any = False
            for p, m in zip(plans, late):
                want = [int(pg) in prev_pages for pg in p.gather.table[:, 0]]
                assert m.tolist() == want
                want_any |= any(want)
            assert any_late == want_any
            n_late += any_late
            n_steps += 1
            prev_pages = set(int(pg) for p in plans for pg in p.scatter.table[:, 0])
        assert n_steps == 10 and n_late > 0          # 40 users: repeats across neighbouring batches are certain
