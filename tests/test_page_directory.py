"""The native page directory against (a) the Python page managers in their 'fast' order
(which the golden fixtures tie to the reference) and (b) the restated Go semantics."""
import random

import pytest

from bikv_b200.coordinator import NativePrefixCacheCoordinator, PrefixCacheCoordinator, PrefixReuseWorkload
from bikv_b200.page_directory import PageDirectory, XorShiftChoice
from bikv_b200.page_manager import MultiPageManager
from oracle.go_page_manager import GoPageManagerOracle


@pytest.mark.parametrize("seed", range(6))
def test_lru_policy_equals_python_page_managers(native, seed):
    rnd = random.Random(seed)
    cache, page, k = rnd.choice([(256, 16, 2), (1024, 16, 4), (4000, 50, 3), (64, 4, 1)])
    py = MultiPageManager(cache, page, k, rng=XorShiftChoice(seed + 1), order="fast")
    nat = PageDirectory(cache, page, k, policy="lru", seed=seed + 1)
    protected = set()
    for step in range(1500):
        iid = rnd.randrange(80)
        x = rnd.random()
        if x < 0.55:
            ln = rnd.randint(1, cache // 3)
            if py.access_item(iid)[0] is not None:       # cached: both just touch it
                assert nat.access_item(iid) == py.access_item(iid)
                continue
            try:
                want = py.load_item(iid, ln)
            except (RuntimeError, ValueError) as e:
                with pytest.raises(type(e)):
                    nat.load_item(iid, ln)
                continue
            got = nat.load_item(iid, ln)
            assert got == (want[0], want[1]), step
            assert not nat.last_was_cached
        elif x < 0.85:
            assert nat.access_item(iid) == py.access_item(iid), step
        elif x < 0.93:
            s, _ = py.access_item(iid)
            if s is not None:
                nat.access_item(iid)
                py.page_managers[s].set_protected(iid)
                nat.set_protected(iid)
                protected.add(iid)
        elif protected:
            iid = protected.pop()
            s, _ = py.access_item(iid)
            nat.access_item(iid)
            if s is not None and py.page_managers[s].page_table[iid]["protected"] > 0:
                py.page_managers[s].remove_protected(iid)
                nat.remove_protected(iid)
        for s in range(k):
            assert nat.free_pages(s) == len(py.page_managers[s].free_pages)
            assert nat.item_count(s) == len(py.page_managers[s].page_table)


@pytest.mark.parametrize("seed", range(6))
def test_tiered_policy_equals_restated_go_semantics(native, seed):
    rnd = random.Random(100 + seed)
    cache, page, k = rnd.choice([(512, 16, 2), (2048, 16, 4), (3000, 50, 3)])
    ttl, p1max = rnd.choice([(50, None), (200, 6), (10, 0)])
    go = GoPageManagerOracle(cache, page, k, XorShiftChoice(seed + 7), ttl=ttl, p1_max_pages=p1max)
    nat = PageDirectory(cache, page, k, policy="tiered", seed=seed + 7, ttl=ttl, p1_max_pages=p1max)
    for step in range(2000):
        iid = rnd.randrange(120)
        x = rnd.random()
        if x < 0.5:
            ln = rnd.randint(1, cache // 4)
            is_user = iid % 3 == 0
            weight, typ = (1, "user cache") if is_user else (0, "item cache")
            try:
                want = go.load_item(iid, ln, weight, typ)
            except RuntimeError:
                with pytest.raises(RuntimeError):
                    nat.load_item(iid, ln, weight, typ)
                # both references leave the evictable items gone in this case
                for s in range(k):
                    assert nat.free_pages(s) == len(go.free[s])
                continue
            got = nat.load_item(iid, ln, weight, typ)
            assert got == (want[0], want[1]), step
            assert nat.last_evicted == want[2], step
        elif x < 0.85:
            assert nat.access_item(iid) == go.access_item(iid), step
        elif x < 0.9:
            now = go.clock + rnd.randint(0, 2 * ttl)
            go.advance_clock(now)
            nat.advance_clock(now)
        else:
            assert nat.priority(iid) == go.priority(iid), step
        if step % 50 == 0:
            for i in range(120):
                assert nat.priority(i) == go.priority(i), (step, i)
            for s in range(k):
                assert nat.free_pages(s) == len(go.free[s])


def test_priority_two_is_never_evicted_until_its_ttl_passes(native):
    d = PageDirectory(16 * 8, 16, 1, policy="tiered", ttl=100, p1_max_pages=8)
    d.load_item(1, 16 * 4, weight=1, item_type="user cache")     # user cache, priority 2
    d.load_item(2, 16 * 4)                                        # item, priority 0
    assert d.priority(1) == 2 and d.priority(2) == 0
    d.load_item(3, 16 * 4)                                        # must evict 2, not 1
    assert d.last_evicted == [2] and d.access_item(1)[0] == 0
    with pytest.raises(RuntimeError):
        d.load_item(4, 16 * 8)                                    # only priority 2 left besides 3
    d.advance_clock(10_000)
    assert d.priority(1) == 1
    d.load_item(5, 16 * 8)
    assert d.access_item(1) == (None, None)


def test_bad_arguments(native):
    assert not native.bikv_pm_create(-1, 16, 1, 0, 0)
    assert not native.bikv_pm_create(64, 0, 1, 0, 0)
    assert not native.bikv_pm_create(64, 16, 0, 0, 0)
    assert not native.bikv_pm_create(64, 16, 1, 7, 0)
    d = PageDirectory(64, 16, 1)
    with pytest.raises(ValueError):
        d.load_item(1, 65)
    assert d.access_item(9) == (None, None)
    with pytest.raises(KeyError):
        d.set_protected(9)


def test_native_batch_planner_equals_python_planner(native):
    """bikv_pm_plan_prefix_batch against PrefixCacheCoordinator.plan_batch (fast order)."""
    wl = PrefixReuseWorkload(seed=5, n_users=500, n_requests=3000, batch=48, n_workers=3,
                             prefix_median=300, prefix_clip=(32, 1500))
    py = PrefixCacheCoordinator(3, 700, 16, order="fast", seed=9, rng=XorShiftChoice(9))
    nat = NativePrefixCacheCoordinator(3, 700, 16, seed=9)
    for batch in wl.batches():
        for k in range(3):
            mine = [r for r in batch if r.worker == k]
            a, b = py.plan_batch(mine), nat.plan_batch(mine)
            assert a.hit == b.hit
            assert a.gather.table.tolist() == b.gather.table.tolist()
            assert a.scatter.table.tolist() == b.scatter.table.tolist()
    assert py.hit_rate == nat.hit_rate and 0.2 < nat.hit_rate < 0.95
