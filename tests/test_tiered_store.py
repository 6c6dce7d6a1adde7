"""HBM tier + host tier behind one page table: items evicted from HBM are copied to the host
tier before their pages are reused, items found only there are copied back on access.  Host
logic on the CPU (the page copies stood in for by the oracle's flat copy), data on the GPU."""
import numpy as np
import pytest
import torch

from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import build_plan
from bikv_b200.tiered_store import TieredPageStore
from oracle import bikv_oracle as O

from helpers import equal_bits, normal

GEOM = KVGeometry(2, 2, 16, 4, torch.float16)


def _drive(store, put, get, rounds=120, n_items=14, seed=0, batch=0):
    """Random stores and fetches; every fetched item must read back exactly what was stored.
    With ``batch`` the accesses run in batches of that many distinct items, copies deferred."""
    rng = np.random.default_rng(seed)
    tokens_of = {i: 1 + (5 * i) % 12 for i in range(n_items)}
    content = store.__dict__.setdefault("_test_content", {})       # survives a second drive of the same store
    if batch:
        for step in range(rounds // batch):
            items = rng.permutation(n_items)[:batch].tolist()
            store.begin_batch()
            got = [(i, store.fetch(i)) for i in items]
            new = [(i, store.store(i, tokens_of[i])) for i, p in got if p is None]
            store.end_batch()
            for i, pages in got:
                if pages is not None:
                    assert equal_bits(get(pages, tokens_of[i]), content[i]), f"batch {step}, item {i}"
            for i, pages in new:
                content[i] = normal(GEOM.worker_shape(tokens_of[i]), GEOM.dtype, 1000 * i + 7)
                put(pages, tokens_of[i], content[i])
        return store.stats
    for step in range(rounds):
        item = int(rng.integers(0, n_items))
        pages = store.fetch(item)
        if pages is None:
            assert store.where(item) is None
            data = normal(GEOM.worker_shape(tokens_of[item]), GEOM.dtype, 1000 * item + 7)
            content[item] = data
            put(store.store(item, tokens_of[item]), tokens_of[item], data)
        else:
            assert item in content, "a fetch hit an item that was never stored"
            assert equal_bits(get(pages, tokens_of[item]), content[item]), f"step {step}, item {item}"
            assert store.where(item) == "hbm"
    return store.stats


def test_directory_logic_with_a_stand_in_copier():
    def copier(src, dst, src_pages, dst_pages, stream):
        pe = GEOM.page_elems
        O.copy_pages_flat(src, dst, [p * pe for p in src_pages], [p * pe for p in dst_pages], pe)

    store = TieredPageStore(GEOM, hbm_pages=8, host_pages=20, device="cpu", copier=copier)

    def put(pages, tokens, data):
        recs = O.plan_records([pages], [tokens], GEOM.page_tokens)
        O.scatter([store.hbm, store.host], GEOM, recs, [data], N.SHARD_BLOCK)

    def get(pages, tokens):
        out = torch.zeros(GEOM.worker_shape(tokens), dtype=GEOM.dtype)
        O.gather([store.hbm, store.host], GEOM, O.plan_records([pages], [tokens], GEOM.page_tokens), [out], N.SHARD_BLOCK)
        return out

    # the two shards of the oracle call must hold the same number of pages
    store.hbm = torch.zeros(GEOM.pool_shape(20), dtype=GEOM.dtype)
    store._per = 20
    st = _drive(store, put, get)
    assert st.demotions > 0 and st.promotions > 0 and st.clean_demotions > 0
    assert st.host_hits == st.promotions and st.hbm_hits > 0 and st.misses > 0
    st = _drive(store, put, get, rounds=150, seed=5, batch=2)      # the same store, now in batches
    assert st.promotions > 20
    assert st.pages_demoted >= st.demotions and st.pages_promoted >= st.promotions
    with pytest.raises(ValueError):
        store.store(next(iter(store._hbm_items)), 4)               # cached KV is immutable


def test_spill_policy_keeps_only_what_proved_reusable():
    moved = []
    store = TieredPageStore(GEOM, hbm_pages=4, host_pages=8, device="cpu", min_hits_to_spill=1,
                            copier=lambda src, dst, sp, dp, st: moved.append((len(sp), src is store.hbm)))
    store.store(1, 8)                      # 2 pages, fetched once below
    store.store(2, 8)                      # 2 pages, never fetched
    assert store.fetch(1) is not None
    store.store(3, 8, spill=False)         # evicts 2 (least recent): not spilled, it never proved reusable
    assert store.where(2) is None and store.stats.not_spilled == 1 and moved == []
    store.store(4, 8)                      # evicts 1: spilled
    assert store.where(1) == "host" and moved == [(2, True)]
    store.store(5, 8)                      # evicts 3: excluded by its own flag
    assert store.where(3) is None and store.stats.not_spilled == 2
    assert store.fetch(1) is not None and store.where(1) == "hbm" and moved[-1] == (2, False)


@pytest.mark.gpu
def test_spill_and_promote_on_the_gpu(cuda):
    import bikv_b200 as B
    store = TieredPageStore(GEOM, hbm_pages=8, host_pages=20, device=cuda)
    mover = store.mover

    def put(pages, tokens, data):
        plan = build_plan([pages], [tokens], GEOM.page_tokens)
        src = data.to(cuda)
        mover.scatter(store.pool, plan, src)
        torch.cuda.synchronize()

    def get(pages, tokens):
        out = torch.zeros(GEOM.worker_shape(tokens), dtype=GEOM.dtype, device=cuda)
        mover.gather(store.pool, build_plan([pages], [tokens], GEOM.page_tokens), out)
        torch.cuda.synchronize()
        return out

    st = _drive(store, put, get, rounds=200, seed=3)
    assert st.demotions > 0 and st.promotions > 0 and st.clean_demotions > 0
    st = _drive(store, put, get, rounds=150, seed=5, batch=2)
    mover.check_status()
    # an item that sits only in the host tier can also be gathered in place, without promotion
    only_host = [i for i in store._host_tokens if store.where(i) == "host"]
    assert only_host
    item = only_host[0]
    _, host_pages = store.dir_host.access_item(item)
    tokens = store.tokens_of(item)
    direct = get(store.global_ids(host_pages, tier=1), tokens)
    promoted = get(store.fetch(item), tokens)
    assert equal_bits(direct, promoted)
