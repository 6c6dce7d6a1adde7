"""Oracle self-consistency and the native plan builder against it (CPU only)."""
import numpy as np
import pytest
import torch

from bikv_b200 import _native as N
from bikv_b200 import workloads as W
from bikv_b200.geometry import GEO_A, GEO_R, KVGeometry
from bikv_b200.plan import Plan, build_plan, flatten_page_lists, plan_from_combined_task
from bikv_b200.pool import global_page_id, shard_of
from oracle import bikv_oracle as O

from helpers import equal_bits, make_shards, make_workers, random_plan


def test_geometry_numbers():
    assert GEO_A.page_bytes == 196608 and GEO_A.bytes_per_token == 12288
    assert W.GEO_B.page_bytes == 917504 and W.GEO_B.bytes_per_token == 57344
    assert W.GEO_C.page_bytes == 5242880
    assert GEO_R.token_shape == (128, 2, 28, 2) and GEO_R.bytes_per_token == 28672  # 128*8*28 in the reference
    assert GEO_R.pool_shape(200) == (10000, 128, 2, 28, 2)


def test_oracle_identity_constant_seven():
    """The one result the reference's tests pin: identity map, constant 7 (test_page_ipc.py)."""
    pe = 50 * GEO_R.token_elems
    src = torch.full((4 * pe,), 7, dtype=torch.float16)
    dst = torch.zeros_like(src)
    off = [i * pe for i in range(4)]
    O.copy_pages_flat(src, dst, off, off, pe)
    assert torch.allclose(dst, torch.full_like(dst, 7))


@pytest.mark.parametrize("layout", [N.POOL_PAGED, N.POOL_TOKEN_MAJOR])
@pytest.mark.parametrize("rule", [N.SHARD_MOD, N.SHARD_BLOCK])
def test_oracle_gather_scatter_round_trip(layout, rule):
    g = KVGeometry(3, 2, 16, 4, torch.float16, layout)
    rng = np.random.default_rng(0)
    lists, tokens = random_plan(rng, g, 3 * 10, 4, 30)
    recs = O.plan_records([l.tolist() for l in lists], tokens.tolist(), 4, item_request=list(range(4)))
    shards = make_shards(g, 3, 10, 1)
    out = make_workers(g, tokens)
    O.gather(shards, g, recs, out, rule)
    fresh = [torch.zeros_like(s) for s in shards]
    O.scatter(fresh, g, recs, out, rule)
    back = make_workers(g, tokens)
    O.gather(fresh, g, recs, back, rule)
    for a, b in zip(out, back):
        assert equal_bits(a, b)
    # element-level spot check of the addressing, straight from the layout definitions
    page_id, valid, req, off = recs[-1]
    s, local = O.locate(page_id, 3, 10, rule)
    l, kv, t, h, d = 2, 1, valid - 1, 1, 7
    if layout == N.POOL_PAGED:
        want = shards[s].view(10, 3, 2, 4, 2, 16)[local, l, kv, t, h, d]
    else:
        want = shards[s].view(40, 16, 2, 3, 2)[local * 4 + t, d, h, l, kv]
    assert out[req][l, kv, off + t, h, d] == want


def test_token_index_form_equals_page_form():
    """The reference's CPU copy (token-indexed advanced indexing, Worker.py:207) moves the
    same tokens as the page-wise oracle."""
    g = KVGeometry(2, 2, 8, 4, torch.float16, N.POOL_TOKEN_MAJOR)
    rng = np.random.default_rng(2)
    lists, tokens = random_plan(rng, g, 20, 3, 19)
    recs = O.plan_records([l.tolist() for l in lists], tokens.tolist(), 4, item_request=[0, 1, 2])
    shards = make_shards(g, 1, 20, 3)
    src, dst = O.token_indices(recs, 4)
    buf = torch.zeros((int(tokens.sum()),) + g.token_shape, dtype=g.dtype)
    O.cpu_gather_tokens(shards[0], buf, src, dst)
    out = make_workers(g, tokens)
    O.gather(shards, g, recs, out)
    at = 0
    for r, t in enumerate(tokens):
        part = buf[at:at + int(t)].permute(3, 4, 0, 2, 1)   # [tok, D, H, L, 2] -> [L, 2, tok, H, D]
        assert equal_bits(part, out[r])
        at += int(t)
    pool2 = torch.zeros_like(shards[0])
    O.cpu_scatter_tokens(pool2, buf, src, dst)
    fresh = [torch.zeros_like(shards[0])]
    O.scatter(fresh, g, recs, out)
    assert equal_bits(pool2, fresh[0])


def test_native_plan_builder_matches_oracle_randomly(native):
    rng = np.random.default_rng(5)
    for trial in range(50):
        P = int(rng.choice([1, 4, 16, 50]))
        n_items = int(rng.integers(1, 12))
        n_req = int(rng.integers(1, 4))
        tokens = rng.integers(0, 6 * P, size=n_items)
        lists = [rng.integers(0, 1000, size=int(rng.integers(0, 7))).tolist() for _ in range(n_items)]
        req = rng.integers(0, n_req, size=n_items)
        shard = rng.integers(0, 4, size=n_items)
        plan = build_plan(lists, tokens, P, item_request=req, n_requests=n_req, item_shard=shard, pages_per_shard=1000)
        want = O.plan_records(lists, tokens.tolist(), P, item_request=req.tolist(), item_shard=shard.tolist(),
                              pages_per_shard=1000)
        assert [tuple(r) for r in plan.table.tolist()] == want


def test_plan_edge_cases(native):
    assert build_plan([], [], 16).n_pages == 0
    assert build_plan([[]], [0], 16).n_pages == 0
    p = build_plan([[3]], [16], 16)
    assert p.table.tolist() == [[3, 16, 0, 0]]
    p = build_plan([[3, 4]], [17], 16)
    assert p.table.tolist() == [[3, 16, 0, 0], [4, 1, 0, 16]]
    with pytest.raises(ValueError):
        build_plan([[1]], [1, 2], 16)
    with pytest.raises(N.BikvError) as e:
        build_plan([[1000]], [1], 16, item_shard=[0], pages_per_shard=1000)
    assert e.value.status == N.ERR_PAGE_RANGE
    with pytest.raises(N.BikvError):
        build_plan([[1]], [1], 16, item_request=[2], n_requests=2)


def test_plan_from_combined_task_dict_and_message(native):
    from bikv_b200 import taskinfo as pb
    task = {"infer_worker": 0, "cache_worker": 2, "token_num": 37, "task_type": 1,
            "id_token_pair": [(7, 20), (9, 17)], "cache_pages_list": [[4, 5], [1, 8]]}
    a = plan_from_combined_task(task, 16)
    assert a.table.tolist() == [[4, 16, 0, 0], [5, 4, 0, 16], [1, 16, 0, 20], [8, 1, 0, 36]]
    msg = pb.CombindedTaskInfo(cache_worker=2, token_num=37,
                               cache_pages_list=[pb.PageList(cache_pages_list=[4, 5]), pb.PageList(cache_pages_list=[1, 8])],
                               id_token_pair=[pb.IdTokenPair(id=7, token_num=20), pb.IdTokenPair(id=9, token_num=17)])
    b = plan_from_combined_task(msg, 16, pages_per_shard=100, block_sharded=True)
    assert b.table[:, 0].tolist() == [204, 205, 201, 208]
    assert b.table[:, 1:].tolist() == a.table[:, 1:].tolist()


def test_shard_maps_are_inverse():
    ids = np.arange(1000)
    for rule in (N.SHARD_MOD, N.SHARD_BLOCK):
        s, l = shard_of(ids, 8, 125, rule)
        assert (global_page_id(s, l, 8, 125, rule) == ids).all()
        assert s.max() == 7 and l.max() == 124


def test_workloads_are_seeded_and_consistent(native):
    a, b = W.config0(), W.config0()
    assert a.request_tokens.tolist() == b.request_tokens.tolist()
    assert all((x == y).all() for x, y in zip(a.page_lists, b.page_lists))
    assert 128 <= a.request_tokens.min() and a.request_tokens.max() <= 1024
    ids = np.concatenate(a.page_lists)
    assert len(set(ids.tolist())) == len(ids)
    w1 = W.config1()
    assert w1.n_requests == 64 and 64 <= w1.request_tokens.min() and w1.request_tokens.max() <= 8192
    assert w1.plan().total_tokens == w1.total_tokens
    # config 2: ranks use disjoint pages, spread over all shards
    ws = [W.config2(r, 4, pages_per_shard=16384) for r in range(4)]
    allids = np.concatenate([np.concatenate(w.page_lists) for w in ws])
    assert len(set(allids.tolist())) == len(allids)
    assert 0.70 < ws[1].remote_fraction(1) < 0.80
    c3 = W.config3(0, 8, n_requests=2)
    assert all(16384 <= w.total_tokens <= 32768 for w in c3)


def test_plan_from_table_roundtrip():
    t = np.array([[3, 16, 0, 0], [4, 2, 0, 16], [9, 5, 1, 0]], dtype=np.int32)
    p = Plan.from_table(t)
    assert p.n_pages == 3 and p.request_tokens.tolist() == [18, 5]
    assert p.recs["page_id"].tolist() == [3, 4, 9]
    flat, begin = flatten_page_lists([[1, 2], [], [3]])
    assert flat.tolist() == [1, 2, 3] and begin.tolist() == [0, 2, 2, 3]


def test_owner_split_covers_every_record_exactly_once(native):
    """Union over owners of the owner-side plans == union of the workers' plans, and an
    oracle gather run owner by owner fills the same worker tensors."""
    from bikv_b200.push import split_plans_by_owner

    g = KVGeometry(2, 2, 8, 4, torch.float16)
    world, per = 3, 16
    perm = np.random.default_rng(0).permutation(world * per * 4)
    tables, nreq, tokens_of = [], [], []
    for r in range(world):
        rng = np.random.default_rng(10 + r)
        tokens = rng.integers(1, 41, size=3)
        counts = (tokens + 3) // 4
        mine = perm[r * per * 4:(r + 1) * per * 4]
        lists, at = [], 0
        for c in counts:
            lists.append(mine[at:at + int(c)].tolist())
            at += int(c)
        tables.append(build_plan(lists, tokens, 4, item_request=[0, 1, 2], n_requests=3).table.copy())
        nreq.append(3)
        tokens_of.append(tokens)

    class _W:      # the two attributes the rest of the test reads
        def __init__(self, t):
            self.request_tokens, self.n_requests = t, len(t)
    ws = [_W(t) for t in tokens_of]
    shards = make_shards(g, world, per * 4, 2)
    want = [make_workers(g, w.request_tokens) for w in ws]
    for r in range(world):
        O.gather(shards, g, [tuple(x) for x in tables[r].tolist()], want[r])
    got = [make_workers(g, w.request_tokens) for w in ws]
    flat = [t for ts in got for t in ts]
    seen = 0
    for owner in range(world):
        push = split_plans_by_owner(tables, nreq, owner, world, per * 4)
        assert ((push[:, 0] % world) == owner).all()
        seen += len(push)
        # destinations interleave: no worker's rows are bunched into one stretch of the sweep,
        # and each worker's rows keep their plan order
        dest = push[:, 2] // 3
        for r in range(world):
            at = np.flatnonzero(dest == r)
            if len(at) >= 2:
                assert at[-1] - at[0] >= (len(push) - 1) // 2
            mine = push[at].copy()
            mine[:, 2] -= 3 * r
            rows_r = tables[r][(tables[r][:, 0] % world) == owner]
            assert np.array_equal(mine, rows_r)
        O.gather(shards, g, [tuple(x) for x in push.tolist()], flat)
    assert seen == sum(len(t) for t in tables)
    for a, b in zip(flat, [t for ts in want for t in ts]):
        assert equal_bits(a, b)


def test_table_views_outlive_their_plan(native):
    """Pinned plan buffers are recycled, but never while a view of one is still around."""
    a = build_plan([[1, 2, 3]], [40], 16).table          # the Plan itself is dropped at once
    b = build_plan([[7, 8, 9]], [48], 16).table
    assert a.tolist() == [[1, 16, 0, 0], [2, 16, 0, 16], [3, 8, 0, 32]]
    assert b.tolist() == [[7, 16, 0, 0], [8, 16, 0, 16], [9, 16, 0, 32]]


def test_page_lists_as_arrays_lists_and_mixed_flatten_alike():
    rng = np.random.default_rng(3)
    arrays = [rng.integers(0, 1000, size=n).astype(np.int32) for n in (5, 0, 17, 1)]
    as_lists = [a.tolist() for a in arrays]
    mixed = [arrays[0], as_lists[1], arrays[2].astype(np.int64), as_lists[3]]
    want_flat = np.concatenate(arrays)
    for form in (arrays, as_lists, mixed, [a.astype(np.int64) for a in arrays]):
        flat, begin = flatten_page_lists(form)
        assert flat.dtype == np.int32 and begin.dtype == np.int64
        assert np.array_equal(flat, want_flat)
        assert begin.tolist() == [0, 5, 5, 22, 23]
    flat, begin = flatten_page_lists([])
    assert len(flat) == 0 and begin.tolist() == [0]
