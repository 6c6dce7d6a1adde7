"""The closed-form pool / worker contents and their checks, against the CPU oracle: what the
checks accept is exactly what the oracle's gather and scatter produce, and they reject the
errors a sum cannot see (right words, wrong place)."""
import numpy as np
import torch

from bikv_b200 import _native as N
from bikv_b200 import selfcheck as S
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import build_plan
from oracle import bikv_oracle as O


class _W:
    def __init__(self, geom, page_lists, request_tokens):
        self.geom, self.page_lists, self.request_tokens = geom, page_lists, request_tokens


def _case(rule, seed=0):
    g = KVGeometry(3, 2, 8, 4, torch.float16)
    n_shards, per = 2, 12
    rng = np.random.default_rng(seed)
    tokens = np.array([9, 4, 13, 1])
    counts = (tokens + g.page_tokens - 1) // g.page_tokens
    perm = rng.permutation(n_shards * per)[: counts.sum()]
    lists, at = [], 0
    for c in counts:
        lists.append(perm[at:at + c])
        at += c
    shards = [torch.zeros(g.pool_shape(per), dtype=g.dtype) for _ in range(n_shards)]
    ids = [S.global_ids_of_shard(s, n_shards, per, rule) for s in range(n_shards)]
    for s in range(n_shards):
        S.fill_pool_(shards[s], g, ids[s], chunk_pages=5)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), g.page_tokens,
                      item_request=np.arange(len(tokens), dtype=np.int32), n_requests=len(tokens))
    recs = [tuple(r) for r in plan.table.tolist()]
    return g, n_shards, per, tokens, lists, shards, ids, recs


def test_gather_of_a_closed_form_pool_is_what_the_check_expects():
    for rule in (N.SHARD_MOD, N.SHARD_BLOCK):
        g, n_shards, per, tokens, lists, shards, ids, recs = _case(rule)
        out = [torch.zeros(g.worker_shape(int(t)), dtype=g.dtype) for t in tokens]
        O.gather(shards, g, recs, out, rule)
        for t, l, n in zip(out, lists, tokens):
            assert S.check_gathered(g, t, l, int(n), max_tokens_per_pass=5)
        # right words, wrong place: two tokens swapped, two planes swapped, pages swapped
        bad = out[0].clone()
        bad[:, :, [0, 1]] = bad[:, :, [1, 0]]
        assert not S.check_gathered(g, bad, lists[0], int(tokens[0]))
        bad = out[0].clone()
        bad[[0, 1]] = bad[[1, 0]]
        assert not S.check_gathered(g, bad, lists[0], int(tokens[0]))
        assert not S.check_gathered(g, out[0], lists[0][::-1], int(tokens[0]))
        bad = out[2].clone()
        bad.view(torch.int16)[1, 1, 12, 1, 7] ^= 1
        assert not S.check_gathered(g, bad, lists[2], int(tokens[2]))


def test_scatter_of_closed_form_workers_is_what_the_pool_check_expects():
    for rule in (N.SHARD_MOD, N.SHARD_BLOCK):
        g, n_shards, per, tokens, lists, shards, ids, recs = _case(rule, seed=3)
        rank = 5
        src = [torch.zeros(g.worker_shape(int(t)), dtype=g.dtype) for t in tokens]
        for r, t in enumerate(src):
            S.fill_worker_(g, t, rank, r, max_tokens_per_pass=3)
        before = [s.clone() for s in shards]
        O.scatter(shards, g, recs, src, rule)
        ws = [None] * rank + [_W(g, lists, tokens)]
        ws = [_W(g, [], np.zeros(0, dtype=np.int64)) if w is None else w for w in ws]
        for s in range(n_shards):
            touched = S.touched_pages(ws, s, n_shards, per, rule)
            assert S.check_scattered_pool(shards[s], g, ids[s], touched, chunk_pages=5)
            assert not S.check_scattered_pool(before[s], g, ids[s], touched) or len(touched) == 0
            assert S.check_scattered_pool(before[s], g, ids[s], touched[:0])
            # a word of an untouched region changed
            bad = shards[s].clone()
            bad.view(-1).view(torch.int16)[-1] ^= 1
            assert not S.check_scattered_pool(bad, g, ids[s], touched)
            # two touched pages exchanged
            if len(touched) >= 2:
                a, b = int(touched[0, 0]), int(touched[1, 0])
                bad = shards[s].clone()
                bad[[a, b]] = bad[[b, a]]
                assert not S.check_scattered_pool(bad, g, ids[s], touched)
        assert sum(len(S.touched_pages(ws, s, n_shards, per, rule)) for s in range(n_shards)) == len(recs)


def test_position_hash_sees_words_that_move():
    t = torch.arange(4096, dtype=torch.int32).view(torch.float16).clone()
    h = S.position_hash(t, chunk_words=500)
    assert h == S.position_hash(t.clone(), chunk_words=4096)
    moved = t.view(torch.int32).clone()
    moved[[3, 900]] = moved[[900, 3]]
    assert moved.sum() == t.view(torch.int32).sum()          # a plain sum is blind to it
    assert S.position_hash(moved) != h
