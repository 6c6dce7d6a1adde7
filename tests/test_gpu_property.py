"""Property test: random geometries, shard counts, layouts and ragged plans, every engine,
against the oracle (hypothesis drives the shapes; data is seeded random bit patterns)."""
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import build_plan
from oracle import bikv_oracle as O

from helpers import equal_bits, make_shards, make_workers

pytestmark = pytest.mark.gpu

DTYPES = {2: torch.bfloat16, 4: torch.float32, 1: torch.uint8}


@st.composite
def cases(draw):
    elt = draw(st.sampled_from([2, 2, 2, 4, 1]))
    layout = draw(st.sampled_from([N.POOL_PAGED, N.POOL_TOKEN_MAJOR]))
    vec = 16 // elt
    dim = vec * draw(st.integers(1, 4))                       # 16-byte vectors along dim
    heads = draw(st.integers(1, 3))
    layers = draw(st.integers(1, 5)) if layout == N.POOL_PAGED else draw(st.sampled_from([1, 2, 3, 4, 8]))
    page_tokens = draw(st.integers(1, 9))
    n_shards = draw(st.integers(1, 4))
    per = draw(st.integers(2, 12))
    rule = draw(st.sampled_from([N.SHARD_MOD, N.SHARD_BLOCK]))
    n_req = draw(st.integers(1, 4))
    total = n_shards * per
    perm = draw(st.permutations(list(range(total))))
    lists, tokens, at = [], [], 0
    for _ in range(n_req):
        n_pages = draw(st.integers(0, min(4, total - at)))
        pages = perm[at:at + n_pages]
        at += n_pages
        tail = draw(st.integers(1, page_tokens)) if n_pages else 0
        lists.append(pages)
        tokens.append((n_pages - 1) * page_tokens + tail if n_pages else 0)
    variant = draw(st.sampled_from([N.VARIANT_LDST, N.VARIANT_BULK]))
    return dict(geom=KVGeometry(layers, heads, dim, page_tokens, DTYPES[elt], layout), n_shards=n_shards, per=per,
                rule=rule, lists=lists, tokens=tokens, variant=variant, seed=draw(st.integers(0, 10_000)))


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture,
                                                                HealthCheck.too_slow, HealthCheck.data_too_large])
@given(case=cases())
def test_random_cases_match_the_oracle(cuda, case):
    g, tokens = case["geom"], case["tokens"]
    plan = build_plan(case["lists"], tokens, g.page_tokens, item_request=list(range(len(tokens))),
                      n_requests=len(tokens))
    recs = [tuple(r) for r in plan.table.tolist()]
    shards_cpu = make_shards(g, case["n_shards"], case["per"], case["seed"], fill="bits")
    shards_gpu = [s.to(cuda) for s in shards_cpu]
    pool = B.ShardedPool.from_tensors(shards_gpu, g, rule=case["rule"])
    mover = B.PageMover(cuda)
    sizes = [max(t, 1) for t in tokens]                       # an empty request still owns a tensor
    out = make_workers(g, sizes, cuda)
    mover.gather(pool, plan, out, variant=case["variant"])
    ref = make_workers(g, sizes)
    O.gather(shards_cpu, g, recs, ref, case["rule"])
    torch.cuda.synchronize()
    for a, b in zip(out, ref):
        assert equal_bits(a, b)
    src = make_workers(g, sizes, fill="normal", seed=case["seed"] + 1) if g.dtype != torch.uint8 else \
        [torch.randint(0, 255, g.worker_shape(t), dtype=torch.uint8) for t in sizes]
    mover.scatter(pool, plan, [t.to(cuda) for t in src], variant=case["variant"])
    O.scatter(shards_cpu, g, recs, src, case["rule"])
    torch.cuda.synchronize()
    mover.check_status()
    for a, b in zip(shards_gpu, shards_cpu):
        assert equal_bits(a, b)
