"""Parity of the CUDA path (through the C ABI) with the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200 import workloads as W
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import Plan, build_plan
from oracle import bikv_oracle as O

from helpers import equal_bits, make_shards, make_workers, random_plan

pytestmark = pytest.mark.gpu

TINY = KVGeometry(2, 1, 8, 4, torch.float16)            # 16-byte rows
SMALL = KVGeometry(3, 2, 64, 16, torch.bfloat16)
GEOS = {"tiny": TINY, "small": SMALL, "A": B.GEO_A, "B": B.GEO_B,
        "C-lite": KVGeometry(4, 8, 128, 16, torch.float16),   # 32 KiB planes -> 2 parts
        "u8": KVGeometry(2, 2, 32, 8, torch.uint8), "f32": KVGeometry(2, 2, 16, 8, torch.float32)}
VARIANTS = {"ldst": N.VARIANT_LDST, "bulk": N.VARIANT_BULK}


def run_case(cuda, geom, n_shards, pages_per_shard, n_requests, max_tokens, variant, rule=N.SHARD_MOD,
             seed=0, fill="bits", min_tokens=1):
    rng = np.random.default_rng(seed)
    lists, tokens = random_plan(rng, geom, n_shards * pages_per_shard, n_requests, max_tokens, min_tokens)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), geom.page_tokens,
                      item_request=np.arange(n_requests, dtype=np.int32), n_requests=n_requests)
    recs = [tuple(r) for r in plan.table.tolist()]
    shards_cpu = make_shards(geom, n_shards, pages_per_shard, seed, fill=fill)
    mover = B.PageMover(cuda)

    # gather
    shards_gpu = [s.to(cuda) for s in shards_cpu]
    pool = B.ShardedPool.from_tensors(shards_gpu, geom, rule=rule)
    out_gpu = make_workers(geom, tokens, cuda)
    mover.gather(pool, plan, out_gpu, variant=variant)
    out_cpu = make_workers(geom, tokens)
    O.gather(shards_cpu, geom, recs, out_cpu, rule)
    torch.cuda.synchronize()
    mover.check_status()
    for a, b in zip(out_gpu, out_cpu):
        assert equal_bits(a, b)
    for a, b in zip(shards_gpu, shards_cpu):
        assert equal_bits(a, b), "gather must not write the pool"

    # scatter fresh worker data into the pool
    src_cpu = make_workers(geom, tokens, fill="normal", seed=seed + 1000)
    src_gpu = [t.to(cuda) for t in src_cpu]
    mover.scatter(pool, plan, src_gpu, variant=variant)
    O.scatter(shards_cpu, geom, recs, src_cpu, rule)
    torch.cuda.synchronize()
    mover.check_status()
    for a, b in zip(shards_gpu, shards_cpu):
        assert equal_bits(a, b)
    for a, b in zip(src_gpu, src_cpu):
        assert equal_bits(a, b), "scatter must not write the worker tensors"


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("geo", GEOS)
def test_paged_single_shard(cuda, geo, variant):
    g = GEOS[geo]
    run_case(cuda, g, 1, 48, 5, 9 * g.page_tokens, VARIANTS[variant], seed=1)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("rule", [N.SHARD_MOD, N.SHARD_BLOCK])
@pytest.mark.parametrize("n_shards", [2, 3, 8, 16])
def test_paged_multi_shard_addressing(cuda, n_shards, rule, variant):
    run_case(cuda, SMALL, n_shards, 11, 7, 6 * 16, VARIANTS[variant], rule=rule, seed=n_shards)


@pytest.mark.parametrize("variant", VARIANTS)
def test_every_tail_length(cuda, variant):
    """One request per tail length 1..page_tokens (and exact multiples)."""
    g = SMALL
    for tail in range(1, g.page_tokens + 1):
        run_case(cuda, g, 1, 8, 1, 16 + tail, VARIANTS[variant], seed=tail, min_tokens=16 + tail)
        run_case(cuda, g, 1, 8, 1, tail, VARIANTS[variant], seed=tail, min_tokens=tail)


@pytest.mark.parametrize("variant", VARIANTS)
def test_config3_full_geometry(cuda, variant):
    """Configuration 3 as stated: 80 layers, 8 KV heads, head 128, fp16, 16-token pages (5 MiB
    each, 32 KiB planes), pool striped over 8 shards, ragged last pages -- against the oracle."""
    run_case(cuda, B.GEO_C, 8, 6, 4, 11 * 16 + 5, VARIANTS[variant], seed=33, min_tokens=16 * 3 + 1)


@pytest.mark.parametrize("variant", VARIANTS)
def test_many_small_requests_more_items_than_grid(cuda, variant):
    run_case(cuda, B.GEO_A, 2, 2048, 64, 1024, VARIANTS[variant], seed=5, fill="normal", min_tokens=128)


@pytest.mark.parametrize("seg", [1024, 4096, 16384, 65536])
@pytest.mark.parametrize("variant", VARIANTS)
def test_segment_sizes(cuda, native, variant, seg):
    old = native.bikv_get_tuning(b"seg_bytes"), native.bikv_get_tuning(b"ldst_seg_bytes")
    try:
        assert native.bikv_set_tuning(b"seg_bytes", seg) == 0 and native.bikv_set_tuning(b"ldst_seg_bytes", seg) == 0
        run_case(cuda, GEOS["C-lite"], 1, 32, 3, 100, VARIANTS[variant], seed=seg)
    finally:
        native.bikv_set_tuning(b"seg_bytes", old[0])
        native.bikv_set_tuning(b"ldst_seg_bytes", old[1])


@pytest.mark.parametrize("stages", [2, 3, 8, 12])
def test_bulk_stage_counts(cuda, native, stages):
    old = native.bikv_get_tuning(b"bulk_stages")
    try:
        assert native.bikv_set_tuning(b"bulk_stages", stages) == 0
        run_case(cuda, B.GEO_B, 1, 64, 4, 200, N.VARIANT_BULK, seed=stages)
    finally:
        native.bikv_set_tuning(b"bulk_stages", old)


def test_packed_single_tensor_like_the_reference(cuda):
    """All items of a combined task land back to back in ONE tensor (the reference's
    running dest_offsets)."""
    g = SMALL
    pages = [[5, 9, 2], [7], [11, 3]]
    tokens = [40, 16, 17]
    plan = build_plan(pages, tokens, g.page_tokens)
    recs = [tuple(r) for r in plan.table.tolist()]
    assert recs == O.plan_records(pages, tokens, g.page_tokens)
    shards_cpu = make_shards(g, 1, 16, 3)
    pool = B.ShardedPool.single(shards_cpu[0].to(cuda), g)
    out = make_workers(g, [73], cuda)
    B.PageMover(cuda).gather(pool, plan, out[0])
    ref = make_workers(g, [73])
    O.gather(shards_cpu, g, recs, ref)
    assert equal_bits(out[0], ref[0])


def test_device_plan_entry_points(cuda):
    """bikv_gather / bikv_scatter with the plan already resident on the device."""
    g = B.GEO_A
    rng = np.random.default_rng(3)
    lists, tokens = random_plan(rng, g, 256, 6, 500)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), g.page_tokens,
                      item_request=np.arange(6, dtype=np.int32), n_requests=6)
    recs = [tuple(r) for r in plan.table.tolist()]
    shards_cpu = make_shards(g, 1, 256, 4)
    shard = shards_cpu[0].to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    out = make_workers(g, tokens, cuda)
    d_recs, d_reqs = mover.upload(plan, g, out)
    for variant in VARIANTS.values():
        for t in out:
            t.zero_()
        mover.gather_dev(pool, d_recs, d_reqs, variant=variant)
        ref = make_workers(g, tokens)
        O.gather(shards_cpu, g, recs, ref)
        for a, b in zip(out, ref):
            assert equal_bits(a, b)
        shard.zero_()
        mover.scatter_dev(pool, d_recs, d_reqs, variant=variant)
        torch.cuda.synchronize()
        zero = [torch.zeros_like(shards_cpu[0])]
        O.scatter(zero, g, recs, ref)
        assert equal_bits(shard, zero[0])
        shard.copy_(shards_cpu[0])


def test_config0_round_trip(cuda):
    """Config 0: gather every request, scatter into a zeroed pool, compare with the
    oracle and with the original pool on the touched tokens."""
    w = W.config0()
    g = w.geom
    pool_cpu = torch.randn(g.pool_shape(w.pages_per_shard), generator=torch.Generator().manual_seed(0)).to(g.dtype)
    plan = w.plan()
    recs = [tuple(r) for r in plan.table.tolist()]
    mover = B.PageMover(cuda)
    shard = pool_cpu.to(cuda)
    out = make_workers(g, w.request_tokens, cuda)
    mover.gather(B.ShardedPool.single(shard, g), plan, out)
    ref = make_workers(g, w.request_tokens)
    O.gather([pool_cpu], g, recs, ref)
    for a, b in zip(out, ref):
        assert equal_bits(a, b)
    fresh = torch.zeros_like(shard)
    mover.scatter(B.ShardedPool.single(fresh, g), plan, out)
    fresh_ref = torch.zeros_like(pool_cpu)
    O.scatter([fresh_ref], g, recs, ref)
    assert equal_bits(fresh, fresh_ref)
    # touched tokens equal the original pool
    t = plan.table
    full = t[t[:, 1] == g.page_tokens, 0]
    assert equal_bits(fresh[full.tolist()], pool_cpu[full.tolist()])


def test_invalid_plans_are_rejected_before_launch(cuda):
    g = SMALL
    shard = torch.zeros(g.pool_shape(8), dtype=g.dtype, device=cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    out = make_workers(g, [32], cuda)
    launches = N.lib().bikv_launch_count()
    for table, status in [([[8, 16, 0, 0]], N.ERR_PAGE_RANGE), ([[0, 16, 0, 17]], N.ERR_DST_RANGE),
                          ([[0, 17, 0, 0]], N.ERR_PLAN), ([[0, 16, 1, 0]], N.ERR_BAD_ARG)]:
        with pytest.raises(B.BikvError) as e:
            mover.gather(pool, Plan.from_table(np.array(table), 1), out)
        assert e.value.status == status
    with pytest.raises(B.BikvError) as e:
        mover.scatter(pool, Plan.from_table(np.array([[1, 16, 0, 0], [1, 16, 0, 16]]), 1), out)
    assert e.value.status == N.ERR_OVERLAP
    assert N.lib().bikv_launch_count() == launches
    assert int(shard.abs().sum()) == 0


def test_full_size_config1_properties(cuda):
    """Config 1 at full size (65,536-page pool, 64 requests): properties that need no
    oracle pass over 10 GB -- (1) scatter(gather(pool)) into a zeroed pool and a second
    gather reproduce the first gather bit for bit, (2) per-request checksums match
    checksums computed directly from the pool pages, (3) untouched pages stay zero."""
    free, _ = torch.cuda.mem_get_info()
    w = W.config1()
    g = w.geom
    need = w.pages_per_shard * g.page_bytes + 2 * w.payload_bytes + (4 << 30)
    if free < need:
        pytest.skip(f"needs {need >> 30} GiB of device memory")
    shard = torch.empty(g.pool_shape(w.pages_per_shard), dtype=g.dtype, device=cuda)
    W.fill_normal_(shard, seed=1)
    plan = w.plan()
    mover = B.PageMover(cuda)
    pool = B.ShardedPool.single(shard, g)
    first = make_workers(g, w.request_tokens, cuda)
    mover.gather(pool, plan, first)
    # (2) checksum of each request against the pool pages read directly with torch
    for r in (0, 17, 63):
        ids = torch.from_numpy(w.page_lists[r].astype(np.int64)).to(cuda)
        pages = shard[ids]                                  # [n, L, 2, P, H, D]
        want = pages.permute(1, 2, 0, 3, 4, 5).reshape(g.n_layers, 2, -1, g.n_kv_heads, g.head_dim)
        want = want[:, :, : int(w.request_tokens[r])]
        assert torch.equal(first[r].view(torch.int16), want.contiguous().view(torch.int16))
    # (1) round trip through a zeroed pool
    touched = torch.from_numpy(np.concatenate(w.page_lists).astype(np.int64)).to(cuda)
    shard.zero_()
    mover.scatter(pool, plan, first)
    second = make_workers(g, w.request_tokens, cuda)
    mover.gather(pool, plan, second)
    torch.cuda.synchronize()
    for a, b in zip(first, second):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # (3) pages outside the plan were not written
    mask = torch.ones(w.pages_per_shard, dtype=torch.bool, device=cuda)
    mask[touched] = False
    untouched = mask.nonzero().flatten()[:: 97]
    assert int(shard[untouched].view(torch.int16).ne(0).sum()) == 0
    mover.check_status()


def test_empty_and_degenerate_plans(cuda):
    """Empty plan, items without tokens, a single one-token page: no faults, no stray writes."""
    g = SMALL
    shard = torch.full(g.pool_shape(4), 3.0, dtype=g.dtype, device=cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    out = make_workers(g, [16], cuda)
    launches = N.lib().bikv_launch_count()
    for plan in (build_plan([], [], 16), build_plan([[]], [0], 16), build_plan([[], []], [0, 0], 16)):
        assert plan.n_pages == 0
        mover.gather(pool, plan, out)
        mover.scatter(pool, plan, out)
    assert N.lib().bikv_launch_count() == launches
    one = build_plan([[2]], [1], 16)
    assert one.table.tolist() == [[2, 1, 0, 0]]
    mover.gather(pool, one, out)
    torch.cuda.synchronize()
    assert float(out[0][:, :, 0].float().min()) == 3.0 and float(out[0][:, :, 1:].float().abs().max()) == 0.0
    out[0].fill_(5.0)
    mover.scatter(pool, one, out)
    torch.cuda.synchronize()
    page = shard[2]                                   # [L, 2, P, H, D]
    assert float(page[:, :, 0].float().min()) == 5.0 and float(page[:, :, 1:].float().max()) == 3.0
    assert float(shard[[0, 1, 3]].float().min()) == 3.0 and float(shard[[0, 1, 3]].float().max()) == 3.0


def test_size_limits_are_refused_not_truncated(native):
    """More chunks than the 32-bit item counter holds: refused on the host (needs no GPU
    memory: the check precedes the launch)."""
    import ctypes as C
    g = N.Geometry(128, 8, 128, 16, 2, N.POOL_PAGED)          # 256 planes, 2 parts of 16 KiB each
    pool = N.PoolDesc()
    pool.shard_base[0] = 0x10000
    pool.n_shards, pool.shard_rule, pool.pages_per_shard = 1, N.SHARD_MOD, 1 << 30
    rc = native.bikv_gather(C.byref(pool), C.byref(g), C.c_void_p(0x1000), 1 << 23, C.c_void_p(0x2000), 1,
                            N.VARIANT_LDST, None, None)
    assert rc in (N.ERR_TOO_LARGE, N.ERR_CUDA)                # too many items, or no device on a CPU box
    big = N.PoolDesc()
    big.shard_base[0] = 0x10000
    big.n_shards, big.shard_rule, big.pages_per_shard = 2, N.SHARD_MOD, 1 << 31
    assert native.bikv_gather(C.byref(big), C.byref(g), C.c_void_p(0x1000), 1, C.c_void_p(0x2000), 1,
                              N.VARIANT_LDST, None, None) == N.ERR_TOO_LARGE


def test_bounded_device_wait_reports_a_timeout_and_the_context_survives(cuda):
    """A wait that nothing satisfies runs out after its limit, the status word carries
    BIKV_ERR_DEVICE_TIMEOUT, check_status raises and clears it, and the GPU keeps working."""
    import ctypes as C
    import time
    mover = B.PageMover(cuda)
    stream = C.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    t0 = time.perf_counter()
    N.check(N.lib().bikv_selftest_wait_timeout(C.c_void_p(mover.status.data_ptr()), 20_000_000, stream))
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.015 < waited < 1.0, waited
    with pytest.raises(B.BikvError) as e:
        mover.check_status()
    assert e.value.status == N.ERR_DEVICE_TIMEOUT
    mover.check_status()                                    # cleared
    run_case(cuda, SMALL, 1, 8, 2, 40, N.VARIANT_BULK, seed=3)     # the context is still usable
    assert N.lib().bikv_selftest_wait_timeout(None, 1000, None) == N.ERR_BAD_ARG
    assert N.lib().bikv_selftest_wait_timeout(C.c_void_p(mover.status.data_ptr()), 2_000_000_000, None) == N.ERR_BAD_ARG


@pytest.mark.parametrize("layout", [N.POOL_PAGED, N.POOL_TOKEN_MAJOR])
@pytest.mark.parametrize("variant", VARIANTS)
def test_bad_records_in_a_device_plan_are_skipped_not_dereferenced(cuda, layout, variant):
    """Plans handed over in device memory cannot be checked on the host.  The kernels check
    each record themselves: a bad one is skipped (no access at all), the first error lands in
    the status word, good records are still served."""
    g = KVGeometry(4, 2, 64, 16, torch.float16, layout)
    shard_cpu = make_shards(g, 1, 8, 1)[0]
    shard = shard_cpu.to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    out = make_workers(g, [48], cuda)
    good = [[3, 16, 0, 0], [5, 7, 0, 16]]
    bad = [[8, 16, 0, 32], [2_000_000_000, 16, 0, 32], [-1, 16, 0, 32],      # page outside the pool
           [1, 0, 0, 32], [1, 17, 0, 32],                                  # valid_tokens out of range
           [1, 16, 1, 32], [1, 16, -5, 32],                                # request index out of range
           [1, 16, 0, 33], [1, 16, 0, -16], [1, 16, 0, 2_000_000_000]]     # token window outside the tensor
    table = torch.tensor(good + bad, dtype=torch.int32, device=cuda)
    reqs = mover.request_table(g, out).to(cuda)
    mover.gather_dev(pool, table, reqs, variant=VARIANTS[variant])
    torch.cuda.synchronize()
    ref = make_workers(g, [48])
    O.gather([shard_cpu], g, [tuple(r) for r in good], ref)
    assert equal_bits(out[0], ref[0])                      # good records served, nothing else written
    with pytest.raises(B.BikvError) as e:
        mover.check_status()
    assert e.value.status in (N.ERR_PAGE_RANGE, N.ERR_PLAN, N.ERR_BAD_ARG, N.ERR_DST_RANGE)
    # the same plan as a scatter must leave the pool untouched outside the good pages
    src = make_workers(g, [48], fill="normal", seed=5)
    src_gpu = [src[0].to(cuda)]                          # must outlive the launch
    mover.scatter_dev(pool, table, mover.request_table(g, src_gpu).to(cuda), variant=VARIANTS[variant])
    torch.cuda.synchronize()
    O.scatter([shard_cpu], g, [tuple(r) for r in good], src)
    assert equal_bits(shard, shard_cpu)
    with pytest.raises(B.BikvError):
        mover.check_status()
    mover.check_status()


# LDST on the paged layout first: its copy loop tolerates any alignment, so this case cannot
# fault even if the check were missing, and a run that stops at the first failure never
# reaches the kernels that issue 16-byte and bulk accesses.
@pytest.mark.parametrize("layout,variant", [(N.POOL_PAGED, "ldst"), (N.POOL_PAGED, "bulk"),
                                            (N.POOL_TOKEN_MAJOR, "ldst")])
def test_bad_request_bases_in_a_device_table_are_skipped_not_dereferenced(cuda, layout, variant):
    """A request table in device memory cannot be checked on the host either.  A record that
    selects a request whose base is NULL or not 16-byte aligned is skipped before any address
    is formed from it; records of the other requests are served."""
    g = KVGeometry(4, 2, 64, 16, torch.float16, layout)
    shard_cpu = make_shards(g, 1, 8, 2)[0]
    shard = shard_cpu.to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    out = make_workers(g, [32], cuda)
    # Backing store for the misaligned request: base + 8 stays inside this allocation.
    backing = torch.zeros(g.token_elems * 33, dtype=g.dtype, device=cuda)
    good = [[3, 16, 0, 0], [5, 9, 0, 16]]
    for bad_base, want in ((backing.data_ptr() + 8, N.ERR_ALIGNMENT), (backing.data_ptr() + 2, N.ERR_ALIGNMENT),
                           (0, N.ERR_BAD_ARG)):
        out[0].zero_()
        reqs = torch.tensor([[out[0].data_ptr(), 32], [bad_base, 32]], dtype=torch.int64, device=cuda)
        table = torch.tensor(good + [[1, 16, 1, 0], [2, 16, 1, 16]], dtype=torch.int32, device=cuda)
        mover.gather_dev(pool, table, reqs, variant=VARIANTS[variant])
        torch.cuda.synchronize()
        ref = make_workers(g, [32])
        O.gather([shard_cpu], g, [tuple(r) for r in good], ref)
        assert equal_bits(out[0], ref[0])
        assert int(backing.view(torch.int16).ne(0).sum()) == 0
        with pytest.raises(B.BikvError) as e:
            mover.check_status()
        assert e.value.status == want
        # scatter: the pool stays as it is outside the good pages
        src = make_workers(g, [32], fill="normal", seed=9)
        src_gpu = src[0].to(cuda)
        reqs = torch.tensor([[src_gpu.data_ptr(), 32], [bad_base, 32]], dtype=torch.int64, device=cuda)
        mover.scatter_dev(pool, table, reqs, variant=VARIANTS[variant])
        torch.cuda.synchronize()
        O.scatter([shard_cpu], g, [tuple(r) for r in good], src)
        assert equal_bits(shard, shard_cpu)
        with pytest.raises(B.BikvError) as e:
            mover.check_status()
        assert e.value.status == want


def test_ldst_kernels_with_32_byte_accesses(cuda, native):
    """`ldst_wide`: 32-byte loads and stores wherever both sides are 32-byte aligned, 16-byte
    ones and byte tails elsewhere (rows of 16 bytes, odd tails, unaligned flat copies)."""
    old = native.bikv_get_tuning(b"ldst_wide")
    try:
        assert native.bikv_set_tuning(b"ldst_wide", 1) == 0
        for name, pages in (("tiny", 48), ("small", 48), ("A", 48), ("B", 48), ("C-lite", 32), ("u8", 48), ("f32", 48)):
            g = GEOS[name]
            run_case(cuda, g, 2, pages // 2, 5, 9 * g.page_tokens, N.VARIANT_LDST, seed=len(name))
        for tail in (1, 7, 15):
            run_case(cuda, SMALL, 1, 8, 1, 16 + tail, N.VARIANT_LDST, seed=tail, min_tokens=16 + tail)
        mover = B.PageMover(cuda)
        src = torch.arange(1 << 20, dtype=torch.int32, device=cuda).view(torch.uint8)
        for so, do, n in ((0, 0, 1 << 20), (32, 64, 100_000), (16, 48, 77_777), (3, 3, 65_537), (1, 2, 4099)):
            dst = torch.zeros(1 << 21, dtype=torch.uint8, device=cuda)
            mover.copy_range(dst.data_ptr() + do, src.data_ptr() + so, n)
            torch.cuda.synchronize()
            assert torch.equal(dst[do:do + n], src[so:so + n]) and int(dst[:do].sum()) == 0 and int(dst[do + n:].sum()) == 0
    finally:
        native.bikv_set_tuning(b"ldst_wide", old)


@pytest.mark.parametrize("span", [2, 3, 4, 8])
def test_bulk_ring_with_several_planes_per_stage(cuda, native, span):
    """The bulk ring may move `bulk_span` adjacent planes of a page per stage (one load
    from the pool for all of them on a gather, one store for a full page on a scatter)."""
    old = native.bikv_get_tuning(b"bulk_span")
    try:
        assert native.bikv_set_tuning(b"bulk_span", span) == 0
        run_case(cuda, SMALL, 3, 11, 7, 6 * 16, N.VARIANT_BULK, seed=span)            # 6 planes: ragged last group
        run_case(cuda, B.GEO_B, 1, 64, 4, 200, N.VARIANT_BULK, seed=span + 1)
        run_case(cuda, TINY, 1, 16, 3, 30, N.VARIANT_BULK, seed=span + 2)
        run_case(cuda, GEOS["C-lite"], 1, 32, 3, 100, N.VARIANT_BULK, seed=span + 3)  # planes in 2 parts: span ignored
        for tail in (1, 7, 15):
            run_case(cuda, SMALL, 1, 8, 1, 16 + tail, N.VARIANT_BULK, seed=tail, min_tokens=16 + tail)
    finally:
        native.bikv_set_tuning(b"bulk_span", old)


def test_request_tables_are_reused_only_for_the_same_live_tensors(cuda):
    """A serving loop hands the mover the same KV tensors again and again: their request
    table is built once.  New tensors -- even at recycled addresses or object ids -- get a
    new one."""
    g = SMALL
    shards_cpu = make_shards(g, 1, 24, 4)
    pool = B.ShardedPool.single(shards_cpu[0].to(cuda), g)
    mover = B.PageMover(cuda)
    plan = build_plan([[3, 9], [5]], [30, 16], g.page_tokens, item_request=[0, 1], n_requests=2)
    recs = [tuple(r) for r in plan.table.tolist()]
    want = make_workers(g, [30, 16])
    O.gather(shards_cpu, g, recs, want)
    out = make_workers(g, [30, 16], cuda)
    first = mover.request_table(g, out).clone()
    kept = mover.request_table(g, out)
    assert mover.request_table(g, out) is kept and torch.equal(kept, first)      # the same objects: the kept table
    assert not torch.equal(mover.request_table(g, list(reversed(out))), first)
    for _ in range(3):
        for t in out:
            t.zero_()
        mover.gather(pool, plan, out)
        torch.cuda.synchronize()
        assert all(equal_bits(a, b) for a, b in zip(out, want))
    for _ in range(5):                                              # fresh tensors each time, old ones dropped
        out = make_workers(g, [30, 16], cuda)
        mover.gather(pool, plan, out)
        torch.cuda.synchronize()
        assert all(equal_bits(a, b) for a, b in zip(out, want))
        del out
    mover.check_status()


def test_one_mover_shared_by_threads_on_their_own_streams(cuda):
    """The reference serves its data methods from a 20-thread gRPC pool
    (distributed_grpc_init.py:127,144).  Eight threads share one PageMover, each on its own
    stream with its own pool, plans of changing size and both kernel variants."""
    import threading
    geom = SMALL
    n_threads, rounds, pages = 8, 6, 40
    mover = B.PageMover(cuda)
    errors = []

    def work(tid):
        try:
            stream = torch.cuda.Stream(device=cuda)
            rng = np.random.default_rng(100 + tid)
            shard_cpu = make_shards(geom, 1, pages, 50 + tid, fill="bits")[0]
            with torch.cuda.stream(stream):
                shard = shard_cpu.to(cuda)
            pool = B.ShardedPool.single(shard, geom)
            for r in range(rounds):
                n_req = int(rng.integers(1, 5))
                lists, tokens = random_plan(rng, geom, pages, n_req, (pages // n_req) * geom.page_tokens)
                plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), geom.page_tokens,
                                  item_request=np.arange(n_req, dtype=np.int32), n_requests=n_req)
                recs = [tuple(x) for x in plan.table.tolist()]
                variant = (N.VARIANT_LDST, N.VARIANT_BULK)[(tid + r) % 2]
                with torch.cuda.stream(stream):
                    out = make_workers(geom, tokens, cuda)
                    mover.gather(pool, plan, out, variant=variant, stream=stream)
                    src_cpu = make_workers(geom, tokens, fill="normal", seed=1000 * tid + r)
                    src = [t.to(cuda, non_blocking=False) for t in src_cpu]
                    mover.scatter(pool, plan, src, variant=variant, stream=stream)
                stream.synchronize()
                want = make_workers(geom, tokens)
                O.gather([shard_cpu], geom, recs, want)
                for a, b in zip(out, want):
                    assert equal_bits(a, b), (tid, r)
                O.scatter([shard_cpu], geom, recs, src_cpu)
                assert equal_bits(shard, shard_cpu), (tid, r)
        except Exception as e:  # noqa: BLE001
            errors.append((tid, repr(e)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(n_threads)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    mover.check_status()
    assert not errors, errors
