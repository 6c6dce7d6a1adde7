"""Flat page copy (the reference kernel's semantics) and the reference's token-major
pool layout, against the oracle."""
import numpy as np
import pytest
import torch

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import build_plan
from oracle import bikv_oracle as O

from helpers import equal_bits, make_shards, make_workers, normal, random_plan

pytestmark = pytest.mark.gpu


def test_reference_identity_check(cuda):
    """The reference's own check (test_page_ipc.py:41-65,127-150): 200 pages of 50 tokens,
    constant 7, identity page map -> 5-D shape kept and every element still 7."""
    g = B.GEO_R
    pages, P = 200, 50
    src = torch.full((pages, P) + g.token_shape, 7, dtype=torch.float16, device=cuda)
    dst = torch.zeros_like(src)
    off = torch.arange(pages, dtype=torch.int64, device=cuda) * (P * g.token_elems)
    B.PageMover(cuda).copy_pages_flat(src, dst, off, off, P * g.token_elems)
    out = dst.view((pages * P,) + g.token_shape)
    assert out.dim() == 5 and tuple(out.shape) == (10000, 128, 2, 28, 2)
    assert torch.allclose(out, torch.full_like(out, 7))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32, torch.uint8])
@pytest.mark.parametrize("page_elems,shift", [(4096, 0), (1000, 0), (777, 1), (50 * 14336, 0), (333, 3), (8, 5)])
def test_flat_copy_random_maps(cuda, dtype, page_elems, shift):
    """Random permutation page map, element offsets with arbitrary alignment."""
    rng = np.random.default_rng(page_elems + shift)
    n_pages, pool_pages = 13, 40
    stride = page_elems + 11
    src = normal((pool_pages * stride + 64,), torch.float32, 1).to(dtype)
    src_off = (rng.permutation(pool_pages)[:n_pages] * stride + shift).astype(np.int64)
    dst_off = (rng.permutation(n_pages) * stride + (shift * 2) % 7).astype(np.int64)
    dst_ref = torch.zeros(n_pages * stride + 64, dtype=dtype)
    O.copy_pages_flat(src, dst_ref, src_off.tolist(), dst_off.tolist(), page_elems)
    dst = torch.zeros_like(dst_ref, device=cuda)
    B.PageMover(cuda).copy_pages_flat(src.to(cuda), dst, torch.from_numpy(src_off).to(cuda),
                                      torch.from_numpy(dst_off).to(cuda), page_elems)
    assert equal_bits(dst, dst_ref)


def test_flat_copy_from_pinned_host(cuda):
    """Source in pinned host memory (the reference's zero_copy_page_kernel)."""
    page_elems, n = 4096, 9
    src = normal((32 * page_elems,), torch.float16, 2).pin_memory()
    rng = np.random.default_rng(0)
    src_off = (rng.permutation(32)[:n] * page_elems).astype(np.int64)
    dst_off = (np.arange(n) * page_elems).astype(np.int64)
    ref = torch.zeros(n * page_elems, dtype=torch.float16)
    O.copy_pages_flat(src, ref, src_off.tolist(), dst_off.tolist(), page_elems)
    dst = torch.zeros_like(ref, device=cuda)
    B.PageMover(cuda).copy_pages_flat(src, dst, torch.from_numpy(src_off).to(cuda),
                                      torch.from_numpy(dst_off).to(cuda), page_elems)
    assert equal_bits(dst, ref)


def test_copy_range(cuda):
    src = normal((1 << 20,), torch.float16, 3).to(cuda)
    dst = torch.zeros_like(src)
    m = B.PageMover(cuda)
    m.copy_range(dst.data_ptr() + 2, src.data_ptr() + 6, 2 * (1 << 20) - 64)
    assert equal_bits(dst[1:1 + (1 << 20) - 32], src[3:3 + (1 << 20) - 32])
    assert int(dst[0]) == 0


TM = N.POOL_TOKEN_MAJOR
TM_GEOS = {
    "R50": B.GEO_R,
    "R16": KVGeometry(28, 2, 128, 16, torch.float16, TM),
    "B": KVGeometry(28, 4, 128, 16, torch.bfloat16, TM),        # 2 slabs
    "C-lite": KVGeometry(80, 8, 128, 4, torch.float16, TM),     # slabs of 64 d x 1 head
    "C": KVGeometry(80, 8, 128, 16, torch.float16, TM),         # configuration 3's full geometry, 5 MiB pages
    "H6": KVGeometry(40, 6, 128, 4, torch.bfloat16, TM),        # slabs of 64 d x 3 heads
    "d64": KVGeometry(24, 2, 64, 16, torch.float16, TM),        # one slab per token
    "d96": KVGeometry(12, 3, 96, 5, torch.float16, TM),         # 12 d-groups: slab rows not a multiple of 8
    "tiny": KVGeometry(1, 1, 8, 3, torch.float16, TM),
    "odd": KVGeometry(3, 3, 24, 5, torch.bfloat16, TM),
    "f32": KVGeometry(2, 2, 8, 4, torch.float32, TM),
    "u8": KVGeometry(2, 3, 32, 4, torch.uint8, TM),
}


@pytest.fixture(params=[1, 0], ids=["one_item_per_cta", "persistent_ring"])
def tm_mode(request, native):
    """Both forms of the 16-byte-unit kernel: one item per CTA (the default) and persistent CTAs
    with a cp.async ring."""
    old = native.bikv_get_tuning(b"tm_single")
    assert native.bikv_set_tuning(b"tm_single", request.param) == 0
    yield request.param
    native.bikv_set_tuning(b"tm_single", old)


@pytest.mark.parametrize("geo", TM_GEOS)
@pytest.mark.parametrize("n_shards", [1, 3])
def test_token_major_gather_scatter(cuda, geo, n_shards, tm_mode):
    g = TM_GEOS[geo]
    rng = np.random.default_rng(len(geo) + n_shards)
    per = 6
    lists, tokens = random_plan(rng, g, n_shards * per, 3, 3 * g.page_tokens)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), g.page_tokens,
                      item_request=np.arange(3, dtype=np.int32), n_requests=3)
    recs = [tuple(r) for r in plan.table.tolist()]
    shards_cpu = make_shards(g, n_shards, per, 9, fill="bits")
    shards_gpu = [s.to(cuda) for s in shards_cpu]
    pool = B.ShardedPool.from_tensors(shards_gpu, g)
    mover = B.PageMover(cuda)
    out = make_workers(g, tokens, cuda)
    mover.gather(pool, plan, out)
    ref = make_workers(g, tokens)
    O.gather(shards_cpu, g, recs, ref)
    for a, b in zip(out, ref):
        assert equal_bits(a, b)
    src_cpu = make_workers(g, tokens, fill="normal", seed=77)
    mover.scatter(pool, plan, [t.to(cuda) for t in src_cpu])
    O.scatter(shards_cpu, g, recs, src_cpu)
    for a, b in zip(shards_gpu, shards_cpu):
        assert equal_bits(a, b)


@pytest.mark.parametrize("staged", [0, 1])
@pytest.mark.parametrize("tile_kib,split_kib,threads", [(8, 8, 0), (8, 16, 64), (16, 32, 96), (100, 100, 256), (48, 96, 0)])
@pytest.mark.parametrize("geo", ["R16", "R50", "B", "H6", "C-lite", "d96"])
def test_token_major_slab_shapes(cuda, native, geo, tile_kib, split_kib, threads, staged, tm_mode):
    """The slab of the 16-byte transposing kernel (d-groups x heads) follows the tile caps;
    every shape, CTA size and scatter mode moves the same bytes."""
    g = TM_GEOS[geo]
    knobs = {b"tm_tile_kib": tile_kib, b"tm_split_tile_kib": split_kib, b"tm_threads": threads,
             b"tm_scatter_staged": staged, b"tm_gather_stages": 2 + staged,
             b"tm_scatter_stages": 3 if threads in (0, 96) else 2}
    old = {k: native.bikv_get_tuning(k) for k in knobs}
    for k, v in knobs.items():
        assert native.bikv_set_tuning(k, v) == 0
    try:
        rng = np.random.default_rng(tile_kib)
        lists, tokens = random_plan(rng, g, 10, 2, 3 * g.page_tokens)
        plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), g.page_tokens,
                          item_request=np.arange(2, dtype=np.int32), n_requests=2)
        recs = [tuple(r) for r in plan.table.tolist()]
        shards_cpu = make_shards(g, 1, 10, 4, fill="bits")
        shards_gpu = [s.to(cuda) for s in shards_cpu]
        pool = B.ShardedPool.from_tensors(shards_gpu, g)
        mover = B.PageMover(cuda)
        out = make_workers(g, tokens, cuda)
        mover.gather(pool, plan, out)
        ref = make_workers(g, tokens)
        O.gather(shards_cpu, g, recs, ref)
        for a, b in zip(out, ref):
            assert equal_bits(a, b)
        src_cpu = make_workers(g, tokens, fill="bits", seed=5)
        mover.scatter(pool, plan, [t.to(cuda) for t in src_cpu])
        O.scatter(shards_cpu, g, recs, src_cpu)
        torch.cuda.synchronize()
        assert equal_bits(shards_gpu[0], shards_cpu[0])
    finally:
        for k, v in old.items():
            native.bikv_set_tuning(k, v)


def test_token_major_equals_paged_after_conversion(cuda):
    """The same logical pool in both layouts gathers to the same worker tensors."""
    gp = KVGeometry(28, 2, 128, 16, torch.float16)
    gt = gp.with_layout(TM)
    n = 12
    paged = normal(gp.pool_shape(n), gp.dtype, 5)                         # [n, L, 2, P, H, D]
    token_major = paged.permute(0, 3, 5, 4, 1, 2).contiguous().view(gt.pool_shape(n))
    rng = np.random.default_rng(1)
    lists, tokens = random_plan(rng, gp, n, 2, 80)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), 16,
                      item_request=np.arange(2, dtype=np.int32), n_requests=2)
    mover = B.PageMover(cuda)
    a = make_workers(gp, tokens, cuda)
    b = make_workers(gp, tokens, cuda)
    mover.gather(B.ShardedPool.single(paged.to(cuda), gp), plan, a)
    mover.gather(B.ShardedPool.single(token_major.to(cuda), gt), plan, b)
    for x, y in zip(a, b):
        assert equal_bits(x, y)
