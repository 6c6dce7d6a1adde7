"""Gather/scatter against the worker's paged KV (one [slot, kv, head, dim] tensor per
layer), and a pool shard living in pinned host memory, against the oracle."""
import numpy as np
import pytest
import torch

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import Plan, build_block_plan, build_plan
from oracle import bikv_oracle as O

from helpers import equal_bits, make_shards, make_workers, normal, random_plan

pytestmark = pytest.mark.gpu

GEOS = {"small": KVGeometry(3, 2, 64, 16, torch.bfloat16), "B": B.GEO_B,
        "row16": KVGeometry(2, 1, 8, 4, torch.float16), "A": B.GEO_A}


@pytest.mark.parametrize("geo", GEOS)
@pytest.mark.parametrize("n_shards", [1, 3])
def test_paged_worker_kv(cuda, geo, n_shards):
    g = GEOS[geo]
    rng = np.random.default_rng(len(geo) + n_shards)
    per, n_blocks = 20, 40
    lists, tokens = random_plan(rng, g, n_shards * per, 4, 6 * g.page_tokens)
    n_pages = sum(len(l) for l in lists)
    blocks = rng.permutation(n_blocks)[:n_pages]
    plan = build_block_plan([l.tolist() for l in lists], tokens.astype(np.int32), g.page_tokens, blocks)
    recs = [tuple(r) for r in plan.table.tolist()]
    assert [r[3] for r in recs] == (blocks * g.page_tokens).tolist()
    shards_cpu = make_shards(g, n_shards, per, 5, fill="bits")
    shards_gpu = [s.to(cuda) for s in shards_cpu]
    pool = B.ShardedPool.from_tensors(shards_gpu, g)
    mover = B.PageMover(cuda)
    slots = n_blocks * g.page_tokens
    layers_cpu = [normal((slots, 2, g.n_kv_heads, g.head_dim), g.dtype, 100 + l) for l in range(g.n_layers)]
    layers_gpu = [t.to(cuda) for t in layers_cpu]
    mover.gather_nhd(pool, plan, layers_gpu)
    O.gather_nhd(shards_cpu, g, recs, layers_cpu)
    torch.cuda.synchronize()
    for a, b in zip(layers_gpu, layers_cpu):
        assert equal_bits(a, b)                      # untouched slots keep their contents
    fresh_cpu = [normal(t.shape, g.dtype, 300 + l) for l, t in enumerate(layers_cpu)]
    mover.scatter_nhd(pool, plan, [t.to(cuda) for t in fresh_cpu])
    O.scatter_nhd(shards_cpu, g, recs, fresh_cpu)
    torch.cuda.synchronize()
    for a, b in zip(shards_gpu, shards_cpu):
        assert equal_bits(a, b)


def test_paged_worker_kv_equals_contiguous_gather_reshaped(cuda):
    """Same pages gathered contiguously and into blocks 0..n-1 hold the same tokens."""
    g = B.GEO_A
    pages = [7, 3, 12, 5]
    plan_c = build_plan([pages], [64], 16)
    plan_b = build_block_plan([pages], [64], 16, [0, 1, 2, 3])
    shard = make_shards(g, 1, 16, 2)[0].to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    cont = make_workers(g, [64], cuda)[0]                                   # [L, 2, 64, H, D]
    layers = [torch.zeros(64, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype, device=cuda) for _ in range(g.n_layers)]
    mover.gather(pool, plan_c, cont)
    mover.gather_nhd(pool, plan_b, layers)
    torch.cuda.synchronize()
    assert equal_bits(torch.stack(layers).permute(0, 2, 1, 3, 4), cont)


def test_paged_worker_plan_is_validated(cuda):
    g = GEOS["small"]
    shard = torch.zeros(g.pool_shape(4), dtype=g.dtype, device=cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    layers = [torch.zeros(32, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype, device=cuda) for _ in range(g.n_layers)]
    launches = N.lib().bikv_launch_count()
    for table, status in [([[0, 16, 0, 17]], N.ERR_DST_RANGE), ([[4, 16, 0, 0]], N.ERR_PAGE_RANGE),
                          ([[0, 0, 0, 0]], N.ERR_PLAN), ([[0, 16, 0, -16]], N.ERR_DST_RANGE)]:
        with pytest.raises(B.BikvError) as e:
            mover.gather_nhd(pool, Plan.from_table(np.array(table), 1), layers)
        assert e.value.status == status
    with pytest.raises(B.BikvError) as e:
        mover.scatter_nhd(pool, Plan.from_table(np.array([[1, 16, 0, 0], [1, 16, 0, 16]]), 1), layers)
    assert e.value.status == N.ERR_OVERLAP
    with pytest.raises(ValueError):
        mover.gather_nhd(pool, Plan.from_table(np.array([[0, 16, 0, 0]]), 1), layers[:-1])
    assert N.lib().bikv_launch_count() == launches


def test_pool_shard_in_pinned_host_memory(cuda):
    """Host tier: a shard whose base is pinned (device-mapped) host memory, as the
    reference's default pool placement (kvcache.py:38-43, read by its zero-copy kernel,
    copy_kernel.cu:39-66).  The ld/st kernels read and write it in place over PCIe."""
    g = GEOS["small"]
    rng = np.random.default_rng(0)
    per = 24
    lists, tokens = random_plan(rng, g, 2 * per, 3, 90)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), 16,
                      item_request=np.arange(3, dtype=np.int32), n_requests=3)
    recs = [tuple(r) for r in plan.table.tolist()]
    shards_cpu = make_shards(g, 2, per, 8)
    host_shard = shards_cpu[0].clone().pin_memory()          # shard 0 on the host
    dev_shard = shards_cpu[1].to(cuda)                        # shard 1 in HBM
    pool = B.ShardedPool([host_shard.data_ptr(), dev_shard.data_ptr()], per, g, device=cuda,
                         keepalive=[host_shard, dev_shard])
    mover = B.PageMover(cuda)
    out = make_workers(g, tokens, cuda)
    mover.gather(pool, plan, out, variant=N.VARIANT_LDST)
    ref = make_workers(g, tokens)
    O.gather(shards_cpu, g, recs, ref)
    torch.cuda.synchronize()
    for a, b in zip(out, ref):
        assert equal_bits(a, b)
    src = make_workers(g, tokens, fill="normal", seed=44)
    mover.scatter(pool, plan, [t.to(cuda) for t in src], variant=N.VARIANT_LDST)
    O.scatter(shards_cpu, g, recs, src)
    torch.cuda.synchronize()
    assert equal_bits(host_shard, shards_cpu[0]) and equal_bits(dev_shard, shards_cpu[1])


def test_paged_worker_bad_device_records_are_skipped(cuda):
    import ctypes as C
    g = GEOS["small"]
    shard_cpu = make_shards(g, 1, 6, 3)[0]
    shard = shard_cpu.to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    layers = [torch.zeros(32, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype, device=cuda) for _ in range(g.n_layers)]
    table, slots, _ = mover.layer_table(g, layers)
    recs = torch.tensor([[2, 16, 0, 0], [6, 16, 0, 16], [1, 16, 0, 17], [1, 16, 0, -1], [1, 40, 0, 0]],
                        dtype=torch.int32, device=cuda)
    gn = g.native()
    rc = N.lib().bikv_gather_nhd(C.byref(pool.desc), C.byref(gn), C.c_void_p(recs.data_ptr()), recs.shape[0],
                                 C.c_void_p(table.data_ptr()), slots, C.c_void_p(mover.status.data_ptr()), None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = [torch.zeros(32, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype) for _ in range(g.n_layers)]
    O.gather_nhd([shard_cpu], g, [(2, 16, 0, 0)], ref)
    for a, b in zip(layers, ref):
        assert equal_bits(a, b)
    with pytest.raises(B.BikvError):
        mover.check_status()


def test_paged_worker_bad_layer_bases_are_skipped(cuda):
    """The layer table of a paged worker cache lives in device memory: an entry that is NULL
    or not 16-byte aligned makes the kernel skip that layer's planes; the other layers are
    served and the status word names the error."""
    import ctypes as C
    g = GEOS["small"]
    shard_cpu = make_shards(g, 1, 6, 4)[0]
    shard = shard_cpu.to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    slots = 32
    gn = g.native()
    for bad, want in ((8, N.ERR_ALIGNMENT), (None, N.ERR_BAD_ARG)):
        layers = [torch.zeros(slots + 1, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype, device=cuda)
                  for _ in range(g.n_layers)]
        bases = [t.data_ptr() for t in layers]
        bases[1] = 0 if bad is None else bases[1] + bad
        table = torch.tensor(bases, dtype=torch.int64, device=cuda)
        recs = torch.tensor([[2, 16, 0, 0], [4, 5, 0, 16]], dtype=torch.int32, device=cuda)
        rc = N.lib().bikv_gather_nhd(C.byref(pool.desc), C.byref(gn), C.c_void_p(recs.data_ptr()), recs.shape[0],
                                     C.c_void_p(table.data_ptr()), slots, C.c_void_p(mover.status.data_ptr()), None)
        assert rc == 0
        torch.cuda.synchronize()
        ref = [torch.zeros(slots + 1, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype) for _ in range(g.n_layers)]
        O.gather_nhd([shard_cpu], g, [(2, 16, 0, 0), (4, 5, 0, 16)], ref)
        ref[1].zero_()                                           # the bad layer is left alone
        for a, b in zip(layers, ref):
            assert equal_bits(a, b)
        with pytest.raises(B.BikvError) as e:
            mover.check_status()
        assert e.value.status == want


def test_paged_worker_layers_aligned_to_16_but_not_32_bytes(cuda):
    """With 32-byte accesses switched on (the default) a layer tensor that starts on a 16-byte
    boundary only is still served, in 16-byte accesses."""
    g = GEOS["small"]
    shards_cpu = make_shards(g, 1, 12, 6)
    shard = shards_cpu[0].to(cuda)
    pool = B.ShardedPool.single(shard, g)
    mover = B.PageMover(cuda)
    slots = 48
    row = 2 * g.n_kv_heads * g.head_dim
    backing = [torch.zeros(slots * row + 8, dtype=g.dtype, device=cuda) for _ in range(g.n_layers)]
    layers = [b[8:].view(slots, 2, g.n_kv_heads, g.head_dim) for b in backing]        # +16 bytes
    assert all(t.data_ptr() % 32 == 16 for t in layers)
    plan = Plan.from_table(np.array([[3, 16, 0, 16], [7, 5, 0, 0], [1, 16, 0, 32]]), 1)
    recs = [tuple(r) for r in plan.table.tolist()]
    mover.gather_nhd(pool, plan, layers)
    torch.cuda.synchronize()
    ref = [torch.zeros(slots, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype) for _ in range(g.n_layers)]
    O.gather_nhd(shards_cpu, g, recs, ref)
    for a, b in zip(layers, ref):
        assert equal_bits(a, b)
    fresh = [normal((slots, 2, g.n_kv_heads, g.head_dim), g.dtype, 90 + l) for l in range(g.n_layers)]
    for t, f in zip(layers, fresh):
        t.copy_(f.to(cuda))
    mover.scatter_nhd(pool, plan, layers)
    torch.cuda.synchronize()
    O.scatter_nhd(shards_cpu, g, recs, fresh)
    assert equal_bits(shard, shards_cpu[0])
    mover.check_status()
