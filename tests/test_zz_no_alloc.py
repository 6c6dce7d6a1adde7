"""bikv_gather_h_static: the gather for callers that cannot allocate device memory.

Some users of this library cannot call cudaMalloc on the transfer path: a serving
engine that has already handed all of HBM to its KV pool has nothing left to give, and
a request handler must not trigger the device-wide synchronisation an allocation or a
free implies.  For them the library carries its own fixed plan staging area and this
entry point uses it.  The test drives the entry point through the C ABI (ctypes, raw
pointers) twice in a row -- the second plan is shorter, so the staging area still
holds the tail of the first -- and requires the worker tensors to equal, bit for bit,
what the ordinary entry point (bikv_gather_h with a caller-provided staging buffer)
produces for the same plans, and what the CPU oracle computes from the same pool and plan,
so the check does not hang on the entry point it mirrors.  This file sorts last so that a run which stops at the
first failure has already run every other test; it does not depend on them.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from oracle import bikv_oracle as O

pytestmark = pytest.mark.gpu


def _plan(rng, geom, total_pages, n_requests, max_tokens):
    tokens = rng.integers(1, max_tokens + 1, size=n_requests)
    counts = (tokens + geom.page_tokens - 1) // geom.page_tokens
    perm = rng.permutation(total_pages)[: int(counts.sum())]
    rows, at = [], 0
    for r, (t, c) in enumerate(zip(tokens, counts)):
        for k in range(int(c)):
            valid = geom.page_tokens if k < c - 1 or t % geom.page_tokens == 0 else int(t % geom.page_tokens)
            rows.append((int(perm[at]), valid, r, k * geom.page_tokens))
            at += 1
    return np.array(rows, dtype=np.int32), tokens


def _gather(lib, fn_name, pool, geom, table, tensors, dev, scratch=None):
    g = geom.native()
    reqs = (N.RequestDesc * len(tensors))()
    for i, t in enumerate(tensors):
        reqs[i].base = t.data_ptr()
        reqs[i].tokens = t.shape[2]
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    recs = C.c_void_p(table.ctypes.data)
    if fn_name == "static":
        rc = lib.bikv_gather_h_static(C.byref(pool), C.byref(g), recs, len(table), reqs, len(tensors), 1,
                                      N.VARIANT_LDST, None, stream)
    else:
        rc = lib.bikv_gather_h(C.byref(pool), C.byref(g), recs, len(table), reqs, len(tensors),
                               C.c_void_p(scratch.data_ptr()), scratch.numel(), 1, N.VARIANT_LDST, None, stream)
    torch.cuda.synchronize(dev)   # the host arrays above must outlive the upload
    return rc


def test_static_gather_matches_ordinary_gather_twice(native, cuda):
    geom = KVGeometry(4, 2, 64, 16, torch.bfloat16)
    n_pages = 256
    gen = torch.Generator().manual_seed(42)
    shard_cpu = torch.randn(geom.pool_shape(n_pages), generator=gen).to(geom.dtype)
    shard = shard_cpu.to(cuda)
    pool = N.PoolDesc()
    pool.shard_base[0] = shard.data_ptr()
    pool.n_shards, pool.shard_rule, pool.pages_per_shard = 1, N.SHARD_MOD, n_pages
    scratch = torch.empty(1 << 16, dtype=torch.uint8, device=cuda)
    rng = np.random.default_rng(7)
    launches = native.bikv_launch_count()
    for call, (n_req, max_tok) in enumerate([(9, 300), (3, 40)]):
        table, tokens = _plan(rng, geom, n_pages, n_req, max_tok)
        want = [torch.zeros(geom.worker_shape(int(t)), dtype=geom.dtype, device=cuda) for t in tokens]
        got = [torch.zeros_like(t) for t in want]
        assert _gather(native, "ordinary", pool, geom, table, want, cuda, scratch) == 0
        assert _gather(native, "static", pool, geom, table, got, cuda) == 0
        oracle = [torch.zeros(geom.worker_shape(int(t)), dtype=geom.dtype) for t in tokens]
        O.gather([shard_cpu], geom, [tuple(r) for r in table.tolist()], oracle)
        for a, b, c in zip(got, want, oracle):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16)), f"call {call}"
            assert torch.equal(a.cpu().view(torch.int16), c.view(torch.int16)), f"call {call} against the oracle"
        assert any(int(t.view(torch.int16).ne(0).sum()) > 0 for t in got)
    assert native.bikv_launch_count() - launches == 4


def test_static_gather_with_an_empty_plan_is_the_start_up_call(native, cuda):
    """n_pages == 0 launches nothing but still resolves the staging array's address on the
    device: the call an engine makes at start-up, before it reserves HBM."""
    geom = KVGeometry(2, 2, 64, 16, torch.float16)
    shard = torch.zeros(geom.pool_shape(4), dtype=geom.dtype, device=cuda)
    pool = N.PoolDesc()
    pool.shard_base[0] = shard.data_ptr()
    pool.n_shards, pool.shard_rule, pool.pages_per_shard = 1, N.SHARD_MOD, 4
    g = geom.native()
    launches = native.bikv_launch_count()
    assert native.bikv_gather_h_static(C.byref(pool), C.byref(g), None, 0, None, 0, 1, N.VARIANT_LDST, None, None) == 0
    assert native.bikv_launch_count() == launches


def test_static_gather_refuses_oversized_plans(native, cuda):
    geom = KVGeometry(2, 2, 64, 16, torch.float16)
    shard = torch.zeros(geom.pool_shape(4), dtype=geom.dtype, device=cuda)
    pool = N.PoolDesc()
    pool.shard_base[0] = shard.data_ptr()
    pool.n_shards, pool.shard_rule, pool.pages_per_shard = 1, N.SHARD_MOD, 4
    g = geom.native()
    out = torch.zeros(geom.worker_shape(16), dtype=geom.dtype, device=cuda)
    reqs = (N.RequestDesc * 1)()
    reqs[0].base, reqs[0].tokens = out.data_ptr(), 16
    table = np.zeros((N.STATIC_MAX_PAGES + 1, 4), dtype=np.int32)
    launches = native.bikv_launch_count()
    rc = native.bikv_gather_h_static(C.byref(pool), C.byref(g), C.c_void_p(table.ctypes.data), len(table), reqs, 1,
                                     1, N.VARIANT_LDST, None, None)
    assert rc == N.ERR_TOO_LARGE
    assert b"maximum" in native.bikv_strerror(rc)
    rc = native.bikv_gather_h_static(C.byref(pool), C.byref(g), C.c_void_p(table.ctypes.data), 1, reqs,
                                     N.STATIC_MAX_REQUESTS + 1, 1, N.VARIANT_LDST, None, None)
    assert rc == N.ERR_TOO_LARGE
    assert native.bikv_launch_count() == launches
