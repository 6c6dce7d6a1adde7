"""The two restatements of the path -- torch slicing (oracle/bikv_oracle.py) and plain C
(oracle/bikv_oracle.c) -- agree byte for byte on random cases."""
import ctypes as C

import numpy as np
import pytest
import torch

from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from oracle import bikv_oracle as O
from oracle import build_c

from helpers import equal_bits, make_shards, make_workers, random_plan


@pytest.fixture(scope="module")
def clib():
    lib = C.CDLL(build_c.build())
    lib.c_plan_records.restype = C.c_int64
    return lib


def _ptrs(tensors):
    arr = (C.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


@pytest.mark.parametrize("layout", [N.POOL_PAGED, N.POOL_TOKEN_MAJOR])
@pytest.mark.parametrize("rule", [N.SHARD_MOD, N.SHARD_BLOCK])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.uint8])
def test_c_and_torch_oracles_agree(clib, layout, rule, dtype):
    g = KVGeometry(3, 2, 16, 5, dtype, layout)
    rng = np.random.default_rng(layout * 7 + rule)
    n_shards, per = 3, 9
    lists, tokens = random_plan(rng, g, n_shards * per, 4, 23)
    # plan
    flat = np.concatenate(lists).astype(np.int32)
    begin = np.concatenate([[0], np.cumsum([len(l) for l in lists])]).astype(np.int64)
    item_tokens = tokens.astype(np.int32)
    item_req = np.arange(4, dtype=np.int32)
    req_tokens = np.zeros(4, dtype=np.int64)
    recs_c = np.zeros((int(begin[-1]), 4), dtype=np.int32)
    n = clib.c_plan_records(flat.ctypes.data_as(C.c_void_p), begin.ctypes.data_as(C.c_void_p),
                            item_tokens.ctypes.data_as(C.c_void_p), item_req.ctypes.data_as(C.c_void_p),
                            4, g.page_tokens, req_tokens.ctypes.data_as(C.c_void_p), recs_c.ctypes.data_as(C.c_void_p))
    recs = O.plan_records([l.tolist() for l in lists], tokens.tolist(), g.page_tokens, item_request=[0, 1, 2, 3])
    assert n == len(recs) and recs_c.tolist() == [list(r) for r in recs]
    assert req_tokens.tolist() == tokens.tolist()
    # gather
    shards = make_shards(g, n_shards, per, 3, fill="bits")
    want = make_workers(g, tokens)
    O.gather(shards, g, recs, want, rule)
    got = make_workers(g, tokens)
    wtok = tokens.astype(np.int64)
    args = (n_shards, C.c_int64(per), rule, layout, g.n_layers, g.n_kv_heads, g.head_dim, g.page_tokens, g.elt_bytes,
            recs_c.ctypes.data_as(C.c_void_p), C.c_int64(n))
    clib.c_move(_ptrs(shards), *args, _ptrs(got), wtok.ctypes.data_as(C.c_void_p), 0)
    for a, b in zip(got, want):
        assert equal_bits(a, b)
    # scatter
    src = make_workers(g, tokens, fill="normal", seed=8) if dtype != torch.uint8 else \
        [torch.randint(0, 255, g.worker_shape(int(t)), dtype=torch.uint8) for t in tokens]
    a_shards = [s.clone() for s in shards]
    b_shards = [s.clone() for s in shards]
    O.scatter(a_shards, g, recs, src, rule)
    clib.c_move(_ptrs(b_shards), *args, _ptrs(src), wtok.ctypes.data_as(C.c_void_p), 1)
    for a, b in zip(a_shards, b_shards):
        assert equal_bits(a, b)


def test_c_flat_copy_agrees(clib):
    src = torch.randn(4000).to(torch.float16)
    so = np.array([100, 1700, 33], dtype=np.int64)
    do = np.array([900, 0, 2500], dtype=np.int64)
    a, b = torch.zeros(4000, dtype=torch.float16), torch.zeros(4000, dtype=torch.float16)
    O.copy_pages_flat(src, a, so.tolist(), do.tolist(), 777)
    clib.c_copy_pages_flat(C.c_void_p(src.data_ptr()), C.c_void_p(b.data_ptr()), so.ctypes.data_as(C.c_void_p),
                           do.ctypes.data_as(C.c_void_p), C.c_int64(3), C.c_int64(777), 2)
    assert equal_bits(a, b)
