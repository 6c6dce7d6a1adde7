"""The C-ABI library loads on a machine without a GPU and exports every symbol the
header declares; host-only entry points behave."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from bikv_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for header in ("bikv.h", "bikv_pm.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(bikv_[a-z_0-9]+)\s*\(", text))
    return sorted(names)


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(N.SIGNATURES)


def test_every_declared_symbol_is_exported(native):
    for name in declared_symbols():
        assert hasattr(native, name), name


def test_version_and_strerror(native):
    assert native.bikv_version() == 1
    assert native.bikv_strerror(0) == b"ok"
    for code in range(-10, 0):
        assert native.bikv_strerror(code) not in (b"", b"unknown status")
    assert native.bikv_strerror(-99) == b"unknown status"


def test_worker_base_rule(native):
    """The predicate the kernels apply to a worker-side base before forming an address."""
    f = native.bikv_check_worker_base
    assert f(None) == N.ERR_BAD_ARG
    for ok in (16, 4096, 0x7F0000000010, (1 << 47) - 16):
        assert f(C.c_void_p(ok)) == 0
    for off in range(1, 16):
        assert f(C.c_void_p(0x7F0000000000 + off)) == N.ERR_ALIGNMENT, off


def test_owner_split_through_the_c_abi(native):
    import ctypes as C
    t0 = np.array([[0, 16, 0, 0], [1, 16, 0, 16], [2, 16, 1, 0], [4, 5, 1, 16]], dtype=np.int32)
    t1 = np.array([[6, 16, 0, 0], [3, 16, 0, 16]], dtype=np.int32)
    ptrs = (C.c_void_p * 2)(t0.ctypes.data, t1.ctypes.data)
    rows = np.array([4, 2], dtype=np.int64)
    reqs = np.array([2, 1], dtype=np.int32)
    out = np.zeros((6, 4), dtype=np.int32)
    call = lambda owner, cap=6, rule=N.SHARD_MOD, shards=2: native.bikv_plan_split_by_owner(
        ptrs, rows.ctypes.data_as(C.c_void_p), reqs.ctypes.data_as(C.c_void_p), 2, owner, shards, 8, rule,
        out.ctypes.data_as(C.c_void_p), cap)
    assert call(0) == 4                    # pages 0, 2, 4 of worker 0 and page 6 of worker 1
    assert sorted(out[:4, 0].tolist()) == [0, 2, 4, 6]
    assert out[out[:, 0] == 6][0].tolist() == [6, 16, 2, 0]           # worker 1's request 0 -> 2
    assert [r for r in out[:4, 0].tolist() if r != 6] == [0, 2, 4]    # worker 0's order kept
    assert call(1) == 2 and sorted(out[:2, 0].tolist()) == [1, 3]
    assert call(0, cap=3) == N.ERR_TOO_LARGE
    assert call(2) == N.ERR_BAD_ARG and call(0, shards=0) == N.ERR_BAD_ARG and call(0, rule=7) == N.ERR_BAD_ARG
    assert call(0, rule=N.SHARD_BLOCK) == 6 and call(1, rule=N.SHARD_BLOCK) == 0     # every id < pages_per_shard


def test_tuning_knobs(native):
    assert native.bikv_set_tuning(b"nope", 1) == N.ERR_BAD_ARG
    old = native.bikv_get_tuning(b"bulk_stages")
    assert native.bikv_set_tuning(b"bulk_stages", 3) == 0
    assert native.bikv_get_tuning(b"bulk_stages") == 3
    assert native.bikv_set_tuning(b"bulk_stages", 1000) == N.ERR_BAD_ARG
    assert native.bikv_set_tuning(b"seg_bytes", 1000) == N.ERR_BAD_ARG
    native.bikv_set_tuning(b"bulk_stages", old)


def test_every_knob_the_header_names_exists(native):
    import os
    import re
    header = open(os.path.join(N.INCLUDE, "bikv.h")).read()
    block = header[header.index("Tuning knobs:"):header.index("int bikv_set_tuning")]
    names = re.findall(r'"([a-z0-9_]+)"', block)
    assert len(names) >= 10
    for name in names:
        value = native.bikv_get_tuning(name.encode())
        assert value >= 0, name
        assert native.bikv_set_tuning(name.encode(), value) == 0, name


def test_scratch_bytes(native):
    assert native.bikv_plan_scratch_bytes(0, 0) == 0
    assert native.bikv_plan_scratch_bytes(1, 1) == 512
    assert native.bikv_plan_scratch_bytes(17, 3) == 512 + 256
    assert native.bikv_plan_scratch_bytes(-1, 0) == N.ERR_BAD_ARG


def _pool(n_shards=1, pages=64, base=0x10000):
    p = N.PoolDesc()
    for s in range(n_shards):
        p.shard_base[s] = base + s * 0x100000
    p.n_shards, p.shard_rule, p.pages_per_shard = n_shards, N.SHARD_MOD, pages
    return p


def _validate(native, table, req_tokens, pool=None, geom=None, overlap=0, bases=None):
    table = np.ascontiguousarray(table, dtype=np.int32).reshape(-1, 4)
    reqs = (N.RequestDesc * len(req_tokens))()
    for i, t in enumerate(req_tokens):
        reqs[i].base = (bases[i] if bases else 0x200000 + 0x1000 * i)
        reqs[i].tokens = t
    pool = pool or _pool()
    geom = geom or N.Geometry(2, 2, 64, 16, 2, N.POOL_PAGED)
    return native.bikv_plan_validate(table.ctypes.data_as(C.c_void_p), len(table), reqs, len(req_tokens),
                                     C.byref(pool), C.byref(geom), overlap)


def test_validate_accepts_good_plan(native):
    assert _validate(native, [[0, 16, 0, 0], [5, 3, 0, 16]], [19]) == 0


@pytest.mark.parametrize("table,req_tokens,expect", [
    ([[64, 16, 0, 0]], [16], N.ERR_PAGE_RANGE),
    ([[-1, 16, 0, 0]], [16], N.ERR_PAGE_RANGE),
    ([[0, 0, 0, 0]], [16], N.ERR_PLAN),
    ([[0, 17, 0, 0]], [32], N.ERR_PLAN),
    ([[0, 16, 1, 0]], [16], N.ERR_BAD_ARG),
    ([[0, 16, 0, 1]], [16], N.ERR_DST_RANGE),
    ([[0, 16, 0, -1]], [16], N.ERR_DST_RANGE),
])
def test_validate_rejects(native, table, req_tokens, expect):
    assert _validate(native, table, req_tokens) == expect


def test_validate_overlap_only_when_asked(native):
    t = [[3, 16, 0, 0], [3, 16, 0, 16]]
    assert _validate(native, t, [32], overlap=0) == 0
    assert _validate(native, t, [32], overlap=1) == N.ERR_OVERLAP


def test_validate_geometry_and_pool(native):
    good = [[0, 16, 0, 0]]
    assert _validate(native, good, [16], geom=N.Geometry(2, 1, 4, 16, 2, N.POOL_PAGED)) == N.ERR_ALIGNMENT
    assert _validate(native, good, [16], geom=N.Geometry(2, 1, 4, 16, 2, N.POOL_TOKEN_MAJOR)) == N.ERR_ALIGNMENT
    assert _validate(native, good, [16], geom=N.Geometry(0, 2, 64, 16, 2, N.POOL_PAGED)) == N.ERR_BAD_ARG
    assert _validate(native, good, [16], geom=N.Geometry(2, 2, 64, 16, 3, N.POOL_PAGED)) == N.ERR_BAD_ARG
    assert _validate(native, good, [16], pool=_pool(base=0x10008)) == N.ERR_ALIGNMENT
    assert _validate(native, good, [16], bases=[0x200004]) == N.ERR_ALIGNMENT
    bad = _pool()
    bad.n_shards = 17
    assert _validate(native, good, [16], pool=bad) == N.ERR_BAD_ARG


def test_empty_plan_is_ok_everywhere(native):
    pool, geom = _pool(), N.Geometry(2, 2, 64, 16, 2, N.POOL_PAGED)
    assert native.bikv_plan_validate(None, 0, None, 0, C.byref(pool), C.byref(geom), 1) == 0
    # zero pages: no launch, no CUDA call, so this works without a GPU
    assert native.bikv_gather(C.byref(pool), C.byref(geom), None, 0, None, 0, 0, None, None) == 0
    assert native.bikv_scatter(C.byref(pool), C.byref(geom), None, 0, None, 0, 0, None, None) == 0
    assert native.bikv_copy_pages_flat(None, None, None, None, 0, 100, 2, None) == 0


def test_bad_arguments_fail_before_any_cuda_call(native):
    pool, geom = _pool(), N.Geometry(2, 2, 64, 16, 2, N.POOL_PAGED)
    assert native.bikv_gather(None, C.byref(geom), None, 1, None, 1, 0, None, None) == N.ERR_BAD_ARG
    assert native.bikv_gather(C.byref(pool), None, None, 1, None, 1, 0, None, None) == N.ERR_BAD_ARG
    assert native.bikv_gather(C.byref(pool), C.byref(geom), None, 1, None, 1, 0, None, None) == N.ERR_BAD_ARG
    assert native.bikv_gather(C.byref(pool), C.byref(geom), None, -1, None, 1, 0, None, None) == N.ERR_BAD_ARG
    assert native.bikv_copy_pages_flat(None, None, None, None, 1, 100, 2, None) == N.ERR_BAD_ARG
    assert native.bikv_copy_pages_flat(None, None, None, None, 1, 100, 0, None) == N.ERR_BAD_ARG
