"""ctypes binding of ``libbikv.so`` (the C ABI declared in ``include/bikv.h``).

The library is built in-tree by :func:`build` (``nvcc`` for ``sm_100a``) and is
the only implementation of the data path: there is no CPU or torch fallback.
If the shared object is missing, :func:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
INCLUDE = os.path.normpath(os.path.join(_HERE, "..", "include"))
# BIKV_LIB points at an alternative build of the library (measurement and debugging).
LIB_PATH = os.environ.get("BIKV_LIB") or os.path.join(CSRC, "libbikv.so")
SOURCES = ["bikv.cu", "bikv_pm.cpp"]
HEADERS = ["bikv_kernels.cuh"]

MAX_SHARDS = 16

OK = 0
ERR_BAD_ARG = -1
ERR_PAGE_RANGE = -2
ERR_DST_RANGE = -3
ERR_ALIGNMENT = -4
ERR_PEER = -5
ERR_CUDA = -6
ERR_OVERLAP = -7
ERR_DEVICE_TIMEOUT = -8
ERR_TOO_LARGE = -9
ERR_PLAN = -10

POOL_PAGED = 0
POOL_TOKEN_MAJOR = 1
SHARD_MOD = 0
SHARD_BLOCK = 1
VARIANT_AUTO = 0
VARIANT_LDST = 1
VARIANT_BULK = 2
STATIC_MAX_PAGES = 32768
STATIC_MAX_REQUESTS = 1024


class Geometry(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32),
        ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("page_tokens", C.c_int32),
        ("elt_bytes", C.c_int32),
        ("pool_layout", C.c_int32),
    ]


class PageRec(C.Structure):
    _fields_ = [
        ("page_id", C.c_int32),
        ("valid_tokens", C.c_int32),
        ("request", C.c_int32),
        ("token_offset", C.c_int32),
    ]


class RequestDesc(C.Structure):
    _fields_ = [("base", C.c_void_p), ("tokens", C.c_int64)]


class PoolDesc(C.Structure):
    _fields_ = [
        ("shard_base", C.c_void_p * MAX_SHARDS),
        ("n_shards", C.c_int32),
        ("shard_rule", C.c_int32),
        ("pages_per_shard", C.c_int64),
    ]


# name -> (restype, argtypes); every symbol include/bikv.h declares.
_P = C.c_void_p
SIGNATURES = {
    "bikv_version": (C.c_int, []),
    "bikv_strerror": (C.c_char_p, [C.c_int]),
    "bikv_last_cuda_error": (C.c_int, []),
    "bikv_launch_count": (C.c_int64, []),
    "bikv_set_tuning": (C.c_int, [C.c_char_p, C.c_int64]),
    "bikv_get_tuning": (C.c_int64, [C.c_char_p]),
    "bikv_plan_build": (
        C.c_int64,
        [_P, _P, _P, _P, _P, C.c_int64, C.c_int32, C.c_int32, _P, C.c_int32, _P, C.c_int64],
    ),
    "bikv_plan_validate": (
        C.c_int,
        [_P, C.c_int64, _P, C.c_int32, C.POINTER(PoolDesc), C.POINTER(Geometry), C.c_int],
    ),
    "bikv_check_worker_base": (C.c_int, [_P]),
    "bikv_plan_split_by_owner": (C.c_int64, [_P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32, _P,
                                             C.c_int64]),
    "bikv_gather": (
        C.c_int,
        [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int32, C.c_int, _P, _P],
    ),
    "bikv_scatter": (
        C.c_int,
        [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int32, C.c_int, _P, _P],
    ),
    "bikv_plan_scratch_bytes": (C.c_int64, [C.c_int64, C.c_int32]),
    "bikv_gather_h": (
        C.c_int,
        [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int32, _P, C.c_int64,
         C.c_int, C.c_int, _P, _P],
    ),
    "bikv_scatter_h": (
        C.c_int,
        [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int32, _P, C.c_int64,
         C.c_int, C.c_int, _P, _P],
    ),
    "bikv_gather_nhd": (C.c_int, [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int64, _P, _P]),
    "bikv_scatter_nhd": (C.c_int, [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int64, _P, _P]),
    "bikv_plan_validate_nhd": (C.c_int, [_P, C.c_int64, C.c_int64, C.POINTER(PoolDesc), C.POINTER(Geometry), C.c_int]),
    "bikv_gather_h_static": (
        C.c_int,
        [C.POINTER(PoolDesc), C.POINTER(Geometry), _P, C.c_int64, _P, C.c_int32, C.c_int, C.c_int, _P, _P],
    ),
    "bikv_copy_pages_flat": (C.c_int, [_P, _P, _P, _P, C.c_int64, C.c_int64, C.c_int32, _P]),
    "bikv_copy_range": (C.c_int, [_P, _P, C.c_int64, _P]),
    "bikv_copy_range_engine": (C.c_int, [_P, _P, C.c_int64, _P]),
    "bikv_host_register": (C.c_int, [_P, C.c_int64]),
    "bikv_host_unregister": (C.c_int, [_P]),
    "bikv_selftest_wait_timeout": (C.c_int, [_P, C.c_int64, _P]),
    "bikv_can_access_peer": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "bikv_enable_peer": (C.c_int, [C.c_int, C.c_int]),
    "bikv_pool_export": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_int64)]),
    "bikv_pool_import": (C.c_int, [C.c_char_p, C.c_int64, C.POINTER(_P)]),
    "bikv_pool_close": (C.c_int, [_P, C.c_int64]),
    # include/bikv_pm.h
    "bikv_pm_create": (_P, [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_uint64]),
    "bikv_pm_destroy": (None, [_P]),
    "bikv_pm_configure_tiers": (C.c_int, [_P, C.c_int64, C.c_int64]),
    "bikv_pm_load_item": (C.c_int64, [_P, C.c_int64, C.c_int64, C.c_int32, C.c_int32, _P, _P, C.c_int64, _P, _P,
                                      C.c_int64, _P]),
    "bikv_pm_access_item": (C.c_int64, [_P, C.c_int64, _P, _P, C.c_int64]),
    "bikv_pm_set_protected": (C.c_int, [_P, C.c_int64]),
    "bikv_pm_remove_protected": (C.c_int, [_P, C.c_int64]),
    "bikv_pm_advance_clock": (C.c_int, [_P, C.c_int64]),
    "bikv_pm_set_clock": (C.c_int, [_P, C.c_int64]),
    "bikv_pm_free_pages": (C.c_int64, [_P, C.c_int32]),
    "bikv_pm_item_count": (C.c_int64, [_P, C.c_int32]),
    "bikv_pm_evictions": (C.c_int64, [_P]),
    "bikv_pm_item_priority": (C.c_int, [_P, C.c_int64]),
    "bikv_pm_plan_prefix_batch": (C.c_int, [_P, _P, _P, _P, C.c_int32, _P, _P, C.c_int64, _P, _P, C.c_int64, _P, _P]),
}
PM_LRU = 0
PM_TIERED = 1
PM_MISS = -100
PM_FULL = -101

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

_lib = None
_lock = threading.Lock()


class BikvError(RuntimeError):
    """A non-zero status from the library (``.status`` holds the code)."""

    def __init__(self, status: int, where: str = ""):
        self.status = int(status)
        msg = {PM_MISS: "item not in the page directory",
               PM_FULL: "page pool full: nothing left to evict"}.get(self.status) or \
            lib().bikv_strerror(self.status).decode()
        if self.status == ERR_CUDA:
            msg += f" [cudaError {lib().bikv_last_cuda_error()}]"
        super().__init__(f"{where + ': ' if where else ''}{msg} ({self.status})")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(INCLUDE, h) for h in
                                                                   ("bikv.h", "bikv_pm.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``libbikv.so`` in-tree for sm_100a; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    tmp = LIB_PATH + f".{os.getpid()}.tmp"        # built aside, then moved into place in one step
    cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-o", tmp]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    if verbose:
        print(res.stderr)
    return LIB_PATH


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: the CUDA library is the only implementation of the "
                    "KV-page path. Build it with `python -c 'import __graft_entry__ as g; g.build()'`."
                )
            l = C.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(l, name)
                fn.restype = res
                fn.argtypes = args
            if l.bikv_version() != 1:
                raise RuntimeError("libbikv.so ABI version mismatch; rebuild it")
            _lib = l
    return _lib


def check(status: int, where: str = "") -> None:
    if status != OK:
        raise BikvError(status, where)
