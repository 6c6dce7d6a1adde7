"""bikv_b200 -- the KV-page gather/scatter path of Bi-KV for NVIDIA B200.

Host layer (this package) mirrors the reference's call surface for the path;
the data movement itself lives in ``csrc/`` (CUDA for sm_100a behind the C ABI
of ``include/bikv.h``) and has no CPU implementation.
"""
from . import _native
from ._native import (BikvError, POOL_PAGED, POOL_TOKEN_MAJOR, SHARD_BLOCK, SHARD_MOD, VARIANT_AUTO,
                      VARIANT_BULK, VARIANT_LDST, build, lib)
from .geometry import GEO_A, GEO_B, GEO_C, GEO_R, KVGeometry
from .page_directory import PageDirectory, XorShiftChoice
from .page_manager import MultiPageManager, PageManager
from .plan import Plan, build_plan, plan_from_combined_task
from .pool import ShardedPool, global_page_id, shard_of

__all__ = [
    "BikvError", "KVGeometry", "GEO_A", "GEO_B", "GEO_C", "GEO_R", "PageManager", "MultiPageManager", "PageDirectory", "XorShiftChoice",
    "Plan", "build_plan", "plan_from_combined_task", "ShardedPool", "shard_of", "global_page_id",
    "PageMover", "build", "lib", "POOL_PAGED", "POOL_TOKEN_MAJOR", "SHARD_MOD", "SHARD_BLOCK",
    "VARIANT_AUTO", "VARIANT_LDST", "VARIANT_BULK",
]


def __getattr__(name):
    if name == "PageMover":
        from .mover import PageMover
        return PageMover
    raise AttributeError(name)
