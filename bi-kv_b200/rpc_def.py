"""Rank / role convention (``rpc_def.py:5-57``): rank 0 scheduler, rank 1
coordinator, even ranks >= 2 workers, odd ranks >= 3 KVCache shards; a role's
gRPC port is ``master_port + rank``."""
import os

KVCACHE_NUM = int(os.environ.get("KVCACHE_NUM", "4"))
WORKER_NUM = int(os.environ.get("WORKER_NUM", "4"))
WORKER_offset = 2
KVCACHE_offset = 3


def get_process_info(rank: int):
    if rank == 0:
        return "LLMScheduler", 0
    if rank == 1:
        return "CacheCoordinator", 0
    return ("Worker" if rank % 2 == 0 else "KVCache"), rank // 2 - 1


def worker_rank(worker_index: int) -> int:
    return 2 * worker_index + WORKER_offset


def kvcache_rank(cache_index: int) -> int:
    return 2 * cache_index + KVCACHE_offset


def generate_rank_map(world_size: int) -> dict:
    out: dict = {}
    for r in range(world_size):
        out.setdefault(get_process_info(r)[0], []).append(r)
    return out
