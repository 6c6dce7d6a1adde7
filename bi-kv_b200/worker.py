"""Worker-side end of the KV-page path.

Keeps the constructor and the four KV-data methods of ``Worker/Worker.py``
(``__init__`` :39-92, ``receive_kvcache_data_batch`` :162-191,
``send_kvcache_data_batch`` :193-218, ``RecvKVCacheData`` / ``SendKVCacheData``
:304-316).  The model forward, scheduler hand-off and coordinator polling of the
reference's Worker are outside this path and are not built.

The worker owns a packed KV buffer ``compute_buffer`` of shape
``[layer, kv, buffer_tokens, head, dim]`` on its GPU.  A combined task's items are
laid out one after another (the reference's running ``dest_offsets``,
``DistributedStorage/kvcache.py:161-174``) inside a token WINDOW of that buffer that
belongs to the task alone: the coordinator splits a batch by shard and the shards serve
their groups concurrently, so one worker receives several combined tasks at once, and
each needs its own place.  (The reference allocates a fresh tensor per call,
``Worker/Worker.py:162-218``; here windows are handed out from the one buffer, front to
back, starting over at token 0 when the end is reached -- the ring discipline of the
reference's staging buffer, ``SharedMemory/CUDA_Shared/ipc_service.cpp:146-168``.)
"""
from __future__ import annotations

import threading
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _native as N
from . import taskinfo as pb
from .geometry import GEO_R, KVGeometry
from .mover import PageMover
from .page_manager import PageManager
from .plan import plan_from_combined_task
from .pool import ShardedPool


class Worker:
    def __init__(self, rank, master_port, cache_size, page_size, coordinator_rank, rank_to_ip, rank_to_ip_rdma,
                 server, *, geometry: Optional[KVGeometry] = None, device=None):
        self.rank = rank
        self.master_port = master_port
        self.worker_index = int(rank / 2) - 1
        self.coordinator_rank = coordinator_rank
        self.server = server
        self.rank_to_ip_grpc = rank_to_ip
        self.rank_to_ip_rdma = rank_to_ip_rdma
        self.device = torch.device(device if device is not None else "cuda:0")
        self.buffer_size = cache_size
        self.page_size = page_size
        base = geometry if geometry is not None else GEO_R
        self.geometry = KVGeometry(base.n_layers, base.n_kv_heads, base.head_dim, page_size, base.dtype,
                                   base.pool_layout)
        self.page_manager = PageManager(cache_size=self.buffer_size, page_size=self.page_size)
        self.compute_buffer = torch.zeros(self.geometry.worker_shape(self.buffer_size), dtype=self.geometry.dtype,
                                          device=self.device)
        self.start_pos = 0
        self.cache_miss_dict: Dict = {}
        self.pool: Optional[ShardedPool] = None
        # Token windows of compute_buffer, one per combined task (see the module text).
        self._window_lock = threading.Lock()
        self._cursor = 0
        self._reserved: Dict[Tuple[int, int], Tuple[int, int]] = {}
        self.windows: Dict[Tuple[int, int], Tuple[int, int]] = {}   # (task_type, cache_worker) -> last (start, tokens)
        self.mover = PageMover(self.device)
        # The model-side paged KV cache (``local_kvcache`` of Worker/Worker.py:68-78): one
        # [blocks * block_size, 2, heads, dim] tensor per layer; allocated on demand.
        self.local_kv_cache_block_size = page_size
        self.local_max_kv_cache_blocks = 0
        self.local_kvcache = []

    # -- wiring --------------------------------------------------------------
    def attach_pool(self, pool: ShardedPool) -> None:
        """The sharded pool as this worker's GPU addresses it.  For the reference's
        item-granular placement build it with ``rule=SHARD_BLOCK`` (a task's
        ``cache_worker`` picks the shard, its page numbers are shard-local)."""
        self.pool = pool

    @staticmethod
    def connect(kvcaches: Sequence, workers: Sequence["Worker"]) -> None:
        """In-process wiring: every worker maps every shard (peer access is enabled where
        GPUs differ) and every shard knows every worker."""
        for w in workers:
            shards = [kv.cuda_cache_data for kv in kvcaches]
            w.attach_pool(ShardedPool.from_tensors(shards, kvcaches[0].geometry, rule=N.SHARD_BLOCK,
                                                   device=w.device))
            for kv in kvcaches:
                kv.attach_worker(w)

    # -- data plane ----------------------------------------------------------
    @staticmethod
    def _task_key(task) -> Tuple[int, int]:
        if isinstance(task, dict):
            return int(task["task_type"]), int(task["cache_worker"])
        return int(task.task_type), int(task.cache_worker)

    @staticmethod
    def _task_tokens(task) -> int:
        if isinstance(task, dict):
            return int(sum(p[1] for p in task["id_token_pair"]))
        return int(sum(p.token_num for p in task.id_token_pair))

    def _bump(self, tokens: int) -> int:
        if tokens > self.buffer_size:
            raise N.BikvError(N.ERR_DST_RANGE, "worker buffer too small for the task")
        if self._cursor + tokens > self.buffer_size:
            self._cursor = 0
        start = self._cursor
        self._cursor += tokens
        return start

    def reserve_window(self, combined_task_info) -> int:
        """Reserves the token window the NEXT pull/push of this task's (task_type,
        cache_worker) will use and returns its first token.  The producer of a RECV's data
        (the model's prefill) calls this, writes ``compute_buffer[:, :, start:start+tokens]``,
        and then lets the task run."""
        tokens = self._task_tokens(combined_task_info)
        with self._window_lock:
            start = self._bump(tokens)
            self._reserved[self._task_key(combined_task_info)] = (start, tokens)
        return start

    def reset_windows(self) -> None:
        """Start handing out windows from token 0 again (between batches)."""
        with self._window_lock:
            self._cursor = 0
            self._reserved.clear()

    def _window(self, task, tokens: int) -> int:
        key = self._task_key(task)
        with self._window_lock:
            got = self._reserved.pop(key, None)
            start = got[0] if got is not None and got[1] == tokens else self._bump(tokens)
            self.windows[key] = (start, tokens)
        return start

    def _plan(self, task):
        if self.pool is None:
            raise RuntimeError(f"worker rank {self.rank}: no pool attached")
        plan = plan_from_combined_task(task, self.page_size, pages_per_shard=self.pool.pages_per_shard,
                                       block_sharded=self.pool.rule == N.SHARD_BLOCK)
        if plan.total_tokens > self.buffer_size:
            raise N.BikvError(N.ERR_DST_RANGE, "worker buffer too small for the task")
        start = self._window(task, plan.total_tokens)
        if start:
            plan.table[:, 3] += start
            plan.request_tokens[0] += start
        return plan, start

    def pull_pages(self, combined_task_info):
        """Gather the task's pages into its own window ``compute_buffer[:, :, start:start+tokens]``;
        returns that view (``windows[(task_type, cache_worker)]`` records the window).
        Asynchronous on this GPU's current stream."""
        plan, start = self._plan(combined_task_info)
        with torch.cuda.device(self.device):
            self.mover.gather(self.pool, plan, self.compute_buffer)
        return self.compute_buffer[:, :, start:plan.total_tokens]

    def push_pages(self, combined_task_info):
        """Scatter the task's window of ``compute_buffer`` into the task's pages: the window
        reserved for it with :meth:`reserve_window`, else the next free one."""
        plan, start = self._plan(combined_task_info)
        with torch.cuda.device(self.device):
            self.mover.scatter(self.pool, plan, self.compute_buffer)
        return plan.total_tokens - start

    def init_local_kvcache(self, max_blocks: int) -> None:
        """Allocates the paged per-layer KV cache with blocks of ``page_size`` tokens (the
        reference uses 10240 blocks of 16 tokens, ``Worker.py:65-66``)."""
        g = self.geometry
        self.local_max_kv_cache_blocks = max_blocks
        self.local_kvcache = [torch.zeros(max_blocks * self.page_size, 2, g.n_kv_heads, g.head_dim, dtype=g.dtype,
                                          device=self.device) for _ in range(g.n_layers)]

    def _block_plan(self, task, block_ids):
        from .plan import build_block_plan

        if self.pool is None or not self.local_kvcache:
            raise RuntimeError(f"worker rank {self.rank}: pool and local_kvcache must be set up first")
        if isinstance(task, dict):
            pages, tokens, cw = task["cache_pages_list"], [p[1] for p in task["id_token_pair"]], task["cache_worker"]
        else:
            pages, tokens, cw = task.cache_pages_list, [p.token_num for p in task.id_token_pair], task.cache_worker
        pages = [getattr(p, "cache_pages_list", p) for p in pages]
        block = self.pool.rule == N.SHARD_BLOCK
        return build_block_plan(pages, tokens, self.page_size, block_ids,
                                item_shard=[cw] * len(tokens) if block else None,
                                pages_per_shard=self.pool.pages_per_shard)

    def pull_pages_to_blocks(self, combined_task_info, block_ids) -> None:
        """Gather the task's pages straight into ``local_kvcache``: the k-th page of the task
        (items in order) fills block ``block_ids[k]`` of every layer -- no intermediate tensor
        between the pool and the cache the model's paged prefill reads."""
        plan = self._block_plan(combined_task_info, block_ids)
        with torch.cuda.device(self.device):
            self.mover.gather_nhd(self.pool, plan, self.local_kvcache)

    def push_pages_from_blocks(self, combined_task_info, block_ids) -> None:
        """Scatter blocks of ``local_kvcache`` into the task's pool pages."""
        plan = self._block_plan(combined_task_info, block_ids)
        with torch.cuda.device(self.device):
            self.mover.scatter_nhd(self.pool, plan, self.local_kvcache)

    def receive_kvcache_data_batch(self, combined_task_info):
        return self.pull_pages(combined_task_info)

    def send_kvcache_data_batch(self, combined_task_info):
        return self.push_pages(combined_task_info)

    # -- gRPC servicer methods of InferWorkerService on this path -------------
    def RecvKVCacheData(self, request, context):
        self.receive_kvcache_data_batch(request)
        return pb.Empty()

    def SendKVCacheData(self, request, context):
        self.send_kvcache_data_batch(request)
        return pb.Empty()

    def ShutDown(self, request, context):
        if self.server is not None:
            self.server.stop(0)
        return pb.Empty()
