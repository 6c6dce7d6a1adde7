"""Worker-side end of the KV-page path.

Keeps the constructor and the four KV-data methods of ``Worker/Worker.py``
(``__init__`` :39-92, ``receive_kvcache_data_batch`` :162-191,
``send_kvcache_data_batch`` :193-218, ``RecvKVCacheData`` / ``SendKVCacheData``
:304-316).  The model forward, scheduler hand-off and coordinator polling of the
reference's Worker are outside this path and are not built.

The worker owns a packed KV buffer ``compute_buffer`` of shape
``[layer, kv, buffer_tokens, head, dim]`` on its GPU.  A combined task's items are
laid out one after another from token 0 (the reference's running ``dest_offsets``,
``DistributedStorage/kvcache.py:161-174``).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from . import _native as N
from . import taskinfo as pb
from .geometry import GEO_R, KVGeometry
from .mover import PageMover
from .page_manager import PageManager
from .plan import plan_from_combined_task
from .pool import ShardedPool
from .rpc_def import KVCACHE_offset


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
        self.mover = PageMover(self.device)

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
    def _plan(self, task):
        if self.pool is None:
            raise RuntimeError(f"worker rank {self.rank}: no pool attached")
        plan = plan_from_combined_task(task, self.page_size, pages_per_shard=self.pool.pages_per_shard,
                                       block_sharded=self.pool.rule == N.SHARD_BLOCK)
        if plan.total_tokens > self.buffer_size:
            raise N.BikvError(N.ERR_DST_RANGE, "worker buffer too small for the task")
        return plan

    def pull_pages(self, combined_task_info):
        """Gather the task's pages into ``compute_buffer[:, :, :tokens]``; returns that view.
        Asynchronous on this GPU's current stream."""
        plan = self._plan(combined_task_info)
        with torch.cuda.device(self.device):
            self.mover.gather(self.pool, plan, self.compute_buffer)
        return self.compute_buffer[:, :, :plan.total_tokens]

    def push_pages(self, combined_task_info):
        """Scatter ``compute_buffer[:, :, :tokens]`` into the task's pages."""
        plan = self._plan(combined_task_info)
        with torch.cuda.device(self.device):
            self.mover.scatter(self.pool, plan, self.compute_buffer)
        return plan.total_tokens

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
