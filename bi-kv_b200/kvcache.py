"""KVCache shard: owns one page pool and routes coordinator tasks.

Keeps the constructor and method names of ``DistributedStorage/kvcache.py``
(``KVCache.__init__`` :32-79, ``send_data_batch`` :96-113, ``receive_data_batch``
:116-130, ``shared_data_batch_pages`` :132-239, ``receive_task_info_batch_gprc``
:368-459, ``_task_info_json_to_pb`` :467-475).  What differs is the data plane:
the pool lives in HBM, and pages move one-sidedly -- the worker GPU's kernel
reads (SEND) or writes (RECV) this shard's memory directly, through a peer
mapping when the worker sits on another GPU.  There is no staging ring, no
RDMA endpoint and no CPU copy.
"""
from __future__ import annotations

import json
from typing import Dict, Optional

import torch

from . import taskinfo as pb
from .geometry import GEO_R, KVGeometry
from .rpc_def import WORKER_offset
from .signals import SIGNAL_RECV, SIGNAL_SEND


class KVCache:
    def __init__(self, rank, cache_size, page_size, master_port, rank_to_ip, rank_to_ip_rdma, server, *,
                 geometry: Optional[KVGeometry] = None, device=None, fill=None):
        """``cache_size`` is in tokens, ``page_size`` in tokens per page, as in the
        reference's ``config.yml`` (``kv_cache.cache_size`` / ``page_size``).  ``geometry``
        defaults to the reference's literals (28 layers, 2 KV heads, head 128, fp16,
        token-major pool) with ``page_size``-token pages.  ``fill``: value the pool starts
        with (the reference fills with the rank; default leaves it uninitialised)."""
        self.rank = rank
        self.cache_index = int(rank / 2) - 1
        self.gpu_index = 0
        self.cache_size = cache_size
        self.page_size = page_size
        base = geometry if geometry is not None else GEO_R
        self.geometry = KVGeometry(base.n_layers, base.n_kv_heads, base.head_dim, page_size, base.dtype,
                                   base.pool_layout)
        self.device = torch.device(device if device is not None else "cuda:0")
        self.num_pages = cache_size // page_size
        self.max_pages = (cache_size + page_size - 1) // page_size
        self.cuda_cache_data = torch.empty(self.geometry.pool_shape(self.num_pages), dtype=self.geometry.dtype,
                                           device=self.device)
        if fill is not None:
            self.cuda_cache_data.fill_(fill)
        self.src_index_pool = torch.full((self.max_pages,), -1, dtype=torch.int64, device=self.device)
        self.dst_index_pool = torch.full((self.max_pages,), -1, dtype=torch.int64, device=self.device)
        self.start_pos = 0
        self.recv_counter = 0
        self.send_counter = 0
        self.master_port = master_port
        self.server = server
        self.rank_to_ip_grpc = rank_to_ip
        self.rank_to_ip_rdma = rank_to_ip_rdma
        self.workers: Dict[int, object] = {}   # in-process workers by worker index
        self.stub_factory = None               # optional: address -> InferWorkerService stub

    # -- wiring --------------------------------------------------------------
    def attach_worker(self, worker) -> None:
        """Registers a worker living in this process (replaces the RDMA connect and
        the shared-memory producer_init of the reference)."""
        self.workers[worker.worker_index] = worker

    def export_handle(self):
        """(64-byte CUDA IPC handle, offset) of this shard's pool for workers in other
        processes."""
        from .pool import ShardedPool
        return ShardedPool.export_handle(self.cuda_cache_data)

    def get_index_tensors(self, num_pages):
        assert num_pages <= self.max_pages, f"Requested {num_pages} exceeds pool size {self.max_pages}"
        return self.src_index_pool[:num_pages], self.dst_index_pool[:num_pages]

    # -- data plane ----------------------------------------------------------
    def _worker_for(self, combined_task_info: Dict):
        w = self.workers.get(combined_task_info["infer_worker"])
        if w is None:
            raise RuntimeError(f"worker {combined_task_info['infer_worker']} is not attached to KVCache "
                               f"rank {self.rank}")
        return w

    def send_data_batch(self, combined_task_info: Dict):
        """SEND: this shard's pages -> the worker's KV buffer.  The copy is issued on the
        worker's GPU (a one-sided read of this pool) and is asynchronous on that GPU's
        current stream; returns the worker-side view of the gathered tokens."""
        return self._worker_for(combined_task_info).pull_pages(combined_task_info)

    def receive_data_batch(self, combined_task_info: Dict):
        """RECV: the worker's KV buffer -> this shard's pages (one-sided write)."""
        return self._worker_for(combined_task_info).push_pages(combined_task_info)

    def shared_data_batch_pages(self, combined_task_info: Dict):
        """Same-host SEND.  In the reference this is a separate CUDA-IPC path; here the
        same kernel serves local and peer shards."""
        return self.send_data_batch(combined_task_info)

    shared_data_batch_pages_cpu2gpu = shared_data_batch_pages

    # -- control plane -------------------------------------------------------
    def receive_task_info_batch_gprc(self, task_info_list):
        """Groups tasks by (infer_worker, SEND/RECV), runs one transfer per group, and
        returns ``{request_id: number of tasks seen}``.  Tasks with ``id == -1`` are
        skipped."""
        combined: Dict[int, Dict[int, Dict]] = {}
        confirmation: Dict[int, int] = {}
        for t in task_info_list:
            if t.id == -1:
                continue
            per_worker = combined.setdefault(t.infer_worker, {})
            if t.task_type in (SIGNAL_SEND, SIGNAL_RECV):
                g = per_worker.get(t.task_type)
                if g is None:
                    per_worker[t.task_type] = {
                        "infer_worker": t.infer_worker, "cache_worker": t.cache_worker,
                        "token_num": t.token_num, "task_type": t.task_type,
                        "id_token_pair": [(t.id, t.token_num)],
                        "cache_pages_list": [t.cache_pages_list],
                    }
                else:
                    g["token_num"] += t.token_num
                    g["id_token_pair"].append((t.id, t.token_num))
                    g["cache_pages_list"].append(t.cache_pages_list)
            confirmation[t.request_id] = confirmation.get(t.request_id, 0) + 1
        for per_worker in combined.values():
            for task in per_worker.values():
                self._dispatch(task)
        return confirmation

    def _dispatch(self, task: Dict) -> None:
        infer_worker = task["infer_worker"]
        message = self._task_info_json_to_pb(task)
        remote = None
        if infer_worker not in self.workers and self.stub_factory is not None:
            rank = 2 * infer_worker + WORKER_offset
            remote = self.stub_factory(f"{self.rank_to_ip_grpc[rank]}:{self.master_port + rank}")
        if task["task_type"] == SIGNAL_SEND:
            if remote is not None:
                remote.RecvKVCacheData(message)
            else:
                self.send_data_batch(task)
            self.send_counter += 1
        else:
            if remote is not None:
                remote.SendKVCacheData(message)
            else:
                self.receive_data_batch(task)
            self.recv_counter += 1

    def ReceiveTasksFromCoordinator(self, request, context):
        confirmation = self.receive_task_info_batch_gprc(request.tasks)
        return pb.ComfirmationMessage(msg=json.dumps(confirmation))

    def _task_info_json_to_pb(self, task_info: Dict):
        m = pb.CombindedTaskInfo()
        m.infer_worker = task_info["infer_worker"]
        m.cache_worker = task_info["cache_worker"]
        m.token_num = task_info["token_num"]
        m.task_type = task_info["task_type"]
        m.cache_pages_list.extend(pb.PageList(cache_pages_list=list(p)) for p in task_info["cache_pages_list"])
        m.id_token_pair.extend(pb.IdTokenPair(id=i, token_num=n) for i, n in task_info["id_token_pair"])
        return m

    def ShutDown(self, request, context):
        if self.server is not None:
            self.server.stop(0)
        return pb.Empty()

    def send_confirmation(self, confirmation_msg):
        return confirmation_msg

    def terminate(self):
        self.show_counter()
        return "Terminated"

    def show_counter(self):
        print(f"[KVCache][RANK {self.rank}] send_counter: {self.send_counter}, recv_counter: {self.recv_counter}")
