"""CacheCoordinatorService on the native page directory.

Decisions and wire behaviour follow the coordinator the reference actually launches, the Go
one (``Go/CacheCoordinator/CacheCoordinator.go``): tasks arriving from a worker get
``cache_worker = (request_id + id) % n_shards`` and are queued (:75-83); the processing loop
(:134-236) turns CHECK into a lookup -- miss: recorded as CACHE_MISS, task left as it is;
hit: CACHE_HIT, task becomes SEND with the item's shard and pages -- and RECV into an
allocation (``LoadItem``), groups the batch by shard, hands each group to that shard's
``KVCacheService.ReceiveTasksFromCoordinator`` (:239-273) and adds the returned counts to the
per-request finished counters; ``PollBatchFromInferWorker`` (:86-124) answers with the
hit/miss table of the polled requests once their counters have reached ``task_num``;
``ReceiveTasksFromScheduler`` (:323-356) reports missed user / item tokens per request.

Differences: the page table is ``PageDirectory`` (tiered policy by default, i.e. the Go page
manager's priorities; ``policy="lru"`` gives the Python coordinator's); waiting is done on a
condition variable instead of spinning; TTL demotion runs when ``gc()`` is called (or every
``gc_interval_s`` seconds on a timer thread).  One time base throughout: the page table's
clock is moved to the monotonic nanosecond clock before every batch of decisions, so the
stamp an entry gets when it is loaded or touched and the ``now`` of a later ``gc()`` are both
nanoseconds, and ``ttl_s`` is an idle time in seconds whenever the first ``gc()`` comes.

A task that cannot be decided (an item larger than a shard, a pool with nothing left to
evict) and a shard whose RPC fails are logged, answered as CACHE_MISS and counted as
finished, so pollers are released and the loop thread lives on; the Go coordinator logs and
returns from the batch in the same situations (``CacheCoordinator.go:239-273``).
"""
from __future__ import annotations

import json
import logging
import threading
import time
from collections import deque
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Dict, List, Optional

from . import taskinfo as pb
from .page_directory import PageDirectory
from .rpc_def import KVCACHE_offset
from .signals import CACHE_HIT, CACHE_MISS, SIGNAL_CHECK, SIGNAL_RECV, SIGNAL_SEND

log = logging.getLogger("bikv.coordinator")


class CacheCoordinator:
    def __init__(self, rank: int, master_port: int, cache_ranks: List[int], infer_ranks: List[int],
                 cache_size: int, page_size: int, rank_to_ip: Dict[int, str], server=None, *,
                 policy: str = "tiered", seed: int = 0, ttl_s: Optional[float] = None,
                 gc_interval_s: Optional[float] = None,
                 kvcache_stub_factory: Optional[Callable[[str], object]] = None):
        """``cache_ranks`` / ``infer_ranks`` are shard / worker INDICES as in the Go coordinator
        (rank = 2*index + offset).  ``kvcache_stub_factory(address)`` returns an object with
        ``ReceiveTasksFromCoordinator`` and ``ShutDown`` (default: a gRPC stub per address)."""
        self.rank, self.master_port = rank, master_port
        self.cache_ranks, self.infer_ranks = list(cache_ranks), list(infer_ranks)
        self.rank_to_ip = rank_to_ip
        self.server = server
        self.kvcache_num = len(self.cache_ranks)
        self.page_manager = PageDirectory(cache_size, page_size, self.kvcache_num, policy=policy, seed=seed,
                                          ttl=None if ttl_s is None else int(ttl_s * 1e9))
        self.cache_miss_dict: Dict[int, Dict[int, int]] = {}
        self.finished_counter_table: Dict[int, int] = {}
        self._queue: deque = deque()
        self._lock = threading.Lock()                 # page directory + tables
        self._wake = threading.Condition(self._lock)  # new tasks, new counts, stop
        self._running = False
        self._thread: Optional[threading.Thread] = None
        self._pool = ThreadPoolExecutor(max_workers=max(1, self.kvcache_num))
        if kvcache_stub_factory is None:
            from . import grpc_services as G
            import grpc
            channels: dict = {}

            def kvcache_stub_factory(address):
                if address not in channels:
                    channels[address] = grpc.insecure_channel(address)
                return G.KVCacheServiceStub(channels[address])
        self._kvcache_stub = kvcache_stub_factory
        self._gc_timer: Optional[threading.Timer] = None
        self.errors = 0                               # tasks answered as misses after a failure
        self._gc_interval_s = gc_interval_s

    # -- helpers ------------------------------------------------------------
    def strategy(self, req_id: int) -> int:
        return req_id % self.kvcache_num

    def _kvcache_address(self, cache_worker: int) -> str:
        rank = 2 * cache_worker + KVCACHE_offset
        return f"{self.rank_to_ip[rank]}:{self.master_port + rank}"

    def gc(self, now_ns: Optional[int] = None) -> None:
        """What the Go coordinator's ttlGc tick does: demote idle user caches, enforce the
        priority-1 quota."""
        with self._lock:
            self.page_manager.advance_clock(time.monotonic_ns() if now_ns is None else now_ns)

    def _gc_tick(self) -> None:
        self.gc()
        if self._running and self._gc_interval_s:
            self._gc_timer = threading.Timer(self._gc_interval_s, self._gc_tick)
            self._gc_timer.daemon = True
            self._gc_timer.start()

    def read_prepared_data(self, data_path: str, index_path: str) -> int:
        """Pre-warms the page table from two JSON files, as the Go coordinator does at start-up
        when configured (``PageManager.go:536-563``): ``data_path`` maps item id (as a string)
        to its token count, ``index_path`` lists ids hottest first; ids from a file whose name
        contains "user" are looked up at ``id + 2000000``.  Items are loaded with weight 0
        until the pages handed out exceed the whole pool.  Returns the number loaded."""
        with open(data_path) as f:
            data = json.load(f)
        with open(index_path) as f:
            ids = json.load(f)
        user_file = "user" in index_path
        limit = self.kvcache_num * self.page_manager.num_pages
        total = loaded = 0
        with self._lock:
            self.page_manager.set_clock(time.monotonic_ns())
            for k in ids:
                tokens = int(data.get(str(k + 2000000 if user_file else k), 0))
                self.page_manager.load_item(int(k), tokens, 0, "prepared")
                loaded += 1
                total += (tokens + self.page_manager.page_size - 1) // self.page_manager.page_size
                if total > limit:
                    break
        return loaded

    # -- service methods ------------------------------------------------------
    def ReceiveTasksFromInferWorker(self, request, context):
        with self._wake:
            for task in request.tasks:
                task.cache_worker = self.strategy(task.request_id + task.id)
                self._queue.append(task)
            self._wake.notify_all()
        return pb.Empty()

    def StartProcessRequest(self, request, context):
        with self._wake:
            if not self._running:
                self._running = True
                self._thread = threading.Thread(target=self._process_requests, name="bikv-coordinator", daemon=True)
                self._thread.start()
        if self._gc_interval_s:
            self._gc_tick()
        return pb.Empty()

    def PollBatchFromInferWorker(self, request, context, timeout_s: float = 600.0):
        want: Dict[int, int] = {}
        for task in request.tasks:
            if want.setdefault(task.request_id, task.task_num) != task.task_num:
                msg = f"conflicting task_num for request id {task.request_id}"
                if context is not None:
                    import grpc
                    context.abort(grpc.StatusCode.INVALID_ARGUMENT, msg)
                raise ValueError(msg)
        deadline = time.monotonic() + timeout_s
        with self._wake:
            while any(self.finished_counter_table.get(r, 0) != n for r, n in want.items()):
                left = deadline - time.monotonic()
                if left <= 0 or not self._wake.wait(timeout=min(left, 1.0)) and time.monotonic() >= deadline:
                    raise TimeoutError("requests did not finish: " + str(
                        {r: (self.finished_counter_table.get(r, 0), n) for r, n in want.items()}))
            out = {r: self.cache_miss_dict.get(r) for r in want}
        return pb.ComfirmationMessage(msg=json.dumps(out))

    def ReceiveTasksFromScheduler(self, request, context):
        miss: Dict[int, Dict[str, int]] = {}
        with self._lock:
            self.page_manager.set_clock(time.monotonic_ns())
            for task in request.tasks:
                entry = miss.setdefault(task.request_id, {"user miss": 0, "item miss": 0})
                if self.page_manager.access_item(task.id)[0] is None:
                    if task.type == "user cache":
                        entry["user miss"] = task.token_num
                    else:
                        entry["item miss"] += task.token_num
        return pb.ComfirmationMessage(msg=json.dumps(miss))

    def ShutDown(self, request, context):
        self.stop()
        if self.server is not None:
            self.server.stop(0)
        return pb.Empty()

    # -- processing loop ------------------------------------------------------
    def _decide(self, task) -> None:
        """CHECK / RECV decision for one task (lock held)."""
        req = task.request_id
        if task.task_type == SIGNAL_CHECK:
            table = self.cache_miss_dict.setdefault(req, {})
            shard, pages = self.page_manager.access_item(task.id)
            if shard is None:
                table[task.id] = CACHE_MISS
            else:
                table[task.id] = CACHE_HIT
                task.task_type = SIGNAL_SEND
                task.cache_worker = shard
                del task.cache_pages_list[:]
                task.cache_pages_list.extend(pages)
        elif task.task_type == SIGNAL_RECV:
            shard, pages = self.page_manager.load_item(task.id, task.token_num, task.weight, task.type)
            task.cache_worker = shard
            del task.cache_pages_list[:]
            task.cache_pages_list.extend(pages)
        self.finished_counter_table.setdefault(req, 0)

    def _give_up(self, tasks: list, why: str) -> None:
        """Tasks that were not carried out: their items read as misses, and they count as
        finished so that nobody waits for them (lock held)."""
        for task in tasks:
            self.cache_miss_dict.setdefault(task.request_id, {})[task.id] = CACHE_MISS
            self.finished_counter_table[task.request_id] = self.finished_counter_table.get(task.request_id, 0) + 1
        self.errors += len(tasks)
        log.error("%d task(s) not carried out: %s", len(tasks), why)

    def _execute(self, cache_worker: int, tasks: list) -> None:
        try:
            stub = self._kvcache_stub(self._kvcache_address(cache_worker))
            reply = stub.ReceiveTasksFromCoordinator(pb.TaskInfoList(tasks=tasks))
            counts = json.loads(reply.msg)
        except Exception as e:  # noqa: BLE001  (a shard that is down, a malformed reply)
            with self._wake:
                self._give_up(tasks, f"shard {cache_worker}: {type(e).__name__}: {e}")
                self._wake.notify_all()
            return
        with self._wake:
            for req, n in counts.items():
                self.finished_counter_table[int(req)] = self.finished_counter_table.get(int(req), 0) + n
            self._wake.notify_all()

    def process_pending(self) -> int:
        """Drains the queue once: decide, group by shard, execute every group, wait for the
        replies.  Returns the number of tasks handled (the loop thread calls this; tests may
        call it directly instead of starting the thread)."""
        groups: Dict[int, list] = {}
        with self._wake:
            n = len(self._queue)
            if n:
                self.page_manager.set_clock(time.monotonic_ns())
            while self._queue:
                task = self._queue.popleft()
                try:
                    self._decide(task)
                except Exception as e:  # noqa: BLE001  (item too large, nothing left to evict)
                    self._give_up([task], f"item {task.id} of request {task.request_id}: {type(e).__name__}: {e}")
                    continue
                groups.setdefault(task.cache_worker, []).append(task)
            if n:
                self._wake.notify_all()
        futures = [self._pool.submit(self._execute, cw, tasks) for cw, tasks in groups.items()]
        for f in futures:
            f.result()
        return n

    def _process_requests(self) -> None:
        while True:
            with self._wake:
                while self._running and not self._queue:
                    self._wake.wait(timeout=0.5)
                if not self._running:
                    return
            try:
                self.process_pending()
            except Exception:  # noqa: BLE001  (the loop must outlive any one batch)
                log.exception("batch failed")

    def stop(self) -> None:
        with self._wake:
            self._running = False
            self._wake.notify_all()
        if self._gc_timer is not None:
            self._gc_timer.cancel()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=5)

    def send_terminate_signal(self) -> None:
        """ShutDown to every shard (CacheCoordinator.go:276-321; workers are left to their
        scheduler here)."""
        for cw in self.cache_ranks:
            try:
                self._kvcache_stub(self._kvcache_address(cw)).ShutDown(pb.Empty())
            except Exception:  # noqa: BLE001  (a shard that is already gone)
                pass
