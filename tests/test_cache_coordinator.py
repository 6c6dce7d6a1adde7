"""CacheCoordinatorService: decisions of the coordinator loop, counters, polling and the
scheduler query, with in-process shard stand-ins and over real gRPC on loopback."""
import json
from concurrent import futures

import grpc
import pytest

from bikv_b200 import grpc_services as G
from bikv_b200 import taskinfo as pb
from bikv_b200.cache_coordinator import CacheCoordinator
from bikv_b200.signals import CACHE_HIT, CACHE_MISS, SIGNAL_CHECK, SIGNAL_RECV, SIGNAL_SEND


class FakeShard:
    """Stands in for a KVCache shard: records what it is told and confirms every task."""

    def __init__(self):
        self.seen = []

    def ReceiveTasksFromCoordinator(self, request, context=None):
        conf = {}
        for t in request.tasks:
            self.seen.append((t.request_id, t.id, t.task_type, t.cache_worker, list(t.cache_pages_list)))
            if t.id != -1:
                conf[t.request_id] = conf.get(t.request_id, 0) + 1
        return pb.ComfirmationMessage(msg=json.dumps(conf))

    def ShutDown(self, request, context=None):
        return pb.Empty()


def make(n_shards=2, **kw):
    shards = {f"127.0.0.1:{5000 + 2 * i + 3}": FakeShard() for i in range(n_shards)}
    cc = CacheCoordinator(1, 5000, list(range(n_shards)), [0], 16 * 64, 16, {2 * i + 3: "127.0.0.1" for i in range(n_shards)},
                          None, kvcache_stub_factory=lambda addr: shards[addr], **kw)
    return cc, list(shards.values())


def task(req, item, typ, tokens=40, task_num=2, kind="item cache", weight=0):
    return pb.TaskInfo(request_id=req, id=item, infer_worker=0, token_num=tokens, task_type=typ, task_num=task_num,
                       type=kind, weight=weight)


def test_check_miss_then_recv_then_check_hit():
    cc, shards = make()
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(1, 10, SIGNAL_CHECK), task(1, 11, SIGNAL_CHECK)]), None)
    assert cc.process_pending() == 2
    assert cc.cache_miss_dict[1] == {10: CACHE_MISS, 11: CACHE_MISS}
    # a missed CHECK keeps its type and goes to shard (request_id + id) % n_shards
    got = sorted(x for s in shards for x in s.seen)
    assert got == [(1, 10, SIGNAL_CHECK, 1, []), (1, 11, SIGNAL_CHECK, 0, [])]
    reply = cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(1, 10, SIGNAL_CHECK), task(1, 11, SIGNAL_CHECK)]), None)
    assert json.loads(reply.msg) == {"1": {"10": CACHE_MISS, "11": CACHE_MISS}}
    # the worker computed them and writes them back
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(2, 10, SIGNAL_RECV), task(2, 11, SIGNAL_RECV)]), None)
    cc.process_pending()
    recv = [x for s in shards for x in s.seen if x[2] == SIGNAL_RECV]
    assert sorted(len(x[4]) for x in recv) == [3, 3]                      # 40 tokens = 3 pages of 16
    placed = {x[1]: (x[3], x[4]) for x in recv}
    # next request: both hit, become SEND with the shard and pages chosen at RECV time
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(3, 10, SIGNAL_CHECK), task(3, 11, SIGNAL_CHECK)]), None)
    cc.process_pending()
    assert cc.cache_miss_dict[3] == {10: CACHE_HIT, 11: CACHE_HIT}
    send = {x[1]: (x[3], x[4]) for s in shards for x in s.seen if x[2] == SIGNAL_SEND}
    assert send == placed
    assert cc.finished_counter_table == {1: 2, 2: 2, 3: 2}


def test_scheduler_query_and_conflicting_task_num():
    cc, _ = make()
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(1, 5, SIGNAL_RECV, tokens=32)]), None)
    cc.process_pending()
    q = pb.TaskInfoList(tasks=[task(9, 5, SIGNAL_CHECK, tokens=32), task(9, 6, SIGNAL_CHECK, tokens=10),
                               task(9, 7, SIGNAL_CHECK, tokens=20), task(9, 8, SIGNAL_CHECK, tokens=99, kind="user cache")])
    assert json.loads(cc.ReceiveTasksFromScheduler(q, None).msg) == {"9": {"user miss": 99, "item miss": 30}}
    with pytest.raises(ValueError):
        cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(1, 5, SIGNAL_CHECK, task_num=1),
                                                           task(1, 6, SIGNAL_CHECK, task_num=2)]), None)
    with pytest.raises(TimeoutError):
        cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(77, 5, SIGNAL_CHECK, task_num=1)]), None, timeout_s=0.2)


def test_user_caches_survive_eviction_until_gc():
    cc, _ = make(n_shards=1, ttl_s=0.0)
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(1, 100, SIGNAL_RECV, tokens=16 * 32, kind="user cache", weight=1),
                                                          task(1, 1, SIGNAL_RECV, tokens=16 * 32)]), None)
    cc.process_pending()                                       # pool of 64 pages is now full
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(2, 2, SIGNAL_RECV, tokens=16 * 32)]), None)
    cc.process_pending()                                       # evicts item 1, never the user cache
    assert cc.page_manager.access_item(100)[0] == 0 and cc.page_manager.access_item(1) == (None, None)
    cc.gc()                                                    # ttl 0: user cache drops to priority 1
    assert cc.page_manager.priority(100) in (0, 1)


def test_over_grpc_with_the_loop_thread():
    shard = FakeShard()
    sserver = grpc.server(futures.ThreadPoolExecutor(max_workers=2))
    G.add_KVCacheServiceServicer_to_server(shard, sserver)
    sport = sserver.add_insecure_port("127.0.0.1:0")
    sserver.start()
    cc = CacheCoordinator(1, sport - 3, [0], [0], 16 * 64, 16, {3: "127.0.0.1"}, None)      # shard rank 3 -> port
    cserver = grpc.server(futures.ThreadPoolExecutor(max_workers=4))
    G.add_CacheCoordinatorServiceServicer_to_server(cc, cserver)
    cport = cserver.add_insecure_port("127.0.0.1:0")
    cserver.start()
    try:
        with grpc.insecure_channel(f"127.0.0.1:{cport}") as ch:
            stub = G.CacheCoordinatorServiceStub(ch)
            stub.StartProcessRequest(pb.StartRequest(msg="go"), timeout=10)
            batch = pb.TaskInfoList(tasks=[task(4, 1, SIGNAL_RECV, task_num=1)])
            stub.ReceiveTasksFromInferWorker(batch, timeout=10)
            reply = stub.PollBatchFromInferWorker(batch, timeout=30)
            assert json.loads(reply.msg) == {"4": None}            # no CHECK was made for request 4
            check = pb.TaskInfoList(tasks=[task(5, 1, SIGNAL_CHECK, task_num=1)])
            stub.ReceiveTasksFromInferWorker(check, timeout=10)
            assert json.loads(stub.PollBatchFromInferWorker(check, timeout=30).msg) == {"5": {"1": CACHE_HIT}}
        assert [x[2] for x in shard.seen] == [SIGNAL_RECV, SIGNAL_SEND]
    finally:
        cc.stop()
        cserver.stop(0)
        sserver.stop(0)


def test_prewarm_from_json(tmp_path):
    cc, _ = make(n_shards=2)
    data = {str(i): 16 * (1 + i % 5) for i in range(30)}             # 90 pages: fits the 128-page pool
    (tmp_path / "item_len.json").write_text(json.dumps(data))
    (tmp_path / "item_hot.json").write_text(json.dumps(list(range(30))))
    n = cc.read_prepared_data(str(tmp_path / "item_len.json"), str(tmp_path / "item_hot.json"))
    assert n == 30
    assert cc.page_manager.access_item(0)[0] is not None           # the hottest item is resident
    q = pb.TaskInfoList(tasks=[task(1, 0, SIGNAL_CHECK), task(1, 1, SIGNAL_CHECK)])
    cc.ReceiveTasksFromInferWorker(q, None)
    cc.process_pending()
    assert cc.cache_miss_dict[1] == {0: CACHE_HIT, 1: CACHE_HIT}
    # ids of a "user" index are looked up at id + 2000000
    udata = {str(2000000 + i): 32 for i in range(5)}
    (tmp_path / "user_len.json").write_text(json.dumps(udata))
    (tmp_path / "user_hot.json").write_text(json.dumps([0, 1, 2, 3, 4]))
    cc2, _ = make(n_shards=1)
    assert cc2.read_prepared_data(str(tmp_path / "user_len.json"), str(tmp_path / "user_hot.json")) == 5
    assert len(cc2.page_manager.access_item(3)[1]) == 2


class FlakyShard(FakeShard):
    """Raises on its first call, like a shard that is down, then serves."""

    def __init__(self):
        super().__init__()
        self.calls = 0

    def ReceiveTasksFromCoordinator(self, request, context=None):
        self.calls += 1
        if self.calls == 1:
            raise ConnectionError("shard unreachable")
        return super().ReceiveTasksFromCoordinator(request, context)


def test_a_failing_shard_or_an_undecidable_task_does_not_stop_the_loop():
    import time
    shard = FlakyShard()
    cc = CacheCoordinator(1, 5000, [0], [0], 16 * 8, 16, {3: "127.0.0.1"}, None,
                          kvcache_stub_factory=lambda addr: shard)
    cc.StartProcessRequest(pb.Empty(), None)
    try:
        # batch 1: the shard's RPC raises; batch 2: an item larger than the shard (9 pages > 8)
        cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(1, 10, SIGNAL_RECV, task_num=1)]), None)
        r = cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(1, 10, SIGNAL_RECV, task_num=1)]), None, timeout_s=10)
        assert json.loads(r.msg) == {"1": {"10": CACHE_MISS}}
        cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(2, 11, SIGNAL_RECV, tokens=16 * 9, task_num=1)]), None)
        r = cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(2, 11, SIGNAL_RECV, task_num=1)]), None, timeout_s=10)
        assert json.loads(r.msg) == {"2": {"11": CACHE_MISS}}
        assert cc.errors == 2
        # the loop thread is alive and a later batch is served normally
        cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(3, 12, SIGNAL_RECV, task_num=1)]), None)
        cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(3, 12, SIGNAL_RECV, task_num=1)]), None, timeout_s=10)
        assert cc._thread.is_alive()
        assert [x[:3] for x in shard.seen] == [(3, 12, SIGNAL_RECV)]
        cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(4, 12, SIGNAL_CHECK, task_num=1)]), None)
        r = cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=[task(4, 12, SIGNAL_CHECK, task_num=1)]), None, timeout_s=10)
        assert json.loads(r.msg) == {"4": {"12": CACHE_HIT}}
    finally:
        cc.stop()


def test_ttl_counts_idle_time_from_the_entry_s_own_stamp():
    """Entries are stamped on the clock gc() compares against: a user cache loaded a moment
    before the first gc() is not demoted, one idle for longer than the TTL is."""
    import time
    cc, shards = make(n_shards=1, ttl_s=5.0)
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=[task(1, 20, SIGNAL_RECV, task_num=1, kind="user cache",
                                                               weight=1)]), None)
    cc.process_pending()
    assert cc.page_manager.priority(20) == 2
    cc.gc()                                               # first gc ever, right after the load
    assert cc.page_manager.priority(20) == 2
    cc.gc(time.monotonic_ns() + int(4e9))                 # idle for 4 s < ttl
    assert cc.page_manager.priority(20) == 2
    cc.gc(time.monotonic_ns() + int(6e9))                 # idle for 6 s > ttl
    assert cc.page_manager.priority(20) == 1
