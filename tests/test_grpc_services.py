"""The control-plane services over real gRPC on loopback: routing, wire format, and (on a
GPU) a coordinator-style client driving KVCache -> Worker transfers through the wire."""
import json
from concurrent import futures

import grpc
import pytest

from bikv_b200 import grpc_services as G
from bikv_b200 import taskinfo as pb
from bikv_b200.signals import SIGNAL_RECV, SIGNAL_SEND


def _serve(register):
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=4))
    register(server)
    port = server.add_insecure_port("127.0.0.1:0")
    server.start()
    return server, f"127.0.0.1:{port}"


def test_kvcache_service_round_trip_on_loopback():
    from bikv_b200.kvcache import KVCache

    kv = KVCache.__new__(KVCache)
    kv.rank, kv.master_port, kv.send_counter, kv.recv_counter = 3, 5000, 0, 0
    kv.workers, kv.stub_factory, kv.server = {}, None, None
    seen = []
    kv.send_data_batch = lambda t: seen.append(("send", t["id_token_pair"], [list(p) for p in t["cache_pages_list"]]))
    kv.receive_data_batch = lambda t: seen.append(("recv", t["id_token_pair"], [list(p) for p in t["cache_pages_list"]]))
    server, addr = _serve(lambda s: G.add_KVCacheServiceServicer_to_server(kv, s))
    try:
        with grpc.insecure_channel(addr) as ch:
            stub = G.KVCacheServiceStub(ch)
            tasks = pb.TaskInfoList(tasks=[
                pb.TaskInfo(request_id=1, id=10, infer_worker=0, cache_worker=0, token_num=20, task_type=SIGNAL_SEND,
                            cache_pages_list=[4, 5]),
                pb.TaskInfo(request_id=1, id=-1, infer_worker=0, token_num=99, task_type=SIGNAL_SEND),
                pb.TaskInfo(request_id=2, id=11, infer_worker=0, cache_worker=0, token_num=16, task_type=SIGNAL_RECV,
                            cache_pages_list=[7]),
            ])
            reply = stub.ReceiveTasksFromCoordinator(tasks, timeout=10)
            assert json.loads(reply.msg) == {"1": 1, "2": 1}
            assert seen == [("send", [(10, 20)], [[4, 5]]), ("recv", [(11, 16)], [[7]])]
            assert isinstance(stub.ShutDown(pb.Empty(), timeout=10), pb.Empty)
    finally:
        server.stop(0)


def test_unimplemented_methods_answer_unimplemented():
    class OnlyShutdown:
        def ShutDown(self, request, context):
            return pb.Empty()

    server, addr = _serve(lambda s: G.add_InferWorkerServiceServicer_to_server(OnlyShutdown(), s))
    try:
        with grpc.insecure_channel(addr) as ch:
            stub = G.InferWorkerServiceStub(ch)
            stub.ShutDown(pb.Empty(), timeout=10)
            with pytest.raises(grpc.RpcError) as e:
                stub.RecvKVCacheData(pb.CombindedTaskInfo(), timeout=10)
            assert e.value.code() == grpc.StatusCode.UNIMPLEMENTED
    finally:
        server.stop(0)


@pytest.mark.gpu
def test_transfers_driven_through_grpc(cuda):
    """KVCache shard and Worker as gRPC servers (threads of this process); the shard reaches
    the worker only through its InferWorkerService stub, as in a deployment."""
    import torch

    from bikv_b200.geometry import KVGeometry
    from bikv_b200.kvcache import KVCache
    from bikv_b200.pool import ShardedPool
    from bikv_b200.worker import Worker
    from bikv_b200 import _native as N
    from helpers import equal_bits, normal

    geom = KVGeometry(2, 2, 64, 16, torch.float16)
    worker = Worker(2, 0, 96, 16, 1, {}, {}, None, geometry=geom)
    wserver, waddr = _serve(lambda s: G.add_InferWorkerServiceServicer_to_server(worker, s))
    wport = int(waddr.split(":")[1])
    kv = KVCache(3, 16 * 12, 16, wport - 2, {2: "127.0.0.1"}, {}, None, geometry=geom, fill=0)   # port = master_port + rank
    worker.attach_pool(ShardedPool.from_tensors([kv.cuda_cache_data], geom, rule=N.SHARD_BLOCK))
    kv.stub_factory = G.worker_stub_factory()
    kserver, kaddr = _serve(lambda s: G.add_KVCacheServiceServicer_to_server(kv, s))
    try:
        data = normal(geom.worker_shape(37), geom.dtype, 1)
        worker.compute_buffer[:, :, :37] = data.to(cuda)
        with grpc.insecure_channel(kaddr) as ch:
            stub = G.KVCacheServiceStub(ch)
            recv = [pb.TaskInfo(request_id=5, id=1, infer_worker=0, cache_worker=0, token_num=20, task_type=SIGNAL_RECV,
                                cache_pages_list=[9, 2]),
                    pb.TaskInfo(request_id=5, id=2, infer_worker=0, cache_worker=0, token_num=17, task_type=SIGNAL_RECV,
                                cache_pages_list=[4, 7])]
            assert json.loads(stub.ReceiveTasksFromCoordinator(pb.TaskInfoList(tasks=recv), timeout=30).msg) == {"5": 2}
            torch.cuda.synchronize()
            worker.compute_buffer.zero_()
            worker.reset_windows()
            send = [pb.TaskInfo(request_id=6, id=t.id, infer_worker=0, cache_worker=0, token_num=t.token_num,
                                task_type=SIGNAL_SEND, cache_pages_list=list(t.cache_pages_list)) for t in recv]
            assert json.loads(stub.ReceiveTasksFromCoordinator(pb.TaskInfoList(tasks=send), timeout=30).msg) == {"6": 2}
        torch.cuda.synchronize()
        assert equal_bits(worker.compute_buffer[:, :, :37], data)
        assert (kv.send_counter, kv.recv_counter) == (1, 1)
    finally:
        kserver.stop(0)
        wserver.stop(0)


def _free_base(ranks):
    """A master_port such that master_port + rank is free for every rank (the reference's
    port convention, rpc_def.py:50-57)."""
    import random
    import socket
    rnd = random.Random()
    for _ in range(200):
        base = rnd.randrange(20000, 50000)
        socks = []
        try:
            for r in ranks:
                s = socket.socket()
                s.bind(("127.0.0.1", base + r))
                socks.append(s)
            return base
        except OSError:
            continue
        finally:
            for s in socks:
                s.close()
    raise RuntimeError("no free port range")


@pytest.mark.gpu
def test_full_chain_coordinator_shards_worker_over_grpc(cuda):
    """Coordinator (rank 1), worker (rank 2) and two shards (ranks 3, 5) as gRPC servers on
    the reference's ports; a client plays the worker's request loop: RECV (write back), then
    CHECK (hit -> SEND).  Data must come back bit for bit."""
    import torch

    from bikv_b200 import _native as N
    from bikv_b200.cache_coordinator import CacheCoordinator
    from bikv_b200.geometry import KVGeometry
    from bikv_b200.kvcache import KVCache
    from bikv_b200.worker import Worker
    from helpers import equal_bits, normal

    geom = KVGeometry(2, 2, 64, 16, torch.float16)
    base = _free_base([1, 2, 3, 5])
    ips = {r: "127.0.0.1" for r in (1, 2, 3, 5)}
    servers = []

    def serve(rank, register):
        s = grpc.server(futures.ThreadPoolExecutor(max_workers=4))
        register(s)
        assert s.add_insecure_port(f"127.0.0.1:{base + rank}") == base + rank
        s.start()
        servers.append(s)

    worker = Worker(2, base, 128, 16, 1, ips, {}, None, geometry=geom)
    kvs = [KVCache(3 + 2 * i, 16 * 16, 16, base, ips, {}, None, geometry=geom, fill=0) for i in range(2)]
    from bikv_b200.pool import ShardedPool
    worker.attach_pool(ShardedPool.from_tensors([k.cuda_cache_data for k in kvs], geom, rule=N.SHARD_BLOCK))
    for k in kvs:
        k.stub_factory = G.worker_stub_factory()
    cc = CacheCoordinator(1, base, [0, 1], [0], 16 * 16, 16, ips, None, policy="lru")
    serve(2, lambda s: G.add_InferWorkerServiceServicer_to_server(worker, s))
    for i, k in enumerate(kvs):
        serve(3 + 2 * i, lambda s, k=k: G.add_KVCacheServiceServicer_to_server(k, s))
    serve(1, lambda s: G.add_CacheCoordinatorServiceServicer_to_server(cc, s))
    try:
        with grpc.insecure_channel(f"127.0.0.1:{base + 1}") as ch:
            stub = G.CacheCoordinatorServiceStub(ch)
            stub.StartProcessRequest(pb.StartRequest(msg="go"), timeout=10)
            data = normal(geom.worker_shape(50), geom.dtype, 7)
            worker.compute_buffer[:, :, :50] = data.to(cuda)
            recv = pb.TaskInfoList(tasks=[pb.TaskInfo(request_id=1, id=42, infer_worker=0, token_num=50,
                                                      task_type=SIGNAL_RECV, task_num=1, type="item cache")])
            stub.ReceiveTasksFromInferWorker(recv, timeout=10)
            stub.PollBatchFromInferWorker(recv, timeout=60)
            torch.cuda.synchronize()
            worker.compute_buffer.zero_()
            worker.reset_windows()
            check = pb.TaskInfoList(tasks=[pb.TaskInfo(request_id=2, id=42, infer_worker=0, token_num=50,
                                                       task_type=4, task_num=1, type="item cache")])
            stub.ReceiveTasksFromInferWorker(check, timeout=10)
            reply = stub.PollBatchFromInferWorker(check, timeout=60)
            assert json.loads(reply.msg) == {"2": {"42": 1}}
        torch.cuda.synchronize()
        assert equal_bits(worker.compute_buffer[:, :, :50], data)
        assert sum(k.recv_counter for k in kvs) == 1 and sum(k.send_counter for k in kvs) == 1
    finally:
        cc.stop()
        for s in servers:
            s.stop(0)
