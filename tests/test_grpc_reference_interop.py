"""Wire compatibility with the reference's GENERATED gRPC code (``Bi-KV/protos/TaskInfo_pb2.py``,
``TaskInfo_pb2_grpc.py``; service and method paths of ``protos/TaskInfo.proto:68-89``, fields
``weight = 10`` and ``cache_pages_list = 11``): the reference's stubs call this repository's
servicers, and this repository's stubs call servicers derived from the reference's generated base
classes.  Needs a checkout of the reference (``$BIKV_REFERENCE_ROOT``, or a directory named
``reference`` beside this repository); skipped without one.  Runs in a child process so that the
reference's generated descriptors do not meet this package's in the test process."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("BIKV_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
PROTOS = os.path.join(REF, "Bi-KV", "protos", "TaskInfo_pb2_grpc.py")

SCRIPT = r"""
import sys, json
sys.argv = ['x']
sys.path.insert(0, {ref!r}); sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
from concurrent import futures
import grpc
from protos import TaskInfo_pb2 as rpb, TaskInfo_pb2_grpc as rgrpc       # the reference's generated code
from bikv_b200 import grpc_services as G, taskinfo as pb
from bikv_b200.cache_coordinator import CacheCoordinator
from bikv_b200.kvcache import KVCache
from bikv_b200.signals import SIGNAL_CHECK, SIGNAL_RECV, SIGNAL_SEND

def serve(register):
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=4))
    register(server)
    port = server.add_insecure_port("127.0.0.1:0")
    server.start()
    return server, f"127.0.0.1:{{port}}"

# 1. reference KVCacheServiceStub -> this repository's KVCache servicer (data methods stubbed: no GPU here)
kv = KVCache.__new__(KVCache)
kv.rank, kv.master_port, kv.send_counter, kv.recv_counter = 3, 5000, 0, 0
kv.workers, kv.stub_factory, kv.server = {{}}, None, None
seen = []
kv.send_data_batch = lambda t: seen.append(("send", t["infer_worker"], t["id_token_pair"], [list(p) for p in t["cache_pages_list"]]))
kv.receive_data_batch = lambda t: seen.append(("recv", t["infer_worker"], t["id_token_pair"], [list(p) for p in t["cache_pages_list"]]))
server, addr = serve(lambda s: G.add_KVCacheServiceServicer_to_server(kv, s))
with grpc.insecure_channel(addr) as ch:
    stub = rgrpc.KVCacheServiceStub(ch)
    tasks = rpb.TaskInfoList(tasks=[
        rpb.TaskInfo(request_id=1, id=10, infer_worker=0, cache_worker=0, token_num=20, task_type=SIGNAL_SEND, weight=3,
                     type="user cache", cache_pages_list=[4, 5]),
        rpb.TaskInfo(request_id=1, id=11, infer_worker=0, cache_worker=0, token_num=16, task_type=SIGNAL_SEND,
                     cache_pages_list=[9]),
        rpb.TaskInfo(request_id=2, id=12, infer_worker=1, cache_worker=0, token_num=40, task_type=SIGNAL_RECV,
                     cache_pages_list=[1, 2, 3]),
        rpb.TaskInfo(request_id=2, id=-1, infer_worker=1, task_type=SIGNAL_RECV)])
    reply = stub.ReceiveTasksFromCoordinator(tasks, timeout=20)
    assert isinstance(reply, rpb.ComfirmationMessage)
    assert json.loads(reply.msg) == {{"1": 2, "2": 1}}, reply.msg
    assert seen == [("send", 0, [(10, 20), (11, 16)], [[4, 5], [9]]), ("recv", 1, [(12, 40)], [[1, 2, 3]])], seen
server.stop(0)

# 2. this repository's stubs -> servicers derived from the reference's generated base classes
class RefKV(rgrpc.KVCacheServiceServicer):
    def ReceiveTasksFromCoordinator(self, request, context):
        t = request.tasks[0]
        return rpb.ComfirmationMessage(msg=json.dumps({{"n": len(request.tasks), "pages": list(t.cache_pages_list),
                                                       "w": t.weight, "type": t.type, "task_num": t.task_num}}))
class RefWorker(rgrpc.InferWorkerServiceServicer):
    def RecvKVCacheData(self, request, context):
        got.append((request.infer_worker, request.cache_worker, request.token_num, request.task_type,
                    [(p.id, p.token_num) for p in request.id_token_pair],
                    [list(p.cache_pages_list) for p in request.cache_pages_list]))
        return rpb.Empty()
got = []
server, addr = serve(lambda s: (rgrpc.add_KVCacheServiceServicer_to_server(RefKV(), s),
                                rgrpc.add_InferWorkerServiceServicer_to_server(RefWorker(), s)))
with grpc.insecure_channel(addr) as ch:
    r = G.KVCacheServiceStub(ch).ReceiveTasksFromCoordinator(
        pb.TaskInfoList(tasks=[pb.TaskInfo(id=3, weight=7, type="item cache", task_num=5, cache_pages_list=[1, 2, 3])]), timeout=20)
    assert json.loads(r.msg) == {{"n": 1, "pages": [1, 2, 3], "w": 7, "type": "item cache", "task_num": 5}}, r.msg
    m = KVCache._task_info_json_to_pb(kv, {{"infer_worker": 2, "cache_worker": 1, "token_num": 37, "task_type": SIGNAL_SEND,
                                           "id_token_pair": [(1, 20), (2, 17)], "cache_pages_list": [[4, 5], [1, 7]]}})
    G.InferWorkerServiceStub(ch).RecvKVCacheData(m, timeout=20)
    assert got == [(2, 1, 37, SIGNAL_SEND, [(1, 20), (2, 17)], [[4, 5], [1, 7]])], got
server.stop(0)

# 3. reference CacheCoordinatorServiceStub -> this repository's coordinator (shard stood in for)
class FakeShard:
    def __init__(self):
        self.seen = []
    def ReceiveTasksFromCoordinator(self, request, context=None):
        conf = {{}}
        for t in request.tasks:
            self.seen.append((t.request_id, t.id, t.task_type, len(t.cache_pages_list)))
            conf[t.request_id] = conf.get(t.request_id, 0) + 1
        return pb.ComfirmationMessage(msg=json.dumps(conf))
shard = FakeShard()
cc = CacheCoordinator(1, 5000, [0], [0], 1024, 16, {{3: "127.0.0.1"}}, None, kvcache_stub_factory=lambda a: shard)
server, addr = serve(lambda s: G.add_CacheCoordinatorServiceServicer_to_server(cc, s))
with grpc.insecure_channel(addr) as ch:
    stub = rgrpc.CacheCoordinatorServiceStub(ch)
    stub.StartProcessRequest(rpb.StartRequest(msg="x"), timeout=20)
    t = rpb.TaskInfoList(tasks=[rpb.TaskInfo(request_id=1, id=7, token_num=40, task_type=SIGNAL_RECV, task_num=1,
                                             type="user cache", weight=1)])
    stub.ReceiveTasksFromInferWorker(t, timeout=20)
    assert json.loads(stub.PollBatchFromInferWorker(t, timeout=30).msg) == {{"1": None}}
    q = rpb.TaskInfoList(tasks=[rpb.TaskInfo(request_id=2, id=7, token_num=40, task_type=SIGNAL_CHECK, task_num=2),
                                rpb.TaskInfo(request_id=2, id=8, token_num=11, task_type=SIGNAL_CHECK, task_num=2)])
    assert json.loads(stub.ReceiveTasksFromScheduler(q, timeout=20).msg) == {{"2": {{"user miss": 0, "item miss": 11}}}}
    stub.ReceiveTasksFromInferWorker(q, timeout=20)
    assert json.loads(stub.PollBatchFromInferWorker(q, timeout=30).msg) == {{"2": {{"7": 1, "8": 0}}}}
assert shard.seen[0] == (1, 7, SIGNAL_RECV, 3) and (2, 7, SIGNAL_SEND, 3) in shard.seen, shard.seen
cc.stop(); server.stop(0)
print("INTEROP_OK")
"""


@pytest.mark.skipif(not os.path.exists(PROTOS), reason="no checkout of the reference's generated gRPC code")
def test_reference_generated_stubs_and_servicers_interoperate():
    script = SCRIPT.format(ref=os.path.join(REF, "Bi-KV"), root=ROOT, tests=os.path.join(ROOT, "tests"))
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "INTEROP_OK" in res.stdout, (res.stdout + res.stderr)[-4000:]
