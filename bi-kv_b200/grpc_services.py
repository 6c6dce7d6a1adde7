"""gRPC plumbing for the three services of ``protos/TaskInfo.proto:68-89``, built on the
messages of ``taskinfo.py`` -- no generated code.  Method paths and wire format are the
reference's (``/KVCacheService/ReceiveTasksFromCoordinator`` and so on: the proto has no
package), so a reference scheduler, coordinator or worker can call a servicer registered
here and the stubs here can call a reference process.

    server = grpc.server(ThreadPoolExecutor(max_workers=20))
    add_KVCacheServiceServicer_to_server(kvcache, server)       # kvcache: bikv_b200.kvcache.KVCache
    add_InferWorkerServiceServicer_to_server(worker, server)    # worker:  bikv_b200.worker.Worker
    server.add_insecure_port(f"[::]:{master_port + rank}")      # port convention of rpc_def.py
"""
from __future__ import annotations

import grpc

from . import taskinfo as pb

_SERVICES = {
    "InferWorkerService": {
        "ReceiveTasksFromScheduler": (pb.TaskInfoList, pb.Empty),
        "StartWriteCacheData": (pb.TaskInfoList, pb.Empty),
        "SendKVCacheData": (pb.CombindedTaskInfo, pb.Empty),
        "RecvKVCacheData": (pb.CombindedTaskInfo, pb.Empty),
        "ShutDown": (pb.Empty, pb.Empty),
    },
    "CacheCoordinatorService": {
        "ReceiveTasksFromInferWorker": (pb.TaskInfoList, pb.Empty),
        "ReceiveTasksFromScheduler": (pb.TaskInfoList, pb.ComfirmationMessage),
        "PollBatchFromInferWorker": (pb.TaskInfoList, pb.ComfirmationMessage),
        "StartProcessRequest": (pb.StartRequest, pb.Empty),
        "ShutDown": (pb.Empty, pb.Empty),
    },
    "KVCacheService": {
        "ReceiveTasksFromCoordinator": (pb.TaskInfoList, pb.ComfirmationMessage),
        "ShutDown": (pb.Empty, pb.Empty),
    },
}


def _unimplemented(name):
    def handler(request, context):
        context.abort(grpc.StatusCode.UNIMPLEMENTED, f"{name} is not implemented by this servicer")
    return handler


def _add(service: str, servicer, server) -> None:
    handlers = {}
    for method, (req, resp) in _SERVICES[service].items():
        fn = getattr(servicer, method, None) or _unimplemented(f"{service}.{method}")
        handlers[method] = grpc.unary_unary_rpc_method_handler(
            fn, request_deserializer=req.FromString, response_serializer=resp.SerializeToString)
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(service, handlers),))


def add_InferWorkerServiceServicer_to_server(servicer, server) -> None:
    _add("InferWorkerService", servicer, server)


def add_CacheCoordinatorServiceServicer_to_server(servicer, server) -> None:
    _add("CacheCoordinatorService", servicer, server)


def add_KVCacheServiceServicer_to_server(servicer, server) -> None:
    _add("KVCacheService", servicer, server)


class _Stub:
    _service = ""

    def __init__(self, channel):
        for method, (req, resp) in _SERVICES[self._service].items():
            setattr(self, method, channel.unary_unary(f"/{self._service}/{method}",
                                                      request_serializer=req.SerializeToString,
                                                      response_deserializer=resp.FromString))


class InferWorkerServiceStub(_Stub):
    _service = "InferWorkerService"


class CacheCoordinatorServiceStub(_Stub):
    _service = "CacheCoordinatorService"


class KVCacheServiceStub(_Stub):
    _service = "KVCacheService"


def worker_stub_factory():
    """For ``KVCache.stub_factory``: address -> InferWorkerService stub, one channel per
    address (the reference's ChannelPool, ``Utils/channelpool.py:5-31``)."""
    channels = {}

    def factory(address: str):
        if address not in channels:
            channels[address] = grpc.insecure_channel(address)
        return InferWorkerServiceStub(channels[address])
    return factory
