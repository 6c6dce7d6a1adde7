"""Wire messages of the control plane, built at import time.

The schema is the one the reference's generated code carries
(``protos/TaskInfo_pb2.py``; note ``TaskInfo.weight = 10`` and
``TaskInfo.cache_pages_list = 11``, which the ``.proto`` text beside it lacks), so a
message serialised here parses in a reference process and the reverse.  The file
descriptor is assembled programmatically -- no ``protoc`` is needed -- and lives in a
private descriptor pool so that it never collides with the reference's own
``TaskInfo.proto`` registration when both are imported in one process.
"""
from google.protobuf import descriptor_pb2 as _d
from google.protobuf import descriptor_pool as _pool
from google.protobuf import message_factory as _mf

_I32, _STR, _MSG = _d.FieldDescriptorProto.TYPE_INT32, _d.FieldDescriptorProto.TYPE_STRING, \
    _d.FieldDescriptorProto.TYPE_MESSAGE
_OPT, _REP = _d.FieldDescriptorProto.LABEL_OPTIONAL, _d.FieldDescriptorProto.LABEL_REPEATED


def _message(fd, name, fields):
    m = fd.message_type.add()
    m.name = name
    for fname, number, ftype, label, type_name in fields:
        f = m.field.add()
        f.name, f.number, f.type, f.label = fname, number, ftype, label
        if type_name:
            f.type_name = type_name


def _build():
    fd = _d.FileDescriptorProto()
    fd.name = "TaskInfo.proto"
    fd.syntax = "proto3"
    common = [("request_id", 1), ("id", 2), ("infer_worker", 3), ("cache_worker", 4), ("token_num", 5),
              ("index", 6), ("task_type", 7)]
    head = [(n, i, _I32, _OPT, None) for n, i in common] + [("type", 8, _STR, _OPT, None),
                                                            ("task_num", 9, _I32, _OPT, None)]
    _message(fd, "IdTokenPair", [("id", 1, _I32, _OPT, None), ("token_num", 2, _I32, _OPT, None)])
    _message(fd, "TaskInfo", head + [("weight", 10, _I32, _OPT, None),
                                     ("cache_pages_list", 11, _I32, _REP, None)])
    _message(fd, "CombindedTaskInfo", head + [("cache_pages_list", 10, _MSG, _REP, ".PageList"),
                                              ("id_token_pair", 11, _MSG, _REP, ".IdTokenPair")])
    _message(fd, "PageList", [("cache_pages_list", 1, _I32, _REP, None)])
    _message(fd, "TaskInfoList", [("tasks", 1, _MSG, _REP, ".TaskInfo")])
    _message(fd, "ComfirmationMessage", [("msg", 1, _STR, _OPT, None)])
    _message(fd, "Empty", [])
    _message(fd, "StartRequest", [("msg", 1, _STR, _OPT, None)])
    pool = _pool.DescriptorPool()
    file_desc = pool.Add(fd) or pool.FindFileByName(fd.name)
    return {n: _mf.GetMessageClass(file_desc.message_types_by_name[n]) for n in
            ("IdTokenPair", "TaskInfo", "CombindedTaskInfo", "PageList", "TaskInfoList",
             "ComfirmationMessage", "Empty", "StartRequest")}


_classes = _build()
IdTokenPair = _classes["IdTokenPair"]
TaskInfo = _classes["TaskInfo"]
CombindedTaskInfo = _classes["CombindedTaskInfo"]
PageList = _classes["PageList"]
TaskInfoList = _classes["TaskInfoList"]
ComfirmationMessage = _classes["ComfirmationMessage"]
Empty = _classes["Empty"]
StartRequest = _classes["StartRequest"]

# gRPC method paths of the three services (protos/TaskInfo.proto:68-89).
KVCACHE_SERVICE = "/KVCacheService"
INFER_WORKER_SERVICE = "/InferWorkerService"
COORDINATOR_SERVICE = "/CacheCoordinatorService"
