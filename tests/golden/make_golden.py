"""Generates the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/Bi-KV-checkout

It imports the reference's Python modules (``<checkout>/Bi-KV``) and records what
they compute, so the fixtures travel to machines that have no checkout:

  page_manager.json   traces of ``PageManager`` / ``MultiPageManager``
                      (DistributedStorage/PageManager.py) under seeded operations
  plan_offsets.json   the ``src_offsets`` / ``dest_offsets`` arrays that
                      ``KVCache.shared_data_batch_pages`` (DistributedStorage/kvcache.py:132-239)
                      hands to its copy kernel, captured with a stub ``ipc_service``
  task_grouping.json  the combined tasks and confirmation counts that
                      ``KVCache.receive_task_info_batch_gprc`` (kvcache.py:368-459) builds,
                      with the serialised ``CombindedTaskInfo`` bytes of
                      ``_task_info_json_to_pb`` (kvcache.py:467-475)
"""
import json
import os
import random
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    sys.argv = ["x"]  # the reference's config.py parses argv at import
    sys.path.insert(0, os.path.join(root, "Bi-KV"))
    captured = {}

    ipc = types.ModuleType("ipc_service")

    class TensorDims:
        pass

    def producer_copy_pages(src, src_off, dst_off, page_size, dims):
        captured["src_offsets"] = src_off.tolist()
        captured["dest_offsets"] = dst_off.tolist()
        captured["page_size"] = page_size
        captured["total_tokens"] = dims.total_tokens

    ipc.TensorDims = TensorDims
    ipc.producer_copy_pages = producer_copy_pages
    sys.modules["ipc_service"] = ipc
    rdma = types.ModuleType("rdma_onesided_transport")
    rdma.RDMAOneSidedEndpoint = object
    sys.modules["rdma_onesided_transport"] = rdma
    model = types.ModuleType("Model")
    qwen = types.ModuleType("Model.qwen2")
    qwen.token_shape = (128, 2, 28, 2)
    qwen.model_params = {"head_size": 128, "num_q_heads": 12, "num_kv_heads": 2, "num_layers": 28}
    model.qwen2 = qwen
    sys.modules["Model"] = model
    sys.modules["Model.qwen2"] = qwen
    return captured


def page_manager_traces():
    import DistributedStorage.PageManager as ref

    traces = []
    for seed, (cache, page) in enumerate([(32, 4), (256, 16), (1000, 50), (4096, 16), (640, 16)]):
        rnd = random.Random(seed)
        pm = ref.PageManager(cache, page)
        ops = []
        for _ in range(300):
            iid = rnd.randrange(24)
            x = rnd.random()
            if x < 0.6:
                ln = rnd.randint(1, max(2, cache // 3))
                try:
                    res = pm.load_item(iid, ln)
                    ops.append(["load", iid, ln, [list(res[0]), list(res[1])]])
                except Exception as e:  # noqa: BLE001
                    ops.append(["load", iid, ln, type(e).__name__])
            elif x < 0.85:
                try:
                    ops.append(["access", iid, 0, list(pm.access_item(iid))])
                except Exception as e:  # noqa: BLE001
                    ops.append(["access", iid, 0, type(e).__name__])
            elif x < 0.93:
                try:
                    pm.set_protected(iid)
                    ops.append(["protect", iid, 0, None])
                except KeyError:
                    ops.append(["protect", iid, 0, "KeyError"])
            else:
                if iid in pm.page_table and pm.page_table[iid]["protected"] > 0:
                    pm.remove_protected(iid)
                    ops.append(["unprotect", iid, 0, None])
        traces.append({"kind": "single", "cache_size": cache, "page_size": page, "ops": ops,
                       "loaded": pm.get_loaded_lists(), "free": list(pm.free_pages)})
    for seed, (cache, page, k) in enumerate([(256, 16, 2), (1024, 16, 4), (4000, 50, 3)]):
        rnd = random.Random(100 + seed)
        ref.random.seed(seed)
        mpm = ref.MultiPageManager(cache, page, k)
        ops = []
        for _ in range(400):
            iid = rnd.randrange(50)
            if rnd.random() < 0.6:
                ln = rnd.randint(1, cache // 3)
                try:
                    res = mpm.load_item(iid, ln)
                    ops.append(["load", iid, ln, [res[0], list(res[1])]])
                except Exception as e:  # noqa: BLE001
                    ops.append(["load", iid, ln, type(e).__name__])
            else:
                s, pages = mpm.access_item(iid)
                ops.append(["access", iid, 0, [s, None if pages is None else list(pages)]])
        traces.append({"kind": "multi", "cache_size": cache, "page_size": page, "shards": k,
                       "random_seed": seed, "ops": ops})
    # The reference's own __main__ demo sequence (PageManager.py:164-203).
    pm = ref.PageManager(cache_size=32, page_size=4)
    demo = []
    for name, ln in (("A", 5), ("B", 7)):
        r = pm.load_item(name, ln)
        demo.append([name, ln, [list(r[0]), list(r[1])], pm.get_loaded_lists()])
    pm.access_item("A")
    for name, ln in (("C", 20), ("D", 30)):
        try:
            r = pm.load_item(name, ln)
            demo.append([name, ln, [list(r[0]), list(r[1])], pm.get_loaded_lists()])
        except Exception as e:  # noqa: BLE001
            demo.append([name, ln, type(e).__name__, pm.get_loaded_lists()])
    traces.append({"kind": "demo", "ops": demo})
    return traces


def plan_offsets(captured):
    import torch
    from DistributedStorage.kvcache import KVCache

    import DistributedStorage.kvcache as kvmod
    kvmod.SM_DEBUG = 0
    cases = []
    rnd = random.Random(7)
    for page_size in (16, 50):
        for _ in range(6):
            kv = KVCache.__new__(KVCache)
            kv.rank, kv.page_size, kv.device = 3, page_size, torch.device("cpu")
            kv.max_pages = 4096
            kv.src_index_pool = torch.empty(kv.max_pages, dtype=torch.int64)
            kv.dst_index_pool = torch.empty(kv.max_pages, dtype=torch.int64)
            kv.cuda_cache_data = torch.zeros(1)
            n_items = rnd.randint(1, 6)
            pairs, pages, next_page = [], [], rnd.randint(0, 100)
            for it in range(n_items):
                tok = rnd.choice([1, page_size - 1, page_size, page_size + 1, 3 * page_size,
                                  rnd.randint(1, 20 * page_size)])
                n = (tok + page_size - 1) // page_size
                ids = rnd.sample(range(4096), n)
                pairs.append((it + 10, tok))
                pages.append(ids)
            task = {"infer_worker": 0, "cache_worker": 0, "token_num": sum(p[1] for p in pairs),
                    "task_type": 1, "id_token_pair": pairs, "cache_pages_list": pages}
            kv.shared_data_batch_pages(task)
            cases.append({"page_size": page_size, "id_token_pair": pairs, "cache_pages_list": pages,
                          "src_offsets": captured["src_offsets"], "dest_offsets": captured["dest_offsets"],
                          "total_tokens": captured["total_tokens"]})
    return cases


def task_grouping():
    from DistributedStorage.kvcache import KVCache
    from protos import TaskInfo_pb2

    class FakeFuture:
        def result(self):
            return None

    sent = []

    class FakeStub:
        def __init__(self, channel):
            pass

        class _M:
            def __init__(self, kind):
                self.kind = kind

            def future(self, pb):
                sent.append([self.kind, pb.SerializeToString().hex()])
                return FakeFuture()

        RecvKVCacheData = _M("RecvKVCacheData")
        SendKVCacheData = _M("SendKVCacheData")

    import DistributedStorage.kvcache as kvmod
    kvmod.TaskInfo_pb2_grpc.InferWorkerServiceStub = FakeStub

    class Pool:
        def get_channel(self, addr):
            return addr

    cases = []
    rnd = random.Random(11)
    for _ in range(5):
        kv = KVCache.__new__(KVCache)
        kv.rank, kv.master_port, kv.send_counter, kv.recv_counter = 3, 5000, 0, 0
        kv.rank_to_ip_grpc = {r: "127.0.0.1" for r in range(12)}
        kv.channelpool = Pool()
        kv.send_data_batch = lambda t: None
        kv.receive_data_batch = lambda t: None
        tasks, plain = [], []
        for i in range(rnd.randint(1, 12)):
            d = dict(request_id=rnd.randint(1, 4), id=rnd.choice([-1, rnd.randint(0, 99)]),
                     infer_worker=rnd.randint(0, 2), cache_worker=0, token_num=rnd.randint(1, 200),
                     index=i, task_type=rnd.choice([1, 2, 5]), type=rnd.choice(["user cache", "item cache"]),
                     task_num=0, weight=1, cache_pages_list=[rnd.randint(0, 500) for _ in range(rnd.randint(1, 5))])
            plain.append(d)
            tasks.append(TaskInfo_pb2.TaskInfo(**d))
        del sent[:]
        conf = kv.receive_task_info_batch_gprc(tasks)
        cases.append({"tasks": plain, "confirmation": {str(k): v for k, v in conf.items()}, "sent": list(sent),
                      "send_counter": kv.send_counter, "recv_counter": kv.recv_counter})
    return cases


def main():
    # The reference checkout: first argument, else $BIKV_REFERENCE_ROOT, else a directory named
    # "reference" beside this repository.
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BIKV_REFERENCE_ROOT") or \
        os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
    captured = load_reference(root)
    out = {
        "page_manager.json": page_manager_traces(),
        "plan_offsets.json": plan_offsets(captured),
        "task_grouping.json": task_grouping(),
    }
    for name, data in out.items():
        with open(os.path.join(HERE, name), "w") as f:
            json.dump(data, f, separators=(",", ":"))
        print(name, os.path.getsize(os.path.join(HERE, name)), "bytes")


if __name__ == "__main__":
    main()
