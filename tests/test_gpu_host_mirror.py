"""The host mirror of the reference's call surface on a GPU: KVCache + Worker driven by
TaskInfo messages and a MultiPageManager plan, the ipc_service-compatible module, and
parity with the reference's own compiled kernel when oracle/_ref holds it."""
import importlib.util
import os
import random

import numpy as np
import pytest
import torch

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200 import ipc_service
from bikv_b200 import taskinfo as pb
from bikv_b200.geometry import KVGeometry
from bikv_b200.kvcache import KVCache
from bikv_b200.signals import SIGNAL_RECV, SIGNAL_SEND
from bikv_b200.worker import Worker
from oracle import bikv_oracle as O

from helpers import equal_bits, normal

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_defaults(cuda):
    kv = KVCache(3, 1000, 50, 5000, {}, {}, None, fill=3)
    assert kv.cache_index == 0 and kv.max_pages == 20
    assert tuple(kv.cuda_cache_data.shape) == (1000, 128, 2, 28, 2) and kv.cuda_cache_data.dtype == torch.float16
    assert float(kv.cuda_cache_data[7, 5, 1, 3, 0]) == 3.0
    src, dst = kv.get_index_tensors(4)
    assert src.data_ptr() != dst.data_ptr() and src.numel() == dst.numel() == 4
    w = Worker(2, 5000, 400, 50, 1, {}, {}, None)
    assert w.worker_index == 0 and tuple(w.compute_buffer.shape) == (28, 2, 400, 2, 128)


@pytest.mark.parametrize("layout", [N.POOL_PAGED, N.POOL_TOKEN_MAJOR])
def test_recv_then_send_through_task_messages(cuda, layout):
    """Two shards, one worker: RECV tasks write worker data into pages chosen by the
    MultiPageManager, SEND tasks read them back; pool and buffers checked against the oracle."""
    geom = KVGeometry(3, 2, 64, 16, torch.float16, layout)
    cache_tokens, page = 16 * 24, 16
    kvs = [KVCache(3 + 2 * i, cache_tokens, page, 5000, {}, {}, None, geometry=geom, fill=0) for i in range(2)]
    worker = Worker(2, 5000, 16 * 40, page, 1, {}, {}, None, geometry=geom)
    Worker.connect(kvs, [worker])
    random.seed(0)
    mpm = B.MultiPageManager(cache_tokens, page, 2)
    rnd = random.Random(1)
    items = [(100 + i, rnd.randint(1, 70)) for i in range(9)]
    tasks = {0: [], 1: []}
    for item_id, tokens in items:
        shard, pages = mpm.load_item(item_id, tokens)
        tasks[shard].append(pb.TaskInfo(request_id=7, id=item_id, infer_worker=0, cache_worker=shard,
                                        token_num=tokens, task_type=SIGNAL_RECV, cache_pages_list=pages))
    shards_ref = [torch.zeros(geom.pool_shape(24), dtype=geom.dtype) for _ in range(2)]
    sent = {}
    for shard in (0, 1):
        if not tasks[shard]:
            continue
        total = sum(t.token_num for t in tasks[shard])
        data = normal(geom.worker_shape(total), geom.dtype, 50 + shard)
        worker.reset_windows()
        worker.compute_buffer[:, :, :total] = data.to(cuda)
        conf = kvs[shard].receive_task_info_batch_gprc(tasks[shard])
        assert conf == {7: len(tasks[shard])}
        torch.cuda.synchronize()
        recs = O.plan_records([list(t.cache_pages_list) for t in tasks[shard]],
                              [t.token_num for t in tasks[shard]], page,
                              item_shard=[shard] * len(tasks[shard]), pages_per_shard=24)
        O.scatter(shards_ref, geom, recs, [data], N.SHARD_BLOCK)
        sent[shard] = (data, recs)
    for i in (0, 1):
        assert equal_bits(kvs[i].cuda_cache_data, shards_ref[i])
    assert kvs[0].recv_counter + kvs[1].recv_counter == len(sent)
    # SEND: same items, looked up through access_item, as a ReceiveTasksFromCoordinator call
    for shard, (data, recs) in sent.items():
        worker.compute_buffer.zero_()
        worker.reset_windows()
        msgs = []
        for t in tasks[shard]:
            s, pages = mpm.access_item(t.id)
            assert s == shard
            msgs.append(pb.TaskInfo(request_id=8, id=t.id, infer_worker=0, cache_worker=s, token_num=t.token_num,
                                    task_type=SIGNAL_SEND, cache_pages_list=pages))
        reply = kvs[shard].ReceiveTasksFromCoordinator(pb.TaskInfoList(tasks=msgs), None)
        assert reply.msg == '{"8": %d}' % len(msgs)
        torch.cuda.synchronize()
        total = data.shape[2]
        assert equal_bits(worker.compute_buffer[:, :, :total], data)
        assert int(worker.compute_buffer[:, :, total:].abs().sum()) == 0
    worker.mover.check_status()


def test_one_batch_spread_over_two_shards_keeps_every_item_apart(cuda):
    """A worker whose items sit on two shards receives one combined task per shard, and the
    coordinator runs the shard groups concurrently: each task has its own window of the
    worker's buffer, in both directions, so no group overwrites or re-reads another's tokens."""
    import json

    from bikv_b200.cache_coordinator import CacheCoordinator
    geom = KVGeometry(2, 2, 64, 16, torch.float16)
    page, per = 16, 16
    kvs = [KVCache(3 + 2 * i, per * page, page, 5000, {}, {}, None, geometry=geom, fill=0) for i in range(2)]
    worker = Worker(2, 5000, 16 * 40, page, 1, {}, {}, None, geometry=geom)
    Worker.connect(kvs, [worker])
    addr = {f"127.0.0.1:{5000 + 3 + 2 * i}": kvs[i] for i in range(2)}

    class Local:          # the shard's servicer called in-process
        def __init__(self, kv):
            self.kv = kv

        def ReceiveTasksFromCoordinator(self, request, context=None):
            return self.kv.ReceiveTasksFromCoordinator(request, context)

    cc = CacheCoordinator(1, 5000, [0, 1], [0], per * page, page, {3: "127.0.0.1", 5: "127.0.0.1"}, None, policy="lru",
                          kvcache_stub_factory=lambda a: Local(addr[a]))
    items = [(10, 33), (11, 16), (12, 50), (13, 7), (14, 40), (15, 21)]       # ids chosen to hit both shards
    recv = [pb.TaskInfo(request_id=1, id=i, infer_worker=0, token_num=n, task_type=SIGNAL_RECV, task_num=len(items),
                        type="item cache") for i, n in items]
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=recv), None)
    # Decide first (page placement), so the worker can stage each shard group's tokens in the
    # window that group will read: what the model's prefill does before the RECV tasks run.
    with cc._wake:
        decided = list(cc._queue)
        cc._queue.clear()
        for t in decided:
            cc._decide(t)
    groups = {}
    for t in decided:
        groups.setdefault(t.cache_worker, []).append(t)
    assert len(groups) == 2, "the case must spread over both shards"
    data = {}
    worker.reset_windows()
    for cw, ts in groups.items():
        n = sum(t.token_num for t in ts)
        combined = {"task_type": SIGNAL_RECV, "cache_worker": cw, "id_token_pair": [(t.id, t.token_num) for t in ts]}
        start = worker.reserve_window(combined)
        data[cw] = normal(geom.worker_shape(n), geom.dtype, 70 + cw)
        worker.compute_buffer[:, :, start:start + n] = data[cw].to(cuda)
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(2) as ex:       # the groups run side by side, as process_pending runs them
        list(ex.map(lambda kv_ts: cc._execute(*kv_ts), groups.items()))
    torch.cuda.synchronize()
    shards_ref = [torch.zeros(geom.pool_shape(per), dtype=geom.dtype) for _ in range(2)]
    for cw, ts in groups.items():
        recs = O.plan_records([list(t.cache_pages_list) for t in ts], [t.token_num for t in ts], page,
                              item_shard=[cw] * len(ts), pages_per_shard=per)
        O.scatter(shards_ref, geom, recs, [data[cw]], N.SHARD_BLOCK)
    for i in (0, 1):
        assert equal_bits(kvs[i].cuda_cache_data, shards_ref[i])
    # SEND through the whole coordinator path: CHECK -> hit -> one group per shard, concurrently
    worker.compute_buffer.zero_()
    worker.reset_windows()
    check = [pb.TaskInfo(request_id=2, id=i, infer_worker=0, token_num=n, task_type=4, task_num=len(items),
                         type="item cache") for i, n in items]
    cc.ReceiveTasksFromInferWorker(pb.TaskInfoList(tasks=check), None)
    assert cc.process_pending() == len(items)
    reply = cc.PollBatchFromInferWorker(pb.TaskInfoList(tasks=check), None, timeout_s=10)
    assert set(json.loads(reply.msg)["2"].values()) == {1}
    torch.cuda.synchronize()
    seen = set()
    for cw in groups:
        start, n = worker.windows[(SIGNAL_SEND, cw)]
        assert n == data[cw].shape[2]
        assert equal_bits(worker.compute_buffer[:, :, start:start + n], data[cw])
        seen |= set(range(start, start + n))
    assert len(seen) == sum(n for _, n in items), "windows must not overlap"
    worker.mover.check_status()


def test_worker_servicer_methods_take_combined_messages(cuda):
    geom = KVGeometry(2, 2, 64, 16, torch.bfloat16)
    kv = KVCache(3, 16 * 8, 16, 5000, {}, {}, None, geometry=geom, fill=0)
    w = Worker(2, 5000, 64, 16, 1, {}, {}, None, geometry=geom)
    Worker.connect([kv], [w])
    msg = kv._task_info_json_to_pb({"infer_worker": 0, "cache_worker": 0, "token_num": 37, "task_type": SIGNAL_RECV,
                                    "id_token_pair": [(1, 20), (2, 17)], "cache_pages_list": [[4, 5], [1, 7]]})
    data = normal(geom.worker_shape(37), geom.dtype, 3)
    w.compute_buffer[:, :, :37] = data.to(cuda)
    w.SendKVCacheData(msg, None)
    w.compute_buffer.zero_()
    w.reset_windows()
    w.RecvKVCacheData(msg, None)
    torch.cuda.synchronize()
    assert equal_bits(w.compute_buffer[:, :, :37], data)
    with pytest.raises(B.BikvError):
        w.pull_pages({"infer_worker": 0, "cache_worker": 0, "token_num": 16, "task_type": SIGNAL_SEND,
                      "id_token_pair": [(1, 16)], "cache_pages_list": [[99]]})   # page outside the shard


def test_ipc_service_compat_flow(cuda):
    """The reference's test_page_ipc.py flow, in one process, through the compat module."""
    P, pages = 50, 40
    g = B.GEO_R
    elems = P * g.token_elems
    ipc_service.consumer_cleanup()
    ipc_service.consumer_init(0, b"/bikv_test", 2 * pages * elems * 2)
    ipc_service.producer_init(0, b"/bikv_test")
    try:
        dims = ipc_service.TensorDims()
        dims.total_tokens, dims.head_size, dims.num_kv_heads, dims.num_layers, dims.kv_pair = pages * P, 128, 2, 28, 2
        cache = torch.full((pages, P) + g.token_shape, 7, dtype=torch.float16, device=cuda)
        ident = torch.arange(pages, dtype=torch.int64, device=cuda) * elems
        ipc_service.producer_copy_pages(cache, ident, ident, P, dims)
        out = ipc_service.consumer_receive()
        assert out.dim() == 5 and tuple(out.shape) == (pages * P, 128, 2, 28, 2)
        assert torch.allclose(out, torch.full_like(out, 7))
        # a real permutation with seeded data (what the reference's test cannot detect)
        cache = normal((pages, P) + g.token_shape, torch.float16, 11).to(cuda)
        perm = torch.randperm(pages, generator=torch.Generator().manual_seed(1))
        src = (perm * elems).to(cuda)
        ipc_service.producer_copy_pages(cache, src, ident, P, dims)
        out = ipc_service.consumer_receive()
        assert equal_bits(out.view(pages, -1), cache.view(pages, -1)[perm.to(cuda)])
        t = normal((3, 5, 7), torch.float16, 2).to(cuda)
        ipc_service.producer_send(t)
        assert equal_bits(ipc_service.consumer_receive(), t)
        pinned = normal((pages, elems), torch.float16, 5).pin_memory()
        ipc_service.producer_zero_copy_pages(pinned, src, ident, P, dims)
        assert equal_bits(ipc_service.consumer_receive().view(pages, -1), pinned[perm])
    finally:
        ipc_service.producer_cleanup()
        ipc_service.consumer_cleanup()


def _reference_kernel():
    path = os.path.join(ROOT, "oracle", "_ref", "bikv_ref_kernel.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/bikv_ref_kernel.so not built (needs a reference checkout at build time)")
    spec = importlib.util.spec_from_file_location("bikv_ref_kernel", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("page_size,n_pages", [(50, 64), (16, 200), (1, 7)])
def test_flat_copy_equals_the_reference_kernel(cuda, page_size, n_pages):
    """bikv_copy_pages_flat against the reference's block_per_page_copy_kernel, compiled
    from the reference's own source, on seeded data and a random page map: bit-exact."""
    ref = _reference_kernel()
    g = B.GEO_R
    elems = page_size * g.token_elems
    pool_pages = 2 * n_pages
    cache = normal((pool_pages * page_size,) + g.token_shape, torch.float16, 21).to(cuda)
    rng = np.random.default_rng(page_size)
    src = torch.from_numpy((rng.permutation(pool_pages)[:n_pages] * elems).astype(np.int64)).to(cuda)
    dst = torch.from_numpy((rng.permutation(n_pages) * elems).astype(np.int64)).to(cuda)
    out_ref = torch.zeros(n_pages * elems, dtype=torch.float16, device=cuda)
    shape = ref.ref_copy_pages(cache, src, dst, out_ref, page_size, 128, 2, 28, 2)
    assert list(shape) == [n_pages * page_size, 128, 2, 28, 2]
    out = torch.zeros_like(out_ref)
    B.PageMover(cuda).copy_pages_flat(cache, out, src, dst, elems)
    torch.cuda.synchronize()
    assert equal_bits(out, out_ref)
    cpu = torch.zeros(n_pages * elems, dtype=torch.float16)
    O.copy_pages_flat(cache.cpu(), cpu, src.tolist(), dst.tolist(), elems)
    assert equal_bits(out_ref, cpu), "oracle disagrees with the reference kernel"


def test_token_major_gather_equals_reference_kernel_plus_permute(cuda):
    """Gather from a reference-layout pool = reference kernel (flat pages) followed by the
    layout permutation, for whole pages."""
    ref = _reference_kernel()
    g = KVGeometry(28, 2, 128, 16, torch.float16, N.POOL_TOKEN_MAJOR)
    pool_pages, n = 48, 20
    cache = normal(g.pool_shape(pool_pages), g.dtype, 31).to(cuda)
    rng = np.random.default_rng(3)
    pages = rng.permutation(pool_pages)[:n]
    src = torch.from_numpy((pages * g.page_elems).astype(np.int64)).to(cuda)
    dst = torch.arange(n, dtype=torch.int64, device=cuda) * g.page_elems
    flat = torch.zeros(n * g.page_elems, dtype=g.dtype, device=cuda)
    ref.ref_copy_pages(cache, src, dst, flat, 16, 128, 2, 28, 2)
    want = flat.view((n * 16,) + g.token_shape).permute(3, 4, 0, 2, 1).contiguous()
    plan = B.build_plan([pages.tolist()], [n * 16], 16)
    got = torch.zeros(g.worker_shape(n * 16), dtype=g.dtype, device=cuda)
    B.PageMover(cuda).gather(B.ShardedPool.single(cache, g), plan, got)
    torch.cuda.synchronize()
    assert equal_bits(got, want)


def test_worker_paged_cache_round_trip(cuda):
    """Worker.local_kvcache filled straight from the pool and drained back into other pages."""
    geom = KVGeometry(3, 2, 64, 16, torch.float16)
    kvs = [KVCache(3 + 2 * i, 16 * 10, 16, 5000, {}, {}, None, geometry=geom, fill=0) for i in range(2)]
    w = Worker(2, 5000, 64, 16, 1, {}, {}, None, geometry=geom)
    Worker.connect(kvs, [w])
    w.init_local_kvcache(12)
    kvs[1].cuda_cache_data.copy_(normal(geom.pool_shape(10), geom.dtype, 9).to(cuda))
    task = {"infer_worker": 0, "cache_worker": 1, "token_num": 40, "task_type": SIGNAL_SEND,
            "id_token_pair": [(1, 24), (2, 16)], "cache_pages_list": [[4, 7], [2]]}
    w.pull_pages_to_blocks(task, [9, 0, 5])
    torch.cuda.synchronize()
    pool1 = kvs[1].cuda_cache_data                                    # [10, L, 2, 16, H, D]
    for l in range(geom.n_layers):
        lay = w.local_kvcache[l]
        assert equal_bits(lay[9 * 16:10 * 16], pool1[4, l].permute(1, 0, 2, 3))
        assert equal_bits(lay[0:8], pool1[7, l, :, :8].permute(1, 0, 2, 3))       # 24 tokens: 16 + 8
        assert int(lay[8:16].abs().sum()) == 0
        assert equal_bits(lay[5 * 16:6 * 16], pool1[2, l].permute(1, 0, 2, 3))
    back = {"infer_worker": 0, "cache_worker": 0, "token_num": 40, "task_type": SIGNAL_RECV,
            "id_token_pair": [(1, 24), (2, 16)], "cache_pages_list": [[1, 3], [8]]}
    w.push_pages_from_blocks(back, [9, 0, 5])
    torch.cuda.synchronize()
    pool0 = kvs[0].cuda_cache_data
    assert equal_bits(pool0[1], pool1[4]) and equal_bits(pool0[8], pool1[2])
    assert equal_bits(pool0[3][:, :, :8], pool1[7][:, :, :8]) and int(pool0[3][:, :, 8:].abs().sum()) == 0
