"""The name-compatible ``ipc_service`` module driven the way the reference drives its own
(``SharedMemory/CUDA_Shared/test_page_ipc.py``): a consumer process and a producer process,
both on ONE GPU, talking through a POSIX shared-memory control block and a CUDA IPC handle."""
import os
import subprocess
import sys
import time
import uuid

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

COMMON = """
import os, sys, time
sys.path.insert(0, {root!r})
import numpy as np, torch
from bikv_b200 import ipc_service
from oracle import bikv_oracle as O
name = {name!r}
params = dict(head_size=128, num_kv_heads=2, num_layers=28, kv_pair=2)
token_elems = 128 * 2 * 28 * 2
def dims(page_size, num_pages):
    d = ipc_service.TensorDims()
    d.total_tokens = num_pages * page_size
    d.head_size, d.num_kv_heads, d.num_layers, d.kv_pair = 128, 2, 28, 2
    return d
def random_case():
    # a seeded pool of 40 pages of 16 tokens and a non-identity map of 23 of them
    page_size, pool_pages, n = 16, 40, 23
    g = torch.Generator().manual_seed(11)
    pool = torch.randn((pool_pages * page_size, 128, 2, 28, 2), generator=g).to(torch.float16)
    rng = np.random.default_rng(5)
    src_pages = rng.permutation(pool_pages)[:n]
    dst_slots = rng.permutation(n)
    pe = page_size * token_elems
    return page_size, n, pool, (src_pages * pe).tolist(), (dst_slots * pe).tolist(), pe
"""

CONSUMER = COMMON + """
ipc_service.consumer_init(0, name, 400 << 20)
open({ready!r}, "w").write("ready")
# 1. the reference's own check: 200 pages of 50 tokens, constant 7, identity map
for i in range(2):
    got = ipc_service.consumer_receive(timeout_s=120)
    assert got.dim() == 5 and tuple(got.shape) == (200 * 50, 128, 2, 28, 2), got.shape
    assert got.dtype == torch.float16 and bool((got == 7).all()), "Data corrupted"
# 2. seeded pool, non-identity page map, against the oracle's flat copy
page_size, n, pool, src_off, dst_off, pe = random_case()
got = ipc_service.consumer_receive(timeout_s=120)
assert tuple(got.shape) == (n * page_size, 128, 2, 28, 2)
want = torch.zeros(n * pe, dtype=torch.float16)
O.copy_pages_flat(pool, want, src_off, dst_off, pe)
assert torch.equal(got.cpu().view(-1).view(torch.int16), want.view(torch.int16)), "page map mismatch"
# 3. the same map read zero-copy from a pinned host pool, and a plain tensor, in bf16
got = ipc_service.consumer_receive(timeout_s=120)
assert torch.equal(got.cpu().view(-1).view(torch.int16), want.view(torch.int16)), "zero-copy mismatch"
got = ipc_service.consumer_receive(timeout_s=120)
assert got.dtype == torch.bfloat16 and tuple(got.shape) == (3, 5, 7)
assert torch.equal(got.cpu().view(torch.int16), torch.arange(105, dtype=torch.float32).view(3, 5, 7).to(torch.bfloat16).view(torch.int16))
# 4. nothing more comes: the wait ends by itself
try:
    ipc_service.consumer_receive(timeout_s=0.3)
    raise SystemExit("expected a timeout")
except TimeoutError:
    pass
ipc_service.consumer_cleanup()
assert not os.path.exists("/dev/shm/" + name.lstrip("/"))
print("CONSUMER_OK")
"""

PRODUCER = COMMON + """
ipc_service.producer_init(0, name)
cache = torch.full((200, 50, 128, 2, 28, 2), 7, dtype=torch.float16, device="cuda")
pe = 50 * token_elems
off = torch.tensor([i * pe for i in range(200)], dtype=torch.int64, device="cuda")
for i in range(2):
    ipc_service.producer_copy_pages(cache, off, off, 50, dims(50, 200))
del cache
page_size, n, pool, src_off, dst_off, pe = random_case()
so = torch.tensor(src_off, dtype=torch.int64, device="cuda")
do = torch.tensor(dst_off, dtype=torch.int64, device="cuda")
ipc_service.producer_copy_pages(pool.cuda(), so, do, page_size, dims(page_size, n))
ipc_service.producer_zero_copy_pages(pool.pin_memory(), so, do, page_size, dims(page_size, n))
ipc_service.producer_send(torch.arange(105, dtype=torch.float32).view(3, 5, 7).to(torch.bfloat16).cuda())
ipc_service.producer_cleanup()
print("PRODUCER_OK")
"""


def test_consumer_and_producer_in_two_processes_on_one_gpu(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    name = "/bikv_test_" + uuid.uuid4().hex[:12]
    ready = str(tmp_path / "ready")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0])
    cons = subprocess.Popen([sys.executable, "-c", CONSUMER.format(root=ROOT, name=name, ready=ready)],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    try:
        t0 = time.time()
        while not os.path.exists(ready):
            assert cons.poll() is None, cons.communicate()[0][-3000:]
            assert time.time() - t0 < 180, "consumer did not come up"
            time.sleep(0.05)
        prod = subprocess.run([sys.executable, "-c", PRODUCER.format(root=ROOT, name=name, ready=ready)],
                              capture_output=True, text=True, timeout=300, env=env)
        assert prod.returncode == 0 and "PRODUCER_OK" in prod.stdout, (prod.stdout + prod.stderr)[-3000:]
        out, _ = cons.communicate(timeout=300)
        assert cons.returncode == 0 and "CONSUMER_OK" in out, out[-3000:]
    finally:
        if cons.poll() is None:
            cons.kill()
        try:
            os.unlink("/dev/shm/" + name.lstrip("/"))
        except FileNotFoundError:
            pass


def test_both_sides_in_one_process_still_work(cuda):
    from bikv_b200 import ipc_service
    name = "/bikv_test_" + uuid.uuid4().hex[:12]
    ipc_service.consumer_init(0, name, 1 << 20)
    try:
        ipc_service.producer_init(0, name)
        x = torch.arange(4096, dtype=torch.float16, device=cuda).view(4, 32, 32)
        ipc_service.producer_send(x)
        got = ipc_service.consumer_receive(timeout_s=10)
        assert torch.equal(got, x)
        with pytest.raises(RuntimeError):
            ipc_service.producer_send(torch.zeros(1 << 20, dtype=torch.float16, device=cuda))   # larger than the ring
    finally:
        ipc_service.producer_cleanup()
        ipc_service.consumer_cleanup()
    with pytest.raises(RuntimeError):
        ipc_service.producer_init(0, name)            # the block is gone
