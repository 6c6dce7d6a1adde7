"""Two or more GPUs: peer-mapped shards in one process, and CUDA-IPC-mapped shards
across processes (one rank per GPU), both against the CPU oracle.  Skipped on a
single-GPU machine."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

import bikv_b200 as B
from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import build_plan
from oracle import bikv_oracle as O

from helpers import equal_bits, make_shards, make_workers, random_plan

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_gpus(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("variant", [N.VARIANT_LDST, N.VARIANT_BULK])
@pytest.mark.parametrize("worker_gpu", [0, 1])
def test_peer_mapped_shards_in_one_process(variant, worker_gpu):
    _need_gpus(2)
    n = min(torch.cuda.device_count(), 4)
    g = KVGeometry(4, 2, 128, 16, torch.bfloat16)
    per = 24
    rng = np.random.default_rng(worker_gpu)
    lists, tokens = random_plan(rng, g, n * per, 5, 150)
    plan = build_plan([l.tolist() for l in lists], tokens.astype(np.int32), 16,
                      item_request=np.arange(5, dtype=np.int32), n_requests=5)
    recs = [tuple(r) for r in plan.table.tolist()]
    shards_cpu = make_shards(g, n, per, 3, fill="bits")
    shards_gpu = [s.to(f"cuda:{i}") for i, s in enumerate(shards_cpu)]
    dev = torch.device(f"cuda:{worker_gpu}")
    with torch.cuda.device(dev):
        pool = B.ShardedPool.from_tensors(shards_gpu, g, device=dev)
        mover = B.PageMover(dev)
        out = make_workers(g, tokens, dev)
        mover.gather(pool, plan, out, variant=variant)
        ref = make_workers(g, tokens)
        O.gather(shards_cpu, g, recs, ref)
        torch.cuda.synchronize(dev)
        for a, b in zip(out, ref):
            assert equal_bits(a, b)
        src_cpu = make_workers(g, tokens, fill="normal", seed=9)
        mover.scatter(pool, plan, [t.to(dev) for t in src_cpu], variant=variant)
        torch.cuda.synchronize(dev)
        mover.check_status()
    O.scatter(shards_cpu, g, recs, src_cpu)
    for a, b in zip(shards_gpu, shards_cpu):
        assert equal_bits(a, b)


RANK_SCRIPT = """
import os, sys
sys.path.insert(0, {root!r})
sys.path.insert(0, os.path.join({root!r}, "tests"))
import numpy as np, torch, torch.distributed as dist
import bikv_b200 as B
from bikv_b200 import _native as N, multi
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import build_plan
from oracle import bikv_oracle as O
from helpers import equal_bits, make_shards, make_workers, random_plan

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device(f"cuda:{{rank}}")
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=rank, world_size=world)
g = KVGeometry(4, 2, 128, 16, torch.bfloat16)
per = 32
shards_cpu = make_shards(g, world, per, 5, fill="bits")          # every rank can rebuild every shard
mine = shards_cpu[rank].to(dev)
pool = B.ShardedPool.exchange(mine, g)
# disjoint pages per rank: rank r owns global ids r*per*... slices of one permutation
perm = np.random.default_rng(0).permutation(world * per)
share = perm[rank * per:(rank + 1) * per]
tokens = np.array([100, 37, 16 * 8])
counts = (tokens + 15) // 16
lists, at = [], 0
for c in counts:
    lists.append(share[at:at + c].tolist()); at += c
plan = build_plan(lists, tokens.astype(np.int32), 16, item_request=np.arange(3, dtype=np.int32), n_requests=3)
recs = [tuple(r) for r in plan.table.tolist()]
mover = B.PageMover(dev)
for variant in (N.VARIANT_LDST, N.VARIANT_BULK):
    out = make_workers(g, tokens, dev)
    mover.gather(pool, plan, out, variant=variant)
    ref = make_workers(g, tokens)
    O.gather(shards_cpu, g, recs, ref)
    torch.cuda.synchronize()
    assert all(equal_bits(a, b) for a, b in zip(out, ref)), "gather mismatch"
multi.host_barrier(timeout_s=60)
src_cpu = make_workers(g, tokens, fill="normal", seed=100 + rank)
mover.scatter(pool, plan, [t.to(dev) for t in src_cpu])
torch.cuda.synchronize()
mover.check_status()
multi.host_barrier(timeout_s=60)            # every rank's writes have landed
everyone = [None] * world
dist.all_gather_object(everyone, (recs, [t.view(torch.int16).numpy() for t in src_cpu]))
for r_recs, r_src in everyone:
    O.scatter(shards_cpu, g, r_recs, [torch.from_numpy(a).view(torch.bfloat16) for a in r_src])
assert equal_bits(mine, shards_cpu[rank]), "scatter mismatch on shard %d" % rank
remote = sum(1 for r in recs if r[0] % world != rank)
print("RANK_OK", rank, "remote pages", remote, "of", len(recs))
multi.host_barrier(timeout_s=60)
pool.close()
dist.destroy_process_group()
"""


def test_ipc_mapped_shards_across_processes():
    _need_gpus(2)
    world = min(torch.cuda.device_count(), 4)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = textwrap.dedent(RANK_SCRIPT).format(root=ROOT, port=port)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for r, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        assert p.returncode == 0 and "RANK_OK" in out, f"rank {r}:\n{out[-3000:]}"


def test_nvlink_ceilings_report():
    """Reference points for the NVLink fractions: one contiguous 4 GiB range moved by
    bikv_copy_range between two GPUs, pulled (loads from the peer) and pushed (stores
    to the peer), one direction at a time and both directions at once.  Prints GB/s per
    direction (run pytest with -s); asserts only that peer traffic is in an NVLink range."""
    _need_gpus(2)
    import ctypes as C
    import time

    lib = N.lib()
    n = 4 << 30
    buf = {d: [torch.zeros(n, dtype=torch.uint8, device=f"cuda:{d}") for _ in range(2)] for d in (0, 1)}
    N.check(lib.bikv_enable_peer(0, 1))
    N.check(lib.bikv_enable_peer(1, 0))
    streams = {d: torch.cuda.Stream(device=f"cuda:{d}") for d in (0, 1)}

    def copy(dev, dst, src):
        with torch.cuda.device(dev):
            N.check(lib.bikv_copy_range(C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), n,
                                        C.c_void_p(streams[dev].cuda_stream)))

    def rate(fn, iters=4):
        fn()
        torch.cuda.synchronize(0), torch.cuda.synchronize(1)
        t = time.perf_counter()
        for _ in range(iters):
            fn()
        torch.cuda.synchronize(0), torch.cuda.synchronize(1)
        return n * iters / (time.perf_counter() - t) / 1e9

    results = {
        "pull, one direction": rate(lambda: copy(0, buf[0][0], buf[1][0])),
        "pull, both directions": rate(lambda: (copy(0, buf[0][0], buf[1][0]), copy(1, buf[1][1], buf[0][1]))),
        "push, one direction": rate(lambda: copy(0, buf[1][0], buf[0][0])),
        "push, both directions": rate(lambda: (copy(0, buf[1][0], buf[0][0]), copy(1, buf[0][1], buf[1][1]))),
    }
    print()
    for k, v in results.items():
        print(f"[nvlink ceiling] contiguous {k}: {v:.1f} GB/s per direction")
    assert all(v > 100 for v in results.values())


PUSH_SCRIPT = """
import ctypes as C, os, sys
sys.path.insert(0, {root!r})
sys.path.insert(0, os.path.join({root!r}, "tests"))
import numpy as np, torch, torch.distributed as dist
import bikv_b200 as B
from bikv_b200 import _native as N, multi
from bikv_b200.geometry import KVGeometry
from bikv_b200.plan import Plan, build_plan
from bikv_b200.pool import ShardedPool
from bikv_b200.push import split_plans_by_owner
from oracle import bikv_oracle as O
from helpers import equal_bits, make_shards, make_workers

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device(f"cuda:{{rank}}")
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=rank, world_size=world)
g = KVGeometry(4, 2, 128, 16, torch.bfloat16)
per = 32
shards_cpu = make_shards(g, world, per, 5, fill="bits")
mine = shards_cpu[rank].to(dev)
pool = ShardedPool.exchange(mine, g)
perm = np.random.default_rng(0).permutation(world * per)
tokens = np.array([100, 37, 16 * 8])
counts = (tokens + 15) // 16
tables = []
for r in range(world):                      # every rank can write down every worker's plan
    share, lists, at = perm[r * per:(r + 1) * per], [], 0
    for c in counts:
        lists.append(share[at:at + c].tolist()); at += c
    tables.append(build_plan(lists, tokens.astype(np.int32), 16, item_request=[0, 1, 2], n_requests=3).table.copy())
# worker tensors of this rank in one arena, mapped by everyone
elems = [g.token_elems * int(t) for t in tokens]
offs = np.concatenate([[0], np.cumsum(elems)[:-1]])
arena = torch.zeros(int(sum(elems)), dtype=g.dtype, device=dev)
handles = [None] * world
dist.all_gather_object(handles, ShardedPool.export_handle(arena))
bases, maps = [], []
for r, h in enumerate(handles):
    if r == rank:
        bases.append(arena.data_ptr()); continue
    out = C.c_void_p()
    N.check(N.lib().bikv_pool_import(h[0], int(h[1]), C.byref(out)))
    bases.append(int(out.value)); maps.append((int(out.value), int(h[1])))
reqs = torch.empty((3 * world, 2), dtype=torch.int64).pin_memory()
for r in range(world):
    for i in range(3):
        reqs[3 * r + i, 0] = bases[r] + int(offs[i]) * 2
        reqs[3 * r + i, 1] = int(tokens[i])
push = split_plans_by_owner(tables, [3] * world, rank, world, per)
mover = B.PageMover(dev)
for variant in (N.VARIANT_LDST, N.VARIANT_BULK):
    arena.zero_()
    torch.cuda.synchronize()
    multi.host_barrier(timeout_s=60)
    mover.gather_table(pool, Plan.from_table(push, 3 * world), reqs, variant=variant)     # owner pushes
    torch.cuda.synchronize()
    mover.check_status()
    multi.host_barrier(timeout_s=60)              # every owner's stores have landed
    ref = make_workers(g, tokens)
    O.gather(shards_cpu, g, [tuple(x) for x in tables[rank].tolist()], ref)
    for i in range(3):
        got = arena[int(offs[i]):int(offs[i]) + elems[i]].view(g.worker_shape(int(tokens[i])))
        assert equal_bits(got, ref[i]), "push gather mismatch, request %d" % i
    multi.host_barrier(timeout_s=60)
remote = int((push[:, 2] // 3 != rank).sum())
print("RANK_OK", rank, "pushed", remote, "remote pages of", len(push))
multi.host_barrier(timeout_s=60)
for ptr, off in maps:
    N.check(N.lib().bikv_pool_close(C.c_void_p(ptr), off))
pool.close()
dist.destroy_process_group()
"""


def test_owner_push_gather_across_processes():
    _need_gpus(2)
    world = min(torch.cuda.device_count(), 4)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = textwrap.dedent(PUSH_SCRIPT).format(root=ROOT, port=port)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world))
        procs.append(subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for r, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        assert p.returncode == 0 and "RANK_OK" in out, f"rank {r}:\\n{out[-3000:]}"
