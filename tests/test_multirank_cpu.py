"""Host logic of the multi-GPU path on two gloo ranks (CPU): handle exchange, workload
partition, reductions, and a barrier that reports a missing rank instead of hanging."""
import os
import socket
import subprocess
import sys
import textwrap


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(body: str, world: int = 2, timeout: int = 120):
    port = _free_port()
    script = textwrap.dedent("""
        import os, sys
        sys.path.insert(0, {root!r})
        import numpy as np, torch, torch.distributed as dist
        import bikv_b200 as B
        from bikv_b200 import _native as N, workloads as W, multi
        from bikv_b200.pool import ShardedPool
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    """).format(root=ROOT, port=port) + textwrap.dedent(body) + textwrap.dedent("""
        dist.barrier()
        dist.destroy_process_group()
    """)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed: timeout]"
        outs.append((p.returncode, out))
    return outs


def test_handle_exchange_builds_the_same_pool_view_on_every_rank(native):
    outs = _run_ranks("""
        g = B.GEO_A
        shard = torch.zeros(g.pool_shape(8), dtype=g.dtype)
        exported = lambda t: (bytes([rank]) * 64, 128 * rank)
        def importer(r, h):
            assert h == (bytes([r]) * 64, 128 * r), h
            return 0x1000000 * (r + 1) + h[1]
        pool = ShardedPool.exchange(shard, g, exporter=exported, importer=importer)
        assert pool.n_shards == world and pool.pages_per_shard == 8 and pool.rule == N.SHARD_MOD
        for r in range(world):
            want = shard.data_ptr() if r == rank else 0x1000000 * (r + 1) + 128 * r
            assert pool.bases[r] == want and pool.desc.shard_base[r] == want
        assert pool.desc.n_shards == world and pool.desc.pages_per_shard == 8
        print("OK", rank)
    """)
    for rc, out in outs:
        assert rc == 0 and "OK" in out, out


def test_config2_partition_is_disjoint_and_mostly_remote(native):
    outs = _run_ranks("""
        w = W.config2(rank, world, pages_per_shard=32768)
        ids = np.concatenate(w.page_lists)
        everyone = [None] * world
        dist.all_gather_object(everyone, ids.tolist())
        flat = [p for ids_r in everyone for p in ids_r]
        assert len(flat) == len(set(flat)), "ranks share pages"
        assert max(flat) < world * 32768
        frac = w.remote_fraction(rank)
        assert abs(frac - (world - 1) / world) < 0.05, frac
        plan = w.plan()
        total = multi.reduce_over_ranks([plan.n_pages, w.payload_bytes], "sum")
        mx = multi.reduce_over_ranks([float(rank + 1)], "max")
        assert mx == [float(world)]
        assert total[0] == sum(len(x) for x in everyone)
        assert multi.worker_of_request(5, world) == 5 % world
        print("OK", rank)
    """)
    for rc, out in outs:
        assert rc == 0 and "OK" in out, out


def test_barrier_reports_a_rank_that_left(native):
    """Rank 1 leaves before the barrier (between steps, nothing in flight); rank 0's barrier
    must end with an error within its timeout instead of hanging."""
    outs = _run_ranks("""
        import time
        multi.host_barrier(timeout_s=30)          # everyone present: passes
        if rank == 1:
            print("LEFT"); sys.stdout.flush(); os._exit(0)
        t = time.time()
        try:
            multi.host_barrier(timeout_s=3)
            print("NO ERROR")
        except RuntimeError as e:
            print("BARRIER ERROR after %.1fs" % (time.time() - t))
        os._exit(0)
    """, timeout=90)
    assert "LEFT" in outs[1][1]
    assert "BARRIER ERROR" in outs[0][1], outs[0][1]


def test_shared_memory_barrier_orders_ranks_and_reports_a_missing_one(native):
    outs = _run_ranks("""
        import time
        b = multi.ShmBarrier()
        # every rank sees the other's write only after the barrier
        flag = torch.zeros(1)
        for k in range(200):
            b.wait(timeout_s=30)
        t0 = time.perf_counter()
        for k in range(2000):
            b.wait(timeout_s=30)
        per = (time.perf_counter() - t0) / 2000
        print("BARRIER_US", round(per * 1e6, 1))
        assert per < 2e-3
        if rank == 1:
            time.sleep(0.3)                  # rank 0 waits for a late rank, then goes on
        b.wait(timeout_s=30)
        if rank == 0:
            try:
                b.wait(timeout_s=0.5)        # rank 1 never enters this one
                raise SystemExit("expected a timeout")
            except RuntimeError as e:
                assert "ranks [1]" in str(e), str(e)
        else:
            time.sleep(1.0)
        b.close()
        print("SHM_BARRIER_OK")
    """, world=2)
    for rc, out in outs:
        assert rc == 0 and "SHM_BARRIER_OK" in out, out[-2000:]
