#!/usr/bin/env python
"""Benchmark of the KV-page gather/scatter path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = gather every request of the batch out of the page pool into per-request
worker tensors [layer, kv, token, head, dim], then scatter them back (a round trip).
N = 1 runs the single-GPU configuration (Qwen2-7B-like geometry, 65,536-page pool, 64
requests); N > 1 (under torchrun, one rank per GPU) stripes the pool by page id over
the ranks and every rank gathers/scatters its own 64 requests, most pages remote.

Prints ONE JSON line on rank 0.  `value` counts payload bytes (valid tokens) moved per
second, both directions, inputs resident in HBM; `roofline.achieved` counts the bytes
the kernel reads plus the bytes it writes (2 x payload per launch); `e2e` is the same
round trip through the Python API from a host-resident plan, with the plan upload and
a status read-back inside the timed region.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "kv_page_gather_scatter_throughput"
UNIT = "GB/s"
# DRAM bytes (read + written) per payload byte of one k_paged_ldst launch, from an ncu capture
# of `bench.py --small` (2,048-page pool, 8 requests, 1.38 GB payload); traffic grows in
# proportion to the bytes copied, so the line scales it to the full launch and says so.
NCU_TRAFFIC_PER_PAYLOAD_BYTE = 1.966
NCU_TRAFFIC_SOURCE = "ncu --set full of k_paged_ldst on `bench.py --small` (1.38 GB payload), scaled by payload"
NVLINK_NOMINAL_GBPS = 900.0     # per direction per GPU


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--variant", default="auto", choices=["auto", "ldst", "bulk"])
    ap.add_argument("--pool-pages", type=int, default=None, help="pages per GPU (default 65536; config3: 8192)")
    ap.add_argument("--requests", type=int, default=None, help="requests per GPU (default 64; config3: 16)")
    ap.add_argument("--host-pages", type=int, default=32768, help="spill: pages of the pinned host tier")
    ap.add_argument("--spill-min-hits", type=int, default=1,
                    help="spill: a prefix evicted from HBM goes to the host tier only after this many hits in HBM")
    ap.add_argument("--workload", default="auto", choices=["auto", "config3", "config4", "spill"],
                    help="auto = configuration 1 (N = 1) or 2 (N > 1), the benchmark; config3 = long-context "
                         "geometry, requests streamed; config4 = coordinator-driven prefix reuse, N/2 shard GPUs + "
                         "N/2 worker GPUs; spill = prefix reuse on one GPU with an HBM tier and a pinned host tier "
                         "(all are additional measurements)")
    ap.add_argument("--c3-order", default="longest", choices=["longest", "arrival"],
                    help="config3: stream each rank's requests longest first (balances the ranks' phases) or in arrival order")
    ap.add_argument("--c4-requests", type=int, default=20000)
    ap.add_argument("--c4-placement", default="striped", choices=["item", "striped"],
                    help="config 4: 'striped' = one page directory over all shards, page id mod shards (every shard serves "
                         "a share of every item); 'item' = an item's pages live on ONE shard, chosen by the multi-shard "
                         "page manager as in the reference (the shard holding the most popular users is the bottleneck)")
    ap.add_argument("--c4-planner", default="native", choices=["native", "python"],
                    help="config4: page directory in C++ (bikv_pm_*) or the Python page managers (order='fast')")
    ap.add_argument("--geometry", default="B", choices=["A", "B", "C", "R"],
                    help="KV geometry (B = the benchmark's; others are side measurements)")
    ap.add_argument("--layout", default="paged", choices=["paged", "token_major"],
                    help="pool layout (token_major = the reference's pool; a side measurement)")
    ap.add_argument("--pages-from", default="all", choices=["all", "remote", "local"],
                    help="N > 1 only: draw pages from all shards (the benchmark), or only remote / only local ones")
    ap.add_argument("--only", default="both", choices=["both", "gather", "scatter"],
                    help="side measurement: time one direction only (all ranks then move data the same way)")
    ap.add_argument("--worker-layout", default="contiguous", choices=["contiguous", "nhd"],
                    help="nhd = the worker's paged KV, one [slot, kv, head, dim] tensor per layer (side measurement)")
    ap.add_argument("--gather-mode", default="push", choices=["pull", "push"],
                    help="N > 1: push = the GPU that owns a page writes it into the worker's tensor, as the reference's "
                         "shard does on SEND (stores over NVLink need no request packets: 6.99 ms per gather on 2 GPUs); "
                         "pull = the worker's GPU reads remote pages (loads over NVLink: 7.70 ms)")
    ap.add_argument("--small", action="store_true", help="profiling-sized case (2,048-page pool, 8 requests)")
    ap.add_argument("--tune", action="append", default=[], metavar="KNOB=VALUE")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--host-kv-steps", type=int, default=2,
                    help="N = 1: also time this many round trips with the worker KV tensors in pinned HOST memory "
                         "(the reference keeps its worker buffer on the CPU); 0 skips it")
    ap.add_argument("--no-sides", action="store_true",
                    help="N = 1: skip the short side runs (token-major pools, paged worker KV) after the headline")
    ap.add_argument("--no-verify", action="store_true", help="skip the closed-form check of one gather and one scatter and the pool hash before and after the run")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


# --------------------------------------------------------------------------- clocks
CLOCK_FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, device_index):
        import torch
        self.proc, self.path = None, None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ident, f"--query-gpu=timestamp,{CLOCK_FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None
        self.t0 = self.t1 = None

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def finish(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        self.out.close()
        import datetime
        rows = []
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), parts[4:9]))
            except ValueError:
                continue
        os.unlink(self.path)
        inside = [r for r in rows if self.t0 is not None and self.t0 - 0.05 <= r[0] <= self.t1 + 0.05]
        use = inside if len(inside) >= 2 else rows
        if not use:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in use for n, v in zip(names, r[3][1:]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[1] for r in use), "sm_max_mhz": max(r[2] for r in use),
                "reasons": reasons, "samples": len(use), "samples_in_timed_region": len(inside)}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_run(steps, warmup, requests, limit_s=20.0):
    """The reference's CPU data path (token rows in host tensors, torch advanced indexing
    over token indices: DistributedStorage/kvcache.py:38-43, Worker/Worker.py:57-62,207) as
    restated in oracle/, on a bounded sample of the single-GPU workload: same geometry and
    request-length distribution, 4,096-page pool, the first `sample_requests` requests."""
    import torch

    from bikv_b200 import workloads as W
    from oracle import bikv_oracle as O

    # All the host cores this process may use (torchrun sets OMP_NUM_THREADS=1 for its ranks).
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        pass
    g = W.GEO_B
    pool_pages, sample_requests = 4096, min(8, requests)
    w = W.config1(seed=0, n_pages=pool_pages, n_requests=sample_requests)
    # The plan comes from the oracle's own restatement of the reference's loop: this arm
    # neither loads nor calls the CUDA library.
    recs = O.plan_records([p.tolist() for p in w.page_lists], [int(t) for t in w.request_tokens], g.page_tokens,
                          item_request=list(range(w.n_requests)))
    src, dst = O.token_indices(recs, g.page_tokens)
    gen = torch.Generator().manual_seed(0)
    # N(0,1) values; one token row drawn per page slot and repeated (a copy's speed does
    # not depend on the values, and drawing 1.9 G normals would dominate the run).
    rows = torch.randn((g.page_tokens,) + g.token_shape, generator=gen, dtype=torch.float32).to(g.dtype)
    pool = rows.repeat((pool_pages,) + (1,) * len(g.token_shape))
    buf = torch.zeros((w.total_tokens,) + g.token_shape, dtype=g.dtype)
    payload = w.payload_bytes

    def step():
        O.cpu_gather_tokens(pool, buf, src, dst)
        O.cpu_scatter_tokens(pool, buf, src, dst)

    for _ in range(max(1, min(warmup, 2))):
        step()
    times, t_all = [], time.perf_counter()
    for _ in range(steps):
        t = time.perf_counter()
        step()
        times.append(time.perf_counter() - t)
        if time.perf_counter() - t_all > limit_s:
            break
    total = sum(times)
    done = len(times)
    gbs = 2 * payload * done / total / 1e9
    sample = (f"{sample_requests} requests ({w.n_pages} pages, {payload / 1e9:.2f} GB payload) of the config-1 "
              f"distribution on a {pool_pages}-page host pool, {done} round trips")
    return {"value": gbs, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample,
            "ms_per_step": total / done * 1e3, "steps_done": done, "pages_per_s": 2 * w.n_pages * done / total,
            "host_cpus": os.cpu_count(), "pool_pages": pool_pages, "requests": sample_requests,
            "pages_per_step": 2 * w.n_pages, "payload_bytes_per_direction": payload}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    if os.environ.get("OMP_NUM_THREADS") and os.environ.get("BIKV_REFERENCE_CHILD") != "1":
        # A launcher (torchrun) pinned this rank to OMP_NUM_THREADS threads, and the OpenMP
        # pool cannot be widened after the fact: run the CPU arm in a child that starts with
        # all host cores and pass its JSON line through.
        env = {k: v for k, v in os.environ.items()
               if k not in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "RANK", "LOCAL_RANK", "WORLD_SIZE")}
        env["BIKV_REFERENCE_CHILD"] = "1"
        res = subprocess.run([sys.executable, os.path.abspath(__file__)] + sys.argv[1:], env=env)
        if res.returncode != 0:
            raise SystemExit(res.returncode)
        return
    base = cpu_reference_run(args.steps, args.warmup, args.requests, limit_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": base["steps_done"], "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": "config1 geometry (28 layers, 4 KV heads, head 128, bf16, 16-token pages) on the "
                               "host: token rows in CPU tensors, torch advanced indexing [BOUNDED SAMPLE of config1]",
                   "sampled_from": "config1", "pool_pages": base["pool_pages"], "requests": base["requests"],
                   "request_lengths": "lognormal(median 2048, sigma 0.8) clipped to [64, 8192]",
                   "step": "gather all requests + scatter them back",
                   "pages_per_step": base["pages_per_step"],
                   "payload_bytes_per_direction": base["payload_bytes_per_direction"]},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "pages_per_s": base["pages_per_s"], "host_cpus": base["host_cpus"],
    }
    print(json.dumps(line), flush=True)


def config_dict(args, w):
    name = "config1: Qwen2-7B-like KV (28 layers, 4 KV heads, head 128, bf16, 16-token pages)" if args.gpus == 1 \
        else f"config2: config-1 geometry, pool striped page_id mod {args.gpus}, {args.gpus - 1}/{args.gpus} of pages remote"
    c = {"workload": name, "pool_pages_per_gpu": args.pool_pages, "requests_per_gpu": args.requests,
         "request_lengths": "lognormal(median 2048, sigma 0.8) clipped to [64, 8192]",
         "step": "gather all requests + scatter them back" + ("" if args.gpus == 1 else
                                                                  "; ranks phase-aligned by a host barrier after each direction"
                                                                  f"; gather by {args.gather_mode}"),
         "l2": "inputs larger than L2 (payload per launch is ~10 GB against 126 MB of L2)"}
    if args.small:
        c["workload"] += " [SMALL profiling case]"
    if args.only != "both":
        c["workload"] += f" [SIDE MEASUREMENT: {args.only} only]"
    if args.gather_mode != "push" and args.gpus > 1:
        c["workload"] += " [SIDE MEASUREMENT: gather pulled by the worker's GPU]"
    if args.worker_layout != "contiguous":
        c["workload"] += " [SIDE MEASUREMENT: worker KV paged, one [slot, kv, head, dim] tensor per layer]"
    if args.pages_from != "all":
        c["workload"] += f" [SIDE MEASUREMENT: {args.pages_from} pages only]"
    if args.geometry != "B" or args.layout != "paged":
        c["workload"] += f" [SIDE MEASUREMENT: geometry {args.geometry}, {args.layout} pool]"
    if w is not None:
        c.update({"pages_per_step_per_gpu": 2 * w.n_pages, "payload_bytes_per_direction_per_gpu": w.payload_bytes,
                  "page_bytes": w.geom.page_bytes})
    return c



# --------------------------------------------------------------------------- additional workloads
def _arena_offsets(geom, tokens_list):
    """Element offsets of worker tensors laid one after another, each start 128-element aligned."""
    out, at = [], 0
    for t in tokens_list:
        out.append(at)
        at += (geom.token_elems * int(t) + 127) // 128 * 128
    return out


def _arena_elems(geom, tokens_list):
    offs = _arena_offsets(geom, tokens_list)
    return offs[-1] + (geom.token_elems * int(tokens_list[-1]) + 127) // 128 * 128 if len(offs) else 0


def _carve(arena, geom, tokens_list):
    """Worker tensors [layer, kv, T, head, dim] laid one after another in a flat arena."""
    import torch
    out, at = [], 0
    for t in tokens_list:
        n = geom.token_elems * int(t)
        out.append(arena[at:at + n].view(geom.worker_shape(int(t))))
        at += (n + 127) // 128 * 128
    if at > arena.numel():
        raise RuntimeError("worker arena too small")
    return out


def run_config3(ctx):
    """Configuration 3: long-context geometry (80 layers, 8 KV heads, head 128, fp16), requests of
    16k-32k tokens, STREAMED one at a time through a reused worker buffer (one request is up to
    10 GiB); pool striped page_id mod N.  A step = every request gathered and scattered back.
    On N > 1 GPUs phase i moves every rank's i-th request; the gather is pushed by the pages'
    owners (`--gather-mode push`, the default) or pulled by the worker, the scatter is the
    worker's push.  Before timing, the first request of every rank is gathered once from a pool
    of closed-form contents and every word checked; the pool's position hash is compared across
    the timed round trips."""
    import ctypes as C

    import numpy as np
    import torch
    import torch.distributed as dist

    import bikv_b200 as B
    from bikv_b200 import _native as N
    from bikv_b200 import multi as multi_mod
    from bikv_b200 import selfcheck as S
    from bikv_b200 import workloads as W
    from bikv_b200.push import split_plans_by_owner

    args, rank, world, dev, lib, multi = (ctx[k] for k in ("args", "rank", "world", "dev", "lib", "multi"))
    geom = W.GEO_C
    shard = B.ShardedPool.allocate_shard(geom, args.pool_pages, dev)
    pool = B.ShardedPool.exchange(shard, geom, group=ctx["cpu_group"]) if multi else B.ShardedPool.single(shard, geom)

    def requests_of(r):
        out = W.config3(r, world, pages_per_shard=args.pool_pages, n_requests=args.requests)
        # Longest first on every rank: phase k then moves every rank's k-th longest request, so
        # the ranks' phases are close in size (max/mean 1.08 instead of 1.23 in arrival order) and
        # the barrier after each phase waits less.
        if args.c3_order == "longest":
            out.sort(key=lambda x: -x.total_tokens)
        return out

    reqs = requests_of(rank)
    arena = torch.zeros(geom.token_elems * max(w.total_tokens for w in reqs), dtype=geom.dtype, device=dev)
    mover = B.PageMover(dev, variant=ctx["variant"])
    staged = []
    for w in reqs:
        t = _carve(arena, geom, [w.total_tokens])
        staged.append(mover.upload(w.plan(), geom, t))
    stream = torch.cuda.current_stream(dev)

    # Owner-push gather: for phase i, this rank's pages of EVERY rank's i-th request go into that
    # rank's arena (mapped here through one IPC handle per rank).
    push = multi and args.gather_mode == "push"
    pushed, arena_maps, pushed_remote_bytes = [], [], 0
    if push:
        everyone = [requests_of(r) if r != rank else reqs for r in range(world)]
        handles = [None] * world
        dist.all_gather_object(handles, B.ShardedPool.export_handle(arena), group=ctx["cpu_group"])
        arena_base = []
        for r, h in enumerate(handles):
            if r == rank:
                arena_base.append(arena.data_ptr())
                continue
            out = C.c_void_p()
            N.check(lib.bikv_pool_import(h[0], int(h[1]), C.byref(out)), "bikv_pool_import")
            arena_base.append(int(out.value))
            arena_maps.append((int(out.value), int(h[1])))
        for i in range(args.requests):
            rows = split_plans_by_owner([everyone[r][i].plan().table for r in range(world)], [1] * world, rank,
                                        world, args.pool_pages)
            table = torch.tensor([[arena_base[r], everyone[r][i].total_tokens] for r in range(world)], dtype=torch.int64)
            pushed.append((torch.from_numpy(rows).to(dev), table.to(dev)))
            pushed_remote_bytes += int(rows[rows[:, 2] != rank, 1].sum()) * geom.bytes_per_token

    def launch_gather(i):
        if push:
            mover.gather_dev(pool, *pushed[i])
        else:
            mover.gather_dev(pool, *staged[i])

    phase_barrier = multi_mod.ShmBarrier(ctx["cpu_group"]) if multi else None

    def phase_end():
        if multi:
            stream.synchronize()
            phase_barrier.wait(timeout_s=ctx.get("barrier_timeout_s", 300))

    def step(events=None):
        for i, (recs, rq) in enumerate(staged):
            if events:
                events[i][0].record(stream)
            launch_gather(i)
            if events:
                events[i][1].record(stream)
            phase_end()
            if events:
                events[i][2].record(stream)
            mover.scatter_dev(pool, recs, rq)
            if events:
                events[i][3].record(stream)
            phase_end()

    def agree(flag):
        if not multi:
            return bool(flag)
        t_ok = torch.tensor([float(bool(flag))], dtype=torch.float64)
        dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
        return bool(t_ok[0])

    # ---- the first request of every rank out of a closed-form pool, every word checked ----
    verified = {"gather_closed_form": None, "pool_hash_unchanged": None}
    if not args.no_verify:
        S.fill_pool_(shard, geom, S.global_ids_of_shard(rank, world, args.pool_pages))
        torch.cuda.synchronize()
        phase_end()
        launch_gather(0)
        phase_end()
        w0 = reqs[0]
        tensor = _carve(arena, geom, [w0.total_tokens])[0]
        verified["gather_closed_form"] = agree(S.check_gathered(geom, tensor, w0.page_lists[0], w0.total_tokens,
                                                                     max_tokens_per_pass=1024))
        if not verified["gather_closed_form"]:
            raise SystemExit("bench.py config3: gathered words differ from what the plan implies")
    W.fill_normal_(shard, seed=99 + rank)
    hash_before = None if args.no_verify else S.position_hash(shard)
    sampler = ClockSampler(ctx["local_rank"]) if rank == 0 else None
    torch.cuda.synchronize()
    torch.cuda.empty_cache()      # scratch left by the pool fill; see main()
    phase_end()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if multi:
        dist.barrier(group=ctx["cpu_group"])
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in staged] for _ in range(args.steps)]
    launches0 = lib.bikv_launch_count()
    if sampler:
        sampler.mark_start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for k in range(args.steps):
        step(ev[k])
    t1.record(stream)
    torch.cuda.synchronize()
    if sampler:
        sampler.mark_end()
    mover.check_status()
    elapsed_ms = t0.elapsed_time(t1)
    g_ms = sum(e[0].elapsed_time(e[1]) for st in ev for e in st) / args.steps
    s_ms = sum(e[2].elapsed_time(e[3]) for st in ev for e in st) / args.steps
    payload = float(sum(w.payload_bytes for w in reqs))
    pages = float(sum(w.n_pages for w in reqs))
    launches = float(lib.bikv_launch_count() - launches0)
    remote = sum(w.remote_fraction(rank) * w.payload_bytes for w in reqs) / payload
    if multi:
        t = torch.tensor([elapsed_ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tot = torch.tensor([payload, pages, launches], dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        elapsed_ms, (tp, tpages, tl) = float(t[0]), tot.tolist()
    else:
        tp, tpages, tl = payload, pages, launches
    clocks = sampler.finish() if sampler else None
    if hash_before is not None:
        phase_end()
        verified["pool_hash_unchanged"] = agree(S.position_hash(shard) == hash_before)
        if not verified["pool_hash_unchanged"]:
            raise SystemExit("bench.py config3: the pool changed across gather->scatter round trips")
    nv_in = remote * payload / (g_ms / 1e3) / 1e9
    if push:       # what this GPU pushed to the others per step, over the time its pushes took
        nv_in = pushed_remote_bytes / (g_ms / 1e3) / 1e9
    if rank == 0:
        peak, peak_kind = measured_peaks()
        secs = elapsed_ms / 1e3
        line = {
            "metric": METRIC, "value": 2 * tp * args.steps / secs / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": {"workload": f"config3: Llama-3-70B-like KV (80 layers, 8 KV heads, head 128, fp16, 16-token pages), "
                                   f"{args.requests} requests per GPU of U[16k,32k] tokens streamed one at a time ({args.c3_order} order), pool "
                                   f"{args.pool_pages} pages per GPU striped page_id mod {world} [ADDITIONAL MEASUREMENT]",
                       "payload_bytes_per_direction_per_gpu": payload, "page_bytes": geom.page_bytes,
                       "l2": "inputs larger than L2 (each request is 5-10 GB)"},
            "pages_per_s": 2 * tpages * args.steps / secs, "gpu_launches": int(tl), "clocks": clocks,
            "roofline": {"bound": "hbm" if not multi else "nvlink", "unit": "GB/s", "gather_ms_per_step": g_ms,
                         "scatter_ms_per_step": s_ms, "remote_fraction": remote,
                         "hbm_achieved": 2 * payload / ((g_ms + s_ms) / 2 / 1e3) / 1e9, "hbm_peak": peak,
                         "hbm_frac": 2 * payload / ((g_ms + s_ms) / 2 / 1e3) / 1e9 / peak, "peak_kind": f"of {peak_kind}",
                         "nvlink_in_GBps_per_gpu": nv_in, "gather_mode": args.gather_mode if multi else None,
                         "nvlink_out_GBps_per_gpu": remote * payload / (s_ms / 1e3) / 1e9},
            "verified": verified,
        }
    else:
        line = None
    if multi:
        dist.barrier(group=ctx["cpu_group"])
        pool.close()
        for ptr, off in arena_maps:
            N.check(lib.bikv_pool_close(C.c_void_p(ptr), off), "bikv_pool_close")
        phase_barrier.close()
    del shard, arena
    return line


def run_config4(ctx):
    """Configuration 4: N/2 KVCache-shard GPUs + N/2 worker GPUs, config-1 geometry.  100,000 users
    ~ Zipf(1.1), cached prefixes lognormal(median 1024, sigma 0.8) in [128, 8192] (sigma is not given
    by the configuration; 0.8 as in configuration 1), new tokens U[32,256] written back, LRU eviction by
    the page directory, batches of 64.  Every page a worker touches is remote.

    Who moves what.  Stores are the better NVLink operation for a kernel, and one GPU that loads and
    stores remotely at the same time gets little more than either alone (two B200s, one GPU driving:
    783 GB/s pulling, 715 pushing, 760-910 doing both; the copy engines reach 1,554 there).  So each
    direction is driven by the GPU that holds the source, with stores only: the SHARD GPUs push the
    hit prefixes of batch k+1 into the workers' tensors (the shard is the active side of a SEND in
    the reference too, ``DistributedStorage/kvcache.py:96-113``) while the WORKER GPUs push batch k's
    missed prefixes and new tokens into the pool.  The two run at the same time -- they load
    opposite directions of every link -- and one host barrier over all ranks ends the pair.

    Hazard: a prefix stored by batch k and read by batch k+1.  The planner sees it (page ids of
    the two plans intersect); those gather rows wait, on every shard, for a barrier behind the
    workers' scatters, the rest overlaps them.  Planning (all workers' shares, replicated on every
    rank so that all hold the same page directory) runs on a host thread ahead of the kernels, and
    every rank builds step k+1's rows and request tables while step k's kernels run.  A
    batch is planned in ONE piece and then split by worker: a user named twice in a batch, by
    requests of two workers, is stored by the first and not read by the second.

    Placement (``--c4-placement``).  By default pages are striped over the shards (one page
    directory, page id mod shards): with Zipf users, an item kept whole on one shard -- the
    reference's ``MultiPageManager.load_item`` -- makes the shard with the most popular prefixes
    push 45 % of all hit bytes on four shards, and a step lasts as long as that shard's push.

    Before the timed run a shorter stream goes through the same pipeline with closed-form
    contents: every prefix a miss stores is a function of (user, token, word), and every prefix
    a later hit receives -- from whichever shard, for whichever worker -- is compared against it
    on the device.  Reports pages/s (wall clock, and device time only) and the hit rate."""
    import ctypes as C
    import queue
    import threading

    import numpy as np
    import torch
    import torch.distributed as dist

    import bikv_b200 as B
    from bikv_b200 import _native as N
    from bikv_b200 import multi as multi_mod
    from bikv_b200 import selfcheck as S
    from bikv_b200 import workloads as W
    from bikv_b200.coordinator import (NativePrefixCacheCoordinator, PrefixCacheCoordinator, PrefixReuseWorkload,
                                       plan_stream)
    from bikv_b200.plan import Plan
    from bikv_b200.push import split_plans_by_owner

    args, rank, world, dev, lib = (ctx[k] for k in ("args", "rank", "world", "dev", "lib"))
    if world < 2 or world % 2:
        raise SystemExit("config4 needs an even number of GPUs >= 2 (half shards, half workers)")
    n_shards = n_workers = world // 2
    is_shard = rank < n_shards
    me = rank if is_shard else rank - n_shards
    geom = W.GEO_B
    group = ctx["cpu_group"]
    per_worker = (64 + n_workers - 1) // n_workers
    arena_elems = geom.token_elems * (8192 + 256) * per_worker

    def note(msg):
        print(f"[config4 rank {rank}] {msg}", file=sys.stderr, flush=True)

    # ---- memory: a shard per shard rank, two arenas per worker rank, everything mapped everywhere needed ----
    shard = arenas = None
    if is_shard:
        shard = torch.zeros(geom.pool_shape(args.pool_pages), dtype=geom.dtype, device=dev)
        mine = [B.ShardedPool.export_handle(shard)]
    else:
        # batch k+1 is gathered into one arena while batch k is scattered out of the other
        arenas = [torch.zeros(arena_elems, dtype=geom.dtype, device=dev) for _ in range(2)]
        mine = [B.ShardedPool.export_handle(a) for a in arenas]
    handles = [None] * world
    dist.all_gather_object(handles, mine, group=group)
    mapped = []

    def open_handle(h):
        out = C.c_void_p()
        N.check(lib.bikv_pool_import(h[0], int(h[1]), C.byref(out)), "bikv_pool_import")
        mapped.append((int(out.value), int(h[1])))
        return int(out.value)

    # Placement.  'item': the multi-shard page manager puts an item on one shard (global page id =
    # shard * pages + page), as ``DistributedStorage/PageManager.py:164-203`` does.  'striped': one
    # directory over all shards' pages and page id mod shards names the shard, so every item -- the
    # most popular users' prefixes too -- is served by all shards alike.
    striped = args.c4_placement == "striped"
    rule = N.SHARD_MOD if striped else N.SHARD_BLOCK
    if is_shard:
        # the pool as this shard addresses it: only its own pages are ever named in its plans
        pool = B.ShardedPool([shard.data_ptr()] * n_shards, args.pool_pages, geom, rule=rule, device=dev,
                             keepalive=[shard])
        arena_base = [[open_handle(h) for h in handles[n_shards + w]] for w in range(n_workers)]
    else:
        pool = B.ShardedPool([open_handle(handles[s][0]) for s in range(n_shards)], args.pool_pages, geom,
                             rule=rule, device=dev)
    # Launches here are short (a batch moves about 1.5 GB per worker): the ld/st kernel, which has no
    # ring to fill and drain, measured 1.58-1.63 M pages/s on 2 + 2 GPUs against 1.51-1.55 M for the bulk ring.
    mover = B.PageMover(dev, variant=N.VARIANT_LDST if args.variant == "auto" else ctx["variant"])
    stream = torch.cuda.Stream(dev)
    step_barrier = multi_mod.ShmBarrier(group)          # microseconds, where a gloo barrier costs a tenth of a step
    tables = [torch.empty((per_worker * (n_workers if is_shard else 1), 2), dtype=torch.int64).pin_memory()
              for _ in range(8)]
    rw = geom.row_elems * geom.elt_bytes // 4
    ok_dev = torch.ones((), dtype=torch.bool, device=dev)

    def make_coordinator():
        dirs, pages = (1, n_shards * args.pool_pages) if striped else (n_shards, args.pool_pages)
        return (NativePrefixCacheCoordinator(dirs, pages, geom.page_tokens, transient_plans=True)
                if args.c4_planner == "native"
                else PrefixCacheCoordinator(dirs, pages, geom.page_tokens, order="fast"))

    def planner(wl, co, out_q):
        """Every worker's share of every batch, and which gather rows read a page the batch before
        writes (decided over ALL workers, so every rank decides alike)."""
        try:
            for step in plan_stream(wl.batches(), co, n_workers, n_shards * args.pool_pages, transient=True):
                out_q.put(step)
        finally:
            out_q.put(None)

    def words(arena, off_elems, tokens):
        n = geom.token_elems * tokens
        return arena[off_elems:off_elems + n].view(torch.int32).view(geom.planes, tokens, rw)

    def prefix_words(user, tokens):
        """Closed form of a user's cached prefix: word (plane, token, w) = mix(user, ...)."""
        return S.worker_words(geom, 0, int(user) & 0xFFFFF, tokens, 0, tokens, dev)

    def shard_rows(plans, masks, k, late):
        """This shard's rows of all workers' gather plans for batch k (the early or the late
        ones), destinations interleaved, and the request table of the workers' arenas."""
        tabs = [p.gather.table[m if late else ~m] for p, m in zip(plans, masks)]
        nreq = [len(p.requests) for p in plans]
        rows = split_plans_by_owner(tabs, nreq, me, n_shards, args.pool_pages, rule=rule)
        return Plan.from_table(rows, sum(nreq), transient=True)

    def run_stream(wl, co, check):
        q = queue.Queue(maxsize=3)
        th = threading.Thread(target=planner, args=(wl, co, q), daemon=True)
        th.start()
        pages = payload = n_steps = n_late = pushed = 0
        spans = []
        launches0 = lib.bikv_launch_count()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        t0 = time.perf_counter()
        bpt = geom.bytes_per_token

        def prepare(item, k):
            """Host work of step k: the request table of the arenas it writes and, on a shard, this
            shard's rows.  Runs while step k-1's kernels do."""
            if item is None:
                return None
            plans, masks, has_late = item
            table = tables[k % len(tables)]
            st = {"has_late": has_late}
            if is_shard:
                tn, at = table.numpy(), 0
                for w, p in enumerate(plans):
                    offs = np.asarray(_arena_offsets(geom, p.tokens), dtype=np.int64)
                    tn[at:at + len(offs), 0] = arena_base[w][k % 2] + offs * geom.elt_bytes
                    tn[at:at + len(offs), 1] = p.tokens
                    at += len(offs)
                st["table"] = table[:at]
                st["early"] = shard_rows(plans, masks, k, late=False)
                st["late"] = shard_rows(plans, masks, k, late=True) if has_late else None
                st["cur"] = True
            else:
                bp = plans[me]
                offs = _arena_offsets(geom, bp.tokens)
                table = table[:len(bp.tokens)]
                tn = table.numpy()
                tn[:, 0] = arenas[k % 2].data_ptr() + np.asarray(offs, dtype=np.int64) * geom.elt_bytes
                tn[:, 1] = bp.tokens
                st["cur"] = (bp, k % 2, table, offs)
                g = bp.gather.table
                st["pages"] = len(g) + bp.scatter.n_pages
                st["payload"] = (int(g[:, 1].sum()) + int(bp.scatter.table[:, 1].sum())) * bpt
            return st

        prev = None          # worker: (share, arena index, table, offsets) whose scatter is due
        k = 0
        nxt = prepare(q.get(), 0)
        drained = nxt is None
        while True:
            st = nxt
            if st is None and prev is None:
                break
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            has_late = st is not None and st["has_late"]
            cur = st["cur"] if st is not None else None
            if st is not None and not is_shard:
                pages += st["pages"]
                payload += st["payload"]
            # -- the stores of this step --
            if is_shard:
                if st is not None:
                    pushed += int(st["early"].table[:, 1].sum()) * bpt
                    mover.gather_table(pool, st["early"], st["table"], stream=stream)
            elif prev is not None:
                pbp, pa, ptable, poffs = prev
                if check:
                    # what the model would have computed: the prefixes this batch stores
                    stored = set(int(r) for r in pbp.scatter.table[pbp.scatter.table[:, 3] == 0, 2])
                    with torch.cuda.stream(stream):
                        for i, r in enumerate(pbp.requests):
                            if i in stored and not pbp.hit[i]:
                                words(arenas[pa], poffs[i], r.tokens)[:, :r.prefix_tokens] = \
                                    prefix_words(r.user, r.prefix_tokens)
                pushed += int(pbp.scatter.table[:, 1].sum()) * bpt
                mover.scatter_table(pool, pbp.scatter, ptable, stream=stream)
            if not has_late:
                e1.record(stream)
            # -- while they run: the host work of the next step --
            if drained:
                nxt = None
            else:
                nxt = prepare(q.get(), k + 1)
                drained = nxt is None
            if has_late:
                # rows that read what the workers are writing right now: once every worker's
                # scatter has landed
                if not is_shard:
                    stream.synchronize()
                step_barrier.wait(timeout_s=ctx.get("barrier_timeout_s", 300))
                if is_shard:
                    pushed += int(st["late"].table[:, 1].sum()) * bpt
                    mover.gather_table(pool, st["late"], st["table"], stream=stream)
                n_late += 1
                e1.record(stream)
            stream.synchronize()
            step_barrier.wait(timeout_s=ctx.get("barrier_timeout_s", 300))
            spans.append((e0, e1))
            n_steps += 1
            if check and not is_shard and cur is not None:
                # This step's gather is complete: every shard has passed the barrier above.  The
                # comparison runs on this stream, which the next step synchronises before its own
                # barrier, i.e. before any shard writes this arena again.
                cbp, ca, _, coffs = cur
                with torch.cuda.stream(stream):
                    for i, r in enumerate(cbp.requests):
                        if cbp.hit[i]:
                            got = words(arenas[ca], coffs[i], r.tokens)[:, :r.prefix_tokens]
                            ok_dev.logical_and_((got == prefix_words(r.user, r.prefix_tokens)).all())
            prev = cur if not is_shard else (True if st is not None else None)
            k += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        th.join()
        mover.check_status()
        dev_ms = sum(a.elapsed_time(b) for a, b in spans)
        return dict(wall=wall, dev_ms=dev_ms, pages=pages, payload=payload, steps=n_steps, late=n_late,
                    launches=lib.bikv_launch_count() - launches0, hit_rate=co.hit_rate, pushed=pushed)

    # ---- closed-form pass over a shorter stream (same pipeline, contents checked) ----
    verified = None
    if not args.no_verify:
        wl = PrefixReuseWorkload(seed=1, n_workers=n_workers, n_requests=min(args.c4_requests, 1920), batch=64)
        run_stream(wl, make_coordinator(), check=True)
        t_ok = torch.tensor([float(bool(ok_dev.item()))], dtype=torch.float64)
        dist.all_reduce(t_ok, op=dist.ReduceOp.MIN, group=group)
        verified = bool(t_ok[0])
        if not verified:
            raise SystemExit("bench.py config4: a gathered prefix differs from what was stored")
    # ---- the timed run ----
    wl = PrefixReuseWorkload(seed=0, n_workers=n_workers, n_requests=args.c4_requests, batch=64)
    co = make_coordinator()
    r = run_stream(wl, co, check=False)
    note(f"{r['steps']} pipeline steps in {r['wall']:.2f} s")
    t = torch.tensor([r["wall"], r["dev_ms"]], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    tot = torch.tensor([float(r["pages"]), float(r["payload"]), float(r["launches"])], dtype=torch.float64)
    dist.all_reduce(tot, op=dist.ReduceOp.SUM, group=group)
    per_rank = [None] * world
    dist.all_gather_object(per_rank, (r["dev_ms"], r["pushed"]), group=group)
    if rank == 0:
        wall, dev_ms = t.tolist()
        line = {
            "metric": "kv_pages_per_second", "value": tot[0].item() / wall, "unit": "pages/s", "n_gpus": world,
            "steps": r["steps"], "warmup": 0, "ms_per_step": wall / r["steps"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": {"workload": f"config4: {n_shards} shard GPUs + {n_workers} worker GPUs, config-1 geometry, "
                                   f"{wl.n_users} users Zipf(1.1), {wl.n_requests} requests in batches of 64, LRU "
                                   f"eviction [ADDITIONAL MEASUREMENT]", "pool_pages_per_shard": args.pool_pages,
                       "placement": ("striped: one page directory over all shards, page id mod shards" if striped else
                                     "item: an item's pages on one shard, chosen by the multi-shard page manager"),
                       "pipeline": "the shard GPUs push batch k+1's hit prefixes while the worker GPUs push batch k's "
                                   "stores (one host barrier over all ranks per pair); gather rows that read a page "
                                   "being stored wait for a second barrier",
                       "pairs_with_late_rows": r["late"]},
            "hit_rate": r["hit_rate"], "GBps_wall": tot[1].item() / wall / 1e9,
            "pages_per_s_device_only": tot[0].item() / (dev_ms / 1e3),
            "GBps_device_only": tot[1].item() / (dev_ms / 1e3) / 1e9,
            "nvlink_GBps_per_worker_device_only": tot[1].item() / n_workers / (dev_ms / 1e3) / 1e9,
            "device_only": "slowest rank's sum over steps of the time its kernels of the step took",
            "host_planning": ("native page directory (bikv_pm_plan_prefix_batch)" if args.c4_planner == "native"
                              else "Python page managers with order='fast'") +
                             ", replicated on every rank, on a host thread ahead of the kernels",
            "gpu_launches": int(tot[2].item()),
            "verified": {"prefixes_closed_form": verified},
            # who is busy: an item lives on one shard, so the shard that holds the most popular users pushes most
            "per_rank": {"role": ["shard"] * n_shards + ["worker"] * n_workers,
                         "GB_pushed": [round(b / 1e9, 2) for _, b in per_rank],
                         "kernel_ms_per_step": [round(ms / r["steps"], 3) for ms, _ in per_rank],
                         "GBps_while_its_kernels_ran": [round(b / 1e6 / ms, 1) if ms else None for ms, b in per_rank]},
        }
    else:
        line = None
    dist.barrier(group=group)
    for ptr, off in mapped:
        N.check(lib.bikv_pool_close(C.c_void_p(ptr), off), "bikv_pool_close")
    step_barrier.close()
    del shard, arenas
    return line


def run_spill(ctx):
    """Side workload: the prefix-reuse stream of configuration 4 on ONE GPU whose HBM pool holds a
    quarter of the pages (16,384) with a host tier behind it (pinned, 32,768 pages by default).
    An item the HBM tier evicts is copied to the host tier before its pages are reused; a prefix
    found only there is copied back and then gathered.  Reports pages/s and where the prefixes
    were found, next to the hit rate the same HBM pool reaches with no host tier behind it.  A
    shorter stream runs first with closed-form prefixes and checks every gathered prefix on the
    device, whichever tier it came back from."""
    import numpy as np
    import torch

    import bikv_b200 as B
    from bikv_b200 import selfcheck as S
    from bikv_b200 import workloads as W
    from bikv_b200.coordinator import PrefixReuseWorkload
    from bikv_b200.page_directory import PageDirectory
    from bikv_b200.plan import build_plan
    from bikv_b200.tiered_store import TieredPageStore

    args, dev, lib = ctx["args"], ctx["dev"], ctx["lib"]
    geom = W.GEO_B
    hbm_pages = args.pool_pages if args.pool_pages != 65536 else 16384
    host_pages = args.host_pages
    mover = B.PageMover(dev, variant=ctx["variant"])
    stream = torch.cuda.current_stream(dev)
    arena = torch.zeros(geom.token_elems * (8192 + 256) * 64, dtype=geom.dtype, device=dev)
    rw = geom.row_elems * geom.elt_bytes // 4
    ok_dev = torch.ones((), dtype=torch.bool, device=dev)
    P = geom.page_tokens

    def words(off_elems, tokens):
        n = geom.token_elems * tokens
        return arena[off_elems:off_elems + n].view(torch.int32).view(geom.planes, tokens, rw)

    def prefix_words(user, tokens):
        return S.worker_words(geom, 0, int(user) & 0xFFFFF, tokens, 0, tokens, dev)

    def run_stream(store, wl, check):
        pages_moved = payload = 0
        next_item = 1 << 40
        ev = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for batch in wl.batches():
            tensors = _carve(arena, geom, [r.tokens for r in batch])
            offs = _arena_offsets(geom, [r.tokens for r in batch])
            g_pages, g_tok, g_req, s_pages, s_tok, s_req, s_first = [], [], [], [], [], [], []
            stored_now, hits, fills = set(), [], []
            store.begin_batch()
            for i, r in enumerate(batch):
                if r.user in stored_now:
                    pass                       # being stored by this very batch: computed again, not read
                else:
                    pages = store.fetch(r.user) if store.tokens_of(r.user) in (None, r.prefix_tokens) else None
                    if pages is not None:
                        g_pages.append(pages), g_tok.append(r.prefix_tokens), g_req.append(i)
                        hits.append(i)
                    else:
                        s_pages.append(store.store(r.user, r.prefix_tokens)), s_tok.append(r.prefix_tokens)
                        s_req.append(i), s_first.append(True)
                        stored_now.add(r.user)
                        fills.append(i)
                s_pages.append(store.store(next_item, r.new_tokens, spill=False)), s_tok.append(r.new_tokens)
                s_req.append(i), s_first.append(False)
                next_item += 1
            store.end_batch(stream)            # demotions, then promotions, ahead of the batch's own copies
            gather = build_plan(g_pages, g_tok, P, item_request=g_req, n_requests=len(batch))
            scatter = build_plan(s_pages, s_tok, P, item_request=s_req, n_requests=len(batch))
            with_prefix = {s_req[k] for k in range(len(s_req)) if s_first[k]}
            table = scatter.table
            for i, r in enumerate(batch):      # a request whose prefix is not stored: new tokens sit behind it
                if i not in with_prefix:
                    table[table[:, 2] == i, 3] += r.prefix_tokens
            e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            e[0].record(stream)
            mover.gather(store.pool, gather, tensors)
            if check:
                for i in hits:
                    r = batch[i]
                    ok_dev.logical_and_((words(offs[i], r.tokens)[:, :r.prefix_tokens] ==
                                         prefix_words(r.user, r.prefix_tokens)).all())
                for i in fills:
                    r = batch[i]
                    words(offs[i], r.tokens)[:, :r.prefix_tokens] = prefix_words(r.user, r.prefix_tokens)
            mover.scatter(store.pool, scatter, tensors)
            e[1].record(stream)
            ev.append(e)
            pages_moved += gather.n_pages + scatter.n_pages
            payload += (int(gather.table[:, 1].sum()) + int(scatter.table[:, 1].sum())) * geom.bytes_per_token
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        mover.check_status()
        return dict(wall=wall, pages=pages_moved, payload=payload, batches=len(ev),
                    dev_ms=sum(a.elapsed_time(b) for a, b in ev))

    verified = None
    if not args.no_verify:
        small = TieredPageStore(geom, 8192, min(16384, host_pages), dev, mover=mover)
        run_stream(small, PrefixReuseWorkload(seed=1, n_workers=1, n_requests=1920, batch=64), check=True)
        verified = bool(ok_dev.item())
        st = small.stats
        if not verified or st.promotions == 0 or st.demotions == 0:
            raise SystemExit(f"bench.py spill: closed-form check failed or did not exercise both moves ({st})")
        del small
    store = TieredPageStore(geom, hbm_pages, host_pages, dev, mover=mover, min_hits_to_spill=args.spill_min_hits)
    launches0 = lib.bikv_launch_count()
    wl = PrefixReuseWorkload(seed=0, n_workers=1, n_requests=args.c4_requests, batch=64)
    r = run_stream(store, wl, check=False)
    st = store.stats
    # the same stream against the same HBM pool with nothing behind it (host logic only)
    alone = PageDirectory(hbm_pages * P, P, 1, policy="lru")
    stored, hit_alone, item = {}, 0, 1 << 40
    for batch in wl.batches():
        for q in batch:
            if alone.access_item(q.user)[0] is not None and stored.get(q.user) == q.prefix_tokens:
                hit_alone += 1
            else:
                alone.load_item(q.user, q.prefix_tokens)
                stored[q.user] = q.prefix_tokens
            alone.load_item(item, q.new_tokens)
            item += 1
    n = wl.n_requests
    line = {
        "metric": "kv_pages_per_second", "value": r["pages"] / r["wall"], "unit": "pages/s", "n_gpus": 1,
        "steps": r["batches"], "warmup": 0, "ms_per_step": r["wall"] / r["batches"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": f"prefix reuse on one GPU with a two-tier pool: {hbm_pages} pages in HBM, {host_pages} in "
                               f"pinned host memory; {wl.n_users} users Zipf(1.1), {n} requests in batches of 64, LRU in "
                               "each tier [ADDITIONAL MEASUREMENT]"},
        "GBps_wall": r["payload"] / r["wall"] / 1e9, "pages_per_s_device_only": r["pages"] / (r["dev_ms"] / 1e3),
        "prefixes_found": {"in_hbm": st.hbm_hits / n, "in_host_tier": st.host_hits / n,
                           "nowhere": 1 - (st.hbm_hits + st.host_hits) / n},
        "hit_rate": (st.hbm_hits + st.host_hits) / n, "hit_rate_same_hbm_pool_without_host_tier": hit_alone / n,
        "tier_moves": {"demotions": st.demotions, "demotions_that_needed_no_copy": st.clean_demotions,
                       "promotions": st.promotions, "pages_demoted": st.pages_demoted,
                       "pages_promoted": st.pages_promoted, "dropped": st.dropped,
                       "evictions_not_spilled": st.not_spilled,
                       "policy": f"prefixes fetched at least {args.spill_min_hits} time(s) while in HBM are kept on "
                                 "eviction; written-back new tokens are not"},
        "gpu_launches": int(lib.bikv_launch_count() - launches0),
        "verified": {"prefixes_closed_form_through_both_tiers": verified},
    }
    return line


# --------------------------------------------------------------------------- side measurements
def peer_copy_ceilings(mover, pool, shard, rank, world, dev, barrier, nbytes=2 << 30, reps=3):
    """What a plain contiguous copy gets out of the links right now: every rank copies one range
    from (pull) or to (push) its right-hand neighbour's shard at the same time -- a ring, so that
    every GPU's link carries data in both directions, as it does under the sharded pool -- once
    with the copy engines (cudaMemcpyAsync: independent of this library's kernels) and once with
    the library's flat copy kernel.  GB/s per GPU, slowest rank, best of `reps` after one untimed
    round.  Runs before the pool is filled: the pushed range overwrites the start of a shard."""
    import torch
    import torch.distributed as dist

    peer = (rank + 1) % world
    nbytes = min(nbytes, shard.numel() * shard.element_size()) >> 20 << 20
    if nbytes <= 0:
        return None
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    main = torch.cuda.current_stream(dev)

    def run(copy, push):
        times = []
        for _ in range(reps + 1):
            torch.cuda.synchronize()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(main)
            remote, local = pool.bases[peer], scratch.data_ptr()
            copy(remote if push else local, local if push else remote, nbytes, stream=main)
            e1.record(main)
            main.synchronize()
            times.append(e0.elapsed_time(e1))
        t = torch.tensor([min(times[1:])], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return nbytes / (float(t[0]) / 1e3) / 1e9

    out = {"engine_pull_GBps_per_gpu": run(mover.copy_range_engine, False),
           "engine_push_GBps_per_gpu": run(mover.copy_range_engine, True),
           "kernel_pull_GBps_per_gpu": run(mover.copy_range, False),
           "kernel_push_GBps_per_gpu": run(mover.copy_range, True),
           "bytes_per_gpu": nbytes,
           "pattern": f"ring over {world} GPUs, every GPU against its right-hand neighbour at once, both link "
                      "directions loaded; engine = cudaMemcpyAsync (copy engines), kernel = bikv_copy_range"}
    torch.cuda.synchronize()
    barrier()
    del scratch
    return out


def side_measure(mover, dev, geom, pool_pages, n_requests, worker_layout, steps=5, warmup=3):
    """One more (pool layout, worker layout) pair on this GPU, after the headline: gather and
    scatter timed separately with CUDA events, the pool's position hash compared across the
    round trips.  Fractions are of the measured HBM copy bandwidth, 2 x payload per launch."""
    import numpy as np
    import torch

    import bikv_b200 as B
    from bikv_b200 import selfcheck as S
    from bikv_b200 import workloads as W
    from bikv_b200.plan import build_block_plan

    shard = B.ShardedPool.allocate_shard(geom, pool_pages, dev)
    W.fill_normal_(shard, seed=4321)
    pool = B.ShardedPool.single(shard, geom)
    w = W.config1(seed=0, n_pages=pool_pages, n_requests=n_requests, geom=geom)
    stream = torch.cuda.current_stream(dev)
    if worker_layout == "nhd":
        blocks = np.random.default_rng(7).permutation(w.n_pages)
        plan = build_block_plan(w.flat(), w.request_tokens.astype("int32"), geom.page_tokens, blocks)
        layers = [torch.zeros((w.n_pages * geom.page_tokens, 2, geom.n_kv_heads, geom.head_dim), dtype=geom.dtype,
                              device=dev) for _ in range(geom.n_layers)]
        gather = lambda: mover.gather_nhd(pool, plan, layers, validate=False)      # noqa: E731
        scatter = lambda: mover.scatter_nhd(pool, plan, layers, validate=False)    # noqa: E731
    else:
        tensors = [torch.zeros(geom.worker_shape(int(t)), dtype=geom.dtype, device=dev) for t in w.request_tokens]
        d_recs, d_reqs = mover.upload(w.plan(), geom, tensors)
        gather = lambda: mover.gather_dev(pool, d_recs, d_reqs)                    # noqa: E731
        scatter = lambda: mover.scatter_dev(pool, d_recs, d_reqs)                  # noqa: E731
    before = S.position_hash(shard)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    for _ in range(warmup):
        gather()
        scatter()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    torch.cuda.synchronize()
    for e in ev:
        e[0].record(stream)
        gather()
        e[1].record(stream)
        scatter()
        e[2].record(stream)
    torch.cuda.synchronize()
    mover.check_status()
    g_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    s_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    peak, peak_kind = measured_peaks()
    same = S.position_hash(shard) == before
    out = {"geometry": f"{geom.n_layers} layers x {geom.n_kv_heads} KV heads x {geom.head_dim}, {geom.elt_bytes}-byte "
                       f"elements, {geom.page_tokens}-token pages",
           "pool_pages": pool_pages, "requests": n_requests, "payload_bytes_per_direction": w.payload_bytes,
           "gather_ms": g_ms, "scatter_ms": s_ms,
           "gather_frac": 2 * w.payload_bytes / (g_ms / 1e3) / 1e9 / peak,
           "scatter_frac": 2 * w.payload_bytes / (s_ms / 1e3) / 1e9 / peak,
           "value_GBps": 2 * w.payload_bytes / ((g_ms + s_ms) / 1e3) / 1e9, "peak_kind": f"of {peak_kind}",
           "steps": steps, "pool_hash_unchanged": same}
    if not same:
        raise SystemExit("bench.py: a side measurement changed its pool across round trips")
    return out


def workload_sides(args, ctx_base):
    """Configurations 3 and 4 (and, on one GPU, the two-tier pool) in a few steps each, so that
    every default run carries a figure for them: configuration 3's geometry (80 layers x 8 KV heads x 128, fp16, 5 MiB pages) with
    two streamed requests per GPU, and -- on an even number of GPUs -- configuration 4's
    shard/worker pipeline over 3,200 requests, its closed-form prefix check included.  A side
    that fails is reported as an error string; it never takes the headline down with it."""
    rank, world = ctx_base["rank"], ctx_base["world"]

    def attempt(fn, **over):
        a = argparse.Namespace(**vars(args))
        for k, v in over.items():
            setattr(a, k, v)
        try:
            return fn(dict(ctx_base, args=a, barrier_timeout_s=60))
        except BaseException as e:  # noqa: BLE001  (SystemExit of a failed check included)
            return {"error": f"{type(e).__name__}: {e}"}

    out = {}
    c3 = attempt(run_config3, workload="config3", pool_pages=8192, requests=2, steps=1, warmup=1)
    if rank == 0 and c3 is not None:
        keep = ("value", "unit", "ms_per_step", "pages_per_s", "error")
        out["config3_geometry_two_requests_per_gpu"] = {k: c3[k] for k in keep if k in c3}
        if "roofline" in c3:
            out["config3_geometry_two_requests_per_gpu"].update(
                {k: c3["roofline"][k] for k in ("hbm_frac", "remote_fraction", "nvlink_in_GBps_per_gpu",
                                               "nvlink_out_GBps_per_gpu", "gather_ms_per_step", "scatter_ms_per_step")},
                workload=c3["config"]["workload"], verified=c3.get("verified"))
    if world == 1:
        sp = attempt(run_spill, workload="spill", pool_pages=8192, host_pages=8192, c4_requests=3200)
        if sp is not None:
            keep = ("value", "unit", "hit_rate", "hit_rate_same_hbm_pool_without_host_tier", "prefixes_found",
                    "tier_moves", "verified", "error")
            out["host_tier_3200_requests"] = {k: sp[k] for k in keep if k in sp}
            if "config" in sp:
                out["host_tier_3200_requests"]["workload"] = sp["config"]["workload"]
    if world >= 2 and world % 2 == 0:
        c4 = attempt(run_config4, workload="config4", c4_requests=3200)
        if rank == 0 and c4 is not None:
            keep = ("value", "unit", "ms_per_step", "hit_rate", "GBps_wall", "pages_per_s_device_only",
                    "nvlink_GBps_per_worker_device_only", "verified", "error")
            out["config4_3200_requests"] = {k: c4[k] for k in keep if k in c4}
            if "config" in c4:
                out["config4_3200_requests"]["workload"] = c4["config"]["workload"]
                out["config4_3200_requests"]["placement"] = c4["config"].get("placement")
    return out


# --------------------------------------------------------------------------- GPU arm
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.small:
        args.pool_pages, args.requests = 2048, 8
    if args.pool_pages is None:
        args.pool_pages = 8192 if args.workload == "config3" else 65536
    if args.requests is None:
        args.requests = 16 if args.workload == "config3" else 64
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}")

    import torch
    import torch.distributed as dist

    import bikv_b200 as B
    from bikv_b200 import _native as N
    from bikv_b200 import multi as multi_mod
    from bikv_b200 import workloads as W
    from bikv_b200.plan import build_plan

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the KV-page path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    lib = N.lib()
    for kv in args.tune:
        k, v = kv.split("=")
        N.check(lib.bikv_set_tuning(k.encode(), int(v)), f"tune {k}")
    variant = {"auto": N.VARIANT_AUTO, "ldst": N.VARIANT_LDST, "bulk": N.VARIANT_BULK}[args.variant]

    multi = world > 1
    if multi:
        # Host-side rendezvous only (handle exchange, barriers, max/sum of a few floats): the
        # data path has no collective, so no NCCL communicator is created.  A rank that is
        # gone makes the others fail after the timeout instead of waiting for ever.
        import datetime
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=300))
        cpu_group = dist.group.WORLD

    if args.workload != "auto":
        ctx = dict(args=args, rank=rank, world=world, dev=dev, lib=lib, variant=variant, multi=multi,
                   cpu_group=cpu_group if multi else None, local_rank=local_rank)
        line = {"config3": run_config3, "config4": run_config4, "spill": run_spill}[args.workload](ctx)
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
        if multi:
            dist.barrier(group=cpu_group)
            dist.destroy_process_group()
        return

    geom = {"A": W.GEO_A, "B": W.GEO_B, "C": W.GEO_C,
            "R": B.KVGeometry(28, 2, 128, 16, torch.float16)}[args.geometry]
    if args.layout == "token_major":
        geom = geom.with_layout(N.POOL_TOKEN_MAJOR)
    shard = B.ShardedPool.allocate_shard(geom, args.pool_pages, dev)
    if multi:
        pool = B.ShardedPool.exchange(shard, geom, group=cpu_group)
        all_w = [W.config2(r, world, seed=0, pages_per_shard=args.pool_pages, n_requests=args.requests, geom=geom,
                           pages_from=args.pages_from) for r in range(world)]
        w = all_w[rank]
    else:
        pool = B.ShardedPool.single(shard, geom)
        w = W.config1(seed=0, n_pages=args.pool_pages, n_requests=args.requests, geom=geom)
    plan = w.plan()
    mover = B.PageMover(dev, variant=variant)
    stream = torch.cuda.current_stream(dev)
    nhd = args.worker_layout == "nhd"
    if nhd:
        # Side measurement: the worker's KV is paged, one [slot, kv, head, dim] tensor per layer.
        import numpy as np
        from bikv_b200.plan import build_block_plan
        blocks = np.random.default_rng(7).permutation(w.n_pages)
        plan = build_block_plan(w.flat(), w.request_tokens.astype("int32"), geom.page_tokens, blocks)
        layers = [torch.zeros((w.n_pages * geom.page_tokens, 2, geom.n_kv_heads, geom.head_dim), dtype=geom.dtype,
                              device=dev) for _ in range(geom.n_layers)]
        tensors = []
        args.no_e2e = True

        def launch_gather():
            mover.gather_nhd(pool, plan, layers, validate=False)

        def launch_scatter():
            mover.scatter_nhd(pool, plan, layers, validate=False)
    else:
        push = multi and args.gather_mode == "push"
        if push:
            # Worker tensors come out of one arena per rank so that one IPC handle maps them all.
            arena = torch.zeros(_arena_elems(geom, w.request_tokens), dtype=geom.dtype, device=dev)
            tensors = _carve(arena, geom, w.request_tokens)
        else:
            tensors = [torch.zeros(geom.worker_shape(int(t)), dtype=geom.dtype, device=dev) for t in w.request_tokens]
        d_recs, d_reqs = mover.upload(plan, geom, tensors)

        def launch_gather():
            mover.gather_dev(pool, d_recs, d_reqs)

        def launch_scatter():
            mover.scatter_dev(pool, d_recs, d_reqs)

        if push:
            import ctypes as C
            import numpy as np
            from bikv_b200.plan import Plan
            from bikv_b200.push import split_plans_by_owner
            handles = [None] * world
            dist.all_gather_object(handles, B.ShardedPool.export_handle(arena), group=cpu_group)
            arena_base, arena_maps = [], []
            for r, h in enumerate(handles):
                if r == rank:
                    arena_base.append(arena.data_ptr())
                    continue
                out = C.c_void_p()
                N.check(lib.bikv_pool_import(h[0], int(h[1]), C.byref(out)), "bikv_pool_import")
                arena_base.append(int(out.value))
                arena_maps.append((int(out.value), int(h[1])))
            # Rows of every worker's plan whose page lives on this GPU; bases of every worker's
            # tensors as mapped here.
            push_table = split_plans_by_owner([x.plan().table for x in all_w], [x.n_requests for x in all_w], rank,
                                              world, args.pool_pages)
            push_reqs = torch.empty((sum(x.n_requests for x in all_w), 2), dtype=torch.int64).pin_memory()
            at = 0
            for r, x in enumerate(all_w):
                for off, t in zip(_arena_offsets(geom, x.request_tokens), x.request_tokens):
                    push_reqs[at, 0] = arena_base[r] + off * geom.elt_bytes
                    push_reqs[at, 1] = int(t)
                    at += 1
            d_push_recs = torch.from_numpy(push_table).to(dev)
            d_push_reqs = push_reqs.to(dev)
            own = (push_table[:, 2] >= rank * args.requests) & (push_table[:, 2] < (rank + 1) * args.requests)
            pushed_remote_bytes = int(push_table[~own, 1].sum()) * geom.bytes_per_token

            def launch_gather():   # noqa: F811  (the owner-side form replaces the pull)
                mover.gather_dev(pool, d_push_recs, d_push_reqs)

    def barrier():
        if multi:
            dist.barrier(group=cpu_group)

    def all_ranks_agree(flag):
        if not multi:
            return bool(flag)
        t_ok = torch.tensor([float(bool(flag))], dtype=torch.float64)
        dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
        return bool(t_ok[0])

    # ---- what the links give a plain contiguous copy (before the pool holds anything) ----
    peer_copy = peer_copy_ceilings(mover, pool, shard, rank, world, dev, barrier) if multi else None

    # ---- content-addressed check of the launches that are timed below ----
    closed_form = {"gather_closed_form": None, "scatter_closed_form": None}
    if not args.no_verify and args.layout == "paged" and not nhd and args.only == "both":
        from bikv_b200 import selfcheck as S
        ids = S.global_ids_of_shard(rank, world, args.pool_pages)
        S.fill_pool_(shard, geom, ids)
        torch.cuda.synchronize()
        barrier()
        launch_gather()
        stream.synchronize()
        barrier()
        ok_g = all(S.check_gathered(geom, t, pl, int(n)) for t, pl, n in zip(tensors, w.page_lists, w.request_tokens))
        for r, t in enumerate(tensors):
            S.fill_worker_(geom, t, rank, r)
        torch.cuda.synchronize()
        barrier()
        launch_scatter()
        stream.synchronize()
        barrier()
        touched = S.touched_pages(all_w if multi else [w], rank, world, args.pool_pages)
        ok_s = S.check_scattered_pool(shard, geom, ids, touched)
        mover.check_status()
        closed_form = {"gather_closed_form": all_ranks_agree(ok_g), "scatter_closed_form": all_ranks_agree(ok_s)}
        if not (closed_form["gather_closed_form"] and closed_form["scatter_closed_form"]):
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": world, "verified": closed_form,
                                  "error": "closed-form check failed"}), flush=True)
            raise SystemExit("bench.py: gathered or scattered words differ from what the plan implies")
        for t in tensors:
            t.zero_()
    W.fill_normal_(shard, seed=1234 + rank)
    torch.cuda.synchronize()
    barrier()

    do_g, do_s = args.only in ("both", "gather"), args.only in ("both", "scatter")
    n_dirs = int(do_g) + int(do_s)

    phase_barrier = multi_mod.ShmBarrier(cpu_group) if multi else None

    def phase_end():
        """N > 1: ranks move data the same way at the same time (all gather, then all
        scatter), as the reference's batch-synchronous scheduler drives its workers.  A
        host barrier between phases keeps them aligned; unaligned ranks load one NVLink
        direction with reads AND writes while the other idles.  The barrier is the
        shared-memory one: a phase lasts milliseconds and a gloo barrier over loopback TCP
        costs a few hundred microseconds of it."""
        if multi:
            stream.synchronize()
            phase_barrier.wait(timeout_s=300)

    def step_resident():
        if do_g:
            launch_gather()
            phase_end()
        if do_s:
            launch_scatter()
            phase_end()

    flat_begin = w.flat()
    item_tokens = w.request_tokens.astype("int32")
    item_req = list(range(w.n_requests))

    def step_e2e():
        p = build_plan(flat_begin, item_tokens, geom.page_tokens, item_request=item_req, n_requests=w.n_requests,
                       transient=True)
        if do_g:
            if multi and args.gather_mode == "push" and not nhd:
                # the shard's share of the batch as the coordinator would deliver it: page records
                mover.gather_table(pool, Plan.from_table(push_table, len(push_reqs), transient=True), push_reqs)
            else:
                mover.gather(pool, p, tensors)
            phase_end()
        if do_s:
            mover.scatter(pool, p, tensors)
            phase_end()
        mover.check_status()          # 16-byte device->host read, synchronises the step

    def shard_checksum():
        """Position-weighted hash of this rank's shard (every 32-bit word weighted by a hash of
        its index, so words that move change it).  A step scatters back exactly what it gathered,
        so the pool must come out of the whole run unchanged (checked after the timed regions,
        on every rank, at full size)."""
        from bikv_b200 import selfcheck as S
        return S.position_hash(shard)

    # nvidia-smi takes a few hundred ms to deliver its first sample: start it well ahead of the timed steps
    sampler = ClockSampler(local_rank) if rank == 0 else None
    checksum_before = shard_checksum() if args.only == "both" and not args.no_verify else None
    # Give back the scratch blocks that filling and checksumming the pool left in torch's
    # caching allocator: with them still mapped the copy kernels measured 2 % slower
    # (0.970 against 0.988 of the HBM copy peak, same box, back to back).
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    for _ in range(args.warmup):
        step_resident()
    torch.cuda.synchronize()

    # ---- timed region: K resident steps, CUDA events on the launching stream ----
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    launches0 = lib.bikv_launch_count()
    barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark_start()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    for k in range(args.steps):
        ev[k][0].record(stream)
        if do_g:
            launch_gather()
        ev[k][1].record(stream)
        if do_g:
            phase_end()
        ev[k][3].record(stream)
        if do_s:
            launch_scatter()
        ev[k][2].record(stream)
        if do_s:
            phase_end()
    t_end.record(stream)
    torch.cuda.synchronize()
    barrier()
    if sampler:
        sampler.mark_end()
    launches = lib.bikv_launch_count() - launches0
    elapsed_ms = t_begin.elapsed_time(t_end)
    gather_ms = [e[0].elapsed_time(e[1]) for e in ev]
    scatter_ms = [e[3].elapsed_time(e[2]) for e in ev]
    mover.check_status()

    # ---- end to end through the Python API, host-resident plan ----
    h2d_plan_bytes = 2 * (plan.n_pages * 16 + w.n_requests * 16)
    e2e = None
    if not args.no_e2e:
        for _ in range(max(1, min(args.warmup, 3))):
            step_e2e()
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_e2e()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        barrier()
        e2e = {"seconds": e2e_s, "h2d_bytes_per_step": h2d_plan_bytes, "d2h_bytes_per_step": 16}

    clocks = sampler.finish() if sampler else None

    # ---- variant: worker KV in pinned host memory, written and read in place over PCIe ----
    host_kv = None
    if not multi and not nhd and args.host_kv_steps > 0 and not args.no_e2e and args.only == "both":
        host = [torch.empty(geom.worker_shape(int(t)), dtype=geom.dtype).pin_memory() for t in w.request_tokens]
        table = torch.empty((len(host), 2), dtype=torch.int64).pin_memory()
        for i, t in enumerate(host):
            table[i, 0], table[i, 1] = t.data_ptr(), t.shape[2]

        def step_host_kv():
            p = build_plan(flat_begin, item_tokens, geom.page_tokens, item_request=item_req, n_requests=w.n_requests,
                           transient=True)
            mover.gather_table(pool, p, table, variant=N.VARIANT_LDST)
            mover.scatter_table(pool, p, table, variant=N.VARIANT_LDST)
            mover.check_status()

        step_host_kv()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.host_kv_steps):
            step_host_kv()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        same = all(torch.equal(a.view(torch.int16), b.cpu().view(torch.int16)) for a, b in
                   list(zip(host, tensors))[:4]) if geom.elt_bytes == 2 else None
        host_kv = {"value": 2 * w.payload_bytes * args.host_kv_steps / dt / 1e9, "unit": UNIT,
                   "steps": args.host_kv_steps, "ms_per_step": dt / args.host_kv_steps * 1e3,
                   "d2h_bytes_per_step": w.payload_bytes, "h2d_bytes_per_step": w.payload_bytes + h2d_plan_bytes,
                   "host_tensors_equal_device_tensors": same,
                   "what": "same round trip with the worker KV tensors in pinned host memory: the gather kernel "
                           "stores into them and the scatter kernel loads from them in place over PCIe "
                           "(the reference keeps its worker buffer on the CPU, Worker/Worker.py:57-62)"}
        del host

    # ---- the reference's own pool layout and the worker's paged KV, one short run each ----
    sides = None
    if not multi and not args.no_sides and args.workload == "auto" and args.geometry == "B" and \
            args.layout == "paged" and not nhd and args.only == "both" and not args.small:
        geo_r = B.KVGeometry(28, 2, 128, 16, torch.float16, N.POOL_TOKEN_MAJOR)
        sides = {
            "token_major_pool_reference_geometry": dict(side_measure(mover, dev, geo_r, 16384, 64, "contiguous"),
                                                        kernel="k_token_major16v"),
            "token_major_pool_config1_geometry": dict(side_measure(mover, dev, W.GEO_B.with_layout(N.POOL_TOKEN_MAJOR),
                                                                   16384, 64, "contiguous"), kernel="k_token_major16v"),
            "paged_pool_to_paged_worker_kv": dict(side_measure(mover, dev, W.GEO_B, 16384, 64, "nhd"),
                                                  kernel="k_paged_nhd"),
        }

    verified = None
    if checksum_before is not None:
        barrier()
        verified = all_ranks_agree(shard_checksum() == checksum_before)
        if not verified:
            raise SystemExit("bench.py: the pool changed across gather->scatter round trips (bits differ)")

    # ---- max over ranks ----
    payload = w.payload_bytes
    pages = w.n_pages
    if multi:
        t = torch.tensor([elapsed_ms, e2e["seconds"] if e2e else 0.0], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tot = torch.tensor([float(payload), float(pages), float(launches)], dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        elapsed_ms = float(t[0])
        if e2e:
            e2e["seconds"] = float(t[1])
        total_payload, total_pages, total_launches = float(tot[0]), float(tot[1]), int(tot[2])
    else:
        total_payload, total_pages, total_launches = float(payload), float(pages), launches

    if rank == 0:
        peak, peak_kind = measured_peaks()
        secs = elapsed_ms / 1e3
        value = n_dirs * total_payload * args.steps / secs / 1e9
        launch_ms = statistics.mean((gather_ms if do_g else []) + (scatter_ms if do_s else []))
        achieved = 2 * payload / (launch_ms / 1e3) / 1e9
        chosen = variant if variant != N.VARIANT_AUTO else int(lib.bikv_get_tuning(b"auto_variant"))
        if chosen == N.VARIANT_AUTO:
            chosen = N.VARIANT_BULK if multi else N.VARIANT_LDST
        kernel = {N.VARIANT_LDST: "k_paged_ldst", N.VARIANT_BULK: "k_paged_bulk"}[chosen]
        if args.layout == "token_major":
            kernel = "k_token_major"
        if nhd:
            kernel = "k_paged_nhd"
        roofline = {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": NCU_TRAFFIC_PER_PAYLOAD_BYTE * payload if kernel == "k_paged_ldst" else None,
            "traffic_source": NCU_TRAFFIC_SOURCE if kernel == "k_paged_ldst" else None,
            "peak_kind": f"of {peak_kind}", "kernel": kernel,
            "algorithmic_bytes_per_launch": 2 * payload, "launch_ms": launch_ms,
            "gather_ms": statistics.mean(gather_ms), "scatter_ms": statistics.mean(scatter_ms),
            "note": "rank 0's launches; local pages are HBM-bound, remote pages NVLink-bound" if multi else
                    "each payload byte is read once and written once",
        }
        if multi:
            remote = w.remote_fraction(rank)
            nv = remote * payload / (statistics.mean(gather_ms) / 1e3) / 1e9
            if args.gather_mode == "push" and not nhd:
                nv = pushed_remote_bytes / (statistics.mean(gather_ms) / 1e3) / 1e9
            out_gbps = remote * payload / (statistics.mean(scatter_ms) / 1e3) / 1e9
            # With (N-1)/N of the pages remote the launches are NVLink-bound, not HBM-bound: the
            # roofline is remote bytes per GPU against the link's nominal rate per direction; what
            # contiguous copies reached on these GPUs a moment ago stands beside it.  The HBM view
            # stays in "hbm".
            roofline = {"bound": "nvlink", "achieved": (nv + out_gbps) / 2, "peak": NVLINK_NOMINAL_GBPS, "unit": "GB/s",
                        "frac": (nv + out_gbps) / 2 / NVLINK_NOMINAL_GBPS, "traffic": None,
                        "peak_kind": "of nominal NVLink 5 (900 GB/s per direction per GPU)",
                        "kernel": kernel, "algorithmic_bytes_per_launch": remote * payload,
                        "launch_ms": launch_ms, "gather_ms": statistics.mean(gather_ms),
                        "scatter_ms": statistics.mean(scatter_ms),
                        "note": "rank 0's launches; achieved = NVLink bytes per GPU per second, mean of the "
                                "gather (ingress) and scatter (egress) launches",
                        "hbm": roofline}
            roofline["nvlink"] = {"remote_fraction": remote, "gather_mode": args.gather_mode,
                                  "gather_ingress_GBps_per_gpu": nv, "gather_frac_of_900_nominal": nv / NVLINK_NOMINAL_GBPS,
                                  "scatter_egress_GBps_per_gpu": out_gbps,
                                  "scatter_frac_of_900_nominal": out_gbps / NVLINK_NOMINAL_GBPS,
                                  "peer_copy_measured_in_this_run": peer_copy}
            if peer_copy:
                best_in = max(peer_copy["engine_pull_GBps_per_gpu"], peer_copy["kernel_pull_GBps_per_gpu"],
                              peer_copy["engine_push_GBps_per_gpu"], peer_copy["kernel_push_GBps_per_gpu"])
                roofline["nvlink"]["gather_frac_of_best_contiguous_copy"] = nv / best_in
                roofline["nvlink"]["scatter_frac_of_best_contiguous_copy"] = out_gbps / best_in
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": config_dict(args, w), "pages_per_s": n_dirs * total_pages * args.steps / secs,
            "roofline": roofline, "gpu_launches": total_launches, "clocks": clocks,
            "verified": dict(closed_form, pool_hash_unchanged=verified),
        }
        if e2e:
            line["e2e"] = {"value": n_dirs * total_payload * args.steps / e2e["seconds"] / 1e9, "unit": UNIT,
                           "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                           "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                           "ms_per_step": e2e["seconds"] / args.steps * 1e3,
                           "what": "build_plan from page lists + PageMover.gather + PageMover.scatter + status read, "
                                   "plan in pinned host memory; the pool and the worker KV tensors stay in HBM"}
        if host_kv:
            line["e2e_host_kv"] = host_kv
        if sides:
            line["side_measurements"] = sides
        if not multi and not args.no_cpu_baseline:
            base = cpu_reference_run(20, 1, args.requests, limit_s=15.0)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    else:
        line = None

    if multi:
        barrier()
        pool.close()
        if args.gather_mode == "push" and not nhd:
            for ptr, off in arena_maps:
                N.check(lib.bikv_pool_close(C.c_void_p(ptr), off), "bikv_pool_close")
        phase_barrier.close()

    # ---- the other configurations, short, once the headline's memory has been given back ----
    eligible = (not args.no_sides and args.geometry == "B" and args.layout == "paged" and not nhd and
                args.only == "both" and not args.small and args.pages_from == "all")
    if eligible:
        shard = pool = tensors = arena = d_recs = d_reqs = d_push_recs = d_push_reqs = None   # noqa: F841
        launch_gather = launch_scatter = None                                                 # noqa: F841
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        more = workload_sides(args, dict(rank=rank, world=world, dev=dev, lib=lib, variant=variant, multi=multi,
                                         cpu_group=cpu_group if multi else None, local_rank=local_rank))
        if rank == 0 and more:
            line.setdefault("side_measurements", {}).update(more)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if multi:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
