"""Host-side pieces of bench.py that need no GPU: argument defaults, the arena carving that the
pushed gather and configuration 4 rely on, what the CPU arm says it ran, and that a run without
a CUDA device refuses instead of falling back to anything."""
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_defaults_and_arena_layout(monkeypatch):
    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert (args.gpus, args.impl, args.gather_mode, args.workload) == (1, "ours", "push", "auto")
    assert args.steps >= 3 and args.warmup >= 3
    import bikv_b200 as B
    g = B.KVGeometry(2, 2, 8, 4, torch.float16)
    tokens = [5, 1, 9]
    offs = bench._arena_offsets(g, tokens)
    assert offs[0] == 0 and all(o % 128 == 0 for o in offs) and offs == sorted(offs)
    arena = torch.arange(bench._arena_elems(g, tokens), dtype=torch.float32).to(torch.float16)
    parts = bench._carve(arena, g, tokens)
    assert [tuple(p.shape) for p in parts] == [g.worker_shape(t) for t in tokens]
    for p, o in zip(parts, offs):
        assert p.data_ptr() == arena.data_ptr() + o * 2 and (o * 2) % 256 == 0
    # no two tensors overlap
    ends = [o + g.token_elems * t for o, t in zip(offs, tokens)]
    assert all(e <= n for e, n in zip(ends, offs[1:] + [arena.numel()]))
    assert bench.NVLINK_NOMINAL_GBPS == 900.0


def test_gpu_arm_refuses_without_a_cuda_device():
    if torch.cuda.is_available():
        return
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode != 0 and "no CPU implementation" in (res.stdout + res.stderr)
    assert not res.stdout.strip().startswith("{")


def test_reference_arm_says_what_it_ran_and_leaves_the_cuda_library_alone():
    """The CPU arm prints the sample it ran (pool, requests), not the GPU arm's configuration,
    and never maps libbikv.so."""
    code = ("import sys, runpy; sys.argv = ['bench.py', '--impl', 'reference', '--steps', '1', '--warmup', '1', "
            "'--requests', '2']\n"
            "try:\n    runpy.run_path(%r, run_name='__main__')\nexcept SystemExit:\n    pass\n"
            "maps = open('/proc/self/maps').read()\n"
            "print('LIBBIKV_MAPPED', 'libbikv' in maps)\n" % os.path.join(ROOT, "bench.py"))
    env = {k: v for k, v in os.environ.items() if k != "OMP_NUM_THREADS"}
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["gpu_launches"] == 0
    assert line["config"]["sampled_from"] == "config1" and line["config"]["pool_pages"] == 4096
    assert line["config"]["requests"] == 2 and "BOUNDED SAMPLE" in line["config"]["workload"]
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
    assert "LIBBIKV_MAPPED False" in res.stdout


def test_a_failing_side_measurement_is_reported_not_raised(monkeypatch):
    """The short runs of the other configurations must never take the headline down: without a
    CUDA device each of them fails, and each failure comes back as an error string."""
    if torch.cuda.is_available():
        return
    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    args.pool_pages, args.requests = 65536, 64
    out = bench.workload_sides(args, dict(rank=0, world=1, dev=torch.device("cuda:0"), lib=None, variant=0,
                                          multi=False, cpu_group=None, local_rank=0))
    assert set(out) == {"config3_geometry_two_requests_per_gpu", "host_tier_3200_requests"}
    assert all("error" in v and isinstance(v["error"], str) for v in out.values())
