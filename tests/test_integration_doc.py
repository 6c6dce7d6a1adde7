"""The ctypes stub printed in the integration guide at the repository root is executed as written (only the library path
is filled in) against a pool in the reference's layout, and checked with the oracle."""
import os
import re
import types

import pytest
import torch

from bikv_b200 import _native as N
from bikv_b200.geometry import KVGeometry
from oracle import bikv_oracle as O

from helpers import equal_bits, normal

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stub_source():
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    code = next(b for b in blocks if "def shared_data_batch_pages" in b)
    return code.replace("/path/to/bi-kv_b200/csrc/libbikv.so", N.LIB_PATH)


def test_stub_parses_and_binds(native):
    ns = {}
    exec(compile(_stub_source(), "integration_stub", "exec"), ns)
    assert callable(ns["shared_data_batch_pages"])


@pytest.mark.gpu
def test_stub_gathers_like_the_oracle(cuda):
    ns = {}
    exec(compile(_stub_source(), "integration_stub", "exec"), ns)
    page_size, pool_pages = 16, 24
    geom = KVGeometry(28, 2, 128, page_size, torch.float16, N.POOL_TOKEN_MAJOR)
    pool_cpu = normal(geom.pool_shape(pool_pages), geom.dtype, 3)
    kv = types.SimpleNamespace(page_size=page_size, cache_size=pool_pages * page_size, device=cuda,
                               cuda_cache_data=pool_cpu.to(cuda))
    task = {"infer_worker": 0, "cache_worker": 0, "token_num": 53, "task_type": 1,
            "id_token_pair": [(7, 37), (9, 16)], "cache_pages_list": [[5, 20, 2], [11]]}
    worker_kv = torch.zeros(geom.worker_shape(53), dtype=geom.dtype, device=cuda)
    ns["shared_data_batch_pages"](kv, task, worker_kv)
    torch.cuda.synchronize()
    want = torch.zeros(geom.worker_shape(53), dtype=geom.dtype)
    recs = O.plan_records(task["cache_pages_list"], [37, 16], page_size)
    O.gather([pool_cpu], geom, recs, [want])
    assert equal_bits(worker_kv, want)
