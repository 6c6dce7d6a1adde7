"""Speed of the flat page copy against the reference's own kernel (compiled from the
reference's source into oracle/_ref) on the reference's micro-benchmark shape: 200 pages
of 50 tokens, 28 layers x 2 KV heads x head 128, fp16 (test_page_ipc.py:41-44).  The new
kernel must not be slower; both rates are printed (run pytest with -s to see them)."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import bikv_b200 as B

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _time(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


@pytest.mark.parametrize("page_size,n_pages", [(50, 200), (16, 2048)])
def test_flat_copy_not_slower_than_reference_kernel(cuda, page_size, n_pages):
    path = os.path.join(ROOT, "oracle", "_ref", "bikv_ref_kernel.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/bikv_ref_kernel.so not built")
    spec = importlib.util.spec_from_file_location("bikv_ref_kernel", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = B.GEO_R
    elems = page_size * g.token_elems
    pool_pages = 2 * n_pages
    cache = torch.randn((pool_pages * page_size,) + g.token_shape, device=cuda, dtype=torch.float16)
    rng = np.random.default_rng(0)
    src = torch.from_numpy((rng.permutation(pool_pages)[:n_pages] * elems).astype(np.int64)).to(cuda)
    dst = torch.from_numpy((rng.permutation(n_pages) * elems).astype(np.int64)).to(cuda)
    out = torch.zeros(n_pages * elems, dtype=torch.float16, device=cuda)
    mover = B.PageMover(cuda)
    # the reference launcher ends with cudaDeviceSynchronize; ours is asynchronous
    t_ref = _time(lambda: ref.ref_copy_pages(cache, src, dst, out, page_size, 128, 2, 28, 2))
    t_new = _time(lambda: mover.copy_pages_flat(cache, out, src, dst, elems))
    nbytes = n_pages * elems * 2
    print(f"\n[flat copy {n_pages} pages x {page_size} tokens = {nbytes / 2**20:.1f} MiB] "
          f"reference kernel {nbytes / t_ref / 1e6:.1f} GB/s ({t_ref:.3f} ms), "
          f"bikv_copy_pages_flat {nbytes / t_new / 1e6:.1f} GB/s ({t_new:.3f} ms), x{t_ref / t_new:.2f}")
    assert t_new <= t_ref * 1.05


def test_gather_against_torch_gpu_ops(cuda):
    """The same gather written with stock torch ops on the GPU (index_select of whole pages,
    permute to [layer, kv, token, head, dim], contiguous) against bikv_gather, config-1
    geometry, 2,048 whole pages into one tensor.  Results must agree bit for bit; both rates
    are printed."""
    from bikv_b200.plan import build_plan

    g = B.GEO_B
    pool_pages, n = 4096, 2048
    shard = torch.randn(g.pool_shape(pool_pages), device=cuda, dtype=torch.float32).to(g.dtype)
    ids = torch.from_numpy(np.random.default_rng(1).permutation(pool_pages)[:n].astype(np.int64)).to(cuda)
    plan = build_plan([ids.tolist()], [n * 16], 16)
    out = torch.zeros(g.worker_shape(n * 16), dtype=g.dtype, device=cuda)
    mover = B.PageMover(cuda)
    pool = B.ShardedPool.single(shard, g)
    d_recs, d_reqs = mover.upload(plan, g, out)

    def torch_ops():
        pages = shard.index_select(0, ids)                                    # [n, L, 2, P, H, D]
        return pages.permute(1, 2, 0, 3, 4, 5).reshape(g.n_layers, 2, n * 16, g.n_kv_heads, g.head_dim).contiguous()

    want = torch_ops()
    mover.gather_dev(pool, d_recs, d_reqs)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    del want
    t_torch = _time(torch_ops)
    t_new = _time(lambda: mover.gather_dev(pool, d_recs, d_reqs))
    nbytes = n * g.page_bytes
    print(f"\n[gather {n} pages = {nbytes / 2**30:.2f} GiB] torch index_select+permute+contiguous "
          f"{nbytes / t_torch / 1e6:.1f} GB/s ({t_torch:.3f} ms), bikv_gather {nbytes / t_new / 1e6:.1f} GB/s "
          f"({t_new:.3f} ms), x{t_torch / t_new:.2f}")
    assert t_new <= t_torch


def test_zero_copy_from_pinned_host_against_reference_kernel(cuda):
    """Source pages in pinned host memory: the reference's zero_copy_page_kernel
    (copy_kernel.cu:39-66) against bikv_copy_pages_flat on the same pinned tensor -- same
    bits; both are bound by the host link, the rates are printed."""
    path = os.path.join(ROOT, "oracle", "_ref", "bikv_ref_kernel.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/bikv_ref_kernel.so not built")
    spec = importlib.util.spec_from_file_location("bikv_ref_kernel", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = B.GEO_R
    page_size, n_pages, pool_pages = 16, 512, 1024
    elems = page_size * g.token_elems
    pinned = torch.randn((pool_pages * page_size,) + g.token_shape, dtype=torch.float32).to(torch.float16).pin_memory()
    rng = np.random.default_rng(2)
    src = torch.from_numpy((rng.permutation(pool_pages)[:n_pages] * elems).astype(np.int64)).to(cuda)
    dst = torch.from_numpy((rng.permutation(n_pages) * elems).astype(np.int64)).to(cuda)
    out_ref = torch.zeros(n_pages * elems, dtype=torch.float16, device=cuda)
    out_new = torch.zeros_like(out_ref)
    mover = B.PageMover(cuda)
    shape = ref.ref_zero_copy_pages(pinned, src, dst, out_ref, page_size, 128, 2, 28, 2)
    assert list(shape) == [n_pages * page_size, 128, 2, 28, 2]
    mover.copy_pages_flat(pinned, out_new, src, dst, elems)
    torch.cuda.synchronize()
    assert torch.equal(out_new.view(torch.int16), out_ref.view(torch.int16))
    t_ref = _time(lambda: ref.ref_zero_copy_pages(pinned, src, dst, out_ref, page_size, 128, 2, 28, 2), iters=5)
    t_new = _time(lambda: mover.copy_pages_flat(pinned, out_new, src, dst, elems), iters=5)
    nbytes = n_pages * elems * 2
    print(f"\n[zero-copy {n_pages} pages x {page_size} tokens = {nbytes / 2**20:.0f} MiB from pinned host memory] "
          f"reference kernel {nbytes / t_ref / 1e6:.1f} GB/s, bikv_copy_pages_flat {nbytes / t_new / 1e6:.1f} GB/s")
    assert t_new <= t_ref * 1.10
