"""Shared helpers for the parity tests: seeded pools, worker tensors, oracle runs."""
import numpy as np
import torch

from oracle import bikv_oracle as O


def random_bits(shape, dtype, seed, device="cpu"):
    """Random 16-bit patterns reinterpreted as ``dtype`` (covers NaN/Inf/denormal
    encodings: the path must pass every bit pattern through)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    n = int(np.prod(shape))
    esz = torch.empty(0, dtype=dtype).element_size()
    raw = torch.randint(0, 256, (n * esz,), dtype=torch.uint8, generator=g)
    return raw.view(dtype).reshape(shape).to(device)


def normal(shape, dtype, seed, device="cpu"):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype).to(device)


def make_shards(geom, n_shards, pages_per_shard, seed, device="cpu", fill="normal"):
    f = normal if fill == "normal" else random_bits
    return [f(geom.pool_shape(pages_per_shard), geom.dtype, seed + 17 * s, device) for s in range(n_shards)]


def make_workers(geom, request_tokens, device="cpu", fill=None, seed=0):
    out = []
    for i, t in enumerate(request_tokens):
        if fill is None:
            out.append(torch.zeros(geom.worker_shape(int(t)), dtype=geom.dtype, device=device))
        else:
            out.append(normal(geom.worker_shape(int(t)), geom.dtype, seed + i, device))
    return out


def equal_bits(a, b):
    return torch.equal(O.bits(a.cpu()), O.bits(b.cpu()))


def random_plan(rng, geom, total_pages, n_requests, max_tokens, min_tokens=1):
    """Random requests with unique pages; returns (page_lists, tokens)."""
    tokens = rng.integers(min_tokens, max_tokens + 1, size=n_requests)
    counts = (tokens + geom.page_tokens - 1) // geom.page_tokens
    perm = rng.permutation(total_pages)[: int(counts.sum())]
    lists, at = [], 0
    for c in counts:
        lists.append(perm[at:at + int(c)].astype(np.int32))
        at += int(c)
    return lists, tokens.astype(np.int64)
