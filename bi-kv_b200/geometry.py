"""KV geometry: what one token, one page and one worker tensor look like.

The reference hard-codes one geometry (head 128, 2 KV heads, 28 layers, K+V,
fp16; ``Model/qwen2.py:512-522``) and repeats it as literals
(``DistributedStorage/kvcache.py:199-206``); here it is a value.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from . import _native as N

_ELT = {torch.float16: 2, torch.bfloat16: 2, torch.int16: 2, torch.uint8: 1, torch.int8: 1,
        torch.float32: 4, torch.int32: 4}


@dataclass(frozen=True)
class KVGeometry:
    n_layers: int
    n_kv_heads: int
    head_dim: int
    page_tokens: int
    dtype: torch.dtype = torch.float16
    pool_layout: int = N.POOL_PAGED

    @property
    def elt_bytes(self) -> int:
        return _ELT[self.dtype]

    @property
    def planes(self) -> int:
        """(layer, kv) pairs."""
        return 2 * self.n_layers

    @property
    def row_elems(self) -> int:
        """Elements of one token in one plane."""
        return self.n_kv_heads * self.head_dim

    @property
    def token_elems(self) -> int:
        return self.planes * self.row_elems

    @property
    def bytes_per_token(self) -> int:
        return self.token_elems * self.elt_bytes

    @property
    def page_elems(self) -> int:
        return self.page_tokens * self.token_elems

    @property
    def page_bytes(self) -> int:
        return self.page_elems * self.elt_bytes

    @property
    def token_shape(self) -> tuple:
        """Per-token shape of the reference pool (``Model/qwen2.py:519-522``)."""
        return (self.head_dim, self.n_kv_heads, self.n_layers, 2)

    def pool_shape(self, n_pages: int) -> tuple:
        if self.pool_layout == N.POOL_PAGED:
            return (n_pages, self.n_layers, 2, self.page_tokens, self.n_kv_heads, self.head_dim)
        return (n_pages * self.page_tokens,) + self.token_shape

    def worker_shape(self, tokens: int) -> tuple:
        return (self.n_layers, 2, tokens, self.n_kv_heads, self.head_dim)

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_tokens - 1) // self.page_tokens

    def with_layout(self, layout: int) -> "KVGeometry":
        return replace(self, pool_layout=layout)

    def native(self) -> N.Geometry:
        return N.Geometry(self.n_layers, self.n_kv_heads, self.head_dim, self.page_tokens,
                          self.elt_bytes, self.pool_layout)


# Geometries of the benchmark configurations (K+V bytes).
GEO_A = KVGeometry(24, 2, 64, 16, torch.float16)     # Qwen2-0.5B-like, 192 KiB/page
GEO_B = KVGeometry(28, 4, 128, 16, torch.bfloat16)   # Qwen2-7B-like, 896 KiB/page
GEO_C = KVGeometry(80, 8, 128, 16, torch.float16)    # Llama-3-70B-like, 5 MiB/page
# The reference's own literals, in its token-major pool layout, 50-token pages.
GEO_R = KVGeometry(28, 2, 128, 50, torch.float16, N.POOL_TOKEN_MAJOR)
