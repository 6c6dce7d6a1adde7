"""PageMover: launches gather / scatter for one worker GPU.

Owns the small device-side state the C ABI leaves to the caller: the status
words a kernel's bounded wait reports into, and the device staging buffer a
host-resident plan is uploaded to.
"""
from __future__ import annotations

import ctypes as C
import threading
import weakref
from typing import Optional, Sequence, Union

import numpy as np
import torch

from . import _native as N
from .geometry import KVGeometry
from .plan import Plan
from .pool import ShardedPool

Tensors = Union[torch.Tensor, Sequence[torch.Tensor]]


class PageMover:
    def __init__(self, device=None, variant: int = N.VARIANT_AUTO):
        if not torch.cuda.is_available():
            raise RuntimeError("PageMover needs a CUDA device: the KV-page path has no CPU implementation")
        N.lib()  # fail now, loudly, if the library is missing
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.variant = variant
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        # Plan staging on the device, one buffer per stream: calls on one stream reuse it in
        # stream order; calls on different streams must not share it.
        self._scratch_by_stream: dict = {}
        # The reference serves its data methods from a 20-thread gRPC pool; one lock keeps
        # this object's host-side state (staging buffers, tables, in-flight list) consistent.
        self._lock = threading.RLock()
        self._req_ring: list = []     # [pinned table, event of the upload that read it]
        self._req_next = 0
        self._req_slot = 0
        self._req_cache: dict = {}    # (geometry, ids of a tensor list) -> (pinned table, weak refs, addresses)
        self._inflight: list = []     # (event, plan): host buffers the GPU may not have read yet
        self._layer_tables: dict = {}

    # -- helpers -----------------------------------------------------------
    def _stream(self, stream) -> int:
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        return int(s.cuda_stream)

    def _scratch_for(self, n_pages: int, n_requests: int, stream=None) -> torch.Tensor:
        need = N.lib().bikv_plan_scratch_bytes(n_pages, n_requests)
        key = self._stream(stream)
        buf = self._scratch_by_stream.get(key)
        if buf is None or buf.numel() < need:
            # A buffer being replaced may still be read by queued work; torch frees it in
            # stream order of ITS allocation stream, so wait for this stream first.
            if buf is not None:
                torch.cuda.current_stream(self.device).synchronize() if stream is None else stream.synchronize()
            buf = torch.empty(max(int(need * 1.5), 1 << 20), dtype=torch.uint8, device=self.device)
            self._scratch_by_stream[key] = buf
        return buf

    def request_table(self, geom: KVGeometry, tensors: Tensors) -> torch.Tensor:
        """Host (pinned) int64 [n, 2] table of (base pointer, tokens) for worker tensors
        of shape ``geom.worker_shape(T)``.  Tables come from a small ring of pinned buffers;
        a buffer is reused only after the upload that last read it has run."""
        ts = [tensors] if isinstance(tensors, torch.Tensor) else list(tensors)
        n = len(ts)
        # The same tensor objects as in an earlier call (a serving loop reuses its KV tensors):
        # their table is kept so that nothing is checked or written again.  Entries hold weak
        # references only, and a hit requires the very same live objects at the same addresses.
        key = (geom, tuple(map(id, ts)))
        hit = self._req_cache.get(key)
        if hit is not None:
            table, refs, ptrs = hit
            if all(r() is t and t.data_ptr() == p for r, t, p in zip(refs, ts, ptrs)):
                self._req_slot = None
                return table
            del self._req_cache[key]
        table = self._build_request_table(geom, ts)
        if n:
            keep = torch.empty((n, 2), dtype=torch.int64).pin_memory()
            keep.copy_(table)
            if len(self._req_cache) >= 8:
                self._req_cache.pop(next(iter(self._req_cache)))
            self._req_cache[key] = (keep, [weakref.ref(t) for t in ts], [t.data_ptr() for t in ts])
        return table

    def _build_request_table(self, geom: KVGeometry, ts: list) -> torch.Tensor:
        n = len(ts)
        slot = self._req_next % 8
        self._req_next += 1
        while len(self._req_ring) <= slot:
            self._req_ring.append([None, None])
        buf, ev = self._req_ring[slot]
        if ev is not None and not ev.query():
            ev.synchronize()
        if buf is None or buf.shape[0] < n:
            buf = torch.empty((max(n, 64), 2), dtype=torch.int64).pin_memory()
        self._req_ring[slot] = [buf, None]
        self._req_slot = slot
        head, tail = (geom.n_layers, 2), (geom.n_kv_heads, geom.head_dim)
        rows = []
        for i, t in enumerate(ts):
            sh = tuple(t.shape)
            if len(sh) != 5 or sh[:2] != head or sh[3:] != tail:
                raise ValueError(f"worker tensor {i} has shape {sh}, want {geom.worker_shape('T')}")
            if t.element_size() != geom.elt_bytes or not t.is_contiguous():
                raise ValueError(f"worker tensor {i} must be contiguous with {geom.elt_bytes}-byte elements")
            if t.device != self.device:
                raise ValueError(f"worker tensor {i} lives on {t.device}, mover on {self.device}")
            rows.append((t.data_ptr(), sh[2]))
        if rows:
            buf.numpy()[:n] = rows
        return buf[:n]

    # -- host-plan path ----------------------------------------------------
    def _run_h(self, fn, pool: ShardedPool, plan: Plan, tensors: Tensors, validate: bool,
               variant: Optional[int], stream) -> None:
        if plan.n_pages == 0:
            return
        with self._lock:
            self._run_h_locked(fn, pool, plan, tensors, validate, variant, stream)

    def _run_h_locked(self, fn, pool, plan, tensors, validate, variant, stream) -> None:
        reqs = self.request_table(pool.geom, tensors)
        if len(reqs) < plan.n_requests:
            raise ValueError(f"plan names {plan.n_requests} worker tensors, {len(reqs)} given")
        scratch = self._scratch_for(plan.n_pages, len(reqs), stream)
        g = pool.geom.native()
        rc = fn(C.byref(pool.desc), C.byref(g), C.c_void_p(plan.host_ptr), plan.n_pages,
                C.c_void_p(reqs.data_ptr()), len(reqs), C.c_void_p(scratch.data_ptr()),
                scratch.numel(), int(validate), self.variant if variant is None else variant,
                C.c_void_p(self.status.data_ptr()), C.c_void_p(self._stream(stream)))
        N.check(rc, fn.__name__)
        self._hold(plan, stream)

    def _hold(self, plan: Plan, stream) -> None:
        """Keeps ``plan`` (its pinned host buffer) alive until the stream has consumed the
        upload, even if the caller drops it right after the call."""
        self._inflight = [(e, p) for e, p in self._inflight if not e.query()]
        ev = torch.cuda.Event()
        ev.record(stream if stream is not None else torch.cuda.current_stream(self.device))
        self._inflight.append((ev, plan))
        if self._req_ring and self._req_slot is not None:
            self._req_ring[self._req_slot][1] = ev

    def gather(self, pool: ShardedPool, plan: Plan, tensors: Tensors, *, validate: bool = True,
               variant: Optional[int] = None, stream=None) -> None:
        """Pool pages -> worker tensors (``[layer, kv, token, head, dim]``), asynchronously."""
        self._run_h(N.lib().bikv_gather_h, pool, plan, tensors, validate, variant, stream)

    def scatter(self, pool: ShardedPool, plan: Plan, tensors: Tensors, *, validate: bool = True,
                variant: Optional[int] = None, stream=None) -> None:
        """Worker tensors -> pool pages (inverse map of :meth:`gather`)."""
        self._run_h(N.lib().bikv_scatter_h, pool, plan, tensors, validate, variant, stream)

    def gather_table(self, pool: ShardedPool, plan: Plan, request_table: torch.Tensor, *, validate: bool = True,
                     variant: Optional[int] = None, stream=None) -> None:
        """:meth:`gather` with a ready request table: host int64 ``[n, 2]`` rows of (base pointer,
        tokens), pinned for an asynchronous upload.  For worker tensors that are not torch tensors
        of this process -- e.g. another GPU's tensors mapped through an IPC handle, when the
        owner of the pages pushes them (``push.py``).  The table must stay unchanged until the
        stream has passed the call."""
        self._run_table(N.lib().bikv_gather_h, pool, plan, request_table, validate, variant, stream)

    def scatter_table(self, pool: ShardedPool, plan: Plan, request_table: torch.Tensor, *, validate: bool = True,
                      variant: Optional[int] = None, stream=None) -> None:
        self._run_table(N.lib().bikv_scatter_h, pool, plan, request_table, validate, variant, stream)

    def _run_table(self, fn, pool, plan, request_table, validate, variant, stream) -> None:
        if plan.n_pages == 0:
            return
        with self._lock:
            self._run_table_locked(fn, pool, plan, request_table, validate, variant, stream)

    def _run_table_locked(self, fn, pool, plan, request_table, validate, variant, stream) -> None:
        if request_table.dtype != torch.int64 or request_table.dim() != 2 or request_table.shape[1] != 2 \
                or not request_table.is_contiguous() or request_table.is_cuda:
            raise ValueError("request_table must be a contiguous host int64 [n, 2] tensor")
        n = request_table.shape[0]
        scratch = self._scratch_for(plan.n_pages, n, stream)
        g = pool.geom.native()
        rc = fn(C.byref(pool.desc), C.byref(g), C.c_void_p(plan.host_ptr), plan.n_pages,
                C.c_void_p(request_table.data_ptr()), n, C.c_void_p(scratch.data_ptr()), scratch.numel(),
                int(validate), self.variant if variant is None else variant,
                C.c_void_p(self.status.data_ptr()), C.c_void_p(self._stream(stream)))
        N.check(rc, fn.__name__)
        ev = torch.cuda.Event()
        ev.record(stream if stream is not None else torch.cuda.current_stream(self.device))
        self._inflight = [(e, p) for e, p in self._inflight if not e.query()]
        self._inflight.append((ev, (plan, request_table)))

    # -- device-plan path --------------------------------------------------
    def upload(self, plan: Plan, geom: KVGeometry, tensors: Tensors):
        """Copies a plan and its request table to fresh device tensors (for repeated
        launches of one plan)."""
        recs = torch.from_numpy(np.ascontiguousarray(plan.table)).to(self.device)
        reqs = self.request_table(geom, tensors).to(self.device)
        return recs, reqs

    def _run_d(self, fn, pool: ShardedPool, recs: torch.Tensor, reqs: torch.Tensor,
               variant: Optional[int], stream) -> None:
        g = pool.geom.native()
        rc = fn(C.byref(pool.desc), C.byref(g), C.c_void_p(recs.data_ptr()), recs.shape[0],
                C.c_void_p(reqs.data_ptr()), reqs.shape[0], self.variant if variant is None else variant,
                C.c_void_p(self.status.data_ptr()), C.c_void_p(self._stream(stream)))
        N.check(rc, fn.__name__)

    def gather_dev(self, pool, recs, reqs, *, variant=None, stream=None) -> None:
        self._run_d(N.lib().bikv_gather, pool, recs, reqs, variant, stream)

    def scatter_dev(self, pool, recs, reqs, *, variant=None, stream=None) -> None:
        self._run_d(N.lib().bikv_scatter, pool, recs, reqs, variant, stream)

    # -- paged worker KV ("NHD": one [slot, kv, head, dim] tensor per layer) ----
    def layer_table(self, geom: KVGeometry, layers: Sequence[torch.Tensor]) -> tuple:
        """(device int64 [n_layers] of base pointers, slots per layer) for a worker's paged
        KV cache; cached per set of tensors."""
        key = tuple(t.data_ptr() for t in layers)
        hit = self._layer_tables.get(key)
        if hit is not None:
            return hit
        if len(layers) != geom.n_layers:
            raise ValueError(f"{len(layers)} layer tensors for {geom.n_layers} layers")
        slots = layers[0].shape[0]
        for i, t in enumerate(layers):
            if tuple(t.shape) != (slots, 2, geom.n_kv_heads, geom.head_dim) or not t.is_contiguous() \
                    or t.element_size() != geom.elt_bytes or t.device != self.device:
                raise ValueError(f"layer tensor {i}: want contiguous [{slots}, 2, {geom.n_kv_heads}, "
                                 f"{geom.head_dim}] on {self.device}, got {tuple(t.shape)} on {t.device}")
        table = torch.tensor(key, dtype=torch.int64).to(self.device)
        if len(self._layer_tables) > 64:
            self._layer_tables.clear()
        self._layer_tables[key] = (table, slots, list(layers))
        return self._layer_tables[key]

    def _run_nhd(self, fn, pool: ShardedPool, plan: Plan, layers, validate: bool, check_overlap: bool, stream) -> None:
        if plan.n_pages == 0:
            return
        with self._lock:
            self._run_nhd_locked(fn, pool, plan, layers, validate, check_overlap, stream)

    def _run_nhd_locked(self, fn, pool, plan, layers, validate, check_overlap, stream) -> None:
        table, slots, _ = self.layer_table(pool.geom, layers)
        g = pool.geom.native()
        if validate:
            N.check(N.lib().bikv_plan_validate_nhd(C.c_void_p(plan.host_ptr), plan.n_pages, slots, C.byref(pool.desc),
                                                   C.byref(g), int(check_overlap)), "bikv_plan_validate_nhd")
        nbytes = plan.n_pages * 16
        scratch = self._scratch_for(plan.n_pages, 0, stream)
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(st):
            scratch[:nbytes].copy_(plan._store.view(torch.uint8).view(-1)[:nbytes], non_blocking=True)
        N.check(fn(C.byref(pool.desc), C.byref(g), C.c_void_p(scratch.data_ptr()), plan.n_pages,
                   C.c_void_p(table.data_ptr()), slots, C.c_void_p(self.status.data_ptr()),
                   C.c_void_p(int(st.cuda_stream))), fn.__name__)
        self._hold(plan, stream)

    def gather_nhd(self, pool: ShardedPool, plan: Plan, layers: Sequence[torch.Tensor], *, validate: bool = True,
                   stream=None) -> None:
        """Pool pages -> the worker's paged KV.  ``plan`` rows are (page_id, valid_tokens, -,
        first slot); ``layers[l]`` is the layer-``l`` tensor ``[slots, 2, heads, dim]``."""
        self._run_nhd(N.lib().bikv_gather_nhd, pool, plan, layers, validate, False, stream)

    def scatter_nhd(self, pool: ShardedPool, plan: Plan, layers: Sequence[torch.Tensor], *, validate: bool = True,
                    stream=None) -> None:
        self._run_nhd(N.lib().bikv_scatter_nhd, pool, plan, layers, validate, True, stream)

    # -- flat copy ---------------------------------------------------------
    def copy_pages_flat(self, src: torch.Tensor, dst: torch.Tensor, src_off: torch.Tensor,
                        dst_off: torch.Tensor, page_elems: int, *, stream=None) -> None:
        """``dst[dst_off[i]+e] = src[src_off[i]+e]`` for ``e < page_elems`` (element offsets)."""
        if src_off.dtype != torch.int64 or dst_off.dtype != torch.int64:
            raise TypeError("offsets must be int64")
        if src_off.shape != dst_off.shape:
            raise ValueError("offset arrays differ in length")
        rc = N.lib().bikv_copy_pages_flat(C.c_void_p(src.data_ptr()), C.c_void_p(dst.data_ptr()),
                                          C.c_void_p(src_off.data_ptr()), C.c_void_p(dst_off.data_ptr()),
                                          src_off.numel(), int(page_elems), src.element_size(),
                                          C.c_void_p(self._stream(stream)))
        N.check(rc, "bikv_copy_pages_flat")

    def copy_range(self, dst_ptr: int, src_ptr: int, nbytes: int, *, stream=None) -> None:
        rc = N.lib().bikv_copy_range(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), int(nbytes),
                                     C.c_void_p(self._stream(stream)))
        N.check(rc, "bikv_copy_range")

    def copy_range_engine(self, dst_ptr: int, src_ptr: int, nbytes: int, *, stream=None) -> None:
        """The same range moved by the copy engines (no kernel, no SM)."""
        rc = N.lib().bikv_copy_range_engine(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), int(nbytes),
                                            C.c_void_p(self._stream(stream)))
        N.check(rc, "bikv_copy_range_engine")

    # -- status ------------------------------------------------------------
    def check_status(self) -> None:
        """Synchronising read of the device status words; raises if a kernel's bounded
        wait ran out, and clears the words."""
        st = self.status.cpu()
        if int(st[0]) != 0:
            self.status.zero_()
            raise N.BikvError(int(st[0]), "device status")
