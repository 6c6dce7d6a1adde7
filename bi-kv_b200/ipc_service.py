"""Drop-in for the reference's ``ipc_service`` extension module
(``SharedMemory/CUDA_Shared/ipc_service.cpp:240-257``): same function names, same
argument order, so ``kvcache.py``-style callers and the two test scripts
(``test_page_ipc.py``, ``test_zero_copy.py``) run against the new kernels -- consumer and
producer in two processes, as the reference runs them, or in one.

How it works, as in the reference (``ipc_service.cpp:20-110,146-168``, ``ipc_wrapper.h:14-28``):
``consumer_init`` creates a POSIX shared-memory block named ``shm_name`` holding two
process-shared semaphores, the ring cursors, the shape of the last transfer and the CUDA
IPC handle of the receive buffer it allocates; ``producer_init`` maps the block and opens
the handle; every transfer reserves a slice of the ring (wrapping to 0 without
back-pressure, ``copy_kernel.cu:87-89``), copies into it, records shape and offsets
(``copy_kernel.cu:116-128``) and posts ``sem_start``; ``consumer_receive`` waits on the
semaphore and returns a non-owning view into the ring.

Differences that a caller can observe:
  * ``consumer_receive`` waits at most ``timeout_s`` (default 60 s) and raises
    ``TimeoutError``, where the reference blocks for ever;
  * the control block also records the element type, and bf16 / fp32 transfers are accepted
    (the reference hard-codes fp16 on the receiving side, ``ipc_service.cpp:155-158``);
  * the block keeps the description (offset, size, shape, type) of each of the last 64
    transfers, not only of the latest, so the k-th ``consumer_receive`` returns the k-th
    transfer even when the producer has run ahead (its DATA is still overwritten once the
    ring wraps onto it, as in the reference);
  * copies run on torch's current stream, which ``producer_*`` synchronises before posting
    (the reference calls ``cudaDeviceSynchronize``);
  * a producer in the consumer's own process attaches to the buffer directly (CUDA does not
    open an IPC handle in the process that exported it).
Offsets are ELEMENT offsets, exactly as the reference kernel reads them
(``copy_kernel.cu:4-8``).
"""
from __future__ import annotations

import ctypes as C
import mmap
import os
import socket
import struct
import time
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from . import _native as N
from .mover import PageMover


@dataclass
class TensorDims:
    total_tokens: int = 0
    head_size: int = 0
    num_kv_heads: int = 0
    num_layers: int = 0
    kv_pair: int = 0


# ---- the control block ---------------------------------------------------------------
# Two sem_t (32 bytes each on glibc/x86-64 and aarch64), then little-endian fields.
_SEM_BYTES = 32
_FIELDS = struct.Struct("<QiiqQQQQQQ5q64sq")
# magic, device_id, dtype_code, consumer_pid, buffer_size, current_offset, last_valid_offset,
# data_size, tensor_dim, transfers, tensor_shape[5], cuda_handle[64], handle_offset
_HOST_AT = 2 * _SEM_BYTES + _FIELDS.size
# One descriptor per transfer in a ring of _DESCS entries: the reference keeps only the LAST
# transfer's shape and offset in the block, so a consumer that lags behind a producer reads a
# later transfer's description; here the k-th receive reads the k-th transfer's own.
_DESC = struct.Struct("<QQQQi5q")          # transfer number (from 1), offset, size, dim, dtype, shape[5]
_DESCS = 64
_DESC_AT = _HOST_AT + 256
_BLOCK_BYTES = _DESC_AT + _DESCS * _DESC.size
_MAGIC = 0x42494B5649504331           # "BIKVIPC1"
_DTYPES = [torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.uint8, torch.int32]
_libc = C.CDLL(None, use_errno=True)
_libc.sem_init.argtypes = [C.c_void_p, C.c_int, C.c_uint]
_libc.sem_post.argtypes = [C.c_void_p]
_libc.sem_destroy.argtypes = [C.c_void_p]


class _Timespec(C.Structure):
    _fields_ = [("tv_sec", C.c_long), ("tv_nsec", C.c_long)]


_libc.sem_timedwait.argtypes = [C.c_void_p, C.POINTER(_Timespec)]


def _shm_path(shm_name) -> str:
    name = shm_name.decode() if isinstance(shm_name, bytes) else str(shm_name)
    name = name.lstrip("/")
    if not name or "/" in name:
        raise RuntimeError(f"bad shared-memory name {shm_name!r}")
    return os.path.join("/dev/shm", name)


class _Control:
    """The mapped control block of one channel."""

    def __init__(self, path: str, create: bool):
        self.path = path
        flags = os.O_RDWR | (os.O_CREAT | os.O_EXCL if create else 0)
        if create:
            try:
                os.unlink(path)                     # the reference unlinks a stale block first
            except FileNotFoundError:
                pass
        try:
            fd = os.open(path, flags, 0o666)
        except OSError as e:
            raise RuntimeError(f"{'consumer' if create else 'producer'}_init shm_open failed: {e}") from e
        try:
            if create:
                os.ftruncate(fd, _BLOCK_BYTES)
            elif os.fstat(fd).st_size < _BLOCK_BYTES:
                raise RuntimeError("producer_init: the shared block is not a bikv ipc_service channel")
            self.map = mmap.mmap(fd, _BLOCK_BYTES)
        finally:
            os.close(fd)
        self._anchor = C.c_char.from_buffer(self.map)
        self.addr = C.addressof(self._anchor)
        self.sem_start = self.addr
        self.sem_complete = self.addr + _SEM_BYTES

    def read(self) -> list:
        return list(_FIELDS.unpack_from(self.map, 2 * _SEM_BYTES))

    def write(self, fields: list) -> None:
        _FIELDS.pack_into(self.map, 2 * _SEM_BYTES, *fields)

    def read_desc(self, transfer: int) -> tuple:
        return _DESC.unpack_from(self.map, _DESC_AT + (transfer % _DESCS) * _DESC.size)

    def write_desc(self, transfer: int, at: int, size: int, shape, dtype_code: int) -> None:
        _DESC.pack_into(self.map, _DESC_AT + (transfer % _DESCS) * _DESC.size, transfer, at, size, len(shape),
                        dtype_code, *(list(shape) + [0] * (5 - len(shape))))

    def close(self) -> None:
        self._anchor = None
        try:
            self.map.close()
        except BufferError:
            pass


class _Consumer:
    def __init__(self, device_id: int, shm_name, buffer_size: int):
        self.device = torch.device(f"cuda:{device_id}")
        self.ctrl = _Control(_shm_path(shm_name), create=True)
        self.buffer = torch.empty(buffer_size, dtype=torch.uint8, device=self.device)
        self.taken = 0                                   # transfers this consumer has received
        handle = C.create_string_buffer(64)
        off = C.c_int64(0)
        N.check(N.lib().bikv_pool_export(C.c_void_p(self.buffer.data_ptr()), handle, C.byref(off)), "bikv_pool_export")
        if _libc.sem_init(self.ctrl.sem_start, 1, 0) or _libc.sem_init(self.ctrl.sem_complete, 1, 0):
            raise RuntimeError("consumer_init sem_init failed")
        self.ctrl.write([_MAGIC, device_id, 0, os.getpid(), buffer_size, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0,
                         bytes(handle.raw), int(off.value)])
        host = socket.gethostname().encode()[:255]
        self.ctrl.map[_HOST_AT:_HOST_AT + 256] = host.ljust(256, b"\0")

    def receive(self, timeout_s: float) -> torch.Tensor:
        deadline = time.time() + timeout_s
        ts = _Timespec(int(deadline), int((deadline % 1) * 1e9))
        while _libc.sem_timedwait(self.ctrl.sem_start, C.byref(ts)) != 0:
            err = C.get_errno()
            if err == 4:          # EINTR
                continue
            if err == 110:        # ETIMEDOUT
                raise TimeoutError(f"consumer_receive: nothing was sent within {timeout_s} s")
            raise RuntimeError(f"consumer_receive sem_wait failed: errno {err}")
        self.taken += 1
        d = self.ctrl.read_desc(self.taken)
        if d[0] != self.taken:
            raise RuntimeError(f"consumer_receive: transfer {self.taken} was overrun (the producer is more than "
                               f"{_DESCS} transfers ahead)")
        at, size, dim, dtype, shape = d[1], d[2], d[3], _DTYPES[d[4]], d[5:10]
        return self.buffer[at:at + size].view(dtype).view(tuple(shape[:dim]))

    def cleanup(self) -> None:
        _libc.sem_destroy(self.ctrl.sem_start)
        _libc.sem_destroy(self.ctrl.sem_complete)
        path = self.ctrl.path
        self.ctrl.close()
        try:
            os.unlink(path)
        except FileNotFoundError:
            pass
        self.buffer = None


class _Producer:
    def __init__(self, device_id: int, shm_name):
        self.device = torch.device(f"cuda:{device_id}")
        self.ctrl = _Control(_shm_path(shm_name), create=False)
        f = self.ctrl.read()
        if f[0] != _MAGIC:
            raise RuntimeError("producer_init: the shared block is not a bikv ipc_service channel")
        host = bytes(self.ctrl.map[_HOST_AT:_HOST_AT + 256]).split(b"\0")[0]
        if host != socket.gethostname().encode()[:255]:
            raise RuntimeError("Processes must run on the same host")
        self.buffer_size = f[4]
        self.mapped = None
        local = _local_consumers.get(self.ctrl.path)
        if f[3] == os.getpid() and local is not None:
            self.base = local.buffer.data_ptr()           # same process: no IPC handle needed
        else:
            out = C.c_void_p()
            with torch.cuda.device(self.device):
                N.check(N.lib().bikv_pool_import(f[15], int(f[16]), C.byref(out)), "bikv_pool_import")
            self.base = int(out.value)
            self.mapped = (self.base, int(f[16]))

    def reserve(self, nbytes: int) -> int:
        if nbytes > self.buffer_size:
            raise RuntimeError("transfer larger than the shared buffer")
        f = self.ctrl.read()
        at = 0 if f[5] + nbytes > self.buffer_size else f[5]    # wraps without back-pressure
        return at

    def publish(self, at: int, nbytes: int, shape, dtype: torch.dtype) -> None:
        f = self.ctrl.read()
        f[2] = _DTYPES.index(dtype)
        f[5], f[6], f[7] = at + nbytes, at, nbytes
        f[8] = len(shape)
        f[9] += 1
        f[10:15] = list(shape) + [0] * (5 - len(shape))
        self.ctrl.write_desc(f[9], at, nbytes, shape, f[2])
        self.ctrl.write(f)
        _libc.sem_post(self.ctrl.sem_start)

    def cleanup(self) -> None:
        if self.mapped is not None:
            N.check(N.lib().bikv_pool_close(C.c_void_p(self.mapped[0]), self.mapped[1]), "bikv_pool_close")
            self.mapped = None
        self.ctrl.close()


_local_consumers: Dict[str, _Consumer] = {}
_consumer: Optional[_Consumer] = None
_producer: Optional[_Producer] = None
_movers: Dict[torch.device, PageMover] = {}


def _mover(device) -> PageMover:
    if device not in _movers:
        _movers[device] = PageMover(device)
    return _movers[device]


def _require(side, role):
    if side is None:
        raise RuntimeError(f"{role} side is not initialised")
    return side


def consumer_init(device_id: int, shm_name, buffer_size: int) -> None:
    """Creates the channel: control block ``shm_name`` and a receive ring of ``buffer_size``
    bytes on ``cuda:device_id`` (``ipc_service.cpp:20-74``)."""
    global _consumer
    path = _shm_path(shm_name)
    if path in _local_consumers:
        raise RuntimeError(f"shared buffer {shm_name!r} already exists")
    if len(shm_name) > 255 or buffer_size <= 0:
        raise RuntimeError("consumer_init: bad name or size")
    _consumer = _local_consumers[path] = _Consumer(device_id, shm_name, buffer_size)


def producer_init(device_id: int, shm_name) -> None:
    """Attaches to a channel a consumer created (``ipc_service.cpp:77-110``)."""
    global _producer
    _producer = _Producer(device_id, shm_name)


def producer_send(tensor: torch.Tensor) -> None:
    """One contiguous tensor into the ring (``ipc_service.cpp:113-143``)."""
    p = _require(_producer, "producer")
    if not tensor.is_cuda:
        raise RuntimeError("Tensor must be on CUDA")
    if not tensor.is_contiguous():
        raise RuntimeError("Tensor must be contiguous")
    if tensor.dtype not in _DTYPES or tensor.dim() > 5:
        raise RuntimeError("Tensor must be a floating tensor of at most 5 dimensions")
    nbytes = tensor.numel() * tensor.element_size()
    at = p.reserve(nbytes)
    with torch.cuda.device(p.device):
        _mover(p.device).copy_range(p.base + at, tensor.data_ptr(), nbytes)
        torch.cuda.current_stream(p.device).synchronize()
    p.publish(at, nbytes, tuple(tensor.shape), tensor.dtype)


def producer_copy_pages(cache_data: torch.Tensor, src_offsets: torch.Tensor, dest_offsets: torch.Tensor,
                        page_size: int, dims: TensorDims) -> None:
    """Pages of a device pool into the ring (``ipc_service.cpp:205-221`` over
    ``copy_kernel.cu:68-129``)."""
    if not cache_data.is_cuda:
        raise RuntimeError("Cache data must be on CUDA")
    _copy_pages(cache_data, src_offsets, dest_offsets, page_size, dims)


def producer_zero_copy_pages(cpu_data: torch.Tensor, page_indices: torch.Tensor, dest_offsets: torch.Tensor,
                             page_size: int, dims: TensorDims) -> None:
    """Pages of a pinned host pool into the ring, read in place over PCIe
    (``ipc_service.cpp:223-239`` over ``copy_kernel.cu:133-196``)."""
    if not cpu_data.is_pinned():
        raise RuntimeError("CPU data must be pinned memory")
    if not page_indices.is_cuda or not dest_offsets.is_cuda:
        raise RuntimeError("Page indices and dest offsets must be on CUDA")
    _copy_pages(cpu_data, page_indices, dest_offsets, page_size, dims)


def _copy_pages(src, src_offsets, dest_offsets, page_size, dims) -> None:
    p = _require(_producer, "producer")
    if not src.is_contiguous():
        raise RuntimeError("Cache data must be contiguous")
    if src.dtype not in _DTYPES:
        raise RuntimeError(f"unsupported pool dtype {src.dtype}")
    if src_offsets.dtype != torch.int64 or dest_offsets.dtype != torch.int64 or src_offsets.numel() != dest_offsets.numel():
        raise RuntimeError("offsets must be int64 arrays of equal length")
    num_pages = src_offsets.numel()
    per_token = dims.head_size * dims.num_kv_heads * dims.num_layers * dims.kv_pair
    page_elems = page_size * per_token
    nbytes = num_pages * page_elems * src.element_size()
    at = p.reserve(nbytes)
    with torch.cuda.device(p.device):
        st = torch.cuda.current_stream(p.device)
        rc = N.lib().bikv_copy_pages_flat(C.c_void_p(src.data_ptr()), C.c_void_p(p.base + at),
                                          C.c_void_p(src_offsets.data_ptr()), C.c_void_p(dest_offsets.data_ptr()),
                                          num_pages, int(page_elems), src.element_size(), C.c_void_p(int(st.cuda_stream)))
        N.check(rc, "bikv_copy_pages_flat")
        st.synchronize()
    p.publish(at, nbytes, (num_pages * page_size, dims.head_size, dims.num_kv_heads, dims.num_layers, dims.kv_pair),
              src.dtype)


def consumer_receive(timeout_s: float = 60.0) -> torch.Tensor:
    """Waits for the next transfer and returns a non-owning view of it inside the ring
    (overwritten when the ring wraps; ``ipc_service.cpp:146-168``)."""
    return _require(_consumer, "consumer").receive(timeout_s)


def producer_cleanup() -> None:
    global _producer
    if _producer is not None:
        _producer.cleanup()
    _producer = None


def consumer_cleanup() -> None:
    global _consumer
    if _consumer is not None:
        for k in [k for k, v in _local_consumers.items() if v is _consumer]:
            del _local_consumers[k]
        _consumer.cleanup()
    _consumer = None
