"""Drop-in for the reference's ``ipc_service`` extension module
(``SharedMemory/CUDA_Shared/ipc_service.cpp:240-257``): same function names, same
argument order, so ``kvcache.py``-style callers and the two test scripts
(``test_page_ipc.py``, ``test_zero_copy.py``) run against the new kernels.

Differences that a caller can observe:
  * there is no POSIX shared-memory control block and no semaphore hand-off; within
    one process ``consumer_init`` allocates the receive buffer and ``producer_init``
    attaches to it by name;
  * copies run on torch's current stream and ``producer_copy_pages`` synchronises
    that stream before returning (the reference calls ``cudaDeviceSynchronize``);
  * bf16 pools are accepted (the reference dispatches fp16/fp32/fp64 only).
Offsets are ELEMENT offsets, exactly as the reference kernel reads them
(``copy_kernel.cu:4-8``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .mover import PageMover


@dataclass
class TensorDims:
    total_tokens: int = 0
    head_size: int = 0
    num_kv_heads: int = 0
    num_layers: int = 0
    kv_pair: int = 0


class _Channel:
    def __init__(self, device, nbytes):
        self.device = torch.device(f"cuda:{device}" if isinstance(device, int) else device)
        self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.current_offset = 0
        self.last_valid_offset = 0
        self.data_size = 0
        self.shape = None
        self.dtype = None


_channels: Dict[bytes, _Channel] = {}
_consumer: Optional[_Channel] = None
_producer: Optional[_Channel] = None
_movers: Dict[torch.device, PageMover] = {}


def _name(shm_name) -> bytes:
    return shm_name if isinstance(shm_name, bytes) else str(shm_name).encode()


def _mover(device) -> PageMover:
    if device not in _movers:
        _movers[device] = PageMover(device)
    return _movers[device]


def consumer_init(device_id: int, shm_name, buffer_size: int) -> None:
    global _consumer
    name = _name(shm_name)
    if name in _channels:
        raise RuntimeError(f"shared buffer {name!r} already exists")
    _consumer = _channels[name] = _Channel(device_id, buffer_size)


def producer_init(device_id: int, shm_name) -> None:
    global _producer
    ch = _channels.get(_name(shm_name))
    if ch is None:
        raise RuntimeError(f"shared buffer {_name(shm_name)!r} has not been created by a consumer")
    _producer = ch


def _reserve(ch: _Channel, nbytes: int) -> int:
    if nbytes > ch.buffer.numel():
        raise RuntimeError("transfer larger than the shared buffer")
    if ch.current_offset + nbytes > ch.buffer.numel():
        ch.current_offset = 0  # the reference wraps without back-pressure (copy_kernel.cu:87-89)
    at = ch.current_offset
    ch.last_valid_offset = at
    ch.current_offset += nbytes
    ch.data_size = nbytes
    return at


def producer_send(tensor: torch.Tensor) -> None:
    ch = _require(_producer, "producer")
    t = tensor.contiguous()
    nbytes = t.numel() * t.element_size()
    at = _reserve(ch, nbytes)
    _mover(ch.device).copy_range(ch.buffer.data_ptr() + at, t.data_ptr(), nbytes)
    ch.shape, ch.dtype = tuple(t.shape), t.dtype
    torch.cuda.current_stream(ch.device).synchronize()


def producer_copy_pages(cache_data: torch.Tensor, src_offsets: torch.Tensor, dest_offsets: torch.Tensor,
                        page_size: int, dims: TensorDims) -> None:
    if not cache_data.is_cuda:
        raise RuntimeError("Cache data must be on CUDA")
    _copy_pages(cache_data, src_offsets, dest_offsets, page_size, dims)


def producer_zero_copy_pages(cpu_data: torch.Tensor, page_indices: torch.Tensor, dest_offsets: torch.Tensor,
                             page_size: int, dims: TensorDims) -> None:
    if not cpu_data.is_pinned():
        raise RuntimeError("CPU data must be pinned memory")
    if not page_indices.is_cuda or not dest_offsets.is_cuda:
        raise RuntimeError("Page indices and dest offsets must be on CUDA")
    _copy_pages(cpu_data, page_indices, dest_offsets, page_size, dims)


def _copy_pages(src, src_offsets, dest_offsets, page_size, dims) -> None:
    ch = _require(_producer, "producer")
    if not src.is_contiguous():
        raise RuntimeError("Cache data must be contiguous")
    num_pages = src_offsets.numel()
    per_token = dims.head_size * dims.num_kv_heads * dims.num_layers * dims.kv_pair
    page_elems = page_size * per_token
    nbytes = num_pages * page_elems * src.element_size()
    at = _reserve(ch, nbytes)
    dst = ch.buffer[at:at + nbytes].view(src.dtype)
    _mover(ch.device).copy_pages_flat(src, dst, src_offsets, dest_offsets, page_elems)
    ch.shape = (num_pages * page_size, dims.head_size, dims.num_kv_heads, dims.num_layers, dims.kv_pair)
    ch.dtype = src.dtype
    torch.cuda.current_stream(ch.device).synchronize()


def consumer_receive() -> torch.Tensor:
    """Non-owning view of the last transfer (overwritten when the buffer wraps)."""
    ch = _require(_consumer, "consumer")
    if ch.shape is None:
        raise RuntimeError("nothing has been sent")
    return ch.buffer[ch.last_valid_offset:ch.last_valid_offset + ch.data_size].view(ch.dtype).view(ch.shape)


def producer_cleanup() -> None:
    global _producer
    _producer = None


def consumer_cleanup() -> None:
    global _consumer
    if _consumer is not None:
        for k in [k for k, v in _channels.items() if v is _consumer]:
            del _channels[k]
    _consumer = None


def _require(ch, role):
    if ch is None:
        raise RuntimeError(f"{role} side is not initialised")
    return ch
