"""Drop-in for the reference's ``rdma_onesided_transport`` extension module
(``NetworkTransport/onesided_rdma_module.cpp:8-85``): class ``RDMAOneSidedEndpoint`` with the
same constructor, method names and argument order, for callers written against it
(``DistributedStorage/kvcache.py:25,88-94``, ``Worker/Worker.py:20,110-139``).

Inside one box there is no NIC between the two ends: a "registered buffer" is memory both
processes can address -- a GPU allocation opened through a CUDA IPC handle, or a POSIX
shared-memory block that each side page-locks for its GPU -- and a one-sided write or read is
ONE contiguous byte-range copy between two such buffers, issued by the server's GPU and
complete when the call returns (``NetworkTransport/onesided_rdma.h:652-759``: one work request
per range, then a busy-poll of the completion queue, ``:955-972``).

Roles, as in the reference.  The SERVER (a KVCache shard) keeps one local cpu buffer and one
local gpu buffer PER CLIENT (``run_server(max_clients, local_cpu_size, local_gpu_size)``); a
CLIENT (a worker) brings one cpu and one gpu buffer (``connect_client(rank, cpu_size,
gpu_size)``).  Only the server posts:
  ``post_rdma_write(rank, size, src_type, dst_type, local_offset, remote_offset)``
      server's local ``src_type`` buffer for that client  ->  the client's ``dst_type`` buffer
  ``post_rdma_read(...)``
      the client's ``src_type`` buffer  ->  server's local ``dst_type`` buffer for that client
Both return 0, or -1 with a line on stderr (unknown rank, range outside a buffer, wrong mode).

The two ends meet over a TCP connection to ``ip:port`` (the reference uses the RDMA
connection manager plus a TCP side channel, ``onesided_rdma.h:560-650``): the client sends
one JSON line naming its buffers, the server maps them and answers.  ``hugepage`` is accepted
and ignored.
"""
from __future__ import annotations

import ctypes as C
import json
import mmap
import os
import socket
import sys
import threading
import uuid
from typing import Dict, Optional

import torch

from . import _native as N

_local_clients: Dict[tuple, "RDMAOneSidedEndpoint"] = {}     # (port, rank) -> client endpoint of this process
_local_lock = threading.Lock()


class _HostBuffer:
    """A byte buffer in a POSIX shared-memory block, page-locked for this process's GPUs."""

    def __init__(self, nbytes: int, name: Optional[str] = None):
        self.created = name is None
        self.name = name or f"bikv_rdma_{os.getpid()}_{uuid.uuid4().hex[:10]}"
        path = os.path.join("/dev/shm", self.name)
        fd = os.open(path, os.O_RDWR | (os.O_CREAT | os.O_EXCL if self.created else 0), 0o600)
        try:
            if self.created:
                os.ftruncate(fd, nbytes)
            self.map = mmap.mmap(fd, nbytes)
        finally:
            os.close(fd)
        self.nbytes = nbytes
        self.tensor = torch.frombuffer(self.map, dtype=torch.uint8)
        self.ptr = self.tensor.data_ptr()
        self.registered = False
        if torch.cuda.is_available():
            N.check(N.lib().bikv_host_register(C.c_void_p(self.ptr), nbytes), "bikv_host_register")
            self.registered = True

    def close(self) -> None:
        if self.registered:
            N.lib().bikv_host_unregister(C.c_void_p(self.ptr))
            self.registered = False
        self.tensor = None
        try:
            self.map.close()
        except BufferError:
            pass
        if self.created:
            try:
                os.unlink(os.path.join("/dev/shm", self.name))
            except FileNotFoundError:
                pass


class _Peer:
    """What the server knows about one client."""

    def __init__(self):
        self.remote = {"cpu": (0, 0), "gpu": (0, 0)}      # type -> (pointer valid here, size)
        self.local = {"cpu": None, "gpu": None}           # type -> uint8 tensor
        self.host_map: Optional[_HostBuffer] = None
        self.gpu_map: Optional[tuple] = None              # (mapped pointer, offset) to close


class RDMAOneSidedEndpoint:
    def __init__(self, ip: str, port: str, mode: str):
        if mode not in ("server", "client"):
            raise ValueError("mode must be 'server' or 'client'")
        self.ip, self.port, self.mode = ip, int(port), mode
        self._peers: Dict[int, _Peer] = {}
        self._listener: Optional[socket.socket] = None
        self._cpu: Optional[_HostBuffer] = None
        self._gpu: Optional[torch.Tensor] = None
        self._rank: Optional[int] = None
        self.use_copy_engine = False      # True: cudaMemcpyAsync instead of the copy kernel
        self.timeout_s = 120.0

    # ------------------------------------------------------------------ server
    def run_server(self, max_clients: int, local_cpu_size: int, local_gpu_size: int, hugepage: bool = False) -> int:
        """Accepts ``max_clients`` clients; for each, allocates the server-side cpu (pinned) and
        gpu buffers of the given sizes and maps the client's buffers."""
        if self.mode != "server":
            print("[Error] run_server on a client endpoint.", file=sys.stderr)
            return -1
        try:
            self._listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            self._listener.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            self._listener.bind(("0.0.0.0" if self.ip in ("", "0.0.0.0") else self.ip, self.port))
            self._listener.listen(max(1, max_clients))
            self._listener.settimeout(self.timeout_s)
            while len(self._peers) < max_clients:
                conn, _ = self._listener.accept()
                with conn:
                    conn.settimeout(self.timeout_s)
                    hello = json.loads(conn.makefile("r").readline())
                    try:
                        self._admit(hello, local_cpu_size, local_gpu_size)
                        conn.sendall(b'{"ok": true}\n')
                    except Exception as e:  # noqa: BLE001  (this client is refused, others may still come)
                        conn.sendall((json.dumps({"ok": False, "error": str(e)}) + "\n").encode())
                        print(f"[Server] client refused: {e}", file=sys.stderr)
            return 0
        except Exception as e:  # noqa: BLE001
            print(f"[Server] run_server failed: {e}", file=sys.stderr)
            return -1
        finally:
            if self._listener is not None:
                self._listener.close()
                self._listener = None

    def _admit(self, hello: dict, local_cpu_size: int, local_gpu_size: int) -> None:
        rank = int(hello["rank"])
        peer = _Peer()
        same_process = hello.get("pid") == os.getpid()
        with _local_lock:
            local = _local_clients.get((self.port, rank)) if same_process else None
        cpu, gpu = hello.get("cpu"), hello.get("gpu")
        if cpu and cpu["size"] > 0:
            if local is not None:
                peer.remote["cpu"] = (local._cpu.ptr, local._cpu.nbytes)
            else:
                peer.host_map = _HostBuffer(int(cpu["size"]), name=cpu["shm"])
                peer.remote["cpu"] = (peer.host_map.ptr, peer.host_map.nbytes)
        if gpu and gpu["size"] > 0:
            if local is not None:
                peer.remote["gpu"] = (local._gpu.data_ptr(), local._gpu.numel())
            else:
                out = C.c_void_p()
                N.check(N.lib().bikv_pool_import(bytes.fromhex(gpu["handle"]), int(gpu["offset"]), C.byref(out)),
                        "bikv_pool_import")
                peer.gpu_map = (int(out.value), int(gpu["offset"]))
                peer.remote["gpu"] = (int(out.value), int(gpu["size"]))
        if local_cpu_size > 0:
            t = torch.empty(local_cpu_size, dtype=torch.uint8)
            peer.local["cpu"] = t.pin_memory() if torch.cuda.is_available() else t
        if local_gpu_size > 0:
            peer.local["gpu"] = torch.empty(local_gpu_size, dtype=torch.uint8, device="cuda")
        self._peers[rank] = peer

    # ------------------------------------------------------------------ client
    def connect_client(self, rank: int, cpu_size: int, gpu_size: int, hugepage: bool = False) -> int:
        """Allocates this client's cpu and gpu buffers (once) and registers them with the
        server at ``ip:port``.  Returns -1 when the server is not there yet, so that callers
        can retry as the reference's worker does (``Worker/Worker.py:118-133``)."""
        if self.mode != "client":
            print("[Error] connect_client on a server endpoint.", file=sys.stderr)
            return -1
        try:
            if self._cpu is None and cpu_size > 0:
                self._cpu = _HostBuffer(cpu_size)
            if self._gpu is None and gpu_size > 0:
                self._gpu = torch.empty(gpu_size, dtype=torch.uint8, device="cuda")
            self._rank = rank
            hello = {"rank": rank, "pid": os.getpid(), "cpu": None, "gpu": None}
            if self._cpu is not None:
                hello["cpu"] = {"size": self._cpu.nbytes, "shm": self._cpu.name}
            if self._gpu is not None:
                handle = C.create_string_buffer(64)
                off = C.c_int64(0)
                N.check(N.lib().bikv_pool_export(C.c_void_p(self._gpu.data_ptr()), handle, C.byref(off)),
                        "bikv_pool_export")
                hello["gpu"] = {"size": self._gpu.numel(), "handle": bytes(handle.raw).hex(), "offset": int(off.value),
                                "device": self._gpu.device.index}
            with _local_lock:
                _local_clients[(self.port, rank)] = self
            with socket.create_connection((self.ip, self.port), timeout=self.timeout_s) as s:
                s.sendall((json.dumps(hello) + "\n").encode())
                reply = json.loads(s.makefile("r").readline())
            if not reply.get("ok"):
                print(f"[Client] refused by the server: {reply.get('error')}", file=sys.stderr)
                return -1
            return 0
        except (ConnectionError, OSError, socket.timeout):
            return -1

    # ------------------------------------------------------------------ one-sided operations
    def _post(self, what: str, rank: int, size: int, src_type: str, dst_type: str, local_offset: int,
              remote_offset: int) -> int:
        if self.mode != "server":
            print(f"[Error] Only server can initiate RDMA {what}.", file=sys.stderr)
            return -1
        peer = self._peers.get(rank)
        if peer is None:
            print(f"[post_rdma_{what}] Client rank {rank} not found.", file=sys.stderr)
            return -1
        local_type, remote_type = (src_type, dst_type) if what == "write" else (dst_type, src_type)
        local = peer.local.get(local_type)
        remote_ptr, remote_size = peer.remote.get(remote_type, (0, 0))
        if size < 0 or local_offset < 0 or remote_offset < 0 or local is None or local_offset + size > local.numel():
            print(f"[post_rdma_{what}] Invalid {'source' if what == 'write' else 'destination'} memory for client.",
                  file=sys.stderr)
            return -1
        if not remote_ptr or remote_offset + size > remote_size:
            print(f"[post_rdma_{what}] Invalid {'destination' if what == 'write' else 'source'} memory.", file=sys.stderr)
            return -1
        if size == 0:
            return 0
        here, there = local.data_ptr() + local_offset, remote_ptr + remote_offset
        dst, src = (there, here) if what == "write" else (here, there)
        try:
            stream = torch.cuda.current_stream()
            fn = N.lib().bikv_copy_range_engine if self.use_copy_engine else N.lib().bikv_copy_range
            N.check(fn(C.c_void_p(dst), C.c_void_p(src), int(size), C.c_void_p(int(stream.cuda_stream))), fn.__name__)
            stream.synchronize()          # the reference returns once the completion has been polled
            return 0
        except Exception as e:  # noqa: BLE001
            print(f"[post_rdma_{what}] copy failed: {e}", file=sys.stderr)
            return -1

    def post_rdma_write(self, rank: int, size: int, src_type: str, dst_type: str, local_offset: int = 0,
                        remote_offset: int = 0) -> int:
        return self._post("write", rank, size, src_type, dst_type, local_offset, remote_offset)

    def post_rdma_read(self, rank: int, size: int, src_type: str, dst_type: str, local_offset: int = 0,
                       remote_offset: int = 0) -> int:
        return self._post("read", rank, size, src_type, dst_type, local_offset, remote_offset)

    # ------------------------------------------------------------------ buffers as tensors
    def get_server_cpu_tensor(self, rank: int) -> torch.Tensor:
        return self._server_tensor(rank, "cpu")

    def get_server_gpu_tensor(self, rank: int) -> torch.Tensor:
        return self._server_tensor(rank, "gpu")

    def _server_tensor(self, rank: int, kind: str) -> torch.Tensor:
        peer = self._peers.get(rank)
        if peer is None or peer.local[kind] is None:
            raise RuntimeError(f"Client rank {rank} not found or its {kind.upper()} memory is not allocated.")
        return peer.local[kind]

    def get_client_cpu_tensor(self) -> torch.Tensor:
        if self._cpu is None:
            raise RuntimeError("Local CPU memory not allocated.")
        return self._cpu.tensor

    def get_client_gpu_tensor(self) -> torch.Tensor:
        if self._gpu is None:
            raise RuntimeError("Local GPU memory not allocated.")
        return self._gpu

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        for peer in self._peers.values():
            if peer.gpu_map is not None:
                N.lib().bikv_pool_close(C.c_void_p(peer.gpu_map[0]), peer.gpu_map[1])
            if peer.host_map is not None:
                peer.host_map.close()
        self._peers.clear()
        if self._rank is not None:
            with _local_lock:
                _local_clients.pop((self.port, self._rank), None)
        if self._cpu is not None:
            self._cpu.close()
            self._cpu = None
        self._gpu = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass
