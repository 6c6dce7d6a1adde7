"""``RDMAOneSidedEndpoint`` (the name-compatible stand-in for the reference's
``rdma_onesided_transport`` module): rendezvous and argument checks on the CPU, data movement
between two processes on one GPU and, where there are two, across GPUs."""
import os
import socket
import subprocess
import sys
import threading
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_rendezvous_and_refusals_without_a_gpu():
    from bikv_b200.rdma_onesided_transport import RDMAOneSidedEndpoint
    port = _free_port()
    server = RDMAOneSidedEndpoint("127.0.0.1", str(port), "server")
    client = RDMAOneSidedEndpoint("127.0.0.1", str(port), "client")
    assert client.connect_client(rank=2, cpu_size=0, gpu_size=0) == -1          # nobody listens yet
    rc = {}
    t = threading.Thread(target=lambda: rc.setdefault("server", server.run_server(1, 0, 0)))
    t.start()
    for _ in range(200):
        if client.connect_client(rank=2, cpu_size=0, gpu_size=0) == 0:
            break
        time.sleep(0.05)
    else:
        pytest.fail("client could not connect")
    t.join(30)
    assert rc["server"] == 0
    # only the server posts; unknown ranks and ranges outside a buffer are refused with -1
    assert client.post_rdma_write(2, 16, "cpu", "cpu") == -1
    assert server.post_rdma_write(9, 16, "cpu", "cpu") == -1
    assert server.post_rdma_write(2, 16, "cpu", "cpu") == -1                  # no buffers were allocated
    assert server.post_rdma_read(2, 16, "gpu", "cpu") == -1
    with pytest.raises(RuntimeError):
        server.get_server_cpu_tensor(2)
    with pytest.raises(RuntimeError):
        client.get_client_gpu_tensor()
    assert server.run_server.__code__.co_varnames[1:5] == ("max_clients", "local_cpu_size", "local_gpu_size", "hugepage")
    assert client.connect_client.__code__.co_varnames[1:5] == ("rank", "cpu_size", "gpu_size", "hugepage")
    assert server.post_rdma_write.__code__.co_varnames[1:7] == ("rank", "size", "src_type", "dst_type", "local_offset",
                                                                 "remote_offset")
    server.close()
    client.close()


CLIENT = """
import os, sys, time
sys.path.insert(0, {root!r})
import torch
from bikv_b200.rdma_onesided_transport import RDMAOneSidedEndpoint
torch.cuda.set_device({client_gpu})
ep = RDMAOneSidedEndpoint("127.0.0.1", "{port}", "client")
for _ in range(400):
    if ep.connect_client(rank=4, cpu_size=1 << 20, gpu_size=1 << 20) == 0:
        break
    time.sleep(0.05)
else:
    raise SystemExit("no server")
cpu, gpu = ep.get_client_cpu_tensor(), ep.get_client_gpu_tensor()
g = torch.Generator().manual_seed(3)
seed = torch.randint(0, 256, (1 << 20,), dtype=torch.uint8, generator=g)
cpu.copy_(seed)
gpu.copy_(seed.flip(0))
torch.cuda.synchronize()
open({ready!r}, "w").write("ready")
while not os.path.exists({done!r}):
    time.sleep(0.02)
# what the server wrote into this client's buffers (see the test body)
torch.cuda.synchronize()
want = torch.arange(1 << 20, dtype=torch.int64).mul(7).remainder(251).to(torch.uint8)
assert torch.equal(gpu[1000:1000 + 77777].cpu(), want[13:13 + 77777]), "write into the client's gpu buffer"
assert torch.equal(cpu[5:5 + 4099], want[100003:100003 + 4099]), "write into the client's cpu buffer"
assert torch.equal(gpu[:1000].cpu(), seed.flip(0)[:1000]) and torch.equal(cpu[:5], seed[:5]), "bytes outside the range"
ep.close()
print("CLIENT_OK")
"""


def _two_process_case(tmp_path, server_gpu, client_gpu):
    from bikv_b200.rdma_onesided_transport import RDMAOneSidedEndpoint
    port = _free_port()
    ready, done = str(tmp_path / "ready"), str(tmp_path / "done")
    child = subprocess.Popen([sys.executable, "-c", CLIENT.format(root=ROOT, port=port, ready=ready, done=done,
                                                                  client_gpu=client_gpu)],
                             stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        torch.cuda.set_device(server_gpu)
        server = RDMAOneSidedEndpoint("127.0.0.1", str(port), "server")
        assert server.run_server(max_clients=1, local_cpu_size=1 << 20, local_gpu_size=1 << 20) == 0
        t0 = time.time()
        while not os.path.exists(ready):
            assert child.poll() is None, child.communicate()[0][-3000:]
            assert time.time() - t0 < 180
            time.sleep(0.02)
        g = torch.Generator().manual_seed(3)
        seed = torch.randint(0, 256, (1 << 20,), dtype=torch.uint8, generator=g)
        for engine in (False, True):
            server.use_copy_engine = engine
            s_cpu, s_gpu = server.get_server_cpu_tensor(4), server.get_server_gpu_tensor(4)
            s_cpu.zero_()
            s_gpu.zero_()
            # READ: client buffers -> server buffers; odd sizes and offsets on purpose
            assert server.post_rdma_read(4, 12345, "cpu", "gpu", local_offset=7, remote_offset=3) == 0
            assert torch.equal(s_gpu[7:7 + 12345].cpu(), seed[3:3 + 12345])
            assert int(s_gpu[:7].sum()) == 0 and int(s_gpu[7 + 12345:].sum()) == 0
            assert server.post_rdma_read(4, 99999, "gpu", "cpu", local_offset=1, remote_offset=17) == 0
            assert torch.equal(s_cpu[1:1 + 99999], seed.flip(0)[17:17 + 99999])
            assert server.post_rdma_read(4, 65536, "gpu", "gpu", local_offset=65536, remote_offset=4096) == 0
            assert torch.equal(s_gpu[65536:2 * 65536].cpu(), seed.flip(0)[4096:4096 + 65536])
            # ranges that leave a buffer are refused, nothing is copied
            assert server.post_rdma_read(4, 2, "cpu", "cpu", local_offset=(1 << 20) - 1) == -1
            assert server.post_rdma_write(4, 1 << 21, "gpu", "gpu") == -1
            assert server.post_rdma_write(4, 16, "gpu", "disk") == -1
        # WRITE: server buffers -> client buffers
        want = torch.arange(1 << 20, dtype=torch.int64).mul(7).remainder(251).to(torch.uint8)
        server.use_copy_engine = False
        server.get_server_cpu_tensor(4).copy_(want)
        server.get_server_gpu_tensor(4).copy_(want)
        torch.cuda.synchronize()
        assert server.post_rdma_write(4, 77777, "cpu", "gpu", local_offset=13, remote_offset=1000) == 0
        server.use_copy_engine = True
        assert server.post_rdma_write(4, 4099, "gpu", "cpu", local_offset=100003, remote_offset=5) == 0
        open(done, "w").write("done")
        out, _ = child.communicate(timeout=120)
        assert child.returncode == 0 and "CLIENT_OK" in out, out[-3000:]
        server.close()
    finally:
        if child.poll() is None:
            child.kill()


@pytest.mark.gpu
def test_write_and_read_between_two_processes_on_one_gpu(cuda, tmp_path):
    _two_process_case(tmp_path, 0, 0)


@pytest.mark.gpu
def test_write_and_read_between_two_gpus(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _two_process_case(tmp_path, 0, 1)
