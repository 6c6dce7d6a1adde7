"""The shared-memory control block of the ``ipc_service`` module, without a GPU: fields
survive a second mapping, the semaphore crosses processes, a wait without a post times out."""
import ctypes as C
import os
import subprocess
import sys
import time
import uuid

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_control_block_fields_and_cross_process_semaphore():
    from bikv_b200 import ipc_service as S
    name = "bikv_ctl_" + uuid.uuid4().hex[:12]
    path = S._shm_path("/" + name)
    a = S._Control(path, create=True)
    try:
        assert S._libc.sem_init(a.sem_start, 1, 0) == 0
        fields = [S._MAGIC, 3, 1, os.getpid(), 1 << 30, 10, 20, 30, 5, 7, 1, 2, 3, 4, 5, bytes(range(64)), 4096]
        a.write(fields)
        b = S._Control(path, create=False)
        assert b.read() == fields
        # a wait nothing posts to ends by itself
        deadline = time.time() + 0.2
        ts = S._Timespec(int(deadline), int((deadline % 1) * 1e9))
        assert S._libc.sem_timedwait(b.sem_start, C.byref(ts)) != 0 and C.get_errno() == 110
        # another process posts
        child = ("import sys; sys.path.insert(0, %r)\n"
                 "from bikv_b200 import ipc_service as S\n"
                 "c = S._Control(%r, create=False); f = c.read(); f[9] += 1; c.write(f); S._libc.sem_post(c.sem_start)\n"
                 % (ROOT, path))
        subprocess.run([sys.executable, "-c", child], check=True, timeout=120)
        deadline = time.time() + 5
        ts = S._Timespec(int(deadline), int((deadline % 1) * 1e9))
        assert S._libc.sem_timedwait(a.sem_start, C.byref(ts)) == 0
        assert a.read()[9] == 8
        b.close()
    finally:
        a.close()
        os.unlink(path)


def test_bad_names_and_missing_blocks_are_errors():
    import pytest
    from bikv_b200 import ipc_service as S
    with pytest.raises(RuntimeError):
        S._shm_path("a/b")
    with pytest.raises(RuntimeError):
        S._Control(S._shm_path("/bikv_no_such_block_" + uuid.uuid4().hex), create=False)
