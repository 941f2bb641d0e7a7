"""Failure handling of the collective layer on machines without a GPU: NCCL is replaced by a stand-in whose calls
fail on demand (tests/fake_nccl.c, loaded through FB_NCCL_LIB), so every error path of fb_comm_* runs for real
through the C ABI: a failing call, an asynchronous error found by polling, an aborted communicator, a missing
library; and two gloo ranks exchange the NCCL id through a process group.  Nothing here touches a GPU."""
import os
import subprocess
import sys
import textwrap

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("fake_nccl") / "libfakenccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", out, os.path.join(HERE, "fake_nccl.c")], check=True)
    return out


def _run(code, lib, **env):
    e = dict(os.environ, FB_NCCL_LIB=lib, PYTHONPATH=ROOT)
    e.update(env)
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=e, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


PRELUDE = """
import ctypes
from faith_b200 import _lib
lib = _lib.load()
def mk(world=2, rank=0):
    idb = ctypes.create_string_buffer(128)
    assert lib.fb_comm_unique_id(idb) == 0
    h = ctypes.c_void_p()
    return lib.fb_comm_create(ctypes.byref(h), idb, rank, world, 0), h
"""


def test_healthy_communicator(fake_lib):
    out = _run(PRELUDE + """
rc, h = mk()
assert rc == 0
r, w, o = ctypes.c_int(), ctypes.c_int(), ctypes.c_int64()
assert lib.fb_comm_info(h, ctypes.byref(r), ctypes.byref(w), ctypes.byref(o)) == 0 and (r.value, w.value, o.value) == (0, 2, 0)
assert lib.fb_allreduce_f32(h, 4096, 16, 0, 0, None) == 0       # the stand-in never touches the buffer
assert lib.fb_allreduce_f32(h, 4096, 16, 0, 1, None) == 5       # one-shot path was not set up: FB_ERR_WORKSPACE
assert lib.fb_allreduce_f32(h, 4096, 16, 3, 0, None) == 1       # unknown reduction: FB_ERR_ARG
assert lib.fb_comm_check(h, 0) == 0
assert lib.fb_comm_destroy(h) == 0
print("ok")
""", fake_lib)
    assert "ok" in out


@pytest.mark.parametrize("what,call", [("init", "ncclCommInitRank"), ("allreduce", "ncclAllReduce")])
def test_failing_call_becomes_fb_err_nccl(fake_lib, what, call):
    out = _run(PRELUDE + """
rc, h = mk()
if rc == 0:
    rc = lib.fb_allreduce_f32(h, 4096, 16, 0, 0, None)
assert rc == 7, rc
print(lib.fb_comm_last_error().decode())
print(lib.fb_status_string(rc).decode())
""", fake_lib, FAKE_NCCL_FAIL=what)
    assert call in out and "unhandled system error" in out and "collective" in out


def test_asynchronous_error_is_found_by_polling(fake_lib):
    out = _run(PRELUDE + """
rc, h = mk()
assert rc == 0
assert lib.fb_allreduce_f32(h, 4096, 16, 0, 0, None) == 0       # first poll: healthy
assert lib.fb_allreduce_f32(h, 4096, 16, 1, 0, None) == 7       # second poll: a peer is gone
print(lib.fb_comm_last_error().decode())
assert lib.fb_comm_check(h, 0) == 7
assert lib.fb_comm_abort(h) == 0
assert lib.fb_allreduce_f32(h, 4096, 16, 0, 0, None) == 7       # an aborted communicator refuses work
print(lib.fb_comm_last_error().decode())
assert lib.fb_comm_destroy(h) == 0
""", fake_lib, FAKE_NCCL_ASYNC_AFTER="2")
    assert "asynchronous NCCL error" in out and "remote process exited" in out and "aborted" in out


def test_missing_library_is_reported(fake_lib):
    out = _run("""
import ctypes
from faith_b200 import _lib
lib = _lib.load()
rc = lib.fb_comm_unique_id(ctypes.create_string_buffer(128))
assert rc == 7, rc
print(lib.fb_comm_last_error().decode())
""", "/nonexistent/libnccl.so.2")
    assert "could not be loaded" in out


def test_bad_arguments(fake_lib):
    _run(PRELUDE + """
idb = ctypes.create_string_buffer(128)
h = ctypes.c_void_p()
assert lib.fb_comm_create(ctypes.byref(h), idb, 2, 2, 0) == 1      # rank outside the world
assert lib.fb_comm_create(ctypes.byref(h), idb, 0, 9, 0) == 1      # more than eight ranks
assert lib.fb_comm_create(ctypes.byref(h), idb, 0, 2, 0) == 7      # an id that did not come from fb_comm_unique_id
assert lib.fb_relax_sharded_f32(None, 0, 0, *([4096] * 9), 1, 4, 8, 2, 3, 0.1, None, None) == 2   # two word blocks
""", fake_lib)


def test_two_ranks_exchange_the_id_over_a_process_group(fake_lib, tmp_path):
    code = """
import os, sys, torch.distributed as dist
rank = int(sys.argv[1])
os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = sys.argv[2]
dist.init_process_group("gloo", rank=rank, world_size=2)
from faith_b200.comm import Comm
c = Comm.from_process_group()          # rank 0 makes the id, rank 1 must receive exactly those bytes
assert (c.rank, c.world) == (rank, 2)
c.check()
c.destroy()
dist.destroy_process_group()
print("rank", rank, "ok")
"""
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent(code))
    e = dict(os.environ, FB_NCCL_LIB=fake_lib, PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "29641"], env=e, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    for r, p in enumerate(procs):
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0 and "rank %d ok" % r in out, out
