"""Failure handling of the communicator behind the C ABI (mcb_comm_*), exercised on the CPU against a stand-in NCCL
(tests/support/fake_nccl.c) that fails on demand: a rendezvous that never completes (a rank that never joins), a
peer that dies (asynchronous NCCL error), a collective that never finishes, an enqueue that fails.  In every case
the call must return within its host deadline with the documented status, the communicator must have been aborted,
and later calls must be refused instead of hanging.  No GPU is involved: nothing here can fault or hang one.

Each case runs in a child process because the library binds its NCCL once per process.
"""
import os
import subprocess
import sys
import textwrap
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), str(ROOT / "tests" / "support" / "fake_nccl.c")],
                   check=True)
    return out


def run_case(fake, mode, body, tmp_path):
    log = tmp_path / f"{mode}.log"
    env = dict(os.environ, MCB_NCCL_LIBRARY=str(fake), FAKE_NCCL_MODE=mode, FAKE_NCCL_LOG=str(log), PYTHONPATH=str(ROOT))
    script = "import time\nfrom metal_candle_b200 import _lib, comm\n" + textwrap.dedent(body)
    t0 = time.perf_counter()
    r = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
    return (log.read_text().split("\n") if log.exists() else []), time.perf_counter() - t0


def test_healthy_path_and_nonblocking_init(fake_nccl, tmp_path):
    log, _ = run_case(fake_nccl, "ok", """
        uid = comm.unique_id()
        assert len(uid) == 128
        c = comm.Communicator(2, 1, uid, timeout_ms=500)
        assert c.info() == {"nranks": 2, "rank": 1, "dead": False, "nccl_version": 22703}
        c.allreduce_bucket(0x1000, 16, 0)
        c.wait()
        c.destroy()
    """, tmp_path)
    assert "init nonblocking" in log and "allreduce" in log and "finalize" in log and "destroy" in log and "abort" not in log


def test_rendezvous_that_completes_late(fake_nccl, tmp_path):
    log, _ = run_case(fake_nccl, "slow_init", """
        c = comm.Communicator(2, 0, comm.unique_id(), timeout_ms=2000)
        assert not c.info()["dead"]
        c.destroy()
    """, tmp_path)
    assert "abort" not in log


def test_rank_that_never_joins_times_out_and_aborts(fake_nccl, tmp_path):
    log, dt = run_case(fake_nccl, "stuck_init", """
        t0 = time.perf_counter()
        try:
            comm.Communicator(2, 0, comm.unique_id(), timeout_ms=300)
            raise SystemExit("the rendezvous should have timed out")
        except comm.CommError as e:
            assert e.code == _lib.MCB_ERR_COMM_TIMEOUT, e
            assert "did not complete within 300 ms" in str(e) and "aborted" in str(e)
        assert 0.25 < time.perf_counter() - t0 < 5.0
    """, tmp_path)
    assert "abort" in log and "destroy" not in log


def test_peer_death_is_reported_and_the_communicator_goes_dead(fake_nccl, tmp_path):
    log, _ = run_case(fake_nccl, "async_error", """
        c = comm.Communicator(4, 2, comm.unique_id(), timeout_ms=500)
        try:
            c.allreduce_bucket(0x1000, 16, 0)
            raise SystemExit("the asynchronous error should have surfaced")
        except comm.CommError as e:
            assert e.code == _lib.MCB_ERR_COMM_BASE + 6, e     # ncclRemoteError
        assert c.info()["dead"]
        for call in (lambda: c.allreduce_bucket(0x1000, 16, 0), lambda: c.wait()):
            try:
                call()
                raise SystemExit("a dead communicator must refuse work")
            except comm.CommError as e:
                assert e.code == _lib.MCB_ERR_COMM_DEAD
        c.destroy()      # frees without touching NCCL again
    """, tmp_path)
    assert log.count("abort") == 1 and "destroy" not in log and "finalize" not in log


def test_collective_that_never_finishes(fake_nccl, tmp_path):
    log, _ = run_case(fake_nccl, "stuck_wait", """
        c = comm.Communicator(2, 0, comm.unique_id(), timeout_ms=250)
        t0 = time.perf_counter()
        try:
            c.allreduce_bucket(0x1000, 16, 0)       # the enqueue itself never settles
            raise SystemExit("should have timed out")
        except comm.CommError as e:
            assert e.code == _lib.MCB_ERR_COMM_TIMEOUT
        assert time.perf_counter() - t0 < 5.0 and c.info()["dead"]
    """, tmp_path)
    assert "abort" in log


def test_enqueue_error_and_explicit_abort(fake_nccl, tmp_path):
    log, _ = run_case(fake_nccl, "enqueue_error", """
        c = comm.Communicator(2, 0, comm.unique_id(), timeout_ms=250)
        try:
            c.allreduce_bucket(0x1000, 16, 0)
            raise SystemExit("should have failed")
        except comm.CommError as e:
            assert e.code == _lib.MCB_ERR_COMM_BASE + 4
        c2 = comm.Communicator(2, 1, comm.unique_id(), timeout_ms=250)
        c2.abort()
        assert c2.info()["dead"]
    """, tmp_path)
    assert log.count("abort") == 2


def test_argument_checks(fake_nccl, tmp_path):
    run_case(fake_nccl, "ok", """
        lib = _lib.load()
        import ctypes as C
        h = C.c_void_p(None)
        assert lib.mcb_comm_init_rank(C.byref(h), 2, 2, b"x" * 128, 100, 0) == -2      # rank out of range
        assert lib.mcb_comm_init_rank(C.byref(h), 0, 0, b"x" * 128, 100, 0) == -2
        assert lib.mcb_comm_unique_id(None) == -1
        assert lib.mcb_comm_allreduce_bucket(None, None, 4, None) == -1
        c = comm.Communicator(1, 0, comm.unique_id(), timeout_ms=100)
        assert lib.mcb_comm_allreduce_bucket(c._h, 0x1000, 0, None) == -2
    """, tmp_path)


def test_missing_library_is_an_error_not_a_fallback(tmp_path):
    env = dict(os.environ, MCB_NCCL_LIBRARY=str(tmp_path / "nope.so"), PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-c", "from metal_candle_b200 import _lib, comm\n"
                        "try:\n    comm.unique_id()\n    raise SystemExit(1)\n"
                        "except comm.CommError as e:\n    assert e.code == _lib.MCB_ERR_COMM_UNAVAILABLE\n"],
                       env=env, capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
