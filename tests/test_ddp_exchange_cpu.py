"""The gradient exchange of the C ABI (fb_ddp_*) on CPU, with a stand-in for
libnccl behind it (tests/cpp/fake_nccl.c, loaded through FB_NCCL_LIBRARY):
the plumbing of pointers and counts, the one-rank world that never touches
NCCL, and every failure path - an NCCL call that returns an error, an
asynchronous error found by a poll, a communicator that is refused after it
has failed - without a GPU and without anything that could hang.

Each case runs in a child process: the library binds NCCL once per process,
so the environment variable has to be in place before the first fb_ddp call.
"""
import os
import subprocess
import sys
import textwrap

import pytest

from ferro_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE_SRC = os.path.join(ROOT, "tests", "cpp", "fake_nccl.c")


@pytest.fixture(scope="module")
def fake(tmp_path_factory):
    build.build()
    out = str(tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-fvisibility=hidden", "-O1", FAKE_SRC, "-o", out], check=True)
    return out


def run_child(fake, body, env_extra=None):
    prelude = f"""
        import ctypes as C, sys
        sys.path.insert(0, {ROOT!r})
        from ferro_b200 import _lib
        lib = _lib.load()
        fake = C.CDLL({fake!r})
        err = lambda: lib.fb_last_error().decode()
        def comm(rank=0, world=2):
            h = C.c_void_p()
            rc = lib.fb_ddp_comm_init(b"x" * 128, rank, world, C.byref(h))
            return rc, h
    """
    code = textwrap.dedent(prelude) + textwrap.dedent(body)
    env = dict(os.environ, FB_NCCL_LIBRARY=fake, **(env_extra or {}))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_allreduce_reaches_nccl_with_the_right_pointer_and_count(fake):
    out = run_child(fake, """
        rc, h = comm(1, 4)
        assert rc == 0, err()
        assert lib.fb_ddp_rank(h) == 1 and lib.fb_ddp_world(h) == 4
        assert lib.fb_ddp_nccl_version() == 99999
        buf = (C.c_float * 10)(*range(10))
        assert lib.fb_ddp_allreduce_bucket(h, None, buf, 10) == 0, err()
        assert list(buf) == [4.0 * i for i in range(10)]           # the stand-in sums `world` equal replicas
        a, b = (C.c_float * 3)(1, 2, 3), (C.c_float * 2)(5, 6)
        ptrs = (C.c_void_p * 3)(C.addressof(a), None, C.addressof(b))
        assert lib.fb_ddp_allreduce_buckets(h, None, ptrs, (C.c_uint64 * 3)(3, 0, 2), 3) == 0, err()
        assert list(a) == [4, 8, 12] and list(b) == [20, 24]
        assert fake.fake_nccl_count(0) == 3
        assert lib.fb_ddp_poll(h) == 0
        assert lib.fb_ddp_allreduce_bucket(h, None, None, 0) == 0   # empty bucket: nothing to do
        assert lib.fb_ddp_allreduce_bucket(h, None, None, 5) == 2   # null bucket
        assert lib.fb_ddp_comm_destroy(h) == 0 and fake.fake_nccl_count(2) == 1
        print("ok")
    """)
    assert "ok" in out


def test_a_world_of_one_never_loads_nccl():
    build.build()
    code = textwrap.dedent(f"""
        import ctypes as C, sys
        sys.path.insert(0, {ROOT!r})
        from ferro_b200 import _lib
        lib = _lib.load()
        h = C.c_void_p()
        assert lib.fb_ddp_comm_init(None, 0, 1, C.byref(h)) == 0
        buf = (C.c_float * 4)(1, 2, 3, 4)
        assert lib.fb_ddp_allreduce_bucket(h, None, buf, 4) == 0
        assert lib.fb_ddp_average_bucket(h, None, buf, 4) == 0
        assert list(buf) == [1, 2, 3, 4] and lib.fb_ddp_poll(h) == 0
        assert lib.fb_ddp_comm_destroy(h) == 0
        # bad ranks are refused before anything else happens
        assert lib.fb_ddp_comm_init(None, 2, 2, C.byref(h)) == 2 and not h.value
        assert lib.fb_ddp_comm_init(None, 0, 0, C.byref(h)) == 2
        print("ok")
    """)
    env = dict(os.environ, FB_NCCL_LIBRARY="/nonexistent/libnccl.so")  # would fail if it were loaded
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


def test_missing_nccl_is_an_error_status_not_a_crash():
    build.build()
    code = textwrap.dedent(f"""
        import ctypes as C, sys
        sys.path.insert(0, {ROOT!r})
        from ferro_b200 import _lib
        lib = _lib.load()
        h = C.c_void_p()
        assert lib.fb_ddp_comm_init(b"x" * 128, 0, 2, C.byref(h)) == 6
        assert b"cannot load" in lib.fb_last_error() and not h.value
        assert lib.fb_ddp_unique_id(C.create_string_buffer(128)) == 6
        assert lib.fb_ddp_nccl_version() == -1
        print("ok")
    """)
    env = dict(os.environ, FB_NCCL_LIBRARY="/nonexistent/libnccl.so")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


def test_a_failing_collective_returns_a_status_and_breaks_the_handle(fake):
    out = run_child(fake, """
        rc, h = comm()
        assert rc == 0, err()
        buf = (C.c_float * 4)(1, 2, 3, 4)
        fake.fake_nccl_fail(2, 6)                                   # ncclAllReduce -> ncclRemoteError
        assert lib.fb_ddp_allreduce_bucket(h, None, buf, 4) == 6
        assert "remote process exited" in err() and "ncclAllReduce" in err()
        assert list(buf) == [1, 2, 3, 4]                            # nothing was modified
        fake.fake_nccl_fail(0, 0)                                   # NCCL is fine again, the handle is not
        assert lib.fb_ddp_allreduce_bucket(h, None, buf, 4) == 6 and "failed before" in err()
        assert lib.fb_ddp_poll(h) == 6
        assert list(buf) == [1, 2, 3, 4] and fake.fake_nccl_count(0) == 0
        # tearing a failed communicator down aborts it instead of flushing it
        assert lib.fb_ddp_comm_destroy(h) == 0
        assert fake.fake_nccl_count(1) == 1 and fake.fake_nccl_count(2) == 0
        print("ok")
    """)
    assert "ok" in out


def test_poll_finds_an_asynchronous_error_between_steps(fake):
    out = run_child(fake, """
        rc, h = comm()
        assert rc == 0 and lib.fb_ddp_poll(h) == 0
        fake.fake_nccl_fail(3, 7)                                   # ncclInProgress: not a failure
        assert lib.fb_ddp_poll(h) == 0
        fake.fake_nccl_fail(3, 6)                                   # a peer died: asynchronous ncclRemoteError
        assert lib.fb_ddp_poll(h) == 6 and "asynchronous" in err()
        fake.fake_nccl_fail(0, 0)
        buf = (C.c_float * 2)(1, 2)
        assert lib.fb_ddp_allreduce_bucket(h, None, buf, 2) == 6    # refused before anything is enqueued
        assert fake.fake_nccl_count(0) == 0
        assert lib.fb_ddp_comm_abort(h) == 0 and fake.fake_nccl_count(1) == 1
        print("ok")
    """)
    assert "ok" in out


def test_init_and_group_failures(fake):
    out = run_child(fake, """
        fake.fake_nccl_fail(1, 2)                                   # ncclCommInitRank -> system error
        rc, h = comm()
        assert rc == 6 and not h.value and "ncclCommInitRank" in err()
        fake.fake_nccl_fail(5, 3)
        assert lib.fb_ddp_unique_id(C.create_string_buffer(128)) == 6
        fake.fake_nccl_fail(0, 0)
        idb = C.create_string_buffer(128)
        assert lib.fb_ddp_unique_id(idb) == 0 and idb.raw == bytes([0x5a]) * 128
        rc, h = comm()
        assert rc == 0
        a = (C.c_float * 2)(1, 2)
        fake.fake_nccl_fail(4, 3)                                   # ncclGroupEnd fails
        assert lib.fb_ddp_allreduce_buckets(h, None, (C.c_void_p * 1)(C.addressof(a)), (C.c_uint64 * 1)(2), 1) == 6
        assert "ncclGroupEnd" in err()
        assert lib.fb_ddp_poll(h) == 6
        print("ok")
    """)
    assert "ok" in out


def test_python_wrapper_raises_comm_error(fake):
    out = run_child(fake, """
        from ferro_b200 import ddp
        from ferro_b200.backend import CommError
        c = ddp.NcclComm(0, 2, share_id=lambda raw: raw)
        buf = (C.c_float * 4)(1, 2, 3, 4)
        c.allreduce_sum(C.addressof(buf), 4, 0)
        assert list(buf) == [2, 4, 6, 8]
        c.poll()
        fake.fake_nccl_fail(3, 6)
        try:
            c.poll()
            raise SystemExit("poll did not raise")
        except CommError as e:
            assert "remote process exited" in str(e)
        try:
            c.allreduce_sum(C.addressof(buf), 4, 0)
            raise SystemExit("exchange on a broken communicator did not raise")
        except CommError:
            pass
        c.abort()
        print("ok")
    """)
    assert "ok" in out
