"""The rank rendezvous and descriptor exchange of the native transport, exercised on the CPU
with memfd files standing in for CUDA allocation handles (world sizes 2 and 4), plus the
host-side failure case: a rank that never joins makes the others return an error by a deadline
instead of blocking forever."""
import ctypes
import multiprocessing as mp
import os
import time
import uuid

import pytest

from mkernel_b200 import _lib


def _rank_main(rank, world, key, q, rounds):
    try:
        lib = _lib.lib()
        comm = ctypes.c_void_p()
        _lib.check(lib.mk_comm_create(key.encode(), rank, world, 0, ctypes.byref(comm)))
        assert lib.mk_comm_rank(comm) == rank and lib.mk_comm_world(comm) == world
        seen = []
        for rnd in range(rounds):
            # bytes all-gather
            mine = bytes([rank, rnd, 0xA5]) * 4
            out = ctypes.create_string_buffer(len(mine) * world)
            _lib.check(lib.mk_comm_allgather(comm, mine, len(mine), out))
            for r in range(world):
                assert out.raw[r * 12:(r + 1) * 12] == bytes([r, rnd, 0xA5]) * 4
            # descriptor all-gather: each rank shares a memfd holding its rank and round
            fd = os.memfd_create(f"mkb-test-{rank}")
            os.write(fd, f"rank{rank}-round{rnd}".encode())
            fds = (ctypes.c_int * world)()
            _lib.check(lib.mk_comm_allgather_fd(comm, fd, fds))
            os.close(fd)
            for r in range(world):
                # descriptors passed between processes share one file offset: read positionally
                seen.append(os.pread(fds[r], 64, 0).decode())
                os.close(fds[r])
            if rank == 0 and rnd == 0:
                time.sleep(0.3)          # a slow rank must not break the others' next round
            _lib.check(lib.mk_comm_barrier(comm))
        lib.mk_comm_destroy(comm)
        q.put((rank, "ok", seen))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put((rank, f"error: {e!r}", []))


@pytest.mark.parametrize("world", [2, 4])
def test_allgather_bytes_and_descriptors(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    key = uuid.uuid4().hex[:12]
    rounds = 3
    procs = [ctx.Process(target=_rank_main, args=(r, world, key, q, rounds)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(30)
    expected = [f"rank{r}-round{rnd}" for rnd in range(rounds) for r in range(world)]
    for rank, status, seen in got:
        assert status == "ok", (rank, status)
        assert seen == expected


def _lonely_rank(key, q):
    os.environ["MKB200_RENDEZVOUS_TIMEOUT_S"] = "1.5"
    lib = _lib.lib()
    comm = ctypes.c_void_p()
    _lib.check(lib.mk_comm_create(key.encode(), 0, 2, 0, ctypes.byref(comm)))
    t0 = time.time()
    rc = lib.mk_comm_barrier(comm)
    q.put((rc, _lib.last_error(), time.time() - t0))
    lib.mk_comm_destroy(comm)


def test_missing_rank_times_out_with_an_error():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_rank, args=(uuid.uuid4().hex[:12], q))
    p.start()
    rc, msg, dt = q.get(timeout=60)
    p.join(30)
    assert rc == -3                       # MK_ERR_TRANSPORT
    assert "timed out" in msg and "rank 1" in msg
    assert 1.0 < dt < 10.0


def test_world_of_one_needs_no_socket():
    lib = _lib.lib()
    comm = ctypes.c_void_p()
    _lib.check(lib.mk_comm_create(b"solo", 0, 1, 0, ctypes.byref(comm)))
    out = ctypes.create_string_buffer(4)
    _lib.check(lib.mk_comm_allgather(comm, b"abcd", 4, out))
    assert out.raw == b"abcd"
    _lib.check(lib.mk_comm_barrier(comm))
    lib.mk_comm_destroy(comm)


def test_two_ranks_cannot_claim_the_same_name():
    lib = _lib.lib()
    key = uuid.uuid4().hex[:12].encode()
    a, b = ctypes.c_void_p(), ctypes.c_void_p()
    _lib.check(lib.mk_comm_create(key, 0, 2, 0, ctypes.byref(a)))
    assert lib.mk_comm_create(key, 0, 2, 0, ctypes.byref(b)) == -3
    assert "bind" in _lib.last_error()
    lib.mk_comm_destroy(a)


def test_long_keys_keep_their_rank_suffix():
    """A rendezvous key longer than a socket name (a fully qualified host name plus a run id)
    must neither cut off the rank suffix nor collide with another long key sharing a prefix."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    prefix = "node-0123.some-cluster.example.internal:29500:" + "x" * 90
    jobs = []
    for tag in ("a", "b"):                      # two jobs whose keys differ only at the very end
        key = prefix + tag
        jobs += [ctx.Process(target=_rank_main, args=(r, 2, key, q, 1)) for r in range(2)]
    for p in jobs:
        p.start()
    got = [q.get(timeout=120) for _ in range(4)]
    for p in jobs:
        p.join(30)
    assert all(status == "ok" for _, status, _ in got), got
