"""Failure detection on the host: every blocking step has a deadline and reports an error code
instead of spinning (the reference spins forever in all of these places: OOB allgather in
src/core/xccl_team_lib.h:114, collective wait in src/team_lib/ucx/xccl_ucx_lib.c:569-571).

Failures are made on the host among CPU ranks: a rank that never joins, a rank that never posts,
a rank that leaves between two collectives. No GPU is involved.
"""
import time

import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team, XcclError
from xccl_b200.utils.launch import run_ranks


def _never_joins(rank, size, job):
    """Rank 1 creates the OOB but never builds a context: rank 0's bootstrap must time out."""
    oob = ShmOob(job, rank, size)
    if rank == 1:
        time.sleep(3.0)
        oob.close()
        return "absent"
    lib = Lib()
    t0 = time.monotonic()
    try:
        ctx = Context(lib, oob, tls=K.TL_UCX)
        Team(ctx, timeout=5.0)
        return "joined"
    except XcclError as e:
        dt = time.monotonic() - t0
        assert e.status == K.ERR_TIMED_OUT, e.status
        assert dt < 2.9, dt
        return "timed out"
    finally:
        lib.close()
        oob.close()


def test_bootstrap_times_out_when_a_rank_never_joins():
    res = run_ranks(_never_joins, 2, timeout=60, env={"XCCL_OOB_TIMEOUT": "1"})
    assert res == ["timed out", "absent"]


def _never_posts(rank, size, job):
    """Every rank builds the team; rank 1 never posts the allreduce. The others' wait ends with
    XCCL_ERR_TIMED_OUT after XCCL_WAIT_TIMEOUT seconds and the library stays usable for queries."""
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    src = np.full(1000, float(rank + 1), dtype=np.float32)
    dst = np.zeros_like(src)
    out = "idle"
    if rank != 1:
        req = team.allreduce(src, dst)
        req.post()
        t0 = time.monotonic()
        try:
            req.wait()
            out = "completed"
        except XcclError as e:
            assert e.status == K.ERR_TIMED_OUT, e.status
            assert 0.9 < time.monotonic() - t0 < 10.0
            out = "timed out"
        assert team.size == size          # queries still answer after the failure
    else:
        time.sleep(2.5)                   # between steps, nothing of this rank in flight
    return out


def test_collective_wait_times_out_when_a_rank_never_posts():
    res = run_ranks(_never_posts, 3, timeout=60, env={"XCCL_WAIT_TIMEOUT": "1"})
    assert res == ["timed out", "idle", "timed out"]


def _leaves_between_steps(rank, size, job):
    """Two allreduces; rank 2 leaves after the first. The survivors complete step one exactly and
    get an error code (not a hang) from step two."""
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    src = np.arange(4096, dtype=np.int32) + rank
    dst = np.zeros_like(src)
    team.allreduce(src, dst).run().finalize()
    want = sum(np.arange(4096, dtype=np.int64) + r for r in range(size)).astype(np.int32)
    assert np.array_equal(dst, want)
    if rank == 2:
        return "left"
    req = team.allreduce(src, dst)
    req.post()
    try:
        req.wait()
        return "completed"
    except XcclError as e:
        assert e.status == K.ERR_TIMED_OUT
        return "detected"


def test_rank_leaving_between_collectives_is_detected():
    res = run_ranks(_leaves_between_steps, 3, timeout=60, env={"XCCL_WAIT_TIMEOUT": "1"})
    assert res == ["detected", "detected", "left"]


def _shrinks_after_a_failure(rank, size, job):
    """Four ranks; rank 2 leaves after the first allreduce. The others get the deadline error from the next one, drop
    the poisoned team and carry on with a new team over the survivors on the SAME context (an endpoint map): no
    rendezvous with the lost rank is needed, because team creation gathers over the members of the new team only."""
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    src = np.arange(1000, dtype=np.int32) + rank
    dst = np.zeros_like(src)
    team.allreduce(src, dst).run().finalize()
    if rank == 2:
        return "left"
    req = team.allreduce(src, dst)
    req.post()
    try:
        req.wait()
        return "completed"
    except XcclError as e:
        assert e.status == K.ERR_TIMED_OUT
    # every later collective of the poisoned team fails at once instead of waiting again
    t0 = time.monotonic()
    with pytest.raises(XcclError):
        team.allreduce(src, dst).run()
    assert time.monotonic() - t0 < 0.5
    survivors = [0, 1, 3]          # known to the survivors from outside (a store, a heartbeat)
    small = Team(ctx, ranks=survivors, timeout=20.0)
    assert small.size == 3 and small.rank == survivors.index(rank)
    for it in range(3):
        dst[:] = 0
        small.allreduce(src + it, dst).run().finalize()
        want = sum(np.arange(1000, dtype=np.int64) + r + it for r in survivors).astype(np.int32)
        assert np.array_equal(dst, want)
    small.barrier().run().finalize()
    small.close()
    return "recovered"


def test_survivors_continue_on_a_smaller_team_of_the_same_context():
    res = run_ranks(_shrinks_after_a_failure, 4, timeout=90, env={"XCCL_WAIT_TIMEOUT": "1"})
    assert res == ["recovered", "recovered", "left", "recovered"]
