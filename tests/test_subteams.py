"""Sub-teams: endpoint ranges (strided, map) over the context's OOB, and non-blocking creation of a split
team interleaved with traffic on another team (the reference's test/test_mpi_create_team_nb.c:16-36 splits
the world by rank parity and creates the halves while point-to-point traffic is in flight)."""
import ctypes as C

import numpy as np

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team, _check
from xccl_b200.utils.launch import run_ranks


def _rank_main(rank, size, job):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    world = Team(ctx)
    L = K.load()
    # post the creation of my parity half without waiting for it ...
    members = [r for r in range(size) if r % 2 == rank % 2]
    arr = (C.c_int * len(members))(*members)
    p = K.TeamParams()
    p.field_mask = K.TEAM_PARAM_EP_RANGE
    p.range.type = K.EP_RANGE_MAP
    p.range.ep_num = len(members)
    p.range.map.map = C.cast(arr, C.POINTER(C.c_int))
    half = C.c_void_p()
    _check(L.xccl_team_create_post(ctx.h, C.byref(p), C.byref(half)), "xccl_team_create_post")
    # ... run a collective on the world team in between (odd and even ranks in different orders, as the
    # reference test does with its sendrecv) ...
    src = np.full(257, rank + 1, dtype=np.int64)
    dst = np.zeros_like(src)
    world.allreduce(src, dst).run().finalize()
    assert np.all(dst == size * (size + 1) // 2)
    # ... then finish the creation
    while True:
        st = L.xccl_team_create_test(half)
        if st == K.OK:
            break
        assert st == K.INPROGRESS, st
        ctx.progress()
    r, s = C.c_int(), C.c_int()
    _check(L.xccl_team_query(half, C.byref(r), C.byref(s)), "xccl_team_query")
    assert (r.value, s.value) == (members.index(rank), len(members))
    # a strided team over the same members through the Python wrapper, used for an allreduce
    args = K.CollArgs()
    args.coll_type = K.ALLREDUCE
    src = np.full(100, float(rank), dtype=np.float32)
    dst = np.zeros_like(src)
    args.buffer_info.src_buffer = src.ctypes.data
    args.buffer_info.dst_buffer = dst.ctypes.data
    args.buffer_info.len = src.nbytes
    args.reduce_info.dt, args.reduce_info.op, args.reduce_info.count = K.DT_FLOAT32, K.OP_SUM, 100
    req = C.c_void_p()
    _check(L.xccl_collective_init(C.byref(args), C.byref(req), half), "xccl_collective_init")
    _check(L.xccl_collective_post(req), "xccl_collective_post")
    _check(L.xccl_collective_wait(req), "xccl_collective_wait")
    _check(L.xccl_collective_finalize(req), "xccl_collective_finalize")
    assert np.all(dst == float(sum(members)))
    L.xccl_team_destroy(half)
    return len(members)


def test_split_team_created_without_blocking_while_the_world_team_works():
    res = run_ranks(_rank_main, 5, timeout=120)
    assert res == [3, 2, 3, 2, 3]


def _small_teams(rank, size, job):
    """Teams of one rank and of every second rank on a context whose first team library is the hierarchy layer: what
    that layer cannot schedule (nothing to exchange) falls through to the host team, the rest runs on the sub-group."""
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX | K.TL_HIER, config={K.TL_HIER: {"ENABLE_NVLINK": "no"}})
    solo = Team(ctx, ranks=[rank])
    assert (solo.rank, solo.size) == (0, 1)
    x = np.arange(10, dtype=np.int32) + rank
    y = np.zeros_like(x)
    solo.allreduce(x, y).run().finalize()
    assert np.array_equal(x, y)
    y[:] = 0
    solo.alltoall(x, y).run().finalize()
    assert np.array_equal(x, y)
    solo.bcast(x, 0).run().finalize()
    solo.barrier().run().finalize()
    solo.close()
    if rank % 2 == 1:
        members = [r for r in range(size) if r % 2 == 1]
        odd = Team(ctx, ranks=members)
        v = np.full(5, rank, np.int32)
        w = np.zeros_like(v)
        odd.allreduce(v, w).run().finalize()
        assert np.all(w == sum(members))
        odd.close()
    ctx.close(); lib.close(); oob.close()
    return True


def test_teams_of_one_and_of_every_second_rank():
    run_ranks(_small_teams, 5, timeout=120)
