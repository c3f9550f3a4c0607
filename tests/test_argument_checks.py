"""Arguments a caller can get wrong: every case ends in a status code on the rank that made the mistake (or on all of
them where all see the same wrong argument), never in a crash or a hang. Host team, CPU ranks. The reference asserts or
reads out of bounds in most of these places (src/team_lib/ucx/xccl_ucx_lib.c:143-160 switches without a default)."""
import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team, XcclError
from xccl_b200.utils.launch import run_ranks


def _rank(rank, size, job):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    out = {}

    # a reduction of zero elements completes and touches nothing
    src = np.zeros(0, np.int32)
    dst = np.full(4, 7, np.int32)
    team.allreduce(src, dst[:0]).run().finalize()
    assert np.all(dst == 7)
    out["zero_count"] = "ok"

    # a root outside the team
    buf = np.arange(16, dtype=np.float32)
    for root in (-1, size, size + 5):
        with pytest.raises(XcclError) as e:
            team.bcast(buf, root).run()
        assert e.value.status in (K.ERR_INVALID_PARAM, K.ERR_UNSUPPORTED), e.value.status
    out["bad_root"] = "ok"

    # a bitwise operation on floating-point data
    a = np.ones(8, np.float32)
    b = np.zeros(8, np.float32)
    with pytest.raises(XcclError) as e:
        team.allreduce(a, b, op=K.OP_BAND).run()
    assert e.value.status in (K.ERR_UNSUPPORTED, K.ERR_NOT_IMPLEMENTED, K.ERR_INVALID_PARAM), e.value.status
    out["float_band"] = "ok"

    # raw argument structures: a missing buffer, a missing count array, a datatype that does not exist
    import ctypes as C
    L = K.load()

    def init_raw(fill):
        a = K.CollArgs()
        fill(a)
        h = C.c_void_p()
        st = L.xccl_collective_init(C.byref(a), C.byref(h), team.h)
        if st == K.OK:
            L.xccl_collective_finalize(h)
        return st

    keep = np.zeros(64, np.int32)

    def no_dst(a):
        a.coll_type = K.ALLREDUCE
        a.buffer_info.src_buffer = keep.ctypes.data
        a.buffer_info.dst_buffer = None
        a.buffer_info.len = keep.nbytes
        a.reduce_info.dt, a.reduce_info.op, a.reduce_info.count = K.DT_INT32, K.OP_SUM, 64
    assert init_raw(no_dst) == K.ERR_INVALID_PARAM

    def no_counts(a):
        a.coll_type = K.ALLTOALLV
        a.buffer_info.src_buffer = keep.ctypes.data
        a.buffer_info.dst_buffer = keep.ctypes.data + 128
        a.buffer_info.src_datatype = a.buffer_info.dst_datatype = K.DT_INT32
    assert init_raw(no_counts) == K.ERR_INVALID_PARAM

    def bad_dt(a):
        a.coll_type = K.ALLREDUCE
        a.buffer_info.src_buffer = keep.ctypes.data
        a.buffer_info.dst_buffer = keep.ctypes.data
        a.buffer_info.len = 64
        a.reduce_info.dt, a.reduce_info.op, a.reduce_info.count = 77, K.OP_SUM, 16
    assert init_raw(bad_dt) in (K.ERR_INVALID_PARAM, K.ERR_UNSUPPORTED)

    def bad_coll(a):
        a.coll_type = 55
    assert init_raw(bad_coll) == K.ERR_INVALID_PARAM

    def ragged_allgather(a):     # the gathered length is no multiple of the team size
        a.coll_type = K.ALLGATHER
        a.buffer_info.src_buffer = keep.ctypes.data
        a.buffer_info.dst_buffer = keep.ctypes.data
        a.buffer_info.len = 4 * size + 1
    assert init_raw(ragged_allgather) == K.ERR_INVALID_PARAM
    out["raw"] = "ok"

    # the Python layer sees the arrays, not just their addresses: a strided view or a buffer that is too short is
    # refused before anything is sent
    big = np.arange(100, dtype=np.int32)
    small = np.zeros(50, np.int32)
    with pytest.raises(ValueError, match="not contiguous"):
        team.allreduce(big[::2], small)
    with pytest.raises(ValueError, match="dst holds 200 bytes"):
        team.allreduce(big, small)
    with pytest.raises(ValueError, match="src holds"):
        team.allgather(small[:3], np.zeros(4 * size, np.int32))
    with pytest.raises(ValueError, match="dst holds"):
        team.alltoallv(big, [10] * size, [10 * i for i in range(size)], small, [30] * size, [30 * i for i in range(size)])
    with pytest.raises(ValueError, match="one count"):
        team.alltoallv(big, [1], [0], small, [1], [0])
    out["python_checks"] = "ok"

    # the request life cycle: a second post while in flight is refused or ordered, finalize refuses a request in
    # flight, a completed request can be posted again
    x = np.arange(50000, dtype=np.int64) + rank
    y = np.zeros_like(x)
    req = team.allreduce(x, y)
    req.post()
    req.wait(timeout=60)
    want = sum(np.arange(50000, dtype=np.int64) + r for r in range(size))
    assert np.array_equal(y, want)
    y[:] = 0
    req.post().wait(timeout=60)
    assert np.array_equal(y, want)
    req.finalize()
    out["lifecycle"] = "ok"

    # the team still works after the refused calls
    team.barrier().run().finalize()
    z = np.full(3, rank + 1, np.int32)
    team.allreduce("in_place", z).run().finalize()
    assert np.all(z == size * (size + 1) // 2)
    team.close(); ctx.close(); lib.close(); oob.close()
    return out


def test_wrong_arguments_end_in_status_codes():
    res = run_ranks(_rank, 3, timeout=120)
    for r in res:
        assert r == {"zero_count": "ok", "bad_root": "ok", "float_band": "ok", "raw": "ok", "python_checks": "ok", "lifecycle": "ok"}
