"""Hierarchy layer: sub-group rules as a pure function, and schedules run by real processes.

One host stands in for several nodes / sockets through XCCL_HIER_FAKE_NODE_ID and
XCCL_FAKE_SOCKET_ID (set per rank before the library reads them). The reference's CI can only
exercise the single-node, unbound layout (.github/workflows/main.yml:43-60); these tests also
cover multi-node and socket levels and non-default node leaders.
"""
import ctypes as C
import os

import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks

NODE, SOCKET, NODE_LEADERS, SOCKET_LEADERS, FLAT = range(5)
NOT_EXISTS, DISABLED, ENABLED = range(3)


def _layout(node, sock, me, leader_id=0):
    L = K.load()
    L.xccl_hier_layout_probe.restype = C.c_int
    n = len(node)
    st, gr, gs = (C.c_int * 5)(), (C.c_int * 5)(), (C.c_int * 5)()
    mem = (C.c_int * (5 * n))()
    nn = L.xccl_hier_layout_probe(n, (C.c_uint64 * n)(*node), (C.c_int * n)(*sock), me, leader_id, st, gr, gs, mem)
    groups = [[mem[s * n + k] for k in range(gs[s])] for s in range(5)]
    return nn, list(st), list(gr), groups


def test_layout_two_nodes_two_sockets():
    node = [1, 1, 1, 1, 2, 2, 2, 2]
    sock = [0, 0, 1, 1, 0, 0, 1, 1]
    nn, st, gr, g = _layout(node, sock, me=3)
    assert nn == 2
    assert g[NODE] == [0, 1, 2, 3] and st[NODE] == ENABLED and gr[NODE] == 3
    assert g[SOCKET] == [2, 3] and gr[SOCKET] == 1
    assert g[NODE_LEADERS] == [0, 4] and st[NODE_LEADERS] == DISABLED
    assert g[SOCKET_LEADERS] == [0, 2] and st[SOCKET_LEADERS] == DISABLED
    assert g[FLAT] == list(range(8))
    nn, st, gr, g = _layout(node, sock, me=4)
    assert st[NODE_LEADERS] == ENABLED and gr[NODE_LEADERS] == 1
    assert g[SOCKET_LEADERS] == [4, 6] and st[SOCKET_LEADERS] == ENABLED and gr[SOCKET_LEADERS] == 0


def test_layout_node_leader_rotation_and_socket_swap():
    node = [7] * 6
    sock = [0, 0, 0, 1, 1, 1]
    # leader is local index 4 (socket 1): the node group is rotated, the leader heads its socket group
    nn, st, gr, g = _layout(node, sock, me=5, leader_id=4)
    assert nn == 1 and st[NODE_LEADERS] == NOT_EXISTS
    assert g[NODE] == [4, 5, 0, 1, 2, 3]
    assert g[SOCKET] == [4, 5, 3]
    assert g[SOCKET_LEADERS] == [4, 0]
    # unbound ranks switch the socket levels off for everybody
    nn, st, gr, g = _layout(node, [0, 0, -1, 1, 1, 1], me=0)
    assert st[SOCKET] == NOT_EXISTS and st[SOCKET_LEADERS] == NOT_EXISTS and st[NODE] == ENABLED


def _data(rank, count, dtype, seed=0):
    rng = np.random.default_rng(seed * 1000 + rank)
    return rng.integers(-8, 9, size=count).astype(dtype)


def _hier_rank(rank, size, job, node_of, sock_of, leader_id):
    os.environ["XCCL_HIER_FAKE_NODE_ID"] = str(node_of[rank])
    os.environ["XCCL_FAKE_SOCKET_ID"] = str(sock_of[rank])
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_HIER | K.TL_UCX,
                  config={K.TL_HIER: {"NODE_LEADER_RANK_ID": str(leader_id), "ENABLE_NVLINK": "no"}})
    team = Team(ctx)
    for coll in (K.ALLREDUCE, K.BCAST, K.BARRIER, K.ALLTOALL):
        assert team.coll_tl(coll, K.MEM_HOST) == K.TL_HIER
    assert team.coll_tl(K.ALLGATHER, K.MEM_HOST) == K.TL_UCX  # hier does not offer it: next in priority
    for count in (1, 33, 5000):
        src = _data(rank, count, np.int32)
        dst = np.zeros_like(src)
        req = team.allreduce(src, dst)
        for _ in range(2):  # persistent: the schedule is re-armed
            dst[:] = 0
            req.post().wait(timeout=60)
            want = np.sum(np.stack([_data(r, count, np.int32) for r in range(size)]), axis=0)
            np.testing.assert_array_equal(dst, want)
        req.finalize()
        buf = _data(rank, count, np.float32, seed=1)
        team.allreduce("in_place", buf, op=K.OP_MAX).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(buf, np.max(np.stack([_data(r, count, np.float32, seed=1) for r in range(size)]), axis=0))
    for root in range(size):
        buf = _data(root, 777, np.float32, seed=2) if rank == root else np.zeros(777, np.float32)
        team.bcast(buf, root).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(buf, _data(root, 777, np.float32, seed=2))
    for _ in range(3):
        team.barrier().post().wait(timeout=60).finalize()
    per = 129
    src = np.arange(per * size, dtype=np.int32) + rank * 100000
    dst = np.zeros_like(src)
    team.alltoall(src, dst).post().wait(timeout=60).finalize()
    want = np.concatenate([(np.arange(per * size, dtype=np.int32) + r * 100000)[rank * per:(rank + 1) * per]
                           for r in range(size)])
    np.testing.assert_array_equal(dst, want)
    team.close()
    ctx.close()
    lib.close()
    oob.close()
    return True


LAYOUTS = {
    "one_node_unbound": ([0] * 4, [-1] * 4, 0),
    "one_node_leader3": ([0] * 5, [-1] * 5, 3),
    "two_nodes_unbound": ([0, 0, 0, 1, 1, 1], [-1] * 6, 0),
    "two_nodes_two_sockets": ([0, 0, 0, 0, 1, 1, 1, 1], [0, 0, 1, 1, 0, 0, 1, 1], 0),
    "uneven_nodes_leader1": ([0, 0, 0, 1, 1, 2], [0, 1, 1, 0, 0, 0], 1),
    "one_rank_per_node": ([0, 1, 2], [0, 0, 0], 0),
}


@pytest.mark.parametrize("name", sorted(LAYOUTS))
def test_hier_collectives(name):
    node_of, sock_of, leader = LAYOUTS[name]
    run_ranks(_hier_rank, len(node_of), node_of, sock_of, leader, timeout=180)


def _pipelined_bcast_rank(rank, size, job):
    os.environ["XCCL_HIER_FAKE_NODE_ID"] = str(rank // 2)
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_HIER | K.TL_UCX,
                  config={K.TL_HIER: {"BCAST_PIPELINE_THRESH": "4k", "BCAST_PIPELINE_DEPTH": "2", "ENABLE_NVLINK": "no"}})
    team = Team(ctx)
    n = 50001  # 200 KB in fragments of 4 KB, two in flight
    for root in (0, 3):
        buf = _data(root, n, np.float32, seed=4) if rank == root else np.zeros(n, np.float32)
        team.bcast(buf, root).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(buf, _data(root, n, np.float32, seed=4))
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


def test_hier_bcast_fragmented_pipeline():
    run_ranks(_pipelined_bcast_rank, 4, timeout=120)


def _sm_get_bcast_rank(rank, size, job, node_of, sock_of, check_window):
    import glob
    os.environ["XCCL_HIER_FAKE_NODE_ID"] = str(node_of[rank])
    os.environ["XCCL_FAKE_SOCKET_ID"] = str(sock_of[rank])
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_HIER | K.TL_UCX,
                  config={K.TL_HIER: {"ENABLE_SHMSEG": "y", "BCAST_SM_GET": "1", "BCAST_SM_GET_THRESH": "1k",
                                      "BCAST_PIPELINE_THRESH": "16k", "BCAST_PIPELINE_DEPTH": "3",
                                      "ENABLE_NVLINK": "no"}})
    team = Team(ctx)
    mine = "/dev/shm/xccl-seg-%d-*" % os.getpid()
    for n, windows in ((100, False), (777, True), (50001, True)):   # 400 B: below the threshold; 200 KB: 13 fragments
        for root in range(size):
            buf = np.zeros(n, np.float32)
            req = team.bcast(buf, root)
            if check_window and rank == root:
                # the root of a node-local level owns one window per region while the request lives
                assert bool(glob.glob(mine)) == windows, (n, root, glob.glob(mine))
            for it in range(3):  # persistent: the same regions and flags serve every post
                buf[:] = _data(root, n, np.float32, seed=10 + it) if rank == root else 0
                req.post().wait(timeout=60)
                np.testing.assert_array_equal(buf, _data(root, n, np.float32, seed=10 + it))
            req.finalize()
            assert not glob.glob(mine)
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


@pytest.mark.parametrize("name", ["one_node_unbound", "two_nodes_two_sockets", "uneven_nodes_leader1"])
def test_hier_bcast_through_fanout_get(name):
    """Host broadcasts whose node-local levels are FANOUT_GETs on the shared-segment team, closed by a FANIN
    (reference: src/team_lib/hier/xccl_hier_schedule_bcast.c:313-485, unreachable there for want of that team)."""
    node_of, sock_of, _ = LAYOUTS[name]
    run_ranks(_sm_get_bcast_rank, len(node_of), node_of, sock_of, name != "uneven_nodes_leader1", timeout=180)
