"""Randomised sweep of the composite team libraries on CPU ranks: the hierarchy layer on faked node / socket
placements, the pod-split layer with several pod sizes and all three allreduce algorithms, the multirail layer with and
without progress threads. All ranks draw the same cases from one seed; every result is checked against numpy on
integer-valued data. The reference has no test of these layers beyond its default CI placement (one node, no sockets)."""
import os

import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks

DTYPES = [np.int32, np.int64, np.float32, np.float64]
OPS = [(K.OP_SUM, np.sum), (K.OP_MAX, np.max), (K.OP_MIN, np.min)]
COUNTS = [1, 3, 31, 257, 1024, 4099, 30000]


def _vals(rank, count, dtype, case):
    rng = np.random.default_rng(case * 977 + rank)
    return rng.integers(-4, 5, size=count).astype(dtype)


def _sweep(team, rank, size, colls, n_cases, seed, tl):
    rng = np.random.default_rng(seed)
    for case in range(n_cases):
        coll = str(rng.choice(colls))
        dtype = DTYPES[rng.integers(len(DTYPES))]
        count = int(rng.choice(COUNTS))
        op, npop = OPS[rng.integers(len(OPS))]
        root = int(rng.integers(size))
        everyone = [_vals(r, count, dtype, case) for r in range(size)]
        tag = f"{K.TL_NAMES.get(tl, tl)} case {case}: {coll} {np.dtype(dtype).name} count={count} op={op} root={root}"
        if coll == "allreduce":
            dst = np.zeros(count, dtype)
            team.allreduce(everyone[rank].copy(), dst, op=op).run().finalize()
            np.testing.assert_array_equal(dst, npop(np.stack(everyone), axis=0).astype(dtype), err_msg=tag)
        elif coll == "bcast":
            buf = everyone[root].copy() if rank == root else np.zeros(count, dtype)
            team.bcast(buf, root).run().finalize()
            np.testing.assert_array_equal(buf, everyone[root], err_msg=tag)
        elif coll == "allgather":
            dst = np.zeros(count * size, dtype)
            team.allgather(everyone[rank].copy(), dst).run().finalize()
            np.testing.assert_array_equal(dst, np.concatenate(everyone), err_msg=tag)
        elif coll == "alltoall":
            full = [_vals(r, count * size, dtype, case + 7777) for r in range(size)]
            dst = np.zeros(count * size, dtype)
            team.alltoall(full[rank].copy(), dst).run().finalize()
            want = np.concatenate([full[s][rank * count:(rank + 1) * count] for s in range(size)])
            np.testing.assert_array_equal(dst, want, err_msg=tag)
        elif coll == "barrier":
            team.barrier().run().finalize()


def _hier_rank(rank, size, job, node_of, sock_of, leader, seed):
    os.environ["XCCL_HIER_FAKE_NODE_ID"] = str(node_of[rank])
    os.environ["XCCL_FAKE_SOCKET_ID"] = str(sock_of[rank])
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_HIER | K.TL_UCX,
                  config={K.TL_HIER: {"NODE_LEADER_RANK_ID": str(leader), "ENABLE_NVLINK": "no", "ENABLE_SHMSEG": "y",
                                      "BCAST_SM_GET": "1", "BCAST_SM_GET_THRESH": "8k", "BCAST_PIPELINE_THRESH": "32k",
                                      "BCAST_PIPELINE_DEPTH": "2"}})
    team = Team(ctx)
    _sweep(team, rank, size, ["allreduce", "bcast", "alltoall", "barrier"], 40, seed, K.TL_HIER)
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


PLACEMENTS = {
    "three_nodes_mixed_sockets": ([0, 0, 0, 1, 1, 2, 2], [0, 0, 1, 0, 1, 1, 1], 0),
    "two_nodes_unbound_leader2": ([0, 0, 0, 1, 1, 1, 1], [-1] * 7, 2),
    "one_node_three_sockets": ([0] * 6, [0, 1, 2, 0, 1, 2], 0),
    "interleaved_nodes": ([0, 1, 0, 1, 0, 1], [0, 0, 1, 1, 0, 0], 1),
}


@pytest.mark.parametrize("name", sorted(PLACEMENTS))
def test_hier_random_cases_on_faked_placements(name):
    node_of, sock_of, leader = PLACEMENTS[name]
    run_ranks(_hier_rank, len(node_of), node_of, sock_of, leader, 11, timeout=240)


def _mpod_rank(rank, size, job, pod, alg, seed):
    os.environ["XCCL_POD_SIZE"] = str(pod)
    os.environ["XCCL_MPOD_ALLREDUCE_ALGORITHM"] = alg
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_MPOD | K.TL_UCX)
    team = Team(ctx)
    assert team.coll_tl(K.ALLREDUCE, K.MEM_HOST) == K.TL_MPOD
    _sweep(team, rank, size, ["allreduce", "bcast", "allgather", "alltoall"], 30, seed, K.TL_MPOD)
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


@pytest.mark.parametrize("size,pod", [(6, 2), (6, 3), (8, 4), (4, 1), (4, 4)])
@pytest.mark.parametrize("alg", ["replicate", "split", "coalesce"])
def test_mpod_random_cases(size, pod, alg):
    run_ranks(_mpod_rank, size, pod, alg, 5, timeout=240)


def _mrail_rank(rank, size, job, threads, replicas, seed):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_MRAIL | K.TL_UCX,
                  config={K.TL_MRAIL: {"THREADS_NUMBER": str(threads), "REPLICAS_NUMBER": str(replicas),
                                       "REPLICATE_TEAM": "ucx"}})
    team = Team(ctx)
    assert team.coll_tl(K.ALLREDUCE, K.MEM_HOST) == K.TL_MRAIL
    _sweep(team, rank, size, ["allreduce", "bcast", "barrier"], 30, seed, K.TL_MRAIL)
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


@pytest.mark.parametrize("threads,replicas", [(0, 2), (2, 3), (1, 4)])
def test_mrail_random_cases(threads, replicas):
    run_ranks(_mrail_rank, 4, threads, replicas, 7, timeout=240)
