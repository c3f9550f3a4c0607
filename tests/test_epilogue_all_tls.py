"""The fused scale / cast epilogue (``xccl_coll_epilogue_t``) gives the same answer whichever team library serves
the reduction: the host team fuses it, the composite team libraries (hier, mpod with its three allreduce
algorithms, mrail) get it applied by the core as a last local step. CPU ranks, numpy oracle."""
import os

import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks


def _data(rank, count, seed=0):
    rng = np.random.default_rng(seed * 1000 + rank)
    return rng.integers(-8, 9, size=count).astype(np.float32)


def _check(team, rank, size, want_tl):
    assert team.coll_tl(K.ALLREDUCE, K.MEM_HOST) == want_tl
    for count in (1, 6, 1000, 4099):
        total = np.sum(np.stack([_data(r, count) for r in range(size)]), axis=0)
        # scale only, out of place; persistent request posted twice
        src, dst = _data(rank, count), np.zeros(count, np.float32)
        req = team.allreduce(src, dst, scale=0.5)
        for _ in range(2):
            dst[:] = 0
            req.post().wait(timeout=60)
            np.testing.assert_array_equal(dst, total * 0.5)
            np.testing.assert_array_equal(src, _data(rank, count))
        req.finalize()
        # scale only, in place
        buf = _data(rank, count)
        team.allreduce("in_place", buf, scale=1.0 / size).post().wait(timeout=60).finalize()
        np.testing.assert_allclose(buf, total / size, rtol=1e-6)
        # scale and cast to a narrower type: dst has half the bytes of the reduction buffer
        src, dst = _data(rank, count), np.zeros(count, np.float16)
        guard = np.full(count + 8, 77, np.float16)   # dst is a view with live elements after it
        view = guard[:count]
        team.allreduce(src, view, scale=0.25, out_dt=K.DT_FLOAT16).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(view, (total * 0.25).astype(np.float16))
        np.testing.assert_array_equal(guard[count:], np.full(8, 77, np.float16))
        # cast to a wider type
        src16, dst32 = _data(rank, count).astype(np.float16), np.zeros(count, np.float32)
        team.allreduce(src16, dst32, out_dt=K.DT_FLOAT32, dt=K.DT_FLOAT16).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(dst32, total)


def _rank(rank, size, job, tls, cfg, want_tl, fake_nodes):
    if fake_nodes:
        os.environ["XCCL_HIER_FAKE_NODE_ID"] = str(fake_nodes[rank])
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=tls, config=cfg)
    team = Team(ctx)
    _check(team, rank, size, want_tl)
    if want_tl == K.TL_UCX:
        # reduce (result on the root only) and reduce-scatter carry the epilogue too
        count = 777
        total = np.sum(np.stack([_data(r, count, 5) for r in range(size)]), axis=0)
        dst = np.zeros(count, np.float16)
        team.reduce(_data(rank, count, 5), dst, root=1, scale=0.5, out_dt=K.DT_FLOAT16).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(dst, (total * 0.5).astype(np.float16) if rank == 1 else np.zeros(count, np.float16))
        per = 50
        total = np.sum(np.stack([_data(r, per * size, 6) for r in range(size)]), axis=0)
        dst = np.zeros(per, np.float32)
        team.reduce_scatter(_data(rank, per * size, 6), dst, scale=0.5).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(dst, total[rank * per:(rank + 1) * per] * 0.5)
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


CASES = {
    "host": (K.TL_UCX, {}, K.TL_UCX, None),
    "hier_one_node": (K.TL_HIER | K.TL_UCX, {K.TL_HIER: {"ENABLE_NVLINK": "no"}}, K.TL_HIER, [0, 0, 0, 0]),
    "hier_two_nodes": (K.TL_HIER | K.TL_UCX, {K.TL_HIER: {"ENABLE_NVLINK": "no"}}, K.TL_HIER, [0, 0, 1, 1]),
    "mpod_replicate": (K.TL_MPOD | K.TL_UCX, {K.TL_MPOD: {"POD_SIZE": "2", "ALLREDUCE_ALGORITHM": "replicate",
                                                          "HOST_HIERARCHY": "y"}}, K.TL_MPOD, None),
    "mpod_split": (K.TL_MPOD | K.TL_UCX, {K.TL_MPOD: {"POD_SIZE": "2", "ALLREDUCE_ALGORITHM": "split",
                                                      "HOST_HIERARCHY": "y"}}, K.TL_MPOD, None),
    "mpod_coalesce": (K.TL_MPOD | K.TL_UCX, {K.TL_MPOD: {"POD_SIZE": "2", "ALLREDUCE_ALGORITHM": "coalesce",
                                                         "HOST_HIERARCHY": "y"}}, K.TL_MPOD, None),
    "mrail_ucx": (K.TL_MRAIL | K.TL_UCX, {K.TL_MRAIL: {"REPLICATE_TEAM": "ucx", "REPLICAS_NUMBER": "3", "THREADS_NUMBER": "0"},
                                          K.TL_HIER: {"ENABLE_NVLINK": "no"}}, K.TL_MRAIL, None),
    "mrail_hier": (K.TL_MRAIL | K.TL_UCX, {K.TL_MRAIL: {"REPLICATE_TEAM": "hier", "REPLICAS_NUMBER": "2", "THREADS_NUMBER": "2"},
                                           K.TL_HIER: {"ENABLE_NVLINK": "no"}}, K.TL_MRAIL, None),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_scale_and_cast_through_every_team_library(name):
    tls, cfg, want, fake = CASES[name]
    run_ranks(_rank, 4, tls, cfg, want, fake, timeout=180)
