"""Pod-split (mpod) and multirail (mrail) team libraries on host buffers, as CPU ranks.

HOST_HIERARCHY makes mpod run its pod algorithms on host memory (pod team and cross-pod team are
both the host team then), so the decomposition logic - pods, slices, shares, transposes, chunk
pipelines, the request FIFO - is checked without GPUs.
"""
import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks


def _data(rank, count, dtype, seed=0):
    rng = np.random.default_rng(seed * 1000 + rank)
    return rng.integers(-8, 9, size=count).astype(dtype)


def _mpod_rank(rank, size, job, pod_size, alg, chunk):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    cfg = {K.TL_MPOD: {"POD_SIZE": str(pod_size), "ALLREDUCE_ALGORITHM": alg, "ALLREDUCE_CHUNK_SIZE": chunk,
                       "HOST_HIERARCHY": "y"}}
    ctx = Context(lib, oob, tls=K.TL_MPOD | K.TL_UCX, config=cfg)
    team = Team(ctx)
    assert team.coll_tl(K.ALLREDUCE, K.MEM_HOST) == K.TL_MPOD
    for count in (pod_size * 6, 1000, 4099):
        src = _data(rank, count, np.int32)
        dst = np.zeros_like(src)
        req = team.allreduce(src, dst)
        for _ in range(2):
            dst[:] = 0
            req.post().wait(timeout=60)
            np.testing.assert_array_equal(dst, np.sum(np.stack([_data(r, count, np.int32) for r in range(size)]), axis=0))
        req.finalize()
    # two requests posted back to back: the FIFO runs them one after the other
    a, b = _data(rank, 300, np.float32, 1), _data(rank, 300, np.float32, 2)
    ra, rb = team.allreduce("in_place", a), team.allreduce("in_place", b, op=K.OP_MAX)
    ra.post(); rb.post()
    rb.wait(timeout=60); ra.wait(timeout=60)
    np.testing.assert_array_equal(a, np.sum(np.stack([_data(r, 300, np.float32, 1) for r in range(size)]), axis=0))
    np.testing.assert_array_equal(b, np.max(np.stack([_data(r, 300, np.float32, 2) for r in range(size)]), axis=0))
    ra.finalize(); rb.finalize()
    per = 77
    src = _data(rank, per, np.int32, 3)
    dst = np.zeros(per * size, np.int32)
    team.allgather(src, dst).post().wait(timeout=60).finalize()
    np.testing.assert_array_equal(dst, np.concatenate([_data(r, per, np.int32, 3) for r in range(size)]))
    for root in range(size):
        buf = _data(root, 513, np.float32, 4) if rank == root else np.zeros(513, np.float32)
        team.bcast(buf, root).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(buf, _data(root, 513, np.float32, 4))
    per = 50
    src = np.arange(per * size, dtype=np.int32) + rank * 100000
    dst = np.zeros_like(src)
    team.alltoall(src, dst).post().wait(timeout=60).finalize()
    want = np.concatenate([(np.arange(per * size, dtype=np.int32) + r * 100000)[rank * per:(rank + 1) * per]
                           for r in range(size)])
    np.testing.assert_array_equal(dst, want)
    team.barrier().post().wait(timeout=60).finalize()
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


@pytest.mark.parametrize("alg", ["replicate", "split", "coalesce"])
def test_mpod_two_pods_of_two(alg):
    run_ranks(_mpod_rank, 4, 2, alg, "256m", timeout=180)


def test_mpod_three_pods_chunked_pipeline():
    run_ranks(_mpod_rank, 6, 2, "split", "1k", timeout=180)


def _mrail_rank(rank, size, job, replicate, threads):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    cfg = {K.TL_MRAIL: {"REPLICATE_TEAM": replicate, "REPLICAS_NUMBER": "3", "THREADS_NUMBER": str(threads)},
           K.TL_HIER: {"ENABLE_NVLINK": "no"}}
    ctx = Context(lib, oob, tls=K.TL_MRAIL | K.TL_UCX, config=cfg)
    team = Team(ctx)
    assert team.coll_tl(K.ALLREDUCE, K.MEM_HOST) == K.TL_MRAIL
    for count in (2, 1000, 30001):
        src = _data(rank, count, np.int64)
        dst = np.zeros_like(src)
        req = team.allreduce(src, dst)
        for _ in range(2):
            dst[:] = 0
            req.post().wait(timeout=60)
            np.testing.assert_array_equal(dst, np.sum(np.stack([_data(r, count, np.int64) for r in range(size)]), axis=0))
        req.finalize()
    for root in (0, size - 1):
        buf = _data(root, 10007, np.float32, 4) if rank == root else np.zeros(10007, np.float32)
        team.bcast(buf, root).post().wait(timeout=60).finalize()
        np.testing.assert_array_equal(buf, _data(root, 10007, np.float32, 4))
    team.barrier().post().wait(timeout=60).finalize()
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


@pytest.mark.parametrize("replicate,threads", [("ucx", 0), ("ucx", 2), ("hier", 0)])
def test_mrail_three_replicas(replicate, threads):
    run_ranks(_mrail_rank, 4, replicate, threads, timeout=180,
              env={"HIER_ucx_XCCL_TEAM_UCX_RING_SIZE": "256k"})
