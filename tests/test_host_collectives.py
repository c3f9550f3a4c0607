"""Host team: every collective against a numpy oracle, as real processes over shared memory.

Mirrors the reference's MPI test programs (test/test_mpi_allreduce.c, test_mpi_reduce.c,
test_mpi_bcast.c, test_mpi_allgather.c, test_mpi_alltoall.c, test_mpi_alltoallv.c,
test_mpi_barrier.c), with the oracle computed from the same seeded data instead of MPI.
"""
import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks


def _data(rank, count, dtype, seed=0):
    rng = np.random.default_rng(seed * 1000 + rank)
    return rng.integers(-8, 9, size=count).astype(dtype)


def _setup(rank, size, job, config=None, tls=K.TL_UCX):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=tls, config=config)
    team = Team(ctx)
    return oob, lib, ctx, team


def _teardown(oob, lib, ctx, team):
    team.close()
    ctx.close()
    lib.close()
    oob.close()


def _allreduce_rank(rank, size, job, counts, config, alg):
    h = _setup(rank, size, job, config)
    team = h[3]
    assert team.coll_tl(K.ALLREDUCE, K.MEM_HOST) == K.TL_UCX
    for dtype in (np.float32, np.int32):
        for count in counts:
            for op, npop in ((K.OP_SUM, np.sum), (K.OP_MAX, np.max)):
                src = _data(rank, count, dtype)
                dst = np.zeros_like(src)
                team.allreduce(src, dst, op=op, alg=alg).run().finalize()
                want = npop(np.stack([_data(r, count, dtype) for r in range(size)]), axis=0)
                np.testing.assert_array_equal(dst, want.astype(dtype), err_msg=f"{dtype} count={count} op={op}")
    # in place, persistent request posted three times
    buf = _data(rank, 1000, np.int64)
    req = team.allreduce("in_place", buf)
    want = np.sum(np.stack([_data(r, 1000, np.int64) for r in range(size)]), axis=0)
    for it in range(3):
        req.run()
        np.testing.assert_array_equal(buf, want * size ** it)
    req.finalize()
    _teardown(*h)
    return True


def test_allreduce_world4_counts_pow2():
    counts = [1 << i for i in range(0, 21, 1)]
    run_ranks(_allreduce_rank, 4, counts, None, None, timeout=300)


@pytest.mark.parametrize("size", [2, 3, 5, 6, 7, 8])
@pytest.mark.parametrize("alg", [K.HOST_ALG_KNOMIAL, K.HOST_ALG_SRA])
def test_allreduce_any_team_size(size, alg):
    run_ranks(_allreduce_rank, size, [1, 3, 7, 64, 1025, 5000], None, alg, timeout=120)


@pytest.mark.parametrize("radix", [2, 3, 8])
def test_allreduce_radix(radix):
    cfg = {K.TL_UCX: {"ALLREDUCE_KN_RADIX": str(radix)}}
    run_ranks(_allreduce_rank, 6, [5, 4096], cfg, None, timeout=120)


def _dtype_ops_rank(rank, size, job):
    h = _setup(rank, size, job)
    team = h[3]
    cases = [(np.int8, K.OP_BAND, np.bitwise_and.reduce), (np.uint16, K.OP_BOR, np.bitwise_or.reduce),
             (np.uint32, K.OP_BXOR, np.bitwise_xor.reduce), (np.int16, K.OP_MIN, np.min),
             (np.uint64, K.OP_PROD, np.prod), (np.float64, K.OP_PROD, np.prod),
             (np.int32, K.OP_LAND, lambda a, axis: np.logical_and.reduce(a != 0, axis=axis)),
             (np.int32, K.OP_LOR, lambda a, axis: np.logical_or.reduce(a != 0, axis=axis)),
             (np.float16, K.OP_SUM, np.sum)]
    for dtype, op, ref in cases:
        rng = np.random.default_rng(rank + 7)
        src = rng.integers(0, 4, size=257).astype(dtype)
        dst = np.zeros_like(src)
        team.allreduce(src, dst, op=op).run().finalize()
        allv = np.stack([np.random.default_rng(r + 7).integers(0, 4, size=257).astype(dtype) for r in range(size)])
        want = ref(allv, axis=0).astype(dtype)
        np.testing.assert_array_equal(dst, want, err_msg=f"{dtype} op={op}")
    _teardown(*h)
    return True


def test_allreduce_dtypes_and_ops():
    run_ranks(_dtype_ops_rank, 4)


def _rooted_rank(rank, size, job):
    h = _setup(rank, size, job)
    team = h[3]
    for count in (1, 32, 3000):
        for root in range(size):
            for alg in (None, K.HOST_ALG_LINEAR):
                # reduce
                src = _data(rank, count, np.int32, seed=root)
                dst = np.full_like(src, -77)
                team.reduce(src, dst, root, alg=alg).run().finalize()
                if rank == root:
                    want = np.sum(np.stack([_data(r, count, np.int32, seed=root) for r in range(size)]), axis=0)
                    np.testing.assert_array_equal(dst, want)
                # bcast (in place on every rank, like test/test_mpi_bcast.c)
                buf = _data(root, count, np.float32, seed=5) if rank == root else np.zeros(count, np.float32)
                team.bcast(buf, root, alg=alg).run().finalize()
                np.testing.assert_array_equal(buf, _data(root, count, np.float32, seed=5))
    _teardown(*h)
    return True


@pytest.mark.parametrize("size", [4, 7])
def test_reduce_and_bcast_every_root(size):
    run_ranks(_rooted_rank, size, timeout=180)


def _gather_scatter_rank(rank, size, job, config):
    h = _setup(rank, size, job, config)
    team = h[3]
    # allgather
    for count in (1, 17, 4096):
        src = _data(rank, count, np.int32)
        dst = np.zeros(count * size, np.int32)
        team.allgather(src, dst).run().finalize()
        np.testing.assert_array_equal(dst, np.concatenate([_data(r, count, np.int32) for r in range(size)]))
    # alltoall, 1024 elements per peer (BASELINE config) and small sizes
    for per in (1, 256, 1024):
        src = np.arange(per * size, dtype=np.int32) + rank * 100000
        dst = np.zeros_like(src)
        req = team.alltoall(src, dst)
        for _ in range(2):
            dst[:] = 0
            req.run()
            want = np.concatenate([(np.arange(per * size, dtype=np.int32) + r * 100000)[rank * per:(rank + 1) * per]
                                   for r in range(size)])
            np.testing.assert_array_equal(dst, want)
        req.finalize()
        # in place -> linear shift algorithm
        buf = src.copy()
        team.alltoall("in_place", buf, bytes_per_peer=per * 4).run().finalize()
        np.testing.assert_array_equal(buf, want)
    # alltoallv with rank-dependent counts: rank s sends (s + d + 1) elements to rank d
    scounts = [rank + d + 1 for d in range(size)]
    sdispl = np.concatenate([[0], np.cumsum(scounts)[:-1]]).tolist()
    rcounts = [s + rank + 1 for s in range(size)]
    rdispl = np.concatenate([[0], np.cumsum(rcounts)[:-1]]).tolist()
    src = np.concatenate([np.full(scounts[d], rank * 100 + d, np.float32) for d in range(size)])
    dst = np.zeros(sum(rcounts), np.float32)
    team.alltoallv(src, scounts, sdispl, dst, rcounts, rdispl).run().finalize()
    want = np.concatenate([np.full(rcounts[s], s * 100 + rank, np.float32) for s in range(size)])
    np.testing.assert_array_equal(dst, want)
    # reduce-scatter (extension)
    src = _data(rank, 64 * size, np.float32)
    dst = np.zeros(64, np.float32)
    team.reduce_scatter(src, dst).run().finalize()
    full = np.sum(np.stack([_data(r, 64 * size, np.float32) for r in range(size)]), axis=0)
    np.testing.assert_array_equal(dst, full[rank * 64:(rank + 1) * 64])
    _teardown(*h)
    return True


@pytest.mark.parametrize("size", [4, 5])
def test_allgather_alltoall_alltoallv(size):
    run_ranks(_gather_scatter_rank, size, None, timeout=180)


@pytest.mark.parametrize("cfg", [{"ALLTOALL_PAIRWISE_CHUNK": "0"}, {"ALLTOALL_PAIRWISE_CHUNK": "2", "ALLTOALL_PAIRWISE_REVERSE": "1"},
                                 {"ALLTOALL_PAIRWISE_BARRIER": "2"}])
def test_alltoall_pairwise_options(cfg):
    run_ranks(_gather_scatter_rank, 6, {K.TL_UCX: cfg}, timeout=180)


def _barrier_rank(rank, size, job):
    import time
    h = _setup(rank, size, job)
    team = h[3]
    # nobody may leave the barrier before the slowest rank entered it
    stamps = np.zeros(size, np.float64)
    time.sleep(0.05 * rank)
    t_in = time.time()
    team.barrier().run().finalize()
    t_out = time.time()
    mine = np.array([t_in, t_out], np.float64)
    allv = np.zeros(2 * size, np.float64)
    team.allgather(mine, allv).run().finalize()
    assert allv[1::2].min() >= allv[0::2].max() - 1e-3, allv
    for root in range(size):
        team.fanin(root).run().finalize()
        team.fanout(root).run().finalize()
    del stamps
    _teardown(*h)
    return True


@pytest.mark.parametrize("size", [3, 4, 8])
def test_barrier_fanin_fanout(size):
    run_ranks(_barrier_rank, size)


def _large_message_rank(rank, size, job):
    # larger than the per-peer ring: the transport must stream
    h = _setup(rank, size, job, {K.TL_UCX: {"RING_SIZE": "64k"}})
    team = h[3]
    n = 1 << 20
    src = _data(rank, n, np.float32)
    dst = np.zeros_like(src)
    for alg in (K.HOST_ALG_KNOMIAL, K.HOST_ALG_SRA):
        team.allreduce(src, dst, alg=alg).run().finalize()
        np.testing.assert_array_equal(dst, np.sum(np.stack([_data(r, n, np.float32) for r in range(size)]), axis=0))
    _teardown(*h)
    return True


def test_streaming_through_small_ring():
    run_ranks(_large_message_rank, 3, timeout=180)


def test_knomial_layout_rules():
    import ctypes as C
    L = K.load()
    out = (C.c_int * 16)()
    role, rounds, partner = C.c_int(), C.c_int(), C.c_int()
    # size 6, radix 4: one full tree of 4, ranks 4 and 5 are extras of proxies 0 and 1, one round
    n = L.xccl_host_knomial_peers(0, 6, 4, 0, out, C.byref(role), C.byref(rounds), C.byref(partner))
    assert (role.value, rounds.value, partner.value) == (1, 1, 4)
    assert sorted(out[:n]) == [1, 2, 3]
    n = L.xccl_host_knomial_peers(5, 6, 4, 0, out, C.byref(role), C.byref(rounds), C.byref(partner))
    assert (role.value, partner.value, n) == (2, 1, 0)
    # size 8, radix 4: two full trees, second round pairs rank r with r +- 4 only
    n = L.xccl_host_knomial_peers(0, 8, 4, 1, out, C.byref(role), C.byref(rounds), C.byref(partner))
    assert (role.value, rounds.value) == (0, 2) and list(out[:n]) == [4]
    n = L.xccl_host_knomial_peers(6, 8, 4, 1, out, C.byref(role), C.byref(rounds), C.byref(partner))
    assert list(out[:n]) == [2]
    # power of the radix: every round has radix-1 peers
    for rnd in range(2):
        n = L.xccl_host_knomial_peers(5, 16, 4, rnd, out, C.byref(role), C.byref(rounds), C.byref(partner))
        assert n == 3 and rounds.value == 2
