"""Randomised sweep of the host team: many (collective, count, type, op, algorithm, root) combinations per
team, all ranks drawing the same cases from one seed, every result checked against numpy. Integer-valued
data keeps sums and products exact in every type."""
import numpy as np
import pytest

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks

DTYPES = [np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint32, np.float32, np.float64]
OPS = [(K.OP_SUM, np.sum), (K.OP_MAX, np.max), (K.OP_MIN, np.min)]


def _vals(rank, count, dtype, case):
    rng = np.random.default_rng(case * 131 + rank)
    lo, hi = (0, 5) if np.issubdtype(dtype, np.unsignedinteger) else (-4, 5)
    return rng.integers(lo, hi, size=count).astype(dtype)


def _rank_main(rank, size, job, n_cases, seed):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    rng = np.random.default_rng(seed)           # same stream on every rank
    done = {}
    for case in range(n_cases):
        coll = rng.choice(["allreduce", "reduce", "bcast", "allgather", "alltoall", "alltoallv"])
        dtype = DTYPES[rng.integers(len(DTYPES))]
        count = int(rng.choice([1, 2, 3, 7, 31, 257, 1024, 4099, 20000]))
        op, npop = OPS[rng.integers(len(OPS))]
        root = int(rng.integers(size))
        alg = [None, K.HOST_ALG_LINEAR, K.HOST_ALG_KNOMIAL, K.HOST_ALG_SRA][rng.integers(4)]
        everyone = [_vals(r, count, dtype, case) for r in range(size)]
        tag = f"case {case}: {coll} {np.dtype(dtype).name} count={count} op={op} root={root} alg={alg}"
        if coll == "allreduce":
            dst = np.zeros(count, dtype)
            team.allreduce(everyone[rank].copy(), dst, op=op, alg=None if alg == K.HOST_ALG_LINEAR else alg).run().finalize()
            np.testing.assert_array_equal(dst, npop(np.stack(everyone), axis=0).astype(dtype), err_msg=tag)
        elif coll == "reduce":
            dst = np.full(count, 3, dtype)
            a = alg if alg in (K.HOST_ALG_LINEAR, K.HOST_ALG_KNOMIAL) else None
            team.reduce(everyone[rank].copy(), dst, root=root, op=op, alg=a).run().finalize()
            if rank == root:
                np.testing.assert_array_equal(dst, npop(np.stack(everyone), axis=0).astype(dtype), err_msg=tag)
        elif coll == "bcast":
            buf = everyone[root].copy() if rank == root else np.zeros(count, dtype)
            a = alg if alg in (K.HOST_ALG_LINEAR, K.HOST_ALG_KNOMIAL) else None
            team.bcast(buf, root, alg=a).run().finalize()
            np.testing.assert_array_equal(buf, everyone[root], err_msg=tag)
        elif coll == "allgather":
            dst = np.zeros(count * size, dtype)
            team.allgather(everyone[rank].copy(), dst).run().finalize()
            np.testing.assert_array_equal(dst, np.concatenate(everyone), err_msg=tag)
        elif coll == "alltoall":
            full = [_vals(r, count * size, dtype, case + 7777) for r in range(size)]
            dst = np.zeros(count * size, dtype)
            a = alg if alg in (K.HOST_ALG_LINEAR, K.HOST_ALG_KNOMIAL) else None
            team.alltoall(full[rank].copy(), dst, alg=a).run().finalize()
            want = np.concatenate([full[s][rank * count:(rank + 1) * count] for s in range(size)])
            np.testing.assert_array_equal(dst, want, err_msg=tag)
        else:
            # counts[s][d]: elements rank s sends to rank d, a function of the case only
            crng = np.random.default_rng(case + 99)
            counts = crng.integers(0, 9, size=(size, size))
            full = [_vals(r, int(counts[r].sum()) + 1, dtype, case + 5555) for r in range(size)]
            sc = counts[rank]
            sd = np.concatenate([[0], np.cumsum(sc)[:-1]])
            rc = counts[:, rank]
            rd = np.concatenate([[0], np.cumsum(rc)[:-1]])
            dst = np.zeros(int(rc.sum()) + 1, dtype)
            team.alltoallv(full[rank].copy(), sc, sd, dst, rc, rd).run().finalize()
            want = []
            for s in range(size):
                off = int(counts[s][:rank].sum())
                want.append(full[s][off:off + int(counts[s][rank])])
            np.testing.assert_array_equal(dst[:int(rc.sum())], np.concatenate(want) if want else dst[:0], err_msg=tag)
        done[coll] = done.get(coll, 0) + 1
    team.close(); ctx.close(); lib.close(); oob.close()
    return done


@pytest.mark.parametrize("size,seed", [(3, 1), (5, 2), (8, 3)])
def test_random_cases_match_numpy(size, seed):
    res = run_ranks(_rank_main, size, 120, seed, timeout=300)
    assert all(r == res[0] for r in res) and sum(res[0].values()) == 120
