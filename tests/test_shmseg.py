"""Global memory map + FANOUT_GET through the shared-segment team (the reference's
test/test_mpi_fanout_get.c cannot pass with the team libraries it ships; this one can)."""
import numpy as np

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks


def _rank(rank, size, job):
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_SHMSEG | K.TL_UCX)
    team = Team(ctx)
    assert team.coll_tl(K.FANOUT_GET, K.MEM_HOST) == K.TL_SHMSEG
    n = 4096
    for root in (0, size - 1):
        region = np.zeros(n, np.int32)
        memh = team.mem_map(region, root)
        for it in range(3):
            if rank == root:
                region[:] = np.arange(n, dtype=np.int32) + it * 1000 + root
            local = np.full(n, -1, np.int32)
            half = n // 2 * 4
            # two half-buffer gets per iteration, like the reference test
            r1 = team.fanout_get(memh, 0, local, half).post()
            r2 = team.fanout_get(memh, half, local[n // 2:], half).post()
            r1.wait(timeout=30); r2.wait(timeout=30)
            r1.finalize(); r2.finalize()
            np.testing.assert_array_equal(local, np.arange(n, dtype=np.int32) + it * 1000 + root)
            team.fanin(root).run().finalize()   # the root may overwrite the region only now
        memh.unmap()
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


def test_fanout_get_over_global_mem_map():
    run_ranks(_rank, 4, timeout=120)
