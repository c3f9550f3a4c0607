"""Thread-multiple mode: several threads of every rank drive their own teams of one shared context
at the same time (the reference's test/test_mt.c:24-144 does the same with pthreads). Exercises the
lock-free progress queue and the locking of the host transport. ctypes releases the GIL inside every
library call, so the calls of different threads really overlap."""
import threading

import numpy as np

from xccl_b200 import _capi as K
from xccl_b200.api import Context, Lib, ShmOob, Team
from xccl_b200.utils.launch import run_ranks

N_THREADS, ITERS = 4, 40


def _rank_main(rank, size, job, tls=K.TL_UCX):
    oob = ShmOob(job, rank, size)
    lib = Lib(thread_mode=K.THREAD_MULTIPLE)
    ctx = Context(lib, oob, tls=tls, thread_mode=K.THREAD_MULTIPLE, config={K.TL_HIER: {"ENABLE_NVLINK": "no"}})
    errors, done = [], []

    def worker(tid: int) -> None:
        try:
            t_oob = ShmOob(f"{job}t{tid}", rank, size)     # every team bootstraps over its own channel
            team = Team(ctx, oob=t_oob)
            count = 1000 + 37 * tid
            src = (np.arange(count, dtype=np.int32) % 17) + rank + tid
            dst = np.zeros_like(src)
            want = sum((np.arange(count, dtype=np.int64) % 17) + r + tid for r in range(size)).astype(np.int32)
            req = team.allreduce(src, dst)                  # persistent: posted ITERS times
            bar = team.barrier()
            for _ in range(ITERS):
                dst[:] = 0
                req.post().wait(timeout=60)
                assert np.array_equal(dst, want), (tid, rank)
                bar.post().wait(timeout=60)
            req.finalize()
            bar.finalize()
            team.close()
            t_oob.close()
            done.append(tid)
        except BaseException as e:  # noqa: BLE001 - reported by the rank below
            errors.append((tid, repr(e)))

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(N_THREADS)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    alive = [t.name for t in threads if t.is_alive()]
    assert not alive, f"threads still running: {alive}"
    assert not errors, errors
    ctx.close()
    lib.close()
    oob.close()
    return sorted(done)


def test_threads_drive_their_own_teams_concurrently():
    res = run_ranks(_rank_main, 3, timeout=240)
    assert res == [list(range(N_THREADS))] * 3


def test_threads_drive_hierarchy_teams_concurrently():
    """The same with the hierarchy layer on top: its schedules run as tasks of the context's lock-free progress queue,
    which any of the threads may pop and progress."""
    res = run_ranks(_rank_main, 3, K.TL_HIER | K.TL_UCX, timeout=240)
    assert res == [list(range(N_THREADS))] * 3
