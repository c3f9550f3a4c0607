"""Run one Python function as N ranks (processes) on this host and collect the results.

This stands in for ``mpirun`` in the reference's tests (test/Makefile.am, CI in
.github/workflows/main.yml:43-60): no MPI exists here, so ranks are forked children that
bootstrap through the shared-memory OOB provider with a fresh job key.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import queue
import time
import traceback
import uuid
from typing import Any, Callable


def _child(fn: Callable, rank: int, size: int, job: str, args: tuple, env: dict, q: Any) -> None:
    try:
        os.environ.update({k: str(v) for k, v in env.items()})
        os.environ["XCCL_JOB_KEY"] = job
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(size)
        res = fn(rank, size, job, *args)
        q.put((rank, True, res))
    except BaseException:  # noqa: BLE001 - the parent reports it
        q.put((rank, False, traceback.format_exc()))


def run_ranks(fn: Callable, size: int, *args: Any, timeout: float = 120.0, env: dict | None = None,
              start_method: str = "fork") -> list:
    """Calls ``fn(rank, size, job_key, *args)`` in `size` processes; returns results by rank.

    Raises RuntimeError with the child's traceback when a rank fails, and TimeoutError (after
    terminating the children it started) when a rank does not finish within `timeout` seconds.
    """
    ctx = mp.get_context(start_method)
    q = ctx.Queue()
    job = uuid.uuid4().hex[:12]
    procs = [ctx.Process(target=_child, args=(fn, r, size, job, args, env or {}, q), daemon=True)
             for r in range(size)]
    for p in procs:
        p.start()
    results: dict[int, Any] = {}
    deadline = time.monotonic() + timeout
    failure = None
    try:
        while len(results) < size:
            left = deadline - time.monotonic()
            if left <= 0:
                raise TimeoutError(f"ranks {sorted(set(range(size)) - set(results))} did not finish in {timeout}s")
            try:
                rank, ok, res = q.get(timeout=min(left, 1.0))
            except queue.Empty:
                dead = [i for i, p in enumerate(procs) if not p.is_alive() and i not in results]
                if dead and q.empty():
                    time.sleep(0.2)
                    if q.empty():
                        raise RuntimeError(f"ranks {dead} exited without a result "
                                           f"(exit codes {[procs[i].exitcode for i in dead]})")
                continue
            if not ok:
                failure = f"rank {rank} failed:\n{res}"
                break
            results[rank] = res
        if failure:
            raise RuntimeError(failure)
    finally:
        for p in procs:
            p.join(timeout=0.5 if failure is None and len(results) == size else 0.1)
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=2.0)
        try:
            os.unlink(f"/dev/shm/xccl-oob-{job}")
        except OSError:
            pass
    return [results[r] for r in range(size)]
