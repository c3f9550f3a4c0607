"""OSU-style latency of the host team (shared-memory transport) on CPU ranks of this machine.

    python -m xccl_b200.bench.host_latency [--ranks 8] [--colls allreduce,bcast] [--max-bytes 32768]

For every size: 200 warm-up and 2000 timed blocking operations per rank; the number is the mean over
ranks of the per-rank mean, in microseconds, as osu_allreduce / osu_bcast report it (the reference
publishes such tables for other machines, README.md:75-132). One JSON line per size.
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np

from .. import _capi as K
from ..utils.launch import run_ranks


def _rank_main(rank: int, size: int, job: str, colls: list, sizes: list, iters: int) -> list:
    from ..api import Context, Lib, ShmOob, Team
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    out = []
    for coll in colls:
        for nbytes in sizes:
            n = max(nbytes // 4, 1)
            src = np.ones(n, dtype=np.float32)
            dst = np.zeros_like(src)
            req = team.allreduce(src, dst) if coll == "allreduce" else team.bcast(dst, 0)
            for _ in range(iters // 10):
                req.run()
            team.barrier().run().finalize()
            t0 = time.perf_counter()
            for _ in range(iters):
                req.run()
            us = (time.perf_counter() - t0) / iters * 1e6
            req.finalize()
            vals = oob.allgather_bytes(np.float64(us).tobytes())
            mean = float(np.mean([np.frombuffer(v, dtype=np.float64)[0] for v in vals]))
            if rank == 0:
                out.append({"bench": "host_latency", "coll": coll, "ranks": size, "bytes": n * 4, "us": round(mean, 2)})
    team.close(); ctx.close(); lib.close(); oob.close()
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--colls", default="allreduce,bcast")
    ap.add_argument("--max-bytes", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=2000)
    a = ap.parse_args()
    sizes, b = [], 4
    while b <= a.max_bytes:
        sizes.append(b)
        b *= 2
    res = run_ranks(_rank_main, a.ranks, a.colls.split(","), sizes, a.iters, timeout=600)
    for r in res[0]:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
