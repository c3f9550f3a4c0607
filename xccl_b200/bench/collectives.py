"""Latency / bus-bandwidth sweep of the collectives: NVLink team (per algorithm) against the
NCCL team, one process per GPU.

    python -m xccl_b200.bench.collectives --gpus 8 [--colls allreduce,alltoall] [--max-bytes 1g]

Every number is device time (CUDA events around `iters` back-to-back posts of one persistent request
on one stream, no host wait between posts; the best of three such batches), the maximum over ranks, after warm-up. Bus bandwidth uses the usual factors: allreduce
2(N-1)/N * S / t, allgather / reduce-scatter / alltoall (N-1)/N * S / t, bcast S / t.
Allreduce runs with the fused 1/N post-scale, as gradient averaging would.
Output: one JSON object per line on stdout (rank 0) and, with --table, a selection table
(`team_size one_shot_max nvls_min`) derived from the measurements.
"""
from __future__ import annotations

import argparse
import json
import struct
import sys

import torch

from .. import _capi as K
from ..utils.launch import run_ranks


def _parse_size(s: str) -> int:
    s = s.lower()
    mult = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1]]) if s[-1] in mult else int(s)


def _sizes(lo: int, hi: int, step: int) -> list[int]:
    out, s = [], lo
    while s <= hi:
        out.append(s)
        s *= step
    return out


def _rank_main(rank: int, size: int, job: str, opts: dict) -> list:
    from ..api import Context, Lib, ShmOob, Team
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    lib = Lib()
    results = []
    impls = []
    # DIRECT_MIN out of reach: the sweep names every algorithm itself ("direct" rows force it)
    cfg = {K.TL_NVLINK: {"WORKSPACE_SIZE": opts["workspace"], "MAX_BLOCKS": str(opts["max_blocks"]),
                         "DIRECT_MIN": "1024g"}}
    ctx_n = Context(lib, oob, tls=K.TL_NVLINK | K.TL_UCX, config=cfg)
    team_n = Team(ctx_n)
    impls.append(("nvlink", team_n))
    ctx_c = Context(lib, oob, tls=K.TL_NCCL | K.TL_UCX)
    team_c = Team(ctx_c)
    impls.append(("nccl", team_c))
    # what a caller gets without naming an algorithm or changing an option: "auto" on ordinary tensors,
    # "symmetric" on buffers from Team.mem_alloc (zero-copy NVLS above the one-shot range)
    ctx_a = Context(lib, oob, tls=K.TL_NVLINK | K.TL_UCX)
    team_a = Team(ctx_a)
    sym_mem = None
    if opts.get("symmetric", True):
        try:
            sym_mem = team_a.mem_alloc(2 * max(opts["sizes"]) + 4096)
        except Exception as e:  # no multicast on this machine
            if rank == 0:
                print(f"symmetric memory unavailable: {e}", file=sys.stderr)
    from .clocks import ClockSampler
    sampler = ClockSampler(rank)
    sampler.start()
    import time as _time
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream

    def max_ranks(v: float) -> float:
        vals = oob.allgather_bytes(struct.pack("d", v))
        return max(struct.unpack("d", b)[0] for b in vals)

    def run_case(coll: str, impl: str, team, nbytes: int, dtype, alg, alg_name: str):
        es = torch.tensor([], dtype=dtype).element_size()
        n = size
        t_begin = _time.monotonic()
        iters = 50 if nbytes <= (1 << 20) else (10 if nbytes <= (64 << 20) else 4)
        if coll == "allreduce":
            count = max(nbytes // es, 1)
            if alg_name == "symmetric":
                half = sym_mem.numel() // 2 // 4096 * 4096
                src = sym_mem[:count * es].view(dtype)
                dst = sym_mem[half:half + count * es].view(dtype)
                src.copy_(torch.randn(count, device=dev).to(dtype))
            else:
                src = torch.randn(count, device=dev).to(dtype)
                dst = torch.empty_like(src)
            kw = dict(alg=alg, stream=sh)
            if impl == "nvlink":
                kw.update(scale=1.0 / n)
            req = team.allreduce(src, dst, **kw)
            factor, total = 2.0 * (n - 1) / n, count * es
        elif coll == "alltoall":
            per = max(nbytes // n // es, 1)
            src = torch.randn(per * n, device=dev).to(dtype)
            dst = torch.empty_like(src)
            req = team.alltoall(src, dst, stream=sh, alg=alg)
            factor, total = (n - 1) / n, per * n * es
        elif coll == "allgather":
            per = max(nbytes // n // es, 1)
            src = torch.randn(per, device=dev).to(dtype)
            dst = torch.empty(per * n, device=dev, dtype=dtype)
            req = team.allgather(src, dst, stream=sh, alg=alg)
            factor, total = (n - 1) / n, per * n * es
        elif coll == "reduce_scatter":
            per = max(nbytes // n // es, 1)
            src = torch.randn(per * n, device=dev).to(dtype)
            dst = torch.empty(per, device=dev, dtype=dtype)
            req = team.reduce_scatter(src, dst, stream=sh, alg=alg)
            factor, total = (n - 1) / n, per * n * es
        elif coll == "bcast":
            if alg_name == "symmetric":
                buf = sym_mem[:max(nbytes // es, 1) * es].view(dtype)
            else:
                buf = torch.randn(max(nbytes // es, 1), device=dev).to(dtype)
            req = team.bcast(buf, 0, stream=sh, alg=alg)
            factor, total = 1.0, buf.numel() * es
        else:
            raise ValueError(coll)
        try:
            # one persistent request cannot be re-posted before it completed: use several
            reqs = [req]
            for _ in range(3):
                warm = reqs[0].post()
                warm.wait()
            torch.cuda.synchronize()
            oob.allgather_bytes(b"x")
            # best of `reps` batches: one stray interruption of a rank (another tenant of the host, a lazily loaded
            # kernel image) would otherwise sit in the average of a 50-post batch
            ms = float("inf")
            for _ in range(opts.get("reps", 3)):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(stream):
                    e0.record(stream)
                    for _ in range(iters):
                        # posts of one request are ordered by its stream: no host wait between them, so the
                        # number is device time per operation, not launch-and-synchronise time
                        req.post()
                    req.wait()
                    e1.record(stream)
                stream.synchronize()
                ms = min(ms, e0.elapsed_time(e1) / iters)
        except Exception as e:  # an algorithm that does not apply at this size
            req.finalize() if hasattr(req, "finalize") else None
            return {"coll": coll, "impl": impl, "alg": alg_name, "bytes": total, "error": str(e)[:80]}
        us = max_ranks(ms * 1e3)
        req.finalize()
        clk = sampler.window(t_begin, _time.monotonic())
        return {"coll": coll, "impl": impl, "alg": alg_name, "dtype": str(dtype).replace("torch.", ""), "gpus": n,
                "bytes": total, "us": round(us, 2), "bus_gbs": round(factor * total / (us * 1e-6) / 1e9, 2),
                "iters": iters, "sm_mhz": clk["sm_mhz"], "clock_reasons": clk["reasons"]}

    dtypes = [getattr(torch, d) for d in opts["dtypes"]]
    for coll in opts["colls"]:
        for dtype in dtypes:
            for nbytes in opts["sizes"]:
                cases = []
                if coll == "allreduce":
                    half = _parse_size(opts["workspace"]) // 2
                    if nbytes * size <= half and nbytes <= (4 << 20):
                        cases.append(("nvlink", team_n, K.NVLINK_ALG_ONE_SHOT, "one_shot"))
                    cases.append(("nvlink", team_n, K.NVLINK_ALG_TWO_SHOT, "two_shot"))
                    if nbytes >= 1024:
                        cases.append(("nvlink", team_n, K.NVLINK_ALG_NVLS, "nvls"))
                elif coll == "bcast":
                    cases.append(("nvlink", team_n, K.NVLINK_ALG_TWO_SHOT, "pull"))
                    cases.append(("nvlink", team_n, K.NVLINK_ALG_NVLS, "multicast"))
                elif coll in ("alltoall", "allgather"):
                    cases.append(("nvlink", team_n, K.NVLINK_ALG_TWO_SHOT, "pull"))
                    if nbytes <= (4 << 20):
                        cases.append(("nvlink", team_n, K.NVLINK_ALG_ONE_SHOT, "push"))
                else:
                    cases.append(("nvlink", team_n, None, "pull"))
                if coll in ("allreduce", "alltoall", "allgather", "reduce_scatter") and nbytes >= (1 << 20):
                    # zero-copy kernels on buffers registered with the peers when the request is initialised
                    cases.append(("nvlink", team_n, K.NVLINK_ALG_DIRECT, "direct"))
                cases.append(("nvlink", team_a, None, "auto"))
                if sym_mem is not None and coll in ("allreduce", "bcast") and nbytes >= 16 and nbytes % 16 == 0:
                    cases.append(("nvlink", team_a, None, "symmetric"))
                cases.append(("nccl", team_c, None, "nccl"))
                for impl, team, alg, name in cases:
                    r = run_case(coll, impl, team, nbytes, dtype, alg, name)
                    if rank == 0:
                        results.append(r)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if rank == 0:
        results.append({"clocks_whole_run": clocks})
    if sym_mem is not None:
        team_a.mem_free(sym_mem)
    team_n.close(); team_c.close(); team_a.close(); ctx_n.close(); ctx_c.close(); ctx_a.close(); lib.close(); oob.close()
    return results


def selection_table(rows: list[dict]) -> dict:
    """Per team size: the largest size where one-shot is fastest, the smallest where NVLS is, and the smallest
    from which the direct (registered-buffer) kernel stays fastest. The file written with --table is what
    XCCL_TEAM_NVLINK_TUNING_FILE reads: lines of `team_size one_shot_max nvls_min direct_min`, -1 = keep the default."""
    out = {}
    ar = [r for r in rows if r.get("coll") == "allreduce" and r.get("impl") == "nvlink" and "us" in r]
    for n in sorted({r["gpus"] for r in ar}):
        by_size: dict[int, dict[str, float]] = {}
        for r in ar:
            if r["gpus"] == n and r["dtype"] == "float32":
                by_size.setdefault(r["bytes"], {})[r["alg"]] = r["us"]
        one_shot_max, nvls_min, direct_min = 0, None, None
        for s in sorted(by_size):
            best = min(by_size[s], key=by_size[s].get)
            if best == "one_shot":
                one_shot_max = s
            if best == "nvls" and nvls_min is None:
                nvls_min = s
            if best == "direct":
                direct_min = s if direct_min is None else direct_min
            elif "direct" in by_size[s]:
                direct_min = None          # something else won again at a larger size
        out[n] = {"one_shot_max": one_shot_max, "nvls_min": nvls_min, "direct_min": direct_min}
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--colls", default="allreduce,alltoall")
    ap.add_argument("--dtypes", default="float32,bfloat16")
    ap.add_argument("--min-bytes", default="4")
    ap.add_argument("--max-bytes", default="1g")
    ap.add_argument("--step", type=int, default=4)
    ap.add_argument("--workspace", default="512m")
    ap.add_argument("--max-blocks", type=int, default=128)
    ap.add_argument("--table", default=None, help="write the derived selection table to this file")
    ap.add_argument("--no-symmetric", action="store_true", help="skip the rows on symmetric memory")
    ap.add_argument("--reps", type=int, default=3, help="batches per case; the best one is reported")
    a = ap.parse_args()
    opts = {"colls": a.colls.split(","), "dtypes": a.dtypes.split(","), "workspace": a.workspace,
            "symmetric": not a.no_symmetric, "reps": a.reps,
            "max_blocks": a.max_blocks, "sizes": _sizes(_parse_size(a.min_bytes), _parse_size(a.max_bytes), a.step)}
    res = run_ranks(_rank_main, a.gpus, opts, timeout=1500, start_method="spawn")
    for r in res[0]:
        print(json.dumps(r), flush=True)
    if a.table:
        tab = selection_table(res[0])
        with open(a.table, "a") as f:
            for n, t in tab.items():
                f.write(f"{n} {t['one_shot_max']} {t['nvls_min'] if t['nvls_min'] is not None else -1} "
                        f"{t['direct_min'] if t['direct_min'] is not None else -1}\n")
        print(json.dumps({"selection_table": tab}), file=sys.stderr)


if __name__ == "__main__":
    main()
