"""Latency / bus-bandwidth sweep of the UNMODIFIED reference library (its NCCL team) on device
buffers: the reference arm of ``python -m xccl_b200.bench.collectives``.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        baseline/ref_sweep.py [--colls allreduce,alltoall] [--dtypes float32] [--min-bytes 4] [--max-bytes 1g] [--step 4]

Same timing rules and bus-bandwidth factors as the sweep of this repository: device time from CUDA
events around ``iters`` back-to-back posts on one stream after a warm-up post (best of three batches), maximum over ranks.
The reference has no bf16 reduction type and no fused post-scale: allreduce runs in fp32 or fp16
with plain sum (a user who wants the average launches a scaling kernel afterwards; that kernel is
NOT charged here). alltoall / allgather / bcast move bytes. One JSON line per case from rank 0,
with ``"impl": "reference"``. Nothing of ``xccl_b200`` is imported.
"""
import argparse
import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import ref_api as R  # noqa: E402


def _parse_size(s: str) -> int:
    s = s.lower()
    mult = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1]]) if s[-1] in mult else int(s)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--colls", default="allreduce,alltoall")
    ap.add_argument("--dtypes", default="float32")
    ap.add_argument("--min-bytes", default="4")
    ap.add_argument("--max-bytes", default="1g")
    ap.add_argument("--step", type=int, default=4)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s = R.RefSession(tls=R.TL_NCCL)
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference library failed to start: {exc}"}))
        return
    stream = torch.cuda.Stream()
    handle = C.c_void_p(stream.cuda_stream)
    sp = C.addressof(handle)
    dts = {"float32": (torch.float32, R.DT_FLOAT32), "float16": (torch.float16, R.DT_FLOAT16)}

    def max_ranks(v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sizes, b = [], _parse_size(a.min_bytes)
    while b <= _parse_size(a.max_bytes):
        sizes.append(b)
        b *= a.step
    n = world
    for coll in a.colls.split(","):
        for dname in a.dtypes.split(","):
            if dname not in dts:
                if rank == 0:
                    print(json.dumps({"impl": "reference", "coll": coll, "dtype": dname,
                                      "unsupported": "the reference has no such reduction type"}), flush=True)
                continue
            tdt, rdt = dts[dname]
            es = torch.tensor([], dtype=tdt).element_size()
            for nbytes in sizes:
                iters = 50 if nbytes <= (1 << 20) else (10 if nbytes <= (64 << 20) else 4)
                if coll == "allreduce":
                    count = max(nbytes // es, 1)
                    src = torch.randn(count, device=dev).to(tdt)
                    dst = torch.empty_like(src)
                    req = s.collective(R.ALLREDUCE, src.data_ptr(), dst.data_ptr(), length=count * es, count=count,
                                       dt=rdt, op=R.OP_SUM, stream_handle_ptr=sp)
                    factor, total = 2.0 * (n - 1) / n, count * es
                elif coll == "alltoall":
                    per = max(nbytes // n // es, 1)
                    src = torch.randn(per * n, device=dev).to(tdt)
                    dst = torch.empty_like(src)
                    req = s.collective(R.ALLTOALL, src.data_ptr(), dst.data_ptr(), length=per * es, stream_handle_ptr=sp)
                    factor, total = (n - 1) / n, per * n * es
                elif coll == "allgather":
                    per = max(nbytes // n // es, 1)
                    src = torch.randn(per, device=dev).to(tdt)
                    dst = torch.empty(per * n, device=dev, dtype=tdt)
                    req = s.collective(R.ALLGATHER, src.data_ptr(), dst.data_ptr(), length=per * n * es, stream_handle_ptr=sp)
                    factor, total = (n - 1) / n, per * n * es
                elif coll == "bcast":
                    count = max(nbytes // es, 1)
                    src = torch.randn(count, device=dev).to(tdt)
                    req = s.collective(R.BCAST, src.data_ptr(), src.data_ptr(), length=count * es, root=0, stream_handle_ptr=sp)
                    factor, total = 1.0, count * es
                else:
                    raise SystemExit(f"the reference's NCCL team has no {coll}")
                try:
                    s.post(req)
                except R.RefError as exc:
                    # the library refused its own call: report it and go on to the next collective
                    if rank == 0:
                        print(json.dumps({"impl": "reference", "coll": coll, "dtype": dname, "bytes": total,
                                          "error": str(exc)}), flush=True)
                    break
                best = float("inf")
                for _ in range(3):   # best of three batches, as in the sweep of the other arm
                    with torch.cuda.stream(stream):
                        stream.synchronize()
                        dist.barrier()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        for _ in range(iters):
                            s.post(req)
                        e1.record(stream)
                        stream.synchronize()
                    best = min(best, e0.elapsed_time(e1) / iters)
                ms = max_ranks(best)
                s.finalize(req)
                if rank == 0:
                    print(json.dumps({"impl": "reference", "alg": "reference_nccl_team", "coll": coll, "dtype": dname,
                                      "gpus": n, "bytes": total, "us": round(ms * 1e3, 2),
                                      "bus_gbs": round(factor * total / (ms * 1e-3) / 1e9, 2), "iters": iters}),
                          flush=True)
                del src
                torch.cuda.empty_cache()
    s.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
