#!/usr/bin/env python
"""Headline benchmark: tensor-parallel Llama-style MLP block step throughput.

Config (fixed): 8192 tokens, hidden 8192, FFN 28672, SwiGLU, bf16, TP = number of GPUs, synthetic
activations ~N(0,1) and random-init weights ~N(0,0.02). One step is the forward of the block:
allgather->GEMM(+SwiGLU) and GEMM->reduce-scatter, each ONE fused tcgen05 kernel of this
repository (with one GPU the same kernels run without communication). Total work is fixed as GPUs
are added (strong scaling); the value is whole-job tokens per second.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl xccl|reference|torch]

For N > 1 launch one process per GPU, e.g.
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W
Rank 0 prints ONE JSON line. `--impl torch` times the same block written with torch collectives
and matmuls (NCCL + cuBLAS) for comparison; `--impl reference` is the unmodified reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import uuid

TOKENS, HIDDEN, FFN = 8192, 8192, 28672
METRIC = "tp_mlp_step_tokens_per_s"


try:
    from xccl_b200.bench.clocks import ClockSampler
except Exception:  # the reference arm runs even where the package cannot be imported
    ClockSampler = None


class _NoClocks:
    def start(self): pass
    def mark_begin(self): pass
    def mark_end(self): pass
    def stop(self): return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampler unavailable"]}


def reference_unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="xccl", choices=["xccl", "reference", "torch"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"],
                    help="fp8: the block-scaled e4m3 variant of the fused kernels (impl xccl only); the headline is bf16")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    ref_root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline")
    if args.impl == "reference" and not os.path.exists(os.path.join(ref_root, "_ref", "lib", "libxccl.so")):
        if int(os.environ.get("RANK", "0")) == 0:
            reference_unavailable("baseline/_ref/lib/libxccl.so is missing: the reference has no pip-installable "
                                  "package; it is built from its unmodified sources by python baseline/build_ref.py")
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            sys.exit("launch one process per GPU with torch.distributed.run for --gpus > 1 (see --help)")
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    oob = None
    ref_session = None
    if args.impl == "reference":
        # the unmodified reference library: its NCCL team for the collectives, cuBLAS (torch.matmul) for the GEMMs
        sys.path.insert(0, ref_root)
        import ref_api
        from ref_tp_mlp import RefTpMlp
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29531")
            dist.init_process_group("gloo", rank=0, world_size=1)
            oob_group = None
        else:
            oob_group = dist.new_group(backend="gloo")
        try:
            ref_session = ref_api.RefSession(group=oob_group, tls=ref_api.TL_NCCL)
        except Exception as exc:  # the library could not bring up its NCCL team here
            if rank == 0:
                reference_unavailable(f"reference library failed to start: {exc}")
            return
        model = RefTpMlp(TOKENS, HIDDEN, FFN, tp=world, rank=rank, session=ref_session)
        model.x_shard.copy_(torch.randn(TOKENS // world, HIDDEN, device=dev).to(torch.bfloat16))
        xp = torch.randn(TOKENS // world, HIDDEN).to(torch.bfloat16).pin_memory()
        yp = [torch.empty(TOKENS // world, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        step = lambda: model.forward()                 # noqa: E731
        e2e_step = lambda: model.forward_from_host(xp)  # noqa: E731
        full_step = lambda: model.forward_from_host_full(xp, yp)  # noqa: E731
        launches_per_step = 0
    elif args.impl == "xccl":
        from xccl_b200.models.tp_mlp import TpMlp, TpMlpFp8
        if world > 1:
            from xccl_b200.api import ShmOob
            key = [uuid.uuid4().hex[:12] if rank == 0 else None]
            dist.broadcast_object_list(key, src=0)
            oob = ShmOob(key[0], rank, world)
        model = (TpMlpFp8 if args.dtype == "fp8" else TpMlp)(TOKENS, HIDDEN, FFN, tp=world, rank=rank, oob=oob)
        x_dev = [torch.randn(TOKENS // world, HIDDEN, device=dev).to(torch.bfloat16)]
        x_pin = [torch.randn(TOKENS // world, HIDDEN).to(torch.bfloat16).pin_memory()]
        y_pin = [[torch.empty(TOKENS // world, HIDDEN, dtype=torch.bfloat16).pin_memory()] for _ in range(2)]
        step = lambda: model.forward(x_dev)           # noqa: E731
        e2e_step = lambda: model.forward_from_host(x_pin)  # noqa: E731
        full_step = lambda: model.forward_from_host_full(x_pin, y_pin)  # noqa: E731
        launches_per_step = 3 if args.dtype == "fp8" else 2
    else:
        from xccl_b200.models.tp_mlp import TorchTpMlp
        model = TorchTpMlp(TOKENS, HIDDEN, FFN, tp=world, rank=rank)
        xd = torch.randn(TOKENS // world, HIDDEN, device=dev).to(torch.bfloat16)
        xp = torch.randn(TOKENS // world, HIDDEN).to(torch.bfloat16).pin_memory()
        yp = [torch.empty(TOKENS // world, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        step = lambda: model.forward(xd)               # noqa: E731
        e2e_step = lambda: model.forward_from_host(xp)  # noqa: E731
        full_step = lambda: model.forward_from_host_full(xp, yp)  # noqa: E731
        launches_per_step = 0

    def timed(fn, n: int, after=None) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        if after is not None:
            after()    # work the steps left on other streams joins the timed stream before the closing event
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    def numerics_check() -> bool:
        """One output shard against the plain fp32 statement of the block on a sample of its rows (the block is
        row-wise, so a rank's output rows depend on its own input rows and on the full weights, which every rank
        can rebuild from the seeds). Outside every timed region."""
        from xccl_b200.models.tp_mlp import _init_weights
        y = model.forward(x_dev)[0]
        torch.cuda.synchronize()
        model.check_error()
        rows = torch.arange(0, TOKENS // world, max(1, TOKENS // world // 48), device=dev)[:48]
        xs = x_dev[0][rows].float()
        want = torch.zeros(rows.numel(), HIDDEN, device=dev, dtype=torch.float32)
        for r in range(world):
            wg, wu, wd = _init_weights(TOKENS, HIDDEN, FFN, world, r, dev)
            h = torch.nn.functional.silu(xs @ wg.float().t()) * (xs @ wu.float().t())
            want += h.to(torch.bfloat16).float() @ wd.float().t()
            del wg, wu, wd, h
        err = float((y[rows].float() - want).abs().max())
        tol = 3e-2 if args.dtype == "bf16" else 1.5e-1
        ok = torch.tensor([1.0 if err <= tol + tol * float(want.abs().max()) else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        return bool(ok.item() == 1.0), err

    def split_times(n: int = 10) -> dict:
        """Device time of each of the two launches of a step, and of the same two GEMM shapes without
        communication, each timed alone over n launches (max over ranks). Outside the headline region."""
        from xccl_b200.ops import gemm as G
        f_local = FFN // world
        out = {}
        model.forward(x_dev)
        out["ag_gemm_swiglu_ms"] = timed(lambda: model.ws.ag_gemm_swiglu(model.w_gate, model.w_up, model.h), n) / n
        out["gemm_rs_ms"] = timed(lambda: model.ws.gemm_rs(model.h, model.w_down, model.y), n) / n
        xa = torch.randn(TOKENS, HIDDEN, device=dev).to(torch.bfloat16)
        hh = torch.empty(TOKENS, f_local, device=dev, dtype=torch.bfloat16)
        yy = torch.empty(TOKENS, HIDDEN, device=dev, dtype=torch.bfloat16)
        G.gemm_swiglu(xa, model.w_gate[0], model.w_up[0], out=hh)
        out["gemm_swiglu_no_comm_ms"] = timed(lambda: G.gemm_swiglu(xa, model.w_gate[0], model.w_up[0], out=hh), n) / n
        G.gemm_bf16(hh, model.w_down[0], out=yy)
        out["gemm_down_no_comm_ms"] = timed(lambda: G.gemm_bf16(hh, model.w_down[0], out=yy), n) / n
        return out

    sampler = ClockSampler(local_rank) if ClockSampler is not None else _NoClocks()
    sampler.start()  # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(args.warmup):
        step()
    sampler.mark_begin()
    ms_total = timed(step, args.steps)
    sampler.mark_end()
    clocks = sampler.stop()
    if args.impl == "xccl":
        model.check_error()

    def all_ranks_ok() -> bool:
        """True when no rank's fused kernels have reported an expired wait (xccl arm; agreed over all ranks, so that
        every rank takes the same branch below)."""
        if args.impl != "xccl":
            return True
        bad = torch.tensor([1.0 if model.ws.error() else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        return bool(bad.item() == 0.0)

    # End-to-end figures. The device-timed number above stands on its own: should the overlapped input path fail on
    # some machine (its waits are bounded and end in an error word), the line is still printed, with the failure named.
    e2e_ms = wall_ms = full_ms = None
    e2e_note = None
    extra = {}
    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    if all_ranks_ok():
        barrier()
        t0 = time.perf_counter()
        e2e_ms = timed(e2e_step, args.steps)
        wall_ms = (time.perf_counter() - t0) * 1e3
        # second end-to-end figure: the same step with the whole output shard read back to pinned host memory
        for _ in range(3):
            full_step()
        model.wait_outputs()
        full_ms = timed(full_step, args.steps, after=lambda: torch.cuda.current_stream().wait_stream(
            model._d2h_stream if args.impl == "xccl" else (model._reader.stream if args.impl == "torch" else model._rd_stream)))
        model.wait_outputs()
    if not all_ranks_ok():
        e2e_ms = wall_ms = full_ms = None
        e2e_note = "a bounded wait expired in a fused kernel during the end-to-end steps (code %#x on rank 0)" % model.ws.error()
    elif args.impl == "xccl" and args.dtype == "bf16":
        ok, err = numerics_check()
        extra["numerics_ok"] = ok
        extra["numerics_max_abs_err"] = err
        extra["split"] = split_times()
        model.check_error()

    ms_per_step = ms_total / args.steps
    value = TOKENS / (ms_per_step * 1e-3)
    e2e_value = TOKENS / (max(e2e_ms, 1e-9) / args.steps * 1e-3) if e2e_ms is not None else None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": args.dtype if args.impl == "xccl" else "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": "llama-style MLP block (SwiGLU)", "global_batch": TOKENS, "seq_len": TOKENS,
                       "hidden": HIDDEN, "ffn": FFN, "parallelism": f"tp{world}",
                       "l2_policy": "operands larger than L2 (weights %.0f MB per GPU)" % (3 * HIDDEN * FFN // world * 2 / 1e6),
                       "step": "forward: allgather->GEMM+SwiGLU, GEMM->reduce-scatter"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": wall_ms / args.steps,
                    "h2d_bytes_per_step": TOKENS // world * HIDDEN * 2, "d2h_bytes_per_step": 4,
                    "result": "scalar metric of the output shard (mean of squares)"} if e2e_ms is not None else {"error": e2e_note},
            "e2e_full_output": {"value": TOKENS / (max(full_ms, 1e-9) / args.steps * 1e-3), "unit": "tokens/s",
                                "ms_per_step": full_ms / args.steps,
                                "h2d_bytes_per_step": TOKENS // world * HIDDEN * 2,
                                "d2h_bytes_per_step": TOKENS // world * HIDDEN * 2,
                                "result": "the whole output shard, read to pinned memory under the next step's kernels"}
            if full_ms is not None else {"error": e2e_note},
            **extra,
            "gpu_launches": launches_per_step * args.steps,
            "tflops_per_gpu": 6.0 * TOKENS * HIDDEN * FFN / world / (ms_per_step * 1e-3) / 1e12,
        }
        print(json.dumps(line), flush=True)
    if args.impl == "xccl":
        model.close()
        if oob is not None:
            oob.close()
    if ref_session is not None:
        model.close()
        ref_session.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
