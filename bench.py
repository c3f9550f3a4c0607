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
import statistics
import subprocess
import sys
import threading
import time
import uuid

TOKENS, HIDDEN, FFN = 8192, 8192, 28672
METRIC = "tp_mlp_step_tokens_per_s"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def mark_begin(self) -> None:
        self.t0 = time.monotonic()

    def mark_end(self) -> None:
        self.t1 = time.monotonic()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t0, t1 = getattr(self, "t0", 0.0), getattr(self, "t1", float("inf"))
        for ts, ln in self.lines:
            if ts < t0 or ts > t1 + 0.15:  # a sample printed just after the region was taken inside it
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args) -> None:
    """The reference (openucx/xccl) is an autotools C library that needs UCX and MPI; neither is in
    this image and it cannot be installed with pip, so there is no reference arm to run."""
    print(json.dumps({"impl": "reference",
                      "unavailable": "openucx/xccl is an autotools C library that requires UCX (configure.ac:92-95) "
                                     "and MPI for any multi-rank run; neither exists in this image and "
                                     "`pip install /root/reference` has no setup.py/pyproject.toml to build"}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="xccl", choices=["xccl", "reference", "torch"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_arm(args)
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
    if args.impl == "xccl":
        from xccl_b200.models.tp_mlp import TpMlp
        if world > 1:
            from xccl_b200.api import ShmOob
            key = [uuid.uuid4().hex[:12] if rank == 0 else None]
            dist.broadcast_object_list(key, src=0)
            oob = ShmOob(key[0], rank, world)
        model = TpMlp(TOKENS, HIDDEN, FFN, tp=world, rank=rank, oob=oob)
        x_dev = [torch.randn(TOKENS // world, HIDDEN, device=dev).to(torch.bfloat16)]
        x_pin = [torch.randn(TOKENS // world, HIDDEN).to(torch.bfloat16).pin_memory()]
        step = lambda: model.forward(x_dev)           # noqa: E731
        e2e_step = lambda: model.forward_from_host(x_pin)  # noqa: E731
        launches_per_step = 2
    else:
        from xccl_b200.models.tp_mlp import TorchTpMlp
        model = TorchTpMlp(TOKENS, HIDDEN, FFN, tp=world, rank=rank)
        xd = torch.randn(TOKENS // world, HIDDEN, device=dev).to(torch.bfloat16)
        xp = torch.randn(TOKENS // world, HIDDEN).to(torch.bfloat16).pin_memory()
        step = lambda: model.forward(xd)               # noqa: E731
        e2e_step = lambda: model.forward_from_host(xp)  # noqa: E731
        launches_per_step = 0

    def timed(fn, n: int) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    sampler = ClockSampler(local_rank)
    sampler.start()  # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(args.warmup):
        step()
    sampler.mark_begin()
    ms_total = timed(step, args.steps)
    sampler.mark_end()
    clocks = sampler.stop()
    if args.impl == "xccl":
        model.check_error()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_ms = timed(e2e_step, args.steps)
    wall_ms = (time.perf_counter() - t0) * 1e3
    if args.impl == "xccl":
        model.check_error()

    ms_per_step = ms_total / args.steps
    value = TOKENS / (ms_per_step * 1e-3)
    e2e_value = TOKENS / (max(e2e_ms, 1e-9) / args.steps * 1e-3)
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": "llama-style MLP block (SwiGLU)", "global_batch": TOKENS, "seq_len": TOKENS,
                       "hidden": HIDDEN, "ffn": FFN, "parallelism": f"tp{world}",
                       "l2_policy": "operands larger than L2 (weights %.0f MB per GPU)" % (3 * HIDDEN * FFN // world * 2 / 1e6),
                       "step": "forward: allgather->GEMM+SwiGLU, GEMM->reduce-scatter"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": wall_ms / args.steps,
                    "h2d_bytes_per_step": TOKENS // world * HIDDEN * 2, "d2h_bytes_per_step": 4},
            "gpu_launches": launches_per_step * args.steps,
            "tflops_per_gpu": 6.0 * TOKENS * HIDDEN * FFN / world / (ms_per_step * 1e-3) / 1e12,
        }
        print(json.dumps(line), flush=True)
    if args.impl == "xccl":
        model.close()
        if oob is not None:
            oob.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
