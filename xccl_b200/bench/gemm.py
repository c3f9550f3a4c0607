"""GEMM micro-benchmark of the tcgen05 kernels against cuBLAS (``torch.matmul``) on one GPU.

    python -m xccl_b200.bench.gemm [--shapes 8192x8192x8192,8192x7168x8192] [--iters 10] [--kinds bf16,swiglu,fp8]

Device time from CUDA events around ``iters`` back-to-back launches after 3 warm-up launches; the
operands of the default shapes are larger than the 126 MB L2, and a 256 MB buffer is rewritten
between the implementations. One JSON line per (kind, shape). ``--no-cublas`` skips the library
arm (used for profiler captures of a single kernel).
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import gemm


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--shapes", default="8192x7168x8192,8192x8192x3584,8192x8192x8192")
    ap.add_argument("--kinds", default="bf16,swiglu,fp8")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-cublas", action="store_true")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for shape in a.shapes.split(","):
        M, N, K = (int(v) for v in shape.lower().split("x"))
        x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        flops = 2.0 * M * N * K
        for kind in a.kinds.split(","):
            row = {"kind": kind, "M": M, "N": N, "K": K, "iters": a.iters}
            if kind == "bf16":
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                ms = _time(lambda: gemm.gemm_bf16(x, w, out), a.iters)
                lib = None if a.no_cublas else (flush.zero_(), _time(lambda: torch.matmul(x, w.t(), out=out), a.iters))[1]
            elif kind == "swiglu":
                # N columns = N/2 gate + N/2 up; output [M, N/2]
                wg, wu = w[: N // 2].contiguous(), w[N // 2:].contiguous()
                out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=dev)
                ms = _time(lambda: gemm.gemm_swiglu(x, wg, wu, out), a.iters)
                lib = None if a.no_cublas else (flush.zero_(), _time(
                    lambda: torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t()), a.iters))[1]
            elif kind == "fp8":
                if K % 128 or N % 128:
                    continue
                a8, sa = gemm.quantize_act_1x128(x.float())
                b8, sb = gemm.quantize_weight_128x128(w.float())
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                ms = _time(lambda: gemm.gemm_fp8_blockscaled(a8, sa, b8, sb, out), a.iters)
                lib = None  # the library arm of this row is the bf16 cuBLAS number of the same shape
            else:
                raise SystemExit(f"unknown kind {kind}")
            row.update(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1), error_word=gemm.last_error())
            if lib is not None:
                row.update(lib_ms=round(lib, 4), lib_tflops=round(flops / lib / 1e9, 1), ratio_vs_lib=round(lib / ms, 3))
            print(json.dumps(row), flush=True)
            flush.zero_()


if __name__ == "__main__":
    main()
