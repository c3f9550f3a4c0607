"""Small, self-terminating cases of each fused kernel for counter captures and device timing on ONE GPU.

    python -m xccl_b200.bench.profile_cases --case ag_gemm [--iters 3]

Each case sets up a small problem (operands larger than L2 where DRAM figures matter, a few hundred MB on the
device at most), runs the kernel `iters` times after one warm-up, checks the kernels' error words and prints one
JSON line with the device time per launch (CUDA events) and the algorithmic bytes / FLOPs of the case. Multi-rank
kernels run with their ranks emulated inside one cooperative launch. The same command line is what a profiler
wraps: `ncu --clock-control none -k regex:<kernel> -c 2 ... python -m xccl_b200.bench.profile_cases --case <case>`.

Cases: gemm, gemm_swiglu, gemm_fp8, ag_gemm, gemm_rs, ag_gemm_fp8, gemm_rs_fp8 (tp=2 emulated), moe_dispatch,
moe_combine (4 emulated ranks), allreduce_one_shot, allreduce_two_shot, allreduce_direct, alltoall_push,
alltoall_pull, allgather_pull, bcast_pull, alltoallv (4 emulated ranks).
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _capi as K


def _timed(fn, iters: int) -> float:
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
    ap.add_argument("--case", required=True)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    out = {"case": a.case, "iters": a.iters}
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)  # noqa: E731

    if a.case in ("gemm", "gemm_swiglu", "gemm_fp8"):
        from ..ops import gemm as G
        M, N, Kd = 4096, 8192, 4096
        x = rnd(M, Kd).to(bf)
        if a.case == "gemm":
            w, c = (rnd(N, Kd) * 0.02).to(bf), torch.empty(M, N, dtype=bf, device=dev)
            ms = _timed(lambda: G.gemm_bf16(x, w, out=c), a.iters)
            out.update(flops=2.0 * M * N * Kd, bytes=2.0 * (M * Kd + N * Kd + M * N))
        elif a.case == "gemm_swiglu":
            wg, wu = (rnd(N // 2, Kd) * 0.02).to(bf), (rnd(N // 2, Kd) * 0.02).to(bf)
            c = torch.empty(M, N // 2, dtype=bf, device=dev)
            ms = _timed(lambda: G.gemm_swiglu(x, wg, wu, out=c), a.iters)
            out.update(flops=2.0 * M * N * Kd, bytes=2.0 * (M * Kd + N * Kd + M * N // 2))
        else:
            a8, sa = G.quantize_act_1x128(x.float())
            b8, sb = G.quantize_weight_128x128(rnd(N, Kd) * 0.02)
            c = torch.empty(M, N, dtype=bf, device=dev)
            ms = _timed(lambda: G.gemm_fp8_blockscaled(a8, sa, b8, sb, out=c), a.iters)
            out.update(flops=2.0 * M * N * Kd, bytes=1.0 * (M * Kd + N * Kd) + 2.0 * M * N)
        out["gemm_error_word"] = G.last_error()
    elif a.case in ("ag_gemm", "gemm_rs", "ag_gemm_fp8", "gemm_rs_fp8"):
        from ..models.tp_mlp import TpMlp, TpMlpFp8
        tokens, hidden, ffn, tp = 4096, 4096, 8192, 2
        fp8 = a.case.endswith("fp8")
        mlp = (TpMlpFp8 if fp8 else TpMlp)(tokens, hidden, ffn, tp=tp, emulate=True)
        xs = [rnd(tokens // tp, hidden).to(bf) for _ in range(tp)]
        mlp.forward(xs)
        torch.cuda.synchronize()
        f_local = ffn // tp
        if a.case == "ag_gemm":
            ms = _timed(lambda: mlp.ws.ag_gemm_swiglu(mlp.w_gate, mlp.w_up, mlp.h), a.iters)
        elif a.case == "gemm_rs":
            ms = _timed(lambda: mlp.ws.gemm_rs(mlp.h, mlp.w_down, mlp.y), a.iters)
        elif a.case == "ag_gemm_fp8":
            ms = _timed(lambda: mlp.ws.ag_gemm_swiglu_fp8q(mlp.w_gate8, mlp.s_gate, mlp.w_up8, mlp.s_up, mlp.h8, mlp.sh), a.iters)
        else:
            ms = _timed(lambda: mlp.ws.gemm_rs_fp8(mlp.h8, mlp.sh, mlp.w_down8, mlp.s_down, mlp.y), a.iters)
        es = 1 if fp8 else 2
        if a.case.startswith("ag_gemm"):
            out.update(flops=tp * 2.0 * tokens * 2 * f_local * hidden,
                       bytes=tp * (es * (tokens * hidden + 2 * f_local * hidden) + es * tokens * f_local),
                       peer_bytes=tp * es * (tokens - tokens // tp) * hidden)
        else:
            out.update(flops=tp * 2.0 * tokens * hidden * f_local,
                       bytes=tp * (es * (tokens * f_local + hidden * f_local) + 2 * tokens * hidden),
                       peer_bytes=tp * 2 * (tokens - tokens // tp) * hidden)
        out["ranks_emulated"] = tp
        mlp.check_error()
        mlp.close()
    elif a.case in ("moe_dispatch", "moe_combine"):
        from ..ops.moe import MoeWorkspace
        n, T, H, E, Kk = 4, 512, 7168, 64, 8
        ws = MoeWorkspace(T, H, E, Kk, emu_ranks=n, cap_rows=n * T * Kk)
        cg = torch.Generator().manual_seed(2)
        xs = [torch.randn(T, H, generator=cg).to(bf).to(dev) for _ in range(n)]
        ids = [torch.stack([torch.randperm(E, generator=cg)[:Kk] for _ in range(T)]).to(torch.int32).to(dev) for _ in range(n)]
        wts = [torch.softmax(torch.randn(T, Kk, generator=cg), -1).to(dev) for _ in range(n)]
        ys = [torch.empty(T, H, dtype=bf, device=dev) for _ in range(n)]
        ws.dispatch(xs, ids)
        torch.cuda.synchronize()
        for r in range(n):
            rows = int(ws.expert_rows(r)[-1].item())
            ws.expert_out(r)[:rows].copy_(ws.recv(r)[:rows])
        if a.case == "moe_dispatch":
            ms = _timed(lambda: ws.dispatch(xs, ids), a.iters)
        else:
            ms = _timed(lambda: ws.combine(ids, wts, ys), a.iters)
        out.update(bytes=2.0 * n * T * Kk * H * 2, ranks_emulated=n, error_word=ws.error())
        ws.close()
    else:
        from ..ops.emu import EmuWorld
        n = 4
        w = EmuWorld(n, 64 << 20)
        if a.case.startswith("allreduce"):
            alg = {"allreduce_one_shot": K.NVLINK_ALG_ONE_SHOT, "allreduce_two_shot": K.NVLINK_ALG_TWO_SHOT,
                   "allreduce_direct": K.NVLINK_ALG_DIRECT}[a.case]
            count = (64 << 10) if alg == K.NVLINK_ALG_ONE_SHOT else (8 << 20)   # fp32 elements: 256 KiB / 32 MiB
            srcs = [rnd(count) for _ in range(n)]
            dsts = [torch.empty_like(s) for s in srcs]
            ms = _timed(lambda: w.allreduce(srcs, dsts, alg=alg, scale=1.0 / n), a.iters)
            out.update(bytes=1.0 * n * count * 4, ranks_emulated=n)
        elif a.case in ("alltoall_push", "alltoall_pull", "allgather_pull", "bcast_pull"):
            per = (16 << 10) if a.case == "alltoall_push" else (4 << 20)
            if a.case.startswith("alltoall"):
                srcs = [torch.randint(0, 255, (per * n,), dtype=torch.uint8, device=dev) for _ in range(n)]
                dsts = [torch.empty_like(s) for s in srcs]
                alg = K.NVLINK_ALG_ONE_SHOT if a.case.endswith("push") else K.NVLINK_ALG_TWO_SHOT
                ms = _timed(lambda: w.alltoall(srcs, dsts, alg=alg), a.iters)
            elif a.case == "allgather_pull":
                srcs = [torch.randint(0, 255, (per,), dtype=torch.uint8, device=dev) for _ in range(n)]
                dsts = [torch.empty(per * n, dtype=torch.uint8, device=dev) for _ in range(n)]
                ms = _timed(lambda: w.allgather(srcs, dsts), a.iters)
            else:
                srcs = [torch.randint(0, 255, (per * n,), dtype=torch.uint8, device=dev) for _ in range(n)]
                dsts = [torch.empty_like(s) for s in srcs]
                ms = _timed(lambda: w.bcast(srcs, dsts, 1), a.iters)
            out.update(bytes=1.0 * n * per * n, ranks_emulated=n)
        elif a.case == "alltoallv":
            per = 1 << 20
            sc = [[per + 4096 * ((s + d) % n) for d in range(n)] for s in range(n)]
            srcs, dsts, metas = [], [], []
            for r in range(n):
                rc = [sc[s][r] for s in range(n)]
                srcs.append(torch.randint(0, 255, (sum(sc[r]),), dtype=torch.uint8, device=dev))
                dsts.append(torch.empty(sum(rc), dtype=torch.uint8, device=dev))
                metas.append(torch.tensor(sc[r] + [sum(sc[r][:d]) for d in range(n)] + rc + [sum(rc[:s]) for s in range(n)],
                                          dtype=torch.int32, device=dev))
            ms = _timed(lambda: w.alltoallv(srcs, dsts, metas, max(s.numel() for s in srcs)), a.iters)
            out.update(bytes=1.0 * sum(sum(x) for x in sc), ranks_emulated=n)
        else:
            raise SystemExit(f"unknown case {a.case}")
        w.close()
    out["ms_per_launch"] = round(ms, 5)
    if "flops" in out:
        out["tflops"] = round(out["flops"] / (ms * 1e-3) / 1e12, 1)
    if "bytes" in out:
        out["algorithmic_gbs"] = round(out["bytes"] / (ms * 1e-3) / 1e9, 1)
    with open("/proc/self/maps") as f:
        out["native_loaded"] = "libxccl.so" in f.read()
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
