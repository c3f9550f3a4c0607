"""MoE expert all-to-all benchmark: fused dispatch + combine kernels against the same exchange
done with alltoallv on the NCCL team plus torch permutation ops.

    python -m xccl_b200.bench.moe --gpus 8 [--tokens 4096 --hidden 7168 --experts 256 --topk 8]

Config of the headline run: 4096 tokens per rank, hidden 7168 (bf16), 256 experts sharded over
the ranks, top-8 routing with expert ids uniform at random (seed 2), gate weights from a softmax
over N(0,1) logits. "Experts" are the identity, so the timed work is exactly dispatch + combine.
Device-timed with CUDA events, maximum over ranks. One JSON line per implementation on stdout.
"""
from __future__ import annotations

import argparse
import json
import struct

import torch

from .. import _capi as K
from ..utils.launch import run_ranks


def _rank_main(rank: int, size: int, job: str, o: dict) -> list:
    from ..api import Context, Lib, ShmOob, Team
    from ..ops.moe import MoeWorkspace
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    T, H, E, Kk = o["tokens"], o["hidden"], o["experts"], o["topk"]
    EL = E // size
    oob = ShmOob(job, rank, size)
    g = torch.Generator(device="cpu").manual_seed(2 * 1000 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    ids = torch.stack([torch.randperm(E, generator=g)[:Kk] for _ in range(T)]).to(torch.int32).to(dev)
    w = torch.softmax(torch.randn(T, Kk, generator=g), -1).to(dev)
    out = []

    def max_ranks(v: float) -> float:
        vals = oob.allgather_bytes(struct.pack("d", v))
        return max(struct.unpack("d", b)[0] for b in vals)

    def timed(fn, iters: int) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        oob.allgather_bytes(b"x")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_ranks(e0.elapsed_time(e1) / iters)

    from .clocks import ClockSampler
    sampler = ClockSampler(rank)
    sampler.start()
    sampler.mark_begin()
    # ---- fused kernels
    ws = MoeWorkspace(T, H, E, Kk, oob=oob, cap_rows=min(size * T * Kk, 2 * T * Kk))
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    rows_view = ws.expert_rows(0)

    # identity expert = EXPERT_OUT must hold RECV: do that copy once outside the timed region by
    # timing dispatch and combine separately and in sequence.
    def dispatch_only():
        ws.dispatch([x], [ids])

    ws.dispatch([x], [ids])
    torch.cuda.synchronize()
    total_rows = int(rows_view[-1].item())
    ws.expert_out(0)[:total_rows].copy_(ws.recv(0)[:total_rows])

    def combine_only():
        ws.combine([ids], [w], [y])

    t_d = timed(dispatch_only, o["iters"])
    # slot order inside an expert depends on arrival order, so the identity expert copies the rows of
    # the LAST dispatch: combine then reads outputs that match the slots it was told about
    torch.cuda.synchronize()
    oob.allgather_bytes(b"x")
    ws.expert_out(0)[:total_rows].copy_(ws.recv(0)[:total_rows])
    torch.cuda.synchronize()
    oob.allgather_bytes(b"x")
    t_c = timed(combine_only, o["iters"])
    err = ws.error()
    want = (x.float() * w.sum(1, keepdim=True)).to(torch.bfloat16)
    ok = bool(torch.allclose(y.float(), want.float(), rtol=3e-2, atol=3e-2))
    routed_bytes = T * Kk * H * 2
    remote = routed_bytes * (size - 1) / size
    if rank == 0:
        out.append({"impl": "xccl_fused", "gpus": size, "dispatch_ms": round(t_d, 4), "combine_ms": round(t_c, 4),
                    "total_ms": round(t_d + t_c, 4), "error_word": err, "numerics_ok": ok,
                    "remote_bytes_each_way": remote, "dispatch_gbs": round(remote / (t_d * 1e-3) / 1e9, 1),
                    "combine_gbs": round(remote / (t_c * 1e-3) / 1e9, 1), "rows_received": total_rows})
    ws.close()

    # ---- baseline: NCCL-team alltoallv + torch permutation (what a user of the reference would write)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_NCCL | K.TL_UCX)
    team = Team(ctx)
    sh = torch.cuda.current_stream().cuda_stream
    flat = ids.flatten().long()
    cnt_buf = torch.zeros(size, dtype=torch.int32, device=dev)
    rcnt_buf = torch.zeros(size, dtype=torch.int32, device=dev)
    cnt_req = team.alltoall(cnt_buf, rcnt_buf, bytes_per_peer=4, stream=sh)
    state = {}

    def base_dispatch():
        order = torch.argsort(flat, stable=True)            # by expert, hence by destination rank
        send = x[order // Kk]                                # permuted copy of the routed rows
        cnt_buf.copy_(torch.bincount(flat // EL, minlength=size).to(torch.int32))
        cnt_req.post().wait()
        sc = cnt_buf.cpu().tolist()                          # host round trip for the counts
        rc = rcnt_buf.cpu().tolist()
        sd = [sum(sc[:i]) * H for i in range(size)]
        rd = [sum(rc[:i]) * H for i in range(size)]
        recv = torch.empty(sum(rc), H, dtype=torch.bfloat16, device=dev)
        req = team.alltoallv(send, [c * H for c in sc], sd, recv, [c * H for c in rc], rd, stream=sh)
        req.post().wait()
        req.finalize()
        state.update(order=order, recv=recv, sc=sc, rc=rc, sd=sd, rd=rd)

    def base_combine():
        back = torch.empty(T * Kk, H, dtype=torch.bfloat16, device=dev)
        req = team.alltoallv(state["recv"], [c * H for c in state["rc"]], state["rd"], back,
                             [c * H for c in state["sc"]], state["sd"], stream=sh)
        req.post().wait()
        req.finalize()
        un = torch.empty_like(back)
        un[state["order"]] = back
        yb = (un.view(T, Kk, H).float() * w[:, :, None]).sum(1).to(torch.bfloat16)
        state["y"] = yb

    tb_d = timed(base_dispatch, o["iters"])
    tb_c = timed(base_combine, o["iters"])
    okb = bool(torch.allclose(state["y"].float(), want.float(), rtol=3e-2, atol=3e-2))
    if rank == 0:
        out.append({"impl": "nccl_alltoallv_torch", "gpus": size, "dispatch_ms": round(tb_d, 4),
                    "combine_ms": round(tb_c, 4), "total_ms": round(tb_d + tb_c, 4), "numerics_ok": okb})
    cnt_req.finalize()
    sampler.mark_end()
    if rank == 0:
        out.append({"clocks_whole_run": sampler.stop()})
    team.close(); ctx.close(); lib.close(); oob.close()
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    res = run_ranks(_rank_main, a.gpus, vars(a), timeout=900, start_method="spawn")
    for r in res[0]:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
