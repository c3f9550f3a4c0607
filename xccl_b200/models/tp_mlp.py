"""Tensor-parallel Llama-style MLP block on the fused kernels.

``y = W_down (silu(W_gate x) * W_up x)`` with the FFN dimension split over ``tp`` ranks and the
activations sharded by tokens (sequence parallel): the up/gate projection is allgather->GEMM with
the SwiGLU fused into the epilogue, the down projection is GEMM->reduce-scatter. Each is ONE
kernel of ``csrc/fused/tp_gemm.cu``; with ``tp == 1`` the same kernels run without communication.

``TorchTpMlp`` is the same block written with torch collectives and matmuls (NCCL + cuBLAS); it
is the comparison point, not a fallback.
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch

from ..ops.tp import TpWorkspace


def _init_weights(tokens: int, hidden: int, ffn: int, tp: int, rank: int, device, seed: int = 0):
    """Random-init shards ~N(0, 0.02) of the named architecture; the same seed gives every
    implementation the same full weights."""
    f_local = ffn // tp
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    mk = lambda *s: (torch.randn(*s, device=device, generator=g) * 0.02).to(torch.bfloat16)  # noqa: E731
    return mk(f_local, hidden), mk(f_local, hidden), mk(hidden, f_local)


class TpMlp:
    """One rank of the block (or, with ``oob=None`` and ``tp > 1``, all ranks emulated on one GPU)."""

    def __init__(self, tokens: int, hidden: int, ffn: int, tp: int = 1, rank: int = 0, oob: Any = None,
                 seed: int = 0, emulate: bool = False):
        if ffn % tp or tokens % tp:
            raise ValueError("tokens and ffn must divide by tp")
        self.tokens, self.hidden, self.ffn, self.tp, self.rank = tokens, hidden, ffn, tp, rank
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.emulate = emulate or (oob is None and tp > 1)
        self.ws = TpWorkspace(tokens, hidden, oob=None if self.emulate else oob, emu_ranks=tp if self.emulate else 1)
        self.n_local = self.ws.n_local
        ranks = range(tp) if self.emulate else [rank]
        ws_ = [_init_weights(tokens, hidden, ffn, tp, r, self.device, seed) for r in ranks]
        self.w_gate = [w[0] for w in ws_]
        self.w_up = [w[1] for w in ws_]
        self.w_down = [w[2] for w in ws_]
        f_local = ffn // tp
        self.h = [torch.empty(tokens, f_local, dtype=torch.bfloat16, device=self.device) for _ in ranks]
        self.y = [torch.empty(tokens // tp, hidden, dtype=torch.bfloat16, device=self.device) for _ in ranks]
        self.x_shards = [self.ws.x_shard(i) for i in range(self.n_local)]
        self.launches = 0
        # forward_from_host overlaps the host->device copy of the input with the first kernel: the kernels are
        # launched first, the chunks follow, and the local rows are walked in growing groups (measured on the
        # 8192 x 8192 x 28672 block on one GPU: 10.2 ms per end-to-end step with copy-then-launch, 9.1 ms with the
        # overlapped copy, 8.8 ms with the growing groups; kernels alone 8.6 ms). XCCL_TP_H2D_OVERLAP=0 turns it off.
        self.overlap_h2d = os.environ.get("XCCL_TP_H2D_OVERLAP") != "0"
        # phases over all shards while every rank's input arrives (copy CTAs, 4 ranks and more); off: no gain measured
        self.h2d_phases = os.environ.get("XCCL_TP_H2D_PHASES", "n").lower() in ("y", "yes", "1", "on", "true")
        self._copy_stream = None
        self._y_alt = None
        self._d2h_stream = None
        self._full_steps = 0

    def forward(self, x_shards: Optional[list] = None) -> list:
        """x_shards: one [tokens/tp, hidden] bf16 tensor per local rank, or None when the input was
        already written into ``self.x_shards``. Returns the [tokens/tp, hidden] output shards."""
        if x_shards is not None:
            for dst, src in zip(self.x_shards, x_shards):
                dst.copy_(src, non_blocking=True)
        self.ws.ag_gemm_swiglu(self.w_gate, self.w_up, self.h)
        self.ws.gemm_rs(self.h, self.w_down, self.y)
        self.launches += 2
        return self.y

    def _forward_with_input(self, x_pinned: list, ramp: bool = True) -> list:
        """The block on input shards that are still in pinned host memory. Overlapped form: the kernels are launched
        first and wait for rows; the copy is enqueued right after on its own stream, chunk by chunk (two driver calls
        per chunk, whose host time would otherwise precede the launch)."""
        if not self.overlap_h2d:
            for dst, src in zip(self.x_shards, x_pinned):
                dst.copy_(src, non_blocking=True)
            return self.forward()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream()
        self.ws.h2d_expect(self._copy_stream, (2 if self.h2d_phases else 1) if ramp else 0)
        try:
            y = self.forward()
        finally:
            self.ws.h2d_issue(x_pinned, self._copy_stream)   # a launched kernel always gets its rows
        return y

    def forward_from_host(self, x_pinned: list) -> torch.Tensor:
        """End-to-end step: host->device copy of this step's input shards from pinned memory,
        the block, and a device->host read of a scalar metric of the result."""
        y = self._forward_with_input(x_pinned)
        # mean of squares in ONE reduction kernel (fp32 accumulation), no fp32 copy of the output
        norm = torch.linalg.vector_norm(y[0], dtype=torch.float32).cpu()   # the device->host read of the step
        return norm.square() / y[0].numel()                                 # finished on the host

    def forward_from_host_full(self, x_pinned: list, y_pinned: list) -> None:
        """End-to-end step whose result is the whole output shard: the input arrives from pinned host memory, the
        [tokens/tp, hidden] output goes back to ``y_pinned[step parity]`` on a copy stream, so the read of step i
        overlaps the kernels of step i+1 (outputs alternate between two device buffers). ``wait_outputs()`` returns
        when every read issued so far has landed."""
        if self._y_alt is None:
            self._y_alt = [torch.empty_like(t) for t in self.y]
            self._d2h_stream = torch.cuda.Stream()
            self._y_free = [torch.cuda.Event(), torch.cuda.Event()]
        k = self._full_steps & 1
        self._full_steps += 1
        main = torch.cuda.current_stream()
        main.wait_event(self._y_free[k])           # the read of step i-2 has left this output buffer
        self.y, self._y_alt = self._y_alt, self.y
        y = self._forward_with_input(x_pinned, ramp=False)   # this copy runs under the previous step's second kernel
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(self._d2h_stream):
            self._d2h_stream.wait_event(done)
            for dst, src in zip(y_pinned[k], y):
                dst.copy_(src, non_blocking=True)
            self._y_free[k].record(self._d2h_stream)

    def wait_outputs(self) -> None:
        if self._d2h_stream is not None:
            self._d2h_stream.synchronize()

    def check_error(self) -> None:
        e = self.ws.error()
        if e:
            raise RuntimeError(f"a bounded wait expired inside a fused TP kernel (code {e:#x})")

    def close(self) -> None:
        self.ws.close()


class TpMlpFp8(TpMlp):
    """The same block on the fp8 tensor cores: activations quantised per row and 128 columns, weights per
    128 x 128 block (e4m3, fp32 scales). Per step: quantise the input shard into the gathered buffer,
    allgather->GEMM+SwiGLU (fp8 rows and scales travel together inside the kernel; its epilogue quantises the
    intermediate, which is written once, as fp8), GEMM->reduce-scatter. Three launches. With
    ``fuse_quant=False`` the intermediate is written as bf16 and quantised by a separate kernel (four launches)."""

    def __init__(self, *args, fuse_quant: bool = True, **kw):
        super().__init__(*args, **kw)
        self.fuse_quant = fuse_quant
        self.overlap_h2d = False   # the input is quantised by a kernel first: it is copied whole, then quantised
        from ..ops.gemm import quantize_weight_128x128
        from ..ops.tp import quantize_rows
        self._quantize_rows = quantize_rows
        qg = [quantize_weight_128x128(w) for w in self.w_gate]
        qu = [quantize_weight_128x128(w) for w in self.w_up]
        qd = [quantize_weight_128x128(w) for w in self.w_down]
        self.w_gate8, self.s_gate = [q[0] for q in qg], [q[1] for q in qg]
        self.w_up8, self.s_up = [q[0] for q in qu], [q[1] for q in qu]
        self.w_down8, self.s_down = [q[0] for q in qd], [q[1] for q in qd]
        f_local = self.ffn // self.tp
        n = self.n_local
        self.x_in = [torch.empty(self.tokens // self.tp, self.hidden, dtype=torch.bfloat16, device=self.device) for _ in range(n)]
        self.x_shards = self.x_in          # the bf16 input of the step; its fp8 form goes into the gathered buffer
        self.x8 = [self.ws.x8_shard(i) for i in range(n)]
        self.sx = [self.ws.sx_shard(i) for i in range(n)]
        self.h8 = [torch.empty(self.tokens, f_local, dtype=torch.float8_e4m3fn, device=self.device) for _ in range(n)]
        self.sh = [torch.empty(self.tokens, f_local // 128, dtype=torch.float32, device=self.device) for _ in range(n)]

    def forward(self, x_shards: Optional[list] = None) -> list:
        if x_shards is not None:
            for dst, src in zip(self.x_in, x_shards):
                dst.copy_(src, non_blocking=True)
        for i in range(self.n_local):
            self._quantize_rows(self.x_in[i], self.x8[i], self.sx[i])
        if self.fuse_quant:
            self.ws.ag_gemm_swiglu_fp8q(self.w_gate8, self.s_gate, self.w_up8, self.s_up, self.h8, self.sh)
        else:
            self.ws.ag_gemm_swiglu_fp8(self.w_gate8, self.s_gate, self.w_up8, self.s_up, self.h)
            for i in range(self.n_local):
                self._quantize_rows(self.h[i], self.h8[i], self.sh[i])
        self.ws.gemm_rs_fp8(self.h8, self.sh, self.w_down8, self.s_down, self.y)
        self.launches += 2 + (1 if self.fuse_quant else 2) * self.n_local
        return self.y


class TorchTpMlp:
    """The same block with torch.distributed collectives and torch matmuls."""

    def __init__(self, tokens: int, hidden: int, ffn: int, tp: int = 1, rank: int = 0, group=None, seed: int = 0):
        import torch.distributed as dist
        self.dist = dist
        self.tokens, self.hidden, self.ffn, self.tp, self.rank, self.group = tokens, hidden, ffn, tp, rank, group
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.w_gate, self.w_up, self.w_down = _init_weights(tokens, hidden, ffn, tp, rank, self.device, seed)
        self.xg = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=self.device)
        self.y = torch.empty(tokens // tp, hidden, dtype=torch.bfloat16, device=self.device)
        self.x_shard = torch.empty(tokens // tp, hidden, dtype=torch.bfloat16, device=self.device)

    def forward(self, x_shard: Optional[torch.Tensor] = None) -> torch.Tensor:
        x_shard = self.x_shard if x_shard is None else x_shard
        if self.tp > 1:
            self.dist.all_gather_into_tensor(self.xg, x_shard, group=self.group)
            x = self.xg
        else:
            x = x_shard
        h = torch.nn.functional.silu(x @ self.w_gate.t()) * (x @ self.w_up.t())
        part = h @ self.w_down.t()
        if self.tp > 1:
            self.dist.reduce_scatter_tensor(self.y, part, group=self.group)
            return self.y
        return part

    def forward_from_host(self, x_pinned: torch.Tensor) -> torch.Tensor:
        self.x_shard.copy_(x_pinned, non_blocking=True)
        y = self.forward()
        return torch.linalg.vector_norm(y, dtype=torch.float32).cpu().square() / y.numel()

    def forward_from_host_full(self, x_pinned: torch.Tensor, y_pinned: list) -> None:
        if getattr(self, "_reader", None) is None:
            self._reader = PipelinedOutputReader(self.y)
        self.x_shard.copy_(x_pinned, non_blocking=True)
        self._reader.read(self.forward(), y_pinned)

    def wait_outputs(self) -> None:
        if getattr(self, "_reader", None) is not None:
            self._reader.wait()


class PipelinedOutputReader:
    """The read-back of ``forward_from_host_full`` for an implementation whose forward returns a fresh or reused
    output tensor: the result is copied to a staging buffer in the main stream's order and read to pinned memory on
    a copy stream, two steps in flight. The comparison arms use it so that all arms overlap the same way."""

    def __init__(self, like: torch.Tensor):
        self.stage = [torch.empty_like(like), torch.empty_like(like)]
        self.stream = torch.cuda.Stream()
        self.free = [torch.cuda.Event(), torch.cuda.Event()]
        self.steps = 0

    def read(self, y: torch.Tensor, y_pinned: list) -> None:
        k = self.steps & 1
        self.steps += 1
        main = torch.cuda.current_stream()
        main.wait_event(self.free[k])
        self.stage[k].copy_(y, non_blocking=True)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(done)
            y_pinned[k].copy_(self.stage[k], non_blocking=True)
            self.free[k].record(self.stream)

    def wait(self) -> None:
        self.stream.synchronize()


def reference_forward_fp32(x_full: torch.Tensor, w_gate_full: torch.Tensor, w_up_full: torch.Tensor,
                           w_down_full: torch.Tensor) -> torch.Tensor:
    """Plain fp32 statement of the block on full (unsharded) tensors: the numerics oracle."""
    x = x_full.float()
    h = torch.nn.functional.silu(x @ w_gate_full.float().t()) * (x @ w_up_full.float().t())
    h = h.to(torch.bfloat16).float()  # the fused kernels round h to bf16 between the two GEMMs
    return h @ w_down_full.float().t()
