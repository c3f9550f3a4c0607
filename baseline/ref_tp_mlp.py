"""The tensor-parallel SwiGLU MLP block as a user of the reference library would run it:
collectives through the reference's NCCL team (``baseline/ref_api.py``), GEMMs through
``torch.matmul`` (cuBLAS). Nothing of ``xccl_b200`` is imported here.

The reference offers allgather, alltoall and allreduce on device buffers (its NCCL team,
``src/team_lib/nccl/xccl_nccl_collective.c``), no reduce-scatter and no bf16 reduction type. The
row-sharded sum after the down projection is therefore written the cheapest way its API allows:
an ``XCCL_ALLTOALL`` of the bf16 partial rows (each rank receives the ``tp`` partials of its own
row block, the same bytes on the wire as a reduce-scatter) followed by a local sum. An
``XCCL_ALLREDUCE`` in fp32 would move four times as many bytes.
"""
import ctypes as C

import torch

import ref_api as R


class RefTpMlp:
    def __init__(self, tokens: int, hidden: int, ffn: int, tp: int, rank: int, session: "R.RefSession", seed: int = 0):
        self.tokens, self.hidden, self.ffn, self.tp, self.rank, self.s = tokens, hidden, ffn, tp, rank, session
        dev = torch.device("cuda", torch.cuda.current_device())
        f_local, m_local = ffn // tp, tokens // tp
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + rank)
        mk = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.02).to(torch.bfloat16)  # noqa: E731
        self.w_gate, self.w_up, self.w_down = mk(f_local, hidden), mk(f_local, hidden), mk(hidden, f_local)
        self.x_shard = torch.empty(m_local, hidden, dtype=torch.bfloat16, device=dev)
        self.xg = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.part = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.recv = torch.empty(tp, m_local, hidden, dtype=torch.bfloat16, device=dev)
        # the reference takes the address of a cudaStream_t; the collectives run on torch's current stream
        self._stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        sp = C.addressof(self._stream)
        self.req_ag = self.req_a2a = None
        self._stage = self._rd_stream = None
        self._steps = 0
        if tp > 1:
            self.req_ag = session.collective(R.ALLGATHER, self.x_shard.data_ptr(), self.xg.data_ptr(),
                                             length=tokens * hidden * 2, stream_handle_ptr=sp)
            self.req_a2a = session.collective(R.ALLTOALL, self.part.data_ptr(), self.recv.data_ptr(),
                                              length=m_local * hidden * 2, stream_handle_ptr=sp)

    def forward(self, x_shard=None) -> torch.Tensor:
        if x_shard is not None and x_shard.data_ptr() != self.x_shard.data_ptr():
            self.x_shard.copy_(x_shard)
        if self.tp > 1:
            self.s.post(self.req_ag)
            x = self.xg
        else:
            x = self.x_shard
        h = torch.nn.functional.silu(x @ self.w_gate.t()) * (x @ self.w_up.t())
        if self.tp == 1:
            return h @ self.w_down.t()
        torch.matmul(h, self.w_down.t(), out=self.part)
        self.s.post(self.req_a2a)
        return torch.sum(self.recv, dim=0, dtype=torch.float32).to(torch.bfloat16)

    def forward_from_host(self, x_pinned: torch.Tensor) -> torch.Tensor:
        self.x_shard.copy_(x_pinned, non_blocking=True)
        y = self.forward()
        return torch.linalg.vector_norm(y, dtype=torch.float32).cpu().square() / y.numel()

    def forward_from_host_full(self, x_pinned: torch.Tensor, y_pinned: list) -> None:
        """The step with the whole output shard read back to pinned memory (two buffers, the read of step i on a
        copy stream under the kernels of step i+1: the same overlap every arm of the benchmark uses)."""
        if self._stage is None:
            like = torch.empty(self.tokens // self.tp, self.hidden, dtype=torch.bfloat16, device=self.x_shard.device)
            self._stage = [like, torch.empty_like(like)]
            self._rd_stream = torch.cuda.Stream()
            self._free = [torch.cuda.Event(), torch.cuda.Event()]
        k = self._steps & 1
        self._steps += 1
        main = torch.cuda.current_stream()
        main.wait_event(self._free[k])
        self.x_shard.copy_(x_pinned, non_blocking=True)
        self._stage[k].copy_(self.forward(), non_blocking=True)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(self._rd_stream):
            self._rd_stream.wait_event(done)
            y_pinned[k].copy_(self._stage[k], non_blocking=True)
            self._free[k].record(self._rd_stream)

    def wait_outputs(self) -> None:
        if self._rd_stream is not None:
            self._rd_stream.synchronize()

    def close(self) -> None:
        torch.cuda.synchronize()
        for r in (self.req_ag, self.req_a2a):
            if r is not None:
                self.s.finalize(r)
        self.req_ag = self.req_a2a = None
