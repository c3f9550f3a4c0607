"""Pipeline-parallel send / receive on NCCL point-to-point (``xccl_p2p_*`` in ``csrc/tl/nccl/nccl_tl.cc``).

The Teams API of the reference has no user-visible send/recv (README.md:14 lists it as a goal); pipeline
stages need one, and NCCL's own p2p over NVLink is the transport for it here. All calls are stream-ordered:
a stage enqueues its receive, its compute and its send on streams and never blocks the host.

    comm = P2PComm(oob)                       # collective over the ranks of `oob`
    with comm.group():                        # one rank sends AND receives: group them, as with NCCL
        comm.recv(act_in, src=stage - 1, stream=s)
        comm.send(act_out, dst=stage + 1, stream=s)

``overlapped_stage_step`` shows the intended use: the activation for micro-batch i+1 is received on a
side stream while micro-batch i is being computed.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import Any, Callable, Optional

import torch

from .. import _capi as K
from ..api import XcclError

K.optional("xccl_p2p_comm_create", C.c_int, C.POINTER(K.Oob), C.POINTER(C.c_void_p))
K.optional("xccl_p2p_comm_destroy", None, C.c_void_p)
K.optional("xccl_p2p_send", C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p)
K.optional("xccl_p2p_recv", C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p)
K.optional("xccl_p2p_group_start", C.c_int)
K.optional("xccl_p2p_group_end", C.c_int)


def _stream(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


class P2PComm:
    def __init__(self, oob: Any):
        self.rank, self.size = oob.rank, oob.size
        self.h = C.c_void_p()
        st = K.load().xccl_p2p_comm_create(C.byref(oob.c), C.byref(self.h))
        if st != K.OK:
            raise XcclError(st, "xccl_p2p_comm_create")

    def send(self, t: torch.Tensor, dst: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        if not t.is_contiguous() or not t.is_cuda:
            raise ValueError("expected a contiguous CUDA tensor")
        st = K.load().xccl_p2p_send(self.h, t.data_ptr(), t.numel() * t.element_size(), dst, _stream(stream))
        if st != K.OK:
            raise XcclError(st, "xccl_p2p_send")

    def recv(self, t: torch.Tensor, src: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        if not t.is_contiguous() or not t.is_cuda:
            raise ValueError("expected a contiguous CUDA tensor")
        st = K.load().xccl_p2p_recv(self.h, t.data_ptr(), t.numel() * t.element_size(), src, _stream(stream))
        if st != K.OK:
            raise XcclError(st, "xccl_p2p_recv")

    @contextlib.contextmanager
    def group(self):
        if K.load().xccl_p2p_group_start() != K.OK:
            raise XcclError(K.ERR_NO_MESSAGE, "xccl_p2p_group_start")
        try:
            yield self
        finally:
            if K.load().xccl_p2p_group_end() != K.OK:
                raise XcclError(K.ERR_NO_MESSAGE, "xccl_p2p_group_end")

    def close(self) -> None:
        if self.h:
            K.load().xccl_p2p_comm_destroy(self.h)
            self.h = C.c_void_p()


def overlapped_stage_step(comm: P2PComm, stage_fn: Callable[[torch.Tensor], torch.Tensor], micro_batches: int,
                          act_shape: tuple, dtype: torch.dtype = torch.bfloat16,
                          first_input: Optional[Callable[[int], torch.Tensor]] = None) -> list:
    """Runs `micro_batches` forward micro-batches through this rank's pipeline stage (stage index = rank).

    Stage 0 takes its inputs from `first_input(i)`; every other stage receives activation i+1 on a side stream
    while it computes micro-batch i; every stage but the last sends its output on a second side stream. Two
    receive buffers alternate. Returns the outputs of the last stage (empty list elsewhere)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    stage, last = comm.rank, comm.size - 1
    compute = torch.cuda.current_stream()
    rx, tx = torch.cuda.Stream(), torch.cuda.Stream()
    bufs = [torch.empty(act_shape, dtype=dtype, device=dev) for _ in range(2)]
    arrived = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    outs, sends = [], []

    def post_recv(i: int) -> None:
        b = i % 2
        if i >= 2:
            rx.wait_event(consumed[b])          # the buffer's previous micro-batch has been read
        comm.recv(bufs[b], src=stage - 1, stream=rx)
        arrived[b].record(rx)

    if stage > 0:
        post_recv(0)
    for i in range(micro_batches):
        b = i % 2
        if stage > 0:
            if i + 1 < micro_batches:
                post_recv(i + 1)                # overlaps with the compute of micro-batch i
            compute.wait_event(arrived[b])
            x = bufs[b]
        else:
            x = first_input(i)
        y = stage_fn(x)
        if stage > 0:
            consumed[b].record(compute)
        if stage < last:
            done = torch.cuda.Event()
            done.record(compute)
            tx.wait_event(done)
            comm.send(y, dst=stage + 1, stream=tx)
            sends.append(y)                     # keep alive until the send stream is done
        else:
            outs.append(y)
    tx.synchronize()
    compute.synchronize()
    return outs
