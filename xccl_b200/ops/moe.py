"""Fused MoE dispatch / combine (``csrc/fused/moe.cu``) on torch tensors."""
from __future__ import annotations

import ctypes as C
from typing import Any, Sequence

import torch

from .. import _capi as K
from ..api import XcclError

_pp = C.POINTER(C.c_void_p)
K.optional("xccl_moe_ws_create", C.c_int, C.POINTER(K.Oob), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _pp)
K.optional("xccl_moe_ws_destroy", None, C.c_void_p)
K.optional("xccl_moe_dispatch", C.c_int, C.c_void_p, _pp, _pp, C.c_void_p)
K.optional("xccl_moe_combine", C.c_int, C.c_void_p, _pp, _pp, _pp, C.c_void_p)
K.optional("xccl_moe_ws_buffer", C.c_void_p, C.c_void_p, C.c_int, C.c_int)
K.optional("xccl_moe_ws_cap_rows", C.c_int, C.c_void_p)
K.optional("xccl_moe_ws_error", C.c_uint32, C.c_void_p)

BUF_RECV, BUF_EXPERT_OUT, BUF_EXPERT_ROWS, BUF_ROW_SOURCE = range(4)


def _ptrs(ts: Sequence[torch.Tensor]):
    arr = (C.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("expected contiguous CUDA tensors")
        arr[i] = t.data_ptr()
    return arr


def _view(ptr: int, shape: tuple, dtype: torch.dtype, device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    typestr = {torch.bfloat16: "<i2", torch.int32: "<i4", torch.uint32: "<u4"}[dtype]

    class _Mem:
        __cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3}

    t = torch.as_tensor(_Mem(), device=device)
    return (t.view(torch.bfloat16) if dtype == torch.bfloat16 else t).view(shape)


class MoeWorkspace:
    """Buffers and state of the fused expert all-to-all for fixed (tokens, hidden, experts, top-k)."""

    def __init__(self, tokens: int, hidden: int, experts: int, topk: int, oob: Any = None, emu_ranks: int = 1,
                 cap_rows: int = 0):
        self.T, self.H, self.E, self.K = tokens, hidden, experts, topk
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.h = C.c_void_p()
        st = K.load().xccl_moe_ws_create(C.byref(oob.c) if oob is not None else None, emu_ranks, tokens, hidden,
                                         experts, topk, cap_rows, C.byref(self.h))
        if st != K.OK:
            raise XcclError(st, "xccl_moe_ws_create")
        self.tp = oob.size if oob is not None else emu_ranks
        self.n_local = 1 if oob is not None else emu_ranks
        self.cap_rows = int(K.load().xccl_moe_ws_cap_rows(self.h))

    def _buf(self, local: int, which: int) -> int:
        return int(K.load().xccl_moe_ws_buffer(self.h, local, which))

    def recv(self, local: int = 0) -> torch.Tensor:
        return _view(self._buf(local, BUF_RECV), (self.cap_rows, self.H), torch.bfloat16, self.device)

    def expert_out(self, local: int = 0) -> torch.Tensor:
        return _view(self._buf(local, BUF_EXPERT_OUT), (self.cap_rows, self.H), torch.bfloat16, self.device)

    def expert_rows(self, local: int = 0) -> torch.Tensor:
        return _view(self._buf(local, BUF_EXPERT_ROWS), (self.E // self.tp + 1,), torch.int32, self.device)

    def row_source(self, local: int = 0) -> torch.Tensor:
        return _view(self._buf(local, BUF_ROW_SOURCE), (self.cap_rows,), torch.int32, self.device)

    def dispatch(self, x: Sequence[torch.Tensor], ids: Sequence[torch.Tensor]) -> None:
        st = K.load().xccl_moe_dispatch(self.h, _ptrs(x), _ptrs(ids), torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_moe_dispatch")

    def combine(self, ids: Sequence[torch.Tensor], weights: Sequence[torch.Tensor], out: Sequence[torch.Tensor]) -> None:
        st = K.load().xccl_moe_combine(self.h, _ptrs(ids), _ptrs(weights), _ptrs(out),
                                       torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_moe_combine")

    def error(self) -> int:
        torch.cuda.synchronize()
        return int(K.load().xccl_moe_ws_error(self.h))

    def close(self) -> None:
        if self.h:
            K.load().xccl_moe_ws_destroy(self.h)
            self.h = C.c_void_p()
