"""Fused tensor-parallel MLP operations (``csrc/fused/tp_mlp.cu``) on torch tensors.

``TpWorkspace`` owns the symmetric buffers. With ``oob=None`` it emulates ``emu_ranks`` ranks on
the current device (every call takes one tensor per rank and is one cooperative launch); with an
out-of-band provider it is one rank of a real group (lists have one entry).
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Optional, Sequence

import torch

from .. import _capi as K
from ..api import XcclError

_pp = C.POINTER(C.c_void_p)
K.optional("xccl_tp_ws_create", C.c_int, C.POINTER(K.Oob), C.c_int, C.c_int, C.c_int, C.c_int, _pp)
K.optional("xccl_tp_ws_destroy", None, C.c_void_p)
K.optional("xccl_tp_ws_x_shard", C.c_void_p, C.c_void_p, C.c_int)
K.optional("xccl_tp_ws_x_full", C.c_void_p, C.c_void_p, C.c_int)
K.optional("xccl_tp_ws_error", C.c_uint32, C.c_void_p)
K.optional("xccl_tp_ag_gemm_swiglu", C.c_int, C.c_void_p, _pp, _pp, _pp, C.c_int, C.c_void_p)
K.optional("xccl_tp_gemm_rs", C.c_int, C.c_void_p, _pp, _pp, _pp, C.c_int, C.c_void_p)
K.optional("xccl_tp_h2d_begin", C.c_int, C.c_void_p, _pp, C.c_void_p)
K.optional("xccl_tp_h2d_expect", C.c_int, C.c_void_p, C.c_void_p, C.c_int)
K.optional("xccl_tp_h2d_issue", C.c_int, C.c_void_p, _pp, C.c_void_p)
K.optional("xccl_tp_quantize_rows", C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p)
K.optional("xccl_tp_ws_x8_shard", C.c_void_p, C.c_void_p, C.c_int)
K.optional("xccl_tp_ws_sx_shard", C.c_void_p, C.c_void_p, C.c_int)
K.optional("xccl_tp_ag_gemm_swiglu_fp8", C.c_int, C.c_void_p, _pp, _pp, _pp, _pp, _pp, C.c_int, C.c_void_p)
K.optional("xccl_tp_ag_gemm_swiglu_fp8q", C.c_int, C.c_void_p, _pp, _pp, _pp, _pp, _pp, _pp, C.c_int, C.c_void_p)
K.optional("xccl_tp_gemm_rs_fp8", C.c_int, C.c_void_p, _pp, _pp, _pp, _pp, _pp, C.c_int, C.c_void_p)


def _ptrs(ts: Sequence[torch.Tensor]):
    arr = (C.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_cuda:
            raise ValueError("expected contiguous CUDA bf16 tensors")
        arr[i] = t.data_ptr()
    return arr


def _raw_ptrs(ts: Sequence[torch.Tensor], dtype: torch.dtype):
    arr = (C.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        if t.dtype != dtype or not t.is_contiguous() or not t.is_cuda:
            raise ValueError(f"expected contiguous CUDA {dtype} tensors")
        arr[i] = t.data_ptr()
    return arr


def quantize_rows(x: torch.Tensor, out8: torch.Tensor, scales: torch.Tensor) -> None:
    """``out8 [rows, K] = e4m3(x / s)``, ``scales [rows, K/128] = amax / 448`` (one CUDA kernel)."""
    rows, Kd = x.shape
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("expected a contiguous bf16 matrix")
    st = K.load().xccl_tp_quantize_rows(x.data_ptr(), rows, Kd, out8.data_ptr(), scales.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    if st != K.OK:
        raise XcclError(st, "xccl_tp_quantize_rows")


def _as_typed(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """A uint8 view of library-owned device memory."""
    class _Mem:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}

    return torch.as_tensor(_Mem(), device=device)


def _as_tensor(ptr: int, shape: tuple, device: torch.device) -> torch.Tensor:
    """A bf16 tensor view of library-owned device memory (no copy, not owned by torch)."""
    n = 1
    for s in shape:
        n *= s

    class _Mem:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<i2", "data": (ptr, False), "version": 3}

    return torch.as_tensor(_Mem(), device=device).view(torch.bfloat16).view(shape)


class TpWorkspace:
    def __init__(self, M: int, hidden: int, oob: Any = None, emu_ranks: int = 1, n_out: Optional[int] = None):
        self.M, self.K, self.N = M, hidden, hidden if n_out is None else n_out
        self.h = C.c_void_p()
        self.device = torch.device("cuda", torch.cuda.current_device())
        L = K.load()
        st = L.xccl_tp_ws_create(C.byref(oob.c) if oob is not None else None, emu_ranks, M, self.K, self.N,
                                 C.byref(self.h))
        if st != K.OK:
            raise XcclError(st, "xccl_tp_ws_create")
        self.tp = oob.size if oob is not None else emu_ranks
        self.n_local = 1 if oob is not None else emu_ranks
        self.rank = oob.rank if oob is not None else 0

    def x_shard(self, local_rank: int = 0) -> torch.Tensor:
        """This rank's rows of the gathered activation buffer: write the layer input here."""
        p = K.load().xccl_tp_ws_x_shard(self.h, local_rank)
        return _as_tensor(p, (self.M // self.tp, self.K), self.device)

    def x_full(self, local_rank: int = 0) -> torch.Tensor:
        p = K.load().xccl_tp_ws_x_full(self.h, local_rank)
        return _as_tensor(p, (self.M, self.K), self.device)

    def ag_gemm_swiglu(self, w_gate: Sequence[torch.Tensor], w_up: Sequence[torch.Tensor],
                       out: Sequence[torch.Tensor]) -> None:
        f_local = w_gate[0].shape[0]
        st = K.load().xccl_tp_ag_gemm_swiglu(self.h, _ptrs(w_gate), _ptrs(w_up), _ptrs(out), f_local,
                                             torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_ag_gemm_swiglu")

    def gemm_rs(self, h: Sequence[torch.Tensor], w_down: Sequence[torch.Tensor], out: Sequence[torch.Tensor]) -> None:
        f_local = h[0].shape[1]
        st = K.load().xccl_tp_gemm_rs(self.h, _ptrs(h), _ptrs(w_down), _ptrs(out), f_local,
                                      torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_gemm_rs")

    def h2d_begin(self, x_pinned: Sequence[torch.Tensor], copy_stream: "torch.cuda.Stream") -> None:
        """Starts the chunked host->device copy of this step's input shards on `copy_stream`; the next
        ``ag_gemm_swiglu`` consumes the rows as they land (no event between the two streams is needed)."""
        arr = (C.c_void_p * len(x_pinned))()
        for i, t in enumerate(x_pinned):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_pinned():
                raise ValueError("expected contiguous pinned bf16 host tensors")
            arr[i] = t.data_ptr()
        st = K.load().xccl_tp_h2d_begin(self.h, arr, copy_stream.cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_h2d_begin")

    def h2d_expect(self, copy_stream: "torch.cuda.Stream", ramp: int = 1) -> None:
        """First half of ``h2d_begin``: the next ``ag_gemm_swiglu`` will wait for the rows of a copy that
        ``h2d_issue`` enqueues AFTER the kernel has been launched, so the host time of issuing the chunks is spent
        while the kernel already runs. Must be followed by the launch and by ``h2d_issue``. ``ramp``: the kernel
        walks the local rows in groups of 1, 1, 2, 4, ... row blocks so that its first tiles need the first chunk only;
        a pipelined caller, whose copy runs under the previous step's kernels, passes 0. 2: phases over all shards
        (copy CTAs; every rank reports its rows block by block; all ranks must ask for the same)."""
        st = K.load().xccl_tp_h2d_expect(self.h, copy_stream.cuda_stream, int(ramp))
        if st != K.OK:
            raise XcclError(st, "xccl_tp_h2d_expect")

    def h2d_issue(self, x_pinned: Sequence[torch.Tensor], copy_stream: "torch.cuda.Stream") -> None:
        arr = (C.c_void_p * len(x_pinned))()
        for i, t in enumerate(x_pinned):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_pinned():
                raise ValueError("expected contiguous pinned bf16 host tensors")
            arr[i] = t.data_ptr()
        st = K.load().xccl_tp_h2d_issue(self.h, arr, copy_stream.cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_h2d_issue")

    # ---- block-scaled fp8 (the same buffers hold [M, K] e4m3 rows followed by [M, K/128] fp32 scales)
    def x8_shard(self, local_rank: int = 0) -> torch.Tensor:
        p = K.load().xccl_tp_ws_x8_shard(self.h, local_rank)
        rows = self.M // self.tp
        return _as_typed(p, rows * self.K, self.device).view(torch.float8_e4m3fn).view(rows, self.K)

    def sx_shard(self, local_rank: int = 0) -> torch.Tensor:
        p = K.load().xccl_tp_ws_sx_shard(self.h, local_rank)
        rows = self.M // self.tp
        return _as_typed(p, rows * (self.K // 128) * 4, self.device).view(torch.float32).view(rows, self.K // 128)

    def ag_gemm_swiglu_fp8(self, w_gate8, s_gate, w_up8, s_up, out: Sequence[torch.Tensor]) -> None:
        f_local = w_gate8[0].shape[0]
        f8, f32 = torch.float8_e4m3fn, torch.float32
        st = K.load().xccl_tp_ag_gemm_swiglu_fp8(self.h, _raw_ptrs(w_gate8, f8), _raw_ptrs(s_gate, f32), _raw_ptrs(w_up8, f8),
                                                 _raw_ptrs(s_up, f32), _ptrs(out), f_local,
                                                 torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_ag_gemm_swiglu_fp8")

    def ag_gemm_swiglu_fp8q(self, w_gate8, s_gate, w_up8, s_up, out8: Sequence[torch.Tensor],
                            out_scales: Sequence[torch.Tensor]) -> None:
        """As ``ag_gemm_swiglu_fp8`` with the output quantised in the epilogue: ``out8`` [M, F_local] e4m3 and
        ``out_scales`` [M, F_local/128] fp32, the activations of ``gemm_rs_fp8``."""
        f_local = w_gate8[0].shape[0]
        f8, f32 = torch.float8_e4m3fn, torch.float32
        st = K.load().xccl_tp_ag_gemm_swiglu_fp8q(self.h, _raw_ptrs(w_gate8, f8), _raw_ptrs(s_gate, f32), _raw_ptrs(w_up8, f8),
                                                  _raw_ptrs(s_up, f32), _raw_ptrs(out8, f8), _raw_ptrs(out_scales, f32),
                                                  f_local, torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_ag_gemm_swiglu_fp8q")

    def gemm_rs_fp8(self, h8, s_h, w_down8, s_down, out: Sequence[torch.Tensor]) -> None:
        f_local = h8[0].shape[1]
        f8, f32 = torch.float8_e4m3fn, torch.float32
        st = K.load().xccl_tp_gemm_rs_fp8(self.h, _raw_ptrs(h8, f8), _raw_ptrs(s_h, f32), _raw_ptrs(w_down8, f8),
                                          _raw_ptrs(s_down, f32), _ptrs(out), f_local,
                                          torch.cuda.current_stream().cuda_stream)
        if st != K.OK:
            raise XcclError(st, "xccl_tp_gemm_rs_fp8")

    def error(self) -> int:
        torch.cuda.synchronize()
        return int(K.load().xccl_tp_ws_error(self.h))

    def close(self) -> None:
        if self.h:
            K.load().xccl_tp_ws_destroy(self.h)
            self.h = C.c_void_p()
