"""tcgen05 GEMM entry points (``csrc/fused/tp_gemm.cu``) on torch tensors."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _capi as K
from ..api import XcclError

K.optional("xccl_gemm_bf16", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p)
K.optional("xccl_gemm_swiglu_bf16", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
           C.c_int, C.c_void_p)
K.optional("xccl_gemm_last_error", C.c_uint32)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_bf16(*ts: torch.Tensor) -> None:
    for t in ts:
        if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous():
            raise ValueError("expected contiguous CUDA bf16 tensors")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ b[N,K].T`` with fp32 accumulation in tensor memory."""
    _check_bf16(a, b)
    M, Kd = a.shape
    N, K2 = b.shape
    if Kd != K2:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    st = K.load().xccl_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, Kd, _stream())
    if st != K.OK:
        raise XcclError(st, "xccl_gemm_bf16")
    return out


def gemm_swiglu(a: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M,F] = silu(a @ w_gate.T) * (a @ w_up.T)`` in one kernel; F must be a multiple of 128."""
    _check_bf16(a, w_gate, w_up)
    M, Kd = a.shape
    F = w_gate.shape[0]
    if out is None:
        out = torch.empty((M, F), dtype=torch.bfloat16, device=a.device)
    st = K.load().xccl_gemm_swiglu_bf16(a.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(), M, F, Kd,
                                        _stream())
    if st != K.OK:
        raise XcclError(st, "xccl_gemm_swiglu_bf16")
    return out


def last_error() -> int:
    """Error word of the GEMM kernels on the current device (0 = none). Synchronises."""
    return int(K.load().xccl_gemm_last_error())
