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


K.optional("xccl_gemm_fp8_blockscaled", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
           C.c_int, C.c_int, C.c_void_p)

FP8_MAX = 448.0  # largest finite e4m3 value


def quantize_act_1x128(x: torch.Tensor):
    """Per-row, per-128-column scaling to e4m3: returns (x8 [M,K] float8_e4m3fn, scales [M,K/128] fp32)."""
    M, Kd = x.shape
    xb = x.float().view(M, Kd // 128, 128)
    s = xb.abs().amax(-1).clamp_min(1e-12) / FP8_MAX
    q = (xb / s[..., None]).to(torch.float8_e4m3fn).view(M, Kd)
    return q.contiguous(), s.contiguous()


def quantize_weight_128x128(w: torch.Tensor):
    """Per 128 x 128 block scaling to e4m3: returns (w8 [N,K], scales [N/128,K/128] fp32)."""
    N, Kd = w.shape
    wb = w.float().view(N // 128, 128, Kd // 128, 128)
    s = wb.abs().amax((1, 3)).clamp_min(1e-12) / FP8_MAX
    q = (wb / s[:, None, :, None]).to(torch.float8_e4m3fn).view(N, Kd)
    return q.contiguous(), s.contiguous()


def dequantize(q: torch.Tensor, s: torch.Tensor, block_rows: int) -> torch.Tensor:
    R, Kd = q.shape
    return (q.float().view(R // block_rows, block_rows, Kd // 128, 128) * s.view(R // block_rows, 1, Kd // 128, 1)).view(R, Kd)


def gemm_fp8_blockscaled(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M,N] (bf16) = dequant(a8, sa) @ dequant(b8, sb).T`` on the fp8 tensor cores; the scales
    are applied per 128-wide K block while fp32 partial products are promoted in registers."""
    M, Kd = a8.shape
    N = b8.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    st = K.load().xccl_gemm_fp8_blockscaled(a8.data_ptr(), sa.data_ptr(), b8.data_ptr(), sb.data_ptr(), out.data_ptr(),
                                            M, N, Kd, _stream())
    if st != K.OK:
        raise XcclError(st, "xccl_gemm_fp8_blockscaled")
    return out
