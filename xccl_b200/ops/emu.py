"""Single-GPU emulation of an N-rank NVLink team (``csrc/tl/nvlink/nvl_emu.cu``).

All ranks' buffers live on the current device and every collective is ONE cooperative kernel
launch whose ``blockIdx.y`` is the rank, so the multi-rank kernels can be exercised on one GPU.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _capi as K
from ..api import XcclError, dtype_of

_pp = C.POINTER(C.c_void_p)
K.optional("xccl_nvlink_emu_create", C.c_int, C.c_int, C.c_size_t, _pp)
K.optional("xccl_nvlink_emu_destroy", None, C.c_void_p)
K.optional("xccl_nvlink_emu_collective", C.c_int, C.c_void_p, C.c_int, _pp, _pp, C.c_size_t, C.c_size_t, C.c_int,
           C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _pp, C.c_size_t, C.c_int, C.c_int, C.c_void_p)
K.optional("xccl_nvlink_emu_timeout_probe", C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_float),
           C.POINTER(C.c_uint32))


def _ptrs(ts: Optional[Sequence[torch.Tensor]], n: int):
    arr = (C.c_void_p * n)()
    if ts is not None:
        for i, t in enumerate(ts):
            arr[i] = t.data_ptr() if t is not None else None
    return arr


class EmuWorld:
    def __init__(self, nranks: int, ws_bytes: int = 64 << 20):
        self.n = nranks
        self.h = C.c_void_p()
        st = K.load().xccl_nvlink_emu_create(nranks, ws_bytes, C.byref(self.h))
        if st != K.OK:
            raise XcclError(st, "xccl_nvlink_emu_create")

    def close(self) -> None:
        if self.h:
            K.load().xccl_nvlink_emu_destroy(self.h)
            self.h = C.c_void_p()

    def _run(self, coll, srcs, dsts, count=0, length=0, dt=K.DT_UINT8, out_dt=K.DT_UNSUPPORTED, op=K.OP_SUM,
             root=0, scale=1.0, alg=0, vmeta=None, max_src_bytes=0, es=1, blocks=0) -> None:
        s = torch.cuda.current_stream().cuda_stream
        st = K.load().xccl_nvlink_emu_collective(self.h, coll, _ptrs(srcs, self.n), _ptrs(dsts, self.n), count,
                                                 length, dt, out_dt, op, root, scale, alg, _ptrs(vmeta, self.n),
                                                 max_src_bytes, es, blocks, s)
        if st != K.OK:
            raise XcclError(st, f"emulated collective {coll}")

    def allreduce(self, srcs, dsts, op=K.OP_SUM, alg=0, scale=1.0, blocks=0) -> None:
        dt, odt = dtype_of(srcs[0]), dtype_of(dsts[0])
        self._run(K.ALLREDUCE, srcs, dsts, count=srcs[0].numel(), dt=dt,
                  out_dt=odt if odt != dt else K.DT_UNSUPPORTED, op=op, alg=alg, scale=scale, blocks=blocks)

    def reduce(self, srcs, dsts, root, op=K.OP_SUM, scale=1.0) -> None:
        self._run(K.REDUCE, srcs, dsts, count=srcs[0].numel(), dt=dtype_of(srcs[0]), op=op, root=root, scale=scale)

    def reduce_scatter(self, srcs, dsts, op=K.OP_SUM, alg=0) -> None:
        self._run(K.REDUCE_SCATTER, srcs, dsts, count=dsts[0].numel(), dt=dtype_of(srcs[0]), op=op, alg=alg)

    def bcast(self, srcs, dsts, root) -> None:
        self._run(K.BCAST, srcs, dsts, length=dsts[0].numel() * dsts[0].element_size(), root=root)

    def allgather(self, srcs, dsts, alg=0) -> None:
        self._run(K.ALLGATHER, srcs, dsts, length=dsts[0].numel() * dsts[0].element_size(), alg=alg)

    def alltoall(self, srcs, dsts, alg=0) -> None:
        self._run(K.ALLTOALL, srcs, dsts, length=dsts[0].numel() * dsts[0].element_size() // self.n, alg=alg)

    def alltoallv(self, srcs, dsts, metas, max_src_bytes) -> None:
        self._run(K.ALLTOALLV, srcs, dsts, vmeta=metas, max_src_bytes=max_src_bytes, es=srcs[0].element_size())

    def barrier(self) -> None:
        self._run(K.BARRIER, None, None)

    def fanin(self, root) -> None:
        self._run(K.FANIN, None, None, root=root)

    def fanout(self, root) -> None:
        self._run(K.FANOUT, None, None, root=root)

    def timeout_probe(self, budget_ms: int):
        ms = C.c_float()
        st4 = (C.c_uint32 * 4)()
        st = K.load().xccl_nvlink_emu_timeout_probe(self.h, budget_ms, C.byref(ms), st4)
        return st, ms.value, list(st4)
