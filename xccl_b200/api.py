"""Object-level Python wrapper of the C API: Lib -> Context -> Team -> Request.

Buffers may be numpy arrays (host memory), torch tensors (host or CUDA) or raw integer
addresses. Every collective returns a persistent :class:`Request` that can be posted again.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Any, Optional, Sequence

from . import _capi as K


class XcclError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: {K.status_str(status)} ({status})")
        self.status = status


def _check(st: int, what: str) -> None:
    if st != K.OK:
        raise XcclError(st, what)


_NP_DT = {"int8": K.DT_INT8, "int16": K.DT_INT16, "int32": K.DT_INT32, "int64": K.DT_INT64,
          "uint8": K.DT_UINT8, "uint16": K.DT_UINT16, "uint32": K.DT_UINT32, "uint64": K.DT_UINT64,
          "float16": K.DT_FLOAT16, "float32": K.DT_FLOAT32, "float64": K.DT_FLOAT64,
          "bfloat16": K.DT_BFLOAT16}


def dtype_of(buf: Any) -> int:
    """XCCL datatype of a numpy array or torch tensor."""
    name = str(getattr(buf, "dtype", "")).replace("torch.", "")
    if name not in _NP_DT:
        raise TypeError(f"no XCCL datatype for {name!r}")
    return _NP_DT[name]


def addr_of(buf: Any) -> int:
    if buf is None:
        return 0
    if isinstance(buf, int):
        return buf
    if hasattr(buf, "data_ptr"):
        return int(buf.data_ptr())
    if hasattr(buf, "ctypes"):
        return int(buf.ctypes.data)
    raise TypeError(f"cannot take the address of {type(buf)}")


def nbytes_of(buf: Any) -> int:
    if hasattr(buf, "nbytes"):
        return int(buf.nbytes)
    return int(buf.numel() * buf.element_size())


def numel_of(buf: Any) -> int:
    return int(buf.size) if hasattr(buf, "ctypes") else int(buf.numel())


def _is_array(buf: Any) -> bool:
    return buf is not None and not isinstance(buf, (int, str)) and (hasattr(buf, "data_ptr") or hasattr(buf, "ctypes"))


def _require(buf: Any, nbytes: int, what: str) -> None:
    """A buffer handed to a collective is one contiguous block of at least `nbytes` bytes: the library sees only its
    address, so a strided view or a short buffer would be read or written past what the caller meant."""
    if not _is_array(buf):
        return  # a raw address or the in-place marker: the caller vouches for it
    if hasattr(buf, "is_contiguous"):
        contiguous = bool(buf.is_contiguous())
    else:
        contiguous = bool(buf.flags["C_CONTIGUOUS"])
    if not contiguous:
        raise ValueError(f"{what} is not contiguous")
    if nbytes_of(buf) < nbytes:
        raise ValueError(f"{what} holds {nbytes_of(buf)} bytes, the collective needs {nbytes}")


class ShmOob:
    """Shared-memory out-of-band provider for ranks of one host (``xccl_oob_shm_create``)."""

    def __init__(self, job_key: str, rank: int, size: int):
        self.c = K.Oob()
        _check(K.load().xccl_oob_shm_create(job_key.encode(), rank, size, C.byref(self.c)), "xccl_oob_shm_create")
        self.rank, self.size = rank, size
        self._alive = True

    def sub(self, parent_ranks: Sequence[int]) -> "SubOob":
        return SubOob(self, parent_ranks)

    def allgather_bytes(self, data: bytes) -> list[bytes]:
        n = len(data)
        sbuf = C.create_string_buffer(data, n)
        rbuf = C.create_string_buffer(n * self.size)
        _check(K.load().xccl_oob_allgather(C.byref(self.c), sbuf, rbuf, n), "xccl_oob_allgather")
        return [rbuf.raw[i * n:(i + 1) * n] for i in range(self.size)]

    def close(self) -> None:
        if self._alive:
            K.load().xccl_oob_shm_destroy(C.byref(self.c))
            self._alive = False


class SubOob:
    """View of a parent OOB restricted to some of its ranks (``xccl_oob_sub_create``)."""

    def __init__(self, parent: Any, parent_ranks: Sequence[int]):
        self.parent = parent
        self.c = K.Oob()
        arr = (C.c_int * len(parent_ranks))(*parent_ranks)
        _check(K.load().xccl_oob_sub_create(C.byref(parent.c), arr, len(parent_ranks), C.byref(self.c)),
               "xccl_oob_sub_create")
        self.rank, self.size = self.c.rank, self.c.size

    allgather_bytes = ShmOob.allgather_bytes

    def close(self) -> None:
        K.load().xccl_oob_sub_destroy(C.byref(self.c))


class Lib:
    def __init__(self, coll_types: Optional[int] = None, thread_mode: Optional[int] = None,
                 team_usage: Optional[int] = None):
        L = K.load()
        p = K.LibParams()
        if coll_types is not None:
            p.field_mask |= K.LIB_PARAM_COLL_TYPES
            p.coll_types = coll_types
        if thread_mode is not None:
            p.field_mask |= K.LIB_PARAM_THREAD_MODE
            p.thread_mode = thread_mode
        if team_usage is not None:
            p.field_mask |= K.LIB_PARAM_TEAM_USAGE
            p.team_usage = team_usage
        self.h = C.c_void_p()
        _check(L.xccl_lib_init(C.byref(p), None, C.byref(self.h)), "xccl_lib_init")

    def tl_list(self) -> list[int]:
        L = K.load()
        arr = C.POINTER(C.c_int)()
        n = C.c_uint()
        _check(L.xccl_get_tl_list(self.h, C.byref(arr), C.byref(n)), "xccl_get_tl_list")
        out = [arr[i] for i in range(n.value)]
        L.xccl_free_tl_list(arr)
        return out

    def close(self) -> None:
        if self.h:
            K.load().xccl_lib_cleanup(self.h)
            self.h = C.c_void_p()


class Context:
    def __init__(self, lib: Lib, oob: Any, tls: int = K.TL_ALL, thread_mode: int = K.THREAD_SINGLE,
                 config: Optional[dict[int, dict[str, str]]] = None, env_prefix: Optional[str] = None):
        L = K.load()
        self.lib, self.oob = lib, oob
        cfg = C.c_void_p()
        _check(L.xccl_context_config_read(lib.h, env_prefix.encode() if env_prefix else None, None, C.byref(cfg)),
               "xccl_context_config_read")
        for tl, opts in (config or {}).items():
            tl_c = C.c_int(tl)
            for name, value in opts.items():
                st = L.xccl_context_config_modify(C.byref(tl_c), cfg, name.encode(), str(value).encode())
                if st not in (K.OK, K.ERR_NO_ELEM):
                    L.xccl_context_config_release(cfg)
                    _check(st, f"xccl_context_config_modify({K.TL_NAMES.get(tl)}, {name})")
        p = K.ContextParams()
        p.field_mask = K.CTX_PARAM_OOB | K.CTX_PARAM_TLS | K.CTX_PARAM_THREAD_MODE
        p.thread_mode = thread_mode
        p.oob = oob.c
        p.tls = tls
        self.h = C.c_void_p()
        st = L.xccl_context_create(lib.h, C.byref(p), cfg, C.byref(self.h))
        L.xccl_context_config_release(cfg)
        _check(st, "xccl_context_create")

    def progress(self) -> None:
        st = K.load().xccl_context_progress(self.h)
        if st < 0:
            raise XcclError(st, "xccl_context_progress")

    def supported_colls(self) -> int:
        a = K.CtxAttr()
        a.field_mask = 1
        _check(K.load().xccl_ctx_query(self.h, C.byref(a)), "xccl_ctx_query")
        return int(a.supported_colls)

    def close(self) -> None:
        if self.h:
            K.load().xccl_context_destroy(self.h)
            self.h = C.c_void_p()


class Request:
    """Persistent collective request (``xccl_collective_init`` .. ``finalize``)."""

    def __init__(self, team: "Team", args: K.CollArgs, keep: tuple):
        self.team, self.args, self._keep = team, args, keep
        self.h = C.c_void_p()
        _check(K.load().xccl_collective_init(C.byref(args), C.byref(self.h), team.h), "xccl_collective_init")

    def post(self) -> "Request":
        _check(K.load().xccl_collective_post(self.h), "xccl_collective_post")
        return self

    def test(self) -> bool:
        st = K.load().xccl_collective_test(self.h)
        if st < 0:
            raise XcclError(st, "xccl_collective_test")
        return st == K.OK

    def wait(self, timeout: Optional[float] = None) -> "Request":
        if timeout is None:
            _check(K.load().xccl_collective_wait(self.h), "xccl_collective_wait")
            return self
        t0 = time.monotonic()
        while not self.test():
            self.team.ctx.progress()
            if time.monotonic() - t0 > timeout:
                raise XcclError(K.ERR_TIMED_OUT, "Request.wait")
        return self

    def run(self) -> "Request":
        return self.post().wait()

    @property
    def elapsed_us(self) -> float:
        return float(K.load().xccl_collective_elapsed_us(self.h))

    def finalize(self) -> None:
        if self.h:
            _check(K.load().xccl_collective_finalize(self.h), "xccl_collective_finalize")
            self.h = C.c_void_p()


class Team:
    def __init__(self, ctx: Context, oob: Any = None, ranks: Optional[Sequence[int]] = None,
                 timeout: float = 120.0):
        """A team over the whole context, over `oob` (its own bootstrap), or over the context
        ranks listed in `ranks` (an endpoint map)."""
        L = K.load()
        self.ctx = ctx
        p = K.TeamParams()
        self._keep: list = []
        if oob is not None:
            p.field_mask |= K.TEAM_PARAM_OOB
            p.oob = oob.c
            self._keep.append(oob)
            p.range.type = K.EP_RANGE_FULL
            p.range.ep_num = oob.size
            p.field_mask |= K.TEAM_PARAM_EP_RANGE
        elif ranks is not None:
            arr = (C.c_int * len(ranks))(*ranks)
            self._keep.append(arr)
            p.field_mask |= K.TEAM_PARAM_EP_RANGE
            p.range.type = K.EP_RANGE_MAP
            p.range.ep_num = len(ranks)
            p.range.map.map = C.cast(arr, C.POINTER(C.c_int))
        self.h = C.c_void_p()
        _check(L.xccl_team_create_post(ctx.h, C.byref(p), C.byref(self.h)), "xccl_team_create_post")
        t0 = time.monotonic()
        while True:
            st = L.xccl_team_create_test(self.h)
            if st == K.OK:
                break
            if st < 0:
                raise XcclError(st, "xccl_team_create_test")
            ctx.progress()
            if time.monotonic() - t0 > timeout:
                raise XcclError(K.ERR_TIMED_OUT, "xccl_team_create_test")
        r, s = C.c_int(), C.c_int()
        _check(L.xccl_team_query(self.h, C.byref(r), C.byref(s)), "xccl_team_query")
        self.rank, self.size = r.value, s.value

    def coll_tl(self, coll: int, mem: int = K.MEM_HOST) -> int:
        return int(K.load().xccl_team_coll_tl(self.h, coll, mem))

    def mem_alloc(self, nbytes: int):
        """Symmetric device memory (``xccl_team_mem_alloc``; collective: every member calls it with the same
        size). Returns a uint8 torch tensor over the memory; view it as any dtype. Collectives whose buffers lie
        in such memory at the same offset on every member run zero-copy through the NVSwitch multicast mapping."""
        import torch
        L = K.load()
        L.xccl_team_mem_alloc.restype = C.c_int
        L.xccl_team_mem_alloc.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]
        p = C.c_void_p()
        _check(L.xccl_team_mem_alloc(self.h, int(nbytes), C.byref(p)), "xccl_team_mem_alloc")
        ptr = int(p.value)

        class _Mem:
            __cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (ptr, False), "version": 3}

        t = torch.as_tensor(_Mem(), device=torch.device("cuda", torch.cuda.current_device()))
        self._sym = getattr(self, "_sym", {})
        self._sym[t.data_ptr()] = ptr
        return t

    def mem_free(self, tensor) -> None:
        """Returns memory of ``mem_alloc`` (collective)."""
        L = K.load()
        L.xccl_team_mem_free.restype = C.c_int
        L.xccl_team_mem_free.argtypes = [C.c_void_p, C.c_void_p]
        ptr = getattr(self, "_sym", {}).pop(tensor.data_ptr(), tensor.data_ptr())
        _check(L.xccl_team_mem_free(self.h, C.c_void_p(ptr)), "xccl_team_mem_free")

    # ------------------------------------------------------------ request builders
    def _args(self, coll: int, src: Any, dst: Any, length: int, alg: Optional[int], stream: Any,
              keep: list) -> K.CollArgs:
        a = K.CollArgs()
        a.coll_type = coll
        a.buffer_info.src_buffer = K.IN_PLACE if (isinstance(src, str) and src == "in_place") else addr_of(src)
        a.buffer_info.dst_buffer = addr_of(dst)
        a.buffer_info.len = length
        if alg is not None:
            a.alg.set_by_user = 1
            a.alg.id = alg
        if stream is not None:
            h = C.c_void_p(int(stream))
            keep.append(h)
            a.field_mask |= K.ARGS_FIELD_STREAM
            a.stream.type = 0
            a.stream.stream = C.cast(C.pointer(h), C.c_void_p)
        keep.extend([src, dst])
        return a

    def allreduce(self, src: Any, dst: Any, op: int = K.OP_SUM, count: Optional[int] = None,
                  dt: Optional[int] = None, alg: Optional[int] = None, stream: Any = None,
                  scale: Optional[float] = None, out_dt: Optional[int] = None) -> Request:
        keep: list = []
        dt = dtype_of(dst if isinstance(src, str) else src) if dt is None else dt
        count = numel_of(dst if isinstance(src, str) else src) if count is None else count
        _require(src, count * K.DT_SIZE[dt], "src")
        _require(dst, count * K.DT_SIZE[dt if out_dt is None or out_dt == K.DT_UNSUPPORTED else out_dt], "dst")
        a = self._args(K.ALLREDUCE, src, dst, count * K.DT_SIZE[dt], alg, stream, keep)
        a.reduce_info.dt, a.reduce_info.op, a.reduce_info.count = dt, op, count
        self._epilogue(a, scale, out_dt)
        return Request(self, a, tuple(keep))

    @staticmethod
    def _epilogue(a, scale: Optional[float], out_dt: Optional[int]) -> None:
        if scale is not None or out_dt is not None:
            a.field_mask |= K.ARGS_FIELD_EPILOGUE
            a.epilogue.scale = 1.0 if scale is None else scale
            a.epilogue.out_dt = K.DT_UNSUPPORTED if out_dt is None else out_dt

    def reduce(self, src: Any, dst: Any, root: int, op: int = K.OP_SUM, count: Optional[int] = None,
               dt: Optional[int] = None, alg: Optional[int] = None, stream: Any = None,
               scale: Optional[float] = None, out_dt: Optional[int] = None) -> Request:
        keep: list = []
        dt = dtype_of(src) if dt is None else dt
        count = numel_of(src) if count is None else count
        _require(src, count * K.DT_SIZE[dt], "src")
        if self.rank == root:
            _require(dst, count * K.DT_SIZE[dt if out_dt is None or out_dt == K.DT_UNSUPPORTED else out_dt], "dst")
        a = self._args(K.REDUCE, src, dst, count * K.DT_SIZE[dt], alg, stream, keep)
        a.reduce_info.dt, a.reduce_info.op, a.reduce_info.count = dt, op, count
        a.root = root
        self._epilogue(a, scale, out_dt)
        return Request(self, a, tuple(keep))

    def reduce_scatter(self, src: Any, dst: Any, op: int = K.OP_SUM, dt: Optional[int] = None,
                       stream: Any = None, alg: Optional[int] = None,
                       scale: Optional[float] = None, out_dt: Optional[int] = None) -> Request:
        keep: list = []
        dt = dtype_of(src) if dt is None else dt
        _require(src, 0, "src")
        _require(dst, numel_of(src) // self.size * K.DT_SIZE[dt if out_dt is None or out_dt == K.DT_UNSUPPORTED else out_dt], "dst")
        a = self._args(K.REDUCE_SCATTER, src, dst, nbytes_of(src), alg, stream, keep)
        a.reduce_info.dt, a.reduce_info.op = dt, op
        a.reduce_info.count = numel_of(src) // self.size
        self._epilogue(a, scale, out_dt)
        return Request(self, a, tuple(keep))

    def bcast(self, buf: Any, root: int, nbytes: Optional[int] = None, alg: Optional[int] = None,
              stream: Any = None) -> Request:
        keep: list = []
        _require(buf, 0 if nbytes is None else nbytes, "buf")
        a = self._args(K.BCAST, buf, buf, nbytes_of(buf) if nbytes is None else nbytes, alg, stream, keep)
        a.root = root
        return Request(self, a, tuple(keep))

    def allgather(self, src: Any, dst: Any, stream: Any = None, alg: Optional[int] = None) -> Request:
        keep: list = []
        _require(dst, 0, "dst")
        _require(src, nbytes_of(dst) // self.size, "src")
        a = self._args(K.ALLGATHER, src, dst, nbytes_of(dst), alg, stream, keep)
        return Request(self, a, tuple(keep))

    def alltoall(self, src: Any, dst: Any, bytes_per_peer: Optional[int] = None, alg: Optional[int] = None,
                 stream: Any = None) -> Request:
        keep: list = []
        per = nbytes_of(dst) // self.size if bytes_per_peer is None else bytes_per_peer
        _require(src, per * self.size, "src")
        _require(dst, per * self.size, "dst")
        a = self._args(K.ALLTOALL, src, dst, per, alg, stream, keep)
        return Request(self, a, tuple(keep))

    def alltoallv(self, src: Any, src_counts: Sequence[int], src_displs: Sequence[int], dst: Any,
                  dst_counts: Sequence[int], dst_displs: Sequence[int], dt: Optional[int] = None,
                  stream: Any = None) -> Request:
        keep: list = []
        dt = dtype_of(src) if dt is None else dt
        if len(src_counts) != self.size or len(src_displs) != self.size or len(dst_counts) != self.size or \
                len(dst_displs) != self.size:
            raise ValueError("alltoallv takes one count and one displacement per team rank")
        es = K.DT_SIZE[dt]
        _require(src, max((int(d) + int(c)) for c, d in zip(src_counts, src_displs)) * es, "src")
        _require(dst, max((int(d) + int(c)) for c, d in zip(dst_counts, dst_displs)) * es, "dst")
        a = self._args(K.ALLTOALLV, src, dst, 0, None, stream, keep)
        arrs = [(C.c_uint32 * self.size)(*map(int, v)) for v in (src_counts, src_displs, dst_counts, dst_displs)]
        keep.extend(arrs)
        u32p = C.POINTER(C.c_uint32)
        a.buffer_info.src_counts = C.cast(arrs[0], u32p)
        a.buffer_info.src_displacements = C.cast(arrs[1], u32p)
        a.buffer_info.dst_counts = C.cast(arrs[2], u32p)
        a.buffer_info.dst_displacements = C.cast(arrs[3], u32p)
        a.buffer_info.src_datatype = dt
        a.buffer_info.dst_datatype = dt
        return Request(self, a, tuple(keep))

    def _sync(self, coll: int, root: int = 0) -> Request:
        a = K.CollArgs()
        a.coll_type = coll
        a.root = root
        return Request(self, a, ())

    def barrier(self) -> Request:
        return self._sync(K.BARRIER)

    def fanin(self, root: int = 0) -> Request:
        return self._sync(K.FANIN, root)

    def fanout(self, root: int = 0) -> Request:
        return self._sync(K.FANOUT, root)

    # ------------------------------------------------------------ global memory
    def mem_map(self, buf: Any, root: int, nbytes: Optional[int] = None, timeout: float = 60.0) -> "MemHandle":
        """Maps `nbytes` of the root's `buf` for the whole team (``xccl_global_mem_map_start/test``)."""
        p = K.MemMapParams()
        p.field_mask = K.MEM_MAP_ADDRESS | K.MEM_MAP_LENGTH | K.MEM_MAP_ROOT
        p.address = addr_of(buf)
        p.length = nbytes_of(buf) if nbytes is None else nbytes
        p.root = root
        h = C.c_void_p()
        _check(K.load().xccl_global_mem_map_start(self.h, p, C.byref(h)), "xccl_global_mem_map_start")
        t0 = time.monotonic()
        while True:
            st = K.load().xccl_global_mem_map_test(h)
            if st == K.OK:
                break
            if st < 0:
                raise XcclError(st, "xccl_global_mem_map_test")
            self.ctx.progress()
            if time.monotonic() - t0 > timeout:
                raise XcclError(K.ERR_TIMED_OUT, "xccl_global_mem_map_test")
        return MemHandle(h, buf)

    def fanout_get(self, memh: "MemHandle", offset: int, local: Any, nbytes: int) -> Request:
        a = K.CollArgs()
        a.coll_type = K.FANOUT_GET
        a.get_info.memh = memh.h
        a.get_info.offset = offset
        a.get_info.local_buffer = addr_of(local)
        a.get_info.len = nbytes
        return Request(self, a, (memh, local))

    def close(self) -> None:
        if self.h:
            K.load().xccl_team_destroy(self.h)
            self.h = C.c_void_p()


class MemHandle:
    def __init__(self, h: C.c_void_p, keep: Any):
        self.h, self._keep = h, keep

    def unmap(self) -> None:
        if self.h:
            _check(K.load().xccl_global_mem_unmap(self.h), "xccl_global_mem_unmap")
            self.h = C.c_void_p()
