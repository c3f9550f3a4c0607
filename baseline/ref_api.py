"""ctypes driver for the UNMODIFIED reference library built by ``baseline/build_ref.py``.

Everything here follows the reference's own public header (``src/api/xccl.h``, ``src/api/xccl_tls.h``
of openucx/xccl): structure layouts, enum values and call order (``xccl_lib_init`` ->
``xccl_context_create`` -> ``xccl_team_create_post/test`` -> ``xccl_collective_init/post/test/
finalize``). Nothing of this repository's own library is loaded by this module; the out-of-band
allgather the reference asks its user for is served by a ``torch.distributed`` (gloo) group.

Used by ``bench.py --impl reference`` and by the collective sweep's reference arm.
"""
import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "lib" / "libxccl.so"

OK, INPROGRESS = 0, 1
(BARRIER, BCAST, ALLREDUCE, REDUCE, ALLTOALL, ALLTOALLV, ALLGATHER, FANIN, FANOUT, FANOUT_GET) = range(10)
OP_MAX, OP_MIN, OP_SUM, OP_PROD = 0, 1, 2, 3
(DT_INT8, DT_INT16, DT_INT32, DT_INT64, DT_INT128, DT_UINT8, DT_UINT16, DT_UINT32, DT_UINT64, DT_UINT128,
 DT_FLOAT16, DT_FLOAT32, DT_FLOAT64) = range(13)
TL_UCX, TL_NCCL = 1 << 0, 1 << 6
THREAD_MODE_SINGLE = 1 << 1
LIB_PARAM_THREAD_MODE, LIB_PARAM_TEAM_USAGE = 1 << 1, 1 << 2
TEAM_USAGE_HW, TEAM_USAGE_SW = 1 << 0, 1 << 1
CTX_PARAM_THREAD_MODE, CTX_PARAM_COMPLETION, CTX_PARAM_OOB, CTX_PARAM_TLS = 1, 2, 4, 8
COMPLETION_NONBLOCKING = 1
TEAM_PARAM_EP_RANGE, TEAM_PARAM_OOB = 1, 2
EP_RANGE_STRIDED = 2
ARGS_FIELD_STREAM = 1


class LibParams(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("reproducible", C.c_uint), ("thread_mode", C.c_uint),
                ("team_usage", C.c_uint64), ("coll_types", C.c_uint64)]


class EpRange(C.Structure):
    """xccl_ep_range_t with its 16-byte union (strided / map / cb) spelled as two words, so that the
    structure can be a by-value callback parameter (24 bytes: passed in memory either way)."""
    _fields_ = [("type", C.c_int), ("ep_num", C.c_int), ("u0", C.c_uint64), ("u1", C.c_uint64)]


ALLGATHER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, EpRange, C.c_void_p,
                           C.POINTER(C.c_void_p))
REQ_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)


class Oob(C.Structure):
    _fields_ = [("allgather", ALLGATHER_FN), ("req_test", REQ_FN), ("req_free", REQ_FN),
                ("coll_context", C.c_void_p), ("rank", C.c_int), ("size", C.c_int)]


class ContextParams(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("thread_mode", C.c_uint), ("completion_type", C.c_int),
                ("oob", Oob), ("tls", C.c_uint64)]


class TeamParams(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("range", EpRange), ("oob", Oob)]


class ReduceInfo(C.Structure):
    _fields_ = [("dt", C.c_int), ("op", C.c_int), ("count", C.c_size_t)]


class BufferInfo(C.Structure):
    _fields_ = [("src_buffer", C.c_void_p), ("src_counts", C.POINTER(C.c_uint32)),
                ("src_displacements", C.POINTER(C.c_uint32)), ("src_datatype", C.c_int),
                ("dst_buffer", C.c_void_p), ("dst_counts", C.POINTER(C.c_uint32)),
                ("dst_displacements", C.POINTER(C.c_uint32)), ("dst_datatype", C.c_int), ("len", C.c_size_t)]


class GetInfo(C.Structure):
    _fields_ = [("memh", C.c_void_p), ("offset", C.c_ssize_t), ("local_buffer", C.c_void_p), ("len", C.c_size_t)]


class _InfoU(C.Union):
    _fields_ = [("buffer_info", BufferInfo), ("get_info", GetInfo)]


class Stream(C.Structure):
    _fields_ = [("type", C.c_int), ("stream", C.c_void_p)]


class CollOpArgs(C.Structure):
    _anonymous_ = ("u",)
    _fields_ = [("field_mask", C.c_uint64), ("coll_type", C.c_int), ("u", _InfoU), ("reduce_info", ReduceInfo),
                ("root", C.c_int), ("alg", C.c_uint8), ("tag", C.c_uint16), ("stream", Stream)]


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise FileNotFoundError(f"{LIB_PATH} is missing: run python baseline/build_ref.py")
    lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
    vp, vpp = C.c_void_p, C.POINTER(C.c_void_p)
    lib.xccl_lib_config_read.argtypes = [C.c_char_p, C.c_char_p, vpp]
    lib.xccl_lib_config_release.argtypes = [vp]
    lib.xccl_lib_config_release.restype = None
    lib.xccl_lib_init.argtypes = [C.POINTER(LibParams), vp, vpp]
    lib.xccl_lib_cleanup.argtypes = [vp]
    lib.xccl_lib_cleanup.restype = None
    lib.xccl_context_config_read.argtypes = [vp, C.c_char_p, C.c_char_p, vpp]
    lib.xccl_context_config_release.argtypes = [vp]
    lib.xccl_context_config_release.restype = None
    lib.xccl_context_create.argtypes = [vp, C.POINTER(ContextParams), vp, vpp]
    lib.xccl_context_progress.argtypes = [vp]
    lib.xccl_context_destroy.argtypes = [vp]
    lib.xccl_team_create_post.argtypes = [vp, C.POINTER(TeamParams), vpp]
    lib.xccl_team_create_test.argtypes = [vp]
    lib.xccl_team_destroy.argtypes = [vp]
    lib.xccl_team_destroy.restype = None
    lib.xccl_collective_init.argtypes = [C.POINTER(CollOpArgs), vpp, vp]
    for f in ("post", "wait", "test", "finalize"):
        getattr(lib, "xccl_collective_" + f).argtypes = [vp]
    return lib


class RefError(RuntimeError):
    pass


def _check(st: int, what: str) -> None:
    if st != OK:
        raise RefError(f"reference {what} failed with status {st}")


class RefSession:
    """Library + context + team of the reference over all ranks of a ``torch.distributed`` group
    (a CPU group: it only carries the out-of-band allgather)."""

    def __init__(self, group=None, tls: int = TL_NCCL):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.lib = load()
        self._keep = []          # ctypes objects the C side points at
        self._oob = self._make_oob()
        lp = LibParams(field_mask=LIB_PARAM_THREAD_MODE | LIB_PARAM_TEAM_USAGE, thread_mode=THREAD_MODE_SINGLE,
                       team_usage=TEAM_USAGE_HW | TEAM_USAGE_SW)
        cfg = C.c_void_p()
        _check(self.lib.xccl_lib_config_read(None, None, C.byref(cfg)), "xccl_lib_config_read")
        self.h_lib = C.c_void_p()
        _check(self.lib.xccl_lib_init(C.byref(lp), cfg, C.byref(self.h_lib)), "xccl_lib_init")
        self.lib.xccl_lib_config_release(cfg)
        cp = ContextParams(field_mask=CTX_PARAM_THREAD_MODE | CTX_PARAM_COMPLETION | CTX_PARAM_OOB | CTX_PARAM_TLS,
                           thread_mode=THREAD_MODE_SINGLE, completion_type=COMPLETION_NONBLOCKING, oob=self._oob,
                           tls=tls)
        self.h_ctx, ctx_cfg = C.c_void_p(), C.c_void_p()
        _check(self.lib.xccl_context_config_read(self.h_lib, None, None, C.byref(ctx_cfg)), "xccl_context_config_read")
        _check(self.lib.xccl_context_create(self.h_lib, C.byref(cp), ctx_cfg, C.byref(self.h_ctx)), "xccl_context_create")
        self.lib.xccl_context_config_release(ctx_cfg)
        tp = TeamParams(field_mask=TEAM_PARAM_EP_RANGE | TEAM_PARAM_OOB, oob=self._oob)
        tp.range.type, tp.range.ep_num = EP_RANGE_STRIDED, self.size
        tp.range.u0 = (1 << 32) | 0   # strided { start = 0, stride = 1 }
        self.h_team = C.c_void_p()
        _check(self.lib.xccl_team_create_post(self.h_ctx, C.byref(tp), C.byref(self.h_team)), "xccl_team_create_post")
        while True:
            st = self.lib.xccl_team_create_test(self.h_team)
            if st == OK:
                break
            if st != INPROGRESS:
                raise RefError(f"reference xccl_team_create_test failed with status {st}")

    def _make_oob(self) -> Oob:
        import torch
        dist, group, size = self.dist, self.group, self.size

        def allgather(src, dst, nbytes, my_rank, ep_range, ctx, req):
            mine = torch.frombuffer(bytearray(C.string_at(src, nbytes)), dtype=torch.uint8)
            out = torch.empty(size * nbytes, dtype=torch.uint8)
            dist.all_gather_into_tensor(out, mine, group=group)
            C.memmove(dst, out.numpy().ctypes.data, size * nbytes)
            req[0] = 1   # finished already: any non-null token
            return 0

        cb_ag, cb_test, cb_free = ALLGATHER_FN(allgather), REQ_FN(lambda r: OK), REQ_FN(lambda r: OK)
        self._keep += [cb_ag, cb_test, cb_free]
        return Oob(allgather=cb_ag, req_test=cb_test, req_free=cb_free, coll_context=None, rank=self.rank,
                   size=self.size)

    # ---- persistent-style collective objects (init once, post many times is NOT offered by the
    # reference's NCCL team: a request is initialised, posted, tested and finalised per call)
    def collective(self, coll_type: int, src: int, dst: int, length: int = 0, count: int = 0, dt: int = DT_UINT8,
                   op: int = OP_SUM, root: int = 0, stream_handle_ptr: int = 0) -> C.c_void_p:
        a = CollOpArgs()
        a.field_mask = ARGS_FIELD_STREAM if stream_handle_ptr else 0
        a.coll_type = coll_type
        a.buffer_info.src_buffer, a.buffer_info.dst_buffer, a.buffer_info.len = src, dst, length
        a.reduce_info.dt, a.reduce_info.op, a.reduce_info.count = dt, op, count
        a.root, a.alg, a.tag = root, 0, 123
        if stream_handle_ptr:
            a.stream.type, a.stream.stream = 0, stream_handle_ptr
        req = C.c_void_p()
        _check(self.lib.xccl_collective_init(C.byref(a), C.byref(req), self.h_team), "xccl_collective_init")
        return req

    def post(self, req) -> None:
        _check(self.lib.xccl_collective_post(req), "xccl_collective_post")

    def test(self, req) -> int:
        return self.lib.xccl_collective_test(req)

    def wait(self, req) -> None:
        while True:
            st = self.lib.xccl_collective_test(req)
            if st == OK:
                return
            if st != INPROGRESS:
                raise RefError(f"reference xccl_collective_test failed with status {st}")
            self.lib.xccl_context_progress(self.h_ctx)

    def finalize(self, req) -> None:
        _check(self.lib.xccl_collective_finalize(req), "xccl_collective_finalize")

    def close(self) -> None:
        if self.h_team:
            self.lib.xccl_team_destroy(self.h_team)
            self.h_team = None
        if self.h_ctx:
            self.lib.xccl_context_destroy(self.h_ctx)
            self.h_ctx = None
        if self.h_lib:
            self.lib.xccl_lib_cleanup(self.h_lib)
            self.h_lib = None
