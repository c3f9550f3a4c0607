"""ctypes view of the public C API in ``include/xccl/xccl.h``.

Only declarations live here: structure layouts, enum values and function prototypes of
``libxccl.so``. The object-level wrapper is :mod:`xccl_b200.api`.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "lib"
_LIB_PATH = _LIB_DIR / "libxccl.so"

# ---------------------------------------------------------------- enums (values of xccl.h)
OK, INPROGRESS = 0, 1
ERR_NO_MESSAGE, ERR_NO_RESOURCE, ERR_NO_MEMORY, ERR_INVALID_PARAM = -1, -2, -4, -5
ERR_UNREACHABLE, ERR_NOT_IMPLEMENTED, ERR_MESSAGE_TRUNCATED, ERR_NO_PROGRESS = -6, -8, -9, -10
ERR_BUFFER_TOO_SMALL, ERR_NO_ELEM = -11, -12
ERR_UNSUPPORTED, ERR_TIMED_OUT = -22, -30

(BARRIER, BCAST, ALLREDUCE, REDUCE, ALLTOALL, ALLTOALLV, ALLGATHER, FANIN, FANOUT, FANOUT_GET,
 REDUCE_SCATTER, COLL_LAST) = range(12)

(OP_MAX, OP_MIN, OP_SUM, OP_PROD, OP_AND, OP_OR, OP_XOR, OP_LAND, OP_LOR, OP_LXOR, OP_BAND, OP_BOR,
 OP_BXOR, OP_MAXLOC, OP_MINLOC, OP_LAST, OP_UNSUPPORTED) = range(17)

(DT_INT8, DT_INT16, DT_INT32, DT_INT64, DT_INT128, DT_UINT8, DT_UINT16, DT_UINT32, DT_UINT64,
 DT_UINT128, DT_FLOAT16, DT_FLOAT32, DT_FLOAT64, DT_BFLOAT16, DT_LAST, DT_UNSUPPORTED) = range(16)

DT_SIZE = {DT_INT8: 1, DT_INT16: 2, DT_INT32: 4, DT_INT64: 8, DT_INT128: 16, DT_UINT8: 1, DT_UINT16: 2,
           DT_UINT32: 4, DT_UINT64: 8, DT_UINT128: 16, DT_FLOAT16: 2, DT_FLOAT32: 4, DT_FLOAT64: 8,
           DT_BFLOAT16: 2}

TL_UCX, TL_HIER, TL_SHARP, TL_HMC, TL_SHMSEG, TL_MRAIL, TL_NCCL, TL_MPOD, TL_NVLINK = (1 << i for i in range(9))
TL_ALL = 511
TL_NAMES = {TL_UCX: "ucx", TL_HIER: "hier", TL_SHARP: "sharp", TL_HMC: "hmc", TL_SHMSEG: "shmseg",
            TL_MRAIL: "mrail", TL_NCCL: "nccl", TL_MPOD: "mpod", TL_NVLINK: "nvlink"}

MEM_HOST, MEM_CUDA = 0, 1
THREAD_MULTIPLE, THREAD_SINGLE = 1, 2
EP_RANGE_UNDEFINED, EP_RANGE_FULL, EP_RANGE_STRIDED, EP_RANGE_MAP, EP_RANGE_CB = range(5)

LIB_PARAM_REPRODUCIBLE, LIB_PARAM_THREAD_MODE, LIB_PARAM_TEAM_USAGE, LIB_PARAM_COLL_TYPES = 1, 2, 4, 16
CTX_PARAM_THREAD_MODE, CTX_PARAM_COMPLETION, CTX_PARAM_OOB, CTX_PARAM_TLS = 1, 2, 4, 8
TEAM_PARAM_EP_RANGE, TEAM_PARAM_OOB = 1, 2
ARGS_FIELD_STREAM, ARGS_FIELD_EPILOGUE = 1, 2
MEM_MAP_ADDRESS, MEM_MAP_LENGTH, MEM_MAP_ROOT = 1, 2, 4
IN_PLACE = 1

HOST_ALG_LINEAR, HOST_ALG_KNOMIAL, HOST_ALG_SRA = 0, 1, 2
NVLINK_ALG_AUTO, NVLINK_ALG_ONE_SHOT, NVLINK_ALG_TWO_SHOT, NVLINK_ALG_NVLS, NVLINK_ALG_DIRECT = 0, 1, 2, 3, 4
NVLINK_ALG_SYMMETRIC = 5


# ---------------------------------------------------------------- structures
class LibParams(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("reproducible", C.c_uint), ("thread_mode", C.c_uint),
                ("team_usage", C.c_uint64), ("coll_types", C.c_uint64)]


class _Strided(C.Structure):
    _fields_ = [("start", C.c_int), ("stride", C.c_int)]


class _Map(C.Structure):
    _fields_ = [("map", C.POINTER(C.c_int))]


RANGE_CB = C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)


class _Cb(C.Structure):
    _fields_ = [("cb", RANGE_CB), ("cb_ctx", C.c_void_p)]


class _RangeU(C.Union):
    _fields_ = [("strided", _Strided), ("map", _Map), ("cb", _Cb)]


class EpRange(C.Structure):
    _anonymous_ = ("u",)
    _fields_ = [("type", C.c_int), ("ep_num", C.c_int), ("u", _RangeU)]


OOB_ALLGATHER = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, EpRange, C.c_void_p,
                            C.POINTER(C.c_void_p))
OOB_TEST = C.CFUNCTYPE(C.c_int, C.c_void_p)
OOB_FREE = C.CFUNCTYPE(C.c_int, C.c_void_p)


class Oob(C.Structure):
    _fields_ = [("allgather", OOB_ALLGATHER), ("req_test", OOB_TEST), ("req_free", OOB_FREE),
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
                ("dst_displacements", C.POINTER(C.c_uint32)), ("dst_datatype", C.c_int),
                ("len", C.c_size_t)]


class GetInfo(C.Structure):
    _fields_ = [("memh", C.c_void_p), ("offset", C.c_ssize_t), ("local_buffer", C.c_void_p),
                ("len", C.c_size_t)]


class _ArgsU(C.Union):
    _fields_ = [("buffer_info", BufferInfo), ("get_info", GetInfo)]


class Alg(C.Structure):
    _fields_ = [("set_by_user", C.c_uint8, 1), ("id", C.c_uint8, 7)]


class Stream(C.Structure):
    _fields_ = [("type", C.c_int), ("stream", C.c_void_p)]


class Epilogue(C.Structure):
    _fields_ = [("scale", C.c_float), ("out_dt", C.c_int)]


class CollArgs(C.Structure):
    _anonymous_ = ("u",)
    _fields_ = [("field_mask", C.c_uint64), ("coll_type", C.c_int), ("u", _ArgsU),
                ("reduce_info", ReduceInfo), ("root", C.c_int), ("alg", Alg), ("tag", C.c_uint16),
                ("stream", Stream), ("epilogue", Epilogue)]


class MemMapParams(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("address", C.c_void_p), ("length", C.c_size_t),
                ("root", C.c_int)]


class CtxAttr(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("supported_colls", C.c_uint64)]


class TlAttr(C.Structure):
    _fields_ = [("field_mask", C.c_uint64), ("context_create_mode", C.c_int), ("devices_count", C.c_int),
                ("devices", C.c_void_p)]


# ---------------------------------------------------------------- library handle
_lib = None


def lib_path() -> Path:
    return _LIB_PATH


def load() -> C.CDLL:
    """Loads libxccl.so (building it first when it is missing and a compiler is present)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _LIB_PATH
    alt = os.environ.get("XCCL_B200_LIB")  # e.g. the sanitizer build, xccl_b200/lib/libxccl_address.so
    if alt:
        path = Path(alt)
    elif not _LIB_PATH.exists():
        from . import build as _build
        _build.build_native()
    _lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    _declare(_lib)
    return _lib


def _declare(L: C.CDLL) -> None:
    vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
    P = C.POINTER

    def fn(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    fn("xccl_status_str", C.c_char_p, i)
    fn("xccl_lib_config_read", i, C.c_char_p, C.c_char_p, P(vp))
    fn("xccl_lib_config_release", None, vp)
    fn("xccl_lib_config_print", None, vp, vp, C.c_char_p, C.c_uint)
    fn("xccl_lib_init", i, P(LibParams), vp, P(vp))
    fn("xccl_lib_cleanup", None, vp)
    fn("xccl_get_tl_list", i, vp, P(P(i)), P(C.c_uint))
    fn("xccl_free_tl_list", None, P(i))
    fn("xccl_tl_query", i, vp, P(i), P(TlAttr))
    fn("xccl_ctx_query", i, vp, P(CtxAttr))
    fn("xccl_context_config_read", i, vp, C.c_char_p, C.c_char_p, P(vp))
    fn("xccl_context_config_modify", i, P(i), vp, C.c_char_p, C.c_char_p)
    fn("xccl_context_config_release", None, vp)
    fn("xccl_context_create", i, vp, P(ContextParams), vp, P(vp))
    fn("xccl_context_progress", i, vp)
    fn("xccl_context_destroy", i, vp)
    fn("xccl_team_create_post", i, vp, P(TeamParams), P(vp))
    fn("xccl_team_create_test", i, vp)
    fn("xccl_team_destroy", None, vp)
    fn("xccl_team_query", i, vp, P(i), P(i))
    fn("xccl_team_coll_tl", i, vp, i, i)
    fn("xccl_collective_init", i, P(CollArgs), P(vp), vp)
    fn("xccl_collective_post", i, vp)
    fn("xccl_collective_wait", i, vp)
    fn("xccl_collective_test", i, vp)
    fn("xccl_collective_finalize", i, vp)
    fn("xccl_collective_elapsed_us", C.c_double, vp)
    fn("xccl_global_mem_map_start", i, vp, MemMapParams, P(vp))
    fn("xccl_global_mem_map_test", i, vp)
    fn("xccl_global_mem_unmap", i, vp)
    fn("xccl_oob_shm_create", i, C.c_char_p, i, i, P(Oob))
    fn("xccl_oob_shm_destroy", None, P(Oob))
    fn("xccl_oob_sub_create", i, P(Oob), P(i), i, P(Oob))
    fn("xccl_oob_sub_destroy", None, P(Oob))
    fn("xccl_oob_allgather", i, P(Oob), vp, vp, sz)
    fn("xccl_mem_reduce", i, vp, vp, vp, sz, i, i)
    fn("xccl_mem_reduce_multi", i, vp, vp, vp, sz, sz, sz, i, i)
    fn("xccl_mem_type", i, vp)
    fn("xccl_host_knomial_peers", i, i, i, i, i, P(i), P(i), P(i), P(i))
    for name, res, args in _OPTIONAL:
        if hasattr(L, name):
            fn(name, res, *args)


# Entry points that exist only once the corresponding component is built in.
_OPTIONAL: list = []


def optional(name, res, *args):
    _OPTIONAL.append((name, res, args))
    if _lib is not None and hasattr(_lib, name):
        f = getattr(_lib, name)
        f.restype = res
        f.argtypes = list(args)


def status_str(st: int) -> str:
    return load().xccl_status_str(st).decode()
