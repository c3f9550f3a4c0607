"""The allocation-free allreduce entry point (``csrc/tl/nvlink/nvl_noalloc.h``).

Some users of the library may not allocate device memory at the moment they need a collective:
they run inside an allocator callback, they are a plugin in a process whose memory pool belongs
to the host application, or they sit on a path where a cudaMalloc (which may synchronise the
device) is not acceptable. For them the library exports one function whose scratch memory is a
static device array. This test calls that function through its C symbol, twice in a row, and
compares every rank's output with what the regular (allocating) emulated allreduce produces for
the same inputs. The file sorts last so that it runs after every other test.
"""
import ctypes as C

import pytest
import torch

from xccl_b200 import _capi as K

pytestmark = pytest.mark.gpu

MAX_RANKS, MAX_COUNT = 8, 16384


def _entry():
    L = K.load()
    fn = L.xccl_emu_allreduce_f32_sum_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_void_p]
    return fn


def _ptrs(ts):
    arr = (C.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        arr[i] = t.data_ptr()
    return arr


def test_no_alloc_allreduce_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from xccl_b200.ops.emu import EmuWorld
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    fn = _entry()
    n, count = 4, 10007
    world = EmuWorld(n, 8 << 20)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        for call in range(2):
            g = torch.Generator(device=dev).manual_seed(100 + call)
            srcs = [torch.randn(count, device=dev, generator=g) for _ in range(n)]
            want = [torch.empty_like(s) for s in srcs]
            got = [torch.full_like(s, float("nan")) for s in srcs]
            world.allreduce(srcs, want, alg=K.NVLINK_ALG_ONE_SHOT)   # the existing entry point
            torch.cuda.synchronize()
            if call == 0:
                st = fn(_ptrs(srcs), _ptrs(got), n, count, stream)    # the allocation-free one; first call: set-up
                assert st == K.OK, K.status_str(st)
            else:
                # free bytes of the device, as the driver sees them: a cudaMalloc inside the library would show
                # here (torch's own counters only see torch's caching allocator)
                free_before = torch.cuda.mem_get_info()[0]
                st = fn(_ptrs(srcs), _ptrs(got), n, count, stream)
                assert st == K.OK, K.status_str(st)
                assert torch.cuda.mem_get_info()[0] == free_before
            for r in range(n):
                torch.testing.assert_close(got[r], want[r], rtol=1e-5, atol=1e-5)
                torch.testing.assert_close(got[r], torch.stack(srcs).double().sum(0).float(), rtol=1e-5, atol=1e-5)
    finally:
        world.close()


def test_no_alloc_allreduce_rejects_sizes_beyond_its_scratch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    fn = _entry()
    t = [torch.zeros(8, device="cuda:0") for _ in range(2)]
    assert fn(_ptrs(t), _ptrs(t), 2, MAX_COUNT + 1, None) == K.ERR_BUFFER_TOO_SMALL
    assert fn(_ptrs(t), _ptrs(t), MAX_RANKS + 1, 8, None) == K.ERR_BUFFER_TOO_SMALL
