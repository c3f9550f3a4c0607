"""GPU tests of the hand-written kernels against plain PyTorch fp32 references.

The multi-rank NVLink kernels run here through the single-GPU emulation (one cooperative launch
whose blockIdx.y is the rank); the real multi-process path has its own test module.
"""
import ctypes as C

import os

import pytest
import torch

from xccl_b200 import _capi as K

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def _loaded_native():
    # fail loudly if the native library is not the thing that runs
    with open("/proc/self/maps") as f:
        assert "libxccl.so" in f.read(), "libxccl.so is not loaded"


# ----------------------------------------------------------------------------- local reduce kernels
@pytest.mark.parametrize("dtype,dt", [(torch.float32, K.DT_FLOAT32), (torch.bfloat16, K.DT_BFLOAT16),
                                      (torch.float16, K.DT_FLOAT16), (torch.int32, K.DT_INT32),
                                      (torch.int64, K.DT_INT64), (torch.uint8, K.DT_UINT8)])
@pytest.mark.parametrize("count", [1, 7, 4099, 1 << 20])
def test_reduce_multi_kernel(dev, dtype, dt, count):
    from xccl_b200.ops import emu  # noqa: F401  (declares optional prototypes)
    L = K.load()
    L.xccl_cuda_reduce_multi.restype = C.c_int
    L.xccl_cuda_reduce_multi.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                         C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    g = torch.Generator(device="cpu").manual_seed(0)
    nvec = 5
    hi = 4 if dtype == torch.uint8 else 9
    a = torch.randint(0, hi, (count,), generator=g).to(dtype).to(dev)
    v = torch.randint(0, hi, (nvec, count), generator=g).to(dtype).to(dev)
    out = torch.empty_like(a)
    for op, ref in ((K.OP_SUM, lambda x: x.sum(0)), (K.OP_MAX, lambda x: x.max(0).values)):
        st = L.xccl_cuda_reduce_multi(a.data_ptr(), v.data_ptr(), out.data_ptr(), nvec, count,
                                      count * a.element_size(), dt, op, 1.0, K.DT_UNSUPPORTED,
                                      torch.cuda.current_stream().cuda_stream)
        assert st == K.OK
        allv = torch.cat([a[None], v]).to(torch.float64 if dtype.is_floating_point else torch.int64)
        want = ref(allv).to(dtype)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (dtype, op, count)
    _loaded_native()


def test_reduce_scale_and_cast(dev):
    L = K.load()
    L.xccl_cuda_reduce_multi.restype = C.c_int
    L.xccl_cuda_reduce_multi.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                         C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    n = 100003
    a = torch.randn(n, device=dev)
    v = torch.randn(3, n, device=dev)
    out = torch.empty(n, device=dev, dtype=torch.bfloat16)
    st = L.xccl_cuda_reduce_multi(a.data_ptr(), v.data_ptr(), out.data_ptr(), 3, n, n * 4, K.DT_FLOAT32, K.OP_SUM,
                                  0.25, K.DT_BFLOAT16, torch.cuda.current_stream().cuda_stream)
    assert st == K.OK
    want = ((a + v.sum(0)) * 0.25).to(torch.bfloat16)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), want.float(), rtol=1e-2, atol=1e-2)


def test_stream_hold_times_out_without_hanging(dev):
    L = K.load()
    L.xccl_cuda_hold_timeout_probe.restype = C.c_int
    L.xccl_cuda_hold_timeout_probe.argtypes = [C.c_int, C.POINTER(C.c_float)]
    ms = C.c_float()
    st = L.xccl_cuda_hold_timeout_probe(50, C.byref(ms))
    assert st == K.ERR_TIMED_OUT
    assert 40.0 <= ms.value < 2000.0
    # the context is still usable
    assert float(torch.ones(4, device=dev).sum()) == 4.0


# ----------------------------------------------------------------------------- emulated NVLink team
@pytest.fixture(scope="module")
def world4(dev):
    from xccl_b200.ops.emu import EmuWorld
    w = EmuWorld(4, 8 << 20)
    yield w
    w.close()


def _ints(n, count, dtype, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randint(-8, 9, (count,), generator=g).to(dtype).to(dev) for _ in range(n)]


@pytest.mark.parametrize("alg", [K.NVLINK_ALG_ONE_SHOT, K.NVLINK_ALG_TWO_SHOT])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
@pytest.mark.parametrize("count", [1, 33, 4096, 262147])
def test_emu_allreduce(world4, dev, alg, dtype, count):
    if alg == K.NVLINK_ALG_ONE_SHOT and count * 4 * 4 > (4 << 20):
        pytest.skip("one-shot needs size x message bytes in one workspace half")
    srcs = _ints(4, count, dtype, dev, seed=count)
    dsts = [torch.full_like(s, 99) for s in srcs]
    world4.allreduce(srcs, dsts, alg=alg)
    want = torch.stack([s.double() for s in srcs]).sum(0).to(dtype)
    for d in dsts:
        assert torch.equal(d, want)
    # max
    world4.allreduce(srcs, dsts, op=K.OP_MAX, alg=alg)
    want = torch.stack(srcs).max(0).values
    for d in dsts:
        assert torch.equal(d, want)


def test_emu_allreduce_chunks_through_small_workspace(world4, dev):
    # 12 MB per rank through a workspace half of 4 MB: three chunks, alternating halves
    count = 3 << 20
    srcs = [torch.randn(count, device=dev) for _ in range(4)]
    dsts = [torch.empty_like(s) for s in srcs]
    world4.allreduce(srcs, dsts, alg=K.NVLINK_ALG_TWO_SHOT)
    want = torch.stack(srcs).double().sum(0).float()
    for d in dsts:
        torch.testing.assert_close(d, want, rtol=1e-5, atol=1e-5)
    assert torch.equal(dsts[0], dsts[3])  # every rank adds in the same order


def test_emu_allreduce_fused_scale_cast_and_unaligned(world4, dev):
    count = 10007
    base = [torch.randn(count + 3, device=dev) for _ in range(4)]
    srcs = [b[3:] for b in base]  # 12-byte offset: not 16-byte aligned
    dsts = [torch.empty(count + 1, device=dev, dtype=torch.bfloat16)[1:] for _ in range(4)]
    for alg in (K.NVLINK_ALG_ONE_SHOT, K.NVLINK_ALG_TWO_SHOT):
        world4.allreduce(srcs, dsts, alg=alg, scale=0.25)
        want = (torch.stack(srcs).double().sum(0) * 0.25).float()
        for d in dsts:
            torch.testing.assert_close(d.float(), want, rtol=1e-2, atol=2e-2)


def test_emu_reduce_and_reduce_scatter(world4, dev):
    count = 5000
    srcs = _ints(4, count, torch.float32, dev, seed=3)
    for root in range(4):
        dsts = [torch.full((count,), -1.0, device=dev) for _ in range(4)]
        world4.reduce(srcs, dsts, root)
        assert torch.equal(dsts[root], torch.stack(srcs).sum(0))
        for r in range(4):
            if r != root:
                assert torch.all(dsts[r] == -1.0)
    per = 1237
    srcs = _ints(4, per * 4, torch.int32, dev, seed=4)
    dsts = [torch.zeros(per, dtype=torch.int32, device=dev) for _ in range(4)]
    world4.reduce_scatter(srcs, dsts)
    full = torch.stack(srcs).sum(0)
    for r in range(4):
        assert torch.equal(dsts[r], full[r * per:(r + 1) * per].to(torch.int32))


def test_emu_bcast_allgather_alltoall(world4, dev):
    n = 4
    for nbytes in (1, 13, 4096, 3 << 20):
        bufs = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev) for _ in range(n)]
        root = 2
        want = bufs[root].clone()
        world4.bcast(bufs, bufs, root)
        for b in bufs:
            assert torch.equal(b, want)
    for per in (3, 1000, 1 << 20):
        srcs = [torch.randint(0, 255, (per,), dtype=torch.uint8, device=dev) for _ in range(n)]
        dsts = [torch.zeros(per * n, dtype=torch.uint8, device=dev) for _ in range(n)]
        world4.allgather(srcs, dsts)
        for d in dsts:
            assert torch.equal(d, torch.cat(srcs))
    for per in (1, 1024, 100003):
        srcs = [torch.randn(per * n, device=dev) for _ in range(n)]
        dsts = [torch.zeros(per * n, device=dev) for _ in range(n)]
        world4.alltoall(srcs, dsts)
        for r in range(n):
            want = torch.cat([srcs[s][r * per:(r + 1) * per] for s in range(n)])
            assert torch.equal(dsts[r], want)


def test_emu_direct_zero_copy_algorithms(world4, dev):
    """The direct kernels read and write the ranks' own buffers (no workspace): allreduce with the fused
    scale and cast, in place, reduce-scatter, allgather (also in place) and alltoall."""
    n = 4
    D = K.NVLINK_ALG_DIRECT
    for dtype, count in ((torch.float32, 4 * 5000), (torch.bfloat16, 8 * 70001), (torch.float16, 8 * 16)):
        srcs = _ints(n, count, dtype, dev, seed=11)
        dsts = [torch.zeros(count, dtype=dtype, device=dev) for _ in range(n)]
        world4.allreduce(srcs, dsts, alg=D)
        want = torch.stack([s.float() for s in srcs]).sum(0)
        for d in dsts:
            assert torch.equal(d.float(), want)
    srcs = [torch.randn(4 * 3000, device=dev) for _ in range(n)]
    want = torch.stack(srcs).sum(0) * 0.25
    outs = [torch.zeros(4 * 3000, dtype=torch.bfloat16, device=dev) for _ in range(n)]
    world4.allreduce(srcs, outs, alg=D, scale=0.25)          # fp32 -> bf16 with the average fused
    for o in outs:
        torch.testing.assert_close(o.float(), want, rtol=1e-2, atol=1e-2)
    bufs = [s.clone() for s in srcs]
    world4.allreduce(bufs, bufs, alg=D, op=K.OP_MAX)        # in place
    for b in bufs:
        assert torch.equal(b, torch.stack(srcs).max(0).values)
    per = 4 * 1237
    srcs = _ints(n, per * n, torch.float32, dev, seed=12)
    dsts = [torch.zeros(per, device=dev) for _ in range(n)]
    world4.reduce_scatter(srcs, dsts, alg=D)
    full = torch.stack(srcs).sum(0)
    for r in range(n):
        assert torch.equal(dsts[r], full[r * per:(r + 1) * per])
    per = 16 * 4099
    srcs = [torch.randint(0, 255, (per,), dtype=torch.uint8, device=dev) for _ in range(n)]
    dsts = [torch.zeros(per * n, dtype=torch.uint8, device=dev) for _ in range(n)]
    world4.allgather(srcs, dsts, alg=D)
    for d in dsts:
        assert torch.equal(d, torch.cat(srcs))
    inplace = [torch.zeros(per * n, dtype=torch.uint8, device=dev) for _ in range(n)]
    for r in range(n):
        inplace[r][r * per:(r + 1) * per] = srcs[r]
    world4.allgather([inplace[r][r * per:(r + 1) * per] for r in range(n)], inplace, alg=D)
    for d in inplace:
        assert torch.equal(d, torch.cat(srcs))
    per = 4 * 25001
    srcs = [torch.randn(per * n, device=dev) for _ in range(n)]
    dsts = [torch.zeros(per * n, device=dev) for _ in range(n)]
    world4.alltoall(srcs, dsts, alg=D)
    for r in range(n):
        assert torch.equal(dsts[r], torch.cat([srcs[s][r * per:(r + 1) * per] for s in range(n)]))


class _Guarded:
    """A byte buffer with 256 sentinel bytes before and after the part a kernel may touch, placed at an odd
    offset so that the payload is not 16-byte aligned: an out-of-bounds pack store shows up in the guards."""
    PAD = 256

    def __init__(self, nbytes, dev, fill=0xA5, skew=3):
        self.raw = torch.full((nbytes + 2 * self.PAD + 16,), fill, dtype=torch.uint8, device=dev)
        self.off = self.PAD + skew
        self.n, self.fill = nbytes, fill

    @property
    def view(self):
        return self.raw[self.off:self.off + self.n]

    def guards_intact(self):
        return bool(torch.all(self.raw[:self.off] == self.fill)) and bool(torch.all(self.raw[self.off + self.n:] == self.fill))


def test_emu_byte_collectives_stay_inside_their_buffers(world4, dev):
    """bcast / allgather / alltoall on unaligned, odd-sized byte buffers: results exact, sources untouched,
    not one byte written outside the destination."""
    n = 4
    for per in (1, 13, 4099, 70001):
        srcs = [_Guarded(per, dev, fill=0x11) for _ in range(n)]
        for r, g in enumerate(srcs):
            g.view.copy_(torch.randint(0, 255, (per,), dtype=torch.uint8, generator=torch.Generator().manual_seed(per + r)).to(dev))
        keep = [g.view.clone() for g in srcs]
        dsts = [_Guarded(per * n, dev) for _ in range(n)]
        world4.allgather([g.view for g in srcs], [g.view for g in dsts])
        for g in dsts:
            assert torch.equal(g.view, torch.cat(keep)) and g.guards_intact(), ("allgather", per)
        a_src = [_Guarded(per * n, dev, fill=0x22) for _ in range(n)]
        for r, g in enumerate(a_src):
            g.view.copy_(torch.randint(0, 255, (per * n,), dtype=torch.uint8, generator=torch.Generator().manual_seed(7 * per + r)).to(dev))
        a_keep = [g.view.clone() for g in a_src]
        a_dst = [_Guarded(per * n, dev) for _ in range(n)]
        world4.alltoall([g.view for g in a_src], [g.view for g in a_dst])
        for r in range(n):
            want = torch.cat([a_keep[s][r * per:(r + 1) * per] for s in range(n)])
            assert torch.equal(a_dst[r].view, want) and a_dst[r].guards_intact(), ("alltoall", per)
        for g, k in zip(srcs + a_src, keep + a_keep):
            assert torch.equal(g.view, k) and g.guards_intact(), ("source modified", per)
        bufs = [_Guarded(per, dev) for _ in range(n)]
        bufs[1].view.copy_(keep[1])
        world4.bcast([g.view for g in bufs], [g.view for g in bufs], root=1)
        for g in bufs:
            assert torch.equal(g.view, keep[1]) and g.guards_intact(), ("bcast", per)


def test_emu_push_allgather_alltoall(world4, dev):
    """The push forms (stores into the destinations' workspaces) on odd, unaligned byte buffers, between pull-form
    calls so that both share the workspace parity bookkeeping."""
    n = 4
    for per in (1, 13, 4099, 70001):
        srcs = [_Guarded(per * n, dev, fill=0x11) for _ in range(n)]
        dsts = [_Guarded(per * n, dev, fill=0x22) for _ in range(n)]
        for r in range(n):
            srcs[r].view.copy_((torch.arange(per * n, device=dev) * 7 + r * 31) % 251)
        world4.alltoall([s.view for s in srcs], [d.view for d in dsts], alg=K.NVLINK_ALG_ONE_SHOT)
        for r in range(n):
            want = torch.cat([srcs[q].view[r * per:(r + 1) * per] for q in range(n)])
            assert torch.equal(dsts[r].view, want) and dsts[r].guards_intact(), ("alltoall push", per, r)
        parts = [_Guarded(per, dev, fill=0x33) for _ in range(n)]
        for r in range(n):
            parts[r].view.copy_((torch.arange(per, device=dev) * 3 + r * 17) % 253)
        world4.allgather([p_.view for p_ in parts], [d.view for d in dsts], alg=K.NVLINK_ALG_ONE_SHOT)
        want = torch.cat([p_.view for p_ in parts])
        for r in range(n):
            assert torch.equal(dsts[r].view, want) and dsts[r].guards_intact(), ("allgather push", per, r)
        world4.allgather([p_.view for p_ in parts], [d.view for d in dsts])   # pull form next to it
        for r in range(n):
            assert torch.equal(dsts[r].view, want)


def test_emu_alltoallv(world4, dev):
    n = 4
    sc = [[(s * 3 + d * 5 + 1) for d in range(n)] for s in range(n)]  # elements rank s sends to rank d
    srcs, dsts, metas, keep = [], [], [], []
    for r in range(n):
        scounts = sc[r]
        sdispl = [sum(scounts[:d]) for d in range(n)]
        rcounts = [sc[s][r] for s in range(n)]
        rdispl = [sum(rcounts[:s]) for s in range(n)]
        srcs.append(torch.cat([torch.full((scounts[d],), float(r * 10 + d), device=dev) for d in range(n)]))
        dsts.append(torch.zeros(sum(rcounts), device=dev))
        metas.append(torch.tensor(scounts + sdispl + rcounts + rdispl, dtype=torch.int32, device=dev))
        keep.append((rcounts,))
    world4.alltoallv(srcs, dsts, metas, max(s.numel() for s in srcs) * 4)
    for r in range(n):
        want = torch.cat([torch.full((sc[s][r],), float(s * 10 + r), device=dev) for s in range(n)])
        assert torch.equal(dsts[r], want)


def test_emu_alltoallv_larger_than_the_workspace(dev):
    """Uneven counts whose streams are several workspace halves long (and of different length per rank, one rank
    sending nothing): the kernel walks the exchange in windows and agrees on the number of rounds from the headers."""
    from xccl_b200.ops.emu import EmuWorld
    n = 4
    w = EmuWorld(n, 256 << 10)   # halves of 128 KiB, 8 KiB of it header
    try:
        for trial in range(2):   # the second exchange starts on the other workspace half
            sc = [[(7919 * (s + 1) + 15013 * d + 3 + trial) * (0 if s == 2 else 1) for d in range(n)] for s in range(n)]
            sc[1][3] = 0
            srcs, dsts, metas = [], [], []
            g = torch.Generator(device=dev).manual_seed(5 + trial)
            for r in range(n):
                scounts = sc[r]
                sdispl = [sum(scounts[:d]) for d in range(n)]
                rcounts = [sc[s][r] for s in range(n)]
                rdispl = [sum(rcounts[:s]) for s in range(n)]
                srcs.append(torch.randn(max(sum(scounts), 1), device=dev, generator=g))
                dsts.append(torch.full((max(sum(rcounts), 1) + 4,), -1.0, device=dev))
                metas.append(torch.tensor(scounts + sdispl + rcounts + rdispl, dtype=torch.int32, device=dev))
            assert max(sum(x) for x in sc) * 4 > 3 * (128 << 10)
            w.alltoallv(srcs, dsts, metas, max(sum(x) for x in sc) * 4)
            for r in range(n):
                parts = []
                for s_ in range(n):
                    o = sum(sc[s_][:r])
                    parts.append(srcs[s_][o:o + sc[s_][r]])
                want = torch.cat(parts)
                assert torch.equal(dsts[r][:want.numel()], want), (trial, r)
                assert torch.all(dsts[r][want.numel():] == -1.0)
            # the workspace parity bookkeeping still holds for what follows
            a = _ints(n, 3000, torch.float32, dev, seed=trial)
            b = [torch.empty_like(x) for x in a]
            w.allreduce(a, b, alg=K.NVLINK_ALG_TWO_SHOT)
            assert torch.equal(b[3], torch.stack(a).sum(0))
    finally:
        w.close()


_BOUNDS_SCRIPT = r"""
import ctypes as C, torch
from xccl_b200 import _capi as K
from xccl_b200.ops.emu import EmuWorld
dev = torch.device("cuda:0")
L = K.load()
rep = (C.c_ulonglong * 4)()
L.xccl_nvlink_debug_bounds_report.restype = C.c_int
assert L.xccl_nvlink_debug_bounds_report(rep) == K.OK, "not a bounds-checking build"
n = 4
w = EmuWorld(n, 1 << 20)            # small halves: the chunk loops, window rounds and parity changes all run
g = torch.Generator(device=dev).manual_seed(0)
for count in (1, 1000, 70001, 300000):
    srcs = [torch.randn(count, device=dev, generator=g) for _ in range(n)]
    dsts = [torch.empty_like(s) for s in srcs]
    for alg in (K.NVLINK_ALG_ONE_SHOT, K.NVLINK_ALG_TWO_SHOT, K.NVLINK_ALG_DIRECT):
        if alg == K.NVLINK_ALG_ONE_SHOT and count * 4 * n > (1 << 19):
            continue
        if alg == K.NVLINK_ALG_DIRECT and count % 4:
            continue
        w.allreduce(srcs, dsts, alg=alg)
        torch.testing.assert_close(dsts[2], torch.stack(srcs).sum(0), rtol=1e-5, atol=1e-5)
    w.reduce(srcs, dsts, root=1)
    rs = [torch.randn(count * n, device=dev, generator=g) for _ in range(n)]
    rd = [torch.empty(count, device=dev) for _ in range(n)]
    w.reduce_scatter(rs, rd)
for per in (13, 4099, 200003):
    bs = [torch.randint(0, 255, (per * n,), dtype=torch.uint8, device=dev) for _ in range(n)]
    bd = [torch.empty_like(b) for b in bs]
    w.alltoall(bs, bd)
    w.alltoall(bs, bd, alg=K.NVLINK_ALG_ONE_SHOT)
    w.bcast(bs, bd, 2)
    ps = [torch.randint(0, 255, (per,), dtype=torch.uint8, device=dev) for _ in range(n)]
    w.allgather(ps, bd)
    w.allgather(ps, bd, alg=K.NVLINK_ALG_ONE_SHOT)
sc = [[(7919 * (s + 1) + 15013 * d + 3) for d in range(n)] for s in range(n)]
srcs, dsts, metas = [], [], []
for r in range(n):
    rc = [sc[s][r] for s in range(n)]
    srcs.append(torch.randn(sum(sc[r]), device=dev, generator=g))
    dsts.append(torch.empty(sum(rc), device=dev))
    metas.append(torch.tensor(sc[r] + [sum(sc[r][:d]) for d in range(n)] + rc + [sum(rc[:s]) for s in range(n)],
                              dtype=torch.int32, device=dev))
w.alltoallv(srcs, dsts, metas, max(s.numel() for s in srcs) * 4)
assert torch.equal(dsts[1][:sc[0][1]], srcs[0][sc[0][0]:sc[0][0] + sc[0][1]])
w.barrier()
assert L.xccl_nvlink_debug_bounds_report(rep) == K.OK
w.close()
print("violations", rep[0], hex(rep[1]), rep[2], rep[3])
assert rep[0] == 0
"""


def test_emu_collectives_under_the_bounds_checking_build(dev):
    """Every NVLink collective with all ranks emulated, on the library built with -DXCCL_DEBUG_BOUNDS: each 16-byte
    access to a workspace or a peer buffer is checked against the ranges of its launch, an access outside them is
    recorded and skipped. Results stay right and the record stays empty."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    lib = root / "xccl_b200" / "lib" / "libxccl_bounds.so"
    if not lib.exists():
        pytest.skip("libxccl_bounds.so is not built (python -m xccl_b200.build --debug-bounds)")
    env = dict(os.environ, XCCL_B200_LIB=str(lib), PYTHONPATH=str(root))
    r = subprocess.run([sys.executable, "-c", _BOUNDS_SCRIPT], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "violations 0" in r.stdout


def test_emu_sync_collectives_and_bounded_wait(world4, dev):
    for _ in range(3):
        world4.barrier()
    for root in range(4):
        world4.fanin(root)
        world4.fanout(root)
    st, ms, st4 = world4.timeout_probe(30)
    assert st == K.ERR_TIMED_OUT and st4[0] == 1
    assert 20.0 <= ms < 2000.0
    # the team still works after the probe
    srcs = _ints(4, 100, torch.float32, dev, seed=9)
    dsts = [torch.empty_like(s) for s in srcs]
    world4.allreduce(srcs, dsts)
    assert torch.equal(dsts[1], torch.stack(srcs).sum(0))


def test_emu_allreduce_eight_ranks(dev):
    from xccl_b200.ops.emu import EmuWorld
    w = EmuWorld(8, 8 << 20)
    try:
        for count, alg in ((1000, K.NVLINK_ALG_ONE_SHOT), (300000, K.NVLINK_ALG_TWO_SHOT)):
            srcs = _ints(8, count, torch.bfloat16, dev, seed=count)
            dsts = [torch.empty_like(s) for s in srcs]
            w.allreduce(srcs, dsts, alg=alg)
            want = torch.stack([s.float() for s in srcs]).sum(0).to(torch.bfloat16)
            for d in dsts:
                assert torch.equal(d, want)
    finally:
        w.close()


# ----------------------------------------------------------------------------- tcgen05 GEMM
@pytest.mark.parametrize("M,N,K_", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (1000, 264, 520)])
def test_gemm_bf16_matches_fp32_reference(dev, M, N, K_):
    from xccl_b200.ops import gemm
    a = (torch.randn(M, K_, device=dev) * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K_, device=dev) * 0.5).to(torch.bfloat16)
    out = gemm.gemm_bf16(a, b)
    assert gemm.last_error() == 0
    want = a.float() @ b.float().t()
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2 * K_ ** 0.5)
    _loaded_native()


def test_gemm_swiglu_matches_fp32_reference(dev):
    from xccl_b200.ops import gemm
    M, F, K_ = 512, 384, 512
    a = (torch.randn(M, K_, device=dev) * 0.5).to(torch.bfloat16)
    wg = (torch.randn(F, K_, device=dev) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(F, K_, device=dev) * 0.05).to(torch.bfloat16)
    out = gemm.gemm_swiglu(a, wg, wu)
    assert gemm.last_error() == 0
    g = a.float() @ wg.float().t()
    u = a.float() @ wu.float().t()
    want = torch.nn.functional.silu(g) * u
    torch.testing.assert_close(out.float(), want, rtol=3e-2, atol=3e-2)


def test_gemm_many_tiles_persistent_schedule(dev):
    from xccl_b200.ops import gemm
    M, N, K_ = 4096, 4096, 512   # 512 tiles over 148 CTAs: several tiles per CTA, both accumulators in use
    a = (torch.randn(M, K_, device=dev) * 0.3).to(torch.bfloat16)
    b = (torch.randn(N, K_, device=dev) * 0.3).to(torch.bfloat16)
    out = gemm.gemm_bf16(a, b)
    assert gemm.last_error() == 0
    want = a.float() @ b.float().t()
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=0.5)


# ----------------------------------------------------------------------------- fused TP-MLP kernels
def _full_weights(mlp):
    wg = torch.cat(mlp.w_gate, 0)
    wu = torch.cat(mlp.w_up, 0)
    wd = torch.cat(mlp.w_down, 1)
    return wg, wu, wd


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_tp_mlp_fused_matches_fp32_reference(dev, tp):
    """allgather->GEMM(+SwiGLU) and GEMM->reduce-scatter, ranks emulated inside one launch."""
    from xccl_b200.models.tp_mlp import TpMlp, reference_forward_fp32
    tokens, hidden, ffn = 1024, 512, 1024
    mlp = TpMlp(tokens, hidden, ffn, tp=tp, emulate=True)
    try:
        g = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(tokens, hidden, device=dev, generator=g).to(torch.bfloat16)
        shards = list(x.chunk(tp, 0))
        for it in range(3):  # repeated launches: sequence numbers, parities and counters advance
            y = mlp.forward(shards)
            mlp.check_error()
            want = reference_forward_fp32(x, *_full_weights(mlp))
            got = torch.cat(y, 0).float()
            torch.testing.assert_close(got, want, rtol=3e-2, atol=3e-2)
        # the gathered buffer of every rank holds every shard
        for i in range(mlp.n_local):
            assert torch.equal(mlp.ws.x_full(i), x)
    finally:
        mlp.close()
    _loaded_native()


def test_tp_mlp_end_to_end_from_pinned_host(dev):
    from xccl_b200.models.tp_mlp import TpMlp
    mlp = TpMlp(512, 256, 512, tp=1)
    try:
        x = torch.randn(512, 256).to(torch.bfloat16).pin_memory()
        m = mlp.forward_from_host([x])
        mlp.check_error()
        assert m.device.type == "cpu" and torch.isfinite(m)
    finally:
        mlp.close()


@pytest.mark.parametrize("tp,phases", [(1, False), (2, False), (4, False), (4, True), (8, False), (8, True)])
def test_tp_mlp_input_arriving_from_host_overlaps_first_kernel(dev, tp, phases, monkeypatch):
    """The chunked host->device copy with stream-ordered flags: the kernel starts before the rows are there and
    must produce the same output as the plain copy-then-launch path, step after step. With copy CTAs (4 and 8
    ranks) and H2D_PHASES every rank reports its rows block by block and the tiles are walked in phases over all shards."""
    from xccl_b200.models.tp_mlp import TpMlp, reference_forward_fp32
    monkeypatch.setenv("XCCL_TP_H2D_OVERLAP", "1")
    monkeypatch.setenv("XCCL_TP_H2D_PHASES", "y" if phases else "n")
    tokens, hidden, ffn = (1024, 512, 1024) if tp <= 2 else (4096, 512, 1024)
    mlp = TpMlp(tokens, hidden, ffn, tp=tp, emulate=(tp > 1))
    try:
        assert mlp.overlap_h2d
        for it in range(3):
            x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(it)).to(torch.bfloat16)
            pinned = [c.contiguous().pin_memory() for c in x.chunk(tp, 0)]
            mlp.forward_from_host(pinned)
            mlp.check_error()
            want = reference_forward_fp32(x.to(dev), *_full_weights(mlp))
            torch.testing.assert_close(torch.cat(mlp.y, 0).float(), want, rtol=3e-2, atol=3e-2)
    finally:
        mlp.close()


def test_tp_mlp_full_output_read_back_is_pipelined_and_exact(dev):
    """forward_from_host_full: input from pinned memory (kernels launched first, rows follow), the whole output shard
    copied back on a copy stream while the next step runs; every step's host copy must hold that step's output."""
    from xccl_b200.models.tp_mlp import TpMlp, reference_forward_fp32
    tokens, hidden, ffn = 1024, 512, 1024
    mlp = TpMlp(tokens, hidden, ffn, tp=1)
    try:
        y_pinned = [[torch.empty(tokens, hidden, dtype=torch.bfloat16).pin_memory()] for _ in range(2)]
        xs = [torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(40 + it)).to(torch.bfloat16) for it in range(4)]
        pinned = [[x.pin_memory()] for x in xs]
        wants = [reference_forward_fp32(x.to(dev), *_full_weights(mlp)) for x in xs]
        for it in range(4):   # no host wait between the steps
            mlp.forward_from_host_full(pinned[it], y_pinned)
        mlp.wait_outputs()
        mlp.check_error()
        # the two host buffers hold the outputs of the last two steps (parity 0: step 2, parity 1: step 3)
        torch.testing.assert_close(y_pinned[0][0].float().to(dev), wants[2], rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(y_pinned[1][0].float().to(dev), wants[3], rtol=3e-2, atol=3e-2)
    finally:
        mlp.close()


# ----------------------------------------------------------------------------- fused MoE all-to-all
@pytest.mark.parametrize("ranks", [1, 2, 4])
def test_moe_dispatch_combine_matches_reference(dev, ranks):
    """Routing, grouping by (expert, source) and the weighted combine, ranks emulated in one launch."""
    from xccl_b200.ops.moe import MoeWorkspace
    T, H, E, Kk = 96, 256, 8 * ranks, 4
    EL = E // ranks
    ws = MoeWorkspace(T, H, E, Kk, emu_ranks=ranks)
    try:
        g = torch.Generator(device="cpu").manual_seed(ranks)
        xs = [torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev) for _ in range(ranks)]
        ids = [torch.stack([torch.randperm(E, generator=g)[:Kk] for _ in range(T)]).to(torch.int32).to(dev) for _ in range(ranks)]
        ws_ = [torch.softmax(torch.randn(T, Kk, generator=g), -1).to(dev) for _ in range(ranks)]
        for it in range(2):
            ws.dispatch(xs, ids)
            assert ws.error() == 0
            # every rank holds, per local expert, exactly the rows routed to it, grouped by source
            for r in range(ranks):
                rows = ws.expert_rows(r).cpu().tolist()
                recv, src = ws.recv(r), ws.row_source(r).cpu()
                row = 0
                for le in range(EL):
                    e = r * EL + le
                    want_n = sum(int((ids[s] == e).sum()) for s in range(ranks))
                    assert rows[le] == want_n
                    last_src = -1
                    for i in range(rows[le]):
                        s, t = divmod(int(src[row + i]), T)
                        assert s >= last_src          # sources appear in rank order inside an expert
                        last_src = s
                        assert bool((ids[s][t] == e).any())
                        assert torch.equal(recv[row + i], xs[s][t])
                    row += rows[le]
                assert rows[EL] == row
                # "experts": scale each row by (1 + global expert id)
                scale = torch.cat([torch.full((rows[le],), 1.0 + r * EL + le) for le in range(EL)]).to(dev)
                ws.expert_out(r)[:row] = (recv[:row].float() * scale[:, None]).to(torch.bfloat16)
            outs = [torch.zeros(T, H, dtype=torch.bfloat16, device=dev) for _ in range(ranks)]
            ws.combine(ids, ws_, outs)
            assert ws.error() == 0
            for r in range(ranks):
                y = (xs[r].float()[:, None, :] * (1.0 + ids[r].float())[:, :, None]).to(torch.bfloat16).float()
                want = (y * ws_[r][:, :, None]).sum(1)
                torch.testing.assert_close(outs[r].float(), want, rtol=2e-2, atol=2e-2)
    finally:
        ws.close()


# ----------------------------------------------------------------------------- block-scaled fp8 GEMM
@pytest.mark.parametrize("M,N,K_", [(128, 128, 128), (256, 384, 512), (1000, 256, 1024), (2048, 1024, 2048)])
def test_gemm_fp8_blockscaled_matches_dequantised_reference(dev, M, N, K_):
    from xccl_b200.ops import gemm
    a = torch.randn(M, K_, device=dev) * torch.rand(M, 1, device=dev) * 3
    b = torch.randn(N, K_, device=dev) * 0.05
    a8, sa = gemm.quantize_act_1x128(a)
    b8, sb = gemm.quantize_weight_128x128(b)
    out = gemm.gemm_fp8_blockscaled(a8, sa, b8, sb)
    assert gemm.last_error() == 0
    want = gemm.dequantize(a8, sa, 1) @ gemm.dequantize(b8, sb, 128).t()
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))


def test_quantize_rows_kernel_matches_torch(dev):
    from xccl_b200.ops import gemm
    from xccl_b200.ops.tp import quantize_rows
    x = (torch.randn(300, 512, device=dev) * torch.rand(300, 1, device=dev) * 5).to(torch.bfloat16)
    x[7, 128:256] = 0  # an all-zero block keeps a finite scale
    out8 = torch.empty(300, 512, dtype=torch.float8_e4m3fn, device=dev)
    s = torch.empty(300, 4, dtype=torch.float32, device=dev)
    quantize_rows(x, out8, s)
    torch.cuda.synchronize()
    q_ref, s_ref = gemm.quantize_act_1x128(x.float())
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    # x / s and x * (1 / s) may round differently by one e4m3 step: compare the dequantised values
    got, want = gemm.dequantize(out8, s, 1), gemm.dequantize(q_ref, s_ref, 1)
    assert float((got - want).abs().max()) <= float(s.max()) * 32 + 1e-6   # one step at the top binade of e4m3
    torch.testing.assert_close(got, x.float(), rtol=0.07, atol=1e-3)
    _loaded_native()


@pytest.mark.parametrize("tp,fuse_quant", [(1, True), (2, True), (4, True), (2, False)])
def test_tp_mlp_fp8_fused_matches_dequantised_reference(dev, tp, fuse_quant):
    """fp8 allgather->GEMM+SwiGLU and GEMM->reduce-scatter (ranks emulated in one launch) against fp32
    products of exactly the quantised operands the kernels consumed."""
    from xccl_b200.models.tp_mlp import TpMlpFp8
    from xccl_b200.ops import gemm
    tokens, hidden, ffn = 1024, 512, 1024
    mlp = TpMlpFp8(tokens, hidden, ffn, tp=tp, emulate=True, fuse_quant=fuse_quant)
    try:
        g = torch.Generator(device=dev).manual_seed(6)
        x = torch.randn(tokens, hidden, device=dev, generator=g).to(torch.bfloat16)
        shards = list(x.chunk(tp, 0))
        for it in range(3):
            y = mlp.forward(shards)
            mlp.check_error()
            xq = gemm.dequantize(torch.cat(mlp.x8, 0), torch.cat(mlp.sx, 0), 1)
            y_want = torch.zeros(tokens, hidden, device=dev)
            for r in range(tp):
                wg = gemm.dequantize(mlp.w_gate8[r], mlp.s_gate[r], 128)
                wu = gemm.dequantize(mlp.w_up8[r], mlp.s_up[r], 128)
                wd = gemm.dequantize(mlp.w_down8[r], mlp.s_down[r], 128)
                h_want = torch.nn.functional.silu(xq @ wg.t()) * (xq @ wu.t())
                if fuse_quant:
                    # the intermediate exists only as e4m3 with 1 x 128 scales: one e4m3 step (2^-3 relative) of the
                    # block maximum at most, and scales that are the block maxima over 448
                    h_got = gemm.dequantize(mlp.h8[r], mlp.sh[r], 1)
                    blk = h_want.view(tokens, -1, 128).abs().amax(-1)
                    torch.testing.assert_close(mlp.sh[r] * 448.0, blk.clamp_min(1e-12 * 448), rtol=3e-2, atol=1e-6)
                    assert float(((h_got - h_want).abs().view(tokens, -1, 128).amax(-1) / blk.clamp_min(1e-6)).max()) <= 0.07
                else:
                    torch.testing.assert_close(mlp.h[r].float(), h_want, rtol=2e-2, atol=2e-2 * float(h_want.abs().max()))
                y_want += gemm.dequantize(mlp.h8[r], mlp.sh[r], 1) @ wd.t()
            got = torch.cat(y, 0).float()
            torch.testing.assert_close(got, y_want, rtol=2e-2, atol=2e-2 * float(y_want.abs().max()))
            # and the whole block stays close to the unquantised fp32 block
            from xccl_b200.models.tp_mlp import reference_forward_fp32
            full = reference_forward_fp32(x, *_full_weights(mlp))
            assert float((got - full).abs().max()) <= 0.08 * float(full.abs().max()) + 1e-3
    finally:
        mlp.close()
    _loaded_native()
