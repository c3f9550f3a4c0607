"""NVLink team with one process per GPU (needs at least 2 GPUs; skipped otherwise).

Every rank checks its results against values it can compute alone from the seeds, so a wrong
answer fails on the rank that sees it. NVLS is exercised when the team reports it.
"""
import os

import pytest
import torch

from xccl_b200 import _capi as K
from xccl_b200.utils.launch import run_ranks

pytestmark = pytest.mark.gpu


def _ngpus():
    try:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def _vals(rank, count, dtype, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed * 100 + rank)
    return torch.randint(-8, 9, (count,), generator=g).to(dtype)


def _rank_main(rank, size, job, tls, nvls):
    from xccl_b200.api import Context, Lib, ShmOob, Team
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    lib = Lib()
    cfg = {K.TL_NVLINK: {"WORKSPACE_SIZE": "32m", "NVLS": "try" if nvls else "no", "TIMING": "y"}}
    ctx = Context(lib, oob, tls=tls, config=cfg)
    team = Team(ctx)
    want_tl = K.TL_NVLINK if (tls & K.TL_NVLINK) else K.TL_NCCL
    assert team.coll_tl(K.ALLREDUCE, K.MEM_CUDA) == want_tl, team.coll_tl(K.ALLREDUCE, K.MEM_CUDA)
    stream = torch.cuda.current_stream().cuda_stream
    out = {}

    algs = [None]
    if tls & K.TL_NVLINK:
        algs = [K.NVLINK_ALG_ONE_SHOT, K.NVLINK_ALG_TWO_SHOT] + ([K.NVLINK_ALG_NVLS] if nvls else [])
    for dtype in (torch.float32, torch.bfloat16):
        for count in (1, 1000, 65536, 1 << 20, (3 << 20) + 5):
            for alg in algs:
                if alg == K.NVLINK_ALG_ONE_SHOT and count * 4 * size > (16 << 20):
                    continue
                src = _vals(rank, count, dtype).to(dev)
                dst = torch.zeros_like(src)
                req = team.allreduce(src, dst, alg=alg, stream=stream)
                try:
                    req.post().wait()
                except Exception as e:  # NVLS may be unavailable on this box: fall back loudly
                    if alg == K.NVLINK_ALG_NVLS:
                        out["nvls"] = f"unavailable: {e}"
                        req.finalize()
                        continue
                    raise
                want = torch.stack([_vals(r, count, dtype).double() for r in range(size)]).sum(0).to(dtype)
                assert torch.equal(dst.cpu(), want), (dtype, count, alg)
                if alg == K.NVLINK_ALG_NVLS:
                    out["nvls"] = "ok"
                req.finalize()
    # fused scale + cast (gradient averaging), persistent request posted 3 times
    src = torch.randn(100000, device=dev, generator=torch.Generator(device=dev).manual_seed(rank))
    dst = torch.empty(100000, device=dev, dtype=torch.bfloat16)
    # (the NCCL team applies it with one kernel on the same stream after the library call; a guard band
    # behind dst shows that nothing wider than the output type was written there)
    guard = torch.full((100000 + 64,), 7.0, device=dev, dtype=torch.bfloat16)
    dst = guard[:100000]
    req = team.allreduce(src, dst, scale=1.0 / size, out_dt=K.DT_BFLOAT16, stream=stream)
    for _ in range(3):
        req.post().wait()
    allv = [torch.randn(100000, device=dev, generator=torch.Generator(device=dev).manual_seed(r)) for r in range(size)]
    want = (torch.stack(allv).double().sum(0) / size).float()
    torch.testing.assert_close(dst.float(), want, rtol=1e-2, atol=2e-2)
    assert torch.all(guard[100000:] == 7.0)
    out["elapsed_us"] = req.elapsed_us
    req.finalize()
    buf = src.clone()
    team.allreduce("in_place", buf, scale=1.0 / size, stream=stream).run().finalize()
    torch.testing.assert_close(buf, want, rtol=1e-5, atol=1e-5)
    # the other collectives
    per = 4099
    src = _vals(rank, per, torch.int32, seed=3).to(dev)
    dst = torch.zeros(per * size, dtype=torch.int32, device=dev)
    team.allgather(src, dst, stream=stream).run().finalize()
    assert torch.equal(dst.cpu(), torch.cat([_vals(r, per, torch.int32, seed=3) for r in range(size)]))
    src = (torch.arange(per * size, dtype=torch.float32) + rank * 1e5).to(dev)
    dst = torch.zeros_like(src)
    team.alltoall(src, dst, stream=stream).run().finalize()
    want = torch.cat([(torch.arange(per * size, dtype=torch.float32) + r * 1e5)[rank * per:(rank + 1) * per]
                      for r in range(size)])
    assert torch.equal(dst.cpu(), want)
    for root in range(size):
        buf = _vals(root, 70001, torch.float32, seed=9).to(dev) if rank == root else torch.zeros(70001, device=dev)
        team.bcast(buf, root, stream=stream).run().finalize()
        assert torch.equal(buf.cpu(), _vals(root, 70001, torch.float32, seed=9))
    if tls & K.TL_NVLINK:
        src = _vals(rank, 5000, torch.float32, seed=4).to(dev)
        dst = torch.zeros_like(src)
        team.reduce(src, dst, root=size - 1, stream=stream).run().finalize()
        if rank == size - 1:
            assert torch.equal(dst.cpu(), torch.stack([_vals(r, 5000, torch.float32, seed=4) for r in range(size)]).sum(0))
        src = _vals(rank, 1237 * size, torch.float32, seed=5).to(dev)
        dst = torch.zeros(1237, device=dev)
        team.reduce_scatter(src, dst, stream=stream).run().finalize()
        full = torch.stack([_vals(r, 1237 * size, torch.float32, seed=5) for r in range(size)]).sum(0)
        assert torch.equal(dst.cpu(), full[rank * 1237:(rank + 1) * 1237])
        # variable counts
        sc = [rank + d + 1 for d in range(size)]
        sd = [sum(sc[:d]) for d in range(size)]
        rc = [s + rank + 1 for s in range(size)]
        rd = [sum(rc[:s]) for s in range(size)]
        src = torch.cat([torch.full((sc[d],), float(rank * 100 + d)) for d in range(size)]).to(dev)
        dst = torch.zeros(sum(rc), device=dev)
        team.alltoallv(src, sc, sd, dst, rc, rd, stream=stream).run().finalize()
        assert torch.equal(dst.cpu(), torch.cat([torch.full((rc[s],), float(s * 100 + rank)) for s in range(size)]))
        # direct (zero-copy) kernels on buffers registered with the peers through CUDA IPC at init;
        # persistent requests posted several times, sub-allocations of torch's caching allocator
        D = K.NVLINK_ALG_DIRECT
        for dtype, count in ((torch.float32, 4 * 100003), (torch.bfloat16, 8 * 300007)):
            src = _vals(rank, count, dtype, seed=21).to(dev)
            dst = torch.zeros_like(src)
            req = team.allreduce(src, dst, alg=D, stream=stream)
            want = torch.stack([_vals(r, count, dtype, seed=21).double() for r in range(size)]).sum(0).to(dtype)
            for _ in range(3):
                dst.zero_()
                req.post().wait()
                assert torch.equal(dst.cpu(), want), ("direct allreduce", dtype)
            req.finalize()
        src = torch.randn(4 * 50000, device=dev, generator=torch.Generator(device=dev).manual_seed(rank + 40))
        out16 = torch.empty(4 * 50000, device=dev, dtype=torch.bfloat16)
        req = team.allreduce(src, out16, alg=D, scale=1.0 / size, out_dt=K.DT_BFLOAT16, stream=stream)
        req.post().wait()
        req.finalize()
        allv = [torch.randn(4 * 50000, device=dev, generator=torch.Generator(device=dev).manual_seed(r + 40)) for r in range(size)]
        torch.testing.assert_close(out16.float(), (torch.stack(allv).double().sum(0) / size).float(), rtol=1e-2, atol=2e-2)
        per = 16 * 4099
        src = _vals(rank, per, torch.int32, seed=23).to(dev)
        dst = torch.zeros(per * size, dtype=torch.int32, device=dev)
        team.allgather(src, dst, stream=stream, alg=D).run().finalize()
        assert torch.equal(dst.cpu(), torch.cat([_vals(r, per, torch.int32, seed=23) for r in range(size)]))
        src = (torch.arange(per * size, dtype=torch.float32) + rank * 1e6).to(dev)
        dst = torch.zeros_like(src)
        req = team.alltoall(src, dst, alg=D, stream=stream)
        for _ in range(2):
            req.post().wait()
        req.finalize()
        want = torch.cat([(torch.arange(per * size, dtype=torch.float32) + r * 1e6)[rank * per:(rank + 1) * per]
                          for r in range(size)])
        assert torch.equal(dst.cpu(), want)
        src = _vals(rank, 4 * 1237 * size, torch.float32, seed=25).to(dev)
        dst = torch.zeros(4 * 1237, device=dev)
        team.reduce_scatter(src, dst, stream=stream, alg=D).run().finalize()
        full = torch.stack([_vals(r, 4 * 1237 * size, torch.float32, seed=25) for r in range(size)]).sum(0)
        assert torch.equal(dst.cpu(), full[rank * 4 * 1237:(rank + 1) * 4 * 1237])
        out["direct"] = "ok"
        # stream-ordered barrier served by the nvlink team
        assert team.coll_tl(K.BARRIER, K.MEM_HOST) == K.TL_NVLINK
        for _ in range(3):
            team.barrier().run().finalize()
    if tls & K.TL_NVLINK:
        # posts that alternate between two streams without a host wait in between: the team orders them, so every
        # rank runs the same sequence of kernels on the shared workspace and pads
        s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
        torch.cuda.synchronize()
        xs = [_vals(rank, 50000 + i, torch.float32, seed=40 + i).to(dev) for i in range(6)]
        ys = [torch.zeros_like(x) for x in xs]
        reqs = [team.allreduce(xs[i], ys[i], stream=(s1 if i % 2 == 0 else s2).cuda_stream,
                               alg=(K.NVLINK_ALG_ONE_SHOT if i % 3 == 0 else K.NVLINK_ALG_TWO_SHOT)) for i in range(6)]
        for _ in range(3):
            for r_ in reqs:
                r_.post()
        for r_ in reqs:
            r_.wait()
        for i in range(6):
            want = torch.stack([_vals(r, 50000 + i, torch.float32, seed=40 + i) for r in range(size)]).sum(0)
            assert torch.equal(ys[i].cpu(), want), ("two streams", i)
            reqs[i].finalize()
        out["two_streams"] = "ok"
        # alltoallv several times larger than the workspace (32 MiB: halves of 16 MiB), uneven counts
        cnt = [(3 << 20) + 1001 * ((rank + 2 * d) % size) for d in range(size)]   # fp32 elements to each peer
        rcnt = [(3 << 20) + 1001 * ((s_ + 2 * rank) % size) for s_ in range(size)]
        src = torch.cat([torch.full((cnt[d],), float(100 * rank + d), device=dev) for d in range(size)])
        dst = torch.zeros(sum(rcnt), device=dev)
        sd = [sum(cnt[:d]) for d in range(size)]
        rd = [sum(rcnt[:s_]) for s_ in range(size)]
        team.alltoallv(src, cnt, sd, dst, rcnt, rd, stream=stream).run().finalize()
        for s_ in range(size):
            assert torch.all(dst[rd[s_]:rd[s_] + rcnt[s_]] == float(100 * s_ + rank)), ("alltoallv", s_)
        out["big_alltoallv"] = "ok"
    if (tls & K.TL_NVLINK) and out.get("nvls") == "ok":
        # reduce to a root and reduce-scatter with the in-switch reduction (multimem.ld_reduce by the reducing rank);
        # counts that are no multiple of a pack and that span several workspace chunks
        for dtype in (torch.float32, torch.bfloat16):
            for count in (5, 70001, (5 << 20) + 3):
                src = _vals(rank, count, dtype, seed=60).to(dev)
                dst = torch.zeros(count, dtype=dtype, device=dev)
                root = count % size
                team.reduce(src, dst, root=root, stream=stream, alg=K.NVLINK_ALG_NVLS, scale=0.5).run().finalize()
                if rank == root:
                    want = (torch.stack([_vals(r, count, dtype, seed=60).double() for r in range(size)]).sum(0) * 0.5).to(dtype)
                    assert torch.equal(dst.cpu(), want), ("nvls reduce", dtype, count)
            per = 40003
            src = _vals(rank, per * size, dtype, seed=61).to(dev)
            dst = torch.zeros(per, dtype=dtype, device=dev)
            team.reduce_scatter(src, dst, stream=stream, alg=K.NVLINK_ALG_NVLS).run().finalize()
            full = torch.stack([_vals(r, per * size, dtype, seed=61).double() for r in range(size)]).sum(0).to(dtype)
            assert torch.equal(dst.cpu(), full[rank * per:(rank + 1) * per]), ("nvls reduce_scatter", dtype)
        out["nvls_reduce"] = "ok"
        # symmetric memory: in-switch reduction and multicast straight on the caller's buffers
        nbytes = 8 << 20
        mem = team.mem_alloc(2 * nbytes)
        for dtype in (torch.float32, torch.bfloat16):
            es = torch.tensor([], dtype=dtype).element_size()
            for count in (4096, 65536 + 8, (1 << 20) + 16):
                src = mem[:count * es].view(dtype)
                dst = mem[nbytes:nbytes + count * es].view(dtype)
                src.copy_(_vals(rank, count, dtype, seed=50).to(dev))
                dst.zero_()
                req = team.allreduce(src, dst, stream=stream, alg=K.NVLINK_ALG_SYMMETRIC, scale=0.5)
                for _ in range(3):
                    req.post()
                req.wait()
                want = (torch.stack([_vals(r, count, dtype, seed=50).double() for r in range(size)]).sum(0) * 0.5).to(dtype)
                assert torch.equal(dst.cpu(), want), ("symmetric", dtype, count)
                req.finalize()
                # in place, chosen without being asked for (size above the one-shot range)
                if count * es > (1 << 20):
                    team.allreduce("in_place", src, stream=stream).run().finalize()
                    assert torch.equal(src.cpu(), (want.double() * 2).to(dtype)), ("symmetric in place", dtype, count)
        buf = mem[:1 << 20]
        if rank == 1:
            buf.copy_(torch.arange(1 << 20, device=dev, dtype=torch.int64).to(torch.uint8))
        else:
            buf.zero_()
        torch.cuda.synchronize()
        team.bcast(buf, 1, stream=stream).run().finalize()
        assert torch.equal(buf.cpu(), torch.arange(1 << 20, dtype=torch.int64).to(torch.uint8))
        # a root whose source is ordinary memory, destinations symmetric
        team.barrier().run().finalize()
        team.mem_free(mem)
        out["symmetric"] = "ok"
    torch.cuda.synchronize()
    team.close()
    ctx.close()
    lib.close()
    oob.close()
    return out


@pytest.mark.parametrize("size", [2, 4, 8])
def test_nvlink_team_collectives(size):
    if _ngpus() < size:
        pytest.skip(f"needs {size} GPUs")
    res = run_ranks(_rank_main, size, K.TL_NVLINK | K.TL_UCX, True, timeout=300, start_method="spawn",
                    env={"NCCL_NVLS_ENABLE": "0"})
    print("nvlink team:", res[0])


def test_nccl_team_collectives():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_rank_main, 2, K.TL_NCCL | K.TL_UCX, False, timeout=300, start_method="spawn")


def _tp_rank_main(rank, size, job):
    """Fused allgather->GEMM+SwiGLU and GEMM->reduce-scatter across real GPUs against the fp32 oracle."""
    from xccl_b200.api import ShmOob
    from xccl_b200.models.tp_mlp import TpMlp, _init_weights, reference_forward_fp32
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    tokens, hidden, ffn = 2048, 1024, 2048
    mlp = TpMlp(tokens, hidden, ffn, tp=size, rank=rank, oob=oob)
    try:
        g = torch.Generator(device="cpu").manual_seed(11)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
        shard = x.chunk(size, 0)[rank].contiguous()
        ws = [_init_weights(tokens, hidden, ffn, size, r, dev) for r in range(size)]
        w_gate = torch.cat([w[0] for w in ws], 0)
        w_up = torch.cat([w[1] for w in ws], 0)
        w_down = torch.cat([w[2] for w in ws], 1)
        want = reference_forward_fp32(x, w_gate, w_up, w_down).chunk(size, 0)[rank]
        errs = []
        for _ in range(4):   # sequence numbers, buffer parities and arrival counters advance
            y = mlp.forward([shard])[0]
            torch.cuda.synchronize()
            mlp.check_error()
            errs.append(float((y.float() - want).abs().max()))
            torch.testing.assert_close(y.float(), want, rtol=3e-2, atol=3e-2)
        # the same block with the input arriving from pinned host memory while the kernel already runs (every rank
        # reports its rows as they land; remote tiles start after the first chunks), a new input every step
        for it in range(3):
            x2 = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(100 + it)).to(torch.bfloat16)
            mine = x2.chunk(size, 0)[rank].contiguous().pin_memory()
            metric = mlp.forward_from_host([mine])
            mlp.check_error()
            want2 = reference_forward_fp32(x2.to(dev), w_gate, w_up, w_down).chunk(size, 0)[rank]
            torch.testing.assert_close(mlp.y[0].float(), want2, rtol=3e-2, atol=3e-2)
            assert torch.isfinite(metric)
        return max(errs)
    finally:
        mlp.close()
        oob.close()


@pytest.mark.parametrize("size", [2, 4, 8])
def test_tp_mlp_fused_across_gpus(size):
    if _ngpus() < size:
        pytest.skip(f"needs {size} GPUs")
    res = run_ranks(_tp_rank_main, size, timeout=300, start_method="spawn")
    print("tp mlp max abs err per rank:", res)


def _registration_release_main(rank, size, job):
    """DIRECT_CACHE=n: the peers' mappings of registered buffers live as long as the requests that use them."""
    import ctypes as C
    from xccl_b200.api import Context, Lib, ShmOob, Team
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_NVLINK | K.TL_UCX, config={K.TL_NVLINK: {"DIRECT_CACHE": "n", "WORKSPACE_SIZE": "32m"}})
    team = Team(ctx)
    count_fn = K.load().xccl_nvlink_peer_mappings
    count_fn.restype, count_fn.argtypes = C.c_int, [C.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    assert count_fn(team.h) == 0
    for it in range(3):   # fresh buffers every round: each is registered, used, released; its memory may then be freed
        n = (1 << 20) + 16 * it
        src = _vals(rank, n, torch.float32, seed=70 + it).to(dev)
        dst = torch.zeros_like(src)
        r1 = team.allreduce(src, dst, stream=stream, alg=K.NVLINK_ALG_DIRECT)
        r2 = team.allreduce(src, dst, stream=stream, alg=K.NVLINK_ALG_DIRECT)   # the same allocations: counted twice
        held = count_fn(team.h)
        assert 1 <= held <= 2 * (size - 1), held
        r1.run()
        want = torch.stack([_vals(r, n, torch.float32, seed=70 + it) for r in range(size)]).sum(0)
        assert torch.equal(dst.cpu(), want)
        r1.finalize()
        assert count_fn(team.h) == held          # r2 still holds them
        r2.run()
        assert torch.equal(dst.cpu(), want)
        r2.finalize()
        assert count_fn(team.h) == 0
        team.barrier().run().finalize()         # every peer has closed its mapping of my buffers
        del src, dst
    team.close(); ctx.close(); lib.close(); oob.close()
    return True


def test_registered_buffers_are_released_with_their_requests():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_registration_release_main, 2, timeout=300, start_method="spawn")


def _host_team_cuda_main(rank, size, job):
    """The host team serving CUDA buffers (the reference's CUDA tests run its UCX team on device memory,
    test/test_mpi_cuda_allreduce.c, test_mpi_cuda_reduce.c): staged through pinned memory, started in
    stream order."""
    from xccl_b200.api import Context, Lib, ShmOob, Team
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    lib = Lib()
    ctx = Context(lib, oob, tls=K.TL_UCX)
    team = Team(ctx)
    assert team.coll_tl(K.ALLREDUCE, K.MEM_CUDA) == K.TL_UCX
    stream = torch.cuda.current_stream().cuda_stream
    for dtype, count in ((torch.float32, 1), (torch.int32, 1000), (torch.float32, 70001)):
        src = _vals(rank, count, dtype, seed=31).to(dev)
        dst = torch.zeros_like(src)
        team.allreduce(src, dst, stream=stream).run().finalize()
        want = torch.stack([_vals(r, count, dtype, seed=31).double() for r in range(size)]).sum(0).to(dtype)
        assert torch.equal(dst.cpu(), want), (dtype, count)
    src = _vals(rank, 5000, torch.float32, seed=32).to(dev)
    dst = torch.zeros_like(src)
    team.reduce(src, dst, root=0, stream=stream).run().finalize()
    if rank == 0:
        assert torch.equal(dst.cpu(), torch.stack([_vals(r, 5000, torch.float32, seed=32) for r in range(size)]).sum(0))
    buf = _vals(1, 4099, torch.float32, seed=33).to(dev) if rank == 1 else torch.zeros(4099, device=dev)
    team.bcast(buf, 1, stream=stream).run().finalize()
    assert torch.equal(buf.cpu(), _vals(1, 4099, torch.float32, seed=33))
    team.close(); ctx.close(); lib.close(); oob.close()
    return "ok"


def test_host_team_serves_cuda_buffers():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_ranks(_host_team_cuda_main, 2, timeout=180, start_method="spawn")
    assert res == ["ok", "ok"]


def _fabric_rank_main(rank, size, job):
    """The in-fabric offload team libraries (ids of the reference's sharp and hmc teams) on NVSwitch: allreduce and
    barrier through the sharp team - bounce path on ordinary tensors, zero-copy on registered memory from
    ZCOPY_THRESH on - and bcast through the hmc team."""
    from xccl_b200.api import Context, Lib, ShmOob, Team, XcclError
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    lib = Lib()
    out = {}
    try:
        ctx = Context(lib, oob, tls=K.TL_SHARP | K.TL_HMC | K.TL_UCX,
                      config={K.TL_SHARP: {"ZCOPY_THRESH": "64k", "BCOPY_BUF_NUM": "4", "BCOPY_BUF_SIZE": "1m"}})
    except XcclError as e:
        return {"skipped": f"no multicast fabric: {e}"}
    team = Team(ctx)
    if team.coll_tl(K.ALLREDUCE, K.MEM_CUDA) != K.TL_SHARP:
        team.close(); ctx.close(); lib.close(); oob.close()
        return {"skipped": "the sharp team did not come up (no multicast)"}
    assert team.coll_tl(K.BCAST, K.MEM_CUDA) == K.TL_HMC
    stream = torch.cuda.current_stream().cuda_stream
    # bounce path: ordinary tensors, also larger than the 4 MiB of bounce buffers
    for count in (1000, 300000, (3 << 20) + 8):
        src = _vals(rank, count, torch.float32, seed=60).to(dev)
        dst = torch.zeros_like(src)
        team.allreduce(src, dst, stream=stream, scale=0.5).run().finalize()
        want = torch.stack([_vals(r, count, torch.float32, seed=60) for r in range(size)]).sum(0) * 0.5
        assert torch.equal(dst.cpu(), want), ("bounce", count)
    # registered memory: below the threshold staged, from it on in place
    mem = team.mem_alloc(16 << 20)
    for count in (4096, 1 << 20):
        src = mem[:count * 4].view(torch.float32)
        dst = mem[8 << 20:(8 << 20) + count * 4].view(torch.float32)
        src.copy_(_vals(rank, count, torch.float32, seed=61).to(dev))
        req = team.allreduce(src, dst, stream=stream)
        for _ in range(2):
            req.post()
        req.wait()
        req.finalize()
        want = torch.stack([_vals(r, count, torch.float32, seed=61) for r in range(size)]).sum(0)
        assert torch.equal(dst.cpu(), want), ("registered", count)
    team.barrier().run().finalize()
    buf = _vals(1, 70000, torch.float32, seed=62).to(dev) if rank == 1 else torch.zeros(70000, device=dev)
    team.bcast(buf, 1, stream=stream).run().finalize()
    assert torch.equal(buf.cpu(), _vals(1, 70000, torch.float32, seed=62))
    torch.cuda.synchronize()
    team.mem_free(mem)
    team.close(); ctx.close()
    # a fabric device that does not exist: the sharp team stays out, the context is served by the rest
    ctx2 = Context(lib, oob, tls=K.TL_SHARP | K.TL_UCX, config={K.TL_SHARP: {"NET_DEVICES": "mlx5_0:1"}})
    team2 = Team(ctx2)
    assert team2.coll_tl(K.ALLREDUCE, K.MEM_CUDA) != K.TL_SHARP
    team2.close(); ctx2.close()
    lib.close(); oob.close()
    out["ok"] = True
    return out


def test_fabric_offload_teams_on_nvswitch():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_ranks(_fabric_rank_main, 2, timeout=240, start_method="spawn", env={"NCCL_NVLS_ENABLE": "0"})
    print("sharp / hmc teams:", res[0])
    assert all(("ok" in r) or ("skipped" in r) for r in res)
