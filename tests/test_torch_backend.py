"""c10d backend "b200xccl" on CPU ranks (store-based OOB + host team), and its DDP hook."""
import os

import pytest
import torch

from xccl_b200.utils.launch import run_ranks


def _more_ops(dist, rank, size, dev):
    """gather, scatter, list-form all_to_all and reduce_scatter, coalesced all_gather, AVG."""
    f = lambda v, n=3: torch.full((n,), float(v), device=dev)
    for root in (0, size - 1):
        outs = [torch.zeros(3, device=dev) for _ in range(size)] if rank == root else None
        dist.gather(f(rank + 1), outs, dst=root)
        if rank == root:
            assert all(torch.all(outs[r] == r + 1) for r in range(size))
        got = torch.zeros(3, device=dev)
        dist.scatter(got, [f(10 * r + root) for r in range(size)] if rank == root else None, src=root)
        assert torch.all(got == 10 * rank + root)
    ins = [f(100 * rank + r, r + 1) for r in range(size)]              # rank sends r+1 elements to rank r
    outs = [torch.zeros(rank + 1, device=dev) for _ in range(size)]
    dist.all_to_all(outs, ins)
    assert all(torch.all(outs[r] == 100 * r + rank) for r in range(size))
    out = torch.zeros(4, device=dev)
    dist.reduce_scatter(out, [f(r + rank, 4) for r in range(size)])
    assert torch.all(out == size * rank + sum(range(size)))
    t = f(rank + 1.0, 5)
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    torch.testing.assert_close(t, f((size + 1) / 2.0, 5))
    o1, o2 = torch.zeros(size * 2, device=dev), torch.zeros(size * 3, device=dev)
    pg = dist.distributed_c10d._get_default_group()
    w = pg.allgather_into_tensor_coalesced([o1, o2], [f(rank, 2), f(-rank, 3)])
    w.wait()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    assert torch.equal(o1.cpu(), torch.arange(size, dtype=torch.float32).repeat_interleave(2))
    assert torch.equal(o2.cpu(), -torch.arange(size, dtype=torch.float32).repeat_interleave(3))


def _pg_rank(rank, size, job, port):
    import torch.distributed as dist

    import xccl_b200.parallel.torch_backend as tb
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "XCCL_TORCH_TLS": "ucx"})
    tb.register()
    dist.init_process_group(tb.BACKEND, rank=rank, world_size=size)
    assert tb.coll_tl(2, False) == "ucx"
    t = torch.full((1000,), float(rank + 1))
    dist.all_reduce(t)
    assert torch.all(t == sum(range(1, size + 1)))
    t = torch.full((7,), float(rank + 1))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert torch.all(t == size)
    b = torch.arange(10, dtype=torch.int64) * (1 if rank == 1 else 0)
    dist.broadcast(b, src=1)
    assert torch.equal(b, torch.arange(10, dtype=torch.int64))
    out = torch.zeros(size * 3)
    dist.all_gather_into_tensor(out, torch.full((3,), float(rank)))
    assert torch.equal(out, torch.arange(size, dtype=torch.float32).repeat_interleave(3))
    lst = [torch.zeros(2) for _ in range(size)]
    dist.all_gather(lst, torch.full((2,), float(rank)))
    assert all(torch.all(lst[r] == r) for r in range(size))
    rs = torch.zeros(4)
    dist.reduce_scatter_tensor(rs, torch.arange(4 * size, dtype=torch.float32))
    assert torch.equal(rs, torch.arange(4 * rank, 4 * rank + 4, dtype=torch.float32) * size)
    a2a = torch.zeros(size * 2)
    dist.all_to_all_single(a2a, torch.arange(size * 2, dtype=torch.float32) + 100 * rank)
    want = torch.cat([torch.arange(2 * rank, 2 * rank + 2, dtype=torch.float32) + 100 * r for r in range(size)])
    assert torch.equal(a2a, want)
    _more_ops(dist, rank, size, torch.device("cpu"))
    # fused scale + cast
    src = torch.full((50,), float(rank + 1))
    dst = torch.zeros(50, dtype=torch.bfloat16)
    tb.allreduce_fused(src, dst, 1.0 / size).wait()
    assert torch.allclose(dst.float(), torch.full((50,), (size + 1) / 2.0), atol=1e-2)
    dist.barrier()
    # DDP with the fused hook: gradients equal the average over ranks
    from torch.nn.parallel import DistributedDataParallel as DDP
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    ddp = DDP(model, bucket_cap_mb=1)
    ddp.register_comm_hook(None, tb.fused_allreduce_hook)
    torch.manual_seed(100 + rank)
    x = torch.randn(8, 16)
    ddp(x).sum().backward()
    g = [p.grad.clone() for p in model.parameters()]
    ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    ref.load_state_dict(model.state_dict())
    acc = [torch.zeros_like(p) for p in ref.parameters()]
    for r in range(size):
        ref.zero_grad()
        torch.manual_seed(100 + r)
        ref(torch.randn(8, 16)).sum().backward()
        for a, p in zip(acc, ref.parameters()):
            a += p.grad / size
    for got, want in zip(g, acc):
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    dist.destroy_process_group()
    return True


def test_c10d_backend_on_cpu_ranks():
    port = 29600 + (os.getpid() % 300)
    run_ranks(_pg_rank, 3, port, timeout=240, start_method="spawn")


def _pg_cuda_rank(rank, size, job, port, tls):
    """The backend on CUDA tensors, one GPU per rank: stream-ordered collectives (reference tests
    test/test_mpi_cuda_allreduce.c, test_mpi_cuda_alltoall.c drive device buffers the same way)."""
    import torch.distributed as dist

    import xccl_b200.parallel.torch_backend as tb
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "XCCL_TORCH_TLS": tls})
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    tb.register()
    dist.init_process_group(tb.BACKEND, rank=rank, world_size=size)
    try:
        assert tb.coll_tl(2, True) == tls.split(",")[0]
        for n in (1, 1000, 1 << 20):
            t = torch.full((n,), float(rank + 1), device=dev)
            dist.all_reduce(t)
            assert torch.all(t == sum(range(1, size + 1)))
        t = torch.full((4099,), float(rank + 1), device=dev, dtype=torch.bfloat16)
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        torch.testing.assert_close(t.float(), torch.full((4099,), (size + 1) / 2.0, device=dev))
        b = torch.arange(1000, device=dev, dtype=torch.int64) * (1 if rank == 1 else 0)
        dist.broadcast(b, src=1)
        assert torch.equal(b, torch.arange(1000, device=dev, dtype=torch.int64))
        rs = torch.zeros(4, device=dev)
        dist.reduce_scatter_tensor(rs, torch.arange(4 * size, dtype=torch.float32, device=dev))
        assert torch.equal(rs.cpu(), torch.arange(4 * rank, 4 * rank + 4, dtype=torch.float32) * size)
        a2a = torch.zeros(size * 2, device=dev)
        dist.all_to_all_single(a2a, torch.arange(size * 2, dtype=torch.float32, device=dev) + 100 * rank)
        want = torch.cat([torch.arange(2 * rank, 2 * rank + 2, dtype=torch.float32) + 100 * r for r in range(size)])
        assert torch.equal(a2a.cpu(), want)
        out = torch.zeros(size * 3, device=dev)
        dist.all_gather_into_tensor(out, torch.full((3,), float(rank), device=dev))
        assert torch.equal(out.cpu(), torch.arange(size, dtype=torch.float32).repeat_interleave(3))
        _more_ops(dist, rank, size, dev)
        # fused scale + cast of a gradient-sized buffer, output narrower than the input
        src = torch.randn(1 << 20, device=dev, generator=torch.Generator(device=dev).manual_seed(rank))
        dst = torch.zeros(1 << 20, dtype=torch.bfloat16, device=dev)
        tb.allreduce_fused(src, dst, 1.0 / size).wait()
        allv = [torch.randn(1 << 20, device=dev, generator=torch.Generator(device=dev).manual_seed(r)) for r in range(size)]
        torch.testing.assert_close(dst.float(), torch.stack(allv).sum(0) / size, rtol=1e-2, atol=2e-2)
        if tls.startswith("nvlink"):
            # tensors in symmetric memory: the same calls, served zero-copy when the fabric has multicast
            try:
                sym = tb.empty_symmetric((1 << 20,), torch.float32)
            except RuntimeError:
                sym = None
            if sym is not None:
                sym.copy_(torch.full((1 << 20,), float(rank + 1), device=dev))
                dist.all_reduce(sym)
                assert torch.all(sym == sum(range(1, size + 1)))
                torch.cuda.synchronize()
                dist.barrier()
                tb.free_symmetric(sym)
        # DDP with the fused hook: gradients equal the average over ranks
        from torch.nn.parallel import DistributedDataParallel as DDP
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 8)).to(dev)
        ddp = DDP(model, device_ids=[rank], bucket_cap_mb=1)
        ddp.register_comm_hook(None, tb.fused_allreduce_hook)
        acc = None
        xs = [torch.randn(16, 64, generator=torch.Generator().manual_seed(100 + r)) for r in range(size)]
        ddp(xs[rank].to(dev)).sum().backward()
        got = [p.grad.clone() for p in model.parameters()]
        ref = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 8)).to(dev)
        ref.load_state_dict(model.state_dict())
        acc = [torch.zeros_like(p) for p in ref.parameters()]
        for r in range(size):
            ref.zero_grad()
            ref(xs[r].to(dev)).sum().backward()
            for a, p in zip(acc, ref.parameters()):
                a += p.grad / size
        for g, w in zip(got, acc):
            torch.testing.assert_close(g, w, rtol=1e-4, atol=1e-5)
        dist.barrier()
        torch.cuda.synchronize()
        return "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("tls", ["nvlink,nccl,ucx", "nccl,ucx"])
def test_c10d_backend_on_cuda_tensors(tls):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29300 + (os.getpid() % 300) + (0 if tls.startswith("nvlink") else 1)
    res = run_ranks(_pg_cuda_rank, 2, port, tls, timeout=240, start_method="spawn", env={"NCCL_NVLS_ENABLE": "0"})
    assert res == ["ok", "ok"]
