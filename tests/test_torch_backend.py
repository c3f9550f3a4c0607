"""c10d backend "b200xccl" on CPU ranks (store-based OOB + host team), and its DDP hook."""
import os

import pytest
import torch

from xccl_b200.utils.launch import run_ranks


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
