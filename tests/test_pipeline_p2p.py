"""Pipeline-parallel send/recv on NCCL p2p (needs 2 GPUs; skipped otherwise)."""
import pytest
import torch

from xccl_b200.utils.launch import run_ranks

pytestmark = pytest.mark.gpu


def _ngpus():
    try:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def _stage_main(rank, size, job):
    from xccl_b200.api import ShmOob
    from xccl_b200.parallel.pipeline import P2PComm, overlapped_stage_step
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    oob = ShmOob(job, rank, size)
    comm = P2PComm(oob)
    try:
        # plain exchange: neighbours swap a tensor inside one group
        mine = torch.full((1 << 16,), float(rank + 1), device=dev)
        theirs = torch.zeros_like(mine)
        peer = rank ^ 1
        with comm.group():
            comm.send(mine, peer)
            comm.recv(theirs, peer)
        torch.cuda.synchronize()
        assert torch.all(theirs == float(peer + 1))
        # a pipeline of `size` stages: stage s multiplies by (s + 2); inputs are i + 1
        n_mb, shape = 6, (256, 512)
        g = torch.Generator(device="cpu").manual_seed(0)
        base = [torch.randn(shape, generator=g).to(torch.bfloat16) for _ in range(n_mb)]
        outs = overlapped_stage_step(comm, lambda x: x * float(rank + 2), n_mb, shape,
                                     first_input=lambda i: base[i].to(dev))
        if rank == size - 1:
            assert len(outs) == n_mb
            for i, o in enumerate(outs):
                want = base[i].to(dev)
                for s in range(size):
                    want = want * float(s + 2)
                torch.testing.assert_close(o.float(), want.float(), rtol=2e-2, atol=1e-2)
        return "ok"
    finally:
        comm.close()
        oob.close()


def test_pipeline_send_recv_two_stages():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_ranks(_stage_main, 2, timeout=180, start_method="spawn", env={"NCCL_NVLS_ENABLE": "0"})
    assert res == ["ok", "ok"]


def _torch_p2p_main(rank, size, job, port):
    import os

    import torch.distributed as dist

    import xccl_b200.parallel.torch_backend as tb
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    tb.register()
    dist.init_process_group(tb.BACKEND, rank=rank, world_size=size)
    try:
        peer = 1 - rank
        for it in range(3):
            t = torch.full((1 << 14,), float(10 * rank + it), device=dev)
            if rank == 0:
                dist.send(t, dst=peer)
                dist.recv(t, src=peer)
                want = float(10 * peer + it)
            else:
                got = torch.empty_like(t)
                dist.recv(got, src=peer)
                dist.send(t, dst=peer)
                t, want = got, float(10 * peer + it)
            torch.cuda.synchronize()
            assert torch.all(t == want)
        return "ok"
    finally:
        dist.destroy_process_group()


def test_torch_backend_send_recv():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_ranks(_torch_p2p_main, 2, 29877, timeout=180, start_method="spawn", env={"NCCL_NVLS_ENABLE": "0"})
    assert res == ["ok", "ok"]
