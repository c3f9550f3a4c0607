"""Data-parallel ResNet-50 training step through a torch.distributed backend: the "b200xccl"
ProcessGroup of this repository (fused scale/cast gradient hook) against torch's "nccl" backend.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m xccl_b200.bench.ddp_resnet --backend b200xccl [--batch 256] [--steps 20] [--warmup 5]

Config of the headline run: 256 images per GPU, 3 x 224 x 224 in bf16 drawn from N(0,1), 1000
classes with uniform random labels, random-init torchvision ResNet-50 in bf16 (channels_last),
SGD with momentum, DistributedDataParallel with 25 MB gradient buckets overlapped with backward.
With ``--backend b200xccl`` the buckets go through ``fused_allreduce_hook`` (sum, 1/world scale
and cast in one NVLink kernel); with ``--backend nccl`` DDP's stock divide + allreduce runs.
The model and its convolution kernels are torch's in both arms: only the gradient collectives differ.
Device-timed with CUDA events, maximum over ranks; rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--backend", default="b200xccl", choices=["b200xccl", "nccl"])
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--no-hook", action="store_true", help="b200xccl backend with DDP's stock divide + allreduce")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    tb = None
    if a.backend == "b200xccl":
        import xccl_b200.parallel.torch_backend as tb
        tb.register()
        dist.init_process_group("b200xccl", rank=rank, world_size=world)
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    import torchvision
    torch.manual_seed(0)
    model = torchvision.models.resnet50(weights=None, num_classes=1000).to(dev).to(torch.bfloat16)
    model = model.to(memory_format=torch.channels_last)
    ddp = DDP(model, device_ids=[local], bucket_cap_mb=a.bucket_mb, gradient_as_bucket_view=True,
              broadcast_buffers=False)
    if tb is not None and not a.no_hook:
        ddp.register_comm_hook(None, tb.fused_allreduce_hook)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.01, momentum=0.9)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = torch.randn(a.batch, 3, 224, 224, device=dev, generator=g).to(torch.bfloat16).contiguous(
        memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (a.batch,), device=dev, generator=g)
    loss_fn = torch.nn.CrossEntropyLoss()

    def step() -> torch.Tensor:
        opt.zero_grad(set_to_none=True)
        loss = loss_fn(ddp(x).float(), y)
        loss.backward()
        opt.step()
        return loss

    from .clocks import ClockSampler
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(a.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    sampler.mark_end()
    clocks = sampler.stop()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], dtype=torch.float32, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    grad_bytes = sum(p.numel() for p in model.parameters()) * 2
    if rank == 0:
        ms_v = float(ms.item())
        print(json.dumps({"bench": "ddp_resnet50", "backend": a.backend, "hook": bool(tb is not None and not a.no_hook),
                          "gpus": world, "batch_per_gpu": a.batch, "dtype": "bf16", "bucket_mb": a.bucket_mb,
                          "ms_per_step": round(ms_v, 3), "images_per_s": round(a.batch * world / (ms_v * 1e-3), 1),
                          "steps_per_s": round(1e3 / ms_v, 3), "grad_bytes": grad_bytes,
                          "loss": float(loss.item()), "data": "synthetic", "clocks": clocks}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
