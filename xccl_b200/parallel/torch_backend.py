"""torch.distributed backend "b200xccl" (``csrc/torch/pg_xccl.cpp``) and the DDP gradient hook.

    import xccl_b200.parallel.torch_backend as tb
    tb.register()                                   # once per process
    dist.init_process_group("b200xccl", ...)        # CPU tensors -> host team, CUDA -> NVLink team
    model = DDP(model, bucket_cap_mb=25)
    model.register_comm_hook(None, tb.fused_allreduce_hook)

The hook replaces DDP's "divide, allreduce, (cast)" by ONE collective whose kernel applies the
1/world scale (and an optional cast) where the reduced value is produced.
"""
import importlib.util
import os
from pathlib import Path
from typing import Any, Optional

import torch
import torch.distributed as dist

from .. import _capi

BACKEND = "b200xccl"
_ext = None


def extension():
    """Loads (building it on first use if needed) the compiled c10d backend module."""
    global _ext
    if _ext is not None:
        return _ext
    _capi.load()
    so = Path(__file__).resolve().parent.parent / "lib" / "xccl_torch.so"
    if not so.exists():
        from .. import build
        build.build_torch_ext()
    spec = importlib.util.spec_from_file_location("xccl_torch", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _ext = mod
    return mod


def register() -> None:
    ext = extension()
    if BACKEND.upper() in dist.Backend.__dict__ or BACKEND in getattr(dist.Backend, "backend_list", []):
        return
    dist.Backend.register_backend(BACKEND, ext.create_backend, devices=["cpu", "cuda"])


def _backend_of(group: Optional[dist.ProcessGroup], device: torch.device):
    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    return pg._get_backend(device)


def allreduce_fused(inp: torch.Tensor, out: torch.Tensor, scale: float, group=None):
    """out = cast(scale * sum_over_ranks(inp)) in one kernel; returns a c10d Work."""
    return extension().allreduce_fused(_backend_of(group, inp.device), inp, out, float(scale))


def empty_symmetric(shape, dtype: torch.dtype = torch.float32, group=None) -> torch.Tensor:
    """A CUDA tensor in the team's symmetric memory (collective: every rank calls it with the same shape).
    ``dist.all_reduce`` / ``broadcast`` on such tensors - the same tensor or the same offset of it on every rank - run
    zero-copy: the NVSwitch adds the ranks' buffers in place and replicates the result. Free with ``free_symmetric``."""
    dev = torch.cuda.current_device()
    n = 1
    for s_ in (shape if isinstance(shape, (tuple, list)) else (shape,)):
        n *= int(s_)
    nbytes = n * torch.tensor([], dtype=dtype).element_size()
    raw = extension().empty_symmetric(_backend_of(group, torch.device("cuda", dev)), (nbytes + 255) // 256 * 256, dev)
    return raw[:nbytes].view(dtype).view(shape)


def free_symmetric(t: torch.Tensor, group=None) -> None:
    """Returns memory of ``empty_symmetric`` (collective)."""
    extension().free_symmetric(_backend_of(group, t.device), t)


def coll_tl(coll: int, cuda: bool, group=None) -> str:
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    return extension().coll_tl(_backend_of(group, dev), coll, cuda)


def fused_allreduce_hook(state: Any, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """DDP communication hook: gradient averaging fused into the allreduce (no separate div)."""
    buf = bucket.buffer()
    world = dist.get_world_size(state if isinstance(state, dist.ProcessGroup) else None)
    work = allreduce_fused(buf, buf, 1.0 / world, state if isinstance(state, dist.ProcessGroup) else None)
    return work.get_future().then(lambda f: f.value()[0])
