"""One process per GPU over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

Replaces the Accelerate layer of the reference (``training/entrypoint.py:321-359``): rank
discovery from the launcher environment, barriers, small host-visible reductions and
object broadcast. Bulk gradient/parameter traffic does not go through here; it belongs
to ``parallel/engine.py`` and the fused kernels.
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

__all__ = ["DistContext", "init_distributed"]


@dataclass
class DistContext:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    backend: str | None = None
    owns_group: bool = False
    fast_vector_sum: Any = None  # set by the engine: sums a short fp32 device vector over ranks in one kernel

    @property
    def is_main_process(self) -> bool:
        return self.rank == 0

    @property
    def distributed(self) -> bool:
        return self.world_size > 1

    # names kept close to what the training loop of the reference calls on its accelerator
    def wait_for_everyone(self) -> None:
        if self.distributed:
            dist.barrier()

    def reduce(self, tensor: torch.Tensor, reduction: str = "sum") -> torch.Tensor:
        """All-reduce a small tensor (sum or mean) and return it; identity for one process."""
        if not self.distributed:
            return tensor
        if (self.fast_vector_sum is not None and tensor.dtype == torch.float32 and tensor.is_cuda
                and 0 < tensor.numel() <= 128):
            t = self.fast_vector_sum(tensor)
            return t / self.world_size if reduction == "mean" else t
        t = tensor.clone()
        if t.device != self.device and self.backend == "nccl":
            t = t.to(self.device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        if reduction == "mean":
            t = t / self.world_size
        return t.to(tensor.device)

    def gather(self, tensor: torch.Tensor) -> torch.Tensor:
        """Concatenate a tensor from every rank along dim 0."""
        if not self.distributed:
            return tensor
        t = tensor.reshape(1) if tensor.ndim == 0 else tensor
        t = t.to(self.device) if self.backend == "nccl" else t
        out = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(out, t)
        return torch.cat(out, dim=0).to(tensor.device)

    def broadcast_object(self, obj: Any, src: int = 0) -> Any:
        if not self.distributed:
            return obj
        box = [obj if self.rank == src else None]
        dist.broadcast_object_list(box, src=src)
        return box[0]

    def shutdown(self) -> None:
        if self.owns_group and dist.is_initialized():
            dist.destroy_process_group()


def init_distributed(*, prefer_cuda: bool = True, timeout_s: float = 1800.0) -> DistContext:
    """Join (or create) the default process group from ``RANK/WORLD_SIZE/LOCAL_RANK/MASTER_*``."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = prefer_cuda and torch.cuda.is_available()
    device = torch.device("cuda", local % max(1, torch.cuda.device_count())) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world <= 1:
        return DistContext(0, 1, local, device, None, False)
    backend = "nccl" if use_cuda else "gloo"
    owns = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw: dict[str, Any] = {"backend": backend, "rank": rank, "world_size": world,
                              "timeout": datetime.timedelta(seconds=timeout_s)}
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group(**kw)
        owns = True
    return DistContext(rank, world, local, device, backend, owns)
