"""Symmetric buffers and the fused gradient collectives that run on them.

``PeerComm`` owns three allocations that exist with the same size on every rank of a node and
are mapped into every rank's address space (``torch.distributed._symmetric_memory`` does the
handle exchange; nothing else of it is used):

* the engine's flat fp32 gradient buffer,
* the engine's flat bf16 parameter buffer,
* a 8 KiB pad of flags and scalars the kernels use to order themselves between GPUs.

On top of those it exposes the three launches of ``csrc/comm.cu``: slab reduction (+ squared
norm), slab AdamW that stores the new bf16 parameters to all ranks, and a tiny vector sum.
They stand in for the bucketed all-reduce / reduce-scatter / all-gather traffic that the
reference gets from DDP and FSDP (``training/entrypoint.py:348-359``, the FSDP launch
configs under ``configs/accelerate``), and for its scalar reductions
(``training/steps.py:62-75,305-310``).

Every call consumes one epoch number; all ranks must issue the same calls in the same order.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch
import torch.distributed as dist

from ..ops import _lib

__all__ = ["PeerComm", "CommCtx", "AdamSegment", "fused_comm_wanted", "MAX_WORLD", "VEC_MAX", "PAD_WORDS"]

MAX_WORLD = 8
VEC_MAX = 128
PAD_WORDS = 2048


class CommCtx(ctypes.Structure):
    _fields_ = [
        ("world", ctypes.c_int),
        ("rank", ctypes.c_int),
        ("grads", ctypes.c_void_p * MAX_WORLD),
        ("params", ctypes.c_void_p * MAX_WORLD),
        ("pads", ctypes.c_void_p * MAX_WORLD),
        ("mc_grads", ctypes.c_void_p),
        ("mc_params", ctypes.c_void_p),
        ("timeout_ns", ctypes.c_ulonglong),
    ]


class AdamSegment(ctypes.Structure):
    _fields_ = [("begin", ctypes.c_longlong), ("end", ctypes.c_longlong), ("lr", ctypes.c_float),
                ("weight_decay", ctypes.c_float)]


def fused_comm_wanted(world_size: int, device: torch.device, enabled: bool = True) -> bool:
    """Fused collectives serve 2..8 GPUs of one node (``train.distributed.fused_collectives``); otherwise NCCL."""
    if not enabled or device.type != "cuda" or not (2 <= world_size <= MAX_WORLD):
        return False
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world_size)))
    return local_world == world_size  # peer mappings need all ranks on one node


class PeerComm:
    """Symmetric gradient / parameter buffers of one rank plus the launches that use them."""

    def __init__(self, n_elems: int, *, rank: int, world_size: int, device: torch.device, want_params: bool = True,
                 use_multicast: bool | None = None, timeout_s: float = 20.0, param_elems: int | None = None) -> None:
        import torch.distributed._symmetric_memory as symm

        self.rank, self.world, self.device = rank, world_size, device
        group = dist.group.WORLD
        self.grads = symm.empty(n_elems, dtype=torch.float32, device=device)
        # full-shard mode keeps only this rank's slabs here (``param_elems``); peers read them through the mapping
        self.params = symm.empty(n_elems if param_elems is None else param_elems, dtype=torch.bfloat16,
                                 device=device) if want_params else None
        self.pad = symm.empty(PAD_WORDS, dtype=torch.int32, device=device)
        self.grads.zero_()
        self.pad.zero_()
        if self.params is not None:
            self.params.zero_()
        torch.cuda.synchronize(device)
        self._handles = [symm.rendezvous(t, group) for t in (self.grads, self.pad) + ((self.params,) if want_params else ())]
        hg, hp = self._handles[0], self._handles[1]
        hw = self._handles[2] if want_params else None
        if use_multicast is None:
            # measured: at 2 ranks plain peer loads/stores are faster (1.11 vs 1.64 ms); at 8 ranks the switch reduction
            # is as fast for the sharded step and faster for the all-reduce (1.43 vs 1.93 ms)
            use_multicast = world_size >= 4
        mc_g = int(getattr(hg, "multicast_ptr", 0) or 0) if use_multicast else 0
        mc_w = int(getattr(hw, "multicast_ptr", 0) or 0) if (use_multicast and hw is not None) else 0
        self.multicast = bool(mc_g)
        ctx = CommCtx()
        ctx.world, ctx.rank = world_size, rank
        for r in range(world_size):
            ctx.grads[r] = int(hg.buffer_ptrs[r])
            ctx.pads[r] = int(hp.buffer_ptrs[r])
            ctx.params[r] = int(hw.buffer_ptrs[r]) if hw is not None else 0
        ctx.mc_grads = mc_g or None
        ctx.mc_params = mc_w or None
        ctx.timeout_ns = int(timeout_s * 1e9)
        self.ctx = ctx
        self.param_ptrs = [int(hw.buffer_ptrs[r]) for r in range(world_size)] if hw is not None else None
        self.epoch = 0
        dist.barrier()  # every pad is zeroed and mapped before the first flag is written

    def self_check(self) -> bool:
        """Run the three launches on a few KiB and compare with ``torch.distributed``; True when all ranks agree.

        Called once by the engine before the buffers carry data: a fabric on which peer access misbehaves is found
        here (and the engine falls back to NCCL collectives) instead of in the middle of a run.
        """
        ok = True
        try:
            world, rank, dev = self.world, self.rank, self.device
            per = 256
            n = per * world
            probe = (torch.arange(n, device=dev, dtype=torch.float32) % 7) + float(rank)
            want = probe.clone()
            dist.all_reduce(want)
            self.grads[:n].copy_(probe)
            dist.barrier()
            norm = torch.zeros(1, device=dev)
            self.reduce(rank * per, per, scale=1.0, to_all=True, extra_share=None, norm_sq_out=norm)
            vec = torch.arange(5, device=dev, dtype=torch.float32) * (rank + 1)
            got_vec = self.vector_sum(vec)
            want_vec = vec.clone()
            dist.all_reduce(want_vec)
            torch.cuda.synchronize(dev)
            ok = bool(torch.allclose(self.grads[:n], want, rtol=1e-5, atol=1e-5)) and \
                bool(torch.allclose(got_vec, want_vec, rtol=1e-6, atol=1e-6)) and \
                abs(float(norm) - float(want.double().pow(2).sum())) <= 1e-3 * float(want.double().pow(2).sum()) + 1e-3
            code = int(_lib.lib().db200_status_read_and_clear())
            ok = ok and code == 0
        except Exception:  # noqa: BLE001
            ok = False
        flag = torch.tensor([1 if ok else 0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        self.grads[: 256 * self.world].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier()
        return bool(int(flag))

    # ---- launches -------------------------------------------------------------------------------
    def _next_epoch(self) -> ctypes.c_uint:
        self.epoch += 1
        return ctypes.c_uint(self.epoch & 0xFFFFFFFF)

    def reduce(self, offset: int, count: int, *, scale: float, to_all: bool, extra_share: torch.Tensor | None,
               norm_sq_out: torch.Tensor | None) -> int:
        """Sum this rank's slab ``[offset, offset+count)`` over all ranks; returns the epoch that was used."""
        e = self._next_epoch()
        _lib.call("db200_comm_reduce", ctypes.byref(self.ctx), ctypes.c_longlong(offset), ctypes.c_longlong(count),
                  ctypes.c_float(scale), ctypes.c_int(1 if to_all else 0), e, _lib.ptr(extra_share),
                  _lib.ptr(norm_sq_out), _lib.stream_ptr())
        return int(e.value)

    def adamw(self, offset: int, count: int, *, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
              segments: Sequence[tuple[int, int, float, float]], betas: tuple[float, float], eps: float, inv_bc1: float,
              inv_sqrt_bc2: float, max_norm: float, epoch: int, norm_sq_out: torch.Tensor | None,
              gate: torch.Tensor | None = None, local_params: torch.Tensor | None = None) -> None:
        """AdamW on the slab reduced under ``epoch``; ``segments`` = (begin, end, lr, weight_decay) inside the slab.

        ``gate``: optional device float, identical on all ranks; the update is skipped when it is not positive.
        """
        if self.params is None and local_params is None:
            raise RuntimeError("PeerComm was built without a parameter buffer")
        arr = (AdamSegment * max(1, len(segments)))()
        for i, (b, en, lr, wd) in enumerate(segments):
            arr[i] = AdamSegment(b, en, lr, wd)
        cf = ctypes.c_float
        _lib.call("db200_comm_adamw", ctypes.byref(self.ctx), ctypes.c_longlong(offset), ctypes.c_longlong(count),
                  _lib.ptr(master), _lib.ptr(exp_avg), _lib.ptr(exp_avg_sq), arr, ctypes.c_int(len(segments)),
                  cf(betas[0]), cf(betas[1]), cf(eps), cf(inv_bc1), cf(inv_sqrt_bc2), cf(max_norm),
                  ctypes.c_uint(epoch & 0xFFFFFFFF), _lib.ptr(norm_sq_out), _lib.ptr(gate), _lib.ptr(local_params), _lib.stream_ptr())

    def vector_sum(self, values: torch.Tensor) -> torch.Tensor:
        """Sum a float vector of at most ``VEC_MAX`` entries over all ranks (result on the device)."""
        n = values.numel()
        if n > VEC_MAX:
            raise ValueError(f"vector_sum takes at most {VEC_MAX} values")
        src = values.detach().to(device=self.device, dtype=torch.float32).reshape(-1).contiguous()
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        _lib.call("db200_comm_vector_sum", ctypes.byref(self.ctx), _lib.ptr(src), _lib.ptr(out), ctypes.c_int(n),
                  self._next_epoch(), _lib.stream_ptr())
        return out.view(values.shape)
