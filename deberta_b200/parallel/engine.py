"""Flat-buffer training engine: parameter storage, gradient synchronisation and AdamW.

This takes the place of ``accelerator.prepare`` + ``torch.optim.AdamW`` + DDP/FSDP of the
reference (``training/entrypoint.py:531-566``, ``training/runtime.py:139-296``) with a
layout chosen for a 180 GB GPU and NVSwitch:

* every trainable parameter lives in ONE flat buffer per dtype role — fp32 master
  weights, fp32 gradients, and (bf16 mode) the bf16 compute copy the kernels read.
  ``param.data`` is a view of the compute buffer, ``param.main_grad`` a view of the
  gradient buffer; weight-gradient GEMMs accumulate straight into it.
* buffers are ordered generator-decay | generator-no-decay | discriminator-decay |
  discriminator-no-decay, so each optimizer (and each phase of decoupled training)
  owns one contiguous range: its gradient reduction is one collective over one range and
  its update is one fused AdamW launch per decay group.
* ``parallelism="ddp"`` all-reduces the range; ``"zero"`` (sharded optimizer state) reduce-scatters it,
  updates the local shard and all-gathers the bf16 compute copy; ``"fsdp"`` (full shard) also keeps the
  compute copy sharded and gathers it layer by layer (``parallel/fsdp.py``).
* the clip coefficient and the non-finite guard are evaluated on the device inside the
  AdamW kernel from the reduced squared norm, so a step needs no host synchronisation;
  the host reads the norm afterwards (or a step later) for logging and LR back-off.
"""

from __future__ import annotations

import ctypes
import hashlib
import math
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from deberta_b200.ops import _lib

from .dist import DistContext
from .peer import PeerComm, fused_comm_wanted

__all__ = ["TrainEngine", "Segment", "OptimizerState", "partition_parameters", "param_order_digest"]

_ALIGN = 64  # elements; keeps every parameter 128-byte (bf16) / 256-byte (fp32) aligned for TMA and vector IO


def is_no_decay_param(name: str, param: torch.Tensor) -> bool:
    """1-D biases, anything named like a norm, and all ≤1-D tensors skip weight decay (``runtime.py:35-52``).

    Two-dimensional tensors called ``bias`` (the GDES embedding deltas) are decayed.
    """
    n = name.lower()
    if n.endswith(".bias") and param.dim() <= 1:
        return True
    if any(k in n for k in ("layernorm", "layer_norm", "rmsnorm", "rms_norm")):
        return True
    return param.dim() <= 1


def is_generator_param(name: str) -> bool:
    return name.startswith(("generator.", "generator_lm_head.", "enhanced_mask_decoder."))


GROUP_ORDER = ("gen_decay", "gen_no_decay", "disc_decay", "disc_no_decay")


def partition_parameters(model: nn.Module) -> dict[str, list[tuple[str, nn.Parameter]]]:
    """Trainable parameters in the four optimizer groups, each Parameter object once (``runtime.py:72-111``)."""
    groups: dict[str, list[tuple[str, nn.Parameter]]] = {k: [] for k in GROUP_ORDER}
    seen: set[int] = set()
    for name, p in model.named_parameters():
        if not p.requires_grad or id(p) in seen:
            continue
        seen.add(id(p))
        key = ("gen" if is_generator_param(name) else "disc") + ("_no_decay" if is_no_decay_param(name, p) else "_decay")
        groups[key].append((name, p))
    return groups


def param_order_digest(model: nn.Module, owners: tuple[str, ...] = ("gen", "disc")) -> str:
    """Digest of parameter names in optimizer order; guards Adam state against silent re-mapping on resume."""
    parts = partition_parameters(model)
    names = [n for key in GROUP_ORDER if key.split("_")[0] in owners for n, _ in parts[key]]
    return hashlib.sha256("\n".join(names).encode()).hexdigest()[:16]


@dataclass
class Segment:
    group: str          # gen_decay | gen_no_decay | disc_decay | disc_no_decay
    start: int
    end: int
    weight_decay: float
    base_lr: float


@dataclass
class OptimizerState:
    """One optimizer = one contiguous range of the flat buffers plus its moments."""

    name: str
    start: int
    end: int
    segments: list[Segment]
    betas: tuple[float, float]
    eps: float
    step: int = 0
    shard: tuple[int, int] = (0, 0)  # range (absolute) whose moments this rank holds
    exp_avg: torch.Tensor | None = None
    exp_avg_sq: torch.Tensor | None = None
    norm_sq: torch.Tensor | None = None  # device float: squared global grad norm of the last sync
    names: list[str] = field(default_factory=list)
    epoch: int = 0  # call number of the last fused reduction (pairs it with the fused update)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class TrainEngine:
    """Owns parameter/gradient/optimizer memory of one model replica on one device."""

    def __init__(self, model: nn.Module, ctx: DistContext, *, compute_dtype: torch.dtype = torch.float32,
                 parallelism: str = "ddp", decoupled: bool = True, lr_generator: float = 5e-4,
                 lr_discriminator: float = 5e-4, weight_decay: float = 0.01, betas: tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, fused_collectives: bool = True, multicast: str = "auto",
                 comm_timeout_s: float = 20.0) -> None:
        if parallelism not in ("ddp", "zero", "fsdp"):
            raise ValueError("parallelism must be 'ddp', 'zero' or 'fsdp'")
        self.model, self.ctx, self.parallelism = model, ctx, parallelism
        self.sharded = parallelism in ("zero", "fsdp")  # optimizer state (and fp32 masters) live on one rank per slab
        self.full_shard = parallelism == "fsdp"
        self.sharder = None
        self.compute_dtype = compute_dtype
        self.device = ctx.device
        self.use_kernels = self.device.type == "cuda"
        model.to(self.device)
        world = ctx.world_size
        parts = partition_parameters(model)
        # ---- layout -----------------------------------------------------------------------
        self.layout: dict[str, tuple[int, int, torch.Size]] = {}
        segs: list[Segment] = []
        bounds: dict[str, tuple[int, int]] = {}
        cursor = 0
        for owner in ("gen", "disc"):
            owner_start = cursor
            for key in (f"{owner}_decay", f"{owner}_no_decay"):
                seg_start = cursor
                for name, p in parts[key]:
                    self.layout[name] = (cursor, p.numel(), p.shape)
                    cursor = _round_up(cursor + p.numel(), _ALIGN)
                wd = weight_decay if key.endswith("_decay") and not key.endswith("no_decay") else 0.0
                segs.append(Segment(key, seg_start, cursor, wd, lr_generator if owner == "gen" else lr_discriminator))
            cursor = _round_up(cursor, _ALIGN * world)  # every optimizer range splits evenly into aligned shards
            if decoupled and (cursor - owner_start) % (world * _ALIGN):
                raise AssertionError("optimizer range is not shard-aligned")
            bounds[owner] = (owner_start, cursor)
        total = cursor
        self.total_elems = total
        dev = self.device
        self.master = torch.zeros(total, dtype=torch.float32, device=dev)
        self.comm = None
        if compute_dtype == torch.bfloat16 and fused_comm_wanted(world, dev, fused_collectives):
            # gradient and parameter buffers live in memory every rank of the node can address
            try:
                self.comm = PeerComm(total, rank=ctx.rank, world_size=world, device=dev,
                                     param_elems=(total // world) if self.full_shard else None,
                                     use_multicast={"on": True, "off": False}.get(str(multicast), None),
                                     timeout_s=float(comm_timeout_s))
            except Exception as e:  # no peer access / symmetric allocator unavailable: NCCL collectives instead
                import logging

                logging.getLogger(__name__).warning("Fused peer-memory collectives unavailable (%s); using NCCL.", e)
                self.comm = None
            # every rank must take the same path
            flag = torch.tensor([1 if self.comm is not None else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag) == 0:
                self.comm = None
            elif not self.comm.self_check():
                import logging

                logging.getLogger(__name__).warning("Fused peer-memory collectives failed their self-check; using NCCL.")
                self.comm = None
        if self.comm is not None:
            self.grads = self.comm.grads
            self.compute = None if self.full_shard else self.comm.params
            ctx.fast_vector_sum = self.comm.vector_sum
        else:
            self.grads = torch.zeros(total, dtype=torch.float32, device=dev)
            self.compute = (torch.zeros(total, dtype=compute_dtype, device=dev)
                            if (compute_dtype != torch.float32 and not self.full_shard) else None)
        self._params: dict[str, nn.Parameter] = {}
        self._owner_bounds = bounds
        for key in GROUP_ORDER:
            for name, p in parts[key]:
                off, n, _ = self.layout[name]
                self.master[off : off + n].copy_(p.data.reshape(-1))
        if world > 1:
            # ranks seed their generators differently (data order, sampling noise), so their freshly initialised
            # weights differ: every replica starts from rank 0's, as DDP / FSDP do when they wrap a module
            dist.broadcast(self.master, src=0)
            for p in model.parameters():
                if not p.requires_grad and p.is_floating_point():
                    dist.broadcast(p.data, src=0)
        for key in GROUP_ORDER:
            for name, p in parts[key]:
                off, n, shape = self.layout[name]
                gview = self.grads[off : off + n].view(shape)
                if self.full_shard:  # storage comes from the sharder's slots below
                    p.grad = None
                    p.main_grad = gview
                    p.register_post_accumulate_grad_hook(_fold_grad_into_main)
                elif self.compute is not None:
                    cview = self.compute[off : off + n]
                    cview.copy_(self.master[off : off + n])
                    p.data = cview.view(shape)
                    p.grad = None
                    p.main_grad = gview
                    p.register_post_accumulate_grad_hook(_fold_grad_into_main)
                else:
                    p.data = self.master[off : off + n].view(shape)
                    p.grad = gview
                self._params[name] = p
        if not self.full_shard:
            self._alias_gdes_bases()
        for p in model.parameters():  # remaining frozen parameters follow the compute dtype
            if not p.requires_grad and p.is_floating_point() and p.dtype != compute_dtype and \
                    (self.compute is not None or self.full_shard):
                p.data = p.data.to(compute_dtype)
        # ---- optimizers ---------------------------------------------------------------------
        self.optimizers: dict[str, OptimizerState] = {}
        specs = ([("generator", "gen"), ("discriminator", "disc")] if decoupled else [("all", None)])
        for opt_name, owner in specs:
            if owner is None:
                start, end = 0, total
                my = segs
            else:
                start, end = bounds[owner]
                my = [s for s in segs if s.group.startswith(owner)]
            if self.sharded and world > 1:
                per = (end - start) // world
                shard = (start + ctx.rank * per, start + (ctx.rank + 1) * per)
            else:
                shard = (start, end)
            n = shard[1] - shard[0]
            names = [nm for s in my for nm, _ in parts[s.group]]
            self.optimizers[opt_name] = OptimizerState(
                opt_name, start, end, my, betas, eps, 0, shard,
                torch.zeros(n, dtype=torch.float32, device=dev), torch.zeros(n, dtype=torch.float32, device=dev),
                torch.zeros(1, dtype=torch.float32, device=dev), names,
            )
        if self.full_shard:
            from .fsdp import ParamSharder

            self.sharder = ParamSharder(self, model, self.layout, self._params, compute_dtype)
            self.sharder.load_from_master(self.master)
            ctx.wait_for_everyone()  # every rank's slabs are filled before anybody gathers
            self.sharder.after_update(None)
            self._alias_gdes_bases()

    def owner_of(self, name: str) -> str:
        """``"gen"`` or ``"disc"``: which backbone's range of the flat layout holds parameter ``name``."""
        off = self.layout[name][0]
        for owner, (a, b) in self._owner_bounds.items():
            if a <= off < b:
                return owner
        raise KeyError(name)

    # ---- GDES ---------------------------------------------------------------------------------
    def _alias_gdes_bases(self) -> None:
        """Point every frozen GDES ``base_weight`` at the generator table it mirrors.

        The base is by definition a copy of the generator embedding refreshed after each
        generator step, and nothing reads it between that step and the refresh; sharing
        the storage makes the refresh (and under sharding its all-gather) disappear.
        """
        for _attr, disc_mod, gen_mod in getattr(self.model, "_gdes_synced_embeddings", []):
            disc_mod.base_weight.data = gen_mod.weight.data

    # ---- gradients ------------------------------------------------------------------------------
    def zero_grad(self, opt_name: str | None = None) -> None:
        if opt_name is None:
            self.grads.zero_()
        else:
            o = self.optimizers[opt_name]
            self.grads[o.start : o.end].zero_()

    def sync_grads(self, opt_name: str, penalty: torch.Tensor | None = None) -> torch.Tensor:
        """Average the optimizer's gradient range over ranks; returns the squared global norm (device scalar).

        ``penalty`` (one device float, 0 or +inf) is added to this rank's share of the squared norm before
        the shares are combined, so that a non-finite loss on any rank makes every rank skip the update.
        Under the fused sharded path the returned scalar is filled in by the following ``step``.
        """
        o = self.optimizers[opt_name]
        world = self.ctx.world_size
        g = self.grads[o.start : o.end]
        if self.comm is not None:
            if self.sharded:
                o.epoch = self.comm.reduce(o.shard[0], o.shard[1] - o.shard[0], scale=1.0 / world, to_all=False,
                                           extra_share=penalty, norm_sq_out=None)
            else:
                per = (o.end - o.start) // world
                o.epoch = self.comm.reduce(o.start + self.ctx.rank * per, per, scale=1.0 / world, to_all=True,
                                           extra_share=penalty, norm_sq_out=o.norm_sq)
            return o.norm_sq
        if world > 1:
            avg = dist.ReduceOp.AVG if self.ctx.backend == "nccl" else dist.ReduceOp.SUM
            if self.sharded:
                out = self.grads[o.shard[0] : o.shard[1]]
                if self.ctx.backend == "nccl":
                    dist.reduce_scatter_tensor(out, g, op=avg)
                else:  # gloo has no reduce-scatter: all-reduce and keep the local shard
                    dist.all_reduce(g, op=avg)
            else:
                dist.all_reduce(g, op=avg)
            if avg == dist.ReduceOp.SUM:
                (self.grads[o.shard[0] : o.shard[1]] if self.sharded else g).mul_(1.0 / world)
        local = self.grads[o.shard[0] : o.shard[1]]
        o.norm_sq.zero_()
        if self.use_kernels:
            _lib.call("db200_sumsq", _lib.ptr(local), ctypes.c_longlong(local.numel()), _lib.ptr(o.norm_sq),
                      _lib.stream_ptr())
        else:
            o.norm_sq.add_(local.double().pow(2).sum().float())
        if world > 1 and self.sharded:
            if penalty is not None:
                o.norm_sq.add_(penalty.to(o.norm_sq.dtype).reshape(1))
            dist.all_reduce(o.norm_sq, op=dist.ReduceOp.SUM)
        elif penalty is not None:
            pen = penalty.to(o.norm_sq.dtype).reshape(1).clone()
            if world > 1:
                dist.all_reduce(pen, op=dist.ReduceOp.SUM)
            o.norm_sq.add_(pen)
        return o.norm_sq

    def grad_norm(self, opt_name: str) -> torch.Tensor:
        return self.optimizers[opt_name].norm_sq.sqrt().squeeze(0)

    # ---- update ---------------------------------------------------------------------------------
    def step(self, opt_name: str, *, lr_scale: float = 1.0, max_grad_norm: float = 0.0,
             gate: torch.Tensor | None = None) -> None:
        """AdamW over the optimizer's (local shard of the) range, clip + finite guard on the device.

        ``gate`` (one float, the same on every rank): the update is skipped when it is not positive. On a GPU the
        decision is taken inside the kernel and the caller corrects ``step`` later; on the CPU it is taken here.
        """
        o = self.optimizers[opt_name]
        o.step += 1
        b1, b2 = o.betas
        inv_bc1 = 1.0 / (1.0 - b1 ** o.step)
        inv_sqrt_bc2 = 1.0 / math.sqrt(1.0 - b2 ** o.step)
        s0, s1 = o.shard
        skipped = False
        if self.comm is not None and self.sharded:
            segs = [(max(sg.start, s0) - s0, min(sg.end, s1) - s0, sg.base_lr * lr_scale, sg.weight_decay)
                    for sg in o.segments if max(sg.start, s0) < min(sg.end, s1)]
            self.comm.adamw(s0, s1 - s0, master=self.master[s0:s1], exp_avg=o.exp_avg, exp_avg_sq=o.exp_avg_sq,
                            segments=segs, betas=o.betas, eps=o.eps, inv_bc1=inv_bc1, inv_sqrt_bc2=inv_sqrt_bc2,
                            max_norm=max_grad_norm, epoch=o.epoch, norm_sq_out=o.norm_sq,
                            gate=None if gate is None else gate.to(torch.float32).reshape(1),
                            local_params=self.sharder.slab_view(opt_name) if self.full_shard else None)
            if self.full_shard:
                self.sharder.after_update(opt_name)
            return
        if gate is not None:
            gate = gate.to(device=self.device, dtype=torch.float32).reshape(1)
        if not self.use_kernels:
            norm = float(o.norm_sq.sqrt())
            if not math.isfinite(norm) or (gate is not None and not float(gate) > 0.0):
                skipped = True
            coef = min(1.0, max_grad_norm / (norm + 1e-6)) if (max_grad_norm > 0 and not skipped) else 1.0
        for seg in o.segments:
            a, b = max(seg.start, s0), min(seg.end, s1)
            if a >= b:
                continue
            lr = seg.base_lr * lr_scale
            p, g = self.master[a:b], self.grads[a:b]
            m, v = o.exp_avg[a - s0 : b - s0], o.exp_avg_sq[a - s0 : b - s0]
            shadow = self.compute[a:b] if self.compute is not None else None
            if self.full_shard:
                shadow = self.sharder.slab_view(opt_name)[a - s0 : b - s0]
            if self.use_kernels:
                c_f = ctypes.c_float
                _lib.call("db200_adamw", _lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), _lib.ptr(shadow),
                          ctypes.c_longlong(b - a), c_f(lr), c_f(seg.weight_decay), c_f(b1), c_f(b2), c_f(o.eps),
                          c_f(inv_bc1), c_f(inv_sqrt_bc2), _lib.ptr(o.norm_sq), c_f(max_grad_norm), c_f(1.0),
                          _lib.ptr(gate), _lib.stream_ptr())
            elif not skipped:
                gg = g * coef if coef != 1.0 else g
                p.mul_(1.0 - lr * seg.weight_decay)
                m.lerp_(gg, 1.0 - b1)
                v.mul_(b2).addcmul_(gg, gg, value=1.0 - b2)
                denom = (v.sqrt() * inv_sqrt_bc2).add_(o.eps)
                p.addcdiv_(m, denom, value=-lr * inv_bc1)
                if shadow is not None:
                    shadow.copy_(p)
        if skipped:
            o.step -= 1
        if self.full_shard:
            if self.ctx.world_size > 1:
                self.ctx.wait_for_everyone()  # every rank's slab is written before any rank reads it
            self.sharder.after_update(opt_name)
        elif self.ctx.world_size > 1 and self.parallelism == "zero":
            # masters stay sharded (only the owner's slice is authoritative); the compute copy is gathered
            buf = self.compute if self.compute is not None else self.master
            mine = buf[s0:s1] if self.ctx.backend == "nccl" else buf[s0:s1].clone()  # only NCCL gathers in place
            dist.all_gather_into_tensor(buf[o.start : o.end], mine)

    def reset_optimizer_state(self, opt_name: str | None = None) -> None:
        for name, o in self.optimizers.items():
            if opt_name in (None, name):
                o.exp_avg.zero_()
                o.exp_avg_sq.zero_()
                o.step = 0

    # ---- state ----------------------------------------------------------------------------------
    def gather_master(self) -> None:
        """Make every rank's fp32 master buffer complete (needed before saving under sharded optimizers)."""
        if self.ctx.world_size > 1 and self.sharded:
            for o in self.optimizers.values():
                dist.all_gather_into_tensor(self.master[o.start : o.end], self.master[o.shard[0] : o.shard[1]].clone())

    def model_state_dict(self) -> dict[str, torch.Tensor]:
        """``model.state_dict()`` with trainable tensors replaced by their fp32 masters (CPU copies)."""
        self.gather_master()
        out: dict[str, torch.Tensor] = {}
        alias = {id(p): n for n, p in self._params.items()}
        for key, t in self.model.state_dict(keep_vars=True).items():
            name = alias.get(id(t))
            if name is not None:
                off, n, shape = self.layout[name]
                out[key] = self.master[off : off + n].view(shape).detach().cpu().clone()
            else:
                out[key] = t.detach().float().cpu().clone() if t.is_floating_point() else t.detach().cpu().clone()
        # frozen GDES bases mirror the generator masters at full precision
        for attr, disc_mod, gen_mod in getattr(self.model, "_gdes_synced_embeddings", []):
            gname = alias.get(id(gen_mod.weight))
            for key, t in self.model.state_dict(keep_vars=True).items():
                if t is disc_mod.base_weight and gname is not None:
                    off, n, shape = self.layout[gname]
                    out[key] = self.master[off : off + n].view(shape).detach().cpu().clone()
        return out

    def load_model_state_dict(self, state: dict[str, torch.Tensor], strict: bool = True) -> None:
        keys = self.model.state_dict(keep_vars=True)
        missing = [k for k in keys if k not in state]
        unexpected = [k for k in state if k not in keys]
        if strict and (missing or unexpected):
            raise RuntimeError(f"state dict mismatch: missing={missing[:5]} unexpected={unexpected[:5]}")
        alias = {id(p): n for n, p in self._params.items()}
        with torch.no_grad():
            for key, t in keys.items():
                if key not in state:
                    continue
                src = state[key].to(self.device)
                name = alias.get(id(t))
                if name is not None:
                    off, n, _ = self.layout[name]
                    self.master[off : off + n].copy_(src.reshape(-1).float())
                    if self.compute is not None:
                        self.compute[off : off + n].copy_(self.master[off : off + n])
                elif any(t is m.base_weight for _, m, _ in getattr(self.model, "_gdes_synced_embeddings", [])):
                    continue  # aliases of generator tables
                else:
                    t.data.copy_(src.to(t.dtype))
        if self.full_shard:
            self.sharder.load_from_master(self.master)
            self.ctx.wait_for_everyone()
            self.sharder.after_update(None)

    def optimizer_state_dict(self) -> dict[str, Any]:
        """This rank's optimizer state in the engine's own flat form (one entry per optimizer)."""
        return {name: {"step": o.step, "shard": list(o.shard), "range": [o.start, o.end], "names": list(o.names),
                       "exp_avg": o.exp_avg.detach().cpu().clone(), "exp_avg_sq": o.exp_avg_sq.detach().cpu().clone()}
                for name, o in self.optimizers.items()}

    def load_optimizer_state_dict(self, state: dict[str, Any]) -> None:
        for name, o in self.optimizers.items():
            s = state[name]
            if list(s["range"]) != [o.start, o.end] or list(s["shard"]) != list(o.shard) or list(s["names"]) != o.names:
                raise RuntimeError(f"optimizer state for {name!r} does not match the current parameter layout")
            o.step = int(s["step"])
            o.exp_avg.copy_(s["exp_avg"].to(self.device))
            o.exp_avg_sq.copy_(s["exp_avg_sq"].to(self.device))

    # ---- optimizer state in the layout of ``torch.optim.AdamW.state_dict()`` --------------------------------
    def _full_moments(self, o: OptimizerState) -> tuple[torch.Tensor, torch.Tensor]:
        """Both moment buffers over the whole optimizer range on every rank (collective under sharding)."""
        if not (self.sharded and self.ctx.world_size > 1):
            return o.exp_avg, o.exp_avg_sq
        out = []
        for part in (o.exp_avg, o.exp_avg_sq):
            full = torch.empty(o.end - o.start, dtype=torch.float32, device=self.device)
            dist.all_gather_into_tensor(full, part.contiguous())
            out.append(full)
        return out[0], out[1]

    def torch_optimizer_state_dicts(self) -> dict[str, dict[str, Any]]:
        """Per optimizer, what ``torch.optim.AdamW(param_groups).state_dict()`` of the reference holds
        (``training/runtime.py:250-296`` there): two parameter groups (decayed, then not decayed), parameters numbered in
        group order, per-parameter ``step`` / ``exp_avg`` / ``exp_avg_sq`` in the parameter's shape. Collective when the
        moments are sharded; every rank returns the full state."""
        out: dict[str, dict[str, Any]] = {}
        for name, o in self.optimizers.items():
            m_full, v_full = self._full_moments(o)
            m_cpu, v_cpu = m_full.detach().cpu(), v_full.detach().cpu()
            groups, state, idx = [], {}, 0
            for seg in o.segments:
                ids = []
                for pname in o.names:
                    off, n, shape = self.layout[pname]
                    if not (seg.start <= off < seg.end):
                        continue
                    if o.step > 0:
                        state[idx] = {"step": torch.tensor(float(o.step)),
                                      "exp_avg": m_cpu[off - o.start : off - o.start + n].view(shape).clone(),
                                      "exp_avg_sq": v_cpu[off - o.start : off - o.start + n].view(shape).clone()}
                    ids.append(idx)
                    idx += 1
                groups.append({"lr": seg.base_lr, "betas": tuple(o.betas), "eps": o.eps, "weight_decay": seg.weight_decay,
                               "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                               "differentiable": False, "fused": None, "decoupled_weight_decay": True, "params": ids})
            out[name] = {"state": state, "param_groups": groups, "param_names": list(o.names)}
        return out

    def load_torch_optimizer_state_dicts(self, states: dict[str, dict[str, Any]]) -> None:
        """Inverse of ``torch_optimizer_state_dicts``; each rank keeps the slice of the moments it owns, so a checkpoint
        can be resumed with any number of ranks and in any parallelism mode."""
        for name, o in self.optimizers.items():
            sd = states[name]
            names = sd.get("param_names")
            if names is not None and list(names) != list(o.names):
                raise RuntimeError(f"optimizer state for {name!r} lists other parameters than the current model")
            order = [pn for seg in o.segments for pn in o.names if seg.start <= self.layout[pn][0] < seg.end]
            n_saved = sum(len(g["params"]) for g in sd["param_groups"])
            if n_saved != len(order):
                raise RuntimeError(f"optimizer state for {name!r} holds {n_saved} parameters, the model has {len(order)}")
            s0, s1 = o.shard
            o.exp_avg.zero_()
            o.exp_avg_sq.zero_()
            step = 0
            for idx, pname in enumerate(order):
                st = sd["state"].get(idx, sd["state"].get(str(idx)))
                if st is None:
                    continue
                step = max(step, int(float(st["step"])))
                off, n, shape = self.layout[pname]
                lo, hi = max(off, s0), min(off + n, s1)
                if lo >= hi:
                    continue
                for key, dst in (("exp_avg", o.exp_avg), ("exp_avg_sq", o.exp_avg_sq)):
                    src = st[key].reshape(-1).float()
                    if src.numel() != n:
                        raise RuntimeError(f"optimizer state of {pname!r} has {src.numel()} elements, expected {n}")
                    dst[lo - s0 : hi - s0].copy_(src[lo - off : hi - off].to(self.device))
            o.step = step


def _fold_grad_into_main(p: torch.Tensor) -> None:
    """Autograd produced ``p.grad`` (ops without a fused weight-gradient path): add it to the fp32 buffer."""
    if p.grad is not None:
        p.main_grad.add_(p.grad)
        p.grad = None
