"""Full-shard data parallelism: compute-dtype parameters exist only as per-rank slabs, gathered per layer.

Counterpart of launching the reference with its FSDP2 configs (``configs/accelerate/fsdp2_*.yaml``:
``fsdp_version: 2``, transformer-layer wrapping, ``fsdp_reshard_after_forward: true``), built on the flat-buffer
engine instead of DTensors:

* sharding follows the optimizer slabs of the engine: rank *r* keeps the fp32 masters, the Adam moments and the
  compute-dtype (bf16) copy of ``[start + r·per, start + (r+1)·per)`` of every optimizer range, nothing else;
* a *unit* is one transformer layer (its weights are two contiguous ranges of the flat layout: decayed and
  non-decayed) or, per backbone, the *root* (embeddings, relative-position table, heads) — the same grouping FSDP's
  ``TRANSFORMER_BASED_WRAP`` produces;
* before a layer unit runs — forward, backward, or the recomputation of activation checkpointing — its ranges are
  copied from the owning ranks into one of two layer-sized slots and the module's parameters are pointed at that slot;
  the next unit's copy is issued on a side stream at the same time, so it lands while the current layer computes.
  After the forward nothing is kept: the slot is simply reused ("reshard"). Weights saved by autograd are views of a
  slot; a unit always lands in the same slot, and is gathered again before its backward, so those views read the
  right numbers when they are used. Root units are gathered after every optimizer step of their backbone and stay;
* the copy is a plain load/store kernel over peer-mapped shard buffers (``csrc/comm.cu::copy_pieces_kernel``; no
  library kernel is handed peer memory, no TMA multicast), or, without peer access (CPU/gloo, several nodes), one
  broadcast per owning rank;
* gradients are produced into the engine's full fp32 gradient buffer during accumulation (FSDP2 under ``no_sync``
  keeps unsharded gradients too) and reduce-scattered onto the slabs once per window by the same fused kernels the
  sharded-optimizer mode uses; the update writes the new bf16 slab locally and nothing is pushed to peers.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from deberta_b200.ops import _lib

__all__ = ["ParamSharder", "Unit", "find_layer_modules"]


def find_layer_modules(backbone: nn.Module) -> list[nn.Module]:
    """The transformer layers of a backbone (``encoder.layer`` of the DeBERTa-v2 model, ``encoder.layers`` of rope)."""
    enc = getattr(backbone, "encoder", None)
    for attr in ("layer", "layers"):
        layers = getattr(enc, attr, None)
        if isinstance(layers, nn.ModuleList):
            return list(layers)
    return []


@dataclass
class Unit:
    name: str
    owner: str                       # "gen" | "disc": which optimizer's step invalidates it
    ranges: list[tuple[int, int]]    # absolute ranges of the flat layout, ascending
    params: list[tuple[nn.Parameter, int, torch.Size]] = field(default_factory=list)  # (parameter, offset in the unit, shape)
    module: nn.Module | None = None  # layer units only
    is_root: bool = False
    size: int = 0                    # elements
    index: int = 0
    stack: int = -1                  # which layer stack (for prefetch neighbours)
    pos: int = -1                    # position inside the stack

    def offset_of(self, flat: int) -> int:
        off = 0
        for a, b in self.ranges:
            if a <= flat < b:
                return off + (flat - a)
            off += b - a
        raise KeyError(flat)


class ParamSharder:
    """Owns the parameter slabs, the gather slots and the hooks of one engine in full-shard mode."""

    def __init__(self, engine: Any, model: nn.Module, layout: dict[str, tuple[int, int, torch.Size]],
                 params: dict[str, nn.Parameter], dtype: torch.dtype) -> None:
        self.engine, self.dtype = engine, dtype
        self.ctx = engine.ctx
        self.device = engine.device
        self.world, self.rank = self.ctx.world_size, self.ctx.rank
        self.es = torch.empty(0, dtype=dtype).element_size()
        # ---- slabs: [(optimizer name, owner, start, per)] and this rank's shard buffer ----
        self.slabs: list[tuple[str, str, int, int, int]] = []  # (opt, owner, start, per, base in the shard buffer)
        base = 0
        for name, o in engine.optimizers.items():
            per = (o.end - o.start) // self.world
            owner = "gen" if name == "generator" else ("disc" if name == "discriminator" else "all")
            self.slabs.append((name, owner, o.start, per, base))
            base += per
        self.shard_elems = base
        comm = engine.comm
        self.peer_shards: list[int] | None = None
        if comm is not None and comm.params is not None:
            self.shard = comm.params[: self.shard_elems]
            self.peer_shards = comm.param_ptrs
        else:
            self.shard = torch.zeros(self.shard_elems, dtype=dtype, device=self.device)
        # ---- units ----
        self.units: list[Unit] = []
        name_of = {id(p): n for n, p in params.items()}
        taken: set[str] = set()
        stacks = [("gen", getattr(model, "generator", None)), ("disc", getattr(model, "discriminator", None))]
        for si, (owner, backbone) in enumerate(stacks):
            if backbone is None:
                continue
            for li, layer in enumerate(find_layer_modules(backbone)):
                names = [name_of[id(p)] for p in layer.parameters() if id(p) in name_of and name_of[id(p)] not in taken]
                if not names:
                    continue
                taken.update(names)
                u = self._make_unit(f"{owner}.layer{li}", owner, names, layout, params)
                u.module, u.stack, u.pos = layer, si, li
                self.units.append(u)
        for owner in ("gen", "disc"):
            names = [n for n in layout if n not in taken and engine.owner_of(n) == owner]
            if names:
                u = self._make_unit(f"{owner}.root", owner, names, layout, params)
                u.is_root = True
                self.units.append(u)
        for i, u in enumerate(self.units):
            u.index = i
        # ---- slots ----
        layer_units = [u for u in self.units if not u.is_root]
        self.slot_elems = max((u.size for u in layer_units), default=0)
        self.slots = [torch.zeros(self.slot_elems, dtype=dtype, device=self.device) for _ in range(2 if layer_units else 0)]
        self.root_bufs = {u.index: torch.zeros(u.size, dtype=dtype, device=self.device) for u in self.units if u.is_root}
        self.slot_holds: list[tuple[int, int] | None] = [None, None]  # (unit index, parameter version) per slot
        self.slot_event: list[Any] = [None, None]    # gather finished (side stream)
        self.slot_free: list[Any] = [None, None]     # last compute that read the slot was enqueued (main stream)
        self.version = {"gen": 0, "disc": 0, "all": 0}
        self._views: dict[tuple[int, int], list[torch.Tensor]] = {}
        self.side = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.gathers = 0  # bookkeeping for tests and reports
        self.bytes_gathered = 0
        for u in self.units:
            if u.is_root:
                self._point(u, self.root_bufs[u.index], key=-1)
            else:
                self._point(u, self.slots[self._slot_of(u)], key=self._slot_of(u))
                u.module.register_forward_pre_hook(lambda _m, _a, u=u: self.prepare(u, backward=False))
                u.module.register_full_backward_pre_hook(lambda _m, _g, u=u: self.prepare(u, backward=True))

    # ---- construction helpers ---------------------------------------------------------------------------------
    def _make_unit(self, name, owner, names, layout, params) -> Unit:
        spans = sorted((layout[n][0], layout[n][0] + layout[n][1], n) for n in names)
        ranges: list[list[int]] = []
        align = 64
        for a, b, _ in spans:
            b = (b + align - 1) // align * align  # the engine pads every parameter to 64 elements
            if ranges and a <= ranges[-1][1]:
                ranges[-1][1] = max(ranges[-1][1], b)
            else:
                ranges.append([a, b])
        u = Unit(name=name, owner=owner, ranges=[(a, b) for a, b in ranges])
        u.size = sum(b - a for a, b in u.ranges)
        for a, _, n in spans:
            u.params.append((params[n], u.offset_of(a), layout[n][2]))
        return u

    def _slot_of(self, u: Unit) -> int:
        return u.pos % 2

    def _point(self, u: Unit, buf: torch.Tensor, key: int) -> None:
        views = self._views.get((u.index, key))
        if views is None:
            views = [buf[off : off + shape.numel()].view(shape) for _, off, shape in u.params]
            self._views[(u.index, key)] = views
        for (p, _, _), v in zip(u.params, views):
            p.data = v

    # ---- gather -----------------------------------------------------------------------------------------------
    def _pieces(self, u: Unit) -> list[tuple[int, int, int, int]]:
        """(owner rank, offset in that rank's shard buffer, offset in the unit, elements) covering the unit."""
        out = []
        for a, b in u.ranges:
            for _name, _owner, start, per, base in self.slabs:
                lo, hi = max(a, start), min(b, start + per * self.world)
                if lo >= hi:
                    continue
                r = (lo - start) // per
                while lo < hi:
                    end = min(hi, start + (r + 1) * per)
                    out.append((r, base + lo - (start + r * per), u.offset_of(lo), end - lo))
                    lo, r = end, r + 1
        return out

    def _gather_into(self, u: Unit, buf: torch.Tensor) -> None:
        """Enqueue the copy of unit ``u`` into ``buf`` on the current stream."""
        pieces = self._pieces(u)
        self.gathers += 1
        self.bytes_gathered += sum(n for r, _, _, n in pieces if r != self.rank) * self.es
        if self.world == 1 or self.peer_shards is not None:
            ptrs = self.peer_shards if self.peer_shards is not None else [self.shard.data_ptr()]
            for i in range(0, len(pieces), 16):
                chunk = pieces[i : i + 16]
                n = len(chunk)
                src = (ctypes.c_void_p * n)(*[ptrs[r] + so * self.es for r, so, _, _ in chunk])
                dst = (ctypes.c_void_p * n)(*[buf.data_ptr() + do * self.es for _, _, do, _ in chunk])
                size = (ctypes.c_longlong * n)(*[cnt * self.es for _, _, _, cnt in chunk])
                if self.device.type == "cuda":
                    _lib.call("db200_comm_copy_pieces", src, dst, size, ctypes.c_int(n), _lib.stream_ptr())
                else:
                    for _, so, do, cnt in chunk:
                        buf[do : do + cnt].copy_(self.shard[so : so + cnt])
            return
        for r, so, do, cnt in pieces:  # no peer mapping: the owner broadcasts its piece
            dst = buf[do : do + cnt]
            if r == self.rank:
                dst.copy_(self.shard[so : so + cnt])
            dist.broadcast(dst, src=r)

    def _neighbour(self, u: Unit, backward: bool) -> Unit | None:
        want = u.pos + (-1 if backward else 1)
        for v in self.units:
            if not v.is_root and v.stack == u.stack and v.pos == want:
                return v
        return None

    def _issue(self, u: Unit, slot: int, on_side: bool) -> None:
        ver = self.version[u.owner]
        if self.slot_holds[slot] == (u.index, ver):
            return
        cuda = self.device.type == "cuda"
        if cuda and on_side and self.peer_shards is not None:
            main = torch.cuda.current_stream(self.device)
            self.side.wait_stream(main)  # whatever last used this slot (and the optimizer that wrote the shards) is ahead of us
            with torch.cuda.stream(self.side):
                self._gather_into(u, self.slots[slot])
                ev = torch.cuda.Event()
                ev.record(self.side)
            self.slot_event[slot] = ev
        else:
            self._gather_into(u, self.slots[slot])
            self.slot_event[slot] = None
        self.slot_holds[slot] = (u.index, ver)

    def prepare(self, u: Unit, backward: bool) -> None:
        """Make unit ``u`` resident in its slot (pre-forward / pre-backward hook) and start on its neighbour."""
        slot = self._slot_of(u)
        self._issue(u, slot, on_side=True)
        ev = self.slot_event[slot]
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            self.slot_event[slot] = None
        self._point(u, self.slots[slot], key=slot)
        nxt = self._neighbour(u, backward)
        if nxt is not None and self.peer_shards is not None and self.device.type == "cuda":
            self._issue(nxt, self._slot_of(nxt), on_side=True)

    # ---- parameter updates -----------------------------------------------------------------------------------
    def slab_view(self, opt_name: str) -> torch.Tensor:
        for name, _owner, _start, per, base in self.slabs:
            if name == opt_name:
                return self.shard[base : base + per]
        raise KeyError(opt_name)

    def after_update(self, opt_name: str | None = None) -> None:
        """The slabs of ``opt_name`` (all when ``None``) changed on every rank: drop stale slots, refresh the roots."""
        owners = {"generator": ("gen",), "discriminator": ("disc",), "all": ("gen", "disc", "all"), None: ("gen", "disc", "all")}[opt_name]
        for o in owners:
            self.version[o] += 1
        if self.world > 1 and self.peer_shards is None and self.device.type != "cuda":
            pass  # broadcasts below order themselves
        for u in self.units:
            if u.is_root and (u.owner in owners):
                self._gather_into(u, self.root_bufs[u.index])

    def load_from_master(self, master: torch.Tensor) -> None:
        """Refill this rank's slabs from the fp32 masters (start of training, checkpoint load)."""
        for name, _owner, start, per, base in self.slabs:
            lo = start + self.rank * per
            self.shard[base : base + per].copy_(master[lo : lo + per])

    def memory_report(self) -> dict[str, int]:
        return {"shard_bytes": self.shard_elems * self.es, "slot_bytes": 2 * self.slot_elems * self.es,
                "root_bytes": sum(b.numel() for b in self.root_bufs.values()) * self.es,
                "full_bytes": self.engine.total_elems * self.es}
