"""One optimizer step of RTD pretraining over a gradient-accumulation window.

Semantics follow the hot loop of the reference (``training/entrypoint.py:1046-1884``):

* decoupled (default): phase 1 runs the generator on every micro-batch, steps the generator
  optimizer, refreshes the shared embeddings; phase 2 runs the discriminator on the cached
  corrupted inputs and steps its optimizer. Coupled: one combined objective, one optimizer.
* token-weighted accumulation (``loop_utils``), gradient clipping over the stepping optimizer's
  parameters, schedulers advance on every window, a non-finite window is skipped with LR
  back-off and periodic optimizer-state reset.

What differs is *where* things happen: losses, token weights, the clip coefficient and the
non-finite guard stay on the device, so the host never waits for the GPU inside a window; it
learns the outcome of a step one window later from a pinned-memory copy. On CPU (tests, smoke
runs) the same code resolves everything synchronously.

Window-level rules of the reference that therefore run on the device:

* a non-finite generator loss or gradient norm on any rank skips the *whole* window
  (``entrypoint.py:1174-1212,1243-1257``): the generator's guard is added to the discriminator's, so
  neither optimizer changes its parameters or moments; the discriminator's forward/backward of that
  window still executes (its result is discarded), which the reference avoids by a host round trip;
* a window in which no rank has a masked token does not step the discriminator
  (``entrypoint.py:1269-1296``): with one process (or on the CPU) the phase is skipped on the host, with
  several GPUs the update kernel is gated by the summed token count and the step counter and schedule
  are corrected when the outcome arrives.

Overlap (``train.distributed.overlap_backward``, GPUs only): the discriminator's gradient collective and its
optimizer kernel are queued on a side stream. Nothing of the next window's generator phase reads a discriminator
parameter or gradient, so that whole phase — forward, backward, the generator's own collective and update — runs
while the discriminator's reduce-scatter, AdamW and parameter all-gather are in flight; the main stream waits for
them where the next discriminator phase (or a checkpoint) begins. The two optimizers' fused collectives share one
set of flags, so the generator's collective is queued behind the discriminator's.

The outcome also carries the kernels' status word: a bounded wait that ran out anywhere since the
previous window raises ``KernelError`` here instead of letting the run continue on partial data.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from deberta_b200.models.mask_utils import AttnMask
from deberta_b200.parallel.dist import DistContext
from deberta_b200.parallel.engine import TrainEngine, param_order_digest
from deberta_b200.utils.trace import nvtx_range

from .loop_utils import (apply_nonfinite_recovery, count_input_tokens_for_batch, count_rtd_tokens_for_batch,
                         micro_loss_scale, recover_lr_mult)
from .schedulers import StepSchedule

__all__ = ["Trainer", "WindowStats"]


@dataclass
class WindowStats:
    """Device-side sums of one window; ``.item()`` them only when a log line is due."""

    gen_loss_tokens: torch.Tensor   # Σ gen_loss_i · g_i
    disc_loss_tokens: torch.Tensor  # Σ disc_loss_i · d_i
    disc_acc_tokens: torch.Tensor   # Σ acc_i · d_i
    disc_pos: torch.Tensor          # Σ positives
    gen_tokens: float
    disc_tokens: float
    input_tokens: float
    zero_gen_window: bool = False
    zero_disc_window: bool = False
    grad_norms: dict[str, torch.Tensor] = field(default_factory=dict)


class _PendingOutcome:
    """Squared grad norms, the discriminator gate and the kernel status word of a finished step on their way to the host."""

    def __init__(self, step: int, norms: dict[str, torch.Tensor], sync: bool, gate: torch.Tensor | None = None) -> None:
        self.step = step
        self.names = list(norms)
        self.has_gate = gate is not None
        parts = [norms[n].reshape(1).float() for n in self.names]
        if gate is not None:
            parts.append(gate.reshape(1).float())
        stacked = torch.cat(parts)
        self.status = None
        if stacked.is_cuda:
            from deberta_b200.ops import _lib

            self.status = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            _lib.call("db200_status_snapshot", _lib.ptr(self.status), _lib.stream_ptr())
        if stacked.is_cuda and not sync:
            self.host = torch.empty(stacked.shape, dtype=stacked.dtype, pin_memory=True)
            self.host.copy_(stacked, non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record()
        else:
            self.host = stacked.detach().cpu()
            self.event = None

    def resolve(self) -> tuple[dict[str, float], float | None, int]:
        """(grad norms by optimizer, gate value or None, kernel status word)."""
        if self.event is not None:
            self.event.synchronize()
        elif self.status is not None:
            torch.cuda.current_stream().synchronize()
        vals = self.host.tolist()
        norms = {n: math.sqrt(v) if (v == v and v >= 0) else float("nan") for n, v in zip(self.names, vals)}
        gate = vals[len(self.names)] if self.has_gate else None
        return norms, gate, (0 if self.status is None else int(self.status[0]))


class Trainer:
    """Holds the model/engine/schedules of a run and executes optimizer steps."""

    def __init__(self, *, model: torch.nn.Module, engine: TrainEngine, ctx: DistContext, train_cfg: Any,
                 optim_cfg: Any, pad_token_id: int | None, synchronous: bool | None = None) -> None:
        self.model, self.engine, self.ctx = model, engine, ctx
        self.train_cfg, self.optim_cfg = train_cfg, optim_cfg
        self.pad_token_id = pad_token_id
        self.decoupled = bool(train_cfg.decoupled_training)
        self.ga_steps = int(train_cfg.gradient_accumulation_steps)
        self.token_weighted = bool(train_cfg.token_weighted_gradient_accumulation)
        o = train_cfg.objective
        self.gen_w, self.disc_w = float(o.gen_loss_weight), float(o.disc_loss_weight)
        self.temperature = float(o.sampling_temperature)
        self.max_grad_norm = float(optim_cfg.max_grad_norm)
        # CPU runs resolve step outcomes immediately; GPU runs defer them by one window
        self.synchronous = (engine.device.type != "cuda") if synchronous is None else bool(synchronous)
        kind, warm, total = optim_cfg.scheduler.type, int(optim_cfg.scheduler.warmup_steps), int(train_cfg.max_steps)
        self.schedules = {name: StepSchedule(kind, warmup_steps=warm, total_steps=total,
                                             base_lr=opt.segments[0].base_lr if opt.segments else 1.0)
                          for name, opt in engine.optimizers.items()}
        self.global_step = 0
        self.lr_mult = 1.0
        self.skip_streak = 0
        self.skipped_steps = 0
        self.consumed_micro_batches = 0
        self._pending: _PendingOutcome | None = None
        di = getattr(train_cfg, "distributed", None)
        self.overlap = bool(getattr(di, "overlap_backward", True)) and engine.device.type == "cuda" and self.decoupled \
            and not self.synchronous
        self._side = torch.cuda.Stream(device=engine.device) if self.overlap else None
        self._disc_done = None  # event: the discriminator's collective + update queued on the side stream have finished
        self.last_outcome: dict[str, float] = {}
        self.on_nonfinite = None  # optional callback(step, norms) for debug artifacts
        self.model.train()

    # ---- helpers ----------------------------------------------------------------------------------
    def optimizer_param_digest(self):
        if self.decoupled:
            return {"generator": param_order_digest(self.model, ("gen",)),
                    "discriminator": param_order_digest(self.model, ("disc",))}
        return param_order_digest(self.model)

    def current_lrs(self) -> dict[str, float]:
        return {n: s.get_last_lr()[0] * self.lr_mult for n, s in self.schedules.items()}

    def _to_device(self, batch: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """Copy a micro-batch to the device. A batch that is still on the host also gets ``masked_idx``, the flat
        positions of its MLM targets: found here on the CPU (16 k integers), they spare the generator phase its two
        ``nonzero`` calls, each of which would stall the host until the device had drained its queue."""
        dev = self.engine.device
        out = {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        labels = batch.get("labels")
        if isinstance(labels, torch.Tensor) and not labels.is_cuda and dev.type == "cuda" and "masked_idx" not in out:
            idx = torch.nonzero(labels.reshape(-1).ne(-100), as_tuple=False).squeeze(-1)
            out["masked_idx"] = idx.pin_memory().to(dev, non_blocking=True)
        return out

    def stage_batch(self, batch: dict[str, torch.Tensor]) -> dict[str, Any]:
        """A host micro-batch made device-resident ahead of time (prefetching loaders, benchmarks that keep their inputs
        on the GPU): the copy of :meth:`_to_device` plus ``_counts``, the token counts that :meth:`train_window`
        would otherwise have to read back from the device, one blocking ``.item()`` each."""
        counts = (*count_rtd_tokens_for_batch(batch, pad_token_id=self.pad_token_id), count_input_tokens_for_batch(batch))
        out: dict[str, Any] = self._to_device(batch)
        out["_counts"] = counts
        return out

    @staticmethod
    def _mask_of(batch: dict[str, torch.Tensor]):
        if batch.get("doc_ids") is not None:
            return AttnMask(doc_ids=batch["doc_ids"])
        return batch.get("attention_mask")

    def _window_denominators(self, gen_total: float, disc_total: float):
        """(gen denom, disc denom, window has masked tokens anywhere) — device tensors when several ranks take part.

        The denominators are the per-rank mean of the window token totals, floored at 1.
        """
        if self.ctx.world_size <= 1:
            return max(gen_total, 1.0), max(disc_total, 1.0), gen_total > 0
        t = torch.tensor([gen_total, disc_total], dtype=torch.float32, device=self.engine.device)
        t = self.ctx.reduce(t, "mean")
        return t[0].clamp(min=1.0), t[1].clamp(min=1.0), (t[0] > 0).to(torch.float32)

    def _finish_optimizer(self, name: str, loss_guard: torch.Tensor | None, *, upstream: torch.Tensor | None = None,
                          gate: torch.Tensor | None = None) -> torch.Tensor:
        """Reduce gradients, fold a non-finite loss into the norm, update, advance the schedule.

        ``upstream``: squared norm of an optimizer that stepped earlier in this window; when it is not finite this
        update is skipped too (the whole window is void). ``gate``: see ``TrainEngine.step``.
        """
        eng = self.engine
        self.wait_for_side_stream()  # the fused collectives of the two optimizers share one set of flags
        penalty = None
        if loss_guard is not None:  # +inf when the window's loss was not finite: every rank then skips the update
            penalty = torch.where(torch.isfinite(loss_guard), 0.0, float("inf")).to(torch.float32).reshape(1)
        if upstream is not None:
            up = torch.where(torch.isfinite(upstream.reshape(1)), 0.0, float("inf")).to(torch.float32)
            penalty = up if penalty is None else penalty + up
        norm_sq = eng.sync_grads(name, penalty)
        eng.step(name, lr_scale=self.schedules[name].scale() * self.lr_mult, max_grad_norm=self.max_grad_norm, gate=gate)
        self.schedules[name].step()
        return norm_sq.clone()

    def wait_for_side_stream(self) -> None:
        """Order the current stream behind the discriminator update that may still run on the side stream."""
        if self._disc_done is not None:
            torch.cuda.current_stream(self.engine.device).wait_event(self._disc_done)
            self._disc_done = None

    def resolve_pending(self) -> None:
        """Apply the host-side consequences of the previous step (LR back-off / recovery, gated updates, kernel errors).

        Every rank must call this at the same points (``train_window`` does; so must a checkpoint save), because it
        can change the optimizer step counters, the LR multiplier and the optimizer moments.
        """
        if self._pending is None:
            return
        norms, gate, status = self._pending.resolve()
        step = self._pending.step
        self._pending = None
        if status != 0:
            from deberta_b200.ops import _lib

            _lib.check_status()  # synchronises, clears the word and raises KernelError with the decoded reason
            raise _lib.KernelError(f"device status {status} recorded during optimizer step {step}")
        self.last_outcome = norms
        if any(not math.isfinite(v) for v in norms.values()):
            self.skip_streak += 1
            self.skipped_steps += 1
            self.lr_mult, reset = apply_nonfinite_recovery(lr_mult=self.lr_mult, skip_streak=self.skip_streak)
            for name, v in norms.items():
                if not math.isfinite(v) and self.engine.use_kernels:
                    self.engine.optimizers[name].step -= 1  # the device guard skipped that update
            if reset:
                self.engine.reset_optimizer_state()
            if self.on_nonfinite is not None:
                self.on_nonfinite(step, norms)
        else:
            self.skip_streak = 0
            self.lr_mult = recover_lr_mult(self.lr_mult)
            if gate is not None and not gate > 0.0 and "discriminator" in self.engine.optimizers:
                # no rank had a masked token: the device gate left the discriminator untouched
                self.engine.optimizers["discriminator"].step -= 1
                self.schedules["discriminator"].step_back()

    _resolve_pending = resolve_pending

    # ---- one optimizer step -------------------------------------------------------------------------
    def train_window(self, batches: list[dict[str, torch.Tensor]]) -> WindowStats:
        """Run one gradient-accumulation window (``len(batches)`` micro-batches) and step the optimizer(s)."""
        self.resolve_pending()
        eng, model, dev = self.engine, self.model, self.engine.device
        device_gate = None
        staged = [b.get("_counts") for b in batches]  # batches from stage_batch() carry their host-side counts
        counts = [c[:2] if c is not None else count_rtd_tokens_for_batch(b, pad_token_id=self.pad_token_id)
                  for b, c in zip(batches, staged)]
        input_tokens = sum(c[2] if c is not None else count_input_tokens_for_batch(b) for b, c in zip(batches, staged))
        gen_total, disc_total = sum(c[0] for c in counts), sum(c[1] for c in counts)
        gen_den, disc_den, has_targets = self._window_denominators(gen_total, disc_total)
        scale = micro_loss_scale(ga_steps=len(batches), token_weighted_ga=self.token_weighted)
        zero = lambda: torch.zeros((), dtype=torch.float32, device=dev)  # noqa: E731
        stats = WindowStats(zero(), zero(), zero(), zero(), gen_total, disc_total, input_tokens,
                            zero_gen_window=gen_total <= 0, zero_disc_window=disc_total <= 0)
        if self.overlap:
            # the discriminator's range was cleared on the side stream right after its update (which may still be
            # reading it); the generator's is cleared after its update below, and both start out as zeros
            pass
        else:
            eng.zero_grad()
        norms: dict[str, torch.Tensor] = {}
        if self.decoupled:
            cached = []
            guard = zero()
            for b, (g_i, d_i) in zip(batches, counts):
                b = self._to_device(b)
                mask = self._mask_of(b)
                with nvtx_range("generator fwd"):
                    out = model(input_ids=b["input_ids"], attention_mask=mask, labels=b["labels"],
                                token_type_ids=b.get("token_type_ids"), sampling_temperature=self.temperature,
                                phase="generator", masked_idx=b.get("masked_idx"))
                w = (g_i / gen_den) if self.token_weighted else 1.0
                with nvtx_range("generator bwd"):
                    (out.gen_loss_raw * (self.gen_w * scale) * w).backward()
                guard = guard + out.gen_loss_raw.detach().float()
                stats.gen_loss_tokens += out.gen_loss_raw.detach().float() * g_i
                cached.append((b, mask, out.corrupted_input_ids, out.disc_labels, g_i, d_i))
            with nvtx_range("generator optimizer"):
                norms["generator"] = self._finish_optimizer("generator", guard)
            model.sync_discriminator_embeddings_from_generator()
            eng.zero_grad("generator")
            guard = zero()
            # does any rank have a masked token in this window? known on the host unless several GPUs take part
            device_gate = None
            if isinstance(has_targets, torch.Tensor):
                if has_targets.is_cuda:
                    device_gate = has_targets
                    run_disc = True
                else:
                    run_disc = bool(float(has_targets) > 0.0)
            else:
                run_disc = bool(has_targets)
            if not run_disc:
                cached = []
            self.wait_for_side_stream()  # last window's discriminator update must have landed before its next forward
            for b, mask, corrupted, labels, g_i, d_i in cached:
                with nvtx_range("discriminator fwd"):
                    out = model(input_ids=b["input_ids"], corrupted_input_ids=corrupted, disc_labels=labels,
                                attention_mask=mask, token_type_ids=b.get("token_type_ids"), phase="discriminator")
                w = (d_i / disc_den) if self.token_weighted else 1.0
                w = w * (1.0 if g_i > 0 else 0.0) * has_targets  # micro-batches / windows without masked tokens carry no RTD signal
                with nvtx_range("discriminator bwd"):
                    (out.disc_loss_raw * (self.disc_w * scale) * w).backward()
                guard = guard + out.disc_loss_raw.detach().float()
                stats.disc_loss_tokens += out.disc_loss_raw.detach().float() * d_i
                stats.disc_acc_tokens += out.disc_accuracy.float() * d_i
                stats.disc_pos += out.disc_positive_count.float()
            if run_disc and self.overlap:
                main = torch.cuda.current_stream(dev)
                self._side.wait_stream(main)  # gradients are final, the generator's update has been queued
                for t in (guard, norms["generator"], device_gate):
                    if isinstance(t, torch.Tensor):
                        t.record_stream(self._side)
                with torch.cuda.stream(self._side), nvtx_range("discriminator optimizer (side stream)"):
                    norms["discriminator"] = self._finish_optimizer("discriminator", guard, upstream=norms["generator"],
                                                                    gate=device_gate)
                    eng.zero_grad("discriminator")
                    self._pending = _PendingOutcome(self.global_step + 1, norms, False, gate=device_gate)
                    self._disc_done = torch.cuda.Event()
                    self._disc_done.record(self._side)
                norms["discriminator"].record_stream(main)
            elif run_disc:
                with nvtx_range("discriminator optimizer"):
                    norms["discriminator"] = self._finish_optimizer("discriminator", guard, upstream=norms["generator"],
                                                                    gate=device_gate)
                eng.zero_grad("discriminator")
        else:
            guard = zero()
            for b, (g_i, d_i) in zip(batches, counts):
                b = self._to_device(b)
                out = model(input_ids=b["input_ids"], attention_mask=self._mask_of(b), labels=b["labels"],
                            token_type_ids=b.get("token_type_ids"), sampling_temperature=self.temperature,
                            gen_loss_weight=self.gen_w, disc_loss_weight=self.disc_w, masked_idx=b.get("masked_idx"))
                if self.token_weighted:
                    obj = self.gen_w * (g_i / gen_den) * out.gen_loss_raw + self.disc_w * (d_i / disc_den) * out.disc_loss_raw
                else:
                    obj = out.loss
                (obj * scale).backward()
                guard = guard + obj.detach().float()
                stats.gen_loss_tokens += out.gen_loss.float() * g_i
                stats.disc_loss_tokens += out.disc_loss.float() * d_i
                stats.disc_acc_tokens += out.disc_accuracy.float() * d_i
                stats.disc_pos += out.disc_positive_count.float()
            norms["all"] = self._finish_optimizer("all", guard)
            model.sync_discriminator_embeddings_from_generator()
            eng.zero_grad()
        if self._disc_done is not None:  # values the caller may read on the main stream
            with torch.cuda.stream(self._side):
                stats.grad_norms = {k: v.sqrt() for k, v in norms.items()}
            for v in stats.grad_norms.values():
                v.record_stream(torch.cuda.current_stream(dev))
        else:
            stats.grad_norms = {k: v.sqrt() for k, v in norms.items()}
        self.global_step += 1
        self.consumed_micro_batches += len(batches)
        if self._pending is None:
            self._pending = _PendingOutcome(self.global_step, norms, self.synchronous,
                                            gate=device_gate if self.decoupled else None)
        if self.synchronous:
            self.resolve_pending()
        return stats

    # ---- state ----------------------------------------------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        """Host-side training state. Call ``resolve_pending()`` on every rank first (``save_training_state`` does)."""
        self.wait_for_side_stream()
        self.resolve_pending()
        from deberta_b200.ops import heads_cuda

        return {"global_step": self.global_step, "lr_mult": self.lr_mult, "skip_streak": self.skip_streak,
                "consumed_micro_batches": self.consumed_micro_batches,
                "sampler_calls": int(heads_cuda._SEED_STATE["counter"]),  # position of the fused sampler's noise stream
                "schedules": {n: s.state_dict() for n, s in self.schedules.items()}}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.global_step = int(state["global_step"])
        self.lr_mult = float(state.get("lr_mult", 1.0))
        self.skip_streak = int(state.get("skip_streak", 0))
        self.consumed_micro_batches = int(state.get("consumed_micro_batches", 0))
        if "sampler_calls" in state:
            from deberta_b200.ops import heads_cuda

            heads_cuda._SEED_STATE["counter"] = int(state["sampler_calls"])
        for n, s in self.schedules.items():
            if n in state.get("schedules", {}):
                s.load_state_dict(state["schedules"][n])
