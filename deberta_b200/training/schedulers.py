"""Learning-rate schedules as pure functions of the step (same shapes as ``transformers.get_scheduler``)."""

from __future__ import annotations

import math
from collections.abc import Callable

SCHEDULER_TYPES = ("linear", "cosine", "cosine_with_restarts", "polynomial", "constant", "constant_with_warmup")


def make_lr_lambda(kind: str, *, warmup_steps: int, total_steps: int, base_lr: float = 1.0) -> Callable[[int], float]:
    """Multiplier of the base LR after ``step`` optimizer steps."""
    kind = str(kind).strip().lower()
    w, t = int(warmup_steps), int(total_steps)
    if kind not in SCHEDULER_TYPES:
        raise ValueError(f"Unknown scheduler type {kind!r}; expected one of {', '.join(SCHEDULER_TYPES)}")

    def warm(step: int) -> float | None:
        return float(step) / float(max(1, w)) if step < w else None

    if kind == "constant":
        return lambda step: 1.0
    if kind == "constant_with_warmup":
        return lambda step: warm(step) if step < w else 1.0
    if kind == "linear":
        return lambda step: warm(step) if step < w else max(0.0, float(t - step) / float(max(1, t - w)))
    if kind == "cosine":
        def f(step: int) -> float:
            if step < w:
                return warm(step)
            prog = float(step - w) / float(max(1, t - w))
            return max(0.0, 0.5 * (1.0 + math.cos(math.pi * 2.0 * 0.5 * prog)))
        return f
    if kind == "cosine_with_restarts":
        def f(step: int) -> float:
            if step < w:
                return warm(step)
            prog = float(step - w) / float(max(1, t - w))
            return 0.0 if prog >= 1.0 else max(0.0, 0.5 * (1.0 + math.cos(math.pi * ((1.0 * prog) % 1.0))))
        return f
    # polynomial (power 1, lr_end 1e-7 as in transformers)
    lr_end, power = 1e-7, 1.0
    lr_init = float(base_lr)

    def f(step: int) -> float:
        if step < w:
            return warm(step)
        if step > t:
            return lr_end / lr_init
        remaining = 1 - (step - w) / max(1, t - w)
        return ((lr_init - lr_end) * remaining**power + lr_end) / lr_init
    return f


class StepSchedule:
    """Scheduler with ``step()`` / ``state_dict()`` over a pure schedule function."""

    def __init__(self, kind: str, *, warmup_steps: int, total_steps: int, base_lr: float) -> None:
        self.fn = make_lr_lambda(kind, warmup_steps=warmup_steps, total_steps=total_steps, base_lr=base_lr)
        self.base_lr = float(base_lr)
        self.last_step = 0

    def step(self) -> None:
        self.last_step += 1

    def step_back(self) -> None:
        """Undo one ``step()`` (an update that turned out not to have happened)."""
        self.last_step = max(0, self.last_step - 1)

    def scale(self) -> float:
        return float(self.fn(self.last_step))

    def get_last_lr(self) -> list[float]:
        return [self.base_lr * self.scale()]

    def state_dict(self) -> dict:
        return {"last_step": self.last_step}

    def load_state_dict(self, state: dict) -> None:
        self.last_step = int(state["last_step"])
