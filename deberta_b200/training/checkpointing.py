"""Resume policy and periodic-save helpers (``training/checkpointing.py`` of the reference)."""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

from .run_management import save_training_checkpoint

logger = logging.getLogger(__name__)


def resolve_data_resume_policy(*, train_cfg: Any, consumed_micro_batches: int, global_step: int) -> tuple[bool, int, str]:
    """(replay the data iterator?, first epoch, reason) for a resume.

    ``replay`` re-iterates exactly the consumed micro-batches; ``restart_epoch`` starts a fresh
    epoch seeded by ``global_step``; ``auto`` replays unless that exceeds
    ``resume_replay_max_micro_batches``.
    """
    strategy = str(getattr(train_cfg, "resume_data_strategy", "auto")).strip().lower()
    limit = int(getattr(train_cfg, "resume_replay_max_micro_batches", 10_000))
    consumed = int(max(0, consumed_micro_batches))
    if strategy == "replay":
        return True, 0, "resume_data_strategy=replay"
    if strategy == "restart_epoch":
        return False, int(global_step), "resume_data_strategy=restart_epoch"
    if consumed <= limit:
        return True, 0, f"auto: replaying {consumed} micro-batches (<= {limit})"
    return False, int(global_step), f"auto: {consumed} micro-batches exceed replay limit {limit}; restarting data epoch"


def normalize_resume_consumed_micro_batches(*, consumed_micro_batches: int, global_step: int, ga_steps: int) -> int:
    """Clamp the stored data position to an optimizer-step boundary (a partial window is never resumed into)."""
    boundary = int(global_step) * int(max(1, ga_steps))
    consumed = int(max(0, consumed_micro_batches))
    if consumed != boundary:
        logger.warning("Checkpoint data position %d is not at an optimizer-step boundary (%d); using the boundary.",
                       consumed, boundary)
    return boundary


def checkpoint_is_due(*, global_step: int, save_steps: int, last_saved_step: int) -> bool:
    """True when ``global_step`` is a multiple of ``save_steps`` that has not been saved yet."""
    return bool(save_steps) and int(save_steps) > 0 and global_step % int(save_steps) == 0 and last_saved_step != global_step


def save_periodic_checkpoint_if_due(*, ctx: Any, save_state, output_dir: Path, global_step: int, save_steps: int,
                                    last_saved_step: int, **kw: Any) -> int:
    """Save ``checkpoint-<step>`` when ``global_step`` hits a multiple of ``save_steps``; returns the last saved step."""
    if not checkpoint_is_due(global_step=global_step, save_steps=save_steps, last_saved_step=last_saved_step):
        return last_saved_step
    save_training_checkpoint(ctx=ctx, save_state=save_state, checkpoint_dir=Path(output_dir) / f"checkpoint-{global_step}",
                             output_dir=Path(output_dir), log_label="periodic", global_step=global_step, **kw)
    return int(global_step)
