"""Experiment trackers: TensorBoard and Weights & Biases, both optional (``training/tracker_utils.py`` of the reference)."""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

logger = logging.getLogger(__name__)


class TrackerSet:
    """Fan-out of ``log(values, step)`` to the configured backends with a monotone step guard."""

    def __init__(self) -> None:
        self.tb = None
        self.wandb_run = None
        self._last_step = -1

    def log(self, values: dict[str, Any], step: int) -> None:
        if step < self._last_step:
            return  # trackers reject steps that go backwards (e.g. crash rows after a resume)
        self._last_step = step
        if self.tb is not None:
            for k, v in values.items():
                if isinstance(v, (int, float)):
                    self.tb.add_scalar(k, v, step)
        if self.wandb_run is not None:
            self.wandb_run.log(values, step=step)

    def finish(self, *, crashed: bool = False) -> None:
        if self.tb is not None:
            self.tb.flush()
            self.tb.close()
        if self.wandb_run is not None:
            if crashed:
                try:
                    self.wandb_run.summary["crashed"] = True
                except Exception:
                    pass
            self.wandb_run.finish(exit_code=1 if crashed else 0)


def init_trackers(*, logging_cfg: Any, logging_dir: Path, run_name: str | None, config_payload: dict[str, Any],
                  is_main_process: bool) -> TrackerSet:
    """Create the trackers named by ``logging.backend`` / ``logging.wandb.enabled`` on the main process."""
    ts = TrackerSet()
    if not is_main_process:
        return ts
    if str(logging_cfg.backend).lower() == "tensorboard":
        try:
            from torch.utils.tensorboard import SummaryWriter

            ts.tb = SummaryWriter(log_dir=str(Path(logging_dir) / "tensorboard"))
        except Exception as e:  # tensorboard is optional
            logger.warning("logging.backend=tensorboard requested but TensorBoard is unavailable: %s", e)
    if bool(logging_cfg.wandb.enabled):
        try:
            import wandb

            ts.wandb_run = wandb.init(project=str(logging_cfg.project_name), name=run_name, config=config_payload,
                                      dir=str(logging_dir))
        except Exception as e:
            logger.warning("logging.wandb.enabled=true but wandb could not be initialised: %s", e)
    return ts


def setup_wandb_watch(*, tracker: TrackerSet, model: Any, watch_mode: str, log_freq: int) -> bool:
    """``wandb.watch`` gradients/parameters/all when W&B is active."""
    mode = str(watch_mode).strip().lower()
    if tracker.wandb_run is None or mode == "none":
        return False
    try:
        import wandb

        wandb.watch(model, log=mode, log_freq=int(log_freq))
        return True
    except Exception as e:
        logger.warning("wandb.watch failed: %s", e)
        return False


def upload_wandb_config_files(*, tracker: TrackerSet, files: list[Path]) -> int:
    """Attach the config snapshots to the W&B run (``run.save`` per file)."""
    n = 0
    if tracker.wandb_run is None:
        return n
    for f in files:
        try:
            if Path(f).exists():
                tracker.wandb_run.save(str(f), policy="now")
                n += 1
        except Exception as e:
            logger.warning("Failed to upload %s to W&B: %s", f, e)
    return n
