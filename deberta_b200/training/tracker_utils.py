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

    def set_summary(self, values: dict[str, Any]) -> None:
        """Run-level facts (crash marker, final step): W&B summary entries; TensorBoard gets them as text."""
        if self.wandb_run is not None:
            for k, v in values.items():
                try:
                    self.wandb_run.summary[k] = v
                except Exception:  # noqa: BLE001
                    pass
        if self.tb is not None:
            try:
                self.tb.add_text("summary", ", ".join(f"{k}={v}" for k, v in values.items()), max(self._last_step, 0))
            except Exception:  # noqa: BLE001
                pass

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


def _unique_existing(paths: list[Path | None]) -> list[Path]:
    seen: set[str] = set()
    out: list[Path] = []
    for p in paths:
        if p is None:
            continue
        p = Path(p).expanduser()
        try:
            key = str(p.resolve())
        except OSError:
            key = str(p)
        if key in seen:
            continue
        seen.add(key)
        if p.is_file():
            out.append(p)
        else:
            logger.warning("W&B config upload skipped missing file: %s", p)
    return out


def upload_wandb_config_files(*, tracker: TrackerSet, logging_dir: Path | None = None, files: list[Path] | None = None,
                              config_source_path: str | Path | None = None, run_name: str | None = None) -> bool:
    """Attach the run's configuration to the W&B run; True when at least one route took the files.

    Files: ``config_resolved.yaml`` of the logging directory, then the config file the user passed (or, when that is
    gone, the ``config_original.yaml`` snapshot), plus any explicit ``files``. Routes, in order
    (``tracker_utils.py:124-244`` of the reference): ``run.save`` per file, the module-level ``wandb.save``, an
    artifact of type ``config``.
    """
    run = tracker.wandb_run
    if run is None:
        return False
    wanted: list[Path | None] = list(files or [])
    if logging_dir is not None:
        wanted.append(Path(logging_dir) / "config_resolved.yaml")
        source = Path(str(config_source_path)).expanduser() if config_source_path else None
        wanted.append(source if source is not None and source.is_file() else Path(logging_dir) / "config_original.yaml")
    todo = _unique_existing(wanted)
    if not todo:
        return False
    module_save = None
    try:
        import wandb

        if getattr(wandb, "run", None) is not None and callable(getattr(wandb, "save", None)):
            module_save = wandb.save
    except Exception:  # noqa: BLE001
        wandb = None  # type: ignore[assignment]
    for save_fn, label in ((getattr(run, "save", None), "run.save"), (module_save, "wandb.save")):
        if not callable(save_fn):
            continue
        sent = 0
        for f in todo:
            try:
                try:
                    save_fn(str(f), base_path=str(f.parent), policy="now")
                except TypeError:  # older clients take the path only
                    save_fn(str(f))
                sent += 1
            except Exception as e:  # noqa: BLE001
                logger.warning("W&B %s failed for %s: %s", label, f, e)
        if sent:
            logger.info("Uploaded %d config file(s) to W&B through %s.", sent, label)
            return True
    log_artifact = getattr(run, "log_artifact", None)
    if callable(log_artifact) and wandb is not None:
        try:
            label = "".join(c if c.isalnum() or c in "-_." else "-" for c in str(run_name or "run")) or "run"
            art = wandb.Artifact(name=f"config-{label}", type="config", metadata={"files": [str(f) for f in todo]})
            for f in todo:
                art.add_file(str(f), name=f.name)
            log_artifact(art)
            logger.info("Uploaded the config files to W&B as artifact config-%s.", label)
            return True
        except Exception as e:  # noqa: BLE001
            logger.warning("W&B artifact upload failed: %s", e)
    logger.warning("The W&B run offers neither save() nor log_artifact(); config files were not uploaded.")
    return False
