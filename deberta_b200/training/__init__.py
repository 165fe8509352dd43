"""Training runtime: loop, checkpoints, metrics."""

from .entrypoint import run_pretraining, run_pretraining_dry_run
from .trainer import Trainer

__all__ = ["run_pretraining", "run_pretraining_dry_run", "Trainer"]
