"""Metric sinks: ``metrics.jsonl.gz`` rows and non-finite debug artifacts (``training/metrics.py`` of the reference)."""

from __future__ import annotations

import gzip
import json
import logging
import time
from pathlib import Path
from typing import Any

import torch

from deberta_b200.utils.io import dump_json

logger = logging.getLogger(__name__)


def append_metrics_jsonl_row(path: Path, row: dict[str, Any]) -> None:
    """Append one JSON row to a gzip member stream (readable with ``gzip.open`` as concatenated members)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with gzip.open(path, "at", encoding="utf-8") as f:
        f.write(json.dumps(row, sort_keys=True, default=float) + "\n")


def flush_loggers() -> None:
    for handler in logging.getLogger().handlers:
        try:
            handler.flush()
        except Exception:
            pass


def _rng_heads() -> dict[str, Any]:
    out: dict[str, Any] = {"torch_cpu": torch.get_rng_state()[:8].tolist()}
    if torch.cuda.is_available():
        try:
            out["torch_cuda"] = torch.cuda.get_rng_state()[:8].tolist()
        except Exception:
            pass
    return out


def write_nonfinite_debug_artifact(*, debug_dir: Path, step: int, what: str, losses: dict[str, float],
                                   lrs: dict[str, float], lr_mult: float, extra: dict[str, Any] | None = None) -> Path:
    """``debug/nonfinite_step_<n>_<what>.json`` with the losses, learning rates and RNG heads at the failure."""
    path = Path(debug_dir) / f"nonfinite_step_{int(step)}_{what}.json"
    payload = {"step": int(step), "what": str(what), "time": time.time(), "losses": losses, "lrs": lrs,
               "lr_mult": float(lr_mult), "rng": _rng_heads(), **(extra or {})}
    dump_json(payload, path)
    return path
