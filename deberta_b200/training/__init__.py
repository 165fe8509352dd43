"""Training runtime of the framework.

The optimizer-step logic lives in ``trainer``, run orchestration (resume, logging, checkpoints, export hook) in
``entrypoint``; the remaining modules are helpers of those two. Names below are loaded lazily.
"""

from __future__ import annotations

import importlib
from typing import Any

# public name -> submodule that defines it; resolved on first access so that importing the package stays cheap
_EXPORTS: dict[str, str] = {
    "Trainer": "trainer",
    "WindowStats": "trainer",
    "run_pretraining": "entrypoint",
    "run_pretraining_dry_run": "entrypoint",
    "StepWatchdog": "watchdog",
    "RankHeartbeat": "watchdog",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str) -> Any:
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(f"{__name__}.{target}"), name)
    globals()[name] = value
    return value


def __dir__() -> list[str]:
    return sorted(set(globals()) | set(_EXPORTS))
