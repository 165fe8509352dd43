"""Optional NVTX ranges around the phases of a training step (``DEBERTA_NVTX=1``).

The reference has no tracing hooks; these ranges make the generator / discriminator / optimizer phases visible
in a timeline profiler without touching the kernels. Disabled (the default) they cost one attribute lookup.
"""

from __future__ import annotations

import contextlib
import os

import torch

__all__ = ["nvtx_range", "nvtx_enabled"]

_ENABLED: bool | None = None


def nvtx_enabled() -> bool:
    global _ENABLED
    if _ENABLED is None:
        _ENABLED = os.environ.get("DEBERTA_NVTX", "0").strip().lower() in ("1", "true", "yes", "on") and torch.cuda.is_available()
    return _ENABLED


@contextlib.contextmanager
def nvtx_range(name: str):
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
