"""Optional NVTX ranges around the phases of a training step (``logging.debug.nvtx: true``).

The reference has no tracing hooks; these ranges make the generator / discriminator / optimizer phases visible
in a timeline profiler without touching the kernels. Disabled (the default) they cost one attribute lookup.
"""

from __future__ import annotations

import contextlib

import torch

__all__ = ["nvtx_range", "nvtx_enabled", "set_nvtx"]

_ENABLED = False


def set_nvtx(enabled: bool) -> None:
    """Switch the ranges on or off for this process (needs a CUDA build of torch to have any effect)."""
    global _ENABLED
    _ENABLED = bool(enabled) and torch.cuda.is_available()


def nvtx_enabled() -> bool:
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
