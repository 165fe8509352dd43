"""Activation lookup (``activations.py:8-21`` of the reference resolves names through HF ``ACT2FN``)."""

from __future__ import annotations

from collections.abc import Callable

import torch


def get_act_fn(name: str | Callable) -> Callable[[torch.Tensor], torch.Tensor]:
    """Resolve an activation by its Hugging Face name (``gelu`` is the exact erf form)."""
    if callable(name):
        return name
    from transformers.activations import ACT2FN

    key = str(name).strip().lower()
    if key not in ACT2FN:
        raise ValueError(f"Unsupported activation {name!r}. Supported: {sorted(ACT2FN.keys())}")
    return ACT2FN[key]
