"""Weight initialisation that cooperates with ``PreTrainedModel.from_pretrained``.

transformers (v5) re-runs ``_init_weights`` over the whole module tree after loading a checkpoint
and expects already-loaded tensors (flagged ``_is_hf_initialized``) to be left alone.
"""

from __future__ import annotations

import torch
from torch import nn


def _fresh(t: torch.Tensor) -> bool:
    return not getattr(t, "_is_hf_initialized", False)


def init_linear_(module: nn.Linear, std: float) -> None:
    if _fresh(module.weight):
        module.weight.data.normal_(mean=0.0, std=std)
    if module.bias is not None and _fresh(module.bias):
        module.bias.data.zero_()


def init_embedding_(module: nn.Embedding, std: float) -> None:
    if _fresh(module.weight):
        module.weight.data.normal_(mean=0.0, std=std)
        if module.padding_idx is not None:
            module.weight.data[module.padding_idx].zero_()


def init_norm_(weight: torch.Tensor | None, bias: torch.Tensor | None = None) -> None:
    if weight is not None and _fresh(weight):
        weight.data.fill_(1.0)
    if bias is not None and _fresh(bias):
        bias.data.zero_()
