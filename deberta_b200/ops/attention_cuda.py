"""Dispatch predicates and launchers for the sm_100a attention kernels."""

from __future__ import annotations

import torch


def disentangled_supported(q, k, v, pos_k, pos_q, heads, pair_keep, dropout_p, training, rel_pos) -> bool:
    return False


def rope_supported(q, k, v, heads, rotary_dim, pair_keep, dropout_p, training) -> bool:
    return False


def disentangled_attention_cuda(*args, **kwargs) -> torch.Tensor:  # pragma: no cover
    raise NotImplementedError


def rope_attention_cuda(*args, **kwargs) -> torch.Tensor:  # pragma: no cover
    raise NotImplementedError
