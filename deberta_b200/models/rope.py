"""Rotary position embeddings: frequency table and cos/sin cache (``rope.py`` of the reference).

Pairing is interleaved (features 2i and 2i+1 rotate together) and ``inv_freq_i =
theta^(-2i/full_dim)`` so partial rotary (``rotary_pct < 1``) keeps the full-head spacing.
The rotation itself happens inside the attention operator.
"""

from __future__ import annotations

import torch
from torch import nn

from deberta_b200.ops.attention import rotate_interleaved

__all__ = ["RotaryEmbedding"]


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, base: float = 10000.0, full_dim: int | None = None) -> None:
        super().__init__()
        self.dim = int(dim)
        if self.dim % 2:
            raise ValueError(f"Rotary dim must be even, got {self.dim}")
        self.base = float(base)
        self.denom = float(full_dim if full_dim is not None else self.dim)
        self.register_buffer("inv_freq", self._inv_freq(), persistent=False)
        self._cache: tuple[torch.Tensor, torch.Tensor] | None = None
        self._key: tuple | None = None

    def _inv_freq(self) -> torch.Tensor:
        return 1.0 / (self.base ** (torch.arange(0, self.dim, 2).float() / self.denom))

    def reset_buffers(self) -> None:
        """Recompute the frequency table in place and drop the cos/sin cache.

        The table is a non-persistent buffer: no checkpoint stores it, so a model that was
        materialised from the meta device (``from_pretrained``) has to write it again.
        """
        self.inv_freq.data.copy_(self._inv_freq().to(self.inv_freq.device))
        self._cache, self._key = None, None

    def _build(self, seq_len: int, device, dtype):
        t = torch.arange(seq_len, device=device, dtype=self.inv_freq.dtype)
        freqs = torch.outer(t, self.inv_freq.to(device))
        emb = torch.repeat_interleave(freqs, 2, dim=-1)  # [f0, f0, f1, f1, ...]
        return emb.cos().to(dtype), emb.sin().to(dtype)

    def prefill_cache(self, seq_len: int, *, device, dtype) -> None:
        """Build the table once for the longest sequence so later calls only slice it."""
        if int(seq_len) <= 0:
            raise ValueError(f"seq_len must be > 0 for rotary cache prefill, got {seq_len}.")
        self._cache = self._build(int(seq_len), device, dtype)
        self._key = (torch.device(device), dtype)

    def get_cos_sin(self, seq_len: int, *, device, dtype) -> tuple[torch.Tensor, torch.Tensor]:
        key = (torch.device(device), dtype)
        if self._cache is None or self._key != key or self._cache[0].shape[0] < seq_len:
            self.prefill_cache(seq_len, device=device, dtype=dtype)
        return self._cache[0][:seq_len], self._cache[1][:seq_len]

    def apply(self, q: torch.Tensor, k: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Rotate ``[B,h,S,d]`` queries and keys (eager helper; the fused operator does this in-kernel)."""
        cos, sin = self.get_cos_sin(q.shape[-2], device=q.device, dtype=q.dtype)
        return (rotate_interleaved(q, cos[None, None], sin[None, None], self.dim),
                rotate_interleaved(k, cos[None, None], sin[None, None], self.dim))
