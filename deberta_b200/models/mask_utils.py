"""Attention-mask normalisation.

Masks are *keep* masks (True/non-zero = attend). Floating-point masks are rejected:
additive masks would silently be misread as keep masks (``mask_utils.py:8-32`` of the
reference has the same contract). ``AttnMask`` condenses whatever layout the caller
passed into the compact description the attention operators consume.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

__all__ = ["normalize_keep_mask", "AttnMask"]


def normalize_keep_mask(mask: torch.Tensor, *, name: str = "attention_mask") -> torch.Tensor:
    """Return ``mask`` as a bool keep-mask; only bool and integer dtypes are accepted."""
    if mask.dtype == torch.bool:
        return mask
    if mask.is_floating_point() or mask.is_complex():
        raise ValueError(
            f"{name} must be a bool or integer keep-mask (1 = attend, 0 = masked); "
            f"floating-point (additive) masks are not supported, got dtype={mask.dtype}."
        )
    return mask.ne(0)


@dataclass
class AttnMask:
    """Compact mask: exactly one of the fields is set (or none for "attend everywhere")."""

    key_keep: torch.Tensor | None = None  # [B,S] bool
    doc_ids: torch.Tensor | None = None  # [B,S] int, 0 = inactive
    pair_keep: torch.Tensor | None = None  # [B,S,S] bool

    @property
    def is_pairwise(self) -> bool:
        return self.doc_ids is not None or self.pair_keep is not None

    def token_keep(self) -> torch.Tensor | None:
        """[B,S] bool activity of each position (None when everything is active)."""
        if self.key_keep is not None:
            return self.key_keep
        if self.doc_ids is not None:
            return self.doc_ids.ne(0)
        if self.pair_keep is not None:
            return torch.diagonal(self.pair_keep, dim1=-2, dim2=-1)
        return None

    def kwargs(self) -> dict:
        return {"key_keep": self.key_keep, "doc_ids": self.doc_ids, "pair_keep": self.pair_keep}

    @classmethod
    def from_any(cls, attention_mask: torch.Tensor | None, doc_ids: torch.Tensor | None = None) -> "AttnMask":
        """Build from ``None``, (B,S), (B,S,S), (B,1|H,1|S,S) keep masks or packed ``doc_ids``."""
        if doc_ids is not None:
            return cls(doc_ids=doc_ids)
        if attention_mask is None:
            return cls()
        if isinstance(attention_mask, AttnMask):
            return attention_mask
        m = normalize_keep_mask(attention_mask)
        if m.ndim == 4:
            m = m[:, 0] if m.shape[1] == 1 else m.any(dim=1)
        if m.ndim == 3:
            if m.shape[-2] == 1:
                m = m[:, 0, :]
            else:
                return cls(pair_keep=m)
        if m.ndim != 2:
            raise ValueError(f"attention_mask must be rank-2/3/4; got rank={attention_mask.ndim}")
        return cls(key_keep=m)
