"""Model zoo: the two backbones (disentangled-attention DeBERTa-v2 and the RoPE encoder), the RTD pretraining
wrapper around a generator/discriminator pair, and the builder that turns a config into both.

Names below are loaded lazily from their submodules.
"""

from __future__ import annotations

import importlib
from typing import Any

# public name -> submodule that defines it; resolved on first access so that importing the package stays cheap
_EXPORTS: dict[str, str] = {
    "DebertaV2Config": "deberta_v2",
    "DebertaV2Model": "deberta_v2",
    "DebertaRoPEConfig": "rope_encoder",
    "DebertaRoPEModel": "rope_encoder",
    "DebertaV3RTDPretrainer": "rtd",
    "build_backbone_configs": "builder",
    "build_backbones": "builder",
    "AttnMask": "mask_utils",
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
