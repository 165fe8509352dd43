"""Input pipeline: where documents come from (``loading``, ``synthetic``), how they become fixed-length token blocks
(``streaming``) and how blocks become masked training batches (``collator``). Names below are loaded lazily.
"""

from __future__ import annotations

import importlib
from typing import Any

# public name -> submodule that defines it; resolved on first access so that importing the package stays cheap
_EXPORTS: dict[str, str] = {
    "load_hf_dataset": "loading",
    "PackedStreamingConfig": "streaming",
    "PackedStreamingDataset": "streaming",
    "SequentialStreamingDataset": "streaming",
    "DebertaV3ElectraCollator": "collator",
    "MLMConfig": "collator",
    "SyntheticTextDataset": "synthetic",
    "SyntheticTokenizer": "synthetic",
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
