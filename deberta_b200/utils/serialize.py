"""Dataclass ↔ plain-mapping conversion for snapshots (``utils/serialize.py`` of the reference)."""

from __future__ import annotations

import dataclasses
from typing import Any, get_type_hints

from .types import coerce_scalar, unwrap_optional_type


def asdict_without_private(obj: Any) -> dict[str, Any]:
    """``dataclasses.asdict`` minus keys starting with ``_`` (recursively)."""
    def strip(v: Any) -> Any:
        if isinstance(v, dict):
            return {k: strip(x) for k, x in v.items() if not str(k).startswith("_")}
        if isinstance(v, (list, tuple)):
            return [strip(x) for x in v]
        return v

    return strip(dataclasses.asdict(obj))


def mapping_from_config_obj(obj: Any) -> dict[str, Any]:
    """Mapping view of a dataclass, mapping, or attribute bag."""
    if obj is None:
        return {}
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return asdict_without_private(obj)
    if isinstance(obj, dict):
        return dict(obj)
    return {k: v for k, v in vars(obj).items() if not k.startswith("_")}


def drop_none_recursive(value: Any) -> Any:
    """Remove ``None`` leaves (and mappings that become empty) from nested mappings."""
    if isinstance(value, dict):
        out = {}
        for k, v in value.items():
            w = drop_none_recursive(v)
            if w is None or (isinstance(w, dict) and not w and isinstance(v, dict)):
                continue
            out[k] = w
        return out
    if isinstance(value, list):
        return [drop_none_recursive(v) for v in value if v is not None]
    return value


def coerce_dataclass_payload_types(cls: type, payload: dict[str, Any]) -> dict[str, Any]:
    """Coerce the scalar leaves of ``payload`` to the annotated field types of dataclass ``cls``."""
    hints = get_type_hints(cls)
    out: dict[str, Any] = {}
    for key, value in payload.items():
        tp = hints.get(key)
        target, _ = unwrap_optional_type(tp) if tp is not None else (None, False)
        if target is not None and dataclasses.is_dataclass(target) and isinstance(value, dict):
            out[key] = coerce_dataclass_payload_types(target, value)
        elif tp is not None and not isinstance(value, (dict, list)):
            out[key] = coerce_scalar(value, tp)
        else:
            out[key] = value
    return out
