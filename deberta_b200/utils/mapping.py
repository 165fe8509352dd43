"""Nested-mapping helpers."""

from __future__ import annotations

from typing import Any


def flatten_mapping(mapping: dict[str, Any], *, prefix: str = "") -> dict[str, Any]:
    """``{"a": {"b": 1}}`` → ``{"a.b": 1}``."""
    out: dict[str, Any] = {}
    for key, value in mapping.items():
        path = f"{prefix}.{key}" if prefix else str(key)
        if isinstance(value, dict):
            out.update(flatten_mapping(value, prefix=path))
        else:
            out[path] = value
    return out


def leaf_paths(value: Any, *, prefix: str = "") -> set[str]:
    """Dotted paths of every non-mapping leaf in a nested mapping."""
    if isinstance(value, dict):
        out: set[str] = set()
        for k, v in value.items():
            out |= leaf_paths(v, prefix=f"{prefix}.{k}" if prefix else str(k))
        return out
    return {prefix} if prefix else set()
