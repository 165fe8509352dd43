"""Scalar coercion used by the CLI flags and dotted overrides (``utils/types.py`` of the reference)."""

from __future__ import annotations

import types
from typing import Any, Union, get_args, get_origin

_TRUE = {"1", "true", "t", "yes", "y", "on"}
_FALSE = {"0", "false", "f", "no", "n", "off"}


def parse_bool(value: Any, *, allow_numeric: bool = True) -> bool:
    """Parse ``true/false/yes/no/on/off`` (and optionally ``1/0``); real bools pass through."""
    if isinstance(value, bool):
        return value
    if isinstance(value, (int, float)) and allow_numeric and value in (0, 1):
        return bool(value)
    text = str(value).strip().lower()
    if not allow_numeric and text in {"0", "1"}:
        raise ValueError(f"Expected a boolean (true/false), got: {value!r}")
    if text in _TRUE:
        return True
    if text in _FALSE:
        return False
    raise ValueError(f"Expected a boolean (true/false), got: {value!r}")


def unwrap_optional_type(tp: Any) -> tuple[Any, bool]:
    """``int | None`` → ``(int, True)``; ``int`` → ``(int, False)``."""
    origin = get_origin(tp)
    if origin in (Union, types.UnionType):
        args = [a for a in get_args(tp) if a is not type(None)]
        allows_none = len(args) != len(get_args(tp))
        if len(args) == 1:
            return args[0], allows_none
        return tp, allows_none
    return tp, False


def coerce_scalar(raw: Any, field_type: Any, *, allow_none: bool = True, allow_bool_numeric: bool = True) -> Any:
    """Cast a raw (usually string) value to the annotated scalar type.

    ``none``/``null`` map to ``None`` for optional fields when ``allow_none`` is set.
    """
    target, optional = unwrap_optional_type(field_type)
    if isinstance(raw, str) and optional and raw.strip().lower() in {"none", "null"}:
        if allow_none or optional:
            return None
    if raw is None:
        if optional:
            return None
        raise ValueError("null is not allowed for this field")
    if target is bool:
        return parse_bool(raw, allow_numeric=allow_bool_numeric)
    if target is int:
        if isinstance(raw, bool):
            raise ValueError(f"Expected an integer, got bool: {raw!r}")
        return int(str(raw).strip()) if isinstance(raw, str) else int(raw)
    if target is float:
        if isinstance(raw, bool):
            raise ValueError(f"Expected a number, got bool: {raw!r}")
        return float(str(raw).strip()) if isinstance(raw, str) else float(raw)
    if target is str:
        return str(raw)
    return raw
