"""Atomic JSON writes and strict JSON-mapping reads."""

from __future__ import annotations

import json
import os
import tempfile
from pathlib import Path
from typing import Any


def dump_json(payload: Any, path: str | Path, *, indent: int = 2, sort_keys: bool = True) -> None:
    """Write JSON via temp file + fsync + ``os.replace`` so readers never see a partial file."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=f".{path.name}.", suffix=".tmp", dir=str(path.parent))
    try:
        with os.fdopen(fd, "w", encoding="utf-8") as f:
            json.dump(payload, f, indent=indent, sort_keys=sort_keys)
            f.write("\n")
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise


def load_json_mapping(path: str | Path) -> dict[str, Any]:
    """Read a JSON file that must contain an object."""
    raw = json.loads(Path(path).read_text(encoding="utf-8"))
    if not isinstance(raw, dict):
        raise ValueError(f"Expected a JSON object in {path}, got {type(raw).__name__}.")
    return raw
