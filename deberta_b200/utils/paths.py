"""Output-directory checks."""

from __future__ import annotations

from pathlib import Path


def validate_existing_output_dir(path: str | Path, *, overwrite: bool, resuming: bool, what: str = "output_dir") -> None:
    """Refuse a non-empty directory unless overwriting or resuming."""
    p = Path(path)
    if not p.exists():
        return
    if not p.is_dir():
        raise ValueError(f"{what} exists and is not a directory: {p}")
    if any(p.iterdir()) and not (overwrite or resuming):
        raise ValueError(
            f"{what} already exists and is not empty: {p}. Set train.checkpoint.overwrite_output_dir=true "
            "or resume with train.checkpoint.resume_from_checkpoint."
        )
