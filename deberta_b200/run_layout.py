"""File names inside a run directory and helpers to locate them (``run_layout.py`` of the reference)."""

from __future__ import annotations

from pathlib import Path

from deberta_b200.config import validate_run_metadata_schema
from deberta_b200.utils.io import load_json_mapping

MODEL_CONFIG_FILE = "model_config.json"
DATA_CONFIG_FILE = "data_config.json"
TRAIN_CONFIG_FILE = "train_config.json"
OPTIM_CONFIG_FILE = "optim_config.json"
LOGGING_CONFIG_FILE = "logging_config.json"
RUN_METADATA_FILE = "run_metadata.json"
RESUME_SOURCE_FILE = "resume_source.json"
CONFIG_ORIGINAL_FILE = "config_original.yaml"
CONFIG_RESOLVED_FILE = "config_resolved.yaml"
DATA_STATE_FILE = "data_state.json"
COMPLETE_MARKER_FILE = ".complete"
CHECKPOINT_PREFIX = "checkpoint-"
FINAL_HF_DIR = "final_hf"


def infer_run_dir_from_checkpoint(checkpoint_dir: str | Path) -> Path:
    """A checkpoint lives directly inside its run directory."""
    return Path(checkpoint_dir).expanduser().resolve().parent


def validate_run_metadata_file(run_dir: str | Path) -> dict:
    """Load ``run_metadata.json`` of a run directory and check its schema version."""
    path = Path(run_dir) / RUN_METADATA_FILE
    if not path.exists():
        raise ValueError(f"Missing {RUN_METADATA_FILE} in {run_dir}; cannot verify the config schema of this run.")
    raw = load_json_mapping(path)
    validate_run_metadata_schema(raw, source=str(path))
    return raw
