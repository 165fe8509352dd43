"""Run-directory config snapshots and resume compatibility checks (``training/run_config.py`` of the reference).

A run directory holds one JSON snapshot per config section plus ``run_metadata.json``
(schema version 4); the logging directory holds ``config_original.yaml`` (the source file,
verbatim) and ``config_resolved.yaml`` (effective values, ``None`` pruned). Resuming checks the
stored model/data/optim snapshots against the current config, ignoring fields that cannot
change the numerics of a resumed run.
"""

from __future__ import annotations

import logging
import shutil
from pathlib import Path
from typing import Any

from deberta_b200 import __version__
from deberta_b200.config import RUN_CONFIG_SCHEMA_VERSION, asdict_without_private, validate_run_metadata_schema
from deberta_b200.run_layout import (CONFIG_ORIGINAL_FILE, CONFIG_RESOLVED_FILE, DATA_CONFIG_FILE, LOGGING_CONFIG_FILE,
                                     MODEL_CONFIG_FILE, OPTIM_CONFIG_FILE, RESUME_SOURCE_FILE, RUN_METADATA_FILE,
                                     TRAIN_CONFIG_FILE, infer_run_dir_from_checkpoint)
from deberta_b200.utils.io import dump_json, load_json_mapping
from deberta_b200.utils.mapping import flatten_mapping
from deberta_b200.utils.serialize import drop_none_recursive

logger = logging.getLogger(__name__)

# fields that may differ between the original run and a resume without invalidating it
_INERT_FIELDS = {
    "train": {"max_steps", "checkpoint.output_dir", "checkpoint.overwrite_output_dir", "checkpoint.save_steps",
              "checkpoint.save_total_limit", "checkpoint.resume_from_checkpoint", "checkpoint.resume_data_strategy",
              "checkpoint.resume_replay_max_micro_batches", "checkpoint.export_hf_final", "dataloader.num_workers",
              "dataloader.pin_memory", "compile.enabled", "compile.mode", "compile.scope", "compile.backend", "tf32",
              "sdpa_kernel", "distributed.parallelism", "distributed.fused_collectives", "distributed.nvls", "distributed.overlap_backward",
              "distributed.comm_timeout_s", "distributed.step_deadline_s", "distributed.heartbeat_s"},
    "model": {"gradient_checkpointing", "hf.attention_kernel", "rope.attention_implementation"},
    "data": {"source.shuffle_buffer_size"},
    "optim": set(),
}


def build_run_metadata(*, effective_compile_scope: str | None = None, compile_scope_reason: str | None = None) -> dict[str, Any]:
    meta: dict[str, Any] = {"config_schema_version": int(RUN_CONFIG_SCHEMA_VERSION), "deberta_version": str(__version__)}
    if effective_compile_scope is not None:
        meta["effective_compile_scope"] = str(effective_compile_scope)
    if compile_scope_reason is not None:
        meta["compile_scope_reason"] = str(compile_scope_reason)
    return meta


def _dump_yaml(payload: dict[str, Any], path: Path) -> None:
    import yaml

    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(yaml.safe_dump(payload, sort_keys=False), encoding="utf-8")


def write_config_yaml_snapshots(*, logging_dir: Path, config_path: Path | None, sections: dict[str, Any]) -> None:
    """``config_original.yaml`` (copy of the user's file, or the defaults) and ``config_resolved.yaml``."""
    logging_dir = Path(logging_dir)
    logging_dir.mkdir(parents=True, exist_ok=True)
    resolved = drop_none_recursive({k: asdict_without_private(v) for k, v in sections.items()})
    if config_path is not None and Path(config_path).exists() and Path(config_path).suffix.lower() in {".yaml", ".yml"}:
        shutil.copyfile(config_path, logging_dir / CONFIG_ORIGINAL_FILE)
    elif config_path is not None and Path(config_path).exists():
        _dump_yaml(load_json_mapping(config_path), logging_dir / CONFIG_ORIGINAL_FILE)
    else:
        _dump_yaml(resolved, logging_dir / CONFIG_ORIGINAL_FILE)
    _dump_yaml(resolved, logging_dir / CONFIG_RESOLVED_FILE)


def write_runtime_resolved_config(*, logging_dir: Path, payload: dict[str, Any]) -> Path:
    """Replace ``config_resolved.yaml`` by the runtime-resolved payload (values only known once the model exists)."""
    path = Path(logging_dir) / CONFIG_RESOLVED_FILE
    _dump_yaml(payload, path)
    return path


def compare_resume_config(*, section: str, stored: dict[str, Any], current: dict[str, Any]) -> list[str]:
    """Dotted paths whose values differ in a way that matters for a resumed run."""
    a, b = flatten_mapping(stored), flatten_mapping(current)
    inert = _INERT_FIELDS.get(section, set())
    return sorted(k for k in set(a) | set(b) if k not in inert and a.get(k) != b.get(k))


def persist_or_validate_run_configs(*, output_dir: Path, logging_dir: Path, sections: dict[str, Any],
                                    config_path: Path | None, resume_checkpoint: str | None, is_main_process: bool,
                                    effective_compile_scope: str | None = None,
                                    compile_scope_reason: str | None = None) -> None:
    """Fresh run: write all snapshots. Resume: validate the stored snapshots first, record cross-run provenance."""
    output_dir = Path(output_dir)
    files = {"model": MODEL_CONFIG_FILE, "data": DATA_CONFIG_FILE, "train": TRAIN_CONFIG_FILE,
             "optim": OPTIM_CONFIG_FILE, "logging": LOGGING_CONFIG_FILE}
    current = {k: asdict_without_private(v) for k, v in sections.items()}
    if resume_checkpoint:
        src_dir = infer_run_dir_from_checkpoint(resume_checkpoint)
        meta_path = src_dir / RUN_METADATA_FILE
        if not meta_path.exists():
            raise ValueError(f"Cannot resume from {resume_checkpoint}: {RUN_METADATA_FILE} is missing in {src_dir}.")
        validate_run_metadata_schema(load_json_mapping(meta_path), source=str(meta_path))
        for name in ("model", "data", "train", "optim"):
            path = src_dir / files[name]
            if not path.exists():
                raise ValueError(f"Cannot resume from {resume_checkpoint}: {files[name]} is missing in {src_dir}.")
            diff = compare_resume_config(section=name, stored=load_json_mapping(path), current=current[name])
            if diff:
                raise ValueError(f"Resume config mismatch in {files[name]} for fields: {', '.join(diff)}. "
                                 "Resume with the original configuration or start a new run.")
        if is_main_process and src_dir.resolve() != output_dir.resolve():
            dump_json({"resume_checkpoint": str(Path(resume_checkpoint).resolve()), "source_run_dir": str(src_dir)},
                      output_dir / RESUME_SOURCE_FILE)
    if not is_main_process:
        return
    output_dir.mkdir(parents=True, exist_ok=True)
    for name, fname in files.items():
        dump_json(current[name], output_dir / fname)
    dump_json(build_run_metadata(effective_compile_scope=effective_compile_scope,
                                 compile_scope_reason=compile_scope_reason), output_dir / RUN_METADATA_FILE)
    write_config_yaml_snapshots(logging_dir=logging_dir, config_path=config_path, sections=sections)
