"""Run directories, resume resolution and transactional checkpoints.

On-disk layout of the reference (``training/run_management.py``): ``checkpoint-<step>/`` with the
model weights, optimizer/scheduler/RNG state, ``data_state.json`` and a ``.complete`` marker that
is written last; a checkpoint is staged in ``.checkpoint-<step>.tmp-<uuid>`` and renamed into
place, old committed checkpoints are rotated, and ``resume_from_checkpoint=auto`` picks the newest
checkpoint that passes the integrity checks. Rank 0 decides; other ranks receive the decision
(or the error) by broadcast.
"""

from __future__ import annotations

import logging
import os
import re
import shutil
import tempfile
import uuid
from contextlib import suppress
from datetime import datetime
from pathlib import Path
from typing import Any

from deberta_b200.run_layout import CHECKPOINT_PREFIX, COMPLETE_MARKER_FILE, DATA_STATE_FILE
from deberta_b200.utils.io import dump_json, load_json_mapping

logger = logging.getLogger(__name__)

_WEIGHT_PATTERNS = ("model.safetensors", "pytorch_model.bin", "model.bin", "*model*.safetensors", "*model*.bin")


def sanitize_run_label(text: str) -> str:
    out = re.sub(r"[^A-Za-z0-9._-]+", "-", str(text).strip()).strip("-.")
    return out or "run"


def resolve_output_dir(*, output_dir: str | None, project_name: str, config_path: str | Path | None,
                       run_name: str | None = None) -> Path:
    """Explicit directory, else ``runs/<project>/<YYYYmmdd_HHMMSS>_<run name or config stem>``."""
    if output_dir is not None and str(output_dir).strip():
        return Path(str(output_dir))
    hint = str(run_name).strip() if run_name else ""
    if not hint and config_path is not None:
        hint = Path(config_path).stem
    stamp = datetime.now().strftime("%Y%m%d_%H%M%S")
    return Path("runs") / sanitize_run_label(project_name) / f"{stamp}_{sanitize_run_label(hint or 'run')}"


def broadcast_rank0_result(ctx: Any, compute, *, broadcast_fn=None) -> Any:
    """Run ``compute`` on rank 0 and hand its value — or its exception — to every rank."""
    if int(getattr(ctx, "world_size", getattr(ctx, "num_processes", 1))) <= 1:
        return compute()
    box: dict[str, Any] = {"ok": True, "value": None, "error_type": None, "error_message": None}
    if bool(getattr(ctx, "is_main_process", False)):
        try:
            box["value"] = compute()
        except Exception as exc:  # forwarded to all ranks below
            box = {"ok": False, "value": None, "error_type": type(exc).__name__, "error_message": str(exc)}
    box = (broadcast_fn or ctx.broadcast_object)(box)
    if not isinstance(box, dict):
        raise RuntimeError("Broadcasted rank-0 payload is malformed.")
    if not box.get("ok", False):
        err = {"ValueError": ValueError, "FileNotFoundError": FileNotFoundError}.get(str(box.get("error_type")), RuntimeError)
        raise err(str(box.get("error_message") or "Unknown error on rank 0."))
    return box.get("value")


def resolve_output_dir_for_ranks(ctx: Any, **kw: Any) -> Path:
    """Same directory on every rank (time-stamped names are decided once, on rank 0)."""
    return Path(broadcast_rank0_result(ctx, lambda: str(resolve_output_dir(**kw))))


# ---- checkpoint inspection ------------------------------------------------------------------------
def parse_checkpoint_step(path: str | Path) -> int:
    m = re.search(rf"{CHECKPOINT_PREFIX}(\d+)", Path(path).name)
    return int(m.group(1)) if m else 0


def list_checkpoints(output_dir: Path) -> list[tuple[int, Path]]:
    return sorted((parse_checkpoint_step(p), p) for p in Path(output_dir).glob(f"{CHECKPOINT_PREFIX}*") if p.is_dir())


def find_latest_checkpoint(output_dir: Path) -> Path | None:
    found = list_checkpoints(output_dir)
    return found[-1][1] if found else None


def checkpoint_weights_appear_valid(checkpoint_dir: Path) -> bool:
    """Structural check: some non-empty model payload exists (single file or sharded directory)."""
    for pat in _WEIGHT_PATTERNS:
        for f in checkpoint_dir.glob(pat):
            with suppress(OSError):
                if f.is_file() and f.stat().st_size > 0:
                    return True
    for sub in checkpoint_dir.glob("pytorch_model_fsdp*"):
        if sub.is_dir():
            for f in sub.rglob("*"):
                with suppress(OSError):
                    if f.is_file() and f.stat().st_size > 0:
                        return True
    return False


def is_checkpoint_committed(checkpoint_dir: Path) -> bool:
    return (Path(checkpoint_dir) / COMPLETE_MARKER_FILE).is_file()


def load_checkpoint_progress_metadata(checkpoint_dir: Path):
    """``(consumed_micro_batches, lr_mult, optimizer_param_digest, global_step, ga_steps)`` from ``data_state.json``."""
    path = Path(checkpoint_dir) / DATA_STATE_FILE
    if not path.exists():
        return None, 1.0, None, None, None
    try:
        raw = load_json_mapping(path)
        consumed = raw.get("consumed_micro_batches")
        consumed = max(0, int(consumed)) if consumed is not None else None
        digest = raw.get("optimizer_param_digest")
        if isinstance(digest, dict):
            digest = {str(k): str(v) for k, v in digest.items()}
        elif digest is not None:
            digest = str(digest)
        step = raw.get("global_step")
        ga = raw.get("gradient_accumulation_steps")
        return (consumed, float(raw.get("lr_mult", 1.0)), digest, max(0, int(step)) if step is not None else None,
                max(1, int(ga)) if ga is not None else None)
    except Exception as exc:
        logger.warning("Checkpoint %s has invalid data_state.json (%s: %s); treating as unresumable.",
                       checkpoint_dir, type(exc).__name__, exc)
        return None, 1.0, None, None, None


def load_checkpoint_data_progress(checkpoint_dir: Path):
    c, m, d, _, _ = load_checkpoint_progress_metadata(checkpoint_dir)
    return c, m, d


def save_checkpoint_data_progress(*, checkpoint_dir: Path, consumed_micro_batches: int, lr_mult: float = 1.0,
                                  optimizer_param_digest=None, global_step: int | None = None,
                                  gradient_accumulation_steps: int | None = None) -> None:
    payload: dict[str, Any] = {"consumed_micro_batches": int(max(0, consumed_micro_batches)), "lr_mult": float(lr_mult)}
    if optimizer_param_digest is not None:
        payload["optimizer_param_digest"] = ({str(k): str(v) for k, v in optimizer_param_digest.items()}
                                             if isinstance(optimizer_param_digest, dict) else str(optimizer_param_digest))
    if global_step is not None:
        payload["global_step"] = int(max(0, global_step))
    if gradient_accumulation_steps is not None:
        payload["gradient_accumulation_steps"] = int(max(1, gradient_accumulation_steps))
    dump_json(payload, Path(checkpoint_dir) / DATA_STATE_FILE)


def is_checkpoint_resumable(checkpoint_dir: Path) -> bool:
    return (is_checkpoint_committed(checkpoint_dir) and load_checkpoint_data_progress(checkpoint_dir)[0] is not None
            and checkpoint_weights_appear_valid(checkpoint_dir))


def find_latest_resumable_checkpoint(output_dir: Path) -> Path | None:
    for _step, ck in reversed(list_checkpoints(output_dir)):
        if is_checkpoint_resumable(ck):
            return ck
        if load_checkpoint_data_progress(ck)[0] is not None and not checkpoint_weights_appear_valid(ck):
            logger.warning("Checkpoint %s has resume metadata but model weights appear missing/empty; skipping.", ck)
    return None


def resolve_resume_checkpoint(*, output_dir: Path, resume_from_checkpoint: str | None, is_main_process: bool) -> str | None:
    """Explicit path (must be committed and intact) or ``auto`` (newest resumable under ``output_dir``)."""
    value = str(resume_from_checkpoint).strip() if resume_from_checkpoint is not None else ""
    if not value:
        return None
    if value.lower() != "auto":
        ck = Path(value).expanduser()
        if not ck.exists():
            raise FileNotFoundError(f"train.resume_from_checkpoint was provided but the checkpoint path does not exist: {ck}")
        if not ck.is_dir():
            raise ValueError(f"train.resume_from_checkpoint must point to a checkpoint directory. Got a non-directory path: {ck}")
        if not is_checkpoint_committed(ck):
            raise ValueError(f"Explicit resume checkpoint '{ck}' is missing .complete marker. "
                             "Only transactionally committed checkpoints are resumable.")
        if load_checkpoint_data_progress(ck)[0] is None:
            raise ValueError(f"Explicit resume checkpoint '{ck}' has .complete marker but failed resume integrity checks "
                             "(missing/invalid data_state.json with consumed_micro_batches).")
        if not checkpoint_weights_appear_valid(ck):
            raise ValueError(f"Explicit resume checkpoint '{ck}' has .complete marker but model weights appear missing or empty.")
        return str(ck.resolve())
    output_dir = Path(output_dir)
    latest = find_latest_checkpoint(output_dir)
    if latest is None:
        if output_dir.exists() and any(output_dir.iterdir()):
            raise ValueError("resume_from_checkpoint=auto was requested but no checkpoint-* directories were found in "
                             f"non-empty output_dir={output_dir}. Clean the directory, enable "
                             "train.overwrite_output_dir=true, or provide an explicit checkpoint path.")
        if is_main_process:
            logger.info("resume_from_checkpoint=auto but no checkpoint-* dirs found; starting from scratch.")
        return None
    good = find_latest_resumable_checkpoint(output_dir)
    if good is None:
        raise ValueError("resume_from_checkpoint=auto found checkpoint-* directories but none are resumable "
                         "(missing .complete marker and/or missing valid data_state.json/model weights). "
                         "Provide an explicit checkpoint path or clean stale/incomplete checkpoints.")
    if is_main_process and good != latest:
        logger.warning("resume_from_checkpoint=auto skipped newest checkpoint %s because resume metadata is "
                       "missing/invalid; falling back to %s.", latest, good)
    return str(good.resolve())


def resolve_resume_checkpoint_for_ranks(ctx: Any, *, output_dir: Path, resume_from_checkpoint: str | None,
                                        broadcast_fn=None) -> str | None:
    if not (str(resume_from_checkpoint).strip() if resume_from_checkpoint is not None else ""):
        return None
    out = broadcast_rank0_result(
        ctx, lambda: resolve_resume_checkpoint(output_dir=output_dir, resume_from_checkpoint=resume_from_checkpoint,
                                               is_main_process=bool(getattr(ctx, "is_main_process", True))),
        broadcast_fn=broadcast_fn)
    if out is not None and not str(out).strip():
        raise RuntimeError("Broadcasted resume checkpoint path is empty.")
    return None if out is None else str(out)


def prepare_output_dir(*, output_dir: Path, overwrite_output_dir: bool, resume_from_checkpoint: str | None,
                       is_main_process: bool) -> None:
    if not is_main_process:
        return
    output_dir = Path(output_dir)
    resuming = bool(str(resume_from_checkpoint).strip()) if resume_from_checkpoint is not None else False
    if output_dir.exists():
        if not output_dir.is_dir():
            raise ValueError(f"Output directory exists and is not a directory: {output_dir}")
        if any(output_dir.iterdir()):
            if not (overwrite_output_dir or resuming):
                raise ValueError(f"Output directory exists and is not empty: {output_dir}. "
                                 "Set train.overwrite_output_dir=true or set train.resume_from_checkpoint.")
            if overwrite_output_dir:
                shutil.rmtree(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)


def rotate_checkpoints(output_dir: Path, *, save_total_limit: int) -> None:
    """Keep the newest ``save_total_limit`` committed checkpoints (uncommitted ones are never counted or deleted)."""
    if save_total_limit <= 0:
        return
    committed = [(s, p) for s, p in list_checkpoints(output_dir) if is_checkpoint_committed(p)]
    for step, p in committed[: max(0, len(committed) - save_total_limit)]:
        try:
            shutil.rmtree(p)
            logger.info("Deleted old checkpoint: %s (step=%d)", p, step)
        except Exception as e:
            logger.warning("Failed to delete checkpoint %s: %s", p, e)


def write_complete_marker(directory: Path) -> None:
    marker = Path(directory) / COMPLETE_MARKER_FILE
    fd, tmp = tempfile.mkstemp(dir=directory, prefix=f".{marker.name}.", suffix=".tmp")
    try:
        with os.fdopen(fd, "w", encoding="utf-8") as f:
            f.write("ok\n")
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, marker)
    except BaseException:
        with suppress(OSError):
            os.unlink(tmp)
        raise


def save_training_checkpoint(*, ctx: Any, save_state, checkpoint_dir: Path, output_dir: Path, consumed_micro_batches: int,
                             save_total_limit: int, log_label: str, lr_mult: float = 1.0, optimizer_param_digest=None,
                             global_step: int | None = None, gradient_accumulation_steps: int | None = None) -> None:
    """Stage → every rank writes its state (``save_state(dir)``) → rank 0 adds metadata, validates, commits, rotates."""
    checkpoint_dir = Path(checkpoint_dir)
    staging = checkpoint_dir.parent / f".{checkpoint_dir.name}.tmp-{uuid.uuid4().hex}"
    staging = Path(ctx.broadcast_object(str(staging))) if getattr(ctx, "distributed", False) else staging
    ctx.wait_for_everyone()
    if ctx.is_main_process:
        if checkpoint_dir.exists():
            if any(checkpoint_dir.iterdir()):
                raise RuntimeError(f"Refusing to overwrite non-empty checkpoint directory: {checkpoint_dir}. "
                                   "Checkpoint directories are immutable; use a new step directory.")
            checkpoint_dir.rmdir()
        staging.mkdir(parents=True, exist_ok=False)
    ctx.wait_for_everyone()
    save_state(str(staging))
    ctx.wait_for_everyone()
    if not ctx.is_main_process:
        # rank 0 validates, commits and rotates alone; the others wait for it so that no rank runs ahead into
        # device-side waits (bounded in seconds) while rank 0 is still deleting old checkpoints
        ctx.wait_for_everyone()
        return
    try:
        save_checkpoint_data_progress(checkpoint_dir=staging, consumed_micro_batches=consumed_micro_batches, lr_mult=lr_mult,
                                      optimizer_param_digest=optimizer_param_digest, global_step=global_step,
                                      gradient_accumulation_steps=gradient_accumulation_steps)
        ok_progress = load_checkpoint_data_progress(staging)[0] is not None
        ok_weights = checkpoint_weights_appear_valid(staging)
        if not (ok_progress and ok_weights):
            raise RuntimeError(f"Post-save structural validation failed for staged checkpoint {staging} "
                               f"(data_state_ok={ok_progress}, weights_ok={ok_weights}).")
        write_complete_marker(staging)
        staging.replace(checkpoint_dir)
        rotate_checkpoints(output_dir, save_total_limit=int(save_total_limit))
        logger.info("Saved %s checkpoint: %s", log_label, checkpoint_dir)
    except Exception:
        shutil.rmtree(staging, ignore_errors=True)
        raise
    finally:
        ctx.wait_for_everyone()
