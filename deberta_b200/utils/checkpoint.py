"""Checkpoint payload I/O.

A training checkpoint directory holds (names follow what Accelerate writes for the reference,
``utils/checkpoint.py`` / ``training/run_management.py`` there, so its tools can read our runs):

* ``model.safetensors``   — full fp32 model state (rank 0); in full-shard mode instead ``pytorch_model_fsdp_0/``, a
  torch distributed-checkpoint directory written by all ranks together (state nested under ``"model"``), which is
  what the reference's FSDP2 runs leave behind (``training/run_management.py:537-625`` there)
* ``optimizer.bin`` / ``optimizer_1.bin`` — generator (or single) / discriminator optimizer state in the layout of
  ``torch.optim.AdamW.state_dict()`` (two parameter groups, per-parameter moments), whole, written by rank 0: any
  number of ranks, in any parallelism mode, can resume from it, and ``torch.optim.AdamW.load_state_dict`` accepts it
* ``scheduler.bin`` / ``scheduler_1.bin``, ``trainer_state.bin``, ``random_states_<rank>.pkl``

Model weights can also be read from the other layouts the reference accepts: ``model.bin`` /
``pytorch_model.bin`` and torch-DCP sharded directories ``pytorch_model_fsdp*`` (state nested under
``"model"``), with ``_orig_mod.`` prefixes of compiled modules stripped.
"""

from __future__ import annotations

import logging
import pickle
import random
from pathlib import Path
from typing import Any

import numpy as np
import torch

logger = logging.getLogger(__name__)

MODEL_SAFETENSORS = "model.safetensors"


def canonicalize_state_dict_keys(state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Strip ``_orig_mod.`` (torch.compile wrappers) and a leading ``model.`` / ``module.`` prefix shared by all keys."""
    out = {k.replace("_orig_mod.", ""): v for k, v in state.items()}
    for prefix in ("model.", "module."):
        if out and all(k.startswith(prefix) for k in out):
            out = {k[len(prefix):]: v for k, v in out.items()}
    return out


def _load_dcp_dir(path: Path) -> dict[str, torch.Tensor]:
    """Read a torch distributed-checkpoint directory without a process group."""
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict_from_keys

    state = _load_state_dict_from_keys(storage_reader=FileSystemReader(str(path)))
    flat: dict[str, torch.Tensor] = {}

    def walk(prefix: str, obj: Any) -> None:
        if isinstance(obj, dict):
            for k, v in obj.items():
                walk(f"{prefix}.{k}" if prefix else str(k), v)
        elif isinstance(obj, torch.Tensor):
            flat[prefix] = obj

    walk("", state)
    return flat


def load_model_state_dict(checkpoint_dir: str | Path) -> dict[str, torch.Tensor]:
    """Model tensors of a checkpoint directory, whichever supported layout it uses (keys canonicalised)."""
    ck = Path(checkpoint_dir)
    st = ck / MODEL_SAFETENSORS
    if st.exists():
        from safetensors.torch import load_file

        return canonicalize_state_dict_keys(load_file(str(st)))
    for name in ("model.bin", "pytorch_model.bin"):
        if (ck / name).exists():
            return canonicalize_state_dict_keys(torch.load(ck / name, map_location="cpu", weights_only=True))
    for sub in sorted(ck.glob("pytorch_model_fsdp*")):
        if sub.is_dir():
            return canonicalize_state_dict_keys(_load_dcp_dir(sub))
    raise FileNotFoundError(f"No model weights found in checkpoint directory: {ck}")


def save_model_state_dict(state: dict[str, torch.Tensor], checkpoint_dir: str | Path) -> Path:
    """Write ``model.safetensors`` (tensors made contiguous and un-aliased first)."""
    from safetensors.torch import save_file

    path = Path(checkpoint_dir) / MODEL_SAFETENSORS
    save_file({k: v.detach().cpu().contiguous().clone() for k, v in state.items()}, str(path))
    return path


def capture_rng_state() -> dict[str, Any]:
    out: dict[str, Any] = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        out["cuda"] = torch.cuda.get_rng_state_all()
    return out


def restore_rng_state(state: dict[str, Any]) -> None:
    random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    torch.set_rng_state(state["torch"])
    if "cuda" in state and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state_all(state["cuda"])
        except Exception as e:  # different GPU count on resume
            logger.warning("Could not restore CUDA RNG state: %s", e)


DCP_MODEL_DIR = "pytorch_model_fsdp_0"


def save_model_state_dict_dcp(state: dict[str, torch.Tensor], checkpoint_dir: str | Path, *, distributed: bool) -> Path:
    """Write the model as a torch distributed-checkpoint directory (collective when ``distributed``: the planner
    spreads the tensors over the ranks' files)."""
    import torch.distributed.checkpoint as dcp

    path = Path(checkpoint_dir) / DCP_MODEL_DIR
    payload = {"model": {k: v.detach().cpu().contiguous() for k, v in state.items()}}
    dcp.save(payload, checkpoint_id=str(path), no_dist=not distributed)
    return path


def save_training_state(directory: str | Path, *, engine: Any, trainer: Any, ctx: Any) -> None:
    """Every rank's part of a checkpoint (collective: gathers fp32 masters and moments under sharding)."""
    d = Path(directory)
    # The outcome of the last window may still be on its way to the host; applying it can roll back an optimizer step,
    # change the LR multiplier or clear the moments, so every rank does it before any rank reads optimizer state.
    if hasattr(trainer, "wait_for_side_stream"):
        trainer.wait_for_side_stream()  # an optimizer update queued on the trainer's side stream
    trainer.resolve_pending()
    model_state = engine.model_state_dict()  # collective
    if getattr(engine, "full_shard", False):
        save_model_state_dict_dcp(model_state, d, distributed=ctx.world_size > 1)
    elif ctx.is_main_process:
        save_model_state_dict(model_state, d)
    opt_states = engine.torch_optimizer_state_dicts()  # collective
    if ctx.is_main_process:
        tstate = trainer.state_dict()
        for i, name in enumerate(engine.optimizers):
            suffix = "" if i == 0 else f"_{i}"
            torch.save(tstate["schedules"][name], d / f"scheduler{suffix}.bin")
            torch.save(opt_states[name], d / f"optimizer{suffix}.bin")
        torch.save(tstate, d / "trainer_state.bin")
    with open(d / f"random_states_{ctx.rank}.pkl", "wb") as f:
        pickle.dump(capture_rng_state(), f)


def load_training_state(directory: str | Path, *, engine: Any, trainer: Any, ctx: Any, strict: bool = True) -> None:
    """Restore model, optimizer moments, schedules and RNG state. The rank count and parallelism mode may differ from
    the run that wrote the checkpoint (each rank slices the whole optimizer state); RNG state is per rank and is
    restored only where a file for this rank exists."""
    d = Path(directory)
    engine.load_model_state_dict(load_model_state_dict(d), strict=strict)
    states: dict[str, Any] = {}
    for i, name in enumerate(engine.optimizers):
        path = d / ("optimizer.bin" if i == 0 else f"optimizer_{i}.bin")
        sd = torch.load(path, map_location="cpu", weights_only=False)
        if "param_groups" not in sd:
            raise RuntimeError(f"{path} is not in torch.optim state-dict layout (written by an older version?).")
        states[name] = sd
    engine.load_torch_optimizer_state_dicts(states)
    ts = d / "trainer_state.bin"
    if ts.exists():
        trainer.load_state_dict(torch.load(ts, map_location="cpu", weights_only=False))
    rng = d / f"random_states_{ctx.rank}.pkl"
    if rng.exists():
        with open(rng, "rb") as f:
            restore_rng_state(pickle.load(f))
