"""Metric sinks: ``metrics.jsonl.gz`` rows and non-finite debug artifacts (``training/metrics.py`` of the reference)."""

from __future__ import annotations

import gzip
import json
import logging
import time
from pathlib import Path
from typing import Any

import torch

from deberta_b200.utils.io import dump_json

logger = logging.getLogger(__name__)


def append_metrics_jsonl_row(path: Path, row: dict[str, Any]) -> None:
    """Append one JSON row to a gzip member stream (readable with ``gzip.open`` as concatenated members)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with gzip.open(path, "at", encoding="utf-8") as f:
        f.write(json.dumps(row, sort_keys=True, default=float) + "\n")


def flush_loggers() -> None:
    for handler in logging.getLogger().handlers:
        try:
            handler.flush()
        except Exception:
            pass


def _rng_heads() -> dict[str, Any]:
    out: dict[str, Any] = {"torch_cpu": torch.get_rng_state()[:8].tolist()}
    if torch.cuda.is_available():
        try:
            out["torch_cuda"] = torch.cuda.get_rng_state()[:8].tolist()
        except Exception:
            pass
    return out


def write_nonfinite_debug_artifact(*, debug_dir: Path, step: int, what: str, losses: dict[str, float],
                                   lrs: dict[str, float], lr_mult: float, extra: dict[str, Any] | None = None) -> Path:
    """``debug/nonfinite_step_<n>_<what>.json`` with the losses, learning rates and RNG heads at the failure."""
    path = Path(debug_dir) / f"nonfinite_step_{int(step)}_{what}.json"
    payload = {"step": int(step), "what": str(what), "time": time.time(), "losses": losses, "lrs": lrs,
               "lr_mult": float(lr_mult), "rng": _rng_heads(), **(extra or {})}
    dump_json(payload, path)
    return path


def _config_mapping(obj: Any) -> dict[str, Any]:
    """Plain mapping of a backbone config object (``to_dict`` of HF configs, ``__dict__`` otherwise)."""
    if obj is None:
        return {}
    if isinstance(obj, dict):
        return dict(obj)
    to_dict = getattr(obj, "to_dict", None)
    if callable(to_dict):
        try:
            return dict(to_dict())
        except Exception:  # noqa: BLE001
            pass
    return {k: v for k, v in vars(obj).items() if not k.startswith("_")}


def build_runtime_resolved_config(*, sections: dict[str, Any], disc_config: Any = None, gen_config: Any = None,
                                  tokenizer: Any = None, runtime: dict[str, Any] | None = None) -> dict[str, Any]:
    """The configuration as the run really uses it, for ``config_resolved.yaml`` and the tracker.

    Starts from the five config sections and fills what only exists once the model is built
    (``training/metrics.py:82-161`` of the reference): the derived generator shape, dropout probabilities, the
    rope position limit and the tokenizer's vocabulary size; blank pretrained paths become absent; ``None`` leaves are
    pruned. ``runtime`` adds facts of this process group (world size, collective path, device).
    """
    from deberta_b200.utils.serialize import asdict_without_private, drop_none_recursive

    payload: dict[str, Any] = {name: asdict_without_private(cfg) for name, cfg in sections.items()}
    model = payload.setdefault("model", {})
    disc, gen = _config_mapping(disc_config), _config_mapping(gen_config)
    gen_out = dict(model.get("generator") or {})
    for key in ("num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads"):
        if gen_out.get(key) is None and gen.get(key) is not None:
            gen_out[key] = int(gen[key])
    model["generator"] = gen_out
    drop = dict(model.get("dropout") or {})
    for ours, theirs in (("hidden_prob", "hidden_dropout_prob"), ("attention_probs_prob", "attention_probs_dropout_prob")):
        if drop.get(ours) is None and disc.get(theirs) is not None:
            drop[ours] = float(disc[theirs])
    model["dropout"] = drop
    rope = dict(model.get("rope") or {})
    if rope.get("max_position_embeddings") is None and disc.get("max_position_embeddings") is not None:
        rope["max_position_embeddings"] = int(disc["max_position_embeddings"])
    model["rope"] = rope
    tok = dict(model.get("tokenizer") or {})
    if tok.get("vocab_target") is None and tokenizer is not None:
        try:
            tok["vocab_target"] = int(len(tokenizer))
        except Exception:  # noqa: BLE001
            pass
    model["tokenizer"] = tok
    pre = dict(model.get("pretrained") or {})
    for key in ("discriminator_path", "generator_path"):
        if not str(pre.get(key) or "").strip():
            pre[key] = None
    model["pretrained"] = pre
    if runtime:
        payload["runtime"] = dict(runtime)
    return drop_none_recursive(payload)
