"""``deberta export``: turn a training checkpoint into standalone Hugging Face artifacts.

Arguments and output layout follow ``export_cli.py`` of the reference. Checkpoints written by this
framework hold the complete fp32 model in ``model.safetensors`` (gathered from the optimizer
shards at save time), so an export is a single-process job; the reference's sharded DCP layout is
readable too. The staged output directory is renamed into place only when everything was written.
"""

from __future__ import annotations

import argparse
import shutil
import uuid
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from deberta_b200.config import load_model_config_snapshot, validate_model_config
from deberta_b200.run_layout import MODEL_CONFIG_FILE, infer_run_dir_from_checkpoint, validate_run_metadata_file
from deberta_b200.utils.io import dump_json, load_json_mapping


@dataclass
class ExportConfig:
    checkpoint_dir: str
    output_dir: str | None = None
    run_dir: str | None = None
    export_what: str = "discriminator"  # discriminator|generator|both
    safe_serialization: bool = True
    offload_to_cpu: bool = True   # accepted for command-line compatibility; checkpoints are already consolidated
    rank0: bool = True            # likewise
    embedding_sharing: str | None = None
    allow_partial_export: bool = False


def add_export_arguments(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("checkpoint_dir", help="Path to checkpoint-<step> directory saved by training.")
    parser.add_argument("--output-dir", default=None,
                        help="Output directory for exported artifacts (must be empty). Defaults to <run_dir>/exported_hf.")
    parser.add_argument("--run-dir", default=None,
                        help="Run directory containing model_config.json. Defaults to the checkpoint's parent.")
    parser.add_argument("--what", "--export-what", dest="export_what", default="discriminator",
                        choices=("discriminator", "generator", "both"), help="Which component(s) to export.")
    for flag, dest, text in (("safe-serialization", "safe_serialization", "Save weights as safetensors."),
                             ("offload-to-cpu", "offload_to_cpu", "Kept for compatibility (no effect)."),
                             ("rank0-only", "rank0", "Kept for compatibility (no effect).")):
        g = parser.add_mutually_exclusive_group()
        g.add_argument(f"--{flag}", dest=dest, action="store_true", help=text)
        g.add_argument(f"--no-{flag}", dest=dest, action="store_false")
        parser.set_defaults(**{dest: True})
    parser.add_argument("--embedding-sharing", default=None, choices=("none", "es", "gdes"),
                        help="Override embedding sharing mode. Defaults to the training config value.")
    parser.add_argument("--allow-partial-export", action="store_true",
                        help="Export the key intersection instead of failing on missing/unexpected backbone keys.")


def namespace_to_export_config(ns: argparse.Namespace) -> ExportConfig:
    return ExportConfig(checkpoint_dir=str(ns.checkpoint_dir), output_dir=ns.output_dir, run_dir=ns.run_dir,
                        export_what=str(ns.export_what), safe_serialization=bool(ns.safe_serialization),
                        offload_to_cpu=bool(ns.offload_to_cpu), rank0=bool(ns.rank0),
                        embedding_sharing=ns.embedding_sharing, allow_partial_export=bool(ns.allow_partial_export))


def _build_export_backbone(backbone_type: str, config: Any) -> torch.nn.Module:
    if backbone_type == "hf_deberta_v2":
        from transformers import AutoModel

        return AutoModel.from_config(config)
    from deberta_b200.models import DebertaRoPEModel

    return DebertaRoPEModel(config)


def _export_component(*, name: str, out_dir: Path, config: Any, own_sd: dict, disc_sd: dict, gen_sd: dict, mode: str,
                      backbone_type: str, cfg: ExportConfig, tokenizer_name: str, step: int | None) -> dict[str, Any]:
    from deberta_b200.models.export_utils import (clean_exported_config, load_intersection_state_dict,
                                                  merge_embeddings_into_export_backbone, write_export_readme)

    model = _build_export_backbone(backbone_type, config)
    state = dict(own_sd)
    if name == "discriminator" and mode == "gdes":
        # GDES checkpoints hold (frozen base, trainable delta) per shared table instead of one weight. The base stands in
        # for the weight during the strict load (every key of the export backbone is then accounted for) and the merge
        # below replaces it by base + delta; the delta ("bias") tensors only feed that merge.
        wanted = set(model.state_dict().keys())
        state = {}
        for k, v in own_sd.items():
            if k.startswith("embeddings.") and k.endswith(".base_weight"):
                target = k[: -len("base_weight")] + "weight"
                if target in wanted and target not in own_sd:
                    state[target] = v
            elif k.startswith("embeddings.") and k.endswith("_embeddings.bias") and k not in wanted:
                continue
            else:
                state[k] = v
    # the stock HF backbone has no absolute-position table when `position_biased_input` is off; the pretrainer keeps one
    # for its Enhanced Mask Decoder. It is not part of the exported encoder, so it is not an unexpected key either.
    missing, unexpected = load_intersection_state_dict(model, state, strict=not cfg.allow_partial_export,
                                                       ignore_unexpected=("embeddings.position_embeddings.weight",))
    if name == "discriminator":
        merge_embeddings_into_export_backbone(export_model=model, disc_sd=disc_sd, gen_sd=gen_sd, mode=mode)
        missing = [k for k in missing if not (mode in {"es", "gdes"} and k.startswith("embeddings.") and k.endswith(".weight"))]
    out_dir.mkdir(parents=True, exist_ok=True)
    model.save_pretrained(str(out_dir), safe_serialization=cfg.safe_serialization)
    clean_exported_config(out_dir / "config.json", strict=True)
    write_export_readme(out_dir, what=name, backbone_type=backbone_type, embedding_sharing=mode, step=step,
                        tokenizer_name=tokenizer_name)
    return {"missing_keys": missing, "unexpected_keys": unexpected}


def run_export(cfg: ExportConfig) -> Path:
    """Export and return the output directory."""
    from deberta_b200.data.synthetic import load_tokenizer
    from deberta_b200.models import build_backbone_configs
    from deberta_b200.models.export_utils import split_pretrainer_state_dict
    from deberta_b200.training.run_management import parse_checkpoint_step
    from deberta_b200.utils.checkpoint import load_model_state_dict

    ck = Path(cfg.checkpoint_dir).expanduser().resolve()
    if not ck.is_dir():
        raise FileNotFoundError(f"Checkpoint directory not found: {ck}")
    run_dir = Path(cfg.run_dir).expanduser().resolve() if cfg.run_dir else infer_run_dir_from_checkpoint(ck)
    validate_run_metadata_file(run_dir)
    model_cfg = load_model_config_snapshot(load_json_mapping(run_dir / MODEL_CONFIG_FILE), source=str(run_dir / MODEL_CONFIG_FILE))
    validate_model_config(model_cfg)
    mode = (cfg.embedding_sharing or model_cfg.embedding_sharing).lower()
    out = Path(cfg.output_dir).expanduser().resolve() if cfg.output_dir else run_dir / "exported_hf"
    if out.exists() and any(out.iterdir()):
        raise ValueError(f"Export output directory must be empty: {out}")
    data_cfg_path = run_dir / "data_config.json"
    max_seq = int(load_json_mapping(data_cfg_path)["packing"]["max_seq_length"]) if data_cfg_path.exists() else 512
    tok = load_tokenizer(model_cfg.tokenizer.name_or_path)
    import dataclasses

    scratch_cfg = dataclasses.replace(model_cfg, from_scratch=True) if model_cfg.from_scratch else model_cfg
    disc_config, gen_config = build_backbone_configs(model_cfg=scratch_cfg, tokenizer=tok, max_position_embeddings=max_seq)
    disc_sd, gen_sd = split_pretrainer_state_dict(load_model_state_dict(ck))
    if not disc_sd or not gen_sd:
        raise RuntimeError(f"Checkpoint {ck} does not contain generator.* and discriminator.* tensors.")
    staged = out.parent / f".{out.name}.tmp-{uuid.uuid4().hex}"
    staged.mkdir(parents=True, exist_ok=False)
    step = parse_checkpoint_step(ck) or None
    meta: dict[str, Any] = {"checkpoint": str(ck), "what": cfg.export_what, "embedding_sharing": mode,
                            "backbone_type": model_cfg.backbone_type, "step": step, "components": {}}
    try:
        todo = ["discriminator", "generator"] if cfg.export_what == "both" else [cfg.export_what]
        for name in todo:
            target = staged / name if cfg.export_what == "both" else staged
            meta["components"][name] = _export_component(
                name=name, out_dir=target, config=disc_config if name == "discriminator" else gen_config,
                own_sd=disc_sd if name == "discriminator" else gen_sd, disc_sd=disc_sd, gen_sd=gen_sd, mode=mode,
                backbone_type=model_cfg.backbone_type, cfg=cfg, tokenizer_name=model_cfg.tokenizer.name_or_path, step=step)
        if hasattr(tok, "save_pretrained"):
            tok.save_pretrained(str(staged))
        dump_json(meta, staged / "export_meta.json")
        if out.exists():
            out.rmdir()
        staged.replace(out)
    except BaseException:
        shutil.rmtree(staged, ignore_errors=True)
        raise
    return out
