"""``deberta train | export`` command line (same surface as ``src/deberta/cli.py`` of the reference).

``train [config] [--preset NAME] [--dry-run] [--section.path VALUE ...]``: one dotted flag
exists for every leaf of the config schema. Precedence: file < preset < flags, then
profile defaults for everything not set explicitly, then validation. When a file value
ends up changed, the change and its reason are printed to stderr.
"""

from __future__ import annotations

import argparse
import copy
import os
import sys
from pathlib import Path
from typing import Any

from deberta_b200.config import (
    Config,
    apply_dotted_override,
    asdict_without_private,
    choices_for,
    iter_leaf_paths_for_dataclass,
    load_config,
    validate_config,
)
from deberta_b200.utils.mapping import flatten_mapping
from deberta_b200.utils.types import parse_bool, unwrap_optional_type

_TRAIN_PRESETS: dict[str, dict[str, dict[str, Any]]] = {
    "deberta-v3-base": {
        "model": {
            "profile": "deberta_v3_parity", "backbone_type": "hf_deberta_v2", "from_scratch": True,
            "embedding_sharing": "gdes", "tokenizer": {"name_or_path": "microsoft/deberta-v3-base"},
            "hf": {"attention_kernel": "dynamic"},
        },
        "data": {
            "source": {"dataset_name": "HuggingFaceFW/fineweb-edu", "dataset_config_name": "default",
                       "train_split": "train", "streaming": True, "text_column_name": "text",
                       "shuffle_buffer_size": 10_000},
            "packing": {"enabled": True, "block_cross_document_attention": False, "max_seq_length": 512},
        },
        "train": {"max_steps": 500_000},
        "logging": {"backend": "none", "wandb": {"enabled": False}},
    }
}
_EXTRA_CHOICE_PATHS = {"model.rope.pretrained.norm_arch": "model.rope.norm_arch",
                       "model.rope.pretrained.ffn_type": "model.rope.ffn_type"}
_FALSE_STRINGS = {"0", "false", "f", "no", "n", "off"}


def _parse_bool(value: str) -> bool:
    try:
        return parse_bool(value, allow_numeric=False)
    except ValueError as exc:
        raise argparse.ArgumentTypeError(f"Expected a boolean value, got: {value}") from exc


def _optional(parser):
    def parse(value: str):
        return None if str(value).strip().lower() in {"none", "null"} else parser(value)
    return parse


def _should_fast_exit_after_train(*, explicit_argv: bool) -> bool:
    """``os._exit(0)`` after a successful console-script run skips slow interpreter teardown.

    Disabled when ``main`` was called with an explicit argv (tests, embedding) or when
    ``DEBERTA_FAST_EXIT_AFTER_TRAIN`` is a false value.
    """
    if explicit_argv:
        return False
    return str(os.getenv("DEBERTA_FAST_EXIT_AFTER_TRAIN", "1")).strip().lower() not in _FALSE_STRINGS


def _flag_text(value: Any) -> str:
    if value is None:
        return "none"
    if isinstance(value, bool):
        return "true" if value else "false"
    return str(value)


def _add_dotflags(parser: argparse.ArgumentParser) -> dict[str, str]:
    """Register ``--section.path`` for every config leaf; returns path → namespace dest."""
    out: dict[str, str] = {}
    for path, tp in iter_leaf_paths_for_dataclass(Config):
        target, optional = unwrap_optional_type(tp)
        conv = {bool: _parse_bool, int: int, float: float}.get(target, str)
        kw: dict[str, Any] = {"type": _optional(conv) if optional else conv}
        choices = choices_for(_EXTRA_CHOICE_PATHS.get(path, path), with_aliases=True)
        if choices and path != "train.mixed_precision":
            kw["choices"] = choices
        dest = "dot__" + path.replace(".", "__")
        parser.add_argument(f"--{path}", dest=dest, default=argparse.SUPPRESS, metavar="VALUE",
                            help=f"Override config field {path}.", **kw)
        out[path] = dest
    return out


def _build_main_parser() -> argparse.ArgumentParser:
    from deberta_b200.export_cli import add_export_arguments

    parser = argparse.ArgumentParser(prog="deberta", description="deberta CLI",
                                     formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    sub = parser.add_subparsers(dest="command", metavar="COMMAND", required=True)
    train = sub.add_parser("train", help="Run RTD pretraining.", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    train.add_argument("config", nargs="?", default=None, help="Path to a YAML/JSON config file.")
    train.add_argument("--preset", choices=tuple(sorted(_TRAIN_PRESETS)), default=None,
                       help="Training preset. With a config file only its model fields apply; without one it "
                            "provides model+data+train+optim+logging defaults.")
    train.add_argument("--dry-run", action="store_true",
                       help="Validate config, output/resume paths, tokenizer+dataset+collator and backbone configs, "
                            "then exit without training or writing checkpoints.")
    parser._dotflag_map = _add_dotflags(train)  # type: ignore[attr-defined]
    export = sub.add_parser("export", help="Consolidate and export a checkpoint to standalone HF artifacts.",
                            formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    add_export_arguments(export)
    return parser


def _apply_preset(*, cfg: Config, preset_name: str, with_config_file: bool) -> tuple[Config, str]:
    preset = _TRAIN_PRESETS.get(str(preset_name).strip().lower())
    if preset is None:
        raise ValueError(f"Unknown train preset: {preset_name!r}. Available presets: {', '.join(sorted(_TRAIN_PRESETS))}.")
    sections = ["model"] if with_config_file else ["model", "data", "train", "optim", "logging"]
    for section in sections:
        for path, value in flatten_mapping(dict(preset.get(section, {})), prefix=section).items():
            cfg = apply_dotted_override(cfg, f"{path}={_flag_text(value)}")
    if with_config_file:
        return cfg, "model-only overrides (config file provided)"
    return cfg, "model+data+train+optim+logging defaults (no config file)"


def _apply_dotflags(*, cfg: Config, ns: argparse.Namespace, dotflag_map: dict[str, str]):
    reasons: dict[str, str] = {}
    for path, dest in dotflag_map.items():
        if hasattr(ns, dest):
            cfg = apply_dotted_override(cfg, f"{path}={_flag_text(getattr(ns, dest))}")
            reasons[path] = f"CLI override (--{path})"
    return cfg, reasons


def _flatten_cfg(cfg: Config) -> dict[str, Any]:
    return flatten_mapping({name: asdict_without_private(getattr(cfg, name))
                            for name in ("model", "data", "train", "optim", "logging")})


def _emit_config_mutation_warnings(*, cfg_path: Path | None, before: Config, after: Config, reasons: dict[str, str]) -> None:
    if cfg_path is None:
        return
    old, new = _flatten_cfg(before), _flatten_cfg(after)
    changes = [(k, v, new[k], reasons.get(k, "runtime normalization/defaulting"))
               for k, v in old.items() if k in new and new[k] != v]
    if not changes:
        return
    print(f"[deberta][config-warning] Loaded config '{cfg_path}' was modified after load:", file=sys.stderr)
    for key, a, b, why in changes:
        print(f"[deberta][config-warning] {key}: {a!r} -> {b!r} ({why})", file=sys.stderr)


def resolve_train_config(ns: argparse.Namespace, dotflag_map: dict[str, str]) -> tuple[Config, Path | None]:
    """file < preset < dotted flags → profile defaults → validation."""
    cfg_path: Path | None = None
    if ns.config is not None:
        cfg_path = Path(ns.config).expanduser().resolve()
        if not cfg_path.exists():
            raise FileNotFoundError(str(cfg_path))
        cfg = load_config(cfg_path)
        baseline = copy.deepcopy(cfg)
    else:
        cfg, baseline = Config(), Config()
    if ns.preset:
        cfg, mode = _apply_preset(cfg=cfg, preset_name=str(ns.preset), with_config_file=cfg_path is not None)
        print(f"Applying train preset '{ns.preset}': {mode}.")
    cfg, reasons = _apply_dotflags(cfg=cfg, ns=ns, dotflag_map=dotflag_map)
    validate_config(cfg)
    _emit_config_mutation_warnings(cfg_path=cfg_path, before=baseline, after=cfg, reasons=reasons)
    return cfg, cfg_path


def _run_train(ns: argparse.Namespace, *, dotflag_map: dict[str, str]) -> None:
    from deberta_b200.training import run_pretraining, run_pretraining_dry_run

    cfg, cfg_path = resolve_train_config(ns, dotflag_map)
    kw = dict(model_cfg=cfg.model, data_cfg=cfg.data, train_cfg=cfg.train, optim_cfg=cfg.optim,
              logging_cfg=cfg.logging, config_path=cfg_path)
    if getattr(ns, "dry_run", False):
        r = run_pretraining_dry_run(**kw)
        print("Dry-run preflight OK: " + ", ".join(f"{k}={r[k]}" for k in (
            "checkpoint_output_dir", "logging_output_dir", "resume_checkpoint", "effective_compile_scope",
            "sample_batch_shape", "sample_active_tokens", "tokenizer_vocab_size")) + ".")
        return
    run_pretraining(**kw)


def main(argv: list[str] | None = None) -> None:
    explicit_argv = argv is not None
    argv = list(sys.argv[1:] if argv is None else argv)
    parser = _build_main_parser()
    args = parser.parse_args(argv)
    if args.command == "train":
        _run_train(args, dotflag_map=dict(parser._dotflag_map))  # type: ignore[attr-defined]
        if _should_fast_exit_after_train(explicit_argv=explicit_argv):
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        return
    if args.command == "export":
        from deberta_b200.export_cli import namespace_to_export_config, run_export

        run_export(namespace_to_export_config(args))


if __name__ == "__main__":
    main()
