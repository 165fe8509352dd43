"""Command-line surface: flag parsing, precedence file < preset < flags, mutation warnings, fast exit, dispatch.

Reference counterparts: ``tests/test_config_and_training_cli.py`` (CLI parse, dotted flags, presets, dry-run, fast-exit)
and ``tests/test_cli_entrypoint.py`` (``python -m`` wiring).
"""

from __future__ import annotations

import argparse
import json

import pytest
import yaml

from deberta_b200 import cli


@pytest.fixture(scope="module")
def parser():
    return cli._build_main_parser()


def _cfg_file(tmp_path, data=None, name="cfg.yaml"):
    data = data or {"model": {"backbone_type": "rope", "tokenizer": {"name_or_path": "synthetic:512"}},
                    "data": {"source": {"dataset_name": "synthetic"}, "packing": {"max_seq_length": 64}},
                    "train": {"max_steps": 5, "mixed_precision": "no"}}
    p = tmp_path / name
    p.write_text(yaml.safe_dump(data) if name.endswith(".yaml") else json.dumps(data))
    return p


def _resolve(parser, argv):
    ns = parser.parse_args(argv)
    return cli.resolve_train_config(ns, dict(parser._dotflag_map))


# ---------------------------------------------------------------------------------------------- parsing
def test_a_subcommand_is_required(parser):
    with pytest.raises(SystemExit):
        parser.parse_args([])
    with pytest.raises(SystemExit):
        parser.parse_args(["fine-tune"])


def test_dotted_flags_are_typed(parser):
    ns = parser.parse_args(["train", "--train.max_steps", "7", "--optim.lr.base", "3e-4", "--train.decoupled_training", "false",
                            "--train.checkpoint.output_dir", "none", "--model.rope.keel_alpha_init", "0.5"])
    assert ns.dot__train__max_steps == 7 and ns.dot__optim__lr__base == 3e-4 and ns.dot__train__decoupled_training is False
    assert ns.dot__train__checkpoint__output_dir is None and ns.dot__model__rope__keel_alpha_init == 0.5
    assert not hasattr(ns, "dot__train__gradient_accumulation_steps")  # flags that were not given leave no trace


@pytest.mark.parametrize("argv", [
    ["train", "--train.max_steps", "many"],
    ["train", "--train.decoupled_training", "1"],           # booleans are words, not digits
    ["train", "--model.backbone_type", "lstm"],             # constrained fields list their choices
    ["train", "--train.no_such_flag", "1"],
    ["train", "--preset", "bert-large"],
])
def test_bad_flag_values_are_usage_errors(parser, argv):
    with pytest.raises(SystemExit) as e:
        parser.parse_args(argv)
    assert e.value.code == 2


def test_choice_flags_accept_aliases_and_mixed_precision_is_free_text(parser):
    ns = parser.parse_args(["train", "--train.mixed_precision", "BF16", "--model.rope.pretrained.ffn_type", "swiglu"])
    assert ns.dot__train__mixed_precision == "BF16" and ns.dot__model__rope__pretrained__ffn_type == "swiglu"


def test_export_subcommand_parses(parser):
    ns = parser.parse_args(["export", "runs/x/checkpoint-10", "--what", "generator", "--output-dir", "out"])
    assert (ns.command, ns.checkpoint_dir, ns.export_what, ns.output_dir) == ("export", "runs/x/checkpoint-10", "generator", "out")
    assert ns.safe_serialization is True and ns.allow_partial_export is False


def test_bool_and_optional_helpers():
    assert cli._parse_bool("Yes") is True and cli._parse_bool("off") is False
    with pytest.raises(argparse.ArgumentTypeError, match="Expected a boolean value"):
        cli._parse_bool("2")
    opt_int = cli._optional(int)
    assert opt_int("none") is None and opt_int("NULL") is None and opt_int("12") == 12
    assert cli._flag_text(None) == "none" and cli._flag_text(True) == "true" and cli._flag_text(3) == "3"


# ---------------------------------------------------------------------------------------------- precedence
def test_flags_override_the_file(parser, tmp_path, capsys):
    p = _cfg_file(tmp_path)
    cfg, path = _resolve(parser, ["train", str(p), "--train.max_steps", "9", "--data.packing.max_seq_length", "128"])
    assert path == p.resolve() and cfg.train.max_steps == 9 and cfg.data.packing.max_seq_length == 128
    err = capsys.readouterr().err
    assert "was modified after load" in err and "train.max_steps: 5 -> 9 (CLI override (--train.max_steps))" in err


def test_unchanged_files_produce_no_warning(parser, tmp_path, capsys):
    _resolve(parser, ["train", str(_cfg_file(tmp_path))])
    assert "config-warning" not in capsys.readouterr().err


def test_missing_config_file(parser, tmp_path):
    with pytest.raises(FileNotFoundError):
        _resolve(parser, ["train", str(tmp_path / "absent.yaml")])


def test_preset_without_a_file_provides_a_full_run(parser, capsys):
    cfg, path = _resolve(parser, ["train", "--preset", "deberta-v3-base"])
    assert path is None and cfg.model.backbone_type == "hf_deberta_v2" and cfg.model.profile == "deberta_v3_parity"
    assert cfg.data.source.dataset_name == "HuggingFaceFW/fineweb-edu" and cfg.train.max_steps == 500_000
    assert cfg.train.objective.mask_token_prob == 1.0 and cfg.optim.scheduler.warmup_steps == 10_000  # parity defaults applied
    assert "model+data+train+optim+logging defaults" in capsys.readouterr().out


def test_preset_with_a_file_touches_only_the_model_section(parser, tmp_path, capsys):
    data = {"data": {"source": {"dataset_name": "synthetic"}, "packing": {"max_seq_length": 64}}, "train": {"max_steps": 5}}
    cfg, _ = _resolve(parser, ["train", str(_cfg_file(tmp_path, data)), "--preset", "deberta-v3-base"])
    assert cfg.model.tokenizer.name_or_path == "microsoft/deberta-v3-base" and cfg.model.backbone_type == "hf_deberta_v2"
    assert cfg.data.source.dataset_name == "synthetic" and cfg.train.max_steps == 5
    assert "model-only overrides" in capsys.readouterr().out


def test_flags_beat_the_preset(parser):
    cfg, _ = _resolve(parser, ["train", "--preset", "deberta-v3-base", "--train.max_steps", "11", "--model.hf.model_size", "small"])
    assert cfg.train.max_steps == 11 and cfg.model.hf.model_size == "small"


def test_unknown_preset_name():
    from deberta_b200.config import Config

    with pytest.raises(ValueError, match="Unknown train preset"):
        cli._apply_preset(cfg=Config(), preset_name="nope", with_config_file=False)


def test_validation_errors_surface_from_resolution(parser, tmp_path):
    with pytest.raises(ValueError, match="No dataset source configured"):
        _resolve(parser, ["train"])
    with pytest.raises(ValueError, match="overwrite_output_dir=true cannot be combined"):
        _resolve(parser, ["train", str(_cfg_file(tmp_path)), "--train.checkpoint.overwrite_output_dir", "true",
                          "--train.checkpoint.resume_from_checkpoint", "auto"])


# ---------------------------------------------------------------------------------------------- dispatch / exit
@pytest.mark.parametrize("env,explicit,want", [(None, False, True), (None, True, False), ("0", False, False), ("false", False, False),
                                               ("1", False, True)])
def test_fast_exit_policy(monkeypatch, env, explicit, want):
    if env is None:
        monkeypatch.delenv("DEBERTA_FAST_EXIT_AFTER_TRAIN", raising=False)
    else:
        monkeypatch.setenv("DEBERTA_FAST_EXIT_AFTER_TRAIN", env)
    assert cli._should_fast_exit_after_train(explicit_argv=explicit) is want


def test_main_dispatches_train_and_export(monkeypatch, tmp_path):
    seen = {}
    import deberta_b200.export_cli as export_cli
    import deberta_b200.training as training

    monkeypatch.setattr(training, "run_pretraining", lambda **kw: seen.setdefault("train", kw))
    monkeypatch.setattr(training, "run_pretraining_dry_run", lambda **kw: {k: "x" for k in (
        "checkpoint_output_dir", "logging_output_dir", "resume_checkpoint", "effective_compile_scope", "sample_batch_shape",
        "sample_active_tokens", "tokenizer_vocab_size")} | seen.setdefault("dry", kw))
    monkeypatch.setattr(export_cli, "run_export", lambda cfg: seen.setdefault("export", cfg))
    p = _cfg_file(tmp_path)
    cli.main(["train", str(p), "--train.max_steps", "3"])  # explicit argv: returns instead of exiting the interpreter
    assert seen["train"]["train_cfg"].max_steps == 3 and seen["train"]["config_path"] == p.resolve()
    assert set(seen["train"]) == {"model_cfg", "data_cfg", "train_cfg", "optim_cfg", "logging_cfg", "config_path"}
    cli.main(["train", str(p), "--dry-run"])
    assert "dry" in seen
    cli.main(["export", str(tmp_path / "checkpoint-1"), "--what", "both"])
    assert seen["export"].export_what == "both" and seen["export"].checkpoint_dir == str(tmp_path / "checkpoint-1")


def test_dry_run_prints_one_summary_line(monkeypatch, tmp_path, capsys):
    import deberta_b200.training as training

    report = {"checkpoint_output_dir": "out", "logging_output_dir": "out/logs", "resume_checkpoint": None,
              "effective_compile_scope": "none", "sample_batch_shape": (2, 64), "sample_active_tokens": 100,
              "tokenizer_vocab_size": 512}
    monkeypatch.setattr(training, "run_pretraining_dry_run", lambda **kw: report)
    cli.main(["train", str(_cfg_file(tmp_path)), "--dry-run"])
    out = capsys.readouterr().out.strip().splitlines()[-1]
    assert out.startswith("Dry-run preflight OK: checkpoint_output_dir=out") and "tokenizer_vocab_size=512" in out


def test_module_entry_point_calls_the_cli(monkeypatch):
    import runpy

    called = []
    monkeypatch.setattr(cli, "main", lambda *a, **k: called.append((a, k)))
    with pytest.raises(SystemExit) as e:
        runpy.run_module("deberta_b200", run_name="__main__")
    assert e.value.code == 0
    assert called == [((), {})]  # plain call: the fast-exit policy sees a console invocation
