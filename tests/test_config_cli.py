"""Config system and CLI contracts (file formats, variables, strictness, flags, presets, shipped configs)."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import yaml

from deberta_b200 import config as C
from deberta_b200.cli import _build_main_parser, _add_dotflags, resolve_train_config  # noqa: F401

REPO = Path(__file__).resolve().parents[1]
BASE = {"model": {"backbone_type": "rope", "tokenizer": {"name_or_path": "synthetic:512"}},
        "data": {"source": {"dataset_name": "synthetic"}, "packing": {"max_seq_length": 64}},
        "train": {"max_steps": 5, "per_device_train_batch_size": 2, "mixed_precision": "no"}}


def _write(tmp_path, data, name="cfg.yaml"):
    p = tmp_path / name
    p.write_text(json.dumps(data) if name.endswith(".json") else yaml.safe_dump(data))
    return p


def test_yaml_and_json_load_to_the_same_config(tmp_path):
    a = C.load_config(_write(tmp_path, BASE))
    b = C.load_config(_write(tmp_path, BASE, "cfg.json"))
    assert C.asdict_without_private(a.train) == C.asdict_without_private(b.train)
    assert a.train.max_steps == 5 and a.data.packing.max_seq_length == 64 and a.model.backbone_type == "rope"


def test_variables_are_interpolated_and_cycles_rejected(tmp_path):
    data = json.loads(json.dumps(BASE))
    data["variables"] = {"seq": 96, "steps": "$variables.n", "n": 7}
    data["data"]["packing"]["max_seq_length"] = "$variables.seq"
    data["train"]["max_steps"] = "$variables.steps"
    cfg = C.load_config(_write(tmp_path, data))
    assert cfg.data.packing.max_seq_length == 96 and cfg.train.max_steps == 7
    data["variables"] = {"a": "$variables.b", "b": "$variables.a"}
    data["train"]["max_steps"] = "$variables.a"
    with pytest.raises(ValueError, match="(?i)cycl|circular"):
        C.load_config(_write(tmp_path, data, "cyc.yaml"))


def test_unknown_keys_and_wrong_types_are_errors(tmp_path):
    bad = json.loads(json.dumps(BASE))
    bad["train"]["max_stepz"] = 3
    with pytest.raises(ValueError, match="max_stepz"):
        C.load_config(_write(tmp_path, bad))
    bad = json.loads(json.dumps(BASE))
    bad["train"]["decoupled_training"] = "yes"  # booleans must be real booleans in files
    with pytest.raises(ValueError, match="decoupled_training"):
        C.load_config(_write(tmp_path, bad, "b.yaml"))
    ok = json.loads(json.dumps(BASE))
    ok["train"]["max_steps"] = "12"  # numeric strings are accepted
    assert C.load_config(_write(tmp_path, ok, "n.yaml")).train.max_steps == 12


def test_legacy_flat_key_gets_a_migration_hint(tmp_path):
    bad = json.loads(json.dumps(BASE))
    bad["train"]["learning_rate"] = 1e-4
    with pytest.raises(ValueError) as e:
        C.load_config(_write(tmp_path, bad))
    assert "optim" in str(e.value)


def test_dotted_overrides_and_explicit_field_tracking(tmp_path):
    cfg = C.load_config(_write(tmp_path, BASE), overrides=["train.max_steps=9", "optim.lr.base=0.001"])
    assert cfg.train.max_steps == 9 and abs(cfg.optim.lr.base - 1e-3) < 1e-12
    assert "max_steps" in C._explicit_fields(cfg.train)
    with pytest.raises(ValueError, match="Unknown override"):
        C.apply_dotted_override(cfg, "train.nope=1")
    with pytest.raises(ValueError, match="section"):
        C.apply_dotted_override(cfg, "trainx.max_steps=1")


def test_every_config_leaf_has_a_cli_flag():
    import argparse

    parser = argparse.ArgumentParser()
    mapping = _add_dotflags(parser)
    leaves = {f"{sec}.{p}" for sec in ("model", "data", "train", "optim", "logging")
              for p, _ in C.iter_leaf_paths_for_dataclass(type(getattr(C.Config(), sec)))}
    assert leaves and leaves <= set(mapping.values()) | set(mapping.keys())
    ns = parser.parse_args(["--train.max_steps", "11", "--model.backbone_type", "rope"])
    assert "11" in vars(ns).values() or 11 in vars(ns).values()


def test_choice_aliases_are_normalised():
    assert C.normalize_mixed_precision("bfloat16") == "bf16"
    assert C.normalize_mixed_precision("none") == "no"
    assert C.normalize_mixed_precision(False) == "no"
    with pytest.raises(ValueError):
        C.normalize_mixed_precision("fp8")


@pytest.mark.parametrize("name", sorted(p.name for p in (REPO / "configs").glob("*.yaml")))
def test_shipped_configs_parse_and_validate(name):
    cfg = C.load_config(REPO / "configs" / name)
    assert cfg.train.max_steps > 0
    assert cfg.model.backbone_type in ("hf_deberta_v2", "rope")


def test_snapshot_loaders_require_exact_keys():
    cfg = C.config_from_mapping(BASE)
    snap = C.asdict_without_private(cfg.train)
    again = C.load_train_config_snapshot(snap, source="test")
    assert again.max_steps == cfg.train.max_steps
    snap.pop("max_steps")
    with pytest.raises(ValueError):
        C.load_train_config_snapshot(snap, source="test")


def test_cli_dry_run_and_preset(tmp_path):
    cfg_path = _write(tmp_path, BASE)
    env = {"PYTHONPATH": str(REPO), "PATH": "/usr/bin:/bin", "CUDA_VISIBLE_DEVICES": ""}
    out = subprocess.run([sys.executable, "-m", "deberta_b200", "train", str(cfg_path), "--dry-run",
                          "--train.max_steps", "3", "--train.checkpoint.output_dir", str(tmp_path / "run")],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-1500:]
    assert not (tmp_path / "run" / "checkpoint-3").exists()
    parser = _build_main_parser()
    ns = parser.parse_args(["train", "--preset", "deberta-v3-base", "--dry-run"])
    assert ns.preset == "deberta-v3-base" and ns.dry_run


def test_readme_and_docs_commands_use_current_flags():
    """Every ``--section.key`` that the docs mention is a real config leaf."""
    import re

    leaves = {f"{sec}.{p}" for sec in ("model", "data", "train", "optim", "logging")
              for p, _ in C.iter_leaf_paths_for_dataclass(type(getattr(C.Config(), sec)))}
    texts = [REPO / "README.md"] + sorted((REPO / "docs").rglob("*.md"))
    texts = [t for t in texts if "api" not in t.parts]
    seen = set()
    for t in texts:
        seen |= set(re.findall(r"--((?:model|data|train|optim|logging)\.[a-z0-9_\.]+)", t.read_text()))
    unknown = sorted(s for s in seen if s not in leaves)
    assert not unknown, unknown
