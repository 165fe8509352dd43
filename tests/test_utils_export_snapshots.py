"""Scalar coercion, JSON/YAML snapshots, checkpoint payload layouts and export helpers.

Reference counterparts: ``tests/test_config_and_training_core.py`` (atomic JSON, data-state round trips, compile-key
remap with a sharded checkpoint written with ``no_dist=True``, snapshot validation), ``tests/test_export_cli.py`` and
``tests/test_export_artifacts.py`` (state-dict split, GDES merge, strict/partial load, staging/cleanup, README content).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path

import pytest
import torch
import yaml

from deberta_b200 import config as C
from deberta_b200 import run_layout as L
from deberta_b200.models import export_utils as X
from deberta_b200.training import run_config as RC
from deberta_b200.utils import checkpoint as CK
from deberta_b200.utils.io import dump_json, load_json_mapping
from deberta_b200.utils.mapping import flatten_mapping, leaf_paths
from deberta_b200.utils.paths import validate_existing_output_dir
from deberta_b200.utils.serialize import (asdict_without_private, coerce_dataclass_payload_types, drop_none_recursive,
                                          mapping_from_config_obj)
from deberta_b200.utils.types import coerce_scalar, parse_bool, unwrap_optional_type


# ---------------------------------------------------------------------------------------------- scalars
@pytest.mark.parametrize("raw,want", [("true", True), ("Yes", True), (" on ", True), ("0", False), ("F", False), (1, True),
                                      (0.0, False), (True, True)])
def test_parse_bool_accepts_common_spellings(raw, want):
    assert parse_bool(raw) is want


@pytest.mark.parametrize("raw", ["maybe", "2", "", 2, None])
def test_parse_bool_rejects_everything_else(raw):
    with pytest.raises(ValueError, match="Expected a boolean"):
        parse_bool(raw)


def test_parse_bool_can_refuse_numeric_spellings():
    with pytest.raises(ValueError):
        parse_bool("1", allow_numeric=False)
    assert parse_bool("true", allow_numeric=False) is True


def test_unwrap_optional_type():
    assert unwrap_optional_type(int | None) == (int, True)
    assert unwrap_optional_type(int) == (int, False)
    tp, opt = unwrap_optional_type(int | str | None)
    assert opt and tp == (int | str | None)


def test_coerce_scalar_matrix():
    assert coerce_scalar(" 12 ", int) == 12 and coerce_scalar("1e-3", float) == 1e-3 and coerce_scalar(5, str) == "5"
    assert coerce_scalar("none", int | None) is None and coerce_scalar("NULL", str | None) is None
    assert coerce_scalar("none", str) == "none"  # only optional fields understand "none"
    assert coerce_scalar(None, float | None) is None
    with pytest.raises(ValueError, match="null is not allowed"):
        coerce_scalar(None, int)
    with pytest.raises(ValueError, match="got bool"):
        coerce_scalar(True, int)
    with pytest.raises(ValueError, match="got bool"):
        coerce_scalar(False, float)
    with pytest.raises(ValueError):
        coerce_scalar("1.5", int)
    assert coerce_scalar("off", bool) is False
    assert coerce_scalar([1], list[int]) == [1]  # non-scalars pass through


# ---------------------------------------------------------------------------------------------- mappings
@dataclass
class _Inner:
    n: int = 1
    opt: float | None = None


@dataclass
class _Outer:
    name: str = "x"
    inner: _Inner = field(default_factory=_Inner)
    _cache: int = 0


def test_mapping_helpers():
    nested = {"a": {"b": 1, "c": {"d": None}}, "e": [1, 2]}
    assert flatten_mapping(nested) == {"a.b": 1, "a.c.d": None, "e": [1, 2]}
    assert leaf_paths(nested) == {"a.b", "a.c.d", "e"}
    assert asdict_without_private(_Outer()) == {"name": "x", "inner": {"n": 1, "opt": None}}
    assert drop_none_recursive(nested) == {"a": {"b": 1}, "e": [1, 2]}
    assert drop_none_recursive({"x": {"y": None}, "z": 0}) == {"z": 0}  # mappings emptied by the pruning go too
    assert mapping_from_config_obj(None) == {} and mapping_from_config_obj({"k": 1}) == {"k": 1}
    assert mapping_from_config_obj(_Outer())["inner"] == {"n": 1, "opt": None}

    class Bag:
        def __init__(self):
            self.a, self._b = 1, 2

    assert mapping_from_config_obj(Bag()) == {"a": 1}


def test_payload_types_are_coerced_against_the_dataclass():
    out = coerce_dataclass_payload_types(_Outer, {"name": 7, "inner": {"n": "3", "opt": "null"}, "extra": "kept"})
    assert out == {"name": "7", "inner": {"n": 3, "opt": None}, "extra": "kept"}


# ---------------------------------------------------------------------------------------------- JSON i/o
def test_dump_json_is_atomic_and_leaves_no_temp_files(tmp_path, monkeypatch):
    target = tmp_path / "deep" / "state.json"
    dump_json({"b": 1, "a": 2}, target)
    assert target.read_text().startswith('{\n  "a": 2') and load_json_mapping(target) == {"a": 2, "b": 1}
    # a failure while writing keeps the previous content and removes the temporary file
    monkeypatch.setattr(os, "replace", lambda *_a: (_ for _ in ()).throw(OSError("disk full")))
    with pytest.raises(OSError, match="disk full"):
        dump_json({"a": 3}, target)
    assert load_json_mapping(target) == {"a": 2, "b": 1}
    assert [p.name for p in target.parent.iterdir()] == ["state.json"]


def test_load_json_mapping_requires_an_object(tmp_path):
    p = tmp_path / "x.json"
    p.write_text("[1, 2]")
    with pytest.raises(ValueError, match="Expected a JSON object"):
        load_json_mapping(p)


def test_validate_existing_output_dir(tmp_path):
    validate_existing_output_dir(tmp_path / "new", overwrite=False, resuming=False)
    validate_existing_output_dir(tmp_path, overwrite=False, resuming=False)  # empty is fine
    (tmp_path / "f").write_text("x")
    with pytest.raises(ValueError, match="not empty"):
        validate_existing_output_dir(tmp_path, overwrite=False, resuming=False)
    validate_existing_output_dir(tmp_path, overwrite=True, resuming=False)
    validate_existing_output_dir(tmp_path, overwrite=False, resuming=True)
    with pytest.raises(ValueError, match="not a directory"):
        validate_existing_output_dir(tmp_path / "f", overwrite=True, resuming=False, what="logging_dir")


# ---------------------------------------------------------------------------------------------- run layout / snapshots
def _sections():
    return {"model": C.ModelConfig(backbone_type="rope"), "data": C.DataConfig(), "train": C.TrainConfig(),
            "optim": C.OptimConfig(), "logging": C.LoggingConfig()}


def test_run_layout_names_and_metadata_validation(tmp_path):
    assert L.infer_run_dir_from_checkpoint(tmp_path / "run" / "checkpoint-5") == (tmp_path / "run").resolve()
    with pytest.raises(ValueError, match="Missing run_metadata.json"):
        L.validate_run_metadata_file(tmp_path)
    dump_json(RC.build_run_metadata(), tmp_path / L.RUN_METADATA_FILE)
    meta = L.validate_run_metadata_file(tmp_path)
    assert meta["config_schema_version"] == RC.RUN_CONFIG_SCHEMA_VERSION and "deberta_version" in meta
    dump_json({"config_schema_version": RC.RUN_CONFIG_SCHEMA_VERSION + 1}, tmp_path / L.RUN_METADATA_FILE)
    with pytest.raises(ValueError):
        L.validate_run_metadata_file(tmp_path)
    dump_json({"deberta_version": "x"}, tmp_path / L.RUN_METADATA_FILE)
    with pytest.raises(ValueError):
        L.validate_run_metadata_file(tmp_path)


def test_run_metadata_records_optional_compile_scope():
    meta = RC.build_run_metadata(effective_compile_scope="backbones", compile_scope_reason="auto")
    assert meta["effective_compile_scope"] == "backbones" and meta["compile_scope_reason"] == "auto"
    assert "effective_compile_scope" not in RC.build_run_metadata()


def test_fresh_run_writes_all_snapshots(tmp_path):
    out, logs = tmp_path / "run", tmp_path / "run" / "logs"
    src = tmp_path / "cfg.yaml"
    src.write_text("# my comment\nmodel:\n  backbone_type: rope\n")
    RC.persist_or_validate_run_configs(output_dir=out, logging_dir=logs, sections=_sections(), config_path=src,
                                       resume_checkpoint=None, is_main_process=True)
    for name in (L.MODEL_CONFIG_FILE, L.DATA_CONFIG_FILE, L.TRAIN_CONFIG_FILE, L.OPTIM_CONFIG_FILE, L.LOGGING_CONFIG_FILE,
                 L.RUN_METADATA_FILE):
        assert (out / name).is_file(), name
    assert load_json_mapping(out / L.MODEL_CONFIG_FILE)["backbone_type"] == "rope"
    assert (logs / L.CONFIG_ORIGINAL_FILE).read_text().startswith("# my comment")  # the user's file, byte for byte
    resolved = yaml.safe_load((logs / L.CONFIG_RESOLVED_FILE).read_text())
    assert resolved["model"]["backbone_type"] == "rope" and set(resolved) == {"model", "data", "train", "optim", "logging"}
    # the snapshot loads back into an equal config object
    again = C.load_model_config_snapshot(load_json_mapping(out / L.MODEL_CONFIG_FILE), source="snap")
    assert asdict_without_private(again) == asdict_without_private(_sections()["model"])


def test_snapshots_without_a_config_file_and_from_json(tmp_path):
    RC.write_config_yaml_snapshots(logging_dir=tmp_path / "a", config_path=None, sections=_sections())
    assert yaml.safe_load((tmp_path / "a" / L.CONFIG_ORIGINAL_FILE).read_text())["model"]["backbone_type"] == "rope"
    js = tmp_path / "c.json"
    js.write_text(json.dumps({"train": {"max_steps": 3}}))
    RC.write_config_yaml_snapshots(logging_dir=tmp_path / "b", config_path=js, sections=_sections())
    assert yaml.safe_load((tmp_path / "b" / L.CONFIG_ORIGINAL_FILE).read_text()) == {"train": {"max_steps": 3}}


def test_non_main_rank_writes_no_snapshots(tmp_path):
    RC.persist_or_validate_run_configs(output_dir=tmp_path / "r", logging_dir=tmp_path / "r" / "logs", sections=_sections(),
                                       config_path=None, resume_checkpoint=None, is_main_process=False)
    assert not (tmp_path / "r").exists()


def test_resume_validates_stored_snapshots(tmp_path):
    out = tmp_path / "run"
    RC.persist_or_validate_run_configs(output_dir=out, logging_dir=out / "logs", sections=_sections(), config_path=None,
                                       resume_checkpoint=None, is_main_process=True)
    ck = out / "checkpoint-2"
    ck.mkdir()
    same = dict(output_dir=out, logging_dir=out / "logs", config_path=None, resume_checkpoint=str(ck), is_main_process=True)
    RC.persist_or_validate_run_configs(sections=_sections(), **same)
    assert not (out / L.RESUME_SOURCE_FILE).exists()  # same run directory: no provenance file
    changed = _sections()
    changed["model"] = C.ModelConfig(backbone_type="rope", hidden_size=512)
    with pytest.raises(ValueError, match="Resume config mismatch in model_config.json for fields: rope.hidden_size"):
        RC.persist_or_validate_run_configs(sections=changed, **same)
    # fields that cannot change the trajectory may differ
    inert = _sections()
    inert["data"] = C.DataConfig(shuffle_buffer_size=77)
    RC.persist_or_validate_run_configs(sections=inert, **same)
    # resuming into a new directory records where the state came from
    other = tmp_path / "continued"
    RC.persist_or_validate_run_configs(output_dir=other, logging_dir=other / "logs", sections=_sections(), config_path=None,
                                       resume_checkpoint=str(ck), is_main_process=True)
    prov = load_json_mapping(other / L.RESUME_SOURCE_FILE)
    assert prov["resume_checkpoint"] == str(ck.resolve()) and prov["source_run_dir"] == str(out.resolve())
    (out / L.OPTIM_CONFIG_FILE).unlink()
    with pytest.raises(ValueError, match="optim_config.json is missing"):
        RC.persist_or_validate_run_configs(sections=_sections(), **same)
    (out / L.RUN_METADATA_FILE).unlink()
    with pytest.raises(ValueError, match="run_metadata.json is missing"):
        RC.persist_or_validate_run_configs(sections=_sections(), **same)


def test_compare_resume_config_reports_added_removed_and_changed_paths():
    stored = {"a": {"x": 1, "y": 2}, "gone": 1}
    current = {"a": {"x": 1, "y": 3}, "new": 5}
    assert RC.compare_resume_config(section="train", stored=stored, current=current) == ["a.y", "gone", "new"]


# ---------------------------------------------------------------------------------------------- checkpoint payloads
def test_state_dict_keys_are_canonicalised():
    t = torch.zeros(1)
    assert set(CK.canonicalize_state_dict_keys({"_orig_mod.a.w": t, "b._orig_mod.w": t})) == {"a.w", "b.w"}
    assert set(CK.canonicalize_state_dict_keys({"model.a": t, "model.b": t})) == {"a", "b"}
    assert set(CK.canonicalize_state_dict_keys({"module._orig_mod.a": t})) == {"a"}
    assert set(CK.canonicalize_state_dict_keys({"model.a": t, "other": t})) == {"model.a", "other"}  # not shared: kept


def test_model_state_loads_from_every_supported_layout(tmp_path):
    state = {"generator.w": torch.arange(6.0).view(2, 3), "discriminator.w": torch.ones(4)}
    a = tmp_path / "safetensors"
    a.mkdir()
    tied = {"x": state["generator.w"], "y": state["generator.w"].t()}  # aliased and non-contiguous tensors are fine
    CK.save_model_state_dict({**state, **tied}, a)
    got = CK.load_model_state_dict(a)
    assert torch.equal(got["y"], state["generator.w"].t()) and torch.equal(got["discriminator.w"], state["discriminator.w"])
    for name in ("model.bin", "pytorch_model.bin"):
        d = tmp_path / name.replace(".", "_")
        d.mkdir()
        torch.save({f"_orig_mod.{k}": v for k, v in state.items()}, d / name)
        assert set(CK.load_model_state_dict(d)) == set(state)
    with pytest.raises(FileNotFoundError, match="No model weights found"):
        CK.load_model_state_dict(tmp_path)


def test_model_state_loads_from_a_sharded_directory_written_without_a_process_group(tmp_path):
    import torch.distributed.checkpoint as dcp

    state = {"generator.w": torch.arange(6.0).view(2, 3), "discriminator.b": torch.ones(4)}
    shard_dir = tmp_path / "pytorch_model_fsdp_0"
    dcp.save({"model": {f"_orig_mod.{k}": v for k, v in state.items()}}, storage_writer=dcp.FileSystemWriter(str(shard_dir)),
             no_dist=True)
    got = CK.load_model_state_dict(tmp_path)
    assert set(got) == set(state) and torch.equal(got["generator.w"], state["generator.w"])


def test_rng_state_round_trip():
    import random

    import numpy as np

    snap = CK.capture_rng_state()
    want = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    CK.restore_rng_state(snap)
    assert (random.random(), float(np.random.rand()), float(torch.rand(1))) == want


# ---------------------------------------------------------------------------------------------- export helpers
def test_exported_config_drops_training_only_keys(tmp_path):
    p = tmp_path / "config.json"
    dump_json({"hidden_size": 8, "hf_attention_kernel": "dynamic", "use_rmsnorm_heads": True, "mask_token_id": 4,
               "pad_token_id": 0}, p)
    X.clean_exported_config(p, strict=True)
    assert load_json_mapping(p) == {"hidden_size": 8, "pad_token_id": 0}
    X.clean_exported_config(tmp_path / "absent.json", strict=True)  # nothing to do
    p.write_text("{broken")
    X.clean_exported_config(p, strict=False)
    with pytest.raises(ValueError, match="Failed to parse exported config"):
        X.clean_exported_config(p, strict=True)


def test_export_readme_and_licence(tmp_path):
    X.write_export_readme(tmp_path, what="discriminator", backbone_type="hf_deberta_v2", embedding_sharing="gdes", step=1200,
                          tokenizer_name="microsoft/deberta-v3-base")
    text = (tmp_path / "README.md").read_text()
    assert text.startswith("---\nlicense: mit") and "training step: 1200" in text and "`gdes`" in text
    assert "AutoModel.from_pretrained" in text and "microsoft/deberta-v3-base" in text
    assert (tmp_path / "LICENSE").read_text().startswith("MIT License")
    X.write_export_readme(tmp_path, what="generator", backbone_type="rope", embedding_sharing="none", step=None, tokenizer_name="t")
    text = (tmp_path / "README.md").read_text()
    assert "training step: unknown" in text and "DebertaRoPEModel.from_pretrained" in text


def test_pretrainer_state_is_split_by_branch():
    t = torch.zeros(1)
    disc, gen = X.split_pretrainer_state_dict({"discriminator.encoder.w": t, "generator.encoder.w": t, "generator_lm_head.w": t,
                                               "rtd_head.w": t})
    assert set(disc) == {"encoder.w"} and set(gen) == {"encoder.w"}


def test_intersection_load_strict_and_partial():
    model = torch.nn.Linear(3, 2)
    full = {"weight": torch.ones(2, 3), "bias": torch.zeros(2)}
    assert X.load_intersection_state_dict(model, full, strict=True) == ([], [])
    assert torch.equal(model.weight.data, torch.ones(2, 3))
    with pytest.raises(RuntimeError, match="Strict export failed: missing=\\['bias'\\] unexpected=\\['extra'\\]"):
        X.load_intersection_state_dict(model, {"weight": full["weight"], "extra": torch.zeros(1)}, strict=True)
    missing, unexpected = X.load_intersection_state_dict(model, {"weight": full["weight"] * 2, "extra": torch.zeros(1)}, strict=False)
    assert (missing, unexpected) == (["bias"], ["extra"]) and float(model.weight.data[0, 0]) == 2.0
    assert X.load_intersection_state_dict(model, {**full, "opt.step": torch.zeros(1)}, strict=True,
                                          ignore_unexpected=(".step",)) == ([], [])
    with pytest.raises(RuntimeError, match="Shape mismatch"):
        X.load_intersection_state_dict(model, {"weight": torch.ones(3, 3), "bias": full["bias"]}, strict=False)


class _Emb(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.embeddings = torch.nn.Module()
        self.embeddings.word_embeddings = torch.nn.Embedding(5, 4)
        self.embeddings.position_embeddings = torch.nn.Embedding(3, 4)


def test_embedding_merge_for_shared_and_delta_modes():
    gen = {"embeddings.word_embeddings.weight": torch.full((5, 4), 2.0), "embeddings.position_embeddings.weight": torch.ones(3, 4)}
    disc = {"embeddings.word_embeddings.bias": torch.full((5, 4), 0.5), "embeddings.position_embeddings.bias": torch.zeros(3, 4)}
    m = _Emb()
    X.merge_embeddings_into_export_backbone(export_model=m, disc_sd=disc, gen_sd=gen, mode="gdes")
    assert torch.equal(m.embeddings.word_embeddings.weight.data, torch.full((5, 4), 2.5))
    m = _Emb()
    X.merge_embeddings_into_export_backbone(export_model=m, disc_sd={}, gen_sd=gen, mode="es")
    assert torch.equal(m.embeddings.word_embeddings.weight.data, torch.full((5, 4), 2.0))
    m = _Emb()
    before = m.embeddings.word_embeddings.weight.data.clone()
    X.merge_embeddings_into_export_backbone(export_model=m, disc_sd=disc, gen_sd=gen, mode="none")
    assert torch.equal(m.embeddings.word_embeddings.weight.data, before)
    with pytest.raises(RuntimeError, match="Missing discriminator bias"):
        X.merge_embeddings_into_export_backbone(export_model=_Emb(), disc_sd={}, gen_sd=gen, mode="gdes")


def test_delta_merge_accumulates_in_fp32():
    gen = {"embeddings.word_embeddings.weight": torch.full((5, 4), 256.0, dtype=torch.bfloat16)}
    disc = {"embeddings.word_embeddings.bias": torch.full((5, 4), 1.0, dtype=torch.bfloat16)}
    m = _Emb()
    X.merge_embeddings_into_export_backbone(export_model=m, disc_sd=disc, gen_sd=gen, mode="gdes", fp32_accumulate=True)
    assert float(m.embeddings.word_embeddings.weight.data[0, 0]) == 257.0  # bf16 arithmetic would give 256 or 258


def test_export_cli_arguments_and_failures(tmp_path):
    import argparse

    from deberta_b200 import export_cli as E

    parser = argparse.ArgumentParser()
    E.add_export_arguments(parser)
    cfg = E.namespace_to_export_config(parser.parse_args(["ck", "--what", "both", "--no-safe-serialization",
                                                          "--embedding-sharing", "es", "--allow-partial-export"]))
    assert (cfg.checkpoint_dir, cfg.export_what, cfg.safe_serialization, cfg.embedding_sharing, cfg.allow_partial_export) == \
        ("ck", "both", False, "es", True)
    assert E.namespace_to_export_config(parser.parse_args(["ck"])).export_what == "discriminator"
    with pytest.raises(SystemExit):
        parser.parse_args(["ck", "--what", "everything"])
    with pytest.raises(FileNotFoundError, match="Checkpoint directory not found"):
        E.run_export(E.ExportConfig(checkpoint_dir=str(tmp_path / "nope")))
    ck = tmp_path / "run" / "checkpoint-1"
    ck.mkdir(parents=True)
    with pytest.raises(ValueError, match="Missing run_metadata.json"):
        E.run_export(E.ExportConfig(checkpoint_dir=str(ck)))
