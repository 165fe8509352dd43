"""Metric sinks, tracker fan-out with fake backends, and the final-export subprocess hook.

Reference counterparts: tracker / W&B fakes and crash handling in ``tests/test_config_and_training_core.py:1241-1444``,
the final-export subprocess check in ``tests/test_config_and_training_resume.py``.
"""

from __future__ import annotations

import gzip
import json
import subprocess
import sys
import types
from pathlib import Path

import pytest

from deberta_b200 import config as C
from deberta_b200.training import export_helpers, metrics, tracker_utils
from deberta_b200.utils.io import load_json_mapping


class FakeRun:
    def __init__(self):
        self.logged, self.saved, self.summary, self.finished = [], [], {}, None

    def log(self, values, step):
        self.logged.append((step, dict(values)))

    def save(self, path, policy="now"):
        self.saved.append((path, policy))

    def finish(self, exit_code=0):
        self.finished = exit_code


class FakeWriter:
    def __init__(self):
        self.scalars, self.closed = [], False

    def add_scalar(self, key, value, step):
        self.scalars.append((key, value, step))

    def flush(self):
        pass

    def close(self):
        self.closed = True


def _fake_wandb(monkeypatch, fail_init=False):
    mod = types.ModuleType("wandb")
    mod.inits, mod.watched = [], []
    run = FakeRun()

    def init(**kw):
        if fail_init:
            raise RuntimeError("no network")
        mod.inits.append(kw)
        return run

    mod.init = init
    mod.watch = lambda model, log, log_freq: mod.watched.append((log, log_freq))
    monkeypatch.setitem(sys.modules, "wandb", mod)
    return mod, run


# ---------------------------------------------------------------------------------------------- metrics
def test_metrics_rows_append_as_gzip_members(tmp_path):
    path = tmp_path / "logs" / "metrics.jsonl.gz"
    metrics.append_metrics_jsonl_row(path, {"step": 1, "loss": 2.5})
    metrics.append_metrics_jsonl_row(path, {"step": 2, "loss": float("nan"), "b": 1})
    with gzip.open(path, "rt") as f:
        rows = [json.loads(line) for line in f]
    assert [r["step"] for r in rows] == [1, 2] and rows[0]["loss"] == 2.5
    assert rows[1]["loss"] != rows[1]["loss"]  # NaN survives the round trip
    assert list(rows[1]) == sorted(rows[1])  # keys are sorted, so rows diff cleanly


def test_nonfinite_debug_artifact(tmp_path):
    p = metrics.write_nonfinite_debug_artifact(debug_dir=tmp_path / "debug", step=12, what="generator",
                                               losses={"gen": float("inf")}, lrs={"generator": 1e-4}, lr_mult=0.5,
                                               extra={"skip_streak": 2})
    assert p.name == "nonfinite_step_12_generator.json"
    raw = load_json_mapping(p)
    assert raw["step"] == 12 and raw["lr_mult"] == 0.5 and raw["skip_streak"] == 2 and len(raw["rng"]["torch_cpu"]) == 8


def test_flush_loggers_tolerates_broken_handlers():
    import logging

    class Broken(logging.Handler):
        def flush(self):
            raise OSError("closed")

    h = Broken()
    logging.getLogger().addHandler(h)
    try:
        metrics.flush_loggers()
    finally:
        logging.getLogger().removeHandler(h)


# ---------------------------------------------------------------------------------------------- trackers
def test_tracker_set_fans_out_and_refuses_steps_that_go_backwards():
    ts = tracker_utils.TrackerSet()
    ts.tb, ts.wandb_run = FakeWriter(), FakeRun()
    ts.log({"loss": 1.0, "note": "text"}, 5)
    ts.log({"loss": 0.9}, 3)  # e.g. a crash row written after a resume
    ts.log({"loss": 0.8}, 5)
    assert ts.tb.scalars == [("loss", 1.0, 5), ("loss", 0.8, 5)]  # only numbers reach TensorBoard
    assert [s for s, _ in ts.wandb_run.logged] == [5, 5]
    ts.finish(crashed=True)
    assert ts.tb.closed and ts.wandb_run.finished == 1 and ts.wandb_run.summary["crashed"] is True


def test_trackers_exist_on_the_main_process_only(tmp_path, monkeypatch):
    mod, run = _fake_wandb(monkeypatch)
    cfg = _with_wandb(C.LoggingConfig(backend="none", project_name="proj"))
    off = tracker_utils.init_trackers(logging_cfg=cfg, logging_dir=tmp_path, run_name="r", config_payload={}, is_main_process=False)
    assert off.wandb_run is None and off.tb is None and mod.inits == []
    on = tracker_utils.init_trackers(logging_cfg=cfg, logging_dir=tmp_path, run_name="r", config_payload={"a": 1}, is_main_process=True)
    assert on.wandb_run is run and mod.inits[0]["project"] == "proj" and mod.inits[0]["name"] == "r" and mod.inits[0]["config"] == {"a": 1}
    on.finish()
    assert run.finished == 0


def _with_wandb(cfg):
    import dataclasses

    return dataclasses.replace(cfg, wandb=dataclasses.replace(cfg.wandb, enabled=True))


def test_wandb_failures_degrade_to_no_tracker(tmp_path, monkeypatch):
    _fake_wandb(monkeypatch, fail_init=True)
    cfg = _with_wandb(C.LoggingConfig(backend="none"))
    ts = tracker_utils.init_trackers(logging_cfg=cfg, logging_dir=tmp_path, run_name=None, config_payload={}, is_main_process=True)
    assert ts.wandb_run is None
    ts.log({"x": 1}, 1)  # a tracker set without backends is inert
    ts.finish()


def test_wandb_watch_and_config_upload(tmp_path, monkeypatch):
    mod, run = _fake_wandb(monkeypatch)
    ts = tracker_utils.TrackerSet()
    assert not tracker_utils.setup_wandb_watch(tracker=ts, model=object(), watch_mode="all", log_freq=10)  # W&B not active
    ts.wandb_run = run
    assert not tracker_utils.setup_wandb_watch(tracker=ts, model=object(), watch_mode="none", log_freq=10)
    assert tracker_utils.setup_wandb_watch(tracker=ts, model=object(), watch_mode=" Gradients ", log_freq=7)
    assert mod.watched == [("gradients", 7)]
    present = tmp_path / "config_resolved.yaml"
    present.write_text("a: 1\n")
    n = tracker_utils.upload_wandb_config_files(tracker=ts, files=[present, tmp_path / "absent.yaml"])
    assert n == 1 and run.saved == [(str(present), "now")]
    assert tracker_utils.upload_wandb_config_files(tracker=tracker_utils.TrackerSet(), files=[present]) == 0


# ---------------------------------------------------------------------------------------------- final export hook
def test_final_export_runs_the_cli_in_a_subprocess(tmp_path, monkeypatch):
    calls = []

    def fake_run(cmd, capture_output, text, timeout):
        calls.append((cmd, timeout))
        return subprocess.CompletedProcess(cmd, 0, "", "")

    monkeypatch.setattr(export_helpers.subprocess, "run", fake_run)
    ok = export_helpers.export_discriminator_hf_subprocess(checkpoint_dir=tmp_path / "checkpoint-9", output_dir=tmp_path / "final_hf",
                                                           timeout_s=30.0)
    cmd, timeout = calls[0]
    assert ok and timeout == 30.0 and cmd[0] == sys.executable and cmd[1:4] == ["-m", "deberta_b200", "export"]
    assert cmd[4] == str(tmp_path / "checkpoint-9") and cmd[cmd.index("--what") + 1] == "discriminator"
    assert cmd[cmd.index("--output-dir") + 1] == str(tmp_path / "final_hf") and "--allow-partial-export" in cmd


def test_final_export_failures_do_not_raise(tmp_path, monkeypatch):
    monkeypatch.setattr(export_helpers.subprocess, "run",
                        lambda cmd, **kw: subprocess.CompletedProcess(cmd, 2, "", "Traceback: boom"))
    assert not export_helpers.export_discriminator_hf_subprocess(checkpoint_dir=tmp_path, output_dir=tmp_path / "o")

    def explode(cmd, **kw):
        raise subprocess.TimeoutExpired(cmd, 1.0)

    monkeypatch.setattr(export_helpers.subprocess, "run", explode)
    assert not export_helpers.export_discriminator_hf_subprocess(checkpoint_dir=tmp_path, output_dir=tmp_path / "o", timeout_s=1.0)
