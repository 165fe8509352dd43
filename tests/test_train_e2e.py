"""End-to-end CPU runs through the public CLI: train → checkpoint → resume → export, and 2-rank gloo runs."""

from __future__ import annotations

import json
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
CFG = ROOT / "configs" / "tiny_cpu_smoke_synthetic.yaml"


def _train(args: list[str], env: dict | None = None, nproc: int = 1, port: int = 29611, cfg: Path | None = None) -> subprocess.CompletedProcess:
    base = [sys.executable]
    if nproc > 1:
        base += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
                 "--master-port", str(port)]
        base += ["-m", "deberta_b200"]
    else:
        base += ["-m", "deberta_b200"]
    e = dict(os.environ, DEBERTA_FAST_EXIT_AFTER_TRAIN="0", PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    e.update(env or {})
    return subprocess.run(base + ["train", str(cfg or CFG), *args], capture_output=True, text=True, cwd=ROOT, env=e, timeout=600)


def test_train_resume_export(tmp_path):
    out = tmp_path / "run"
    common = ["--train.checkpoint.output_dir", str(out), "--train.checkpoint.save_steps", "2", "--logging.logging_steps", "1",
              "--train.checkpoint.save_total_limit", "2", "--logging.debug.metrics", "true"]
    r = _train([*common, "--train.max_steps", "4", "--train.checkpoint.export_hf_final", "false"])
    assert r.returncode == 0, r.stderr[-3000:]
    assert (out / "checkpoint-4" / ".complete").read_text() == "ok\n"
    assert sorted(p.name for p in out.glob("checkpoint-*")) == ["checkpoint-2", "checkpoint-4"]
    state = json.loads((out / "checkpoint-4" / "data_state.json").read_text())
    assert state["global_step"] == 4 and state["consumed_micro_batches"] == 4 and state["gradient_accumulation_steps"] == 1
    assert set(state["optimizer_param_digest"]) == {"generator", "discriminator"}
    assert json.loads((out / "run_metadata.json").read_text())["config_schema_version"] == 4
    for name in ("model", "data", "train", "optim", "logging"):
        assert (out / f"{name}_config.json").exists()
    assert (out / "logs" / "config_original.yaml").exists() and (out / "logs" / "config_resolved.yaml").exists()
    # resume: overwrite must be off, output dir is reused
    r = _train([*common, "--train.max_steps", "6", "--train.checkpoint.overwrite_output_dir", "false",
                "--train.checkpoint.resume_from_checkpoint", "auto"])
    assert r.returncode == 0, r.stderr[-3000:]
    assert "Resumed from" in r.stderr and (out / "checkpoint-6" / ".complete").exists()
    assert sorted(p.name for p in out.glob("checkpoint-*")) == ["checkpoint-4", "checkpoint-6"]  # rotation keeps 2
    hf = out / "final_hf"
    assert (hf / "model.safetensors").exists() and (hf / "README.md").exists() and (hf / "export_meta.json").exists()
    cfg = json.loads((hf / "config.json").read_text())
    assert "use_rmsnorm_heads" not in cfg and cfg["model_type"] == "deberta-rope"
    # the exported backbone loads and its word embeddings are generator table + discriminator delta
    from safetensors.torch import load_file

    from deberta_b200.models import DebertaRoPEModel

    model = DebertaRoPEModel.from_pretrained(str(hf))
    ck = load_file(str(out / "checkpoint-6" / "model.safetensors"))
    want = ck["generator.embeddings.word_embeddings.weight"] + ck["discriminator.embeddings.word_embeddings.bias"]
    torch.testing.assert_close(model.embeddings.word_embeddings.weight.data, want)
    # a resume with a changed model must be refused
    r = _train([*common, "--train.max_steps", "8", "--train.checkpoint.overwrite_output_dir", "false",
                "--train.checkpoint.resume_from_checkpoint", "auto", "--model.rope.num_hidden_layers", "3"])
    assert r.returncode != 0 and "Resume config mismatch" in r.stderr


@pytest.mark.parametrize("parallelism", ["ddp", "zero", "fsdp"])
def test_two_rank_gloo_matches_layout(tmp_path, parallelism):
    out = tmp_path / f"run_{parallelism}"
    r = _train(["--train.checkpoint.output_dir", str(out), "--train.max_steps", "3", "--train.checkpoint.save_steps", "0",
                "--train.checkpoint.export_hf_final", "false", "--train.gradient_accumulation_steps", "2",
                "--logging.logging_steps", "1", "--train.distributed.parallelism", parallelism], nproc=2,
               port=29611 + ["ddp", "zero", "fsdp"].index(parallelism))
    assert r.returncode == 0, r.stderr[-3000:]
    ck = out / "checkpoint-3"
    assert (ck / ".complete").exists()
    names = {p.name for p in ck.iterdir()}
    # the model: one safetensors file, or (full shard) a distributed-checkpoint directory all ranks wrote into
    assert ("pytorch_model_fsdp_0" in names and (ck / "pytorch_model_fsdp_0" / ".metadata").exists()) if parallelism == "fsdp" \
        else "model.safetensors" in names
    # optimizer state is whole and in torch.optim layout whatever the sharding was
    assert {"optimizer.bin", "optimizer_1.bin"} <= names and not any(n.startswith("optimizer_shard") for n in names)
    sd = torch.load(ck / "optimizer_1.bin", map_location="cpu", weights_only=False)
    assert len(sd["param_groups"]) == 2 and sd["param_groups"][1]["weight_decay"] == 0.0
    assert sd["state"] and all(set(v) == {"step", "exp_avg", "exp_avg_sq"} for v in sd["state"].values())
    assert {"random_states_0.pkl", "random_states_1.pkl"} <= names
    assert "step 3" in r.stderr
    losses = [float(m) for m in re.findall(r"step \d+ \| loss ([0-9.]+)", r.stderr)]
    assert len(losses) == 3
    _TWO_RANK_LOSSES[parallelism] = losses
    if len(_TWO_RANK_LOSSES) > 1:  # replicated, sharded-optimizer and full-shard runs are the same computation
        ref = next(iter(_TWO_RANK_LOSSES.values()))
        for other in _TWO_RANK_LOSSES.values():
            assert all(abs(a - b) < 2e-4 * max(1.0, abs(a)) for a, b in zip(ref, other)), _TWO_RANK_LOSSES


_TWO_RANK_LOSSES: dict[str, list[float]] = {}


def test_resume_with_another_rank_count_and_mode(tmp_path):
    """A checkpoint written by two full-shard ranks resumes in one replicated process (and the other way round the
    optimizer moments are sliced again): the run continues from the same step with finite losses."""
    out = tmp_path / "run"
    common = ["--train.checkpoint.output_dir", str(out), "--train.checkpoint.export_hf_final", "false",
              "--train.gradient_accumulation_steps", "2", "--logging.logging_steps", "1", "--train.checkpoint.save_steps", "2"]
    r = _train([*common, "--train.max_steps", "2", "--train.distributed.parallelism", "fsdp"], nproc=2, port=29621)
    assert r.returncode == 0, r.stderr[-3000:]
    resume = ["--train.checkpoint.resume_from_checkpoint", "auto", "--train.checkpoint.overwrite_output_dir", "false"]
    r = _train([*common, "--train.max_steps", "3", "--train.distributed.parallelism", "ddp", *resume])
    assert r.returncode == 0, r.stderr[-3000:]
    assert "Resumed from" in r.stderr and "step 3 |" in r.stderr and (out / "checkpoint-3" / "model.safetensors").exists()
    sd = torch.load(out / "checkpoint-3" / "optimizer.bin", map_location="cpu", weights_only=False)
    assert int(float(next(iter(sd["state"].values()))["step"])) == 3
    r = _train([*common, "--train.max_steps", "4", "--train.distributed.parallelism", "zero", *resume], nproc=2, port=29622)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "step 4 |" in r.stderr


def test_dry_run_reports_batch_shape(tmp_path, capsys):
    from deberta_b200.cli import main

    main(["train", str(CFG), "--dry-run", "--train.checkpoint.output_dir", str(tmp_path / "never")])
    text = capsys.readouterr().out
    assert "Dry-run preflight OK" in text and "sample_batch_shape=(4, 128)" in text
    assert not (tmp_path / "never").exists()


@pytest.mark.parametrize("nproc", [1, 2])
def test_tiny_hf_deberta_v2_smoke_config_trains(tmp_path, nproc):
    """The 2-layer / 64-wide DeBERTa-v2 family model with the 128 100-entry vocabulary: one process, and two gloo ranks."""
    cfg = ROOT / "configs" / "tiny_cpu_smoke_hf_deberta_v2.yaml"
    r = _train(["--train.checkpoint.output_dir", str(tmp_path / "run"), "--train.max_steps", "3"], nproc=nproc, port=29631,
               cfg=cfg)
    assert r.returncode == 0, r.stderr[-3000:]
    rows = re.findall(r"step (\d+) \| loss ([0-9.]+) \| gen ([0-9.]+) \| disc ([0-9.]+)", r.stderr)
    assert [int(x[0]) for x in rows] == [1, 2, 3]
    gen = [float(x[2]) for x in rows]
    assert all(11.0 < g < 12.5 for g in gen)  # ln(128100) = 11.76 at initialisation
    assert abs(float(rows[0][1]) - (float(rows[0][2]) + 50.0 * float(rows[0][3]))) < 2e-3 * float(rows[0][1])  # loss = gen + 50 disc


def test_hf_deberta_v2_checkpoint_exports_with_stock_transformers_classes(tmp_path):
    """``deberta export`` on a GDES checkpoint of the DeBERTa-v2 family, strict mode, both components: the artifacts load
    with ``transformers.AutoModel`` and the discriminator's word embeddings are generator table + delta (the checkpoint
    itself only holds ``base_weight`` / ``bias`` for shared tables, and the pretrainer's absolute-position table, which
    the stock backbone does not have, is not an unexpected key)."""
    cfg = ROOT / "configs" / "tiny_cpu_smoke_hf_deberta_v2.yaml"
    out = tmp_path / "run"
    r = _train(["--train.checkpoint.output_dir", str(out), "--train.max_steps", "2", "--train.checkpoint.save_steps", "2",
                "--train.checkpoint.export_hf_final", "false"], cfg=cfg)
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    exp = tmp_path / "exported"
    r = subprocess.run([sys.executable, "-m", "deberta_b200", "export", str(out / "checkpoint-2"), "--what", "both",
                        "--output-dir", str(exp)], capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    from safetensors.torch import load_file
    from transformers import AutoModel

    disc = AutoModel.from_pretrained(str(exp / "discriminator"))
    gen = AutoModel.from_pretrained(str(exp / "generator"))
    ck = load_file(str(out / "checkpoint-2" / "model.safetensors"))
    want = ck["generator.embeddings.word_embeddings.weight"].float() + ck["discriminator.embeddings.word_embeddings.bias"].float()
    torch.testing.assert_close(disc.embeddings.word_embeddings.weight.data.float(), want)
    torch.testing.assert_close(gen.embeddings.word_embeddings.weight.data, ck["generator.embeddings.word_embeddings.weight"])
    meta = json.loads((exp / "export_meta.json").read_text())
    assert meta["components"]["discriminator"]["unexpected_keys"] == [] and meta["components"]["discriminator"]["missing_keys"] == []
