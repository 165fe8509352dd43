"""The benchmark script's contract, as far as it can be checked without a GPU: flags, defaults, the synthetic batches it
feeds to both arms, the configuration it builds, and the reference arm's one-line answer on a machine without CUDA."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(REPO))
import bench  # noqa: E402


def _args(*argv):
    old = sys.argv
    sys.argv = ["bench.py", *argv]
    try:
        return bench.parse_args()
    finally:
        sys.argv = old


def test_defaults_name_the_headline_configuration():
    a = _args()
    assert (a.gpus, a.impl, a.backbone, a.model_size, a.parallelism) == (1, "ours", "hf_deberta_v2", "base", "zero")
    assert a.micro_batch == 32 and a.seq_len == 512 and a.warmup >= 3 and a.steps >= 1 and not a.block_docs
    b = _args("--gpus", "8", "--steps", "20", "--warmup", "5", "--impl", "reference")
    assert (b.gpus, b.steps, b.warmup, b.impl) == (8, 20, 5, "reference")


def test_synthetic_batches_come_from_the_real_packer_and_collator():
    batches = bench.synthetic_batches(2, 3, 128, seed=7, pin=False)
    assert len(batches) == 2
    for b in batches:
        assert b["input_ids"].shape == (3, 128) and b["labels"].shape == (3, 128) and "doc_ids" not in b
        picked = b["labels"].ne(-100)
        assert 0 < int(picked.sum()) <= 3 * 20 and bool((b["input_ids"][picked] == 4).all())  # 15 % budget, all [MASK]
        assert bool((b["input_ids"][:, 0] == 1).all())
    again = bench.synthetic_batches(2, 3, 128, seed=7, pin=False)
    assert all(torch.equal(x["input_ids"], y["input_ids"]) for x, y in zip(batches, again))  # seeded: both arms see the same data
    other = bench.synthetic_batches(1, 3, 128, seed=8, pin=False)
    assert not torch.equal(other[0]["input_ids"], batches[0]["input_ids"])  # each rank (seed) has its own stream


def test_block_docs_batches_carry_document_ids():
    b = bench.synthetic_batches(1, 2, 256, seed=3, pin=False, block_docs=True)[0]
    doc = b["doc_ids"]
    assert doc.shape == (2, 256) and int(doc.min()) >= 0 and int(doc.max()) >= 2
    assert bool((doc[:, 1:] >= doc[:, :-1]).logical_or(doc[:, 1:] == 0).all())  # ids grow along a row, 0 marks padding


@pytest.mark.parametrize("backbone", ["hf_deberta_v2", "rope"])
def test_benchmark_configuration_is_the_published_recipe(backbone):
    cfg = bench.build_config(_args("--backbone", backbone, "--seq-len", "512"))
    assert cfg.model.backbone_type == backbone and cfg.model.embedding_sharing == "gdes"
    assert cfg.train.mixed_precision == "bf16" and cfg.train.decoupled_training is True
    assert cfg.train.per_device_train_batch_size == 32 and cfg.train.gradient_accumulation_steps == 8
    # the RTD weight follows the profile default of the backbone (10 for DeBERTa-v2, 50 for rope)
    assert cfg.train.objective.disc_loss_weight == (10.0 if backbone == "hf_deberta_v2" else 50.0)
    assert cfg.train.objective.mask_token_prob == 1.0
    assert cfg.optim.lr.base == 2e-4 and cfg.optim.adam.beta2 == 0.98 and cfg.data.packing.max_seq_length == 512
    if backbone == "hf_deberta_v2":
        assert cfg.model.hf.model_size == "base" and cfg.model.profile == "deberta_v3_parity"


def test_reference_arm_answers_in_one_json_line_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without CUDA")
    res = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference"], capture_output=True, text=True,
                         timeout=600, cwd=str(REPO))
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def test_own_arm_refuses_to_run_on_cpu():
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without CUDA")
    res = subprocess.run([sys.executable, str(REPO / "bench.py"), "--steps", "1", "--warmup", "1"], capture_output=True, text=True,
                         timeout=600, cwd=str(REPO))
    assert res.returncode != 0 and "needs a CUDA device" in (res.stderr + res.stdout)  # never a silent CPU number
