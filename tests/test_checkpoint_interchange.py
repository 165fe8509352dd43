"""Checkpoints written here are read by the reference's own loaders and by ``torch.optim.AdamW`` built the reference's
way; optimizer state survives a change of sharding."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from deberta_b200 import config as C
from deberta_b200.parallel.dist import DistContext
from deberta_b200.parallel.engine import TrainEngine
from deberta_b200.utils.checkpoint import load_training_state, save_training_state

from ._ref import import_reference
from .test_rtd_parity import _batch, _build


class _Trainer:
    """The slice of the trainer a checkpoint touches."""

    def __init__(self, engine):
        self.engine, self.global_step = engine, 2

    def resolve_pending(self):
        pass

    def state_dict(self):
        return {"global_step": self.global_step, "schedules": {n: {"last_step": 2} for n in self.engine.optimizers}}

    def load_state_dict(self, s):
        self.global_step = int(s["global_step"])


def _train_two_steps(engine, model):
    ids, labels, mask = _batch()
    for _ in range(2):
        engine.zero_grad()
        gen = model(input_ids=ids, attention_mask=mask, labels=labels, phase="generator")
        gen.gen_loss_raw.backward()
        disc = model(input_ids=ids, corrupted_input_ids=gen.corrupted_input_ids, disc_labels=gen.disc_labels,
                     attention_mask=mask, phase="discriminator")
        disc.disc_loss_raw.backward()
        for name in engine.optimizers:
            engine.sync_grads(name)
            engine.step(name, lr_scale=1.0, max_grad_norm=1.0)


@pytest.mark.parametrize("backbone", ["hf", "rope"])
def test_reference_loaders_accept_our_checkpoint(tmp_path: Path, backbone):
    ref_pkg = import_reference()
    from deberta.training.runtime import _build_decoupled_optimizers
    from deberta.utils.checkpoint import load_checkpoint_model_state_dict

    ref, ours = _build(backbone, "gdes")
    engine = TrainEngine(ours, DistContext(), compute_dtype=torch.float32, parallelism="ddp", decoupled=True,
                         lr_generator=1e-3, lr_discriminator=2e-3, weight_decay=0.01, betas=(0.9, 0.98), eps=1e-6)
    _train_two_steps(engine, ours)
    save_training_state(tmp_path, engine=engine, trainer=_Trainer(engine), ctx=DistContext())
    # ---- model weights through the reference's loader into the reference's model ----
    state = load_checkpoint_model_state_dict(tmp_path)
    missing, unexpected = ref.load_state_dict(state, strict=True)
    assert not missing and not unexpected
    want = engine.model_state_dict()
    for k, v in ref.state_dict().items():
        torch.testing.assert_close(v, want[k])
    # ---- optimizer files into AdamW objects built by the reference's own builder ----
    train_cfg = ref_pkg.config.TrainConfig(decoupled_training=True, mixed_precision="no")
    for name, value in (("learning_rate", 1e-3), ("generator_learning_rate", 1e-3), ("discriminator_learning_rate", 2e-3),
                        ("weight_decay", 0.01), ("adam_beta1", 0.9), ("adam_beta2", 0.98), ("adam_epsilon", 1e-6)):
        object.__setattr__(train_cfg, name, value)
    gen_opt, disc_opt = _build_decoupled_optimizers(ref, train_cfg, mixed_precision="no")
    for opt, fname, ours_name in ((gen_opt, "optimizer.bin", "generator"), (disc_opt, "optimizer_1.bin", "discriminator")):
        sd = torch.load(tmp_path / fname, map_location="cpu", weights_only=False)
        assert [len(g["params"]) for g in sd["param_groups"]] == [len(g["params"]) for g in opt.param_groups]
        opt.load_state_dict({"state": sd["state"], "param_groups": sd["param_groups"]})
        o = engine.optimizers[ours_name]
        flat = [p for g in opt.param_groups for p in g["params"]]
        assert len(flat) == len(o.names)
        by_name = dict(ref.named_parameters())
        order = [n for seg in o.segments for n in o.names if seg.start <= engine.layout[n][0] < seg.end]
        for p, n in zip(flat, order):  # the i-th parameter of the reference's optimizer is the i-th of ours
            assert p is by_name[n], n
            off, cnt, shape = engine.layout[n]
            torch.testing.assert_close(opt.state[p]["exp_avg"], o.exp_avg[off - o.start: off - o.start + cnt].view(shape))
            assert int(opt.state[p]["step"]) == 2
        assert opt.param_groups[1]["weight_decay"] == 0.0 and opt.param_groups[0]["weight_decay"] == 0.01


def test_optimizer_state_round_trip_is_exact_and_reshards(tmp_path: Path):
    _, ours = _build("rope", "gdes")
    ctx = DistContext()
    engine = TrainEngine(ours, ctx, compute_dtype=torch.float32, parallelism="ddp", decoupled=True)
    _train_two_steps(engine, ours)
    save_training_state(tmp_path, engine=engine, trainer=_Trainer(engine), ctx=ctx)
    _, other = _build("rope", "gdes")
    eng2 = TrainEngine(other, ctx, compute_dtype=torch.float32, parallelism="fsdp", decoupled=True)
    load_training_state(tmp_path, engine=eng2, trainer=_Trainer(eng2), ctx=ctx)
    assert torch.equal(eng2.master, engine.master)
    for name, o in engine.optimizers.items():
        o2 = eng2.optimizers[name]
        assert o2.step == o.step == 2 and torch.equal(o2.exp_avg, o.exp_avg) and torch.equal(o2.exp_avg_sq, o.exp_avg_sq)
    # a rank that owns the second half of every range keeps exactly that slice of the saved moments
    states = engine.torch_optimizer_state_dicts()
    o = eng2.optimizers["discriminator"]
    half = (o.end - o.start) // 2
    keep_m = o.exp_avg.clone()
    o.shard = (o.start + half, o.end)
    o.exp_avg, o.exp_avg_sq = torch.zeros(o.end - o.start - half), torch.zeros(o.end - o.start - half)
    eng2.load_torch_optimizer_state_dicts(states)
    assert torch.equal(o.exp_avg, keep_m[half:])
