"""Optimizer grouping, flat-buffer engine and one-window trainer semantics on CPU (fp32, single process).

Reference counterparts: ``tests/test_config_and_training_core.py`` (optimizer partition / parameter-order digest),
``tests/test_config_and_training_runtime.py`` (no-decay and generator rules, LR resolution) and
``tests/test_config_and_training_resume.py:419-632`` (decoupled loop order, scaling, non-finite skip protocol).
"""

from __future__ import annotations

import copy
import math

import pytest
import torch

from deberta_b200 import config as C
from deberta_b200.data.synthetic import SyntheticTokenizer
from deberta_b200.parallel.dist import DistContext
from deberta_b200.parallel.engine import (GROUP_ORDER, is_generator_param, is_no_decay_param, param_order_digest,
                                          partition_parameters)
from deberta_b200.training.runtime import build_engine, build_model, resolve_learning_rates
from deberta_b200.training.trainer import Trainer

VOCAB = 200


def _configs(decoupled=True, ga=2, token_weighted=True, sharing="gdes", **optim):
    model = C.ModelConfig(backbone_type="rope", hidden_size=32, num_hidden_layers=3, num_attention_heads=2,
                          intermediate_size=64, embedding_sharing=sharing, tokenizer_name_or_path=f"synthetic:{VOCAB}")
    train = C.TrainConfig(max_steps=20, per_device_train_batch_size=2, gradient_accumulation_steps=ga,
                          decoupled_training=decoupled, token_weighted_gradient_accumulation=token_weighted,
                          mixed_precision="no")
    opt = C.OptimConfig(**{"learning_rate": 1e-3, "warmup_steps": 0, "lr_scheduler_type": "constant", **optim})
    return model, train, opt


def _setup(seed=0, **kw):
    model_cfg, train_cfg, optim_cfg = _configs(**kw)
    torch.manual_seed(seed)
    tok = SyntheticTokenizer(VOCAB)
    model, _, _ = build_model(model_cfg=model_cfg, tokenizer=tok, max_seq_length=32)
    ctx = DistContext()
    engine = build_engine(model=model, ctx=ctx, train_cfg=train_cfg, optim_cfg=optim_cfg, parallelism="ddp")
    trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=train_cfg, optim_cfg=optim_cfg, pad_token_id=0)
    return model, engine, trainer


def _batches(n=2, seed=3, masked=True):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(5, VOCAB, (2, 16), generator=g)
        labels = torch.full_like(ids, -100)
        if masked:
            pick = torch.rand(2, 16, generator=g) < 0.3
            pick[:, 0] = False
            pick[0, 1] = True
            labels[pick] = ids[pick]
            ids = ids.masked_fill(pick, 4)
        out.append({"input_ids": ids, "labels": labels})
    return out


# ---------------------------------------------------------------------------------------------- grouping
def test_no_decay_and_generator_rules():
    w, b, delta = torch.nn.Parameter(torch.zeros(4, 4)), torch.nn.Parameter(torch.zeros(4)), torch.nn.Parameter(torch.zeros(9, 4))
    assert not is_no_decay_param("encoder.layer.0.dense.weight", w)
    assert is_no_decay_param("encoder.layer.0.dense.bias", b)
    assert is_no_decay_param("encoder.LayerNorm.weight", b) and is_no_decay_param("x.rms_norm.weight", b)
    assert is_no_decay_param("keel_alpha", torch.nn.Parameter(torch.zeros(())))
    assert not is_no_decay_param("discriminator.embeddings.word_embeddings.bias", delta)  # 2-D deltas are decayed
    assert is_generator_param("generator.encoder.x") and is_generator_param("generator_lm_head.bias")
    assert is_generator_param("enhanced_mask_decoder.q") and not is_generator_param("discriminator_head.dense.weight")


def test_partition_covers_every_trainable_parameter_once():
    model, _, _ = _setup()
    groups = partition_parameters(model)
    assert tuple(groups) == GROUP_ORDER
    ids = [id(p) for g in groups.values() for _, p in g]
    trainable = {id(p) for p in model.parameters() if p.requires_grad}
    assert len(ids) == len(set(ids)) and set(ids) == trainable
    assert all(is_generator_param(n) for n, _ in groups["gen_decay"] + groups["gen_no_decay"])
    assert all(p.dim() >= 2 for _, p in groups["disc_decay"])
    frozen = next(iter(model.parameters()))
    frozen.requires_grad_(False)
    assert id(frozen) not in {id(p) for g in partition_parameters(model).values() for _, p in g}


def test_shared_embedding_is_owned_by_the_generator_only():
    model, _, _ = _setup(sharing="es", decoupled=False)
    groups = partition_parameters(model)
    shared = model.generator.embeddings.word_embeddings.weight
    owners = [k for k, g in groups.items() if any(p is shared for _, p in g)]
    assert owners == ["gen_decay"]


def test_param_order_digest_tracks_names_and_owners():
    model, _, _ = _setup()
    full, gen, disc = param_order_digest(model), param_order_digest(model, ("gen",)), param_order_digest(model, ("disc",))
    assert len({full, gen, disc}) == 3 and len(full) == 16
    again, _, _ = _setup()
    assert param_order_digest(again) == full  # a function of names and order only, not of values
    model.discriminator_head.register_parameter("extra", torch.nn.Parameter(torch.zeros(3)))
    assert param_order_digest(model, ("disc",)) != disc and param_order_digest(model, ("gen",)) == gen


def test_learning_rate_resolution():
    assert resolve_learning_rates(C.OptimConfig(learning_rate=2e-4)) == (2e-4, 2e-4)
    assert resolve_learning_rates(C.OptimConfig(learning_rate=2e-4, generator_learning_rate=1e-4,
                                                discriminator_learning_rate=5e-4)) == (1e-4, 5e-4)


# ---------------------------------------------------------------------------------------------- engine
def test_engine_layout_one_or_two_optimizers_with_group_hyperparameters():
    _, eng, _ = _setup(decoupled=True, weight_decay=0.02, generator_learning_rate=5e-4)
    assert list(eng.optimizers) == ["generator", "discriminator"]
    g, d = eng.optimizers["generator"], eng.optimizers["discriminator"]
    assert g.end <= d.start  # disjoint, contiguous ranges of the flat buffers
    by_group = {s.group: s for o in (g, d) for s in o.segments}
    assert by_group["gen_decay"].weight_decay == 0.02 and by_group["gen_no_decay"].weight_decay == 0.0
    assert by_group["gen_decay"].base_lr == 5e-4 and by_group["disc_decay"].base_lr == 1e-3
    _, eng1, _ = _setup(decoupled=False)
    assert list(eng1.optimizers) == ["all"]


def test_parameters_are_views_of_the_flat_master_buffer():
    model, eng, _ = _setup()
    p = model.discriminator_head.dense.weight
    lo, hi = eng.master.data_ptr(), eng.master.data_ptr() + eng.master.numel() * 4
    assert lo <= p.data_ptr() < hi
    with torch.no_grad():
        eng.master.zero_()
    assert float(p.abs().sum()) == 0.0  # writing the buffer changes the module's weights


def test_engine_step_matches_torch_adamw_with_clipping():
    model, eng, _ = _setup(decoupled=False, weight_decay=0.01, max_grad_norm=0.5)
    ref = copy.deepcopy(model)
    groups = partition_parameters(ref)
    torch_opt = torch.optim.AdamW(
        [{"params": [p for _, p in groups[k]], "weight_decay": 0.0 if k.endswith("no_decay") else 0.01} for k in GROUP_ORDER],
        lr=1e-3, betas=(eng.optimizers["all"].betas), eps=eng.optimizers["all"].eps)
    batch = _batches(1)[0]
    for step in range(3):
        for m in (model, ref):
            torch.manual_seed(100 + step)
            m(input_ids=batch["input_ids"], labels=batch["labels"]).loss.backward()
        eng.sync_grads("all")
        eng.step("all", lr_scale=1.0, max_grad_norm=0.5)
        eng.zero_grad()
        model.sync_discriminator_embeddings_from_generator()
        torch.nn.utils.clip_grad_norm_([p for g in groups.values() for _, p in g], 0.5)
        torch_opt.step()
        torch_opt.zero_grad()
        ref.sync_discriminator_embeddings_from_generator()
    for (n, a), (_, b) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(a, b, rtol=2e-4, atol=2e-6), n


def test_engine_skips_the_update_when_the_norm_is_not_finite():
    model, eng, _ = _setup(decoupled=False)
    batch = _batches(1)[0]
    model(input_ids=batch["input_ids"], labels=batch["labels"]).loss.backward()
    before = eng.master.clone()
    norm_sq = eng.sync_grads("all", torch.tensor([float("inf")]))
    eng.step("all", lr_scale=1.0, max_grad_norm=1.0)
    assert not math.isfinite(float(norm_sq)) and torch.equal(eng.master, before) and eng.optimizers["all"].step == 0


def test_engine_state_round_trip():
    model, eng, trainer = _setup()
    trainer.train_window(_batches())
    model_state, opt_state = eng.model_state_dict(), eng.optimizer_state_dict()
    assert "discriminator.embeddings.word_embeddings.bias" in model_state
    model2, eng2, _ = _setup(seed=9)
    eng2.load_model_state_dict(model_state)
    eng2.load_optimizer_state_dict(opt_state)
    assert torch.equal(eng2.master, eng.master)
    for name in eng.optimizers:
        assert eng2.optimizers[name].step == eng.optimizers[name].step
        assert torch.equal(eng2.optimizers[name].exp_avg, eng.optimizers[name].exp_avg)
    bad = dict(model_state)
    bad.pop("discriminator_head.classifier.bias")
    with pytest.raises((KeyError, RuntimeError, ValueError)):
        eng2.load_model_state_dict(bad, strict=True)


# ---------------------------------------------------------------------------------------------- trainer
def test_decoupled_window_steps_generator_before_discriminator_and_counts_progress():
    model, eng, trainer = _setup(decoupled=True, ga=2)
    order = []
    real_step = eng.step
    eng.step = lambda name, **kw: (order.append(name), real_step(name, **kw))[1]
    gen_before = model.generator.embeddings.word_embeddings.weight.detach().clone()
    stats = trainer.train_window(_batches(2))
    assert order == ["generator", "discriminator"]
    assert trainer.global_step == 1 and trainer.consumed_micro_batches == 2
    assert set(stats.grad_norms) == {"generator", "discriminator"} and all(float(v) > 0 for v in stats.grad_norms.values())
    assert stats.gen_tokens > 0 and stats.disc_tokens == 2 * 2 * 16 and stats.input_tokens == 64
    # the discriminator saw the refreshed generator embeddings
    emb = model.discriminator.embeddings.word_embeddings
    gen_after = model.generator.embeddings.word_embeddings.weight.detach()
    assert not torch.equal(gen_after, gen_before) and torch.allclose(emb.weight, gen_after + emb.bias)
    assert all(p.grad is None or float(p.grad.abs().sum()) == 0.0 for p in model.parameters())  # gradients cleared


def test_coupled_window_uses_one_optimizer():
    _, eng, trainer = _setup(decoupled=False)
    stats = trainer.train_window(_batches(2))
    assert set(stats.grad_norms) == {"all"} and eng.optimizers["all"].step == 1


def test_token_weighting_makes_the_window_independent_of_how_it_is_split():
    """Two micro-batches of unequal masked counts give the same update as their concatenation in one micro-batch."""
    a, b = _batches(2, seed=8)
    b["labels"][:, 8:] = -100  # make the masked counts differ
    merged = {k: torch.cat([a[k], b[k]]) for k in a}
    results = []
    for window in ([a, b], [merged]):
        model, eng, trainer = _setup(decoupled=False, ga=len(window))
        # sampling noise must not differ between the layouts: freeze it with a near-greedy temperature
        trainer.temperature = 1e-6
        trainer.train_window(window)
        results.append(eng.master.clone())
    assert torch.allclose(results[0], results[1], rtol=1e-4, atol=1e-6)


def test_plain_mean_accumulation_divides_by_the_number_of_micro_batches():
    _, eng_w, t_w = _setup(token_weighted=True, decoupled=False)
    _, eng_m, t_m = _setup(token_weighted=False, decoupled=False)
    for t in (t_w, t_m):
        t.temperature = 1e-6
    same = _batches(1, seed=4) * 2  # identical micro-batches: both normalisations agree exactly
    t_w.train_window(same)
    t_m.train_window(same)
    assert torch.allclose(eng_w.master, eng_m.master, rtol=1e-5, atol=1e-7)


def test_nonfinite_window_is_skipped_with_backoff_then_recovers():
    model, eng, trainer = _setup(decoupled=True)
    seen = []
    trainer.on_nonfinite = lambda step, norms: seen.append((step, dict(norms)))
    before = eng.master.clone()
    with torch.no_grad():
        model.generator_lm_head.bias.fill_(float("nan"))  # poisons the generator loss only
    trainer.train_window(_batches(2))
    assert trainer.skipped_steps == 1 and trainer.skip_streak == 1 and trainer.lr_mult == 0.5
    assert seen and seen[0][0] == 1 and not math.isfinite(seen[0][1]["generator"])
    gen = eng.optimizers["generator"]
    assert gen.step == 0  # the update did not happen
    lo, hi = gen.start, gen.end
    bias = model.generator_lm_head.bias
    keep = torch.ones(hi - lo, dtype=torch.bool)
    off = (bias.data_ptr() - eng.master.data_ptr()) // 4 - lo
    keep[off:off + bias.numel()] = False
    assert torch.equal(eng.master[lo:hi][keep], before[lo:hi][keep])
    assert trainer.global_step == 1  # the window still counts (schedules advance, data was consumed)
    with torch.no_grad():
        bias.zero_()
    trainer.train_window(_batches(2, seed=6))
    assert trainer.skip_streak == 0 and math.isclose(trainer.lr_mult, 0.55) and gen.step == 1


def test_every_fourth_consecutive_skip_clears_the_optimizer_moments():
    model, eng, trainer = _setup(decoupled=False)
    trainer.train_window(_batches(2))
    assert float(eng.optimizers["all"].exp_avg.abs().sum()) > 0
    with torch.no_grad():
        model.generator_lm_head.bias.fill_(float("nan"))
    for i in range(4):
        trainer.train_window(_batches(2, seed=20 + i))
    assert trainer.skip_streak == 4 and math.isclose(trainer.lr_mult, 0.5 ** 4)
    assert float(eng.optimizers["all"].exp_avg.abs().sum()) == 0.0 and eng.optimizers["all"].step == 0


def test_window_without_masked_tokens_trains_nothing_but_advances():
    model, eng, trainer = _setup(decoupled=True)
    trainer.train_window(_batches(2))  # moments and step counters are non-trivial from here on
    disc = eng.optimizers["discriminator"]
    lo, hi = disc.start, disc.end
    before, m_before, v_before = eng.master[lo:hi].clone(), disc.exp_avg.clone(), disc.exp_avg_sq.clone()
    sched_before = trainer.schedules["discriminator"].last_step
    stats = trainer.train_window(_batches(2, masked=False))
    assert stats.zero_gen_window and not stats.zero_disc_window and trainer.global_step == 2
    # no rank has a generator target: the discriminator neither steps nor decays (reference entrypoint.py:1269-1296)
    assert torch.equal(eng.master[lo:hi], before) and torch.equal(disc.exp_avg, m_before)
    assert torch.equal(disc.exp_avg_sq, v_before) and disc.step == 1
    assert trainer.schedules["discriminator"].last_step == sched_before
    assert trainer.skipped_steps == 0 and trainer.lr_mult == 1.0  # not a non-finite skip


def test_device_gate_switches_the_update_off_and_the_outcome_corrects_the_counters():
    """The path several GPUs take: the decision sits in a tensor, the update is gated where it runs, and the step
    counter / schedule are corrected when the outcome is read."""
    model, eng, trainer = _setup(decoupled=True)
    trainer.train_window(_batches(2))
    disc = eng.optimizers["discriminator"]
    before = eng.master[disc.start:disc.end].clone()
    real = trainer._window_denominators
    trainer._window_denominators = lambda g, d: (torch.tensor(max(g, 1.0)), torch.tensor(max(d, 1.0)),
                                                 torch.tensor(1.0 if g > 0 else 0.0))
    trainer.train_window(_batches(2, masked=False))
    assert torch.equal(eng.master[disc.start:disc.end], before) and disc.step == 1
    trainer.train_window(_batches(2, seed=9))
    assert disc.step == 2 and not torch.equal(eng.master[disc.start:disc.end], before)
    trainer._window_denominators = real
    g = torch.tensor([0.0])
    m0 = eng.master.clone()
    eng.sync_grads("discriminator")
    eng.step("discriminator", gate=g)
    assert torch.equal(eng.master, m0) and disc.step == 2


def test_nonfinite_generator_voids_the_whole_window():
    """A NaN generator loss: discriminator weights and Adam moments stay bit-identical, both counters stay put."""
    model, eng, trainer = _setup(decoupled=True)
    trainer.train_window(_batches(2))
    disc, gen = eng.optimizers["discriminator"], eng.optimizers["generator"]
    w, m, v = eng.master[disc.start:disc.end].clone(), disc.exp_avg.clone(), disc.exp_avg_sq.clone()
    with torch.no_grad():
        model.generator_lm_head.bias.fill_(float("nan"))
    trainer.train_window(_batches(2, seed=5))
    assert torch.equal(eng.master[disc.start:disc.end], w) and torch.equal(disc.exp_avg, m) and torch.equal(disc.exp_avg_sq, v)
    assert disc.step == 1 and gen.step == 1 and trainer.skipped_steps == 1 and trainer.lr_mult == 0.5
    assert not math.isfinite(trainer.last_outcome["discriminator"])  # the generator's guard reached the discriminator
    assert trainer.schedules["discriminator"].last_step == 2  # schedules advance on a skipped window


def test_kernel_status_word_raises_when_the_outcome_is_read(monkeypatch):
    from deberta_b200.ops import _lib
    from deberta_b200.training import trainer as T

    _, _, trainer = _setup()
    trainer.train_window(_batches(2))

    class Outcome:
        step = 7

        def resolve(self):
            return {"generator": 1.0}, None, 5

    monkeypatch.setattr(_lib, "check_status", lambda: (_ for _ in ()).throw(_lib.KernelError("device status 5")))
    trainer._pending = Outcome()
    with pytest.raises(_lib.KernelError):
        trainer.resolve_pending()
    assert trainer._pending is None and T.Trainer.resolve_pending is T.Trainer._resolve_pending


def test_logged_row_matches_a_hand_computation():
    from deberta_b200.training.entrypoint import _reduce_window_stats
    from deberta_b200.training.trainer import WindowStats

    t = lambda x: torch.tensor(float(x))  # noqa: E731
    w1 = WindowStats(t(2.0 * 10), t(0.5 * 100), t(0.9 * 100), t(12), gen_tokens=10, disc_tokens=100, input_tokens=100)
    w2 = WindowStats(t(4.0 * 30), t(0.25 * 300), t(0.7 * 300), t(20), gen_tokens=30, disc_tokens=300, input_tokens=300)
    row = _reduce_window_stats(DistContext(), [w1, w2], torch.device("cpu"), loss_weights=(1.0, 50.0))
    gen = (2.0 * 10 + 4.0 * 30) / 40
    disc = (0.5 * 100 + 0.25 * 300) / 400
    assert math.isclose(row["gen_loss"], gen) and math.isclose(row["disc_loss"], disc)
    assert math.isclose(row["loss"], 1.0 * gen + 50.0 * disc, rel_tol=1e-6)
    assert math.isclose(row["disc_acc"], (90 + 210) / 400) and math.isclose(row["disc_pos_frac"], 32 / 400)


def test_trainer_state_round_trip_and_lr_reporting():
    _, _, trainer = _setup(generator_learning_rate=5e-4)
    trainer.train_window(_batches(2))
    trainer.lr_mult = 0.25
    assert trainer.current_lrs() == {"generator": 5e-4 * 0.25, "discriminator": 1e-3 * 0.25}
    state = trainer.state_dict()
    _, _, other = _setup(generator_learning_rate=5e-4)
    other.load_state_dict(state)
    assert (other.global_step, other.lr_mult, other.consumed_micro_batches) == (1, 0.25, 2)
    assert other.schedules["generator"].last_step == 1
    digest = trainer.optimizer_param_digest()
    assert set(digest) == {"generator", "discriminator"} and digest == other.optimizer_param_digest()


def test_full_shard_mode_gathers_layers_on_demand_and_matches_replicated():
    """One process: the same windows through ``ddp`` and ``fsdp`` engines end in bit-identical masters; the sharder
    gathered layer units into its two slots and kept the roots resident."""
    def run(parallelism):
        model_cfg, train_cfg, optim_cfg = _configs()
        torch.manual_seed(0)
        model, _, _ = build_model(model_cfg=model_cfg, tokenizer=SyntheticTokenizer(VOCAB), max_seq_length=32)
        ctx = DistContext()
        engine = build_engine(model=model, ctx=ctx, train_cfg=train_cfg, optim_cfg=optim_cfg, parallelism=parallelism)
        trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=train_cfg, optim_cfg=optim_cfg, pad_token_id=0)
        losses = []
        for i in range(3):
            torch.manual_seed(100 + i)
            losses.append(float(trainer.train_window(_batches(2, seed=3 + i)).gen_loss_tokens))
        return losses, engine, model

    ref_losses, ref_eng, _ = run("ddp")
    losses, eng, model = run("fsdp")
    assert losses == ref_losses and torch.equal(eng.master, ref_eng.master)
    sh = eng.sharder
    names = [u.name for u in sh.units]
    assert names == ["gen.layer0", "disc.layer0", "disc.layer1", "disc.layer2", "gen.root", "disc.root"]
    covered = sorted(r for u in sh.units for r in u.ranges)
    assert covered[0][0] == 0 and all(a[1] == b[0] for a, b in zip(covered, covered[1:])) and covered[-1][1] == eng.total_elems
    assert eng.compute is None and len(sh.slots) == 2 and sh.slot_elems == max(u.size for u in sh.units if not u.is_root)
    assert sh.gathers > 3 * 2 * 4  # every layer unit, forward and backward, every window (plus roots after each update)
    # a layer's parameters live in a slot, a root's in its own buffer; the GDES base aliases the generator's table
    lay = model.discriminator.encoder.layers[1]
    p0 = next(lay.parameters())
    assert sh.slots[1].data_ptr() <= p0.data_ptr() < sh.slots[1].data_ptr() + sh.slots[1].numel() * 4
    emb = model.discriminator.embeddings.word_embeddings
    assert emb.base_weight.data_ptr() == model.generator.embeddings.word_embeddings.weight.data_ptr()
    rep = sh.memory_report()
    assert rep["shard_bytes"] == eng.total_elems * 4 and rep["slot_bytes"] == 2 * sh.slot_elems * 4
