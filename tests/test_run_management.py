"""Output-directory, checkpoint-commit and resume-resolution contracts, plus loop arithmetic and schedules.

The reference pins these in ``tests/test_config_and_training_core.py:288-347`` (rank-0 broadcast with an
injected ``broadcast_fn``), ``tests/test_config_and_training_runtime.py`` (resume policy, loop math, flag
logic) and ``tests/test_config_and_training_resume.py:1746-1868`` (transactional save on a non-main rank).
"""

from __future__ import annotations

import json
import math
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

from deberta_b200.training import loop_utils as lu
from deberta_b200.training import run_management as rm
from deberta_b200.training.checkpointing import (normalize_resume_consumed_micro_batches, resolve_data_resume_policy,
                                                 save_periodic_checkpoint_if_due)
from deberta_b200.training.schedulers import SCHEDULER_TYPES, StepSchedule, make_lr_lambda


class Ctx:
    """Single-process stand-in for the distributed context; records barrier calls."""

    def __init__(self, rank=0, world=1):
        self.rank, self.world_size, self.is_main_process, self.distributed = rank, world, rank == 0, world > 1
        self.barriers = 0
        self.sent = []

    def wait_for_everyone(self):
        self.barriers += 1

    def broadcast_object(self, obj):
        self.sent.append(obj)
        return obj


def _write_ckpt(out: Path, step: int, *, weights=True, state=True, complete=True, consumed=None) -> Path:
    ck = out / f"checkpoint-{step}"
    ck.mkdir(parents=True)
    if weights:
        (ck / "model.safetensors").write_bytes(b"x" * 16)
    if state:
        rm.save_checkpoint_data_progress(checkpoint_dir=ck, consumed_micro_batches=step * 2 if consumed is None else consumed,
                                         lr_mult=0.5, global_step=step, gradient_accumulation_steps=2)
    if complete:
        rm.write_complete_marker(ck)
    return ck


# ---------------------------------------------------------------------------------------------- output dir
def test_sanitize_run_label():
    assert rm.sanitize_run_label("  my run/№1 ") == "my-run-1"
    assert rm.sanitize_run_label("...") == "run"
    assert rm.sanitize_run_label("ok_name-1.2") == "ok_name-1.2"


def test_resolve_output_dir_explicit_and_generated():
    assert rm.resolve_output_dir(output_dir="x/y", project_name="p", config_path=None) == Path("x/y")
    auto = rm.resolve_output_dir(output_dir=None, project_name="my proj", config_path="configs/base v3.yaml")
    assert auto.parts[0] == "runs" and auto.parts[1] == "my-proj" and auto.name.endswith("_base-v3")
    named = rm.resolve_output_dir(output_dir="  ", project_name="p", config_path="c.yaml", run_name="trial 7")
    assert named.name.endswith("_trial-7")
    bare = rm.resolve_output_dir(output_dir=None, project_name="p", config_path=None)
    assert bare.name.endswith("_run")


def test_rank0_result_is_computed_once_and_broadcast():
    calls = []
    main, other = Ctx(0, 2), Ctx(1, 2)
    wire = {}

    def bcast_main(box):
        wire["box"] = box
        return box

    got0 = rm.broadcast_rank0_result(main, lambda: calls.append(1) or "dir-A", broadcast_fn=bcast_main)
    got1 = rm.broadcast_rank0_result(other, lambda: calls.append(2) or "dir-B", broadcast_fn=lambda _own: wire["box"])
    assert got0 == got1 == "dir-A" and calls == [1]  # the non-main rank never computes


@pytest.mark.parametrize("exc,expected", [(ValueError("bad"), ValueError), (FileNotFoundError("gone"), FileNotFoundError),
                                          (KeyError("k"), RuntimeError)])
def test_rank0_errors_reach_every_rank_with_their_type(exc, expected):
    wire = {}

    def boom():
        raise exc

    with pytest.raises(expected):
        rm.broadcast_rank0_result(Ctx(0, 2), boom, broadcast_fn=lambda b: wire.setdefault("box", b))
    with pytest.raises(expected):
        rm.broadcast_rank0_result(Ctx(1, 2), lambda: "unused", broadcast_fn=lambda _b: wire["box"])


def test_rank0_broadcast_rejects_malformed_payloads_and_skips_single_process():
    with pytest.raises(RuntimeError, match="malformed"):
        rm.broadcast_rank0_result(Ctx(1, 2), lambda: 1, broadcast_fn=lambda _b: "not a dict")
    assert rm.broadcast_rank0_result(Ctx(0, 1), lambda: 41 + 1, broadcast_fn=lambda _b: pytest.fail("no broadcast")) == 42


def test_prepare_output_dir_matrix(tmp_path):
    out = tmp_path / "run"
    rm.prepare_output_dir(output_dir=out, overwrite_output_dir=False, resume_from_checkpoint=None, is_main_process=True)
    assert out.is_dir()
    (out / "junk.txt").write_text("x")
    with pytest.raises(ValueError, match="not empty"):
        rm.prepare_output_dir(output_dir=out, overwrite_output_dir=False, resume_from_checkpoint=None, is_main_process=True)
    # resuming keeps the content
    rm.prepare_output_dir(output_dir=out, overwrite_output_dir=False, resume_from_checkpoint="auto", is_main_process=True)
    assert (out / "junk.txt").exists()
    # non-main ranks never touch the directory
    rm.prepare_output_dir(output_dir=out, overwrite_output_dir=True, resume_from_checkpoint=None, is_main_process=False)
    assert (out / "junk.txt").exists()
    rm.prepare_output_dir(output_dir=out, overwrite_output_dir=True, resume_from_checkpoint=None, is_main_process=True)
    assert out.is_dir() and not any(out.iterdir())
    f = tmp_path / "file"
    f.write_text("x")
    with pytest.raises(ValueError, match="not a directory"):
        rm.prepare_output_dir(output_dir=f, overwrite_output_dir=False, resume_from_checkpoint=None, is_main_process=True)


# ---------------------------------------------------------------------------------------------- checkpoints
def test_checkpoint_listing_orders_by_step_number(tmp_path):
    for s in (900, 1000, 50):
        (tmp_path / f"checkpoint-{s}").mkdir()
    (tmp_path / "checkpoint-7").write_text("a file, not a directory")
    assert [s for s, _ in rm.list_checkpoints(tmp_path)] == [50, 900, 1000]
    assert rm.find_latest_checkpoint(tmp_path).name == "checkpoint-1000"
    assert rm.parse_checkpoint_step("a/b/checkpoint-123") == 123 and rm.parse_checkpoint_step("other") == 0
    assert rm.find_latest_checkpoint(tmp_path / "none") is None


def test_weights_validity_patterns(tmp_path):
    assert not rm.checkpoint_weights_appear_valid(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"")
    assert not rm.checkpoint_weights_appear_valid(tmp_path)  # empty payloads do not count
    shard = tmp_path / "pytorch_model_fsdp_0"
    shard.mkdir()
    (shard / "__0_0.distcp").write_bytes(b"abc")
    assert rm.checkpoint_weights_appear_valid(tmp_path)


def test_progress_metadata_round_trip_and_invalid_files(tmp_path):
    rm.save_checkpoint_data_progress(checkpoint_dir=tmp_path, consumed_micro_batches=-3, lr_mult=0.25,
                                     optimizer_param_digest={"gen": 1, "disc": "ab"}, global_step=9,
                                     gradient_accumulation_steps=0)
    consumed, mult, digest, step, ga = rm.load_checkpoint_progress_metadata(tmp_path)
    assert (consumed, mult, digest, step, ga) == (0, 0.25, {"gen": "1", "disc": "ab"}, 9, 1)
    (tmp_path / "data_state.json").write_text("{not json")
    assert rm.load_checkpoint_progress_metadata(tmp_path) == (None, 1.0, None, None, None)
    (tmp_path / "data_state.json").write_text(json.dumps({"lr_mult": 0.5}))
    assert rm.load_checkpoint_data_progress(tmp_path)[0] is None  # a position is required
    empty = tmp_path / "none"
    empty.mkdir()
    assert rm.load_checkpoint_progress_metadata(empty) == (None, 1.0, None, None, None)


def test_resumable_needs_marker_state_and_weights(tmp_path):
    assert rm.is_checkpoint_resumable(_write_ckpt(tmp_path, 1))
    assert not rm.is_checkpoint_resumable(_write_ckpt(tmp_path, 2, complete=False))
    assert not rm.is_checkpoint_resumable(_write_ckpt(tmp_path, 3, state=False))
    assert not rm.is_checkpoint_resumable(_write_ckpt(tmp_path, 4, weights=False))
    assert rm.find_latest_resumable_checkpoint(tmp_path).name == "checkpoint-1"


def test_resume_auto_picks_newest_resumable_and_explains_failures(tmp_path):
    out = tmp_path / "out"
    assert rm.resolve_resume_checkpoint(output_dir=out, resume_from_checkpoint=None, is_main_process=True) is None
    assert rm.resolve_resume_checkpoint(output_dir=out, resume_from_checkpoint="  ", is_main_process=True) is None
    assert rm.resolve_resume_checkpoint(output_dir=out, resume_from_checkpoint="auto", is_main_process=True) is None
    out.mkdir()
    (out / "notes.txt").write_text("x")
    with pytest.raises(ValueError, match="no checkpoint-\\* directories were found"):
        rm.resolve_resume_checkpoint(output_dir=out, resume_from_checkpoint="auto", is_main_process=True)
    _write_ckpt(out, 10)
    _write_ckpt(out, 20, complete=False)
    got = rm.resolve_resume_checkpoint(output_dir=out, resume_from_checkpoint="AUTO", is_main_process=True)
    assert Path(got).name == "checkpoint-10" and Path(got).is_absolute()
    bad = tmp_path / "bad"
    _write_ckpt(bad, 5, complete=False)
    with pytest.raises(ValueError, match="none are resumable"):
        rm.resolve_resume_checkpoint(output_dir=bad, resume_from_checkpoint="auto", is_main_process=True)


def test_resume_explicit_path_integrity_checks(tmp_path):
    with pytest.raises(FileNotFoundError):
        rm.resolve_resume_checkpoint(output_dir=tmp_path, resume_from_checkpoint=str(tmp_path / "nope"), is_main_process=True)
    f = tmp_path / "f"
    f.write_text("x")
    with pytest.raises(ValueError, match="non-directory"):
        rm.resolve_resume_checkpoint(output_dir=tmp_path, resume_from_checkpoint=str(f), is_main_process=True)
    with pytest.raises(ValueError, match="missing .complete marker"):
        rm.resolve_resume_checkpoint(output_dir=tmp_path, resume_from_checkpoint=str(_write_ckpt(tmp_path, 1, complete=False)),
                                     is_main_process=True)
    with pytest.raises(ValueError, match="integrity checks"):
        rm.resolve_resume_checkpoint(output_dir=tmp_path, resume_from_checkpoint=str(_write_ckpt(tmp_path, 2, state=False)),
                                     is_main_process=True)
    with pytest.raises(ValueError, match="weights appear missing"):
        rm.resolve_resume_checkpoint(output_dir=tmp_path, resume_from_checkpoint=str(_write_ckpt(tmp_path, 3, weights=False)),
                                     is_main_process=True)
    good = _write_ckpt(tmp_path, 4)
    assert rm.resolve_resume_checkpoint(output_dir=tmp_path, resume_from_checkpoint=str(good), is_main_process=True) == str(good.resolve())


def test_resume_resolution_for_ranks_uses_rank0_answer(tmp_path):
    good = _write_ckpt(tmp_path, 4)
    wire = {}
    a = rm.resolve_resume_checkpoint_for_ranks(Ctx(0, 2), output_dir=tmp_path, resume_from_checkpoint="auto",
                                               broadcast_fn=lambda b: wire.setdefault("b", b))
    b = rm.resolve_resume_checkpoint_for_ranks(Ctx(1, 2), output_dir=tmp_path / "elsewhere", resume_from_checkpoint="auto",
                                               broadcast_fn=lambda _b: wire["b"])
    assert a == b == str(good.resolve())
    assert rm.resolve_resume_checkpoint_for_ranks(Ctx(1, 2), output_dir=tmp_path, resume_from_checkpoint=None,
                                                  broadcast_fn=lambda _b: pytest.fail("no broadcast")) is None
    with pytest.raises(RuntimeError, match="empty"):
        rm.resolve_resume_checkpoint_for_ranks(Ctx(1, 2), output_dir=tmp_path, resume_from_checkpoint="auto",
                                               broadcast_fn=lambda _b: {"ok": True, "value": " "})


def test_rotation_keeps_newest_committed_and_ignores_uncommitted(tmp_path):
    for s in (1, 2, 3, 4):
        _write_ckpt(tmp_path, s)
    _write_ckpt(tmp_path, 5, complete=False)
    rm.rotate_checkpoints(tmp_path, save_total_limit=2)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["checkpoint-3", "checkpoint-4", "checkpoint-5"]
    rm.rotate_checkpoints(tmp_path, save_total_limit=0)  # 0 = keep everything
    assert len(list(tmp_path.iterdir())) == 3


def _save_state(files=("model.safetensors",)):
    def fn(d):
        for f in files:
            (Path(d) / f).write_bytes(b"w" * 8)
    return fn


def test_transactional_save_commits_atomically_and_rotates(tmp_path):
    ctx = Ctx()
    for s in (1, 2, 3):
        rm.save_training_checkpoint(ctx=ctx, save_state=_save_state(), checkpoint_dir=tmp_path / f"checkpoint-{s}",
                                    output_dir=tmp_path, consumed_micro_batches=4 * s, save_total_limit=2, log_label="t",
                                    lr_mult=0.5, optimizer_param_digest="abc", global_step=s, gradient_accumulation_steps=4)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["checkpoint-2", "checkpoint-3"]  # no staging leftovers
    ck = tmp_path / "checkpoint-3"
    assert rm.is_checkpoint_resumable(ck)
    assert rm.load_checkpoint_progress_metadata(ck) == (12, 0.5, "abc", 3, 4)
    assert ctx.barriers == 12  # four barriers per save: the last one holds the other ranks until rank 0 has committed


def test_transactional_save_refuses_to_overwrite_and_cleans_up_failures(tmp_path):
    ctx = Ctx()
    kw = dict(ctx=ctx, output_dir=tmp_path, consumed_micro_batches=1, save_total_limit=0, log_label="t")
    rm.save_training_checkpoint(save_state=_save_state(), checkpoint_dir=tmp_path / "checkpoint-1", **kw)
    with pytest.raises(RuntimeError, match="Refusing to overwrite"):
        rm.save_training_checkpoint(save_state=_save_state(), checkpoint_dir=tmp_path / "checkpoint-1", **kw)
    # a save that produced no weights fails validation, leaves no checkpoint and no staging directory
    with pytest.raises(RuntimeError, match="structural validation failed"):
        rm.save_training_checkpoint(save_state=_save_state(files=()), checkpoint_dir=tmp_path / "checkpoint-2", **kw)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["checkpoint-1"]
    # an empty directory of the same name is replaced
    (tmp_path / "checkpoint-3").mkdir()
    rm.save_training_checkpoint(save_state=_save_state(), checkpoint_dir=tmp_path / "checkpoint-3", **kw)
    assert rm.is_checkpoint_committed(tmp_path / "checkpoint-3")


def test_transactional_save_on_non_main_rank_writes_state_but_no_metadata(tmp_path):
    staging = tmp_path / ".checkpoint-1.tmp-shared"
    staging.mkdir()

    class Other(Ctx):
        def broadcast_object(self, obj):
            return str(staging)  # the name rank 0 chose

    ctx = Other(1, 2)
    seen = []
    rm.save_training_checkpoint(ctx=ctx, save_state=lambda d: seen.append(d), checkpoint_dir=tmp_path / "checkpoint-1",
                                output_dir=tmp_path, consumed_micro_batches=1, save_total_limit=1, log_label="t")
    assert seen == [str(staging)] and ctx.barriers == 4
    assert not (tmp_path / "checkpoint-1").exists() and not (staging / "data_state.json").exists()


def test_periodic_save_only_on_multiples_and_once_per_step(tmp_path):
    ctx = Ctx()
    kw = dict(ctx=ctx, save_state=_save_state(), output_dir=tmp_path, consumed_micro_batches=0, save_total_limit=0)
    assert save_periodic_checkpoint_if_due(global_step=3, save_steps=2, last_saved_step=0, **kw) == 0
    assert save_periodic_checkpoint_if_due(global_step=4, save_steps=2, last_saved_step=0, **kw) == 4
    assert save_periodic_checkpoint_if_due(global_step=4, save_steps=2, last_saved_step=4, **kw) == 4
    assert save_periodic_checkpoint_if_due(global_step=6, save_steps=0, last_saved_step=4, **kw) == 4
    assert [p.name for p in tmp_path.iterdir()] == ["checkpoint-4"]


# ---------------------------------------------------------------------------------------------- resume policy
def test_data_resume_policy():
    cfg = SimpleNamespace(resume_data_strategy="auto", resume_replay_max_micro_batches=100)
    assert resolve_data_resume_policy(train_cfg=cfg, consumed_micro_batches=100, global_step=50)[:2] == (True, 0)
    replay, epoch, why = resolve_data_resume_policy(train_cfg=cfg, consumed_micro_batches=101, global_step=50)
    assert (replay, epoch) == (False, 50) and "exceed replay limit" in why
    cfg.resume_data_strategy = "replay"
    assert resolve_data_resume_policy(train_cfg=cfg, consumed_micro_batches=10**9, global_step=7)[:2] == (True, 0)
    cfg.resume_data_strategy = "restart_epoch"
    assert resolve_data_resume_policy(train_cfg=cfg, consumed_micro_batches=0, global_step=7)[:2] == (False, 7)


def test_resume_position_is_clamped_to_an_optimizer_step_boundary():
    assert normalize_resume_consumed_micro_batches(consumed_micro_batches=40, global_step=10, ga_steps=4) == 40
    assert normalize_resume_consumed_micro_batches(consumed_micro_batches=43, global_step=10, ga_steps=4) == 40
    assert normalize_resume_consumed_micro_batches(consumed_micro_batches=-1, global_step=3, ga_steps=0) == 3


# ---------------------------------------------------------------------------------------------- loop arithmetic
def test_token_weighted_objective_equals_full_batch_normalisation():
    torch.manual_seed(0)
    gen_tok = [torch.rand(n) for n in (5, 11, 2)]     # per-token losses of three micro-batches
    disc_tok = [torch.rand(n) for n in (40, 64, 9)]
    g_total, d_total = sum(t.numel() for t in gen_tok), sum(t.numel() for t in disc_tok)
    window = sum(lu.token_weighted_micro_objective(gen_loss=g.mean(), disc_loss=d.mean(), gen_count=g.numel(), disc_count=d.numel(),
                                                   gen_window_tokens_per_rank=g_total, disc_window_tokens_per_rank=d_total,
                                                   gen_loss_weight=1.0, disc_loss_weight=50.0)
                 for g, d in zip(gen_tok, disc_tok))
    want = torch.cat(gen_tok).mean() + 50.0 * torch.cat(disc_tok).mean()
    assert abs(float(window) - float(want)) < 1e-5


def test_window_denominators_and_loss_scales():
    assert lu.resolve_window_token_denominators(gen_window_tokens_per_rank_raw=0.0, disc_window_tokens_per_rank_raw=12.5) == \
        (1.0, 12.5, True, False)
    assert lu.micro_loss_scale(ga_steps=4, token_weighted_ga=True) == 1.0
    assert lu.micro_loss_scale(ga_steps=4, token_weighted_ga=False) == 0.25
    assert lu.micro_loss_scale(ga_steps=0, token_weighted_ga=False) == 1.0
    assert lu.finalize_window_metric_loss(accumulated_loss=8.0, ga_steps=4, token_weighted_ga=False) == 2.0
    assert lu.finalize_window_metric_loss(accumulated_loss=8.0, ga_steps=4, token_weighted_ga=True) == 8.0


def test_clip_decision_and_nonfinite_backoff_recovery():
    assert lu.should_clip_gradients(sync_gradients=True, max_grad_norm=1.0)
    assert not lu.should_clip_gradients(sync_gradients=False, max_grad_norm=1.0)
    assert not lu.should_clip_gradients(sync_gradients=True, max_grad_norm=None)
    assert not lu.should_clip_gradients(sync_gradients=True, max_grad_norm=0.0)
    mult, resets = 1.0, []
    for streak in range(1, 10):
        mult, reset = lu.apply_nonfinite_recovery(lr_mult=mult, skip_streak=streak)
        resets.append(reset)
    assert mult == lu.NONFINITE_LR_MULT_FLOOR  # halves per skip, never below the floor
    assert [i + 1 for i, r in enumerate(resets) if r] == [4, 8]
    for _ in range(60):
        mult = lu.recover_lr_mult(mult)
    assert mult == 1.0


def test_token_counts_for_padding_masks_and_document_ids():
    batch = {"input_ids": torch.tensor([[1, 9, 9, 2, 0, 0], [1, 9, 2, 9, 9, 2]]),
             "labels": torch.tensor([[-100, 9, -100, -100, -100, -100], [-100, -100, -100, 9, 9, -100]]),
             "attention_mask": torch.tensor([[1, 1, 1, 1, 0, 0], [1] * 6])}
    assert lu.count_rtd_tokens_for_batch(batch, pad_token_id=0) == (3.0, 10.0)
    assert lu.count_input_tokens_for_batch(batch) == 10.0
    del batch["attention_mask"]
    assert lu.count_rtd_tokens_for_batch(batch, pad_token_id=0) == (3.0, 10.0)  # falls back to pad id
    batch["doc_ids"] = torch.tensor([[1, 1, 1, 1, 0, 0], [1, 1, 1, 2, 2, 2]])
    assert lu.count_rtd_tokens_for_batch(batch, pad_token_id=0) == (3.0, 10.0)
    assert lu.count_input_tokens_for_batch(batch) == 10.0


# ---------------------------------------------------------------------------------------------- schedules
@pytest.mark.parametrize("kind", SCHEDULER_TYPES)
def test_schedules_match_transformers(kind):
    transformers = pytest.importorskip("transformers")
    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=2e-4)
    sched = transformers.get_scheduler(kind, opt, num_warmup_steps=5, num_training_steps=40)
    ours = StepSchedule(kind, warmup_steps=5, total_steps=40, base_lr=2e-4)
    for _ in range(45):
        assert math.isclose(ours.get_last_lr()[0], sched.get_last_lr()[0], rel_tol=1e-6, abs_tol=1e-12)
        opt.step()
        sched.step()
        ours.step()


def test_schedule_state_round_trip_and_unknown_kind():
    s = StepSchedule("linear", warmup_steps=2, total_steps=10, base_lr=1.0)
    for _ in range(6):
        s.step()
    t = StepSchedule("linear", warmup_steps=2, total_steps=10, base_lr=1.0)
    t.load_state_dict(s.state_dict())
    assert t.scale() == s.scale() == 0.5
    with pytest.raises(ValueError, match="Unknown scheduler type"):
        make_lr_lambda("exotic", warmup_steps=0, total_steps=1)
    assert make_lr_lambda("linear", warmup_steps=0, total_steps=0)(0) == 0.0  # degenerate lengths do not divide by zero
