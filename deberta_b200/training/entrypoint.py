"""``run_pretraining`` / ``run_pretraining_dry_run``: the training program behind ``deberta train``.

Follows the stages of ``training/entrypoint.py`` of the reference: process group → validation →
output/resume resolution → config snapshots → seed → tokenizer → data → model → engine/optimizers →
trackers → resume (weights, optimizer, schedules, RNG, data position) → step loop with periodic
logging/checkpoints → final checkpoint → HF export. Distribution is this package's own engine
(``parallel/engine.py``) instead of Accelerate.
"""

from __future__ import annotations

import contextlib
import logging
import time
from pathlib import Path
from typing import Any

import torch

from deberta_b200.config import (Config, DataConfig, LoggingConfig, ModelConfig, OptimConfig, TrainConfig,
                                 _sync_legacy_train_aliases, validate_config)
from deberta_b200.parallel.dist import DistContext, init_distributed
from deberta_b200.run_layout import FINAL_HF_DIR
from deberta_b200.utils.checkpoint import load_training_state, save_training_state
from deberta_b200.utils.log import setup_process_logging
from deberta_b200.utils.trace import set_nvtx

from .compile import maybe_compile_model, resolve_compile_scope
from .checkpointing import (checkpoint_is_due, normalize_resume_consumed_micro_batches, resolve_data_resume_policy,
                            save_periodic_checkpoint_if_due)
from .export_helpers import export_discriminator_hf_subprocess
from .metrics import (append_metrics_jsonl_row, build_runtime_resolved_config, flush_loggers,
                      write_nonfinite_debug_artifact)
from .run_config import persist_or_validate_run_configs, write_runtime_resolved_config
from .run_management import (load_checkpoint_progress_metadata, prepare_output_dir, resolve_output_dir_for_ranks,
                             resolve_resume_checkpoint_for_ranks, save_training_checkpoint)
from .runtime import (build_dataloader, build_engine, build_model, build_tokenizer, build_training_dataset_and_collator,
                      cycle_dataloader)
from .tracker_utils import init_trackers, setup_wandb_watch, upload_wandb_config_files
from .trainer import Trainer

logger = logging.getLogger(__name__)


def _resolve_dirs(ctx: DistContext, train_cfg: TrainConfig, logging_cfg: LoggingConfig, config_path) -> tuple[Path, Path]:
    out = resolve_output_dir_for_ranks(ctx, output_dir=train_cfg.checkpoint.output_dir,
                                       project_name=logging_cfg.project_name, config_path=config_path,
                                       run_name=logging_cfg.run_name)
    log_dir = Path(logging_cfg.output_dir) if logging_cfg.output_dir else out / "logs"
    return out, log_dir


def _validate(model_cfg, data_cfg, train_cfg, optim_cfg, logging_cfg) -> None:
    validate_config(Config(model=model_cfg, data=data_cfg, train=train_cfg, optim=optim_cfg, logging=logging_cfg))


def run_pretraining_dry_run(*, model_cfg: ModelConfig, data_cfg: DataConfig, train_cfg: TrainConfig,
                            optim_cfg: OptimConfig | None = None, logging_cfg: LoggingConfig | None = None,
                            config_path: str | Path | None = None) -> dict[str, Any]:
    """Preflight without training or writing: config, paths, resume target, tokenizer + one collated batch, backbone configs."""
    optim_cfg, logging_cfg = optim_cfg or OptimConfig(), logging_cfg or LoggingConfig()
    _validate(model_cfg, data_cfg, train_cfg, optim_cfg, logging_cfg)
    ctx = DistContext()
    out, log_dir = _resolve_dirs(ctx, train_cfg, logging_cfg, config_path)
    resume = resolve_resume_checkpoint_for_ranks(ctx, output_dir=out,
                                                 resume_from_checkpoint=train_cfg.checkpoint.resume_from_checkpoint)
    if out.exists() and any(out.iterdir()) and not (train_cfg.checkpoint.overwrite_output_dir or resume):
        raise ValueError(f"Output directory exists and is not empty: {out}. "
                         "Set train.overwrite_output_dir=true or set train.resume_from_checkpoint.")
    tok = build_tokenizer(model_cfg)
    dataset, collator = build_training_dataset_and_collator(data_cfg=data_cfg, train_cfg=train_cfg, tokenizer=tok,
                                                            process_index=0, num_processes=1)
    it = iter(dataset)
    batch = collator([next(it) for _ in range(int(train_cfg.per_device_train_batch_size))])
    from deberta_b200.models import build_backbone_configs

    from .loop_utils import count_input_tokens_for_batch

    build_backbone_configs(model_cfg=model_cfg, tokenizer=tok, max_position_embeddings=int(data_cfg.packing.max_seq_length))
    return {
        "checkpoint_output_dir": str(out), "logging_output_dir": str(log_dir), "resume_checkpoint": resume,
        "effective_compile_scope": (resolve_compile_scope(
            requested_scope=train_cfg.compile.scope, backbone_type=model_cfg.backbone_type,
            block_cross_document_attention=bool(data_cfg.packing.block_cross_document_attention))[0]
            if train_cfg.compile.enabled else "none (compile disabled; hot operators are precompiled sm_100a kernels)"),
        "sample_batch_shape": tuple(batch["input_ids"].shape),
        "sample_active_tokens": int(count_input_tokens_for_batch(batch)), "tokenizer_vocab_size": len(tok),
    }


def run_pretraining(*, model_cfg: ModelConfig, data_cfg: DataConfig, train_cfg: TrainConfig,
                    optim_cfg: OptimConfig | None = None, logging_cfg: LoggingConfig | None = None,
                    config_path: str | Path | None = None, hf_dataset: Any = None) -> dict[str, Any]:
    """Train until ``train.max_steps``; returns a small summary (final step, losses, output directory)."""
    optim_cfg, logging_cfg = optim_cfg or OptimConfig(), logging_cfg or LoggingConfig()
    ctx = init_distributed()
    setup_process_logging(ctx.is_main_process)
    _validate(model_cfg, data_cfg, train_cfg, optim_cfg, logging_cfg)
    _sync_legacy_train_aliases(train_cfg=train_cfg, optim_cfg=optim_cfg, logging_cfg=logging_cfg)
    if train_cfg.tf32 and torch.cuda.is_available():
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    ck = train_cfg.checkpoint
    out_dir, log_dir = _resolve_dirs(ctx, train_cfg, logging_cfg, config_path)
    prepare_output_dir(output_dir=out_dir, overwrite_output_dir=ck.overwrite_output_dir,
                       resume_from_checkpoint=ck.resume_from_checkpoint, is_main_process=ctx.is_main_process)
    ctx.wait_for_everyone()
    resume = resolve_resume_checkpoint_for_ranks(ctx, output_dir=out_dir, resume_from_checkpoint=ck.resume_from_checkpoint)
    sections = {"model": model_cfg, "data": data_cfg, "train": train_cfg, "optim": optim_cfg, "logging": logging_cfg}
    persist_or_validate_run_configs(output_dir=out_dir, logging_dir=log_dir, sections=sections,
                                    config_path=Path(config_path) if config_path else None, resume_checkpoint=resume,
                                    is_main_process=ctx.is_main_process)
    ctx.wait_for_everyone()
    torch.manual_seed(int(train_cfg.seed) + ctx.rank)  # device-specific seeds, as `set_seed(device_specific=True)`
    tok = build_tokenizer(model_cfg)
    dataset, collator = build_training_dataset_and_collator(data_cfg=data_cfg, train_cfg=train_cfg, tokenizer=tok,
                                                            process_index=ctx.rank, num_processes=ctx.world_size,
                                                            hf_dataset=hf_dataset)
    loader = build_dataloader(dataset=dataset, collator=collator, train_cfg=train_cfg)
    model, disc_cfg, gen_cfg = build_model(model_cfg=model_cfg, tokenizer=tok,
                                           max_seq_length=int(data_cfg.packing.max_seq_length),
                                           load_pretrained_weights=resume is None)
    set_nvtx(bool(logging_cfg.debug.nvtx))
    engine = build_engine(model=model, ctx=ctx, train_cfg=train_cfg, optim_cfg=optim_cfg)
    trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=train_cfg, optim_cfg=optim_cfg,
                      pad_token_id=getattr(tok, "pad_token_id", None))
    model.sync_discriminator_embeddings_from_generator()
    compile_scope, compile_reason, _ = maybe_compile_model(model, train_cfg=train_cfg, model_cfg=model_cfg, data_cfg=data_cfg)
    if compile_scope is not None and ctx.is_main_process:
        from deberta_b200.run_layout import RUN_METADATA_FILE
        from deberta_b200.utils.io import dump_json

        from .run_config import build_run_metadata

        dump_json(build_run_metadata(effective_compile_scope=compile_scope, compile_scope_reason=compile_reason),
                  out_dir / RUN_METADATA_FILE)
    # what the run really uses (derived generator shape, vocabulary size, collective path) goes to config_resolved.yaml
    # and to the tracker instead of the raw sections (``entrypoint.py:619-633`` of the reference)
    resolved = build_runtime_resolved_config(
        sections=sections, disc_config=disc_cfg, gen_config=gen_cfg, tokenizer=tok,
        runtime={"world_size": ctx.world_size, "device": str(engine.device), "parallelism": engine.parallelism,
                 "compute_dtype": str(engine.compute_dtype).replace("torch.", ""),
                 "collectives": ("peer-memory kernels" + (" (multimem)" if engine.comm.multicast else ""))
                 if engine.comm is not None else ("nccl" if ctx.backend == "nccl" else (ctx.backend or "none"))})
    if ctx.is_main_process:
        write_runtime_resolved_config(logging_dir=log_dir, payload=resolved)
    trackers = init_trackers(logging_cfg=logging_cfg, logging_dir=log_dir, run_name=logging_cfg.run_name,
                             config_payload=resolved, is_main_process=ctx.is_main_process)
    setup_wandb_watch(tracker=trackers, model=model, watch_mode=logging_cfg.wandb.watch,
                      log_freq=logging_cfg.wandb.watch_log_freq)
    if ctx.is_main_process and logging_cfg.wandb.enabled:
        upload_wandb_config_files(tracker=trackers, logging_dir=log_dir, config_source_path=config_path,
                                  run_name=logging_cfg.run_name)
    metrics_path = log_dir / "metrics.jsonl.gz"
    debug_dir = log_dir / "debug"
    # a skipped (non-finite) window always leaves a debug record, as in the reference (``training/metrics.py:195-272``)
    trainer.on_nonfinite = lambda step, norms: ctx.is_main_process and write_nonfinite_debug_artifact(
        debug_dir=debug_dir, step=step, what="grad_norm", losses={}, lrs=trainer.current_lrs(),
        lr_mult=trainer.lr_mult, extra={"grad_norms": {k: repr(v) for k, v in norms.items()}})

    # ---- resume --------------------------------------------------------------------------------------
    start_epoch = 0
    ga = int(train_cfg.gradient_accumulation_steps)
    digest = trainer.optimizer_param_digest()
    if resume:
        load_training_state(resume, engine=engine, trainer=trainer, ctx=ctx)
        model.sync_discriminator_embeddings_from_generator()
        consumed, lr_mult, stored_digest, step, stored_ga = load_checkpoint_progress_metadata(Path(resume))
        if stored_digest is not None and stored_digest != digest:
            raise RuntimeError("Optimizer parameter order of the checkpoint differs from the current model "
                               f"(checkpoint={stored_digest}, current={digest}); refusing to reuse Adam state.")
        if stored_ga is not None and stored_ga != ga:
            raise ValueError(f"Checkpoint was written with gradient_accumulation_steps={stored_ga}, current is {ga}.")
        if step is not None:
            trainer.global_step = int(step)
        trainer.lr_mult = float(lr_mult)
        consumed = normalize_resume_consumed_micro_batches(consumed_micro_batches=consumed or 0,
                                                           global_step=trainer.global_step, ga_steps=ga)
        replay, start_epoch, why = resolve_data_resume_policy(train_cfg=ck, consumed_micro_batches=consumed,
                                                              global_step=trainer.global_step)
        trainer.consumed_micro_batches = consumed
        logger.info("Resumed from %s at step %d (%s)", resume, trainer.global_step, why)
    batches = cycle_dataloader(loader, start_epoch=start_epoch)
    if resume and replay:
        for _ in range(trainer.consumed_micro_batches):
            next(batches)

    # ---- loop ------------------------------------------------------------------------------------------
    max_steps, log_every = int(train_cfg.max_steps), int(logging_cfg.logging_steps)
    pending: list[Any] = []
    t_last, tok_last, tokens_seen, last_saved = time.perf_counter(), 0.0, 0.0, -1
    summary: dict[str, Any] = {"output_dir": str(out_dir)}
    crashed = False

    def save_state(directory: str) -> None:
        save_training_state(directory, engine=engine, trainer=trainer, ctx=ctx)

    save_kw = dict(save_total_limit=int(ck.save_total_limit), optimizer_param_digest=digest, gradient_accumulation_steps=ga)
    watchdog = heartbeat = None
    di = train_cfg.distributed
    if float(di.step_deadline_s) > 0:  # host-side liveness report when no optimizer step completes in time
        from .watchdog import StepWatchdog

        watchdog = StepWatchdog(float(di.step_deadline_s), report_dir=out_dir / "watchdog").start()
    if float(di.heartbeat_s) > 0 and ctx.distributed:
        # every rank reports (step, time) through the process-group store; a rank whose report is older than the
        # limit is named in an error before the next window is queued, instead of a collective waiting for it
        import torch.distributed as dist

        from .watchdog import RankHeartbeat

        heartbeat = RankHeartbeat(dist.distributed_c10d._get_default_store(), ctx.rank, ctx.world_size)
        heartbeat.beat(trainer.global_step)
        ctx.wait_for_everyone()
    weights = (float(train_cfg.objective.gen_loss_weight), float(train_cfg.objective.disc_loss_weight))
    tokens_seen_global = 0.0
    try:
        while trainer.global_step < max_steps:
            if heartbeat is not None:
                stale = heartbeat.stale_ranks(float(di.heartbeat_s))
                if stale:
                    raise RuntimeError(f"rank(s) {stale} sent no heartbeat for {float(di.heartbeat_s):.0f} s "
                                       f"(last completed step {trainer.global_step}); stopping before the next collective.")
            stats = trainer.train_window([next(batches) for _ in range(ga)])
            if watchdog is not None:
                watchdog.beat(trainer.global_step)
            if heartbeat is not None:
                heartbeat.beat(trainer.global_step)
            pending.append(stats)
            tokens_seen += stats.input_tokens
            step = trainer.global_step
            if log_every > 0 and (step % log_every == 0 or step == max_steps):
                row = _reduce_window_stats(ctx, pending, engine.device, loss_weights=weights)
                now = time.perf_counter()
                global_tokens = float(ctx.reduce(torch.tensor([tokens_seen - tok_last], dtype=torch.float64), "sum")[0])
                tokens_seen_global += global_tokens
                lrs = trainer.current_lrs()
                # `lr` is the discriminator's (the schedule the reference reports, ``entrypoint.py:1493-1501``)
                row.update(step=step, lr=float(lrs.get("discriminator", next(iter(lrs.values())))), lr_mult=trainer.lr_mult,
                           input_tokens_per_sec=global_tokens / max(now - t_last, 1e-9),
                           input_tokens_seen=tokens_seen_global, skipped_steps=trainer.skipped_steps,
                           **{f"lr_{name}": float(v) for name, v in lrs.items()})
                t_last, tok_last, pending = now, tokens_seen, []
                if ctx.is_main_process:
                    logger.info("step %d | loss %.4f | gen %.4f | disc %.4f | acc %.4f | lr %.3e | %.0f tok/s", step,
                                row["loss"], row["gen_loss"], row["disc_loss"], row["disc_acc"], row["lr"],
                                row["input_tokens_per_sec"])
                    trackers.log({k: v for k, v in row.items() if isinstance(v, (int, float))}, step)
                    if logging_cfg.debug.metrics:
                        append_metrics_jsonl_row(metrics_path, row)
                summary.update(row)
            if checkpoint_is_due(global_step=step, save_steps=int(ck.save_steps), last_saved_step=last_saved):
                trainer.resolve_pending()  # on every rank, before anything of the optimizer or the LR multiplier is read
                last_saved = save_periodic_checkpoint_if_due(
                    ctx=ctx, save_state=save_state, output_dir=out_dir, global_step=step, save_steps=int(ck.save_steps),
                    last_saved_step=last_saved, consumed_micro_batches=trainer.consumed_micro_batches,
                    lr_mult=trainer.lr_mult, **save_kw)
        trainer.resolve_pending()  # the last window's outcome (kernel status, skipped update) before the run ends
    except BaseException as exc:
        crashed = True
        if ctx.is_main_process:
            crash_row = {"event": "crash", "step": trainer.global_step, "crash": 1,
                         "error": f"{type(exc).__name__}: {exc}"}
            append_metrics_jsonl_row(metrics_path, crash_row)
            with contextlib.suppress(Exception):  # the tracker gets the row too (``entrypoint.py:1886-2005``)
                trackers.log({"crash": 1, "crash_step": trainer.global_step}, trainer.global_step)
                trackers.set_summary({"crashed": True, "crash_type": type(exc).__name__, "crash_step": trainer.global_step})
        raise
    finally:
        if watchdog is not None:
            watchdog.stop()
        flush_loggers()
        # a crash checkpoint is only safe without peers (a collective save could deadlock on a dead rank)
        if (not crashed or ctx.world_size == 1) and trainer.global_step > 0 and last_saved != trainer.global_step:
            try:
                with contextlib.suppress(Exception):
                    trainer.resolve_pending()
                save_training_checkpoint(ctx=ctx, save_state=save_state,
                                         checkpoint_dir=out_dir / f"checkpoint-{trainer.global_step}", output_dir=out_dir,
                                         consumed_micro_batches=trainer.consumed_micro_batches, log_label="final",
                                         lr_mult=trainer.lr_mult, global_step=trainer.global_step, **save_kw)
                last_saved = trainer.global_step
            except Exception as e:  # never mask the original error
                logger.warning("Final checkpoint failed: %s", e)
        trackers.finish(crashed=crashed)
    if ck.export_hf_final and ctx.is_main_process and last_saved > 0:
        export_discriminator_hf_subprocess(checkpoint_dir=out_dir / f"checkpoint-{last_saved}",
                                           output_dir=out_dir / FINAL_HF_DIR)
    ctx.wait_for_everyone()
    summary.update(global_step=trainer.global_step, last_checkpoint=str(out_dir / f"checkpoint-{last_saved}"))
    ctx.shutdown()
    return summary


def _reduce_window_stats(ctx: DistContext, windows: list[Any], device: torch.device,
                         loss_weights: tuple[float, float] = (1.0, 1.0)) -> dict[str, float]:
    """Globally token-weighted means over the windows since the last log line (one small all-reduce).

    ``loss`` is the combined objective ``w_g·gen + w_d·disc`` (``rtd.py:1241-1244`` of the reference).
    """
    acc = torch.zeros(6, dtype=torch.float32, device=device)
    zero_gen = zero_disc = 0
    for w in windows:
        acc += torch.stack([w.gen_loss_tokens, w.disc_loss_tokens, w.disc_acc_tokens, w.disc_pos,
                            torch.tensor(w.gen_tokens, device=device), torch.tensor(w.disc_tokens, device=device)])
        zero_gen += int(w.zero_gen_window)
        zero_disc += int(w.zero_disc_window)
    acc = ctx.reduce(acc, "sum").cpu()
    g_tok, d_tok = max(float(acc[4]), 1.0), max(float(acc[5]), 1.0)
    gen, disc = float(acc[0]) / g_tok, float(acc[1]) / d_tok
    return {"gen_loss": gen, "disc_loss": disc, "loss": loss_weights[0] * gen + loss_weights[1] * disc,
            "disc_acc": float(acc[2]) / d_tok,
            "disc_pos_frac": float(acc[3]) / d_tok, "zero_gen_windows": zero_gen, "zero_disc_windows": zero_disc}
