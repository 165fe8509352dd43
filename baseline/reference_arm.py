"""Reference arm of ``bench.py``: the unmodified reference package under ``baseline/_ref``.

The reference's own entry point (``deberta train``) needs the ``accelerate`` package, which
is not installed on this image, so its training loop cannot be started as is. This arm
therefore drives the reference's public building blocks exactly the way that loop does
(``training/entrypoint.py:1046-1514`` of the reference): its config classes, its backbone
builders and ``DebertaV3RTDPretrainer``, its optimizer/scheduler builders, its token-weighted
objective helpers, bf16 autocast with fp32 parameters, torch DDP (``find_unused_parameters``
as the reference sets for decoupled training, ``no_sync`` on non-final micro-batches) for
N > 1, ``clip_grad_norm_`` and fused ``torch.optim.AdamW``. Nothing from ``deberta_b200``
runs on this path except the synthetic data source that produces the shared input batches.
"""

from __future__ import annotations

import contextlib
import json
import os
import sys
import time
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"


def unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


class _StubTokenizer:
    """Vocabulary size and special ids only (what the reference's builder reads from a tokenizer)."""

    pad_token_id, cls_token_id, sep_token_id, unk_token_id, mask_token_id = 0, 1, 2, 3, 4
    bos_token_id = eos_token_id = None
    all_special_ids = [0, 1, 2, 3, 4]

    def __init__(self, vocab: int) -> None:
        self.vocab = vocab

    def __len__(self) -> int:
        return self.vocab


def run_reference(args) -> dict:
    if not (REF_DIR / "deberta").exists():
        return unavailable("reference package is not installed under baseline/_ref")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    sys.path.insert(0, str(REF_DIR))
    try:
        from deberta.config import ModelConfig, TrainConfig
        from deberta.modeling.builder import build_backbone_configs, build_backbones
        from deberta.modeling.rtd import DebertaV3RTDPretrainer
        from deberta.training.loop_utils import _count_rtd_tokens_for_batch, _scale_loss_for_backward
        from deberta.training.runtime import _build_decoupled_optimizers, _build_scheduler
    except Exception as e:  # pragma: no cover - depends on the image
        return unavailable(f"reference import failed: {type(e).__name__}: {e}")
    import torch.distributed as dist

    import bench

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(1234)
    if getattr(args, "backbone", "hf_deberta_v2") == "rope":
        model_cfg = ModelConfig(backbone_type="rope", embedding_sharing="gdes",
                                rope={"ffn_type": getattr(args, "rope_ffn", "mlp")},
                                generator=({"num_hidden_layers": int(args.gen_layers)} if getattr(args, "gen_layers", 0) else {}),
                                gradient_checkpointing=bool(getattr(args, "grad_ckpt", False)))
    else:
        model_cfg = ModelConfig(profile="deberta_v3_parity", backbone_type="hf_deberta_v2", embedding_sharing="gdes",
                                hf={"model_size": args.model_size},
                                generator=({"num_hidden_layers": int(args.gen_layers)} if getattr(args, "gen_layers", 0) else {}),
                                gradient_checkpointing=bool(getattr(args, "grad_ckpt", False)))
    train_cfg = TrainConfig(per_device_train_batch_size=args.micro_batch, gradient_accumulation_steps=args.ga,
                            mixed_precision="bf16", max_steps=10_000)
    for k, v in dict(learning_rate=2e-4, generator_learning_rate=-1.0, discriminator_learning_rate=-1.0, weight_decay=0.01,
                     adam_beta1=0.9, adam_beta2=0.98, adam_epsilon=1e-6,
                     warmup_steps=(bench.curve_warmup(args) if getattr(args, "curve", 0) else 10_000),
                     lr_scheduler_type="linear", max_grad_norm=1.0).items():
        object.__setattr__(train_cfg, k, v)
    tok = _StubTokenizer(bench.VOCAB)
    disc_cfg, gen_cfg = build_backbone_configs(model_cfg=model_cfg, tokenizer=tok, max_position_embeddings=args.seq_len)
    disc, gen = build_backbones(model_cfg=model_cfg, disc_config=disc_cfg, gen_config=gen_cfg)
    if model_cfg.gradient_checkpointing:  # as the reference's entrypoint does (training/entrypoint.py:505-510)
        for backbone in (disc, gen):
            try:
                backbone.gradient_checkpointing_enable()
            except (TypeError, AttributeError):
                # transformers >= 5 walks the tree with nn.Module.apply(fn), which the reference's RotaryEmbedding shadows
                # with its own apply(q, k); the encoder's forward only reads this flag (modeling/rope_encoder.py:474-475)
                for mod in backbone.modules():
                    if hasattr(mod, "gradient_checkpointing"):
                        mod.gradient_checkpointing = True
    model = DebertaV3RTDPretrainer(discriminator_backbone=disc, generator_backbone=gen, disc_config=disc_cfg,
                                   gen_config=gen_cfg, embedding_sharing="gdes", tie_generator_word_embeddings=True,
                                   additional_forbidden_token_ids=tok.all_special_ids).to(device)
    gen_opt, disc_opt = _build_decoupled_optimizers(model, train_cfg, mixed_precision="bf16")
    gen_sched, disc_sched = _build_scheduler(gen_opt, train_cfg), _build_scheduler(disc_opt, train_cfg)
    wrapped = model
    if world > 1:
        wrapped = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], find_unused_parameters=True)
    model.sync_discriminator_embeddings_from_generator()
    model.train()
    block_docs = bool(getattr(args, "block_docs", False))
    host = bench.synthetic_batches(args.ga, args.micro_batch, args.seq_len, seed=100 + rank, pin=True, block_docs=block_docs,
                                   mean_doc_len=getattr(args, "mean_doc_len", 60))
    from deberta.training.compile import _build_doc_block_mask  # the reference loop turns document ids into [B,S,S] masks

    def mask_of(b):
        doc = b.get("doc_ids")
        return _build_doc_block_mask(doc) if doc is not None else b.get("attention_mask")

    dev = [{k: v.to(device) for k, v in b.items()} for b in host]
    # loss weights as the reference's profile defaults resolve them: 10 for the DeBERTa-v2 backbone, 50 otherwise
    gen_w, disc_w, ga = 1.0, (10.0 if getattr(args, "backbone", "hf_deberta_v2") == "hf_deberta_v2" else 50.0), args.ga
    if getattr(args, "curve", 0):
        disc_w = 50.0  # loss curves are compared at the objective weights the other arm uses

    def window(batches, counts):
        gen_tot = max(sum(c[0] for c in counts), 1.0)
        disc_tot = max(sum(c[1] for c in counts), 1.0)
        gen_opt.zero_grad(set_to_none=True)
        disc_opt.zero_grad(set_to_none=True)
        cached = []
        last = None
        for i, (b, (g_i, d_i)) in enumerate(zip(batches, counts)):
            b = {k: v.to(device, non_blocking=True) for k, v in b.items()}
            sync = (i == len(batches) - 1) or world == 1
            ctx = contextlib.nullcontext() if sync else wrapped.no_sync()
            with ctx:
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    b["_mask"] = mask_of(b)  # built once per micro-batch, as in the reference loop (entrypoint.py:1119-1121)
                    out = wrapped(input_ids=b["input_ids"], attention_mask=b["_mask"], labels=b["labels"],
                                  phase="generator")
                obj = out.gen_loss_raw * (g_i / gen_tot)
                loss = _scale_loss_for_backward(loss=gen_w * obj, ga_steps=ga, token_weighted_ga=True) / ga
                loss.backward()
            cached.append((b, out.corrupted_input_ids, out.disc_labels, d_i))
            last = out.gen_loss_raw.detach()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        gen_opt.step()
        gen_sched.step()
        gen_opt.zero_grad(set_to_none=True)
        model.sync_discriminator_embeddings_from_generator()
        for i, (b, corrupted, labels, d_i) in enumerate(cached):
            sync = (i == len(cached) - 1) or world == 1
            ctx = contextlib.nullcontext() if sync else wrapped.no_sync()
            with ctx:
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    out = wrapped(input_ids=b["input_ids"], corrupted_input_ids=corrupted, disc_labels=labels,
                                  attention_mask=b["_mask"], phase="discriminator")
                obj = out.disc_loss_raw * (d_i / disc_tot)
                loss = _scale_loss_for_backward(loss=disc_w * obj, ga_steps=ga, token_weighted_ga=True) / ga
                loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        disc_opt.step()
        disc_sched.step()
        disc_opt.zero_grad(set_to_none=True)
        return last, out.disc_loss_raw.detach()

    counts = [_count_rtd_tokens_for_batch(b, pad_token_id=0) for b in host]

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if getattr(args, "curve", 0):  # fixed-seed loss curve instead of timing: same batches as the other arm
        rows = []
        for batches in bench.curve_batches(args, rank):
            g, d = window(batches, [_count_rtd_tokens_for_batch(b, pad_token_id=0) for b in batches])
            rows.append(torch.stack([g.float(), d.float()]))
        vals = torch.stack(rows).cpu().tolist()
        return bench.curve_report(args, "reference", [v[0] for v in vals], [v[1] for v in vals], world) if rank == 0 else {}
    try:
        for _ in range(args.warmup):
            window(dev, counts)
        sampler = bench.ClockSampler(local)
        sync_all()
        if rank == 0:
            sampler.start()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            window(dev, counts)
        e.record()
        sync_all()
        clocks = sampler.stop() if rank == 0 else {}
        ms = torch.tensor([s.elapsed_time(e)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = float(ms)
        sync_all()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            g, d = window(host, counts)
            out = torch.stack([g.float(), d.float()]).cpu()
        sync_all()
        e2e = torch.tensor([time.perf_counter() - t0], device=device)
        if world > 1:
            dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
        e2e = float(e2e)
    except torch.cuda.OutOfMemoryError as err:
        return unavailable(f"reference ran out of GPU memory at micro-batch {args.micro_batch}: {err}")
    tokens = args.ga * args.micro_batch * args.seq_len * world * args.steps
    h2d = sum(v.numel() * v.element_size() for b in host for v in b.values())
    result = {
        "metric": (f"RTD pretrain tokens/s, DeBERTa-v3-{args.model_size} seq{args.seq_len}, max over ranks"
                   if getattr(args, "backbone", "hf_deberta_v2") == "hf_deberta_v2"
                   else f"RTD pretrain tokens/s, rope backbone seq{args.seq_len}, max over ranks"), "value": tokens / (ms / 1e3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic packed Zipf(1.1) token streams, random-init weights", "impl": "reference",
        "config": {"model": ((f"deberta-v3-{args.model_size} RTD" if getattr(args, "backbone", "hf_deberta_v2") == "hf_deberta_v2"
                              else f"rope RTD ({getattr(args, 'rope_ffn', 'mlp')} FFN"
                                   + (", activation checkpointing" if getattr(args, "grad_ckpt", False) else "") + ")")
                             + " (reference modules, eager, bf16 autocast)"),
                   "preset": getattr(args, "preset", None), "mean_doc_len": getattr(args, "mean_doc_len", 60),
                   "global_batch": args.micro_batch * args.ga * world, "micro_batch": args.micro_batch,
                   "grad_accum": args.ga, "seq_len": args.seq_len, "block_cross_document_attention": block_docs,
                   "parallelism": f"ddp{world}",
                   "driver": "reference building blocks driven as in its decoupled loop; `accelerate` is not installed"},
        "clocks": clocks,
        "e2e": {"value": tokens / e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
        "gpu_launches": 0, "final_gen_loss": float(out[0]),
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}
