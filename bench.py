"""Headline benchmark: RTD pretraining tokens/s, DeBERTa-v3-base, seq 512, micro-batch 32 per GPU.

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run`` for N > 1)
runs K optimizer steps of the flagship configuration on synthetic packed Zipf(1.1) token
streams with random-init weights and prints ONE JSON line on rank 0. A step is one
gradient-accumulation window of ``--ga`` micro-batches followed by the generator and
discriminator optimizer updates (decoupled training, two AdamW optimizers, clipping).

Two numbers are measured for this framework:
* ``value``  — device-timed (CUDA events, max over ranks) with micro-batches already on the GPU;
* ``e2e``    — the same steps through ``Trainer.train_window`` fed from pinned host memory, with
  the host→device copy of every micro-batch and a device→host read of the step's losses inside
  the timed region.

``--impl reference`` runs the unmodified reference package installed under ``baseline/_ref``
(its model classes, optimizer builders and eager code path) on the same data and schedule.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
import warnings
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

SEQ_LEN = 512
MICRO_BATCH = 32
VOCAB = 128_100
BASELINE_TOKENS_PER_S = None  # the reference publishes no number
# Secondary configurations (per-GPU micro-batch as named; grad-accum 2 keeps a run short).
PRESETS = {
    "v3-small": dict(model_size="small", micro_batch=64, ga=2, parallelism="ddp"),
    "rope-2048": dict(backbone="rope", seq_len=2048, micro_batch=8, ga=2, rope_ffn="swiglu", gen_layers=6, block_docs=True,
                      mean_doc_len=600),
    "rope-4096": dict(backbone="rope", seq_len=4096, micro_batch=4, ga=2, rope_ffn="swiglu", gen_layers=6, block_docs=True,
                      mean_doc_len=1200, grad_ckpt=True),
}


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=4)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--ga", type=int, default=8, help="micro-batches per optimizer step (2048-sequence global batch at 8 GPUs)")
    p.add_argument("--impl", choices=("ours", "reference"), default="ours")
    p.add_argument("--micro-batch", type=int, default=MICRO_BATCH)
    p.add_argument("--seq-len", type=int, default=SEQ_LEN)
    p.add_argument("--model-size", default="base")
    p.add_argument("--backbone", choices=("hf_deberta_v2", "rope"), default="hf_deberta_v2",
                   help="rope: the RoPE/RMSNorm/SwiGLU family at its config defaults (secondary benchmark)")
    p.add_argument("--parallelism", choices=("ddp", "zero", "fsdp"), default="zero")
    p.add_argument("--block-docs", action="store_true",
                   help="rope backbone only: packed documents do not attend to each other (data.packing."
                        "block_cross_document_attention); the collator then emits document ids")
    p.add_argument("--rope-ffn", choices=("mlp", "swiglu"), default="mlp", help="feed-forward type of the rope backbone")
    p.add_argument("--gen-layers", type=int, default=0, help="generator depth (0: derived from the discriminator)")
    p.add_argument("--grad-ckpt", action="store_true", help="activation checkpointing per layer (both arms)")
    p.add_argument("--mean-doc-len", type=int, default=60, help="mean length of the synthetic documents (tokens)")
    p.add_argument("--preset", choices=tuple(PRESETS), default=None,
                   help="one of the secondary benchmark configurations (sets the flags above)")
    p.add_argument("--curve", type=int, default=0,
                   help="instead of timing: train this many steps at a fixed seed and print the loss curve (JSON)")
    p.add_argument("--no-dependent-launch", action="store_true",
                   help="launch every kernel the ordinary way (A/B switch for programmatic dependent launch)")
    args = p.parse_args()
    if args.preset:
        for k, v in PRESETS[args.preset].items():
            setattr(args, k, v)
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for name, val in zip(names, r[5:9]):
                    if val.lower() == "active":
                        reasons.add(name)
        smax = next((float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()), None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def synthetic_batches(n: int, micro_batch: int, seq_len: int, seed: int, pin: bool,
                      block_docs: bool = False, mean_doc_len: int = 60) -> list[dict[str, torch.Tensor]]:
    """``n`` collated micro-batches from the synthetic corpus through the real packer + collator."""
    from deberta_b200.data import DebertaV3ElectraCollator, MLMConfig, PackedStreamingConfig, PackedStreamingDataset
    from deberta_b200.data.synthetic import SyntheticTextDataset, SyntheticTokenizer

    tok = SyntheticTokenizer(VOCAB)
    ds = PackedStreamingDataset(hf_dataset=SyntheticTextDataset(vocab_size=VOCAB, zipf_s=1.1, mean_doc_len=int(mean_doc_len), seed=seed),
                                tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=seq_len, seed=seed))
    col = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(mlm_probability=0.15, mask_token_prob=1.0,
                                                                random_token_prob=0.0), packed_sequences=True,
                                   block_cross_document_attention=bool(block_docs))
    it = iter(ds)
    out = []
    torch.manual_seed(seed)
    for _ in range(n):
        b = col([next(it) for _ in range(micro_batch)])
        if pin:
            b = {k: v.pin_memory() for k, v in b.items()}
        out.append(b)
    return out


def curve_warmup(args: argparse.Namespace) -> int:
    """Warm-up length of a loss-curve run (a tenth of it), the same in both arms."""
    return max(1, int(args.curve) // 10)


def curve_batches(args: argparse.Namespace, rank: int):
    """The micro-batches of a loss-curve run, window by window: the same stream in both arms."""
    per = 64  # windows generated at a time
    done = 0
    while done < args.curve:
        n = min(per, args.curve - done)
        chunk = synthetic_batches(n * args.ga, args.micro_batch, args.seq_len, seed=5000 + 97 * rank + done, pin=False,
                                  block_docs=getattr(args, "block_docs", False), mean_doc_len=args.mean_doc_len)
        for w in range(n):
            yield chunk[w * args.ga:(w + 1) * args.ga]
        done += n


def curve_report(args: argparse.Namespace, impl: str, gen: list[float], disc: list[float], world: int) -> dict:
    """One JSON object for ``--curve``: per-step generator loss, 100-step means of both losses."""
    mean = lambda xs: sum(xs) / max(len(xs), 1)  # noqa: E731
    return {"impl": impl, "curve_steps": len(gen), "n_gpus": world, "seed": 1234,
            "config": {"model_size": args.model_size, "backbone": args.backbone, "micro_batch": args.micro_batch,
                       "grad_accum": args.ga, "seq_len": args.seq_len, "lr": 2e-4, "warmup_steps": curve_warmup(args)},
            "gen_loss": [round(x, 5) for x in gen], "disc_loss": [round(x, 5) for x in disc],
            "gen_loss_mean100": [round(mean(gen[i:i + 100]), 5) for i in range(0, len(gen), 100)],
            "disc_loss_mean100": [round(mean(disc[i:i + 100]), 5) for i in range(0, len(disc), 100)]}


def build_config(args: argparse.Namespace):
    from deberta_b200.config import Config, DataConfig, ModelConfig, OptimConfig, TrainConfig, validate_config

    cfg = Config(
        model=(ModelConfig(profile="deberta_v3_parity", backbone_type="hf_deberta_v2", embedding_sharing="gdes",
                           hf={"model_size": args.model_size}, tokenizer={"name_or_path": f"synthetic:{VOCAB}"})
               if args.backbone == "hf_deberta_v2" else
               ModelConfig(backbone_type="rope", embedding_sharing="gdes", tokenizer={"name_or_path": f"synthetic:{VOCAB}"},
                           rope={"ffn_type": args.rope_ffn})),
        data=DataConfig(dataset_name="synthetic", dataset_config_name=f"zipf1.1-mean60-vocab{VOCAB}",
                        max_seq_length=args.seq_len),
        train=TrainConfig(per_device_train_batch_size=args.micro_batch, gradient_accumulation_steps=args.ga,
                          mixed_precision="bf16", max_steps=10_000, disc_loss_weight=50.0, mask_token_prob=1.0,
                          random_token_prob=0.0, dataloader_num_workers=0),
        optim=OptimConfig(learning_rate=2e-4, adam_beta2=0.98, adam_epsilon=1e-6,
                          warmup_steps=curve_warmup(args) if args.curve else 10_000),
    )
    from deberta_b200.config import apply_dotted_override

    if args.gen_layers > 0:
        cfg = apply_dotted_override(cfg, f"model.generator.num_hidden_layers={int(args.gen_layers)}")
    if args.grad_ckpt:
        cfg = apply_dotted_override(cfg, "model.gradient_checkpointing=true")
    if args.block_docs:
        cfg = apply_dotted_override(cfg, "data.packing.block_cross_document_attention=true")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        validate_config(cfg)
    return cfg


def describe_model(args: argparse.Namespace) -> str:
    if args.backbone == "hf_deberta_v2":
        return f"deberta-v3-{args.model_size} RTD (GDES, EMD" + (f", {args.gen_layers}L gen" if args.gen_layers else "") + ")"
    return (f"rope RTD (12L, {args.rope_ffn} FFN, " + (f"{args.gen_layers}L gen" if args.gen_layers else "derived gen") +
            (", activation checkpointing" if args.grad_ckpt else "") + ", GDES)")


def run_ours(args: argparse.Namespace) -> dict:
    from deberta_b200.ops import _lib
    from deberta_b200.parallel.dist import init_distributed
    from deberta_b200.training.runtime import build_engine, build_model, build_tokenizer
    from deberta_b200.training.trainer import Trainer

    ctx = init_distributed()
    if ctx.device.type != "cuda":
        raise SystemExit("bench.py needs a CUDA device")
    if getattr(args, "no_dependent_launch", False):
        _lib.set_dependent_launch(False)
    cfg = build_config(args)
    torch.manual_seed(1234)
    tok = build_tokenizer(cfg.model)
    model, _, _ = build_model(model_cfg=cfg.model, tokenizer=tok, max_seq_length=args.seq_len)
    engine = build_engine(model=model, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim, parallelism=args.parallelism)
    trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim,
                      pad_token_id=tok.pad_token_id)
    if args.curve:
        rows = []
        for window in curve_batches(args, ctx.rank):
            st = trainer.train_window(window)
            rows.append(torch.stack([st.gen_loss_tokens / max(st.gen_tokens, 1.0), st.disc_loss_tokens / max(st.disc_tokens, 1.0)]))
        trainer.wait_for_side_stream()
        trainer.resolve_pending()
        vals = torch.stack(rows).cpu().tolist()
        _lib.check_status()
        ctx.shutdown()
        return curve_report(args, "ours", [v[0] for v in vals], [v[1] for v in vals], ctx.world_size) if ctx.is_main_process else {}
    host = synthetic_batches(args.ga, args.micro_batch, args.seq_len, seed=100 + ctx.rank, pin=True,
                             block_docs=getattr(args, "block_docs", False), mean_doc_len=args.mean_doc_len)
    dev = [trainer.stage_batch(b) for b in host]  # device-resident inputs with their host-side token counts attached
    tokens_per_step = args.ga * args.micro_batch * args.seq_len
    h2d = sum(v.numel() * v.element_size() for b in host for v in b.values())

    def sync_all() -> None:
        ctx.wait_for_everyone()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.train_window(dev)
    # ---- device-timed: inputs resident on the GPU, CUDA events, max over ranks --------------------
    sampler = ClockSampler(ctx.local_rank)
    sync_all()
    if ctx.is_main_process:
        sampler.start()
    launches0 = _lib.LAUNCH_COUNT
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        stats = trainer.train_window(dev)
    end.record()
    sync_all()
    clocks = sampler.stop() if ctx.is_main_process else {}
    launches = _lib.LAUNCH_COUNT - launches0
    ms = torch.tensor([start.elapsed_time(end)], device=ctx.device)
    ms = float(ctx.gather(ms).max())
    # ---- end to end: pinned host batches in, losses out, every step ---------------------------------
    sync_all()
    t0 = time.perf_counter()
    d2h = 0
    for _ in range(args.steps):
        stats = trainer.train_window(host)
        out = torch.stack([stats.gen_loss_tokens, stats.disc_loss_tokens, stats.disc_acc_tokens]).cpu()
        d2h = out.numel() * out.element_size()
    sync_all()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=ctx.device)
    e2e_s = float(ctx.gather(e2e_s).max())
    _lib.check_status()
    gen_loss = float(stats.gen_loss_tokens) / max(stats.gen_tokens, 1.0)
    value = tokens_per_step * ctx.world_size * args.steps / (ms / 1e3)
    result = {
        "metric": (f"RTD pretrain tokens/s, DeBERTa-v3-{args.model_size} seq{args.seq_len}, max over ranks" if args.backbone == "hf_deberta_v2"
                   else f"RTD pretrain tokens/s, rope backbone seq{args.seq_len}, max over ranks"), "value": value, "unit": "tokens/s",
        "n_gpus": ctx.world_size, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic packed Zipf(1.1) token streams, random-init weights", "impl": "ours",
        "config": {"model": ("deberta-v3-base RTD (12L disc + 6L gen, GDES, EMD)"
                             if (args.backbone == "hf_deberta_v2" and args.model_size == "base" and not args.gen_layers)
                             else describe_model(args)),
                   "preset": args.preset, "mean_doc_len": args.mean_doc_len,
                   "global_batch": args.micro_batch * args.ga * ctx.world_size, "micro_batch": args.micro_batch,
                   "grad_accum": args.ga, "seq_len": args.seq_len, "block_cross_document_attention": bool(args.block_docs),
                   "parallelism": f"dp{ctx.world_size}" + {"zero": "-zero1", "fsdp": "-fullshard", "ddp": "-replicated"}[args.parallelism],
                   "collectives": ("none (1 GPU)" if ctx.world_size == 1 else
                                   ("fused peer-memory kernels" + (" (multimem)" if engine.comm.multicast else "")
                                    if getattr(engine, "comm", None) is not None else "NCCL")),
                   "l2": "activations of one micro-batch (>1 GB) exceed the 126 MB L2 between kernels"},
        "clocks": clocks,
        "e2e": {"value": tokens_per_step * ctx.world_size * args.steps / e2e_s, "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches, "final_gen_loss": gen_loss,
        "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2),
    }
    if getattr(engine, "sharder", None) is not None:
        result["config"]["param_shard_bytes"] = engine.sharder.memory_report()
    ctx.shutdown()
    return result if ctx.is_main_process else {}


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        result = run_reference(args)
    else:
        result = run_ours(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
