"""Step-by-step comparison of the two execution paths: fp32 PyTorch oracle vs bf16 sm_100a kernels.

Usage::

    python -m deberta_b200.tools.kernel_drift_probe [--config CFG.yaml] [--steps 8] [--micro-batch 8] [--seq-len 128]
        [--model-size xsmall|small|base] [--backbone hf_deberta_v2|rope] [--tolerance 0.05] [--json]

Both arms build the same model from the same seed, see the same synthetic batches and take the same optimizer
steps through the real trainer; the probe prints per step the generator / discriminator losses and gradient norms
of both arms, their relative difference, and the step time (``perf_counter`` around a device synchronise, after
one warm-up step). It is the counterpart of the reference's eager-vs-compiled probe
(``tools/compile_drift_probe.py:382-473``): here the two paths are "PyTorch ops" and "hand-written kernels".
Without a GPU both arms run the PyTorch path (the drift is then the run-to-run noise floor, normally 0).
Exit status 1 when the largest relative loss difference exceeds ``--tolerance``.
"""

from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def _build_cfg(args: argparse.Namespace, precision: str):
    from deberta_b200.config import Config, DataConfig, ModelConfig, OptimConfig, TrainConfig, load_config, validate_config

    if args.config:
        from deberta_b200.config import apply_dotted_override

        cfg = apply_dotted_override(load_config(args.config), f"train.mixed_precision={precision}")
        validate_config(cfg)
        return cfg
    hf = {"model_size": args.model_size} if args.backbone == "hf_deberta_v2" else {}
    cfg = Config(
        model=ModelConfig(backbone_type=args.backbone, embedding_sharing="gdes", hf=hf,
                          tokenizer={"name_or_path": f"synthetic:{args.vocab}"}),
        data=DataConfig(dataset_name="synthetic", max_seq_length=args.seq_len),
        train=TrainConfig(mixed_precision=precision, per_device_train_batch_size=args.micro_batch,
                          gradient_accumulation_steps=1, decoupled_training=True, dataloader_num_workers=0),
        optim=OptimConfig(),
    )
    validate_config(cfg)
    return cfg


def _run_arm(args: argparse.Namespace, precision: str, device: torch.device) -> list[dict[str, float]]:
    from deberta_b200.parallel.dist import DistContext
    from deberta_b200.training.runtime import build_engine, build_model, build_tokenizer
    from deberta_b200.training.trainer import Trainer

    cfg = _build_cfg(args, precision)
    torch.manual_seed(args.seed)
    tok = build_tokenizer(cfg.model)
    model, _, _ = build_model(model_cfg=cfg.model, tokenizer=tok, max_seq_length=args.seq_len)
    ctx = DistContext(device=device)
    engine = build_engine(model=model, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim)
    trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim,
                      pad_token_id=tok.pad_token_id, synchronous=True)
    batches = _batches(args, tok)
    rows = []
    for i, b in enumerate(batches):
        torch.manual_seed(args.seed + 1000 + i)  # same sampling noise stream in both arms
        if device.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        st = trainer.train_window([{k: v.to(device) for k, v in b.items()}])
        if device.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        rows.append({"step": i, "gen_loss": float(st.gen_loss_tokens) / max(st.gen_tokens, 1.0),
                     "disc_loss": float(st.disc_loss_tokens) / max(st.disc_tokens, 1.0),
                     "gen_grad_norm": float(st.grad_norms.get("generator", torch.zeros(()))),
                     "disc_grad_norm": float(st.grad_norms.get("discriminator", torch.zeros(()))), "ms": dt * 1e3})
    return rows


def _batches(args: argparse.Namespace, tok):
    from deberta_b200.data import DebertaV3ElectraCollator, MLMConfig, PackedStreamingConfig, PackedStreamingDataset
    from deberta_b200.data.synthetic import SyntheticTextDataset

    ds = PackedStreamingDataset(hf_dataset=SyntheticTextDataset(vocab_size=args.vocab, zipf_s=1.1, mean_doc_len=40, seed=args.seed),
                                tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=args.seq_len, seed=args.seed))
    col = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(mlm_probability=0.15), packed_sequences=True,
                                   block_cross_document_attention=False)
    it = iter(ds)
    torch.manual_seed(args.seed)
    return [col([next(it) for _ in range(args.micro_batch)]) for _ in range(args.steps)]


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", default=None, help="YAML/JSON config; default: a scratch model of --model-size")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--model-size", default="xsmall")
    ap.add_argument("--backbone", default="hf_deberta_v2", choices=("hf_deberta_v2", "rope"))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tolerance", type=float, default=0.05)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    gpu = torch.cuda.is_available()
    device = torch.device("cuda" if gpu else "cpu")
    ref = _run_arm(args, "no", device)
    ker = _run_arm(args, "bf16" if gpu else "no", device)
    worst = 0.0
    rows = []
    for a, b in zip(ref, ker):
        rel = max(abs(a[k] - b[k]) / max(abs(a[k]), 1e-6) for k in ("gen_loss", "disc_loss"))
        worst = max(worst, rel)
        rows.append({"step": a["step"], "ref": a, "kernels": b, "rel_loss_diff": rel})
    if args.json:
        print(json.dumps({"kernel_path": gpu, "max_rel_loss_diff": worst, "steps": rows}, indent=1))
    else:
        print(f"arms: fp32 PyTorch ops vs {'bf16 sm_100a kernels' if gpu else 'fp32 PyTorch ops (no GPU here)'}")
        print(f"{'step':>4} {'gen ref':>9} {'gen ker':>9} {'disc ref':>9} {'disc ker':>9} {'|g| ref':>9} {'|g| ker':>9} {'rel':>8} {'ms ref':>8} {'ms ker':>8}")
        for r in rows:
            a, b = r["ref"], r["kernels"]
            print(f"{r['step']:>4} {a['gen_loss']:>9.4f} {b['gen_loss']:>9.4f} {a['disc_loss']:>9.4f} {b['disc_loss']:>9.4f} "
                  f"{a['disc_grad_norm']:>9.3f} {b['disc_grad_norm']:>9.3f} {r['rel_loss_diff']:>8.4f} {a['ms']:>8.1f} {b['ms']:>8.1f}")
        print(f"max relative loss difference: {worst:.4f} (tolerance {args.tolerance})")
    return 0 if worst <= args.tolerance else 1


if __name__ == "__main__":
    sys.exit(main())
