"""Kernel time shares of one optimizer step (``torch.profiler`` on one gradient-accumulation window).

Usage::

    python -m deberta_b200.tools.step_kernel_shares [--backbone hf_deberta_v2|rope] [--model-size base] [--seq-len 512]
        [--micro-batch 32] [--ga 2] [--top 40] [--callers] [--gaps] [--no-dependent-launch]

Builds the RTD pretrainer from the config defaults on synthetic packed data, runs three warm-up windows, profiles the
fourth and prints, per kernel name, the launch count, total and mean device time and the share of the window. The
shares say where a step spends its time; absolute times under the profiler are not benchmark numbers. ``--callers``
also lists the ATen operators that launched kernels (fills, adds, copies: what is left outside the library's own
kernels) with the line of this package that called each of them; ``--gaps`` lists where the GPU sat idle inside the
window (time between the end of one kernel and the start of the next, grouped by the pair of kernels around it; the
profiler slows the host down, so these are upper bounds). The reference
has no counterpart (it ships no profiling hooks; its closest tool is ``tools/compile_drift_probe.py:363-366``, which
times whole steps).
"""

from __future__ import annotations

import argparse
import collections
import warnings

import torch

VOCAB = 128_100


def _config(a: argparse.Namespace):
    from deberta_b200.config import Config, DataConfig, ModelConfig, OptimConfig, TrainConfig, validate_config

    model = (ModelConfig(profile="deberta_v3_parity", backbone_type="hf_deberta_v2", hf={"model_size": a.model_size},
                         tokenizer={"name_or_path": f"synthetic:{VOCAB}"}) if a.backbone == "hf_deberta_v2"
             else ModelConfig(backbone_type="rope", tokenizer={"name_or_path": f"synthetic:{VOCAB}"}))
    cfg = Config(model=model, data=DataConfig(dataset_name="synthetic", max_seq_length=a.seq_len),
                 train=TrainConfig(per_device_train_batch_size=a.micro_batch, gradient_accumulation_steps=a.ga,
                                   mixed_precision="bf16", max_steps=10_000, dataloader_num_workers=0),
                 optim=OptimConfig(learning_rate=2e-4, warmup_steps=10_000))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        validate_config(cfg)
    return cfg


def _batches(a: argparse.Namespace, device: torch.device) -> list[dict[str, torch.Tensor]]:
    from deberta_b200.data import DebertaV3ElectraCollator, MLMConfig, PackedStreamingConfig, PackedStreamingDataset
    from deberta_b200.data.synthetic import SyntheticTextDataset, SyntheticTokenizer

    tok = SyntheticTokenizer(VOCAB)
    ds = iter(PackedStreamingDataset(hf_dataset=SyntheticTextDataset(vocab_size=VOCAB, mean_doc_len=60, seed=100), tokenizer=tok,
                                     cfg=PackedStreamingConfig(max_seq_length=a.seq_len, seed=100)))
    col = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(mask_token_prob=1.0, random_token_prob=0.0),
                                   packed_sequences=True, block_cross_document_attention=False)
    torch.manual_seed(100)
    return [dict(col([next(ds) for _ in range(a.micro_batch)])) for _ in range(a.ga)]  # host batches


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--backbone", choices=("hf_deberta_v2", "rope"), default="hf_deberta_v2")
    p.add_argument("--model-size", default="base")
    p.add_argument("--seq-len", type=int, default=512)
    p.add_argument("--micro-batch", type=int, default=32)
    p.add_argument("--ga", type=int, default=2)
    p.add_argument("--top", type=int, default=40)
    p.add_argument("--callers", action="store_true", help="attribute ATen kernels to the package line that launched them")
    p.add_argument("--gaps", action="store_true", help="list the idle intervals of the GPU inside the window")
    p.add_argument("--no-dependent-launch", action="store_true",
                   help="ordinary launches: with programmatic dependent launch a kernel's recorded duration includes its "
                        "wait for the predecessor, which inflates the per-kernel shares")
    a = p.parse_args(argv)
    if not torch.cuda.is_available():
        print("step_kernel_shares needs a CUDA device")
        return 2
    from torch.profiler import ProfilerActivity, profile

    from deberta_b200.parallel.dist import init_distributed
    from deberta_b200.training.runtime import build_engine, build_model, build_tokenizer
    from deberta_b200.training.trainer import Trainer

    ctx = init_distributed()
    if a.no_dependent_launch:
        from deberta_b200.ops import _lib

        _lib.set_dependent_launch(False)
    cfg = _config(a)
    torch.manual_seed(1234)
    tok = build_tokenizer(cfg.model)
    model, _, _ = build_model(model_cfg=cfg.model, tokenizer=tok, max_seq_length=a.seq_len)
    engine = build_engine(model=model, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim, parallelism="zero")
    trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim, pad_token_id=tok.pad_token_id)
    window = [trainer.stage_batch(b) for b in _batches(a, ctx.device)]
    for _ in range(3):
        trainer.train_window(window)
    torch.cuda.synchronize()
    extra = {}
    if a.callers:  # Python stacks are only recorded with the verbose collector
        extra = dict(with_stack=True, experimental_config=torch._C._profiler._ExperimentalConfig(verbose=True))
    # host-side events are only needed to name callers; without them the profiler barely slows the launching thread,
    # which is what the idle-gap report wants
    acts = [ProfilerActivity.CUDA] + ([ProfilerActivity.CPU] if a.callers else [])
    with profile(activities=acts, **extra) as prof:
        trainer.train_window(window)
        torch.cuda.synchronize()
    agg: dict[str, list[float]] = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            slot = agg[ev.name[:96]]
            slot[0] += 1
            slot[1] += ev.device_time
    total = sum(v[1] for v in agg.values())
    launches = int(sum(v[0] for v in agg.values()))
    print(f"window of {a.ga} micro-batches ({a.micro_batch} x {a.seq_len}): {total / 1e3:.1f} ms of device time over {launches} launches")
    for name, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[: a.top]:
        print(f"{t / total * 100:5.1f} %  {t / 1e3:8.2f} ms  n={int(n):5d}  mean {t / n:8.1f} us  {name}")
    if a.gaps:
        spans = sorted((ev.time_range.start, ev.time_range.end, ev.name) for ev in prof.events()
                       if ev.device_type == torch.autograd.DeviceType.CUDA)
        idle: dict[tuple[str, str], list[float]] = collections.defaultdict(lambda: [0, 0.0])
        busy_until, prev = spans[0][1], spans[0][2]
        for start, end, name in spans[1:]:
            if start > busy_until + 1.0:  # more than a microsecond with nothing running
                slot = idle[(prev[:60], name[:60])]
                slot[0] += 1
                slot[1] += start - busy_until
            if end > busy_until:
                busy_until, prev = end, name
        gap_total = sum(v[1] for v in idle.values())
        print(f"GPU idle inside the window: {gap_total / 1e3:.2f} ms in {int(sum(v[0] for v in idle.values()))} intervals "
              f"({gap_total / (spans[-1][1] - spans[0][0]) * 100:.1f} % of its span)")
        for (before, after), (n, t) in sorted(idle.items(), key=lambda kv: -kv[1][1])[: a.top]:
            print(f"{t / 1e3:8.2f} ms  n={int(n):4d}  after {before}  before {after}")
    if a.callers:
        rows: dict[tuple[str, str], list[float]] = collections.defaultdict(lambda: [0, 0.0])
        for ev in prof.key_averages(group_by_stack_n=24):
            if not ev.key.startswith("aten::") or ev.self_device_time_total <= 0:
                continue
            site = next((f.strip() for f in ev.stack if "deberta_b200" in f and "step_kernel_shares" not in f),
                        "(autograd engine or outside the package)")
            slot = rows[(ev.key, site[-110:])]
            slot[0] += ev.count
            slot[1] += ev.self_device_time_total
        print("ATen operators that launched kernels, by calling line:")
        for (op, site), (n, t) in sorted(rows.items(), key=lambda kv: -kv[1][1])[: a.top]:
            print(f"{t / 1e3:8.2f} ms  n={int(n):5d}  {op:28s} {site}")
    ctx.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
