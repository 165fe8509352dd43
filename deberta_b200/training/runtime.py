"""Builders for the pieces a training run needs (``training/runtime.py`` of the reference):
tokenizer, dataset + collator, the endless batch iterator, and the model/engine pair."""

from __future__ import annotations

import logging
from collections.abc import Iterator
from typing import Any

import torch

from deberta_b200.config import DataConfig, ModelConfig, OptimConfig, TrainConfig
from deberta_b200.data import (DebertaV3ElectraCollator, MLMConfig, PackedStreamingConfig, PackedStreamingDataset,
                               SequentialStreamingDataset, load_hf_dataset)
from deberta_b200.data.synthetic import load_tokenizer
from deberta_b200.models import DebertaV3RTDPretrainer, build_backbone_configs, build_backbones
from deberta_b200.parallel.dist import DistContext
from deberta_b200.parallel.engine import TrainEngine

logger = logging.getLogger(__name__)


def build_tokenizer(model_cfg: ModelConfig) -> Any:
    tok = load_tokenizer(model_cfg.tokenizer.name_or_path)
    if getattr(tok, "pad_token_id", None) is None:
        raise ValueError("Tokenizer must define a pad token for pretraining.")
    return tok


def build_training_dataset_and_collator(*, data_cfg: DataConfig, train_cfg: TrainConfig, tokenizer: Any,
                                        process_index: int, num_processes: int, hf_dataset: Any = None):
    """(iterable dataset of token blocks, masking collator) for this rank."""
    ds = hf_dataset if hf_dataset is not None else load_hf_dataset(cfg=data_cfg)
    pcfg = PackedStreamingConfig(text_column_name=data_cfg.source.text_column_name,
                                 max_seq_length=int(data_cfg.packing.max_seq_length), seed=int(train_cfg.seed),
                                 shuffle_buffer_size=int(data_cfg.source.shuffle_buffer_size))
    cls = PackedStreamingDataset if data_cfg.packing.enabled else SequentialStreamingDataset
    dataset = cls(hf_dataset=ds, tokenizer=tokenizer, cfg=pcfg, process_index=process_index, num_processes=num_processes)
    o = train_cfg.objective
    collator = DebertaV3ElectraCollator(
        tokenizer=tokenizer,
        cfg=MLMConfig(mlm_probability=float(o.mlm_probability), mask_token_prob=float(o.mask_token_prob),
                      random_token_prob=float(o.random_token_prob), max_ngram=int(o.mlm_max_ngram)),
        packed_sequences=bool(data_cfg.packing.enabled),
        block_cross_document_attention=bool(data_cfg.packing.block_cross_document_attention),
    )
    return dataset, collator


def build_dataloader(*, dataset: Any, collator: Any, train_cfg: TrainConfig) -> torch.utils.data.DataLoader:
    workers = int(train_cfg.dataloader.num_workers)
    return torch.utils.data.DataLoader(
        dataset, batch_size=int(train_cfg.per_device_train_batch_size), collate_fn=collator, num_workers=workers,
        pin_memory=bool(train_cfg.dataloader.pin_memory) and torch.cuda.is_available(), drop_last=True,
        persistent_workers=workers > 0,
    )


def cycle_dataloader(loader: Any, *, start_epoch: int = 0) -> Iterator[dict[str, torch.Tensor]]:
    """Endless batches; every pass over the data is a new epoch with its own shuffle seed."""
    epoch = int(start_epoch)
    while True:
        ds = getattr(loader, "dataset", None)
        if hasattr(ds, "set_epoch"):
            ds.set_epoch(epoch)
        seen = False
        for batch in loader:
            seen = True
            yield batch
        if not seen:
            raise RuntimeError("The training dataloader produced no batches (dataset too small for one batch?).")
        epoch += 1


def build_model(*, model_cfg: ModelConfig, tokenizer: Any, max_seq_length: int, load_pretrained_weights: bool = True):
    """RTD pretrainer with both backbones built from the config (scratch or pretrained)."""
    disc_cfg, gen_cfg = build_backbone_configs(model_cfg=model_cfg, tokenizer=tokenizer,
                                               max_position_embeddings=int(max_seq_length))
    disc, gen = build_backbones(model_cfg=model_cfg, disc_config=disc_cfg, gen_config=gen_cfg,
                                load_pretrained_weights=load_pretrained_weights)
    if model_cfg.gradient_checkpointing:
        for m in (disc, gen):
            m.gradient_checkpointing_enable()
    model = DebertaV3RTDPretrainer(
        discriminator_backbone=disc, generator_backbone=gen, disc_config=disc_cfg, gen_config=gen_cfg,
        embedding_sharing=model_cfg.embedding_sharing, tie_generator_word_embeddings=True,
        additional_forbidden_token_ids=getattr(tokenizer, "all_special_ids", None),
    )
    return model, disc_cfg, gen_cfg


def resolve_learning_rates(optim_cfg: OptimConfig) -> tuple[float, float]:
    base = float(optim_cfg.lr.base)
    g, d = float(optim_cfg.lr.generator), float(optim_cfg.lr.discriminator)
    return (g if g > 0 else base), (d if d > 0 else base)


def build_engine(*, model: torch.nn.Module, ctx: DistContext, train_cfg: TrainConfig, optim_cfg: OptimConfig,
                 parallelism: str | None = None) -> TrainEngine:
    """Engine with the optimizer layout of the run: two optimizers when decoupled, one otherwise.

    ``train.distributed`` chooses the parallelism and the collective path (``parallelism`` overrides the former).
    """
    di = train_cfg.distributed
    parallelism = str(di.parallelism) if parallelism is None else parallelism
    bf16 = str(train_cfg.mixed_precision) == "bf16" and ctx.device.type == "cuda"
    if str(train_cfg.mixed_precision) == "bf16" and not bf16:
        logger.warning("train.mixed_precision=bf16 needs a CUDA device; running this process in fp32.")
    eps = float(optim_cfg.adam.epsilon)
    if bf16:
        eps = max(eps, 1e-6)  # moments of bf16-rounded gradients make smaller eps unstable
    lr_g, lr_d = resolve_learning_rates(optim_cfg)
    return TrainEngine(model, ctx, compute_dtype=torch.bfloat16 if bf16 else torch.float32, parallelism=parallelism,
                       decoupled=bool(train_cfg.decoupled_training), lr_generator=lr_g, lr_discriminator=lr_d,
                       weight_decay=float(optim_cfg.weight_decay),
                       betas=(float(optim_cfg.adam.beta1), float(optim_cfg.adam.beta2)), eps=eps,
                       fused_collectives=bool(di.fused_collectives), multicast=str(di.nvls),
                       comm_timeout_s=float(di.comm_timeout_s))
