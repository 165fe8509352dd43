"""Configuration schema: ``model / data / train / optim / logging`` (schema version 4).

The schema, defaults, aliases and validation rules are those of ``src/deberta/config.py``
of the reference, so its YAML/JSON files load unchanged. The implementation is generic:
every section is a frozen dataclass derived from ``Section``, whose constructor accepts
nested mappings, dotted keys and the legacy flat names (``ModelConfig(hidden_size=64)``),
and whose attribute lookup resolves the same legacy names for reading.
"""

from __future__ import annotations

import dataclasses
import re
import warnings
from collections.abc import Callable
from dataclasses import asdict, dataclass, field, fields, replace
from pathlib import Path
from typing import Any, ClassVar, get_type_hints

from deberta_b200.utils.io import load_json_mapping
from deberta_b200.utils.mapping import flatten_mapping, leaf_paths
from deberta_b200.utils.serialize import asdict_without_private
from deberta_b200.utils.types import coerce_scalar, unwrap_optional_type

RUN_CONFIG_SCHEMA_VERSION = 4
_DENSE_DOC_BLOCK_WARN_SEQ_LEN = 2048

# ---------------------------------------------------------------------------------------------
# choices and aliases
# ---------------------------------------------------------------------------------------------
_CHOICES: dict[str, set[str]] = {
    "model.backbone_type": {"rope", "hf_deberta_v2"},
    "model.profile": {"modern", "deberta_v3_parity"},
    "model.embedding_sharing": {"none", "es", "gdes"},
    "model.hf.model_size": {"xsmall", "small", "base", "large"},
    "model.hf.attention_kernel": {"dynamic", "cached_bmm", "stable"},
    "model.rope.norm_arch": {"post", "keel"},
    "model.rope.attention_implementation": {"sdpa", "eager"},
    "model.rope.ffn_type": {"swiglu", "mlp"},
    "train.mixed_precision": {"bf16", "no"},
    "train.sdpa_kernel": {"auto", "flash", "mem_efficient", "math"},
    "train.compile.mode": {"default", "reduce-overhead", "max-autotune", "max-autotune-no-cudagraphs"},
    "train.compile.scope": {"auto", "backbones", "encoder", "gen_encoder", "disc_encoder", "ffn", "gen_ffn", "disc_ffn"},
    "train.compile.backend": {"inductor", "aot_eager"},
    "train.checkpoint.resume_data_strategy": {"auto", "replay", "restart_epoch"},
    "train.distributed.parallelism": {"ddp", "zero", "fsdp"},
    "train.distributed.nvls": {"auto", "on", "off"},
    "optim.scheduler.type": {"linear", "cosine", "cosine_with_restarts", "polynomial", "constant", "constant_with_warmup"},
    "logging.backend": {"none", "tensorboard"},
    "logging.wandb.watch": {"none", "gradients", "parameters", "all"},
}
_ALIASES: dict[str, dict[str, str]] = {
    "model.hf.attention_kernel": {"default": "dynamic", "cache": "cached_bmm", "cached": "cached_bmm",
                                  "safe": "stable", "compile_safe": "stable"},
    "train.sdpa_kernel": {"mem": "mem_efficient", "mem-efficient": "mem_efficient", "efficient": "mem_efficient",
                          "flashattention": "flash", "flash_attention": "flash"},
    "train.compile.mode": {"reduce_overhead": "reduce-overhead", "max_autotune": "max-autotune",
                           "max_autotune_no_cudagraphs": "max-autotune-no-cudagraphs"},
    "train.compile.scope": {"both": "backbones", "backbone": "backbones", "full": "backbones", "encoders": "encoder",
                            "generator_encoder": "gen_encoder", "discriminator_encoder": "disc_encoder",
                            "ffns": "ffn", "generator_ffn": "gen_ffn", "discriminator_ffn": "disc_ffn"},
    "train.compile.backend": {"aot-eager": "aot_eager"},
    "train.distributed.parallelism": {"replicated": "ddp", "zero1": "zero", "sharded_optimizer": "zero",
                                      "full_shard": "fsdp", "fsdp2": "fsdp", "zero3": "fsdp"},
    "train.distributed.nvls": {"true": "on", "1": "on", "yes": "on", "false": "off", "0": "off", "no": "off"},
    "logging.wandb.watch": {"off": "none", "disabled": "none", "false": "none", "0": "none", "grad": "gradients",
                            "gradient": "gradients", "weights": "parameters", "params": "parameters",
                            "param": "parameters"},
    "train.mixed_precision": {"bfloat16": "bf16", "true": "bf16", "1": "bf16", "yes": "bf16", "y": "bf16",
                              "on": "bf16", "none": "no", "false": "no", "0": "no", "off": "no", "n": "no"},
}
_HYPHEN_TO_UNDERSCORE = {"train.compile.scope", "train.compile.backend", "logging.wandb.watch",
                         "model.hf.attention_kernel"}
_HF_DEBERTA_PRETRAINED_PREFIXES = ("microsoft/deberta-v2", "microsoft/deberta-v3", "microsoft/mdeberta-v3")


def choices_for(path: str, *, with_aliases: bool = False) -> list[str] | None:
    """Allowed values of a constrained string field (used for CLI ``choices``)."""
    if path not in _CHOICES:
        return None
    out = set(_CHOICES[path])
    if with_aliases:
        out |= set(_ALIASES.get(path, {}))
    return sorted(out)


def normalize_choice(path: str, value: Any) -> str:
    """Lower-case, alias-resolve and validate a constrained string option."""
    v = str(value).strip().lower()
    if path in _HYPHEN_TO_UNDERSCORE:
        v = v.replace("-", "_")
    v = _ALIASES.get(path, {}).get(v, v)
    if v not in _CHOICES[path]:
        raise ValueError(f"{path} must be one of: {'|'.join(sorted(_CHOICES[path]))}. Got: {value}")
    return v


def normalize_mixed_precision(value: object) -> str:
    """``bf16|no`` plus boolean-ish aliases (``true/false/yes/no/on/off/1/0``)."""
    if isinstance(value, bool):
        return "bf16" if value else "no"
    v = str(value).strip().lower()
    v = _ALIASES["train.mixed_precision"].get(v, v)
    if v not in _CHOICES["train.mixed_precision"]:
        raise ValueError("train.mixed_precision must be one of: bf16|no (or aliases true|false|yes|no|on|off|1|0).")
    return v


def resolve_effective_mixed_precision(value: object, *, bf16_sanity_check: Callable[[], bool] | None = None) -> str:
    """Normalise mixed precision and fail loudly when bf16 was asked for but cannot run."""
    mp = normalize_mixed_precision(value)
    if mp == "bf16" and bf16_sanity_check is not None and not bf16_sanity_check():
        raise RuntimeError(
            "train.mixed_precision=bf16 requested but bf16 preflight failed. "
            "Set train.mixed_precision=no explicitly if you want to continue in full precision."
        )
    return mp


_normalize_hf_attention_kernel = lambda v: normalize_choice("model.hf.attention_kernel", v)  # noqa: E731
_normalize_sdpa_kernel = lambda v: normalize_choice("train.sdpa_kernel", v)  # noqa: E731
_normalize_torch_compile_mode = lambda v: normalize_choice("train.compile.mode", v)  # noqa: E731
_normalize_torch_compile_scope = lambda v: normalize_choice("train.compile.scope", v)  # noqa: E731
_normalize_torch_compile_backend = lambda v: normalize_choice("train.compile.backend", v)  # noqa: E731
_normalize_wandb_watch = lambda v: normalize_choice("logging.wandb.watch", v)  # noqa: E731


# ---------------------------------------------------------------------------------------------
# generic section machinery
# ---------------------------------------------------------------------------------------------
def _set(obj: Any, name: str, value: Any) -> None:
    object.__setattr__(obj, name, value)


def _nested_get(obj: Any, path: str) -> Any:
    for part in path.split("."):
        obj = getattr(obj, part)
    return obj


def _replace_path(obj: Any, parts: list[str], value: Any) -> Any:
    key = parts[0]
    if not dataclasses.is_dataclass(obj) or key not in {f.name for f in fields(obj)}:
        raise TypeError(f"Unknown field {key!r} for {type(obj).__name__}.")
    if len(parts) == 1:
        return replace(obj, **{key: value})
    return replace(obj, **{key: _replace_path(getattr(obj, key), parts[1:], value)})


def _apply_dotted(obj: Any, updates: dict[str, Any]) -> Any:
    for path, value in updates.items():
        parts = [p.strip() for p in str(path).split(".") if p.strip()]
        if parts:
            obj = _replace_path(obj, parts, value)
    return obj


class Section:
    """Base of all config dataclasses: mapping/legacy-aware constructor and legacy reads."""

    _LEGACY: ClassVar[dict[str, str]] = {}
    _DYNAMIC_DEFAULTS: ClassVar[dict[str, Any]] = {}

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        flds = fields(self)  # type: ignore[arg-type]
        names = [f.name for f in flds]
        if len(args) > len(names):
            raise TypeError(f"{type(self).__name__}.__init__ takes at most {len(names)} positional arguments")
        for name, val in zip(names, args):
            if name in kwargs:
                raise TypeError(f"{type(self).__name__}.__init__ got multiple values for {name!r}")
            kwargs[name] = val
        hints = get_type_hints(type(self))
        values: dict[str, Any] = {}
        for f in flds:
            target, _ = unwrap_optional_type(hints[f.name])
            is_sub = isinstance(target, type) and issubclass(target, Section)
            if f.name in kwargs:
                v = kwargs.pop(f.name)
                if is_sub:
                    if v is None:
                        v = target()
                    elif isinstance(v, dict):
                        v = _apply_dotted(target(), flatten_mapping(v))
                    elif not isinstance(v, target):
                        raise TypeError(f"{f.name} must be a {target.__name__} or mapping, got {type(v).__name__}.")
                elif v is not None and target in (int, float, str, bool) and not isinstance(v, target):
                    v = target(v)
            elif f.default is not dataclasses.MISSING:
                v = f.default
            else:
                v = f.default_factory()  # type: ignore[misc]
            values[f.name] = v
        kwargs = self._translate_legacy_kwargs(kwargs, values)
        dotted: dict[str, Any] = {}
        unknown: list[str] = []
        for key, v in kwargs.items():
            path = self._LEGACY.get(key, key if "." in key else None)
            if path is None or path.split(".")[0] not in values:
                unknown.append(key)
            elif "." in path:
                dotted[path] = v
            else:
                values[path] = v
        if unknown:
            raise TypeError(
                f"{type(self).__name__}.__init__ got unexpected keyword argument(s): {', '.join(sorted(unknown))}"
            )
        for name, v in values.items():
            _set(self, name, v)
        for path, v in dotted.items():
            root, rest = path.split(".", 1)
            _set(self, root, _apply_dotted(getattr(self, root), {rest: v}))

    def _translate_legacy_kwargs(self, kwargs: dict[str, Any], values: dict[str, Any]) -> dict[str, Any]:
        return kwargs

    def __getattr__(self, name: str) -> Any:
        # only reached when normal lookup failed: legacy flat names
        cls = type(self)
        path = cls._LEGACY.get(name)
        if path is not None:
            return _nested_get(self, path)
        if name in cls._DYNAMIC_DEFAULTS:
            return cls._DYNAMIC_DEFAULTS[name]
        raise AttributeError(name)


def _cfg(cls):
    """``@dataclass(frozen=True)`` that keeps ``Section.__init__``."""
    return dataclass(frozen=True, init=False)(cls)


# ---------------------------------------------------------------------------------------------
# model
# ---------------------------------------------------------------------------------------------
@_cfg
class ModelTokenizerConfig(Section):
    name_or_path: str = "microsoft/deberta-v3-base"
    allow_vocab_resize: bool = False
    vocab_target: int | None = None
    vocab_multiple: int = 1


@_cfg
class ModelHFScratchConfig(Section):
    """Shape overrides for a from-scratch ``hf_deberta_v2`` discriminator (all optional). The reference's schema only
    offers the size presets, and builds its tiny test models in code (``tests/test_smoke.py:1773-1851``); these leaves
    make such a model expressible in a config file (``configs/tiny_cpu_smoke_hf_deberta_v2.yaml``)."""

    hidden_size: int | None = None
    num_hidden_layers: int | None = None
    num_attention_heads: int | None = None
    intermediate_size: int | None = None
    position_buckets: int | None = None


@_cfg
class ModelHFConfig(Section):
    model_size: str = "base"
    attention_kernel: str = "dynamic"
    max_position_embeddings: int | None = None
    scratch: ModelHFScratchConfig = field(default_factory=ModelHFScratchConfig)


@_cfg
class ModelPretrainedConfig(Section):
    discriminator_path: str = ""
    generator_path: str | None = None


@_cfg
class ModelGeneratorConfig(Section):
    num_hidden_layers: int | None = None
    hidden_size: int | None = None
    intermediate_size: int | None = None
    num_attention_heads: int | None = None


@_cfg
class ModelRopePretrainedConfig(Section):
    max_position_embeddings: int | None = None
    rope_theta: float | None = None
    rotary_pct: float | None = None
    use_absolute_position_embeddings: bool | None = None
    type_vocab_size: int | None = None
    norm_arch: str | None = None
    norm_eps: float | None = None
    keel_alpha_init: float | None = None
    keel_alpha_learnable: bool | None = None
    ffn_type: str | None = None
    use_bias: bool | None = None
    initializer_range: float | None = None


@_cfg
class ModelRopeConfig(Section):
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    hidden_act: str = "gelu"
    rope_theta: float = 10000.0
    rotary_pct: float = 1.0
    use_absolute_position_embeddings: bool = False
    max_position_embeddings: int | None = None
    type_vocab_size: int = 2
    norm_arch: str = "post"
    norm_eps: float = 1e-6
    keel_alpha_init: float | None = None
    keel_alpha_learnable: bool = False
    attention_implementation: str = "sdpa"
    ffn_type: str = "mlp"
    use_bias: bool = False
    swiglu_adjust_intermediate: bool = True
    initializer_range: float = 0.02
    pretrained: ModelRopePretrainedConfig = field(default_factory=ModelRopePretrainedConfig)


@_cfg
class ModelDropoutConfig(Section):
    hidden_prob: float | None = 0.0
    attention_probs_prob: float | None = 0.0


_ROPE_FLAT = ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "hidden_act",
              "rope_theta", "rotary_pct", "use_absolute_position_embeddings", "max_position_embeddings",
              "type_vocab_size", "norm_arch", "norm_eps", "keel_alpha_init", "keel_alpha_learnable",
              "attention_implementation", "ffn_type", "use_bias", "swiglu_adjust_intermediate", "initializer_range")


@_cfg
class ModelConfig(Section):
    profile: str = "modern"
    backbone_type: str = "hf_deberta_v2"
    from_scratch: bool = True
    embedding_sharing: str = "gdes"
    gradient_checkpointing: bool = False
    tokenizer: ModelTokenizerConfig = field(default_factory=ModelTokenizerConfig)
    hf: ModelHFConfig = field(default_factory=ModelHFConfig)
    pretrained: ModelPretrainedConfig = field(default_factory=ModelPretrainedConfig)
    generator: ModelGeneratorConfig = field(default_factory=ModelGeneratorConfig)
    rope: ModelRopeConfig = field(default_factory=ModelRopeConfig)
    dropout: ModelDropoutConfig = field(default_factory=ModelDropoutConfig)

    _LEGACY: ClassVar[dict[str, str]] = {
        **{f"tokenizer_{k}": f"tokenizer.{k}" for k in ("name_or_path", "allow_vocab_resize", "vocab_target", "vocab_multiple")},
        **{f"hf_{k}": f"hf.{k}" for k in ("attention_kernel", "model_size", "max_position_embeddings")},
        "pretrained_discriminator_path": "pretrained.discriminator_path",
        "pretrained_generator_path": "pretrained.generator_path",
        **{f"generator_{k}": f"generator.{k}" for k in ("num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads")},
        **{k: f"rope.{k}" for k in _ROPE_FLAT},
        **{f"pretrained_{f.name}": f"rope.pretrained.{f.name}" for f in fields(ModelRopePretrainedConfig)},
        "hidden_dropout_prob": "dropout.hidden_prob",
        "attention_probs_dropout_prob": "dropout.attention_probs_prob",
    }


# ---------------------------------------------------------------------------------------------
# data
# ---------------------------------------------------------------------------------------------
@_cfg
class DataSourceConfig(Section):
    dataset_name: str | None = None
    dataset_config_name: str | None = None
    data_files: str | None = None
    load_from_disk: str | None = None
    train_split: str = "train"
    text_column_name: str = "text"
    streaming: bool = True
    shuffle_buffer_size: int = 10_000


@_cfg
class DataPackingConfig(Section):
    enabled: bool = True
    max_seq_length: int = 512
    block_cross_document_attention: bool = False


@_cfg
class DataConfig(Section):
    source: DataSourceConfig = field(default_factory=DataSourceConfig)
    packing: DataPackingConfig = field(default_factory=DataPackingConfig)

    _LEGACY: ClassVar[dict[str, str]] = {
        **{f.name: f"source.{f.name}" for f in fields(DataSourceConfig)},
        "pack_sequences": "packing.enabled",
        "max_seq_length": "packing.max_seq_length",
        "block_cross_document_attention": "packing.block_cross_document_attention",
    }


# ---------------------------------------------------------------------------------------------
# train
# ---------------------------------------------------------------------------------------------
@_cfg
class TrainDataloaderConfig(Section):
    num_workers: int = 2
    pin_memory: bool = True


@_cfg
class TrainCompileConfig(Section):
    enabled: bool = False
    mode: str = "default"
    scope: str = "auto"
    backend: str = "inductor"


@_cfg
class TrainObjectiveConfig(Section):
    mlm_probability: float = 0.15
    mask_token_prob: float = 0.8
    random_token_prob: float = 0.1
    mlm_max_ngram: int = 1
    sampling_temperature: float = 1.0
    gen_loss_weight: float = 1.0
    disc_loss_weight: float = 50.0


@_cfg
class TrainCheckpointConfig(Section):
    output_dir: str | None = None
    overwrite_output_dir: bool = False
    save_steps: int = 1_000
    save_total_limit: int = 3
    resume_from_checkpoint: str | None = None
    resume_data_strategy: str = "auto"
    resume_replay_max_micro_batches: int = 10_000
    export_hf_final: bool = True


@_cfg
class TrainDistributedConfig(Section):
    """How the ranks of one node share the work (this package's engine; the reference delegates this to its
    Accelerate launch files ``configs/accelerate/fsdp2_*.yaml``)."""

    parallelism: str = "zero"       # ddp: replicated optimizer | zero: sharded optimizer state | fsdp: parameters sharded too
    fused_collectives: bool = True  # peer-memory kernels instead of NCCL for gradients / parameters (one node, 2..8 GPUs)
    nvls: str = "auto"              # in-switch reduction (multimem) path of those kernels: auto = from 4 ranks on
    overlap_backward: bool = True   # reduce gradient buckets on a side stream while backward still runs
    comm_timeout_s: float = 20.0    # longest device-side wait for a peer before the step fails
    step_deadline_s: float = 0.0    # host watchdog: report when no optimizer step completes in this time (0 = off)
    heartbeat_s: float = 0.0        # rank heartbeats through the process-group store (0 = off)


@_cfg
class TrainConfig(Section):
    seed: int = 42
    max_steps: int = 10_000
    per_device_train_batch_size: int = 4
    gradient_accumulation_steps: int = 1
    token_weighted_gradient_accumulation: bool = True
    mixed_precision: str = "bf16"
    tf32: bool = True
    sdpa_kernel: str = "auto"
    decoupled_training: bool = True
    dataloader: TrainDataloaderConfig = field(default_factory=TrainDataloaderConfig)
    compile: TrainCompileConfig = field(default_factory=TrainCompileConfig)
    objective: TrainObjectiveConfig = field(default_factory=TrainObjectiveConfig)
    checkpoint: TrainCheckpointConfig = field(default_factory=TrainCheckpointConfig)
    distributed: TrainDistributedConfig = field(default_factory=TrainDistributedConfig)

    _LEGACY: ClassVar[dict[str, str]] = {
        "dataloader_num_workers": "dataloader.num_workers",
        "dataloader_pin_memory": "dataloader.pin_memory",
        "torch_compile": "compile.enabled",
        "torch_compile_mode": "compile.mode",
        "torch_compile_scope": "compile.scope",
        "torch_compile_backend": "compile.backend",
        **{f.name: f"objective.{f.name}" for f in fields(TrainObjectiveConfig)},
        **{f.name: f"checkpoint.{f.name}" for f in fields(TrainCheckpointConfig)},
    }
    # optimiser / logging values mirrored onto TrainConfig by ``_sync_legacy_train_aliases``;
    # these are the values seen before any mirroring happened.
    _DYNAMIC_DEFAULTS: ClassVar[dict[str, Any]] = {
        "learning_rate": 5e-4, "generator_learning_rate": -1.0, "discriminator_learning_rate": -1.0,
        "weight_decay": 0.01, "adam_beta1": 0.9, "adam_beta2": 0.999, "adam_epsilon": 1e-8, "warmup_steps": 1_000,
        "lr_scheduler_type": "linear", "max_grad_norm": 1.0, "project_name": "deberta-train", "run_name": None,
        "logging_steps": 50, "report_to": "none", "wandb_watch": "gradients", "wandb_watch_log_freq": 100,
        "debug_metrics": False, "logging_output_dir": None,
    }

    def _translate_legacy_kwargs(self, kwargs, values):
        # mixed_precision accepts real booleans in constructors
        if isinstance(values.get("mixed_precision"), bool):
            values["mixed_precision"] = "bf16" if values["mixed_precision"] else "no"
        return kwargs


# ---------------------------------------------------------------------------------------------
# optim / logging
# ---------------------------------------------------------------------------------------------
@_cfg
class OptimLRConfig(Section):
    base: float = 5e-4
    generator: float = -1.0
    discriminator: float = -1.0


@_cfg
class OptimAdamConfig(Section):
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8


@_cfg
class OptimSchedulerConfig(Section):
    type: str = "linear"
    warmup_steps: int = 1_000


@_cfg
class OptimConfig(Section):
    lr: OptimLRConfig = field(default_factory=OptimLRConfig)
    adam: OptimAdamConfig = field(default_factory=OptimAdamConfig)
    scheduler: OptimSchedulerConfig = field(default_factory=OptimSchedulerConfig)
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0

    _LEGACY: ClassVar[dict[str, str]] = {
        "learning_rate": "lr.base", "generator_learning_rate": "lr.generator",
        "discriminator_learning_rate": "lr.discriminator", "adam_beta1": "adam.beta1", "adam_beta2": "adam.beta2",
        "adam_epsilon": "adam.epsilon", "lr_scheduler_type": "scheduler.type", "warmup_steps": "scheduler.warmup_steps",
    }


@_cfg
class LoggingWandbConfig(Section):
    enabled: bool = False
    watch: str = "gradients"
    watch_log_freq: int = 100


@_cfg
class LoggingDebugConfig(Section):
    metrics: bool = False
    nvtx: bool = False  # NVTX ranges around the phases of a step


@_cfg
class LoggingConfig(Section):
    project_name: str = "deberta-train"
    run_name: str | None = None
    output_dir: str | None = None
    logging_steps: int = 50
    backend: str = "none"
    wandb: LoggingWandbConfig = field(default_factory=LoggingWandbConfig)
    debug: LoggingDebugConfig = field(default_factory=LoggingDebugConfig)

    _LEGACY: ClassVar[dict[str, str]] = {
        "wandb_watch": "wandb.watch", "wandb_watch_log_freq": "wandb.watch_log_freq", "debug_metrics": "debug.metrics",
    }

    def _translate_legacy_kwargs(self, kwargs, values):
        # ``report_to=wandb`` switches W&B on; any other value names the plain backend
        if "report_to" in kwargs:
            kwargs = dict(kwargs)
            target = str(kwargs.pop("report_to")).strip().lower()
            kwargs["wandb.enabled"] = target == "wandb"
            if target != "wandb":
                values["backend"] = target
        return kwargs


@dataclass(frozen=True)
class Config:
    """Top-level bundle of the five sections."""

    model: ModelConfig = field(default_factory=ModelConfig)
    data: DataConfig = field(default_factory=DataConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    logging: LoggingConfig = field(default_factory=LoggingConfig)


def _sync_legacy_train_aliases(*, train_cfg: TrainConfig, optim_cfg: OptimConfig, logging_cfg: LoggingConfig) -> None:
    """Mirror optimiser/logging values onto ``TrainConfig`` under their flat historical names."""
    mirror = {
        "learning_rate": float(optim_cfg.lr.base), "generator_learning_rate": float(optim_cfg.lr.generator),
        "discriminator_learning_rate": float(optim_cfg.lr.discriminator), "weight_decay": float(optim_cfg.weight_decay),
        "adam_beta1": float(optim_cfg.adam.beta1), "adam_beta2": float(optim_cfg.adam.beta2),
        "adam_epsilon": float(optim_cfg.adam.epsilon), "warmup_steps": int(optim_cfg.scheduler.warmup_steps),
        "lr_scheduler_type": str(optim_cfg.scheduler.type), "max_grad_norm": float(optim_cfg.max_grad_norm),
        "project_name": str(logging_cfg.project_name), "run_name": logging_cfg.run_name,
        "logging_output_dir": logging_cfg.output_dir, "logging_steps": int(logging_cfg.logging_steps),
        "report_to": "wandb" if logging_cfg.wandb.enabled else str(logging_cfg.backend).strip().lower(),
        "wandb_watch": str(logging_cfg.wandb.watch), "wandb_watch_log_freq": int(logging_cfg.wandb.watch_log_freq),
        "debug_metrics": bool(logging_cfg.debug.metrics),
    }
    for k, v in mirror.items():
        _set(train_cfg, k, v)


def _explicit_fields(cfg_obj: Any) -> set[str]:
    raw = getattr(cfg_obj, "_explicit_fields", None) if cfg_obj is not None else None
    return {str(x) for x in raw} if isinstance(raw, (set, frozenset, list, tuple)) else set()


def _mark_explicit_fields(cfg_obj: Any, explicit: set[str]) -> None:
    _set(cfg_obj, "_explicit_fields", {str(x) for x in explicit})


# ---------------------------------------------------------------------------------------------
# validation
# ---------------------------------------------------------------------------------------------
def _looks_like_hf_deberta_checkpoint(value: str) -> bool:
    """Hub ids / URLs / cache paths of Microsoft DeBERTa v2/v3 checkpoints."""
    v = str(value).strip().lower().replace("\\", "/")
    if not v:
        return False
    if v.startswith("hf://"):
        v = v[5:]
    if "huggingface.co/" in v and v.startswith(("https://", "http://")):
        v = v.split("huggingface.co/", 1)[1]
    v = v.lstrip("/")
    if any(v == p or v.startswith(f"{p}-") or v.startswith(f"{p}/") for p in _HF_DEBERTA_PRETRAINED_PREFIXES):
        return True
    return any(f"/models--microsoft--{m}" in f"/{v}/" for m in ("deberta-v2", "deberta-v3", "mdeberta-v3"))


def _warn(msg: str) -> None:
    warnings.warn(msg, UserWarning, stacklevel=3)


def validate_model_config(cfg: ModelConfig) -> None:
    """Normalise constrained values in place and reject inconsistent model options."""
    for name in ("backbone_type", "profile", "embedding_sharing"):
        _set(cfg, name, normalize_choice(f"model.{name}", getattr(cfg, name)))
    _set(cfg.hf, "attention_kernel", normalize_choice("model.hf.attention_kernel", cfg.hf.attention_kernel))
    _set(cfg.hf, "model_size", normalize_choice("model.hf.model_size", cfg.hf.model_size))
    for name in ("norm_arch", "attention_implementation", "ffn_type"):
        _set(cfg.rope, name, normalize_choice(f"model.rope.{name}", getattr(cfg.rope, name)))
    _set(cfg.tokenizer, "name_or_path", str(cfg.tokenizer.name_or_path).strip())
    _set(cfg.pretrained, "discriminator_path", str(cfg.pretrained.discriminator_path or "").strip())
    if cfg.pretrained.generator_path is not None:
        _set(cfg.pretrained, "generator_path", str(cfg.pretrained.generator_path).strip() or None)
    if not cfg.tokenizer.name_or_path:
        raise ValueError("model.tokenizer.name_or_path must be a non-empty tokenizer source.")
    if not cfg.from_scratch and not cfg.pretrained.discriminator_path:
        raise ValueError(
            "model.pretrained.discriminator_path must be set when model.from_scratch=false "
            "(weights are loaded from this source)."
        )
    if cfg.rope.max_position_embeddings is not None and int(cfg.rope.max_position_embeddings) <= 0:
        raise ValueError("model.rope.max_position_embeddings must be > 0 when provided.")
    if not 0.0 < float(cfg.rope.rotary_pct) <= 1.0:
        raise ValueError("model.rope.rotary_pct must be in (0, 1].")
    if int(cfg.tokenizer.vocab_multiple) <= 0:
        raise ValueError("model.tokenizer.vocab_multiple must be >= 1.")
    if cfg.tokenizer.vocab_target is not None and int(cfg.tokenizer.vocab_target) <= 0:
        raise ValueError("model.tokenizer.vocab_target must be > 0 when provided.")
    d = ModelConfig()
    if cfg.backbone_type == "hf_deberta_v2":
        mpe = cfg.hf.max_position_embeddings
        if mpe is not None and int(mpe) <= 0:
            raise ValueError("model.hf.max_position_embeddings must be > 0 when provided.")
        if mpe is not None and not cfg.from_scratch:
            raise ValueError(
                "model.hf.max_position_embeddings is only supported when model.from_scratch=true for hf_deberta_v2 runs."
            )
        sc = cfg.hf.scratch
        given = {k: v for k, v in asdict(sc).items() if v is not None}
        if given and not cfg.from_scratch:
            raise ValueError("model.hf.scratch.* is only supported when model.from_scratch=true.")
        for k, v in given.items():
            if int(v) <= 0:
                raise ValueError(f"model.hf.scratch.{k} must be > 0 when provided.")
        if sc.hidden_size is not None and sc.num_attention_heads is not None and int(sc.hidden_size) % int(sc.num_attention_heads):
            raise ValueError("model.hf.scratch.hidden_size must be divisible by model.hf.scratch.num_attention_heads.")
        if asdict(cfg.rope) != asdict(d.rope):
            raise ValueError("These options are only valid when model.backbone_type='rope': model.rope.*")
    else:
        for name in ("attention_kernel", "max_position_embeddings", "model_size"):
            if getattr(cfg.hf, name) != getattr(d.hf, name):
                _warn(
                    f"model.hf.{name} only applies when model.backbone_type='hf_deberta_v2'. "
                    f"Current value ({getattr(cfg.hf, name)!r}) has no effect on the rope backbone."
                )
    if cfg.backbone_type == "rope" and cfg.from_scratch and asdict(cfg.rope.pretrained) != asdict(d.rope.pretrained):
        raise ValueError("These options apply only when model.from_scratch=false: model.rope.pretrained.*")
    if cfg.backbone_type == "rope" and not cfg.from_scratch:
        bad = [f"{n}={getattr(cfg.pretrained, n)}" for n in ("discriminator_path", "generator_path")
               if getattr(cfg.pretrained, n) and _looks_like_hf_deberta_checkpoint(str(getattr(cfg.pretrained, n)))]
        if bad:
            raise ValueError(
                "model.from_scratch=false with model.backbone_type='rope' requires DebertaRoPE checkpoints, "
                "not HF DeBERTa v2/v3 checkpoints. Use model.backbone_type='hf_deberta_v2' for HF DeBERTa weights, "
                "or keep model.from_scratch=true for RoPE model initialization. Invalid sources: " + ", ".join(sorted(bad))
            )
        if asdict(replace(cfg.rope, pretrained=d.rope.pretrained)) != asdict(d.rope):
            raise ValueError(
                "These options only affect scratch RoPE initialization and are not applied when "
                "model.from_scratch=false. Use explicit model.rope.pretrained.* overrides instead."
            )
        pre = cfg.rope.pretrained
        if pre.max_position_embeddings is not None and int(pre.max_position_embeddings) <= 0:
            raise ValueError("model.rope.pretrained.max_position_embeddings must be > 0 when provided.")
        if pre.rotary_pct is not None and not 0.0 < float(pre.rotary_pct) <= 1.0:
            raise ValueError("model.rope.pretrained.rotary_pct must be in (0, 1] when provided.")
        for name in ("norm_arch", "ffn_type"):
            if getattr(pre, name) is not None:
                v = str(getattr(pre, name)).strip().lower()
                if v not in _CHOICES[f"model.rope.{name}"]:
                    raise ValueError(
                        f"model.rope.pretrained.{name} must be one of: "
                        f"{'|'.join(sorted(_CHOICES[f'model.rope.{name}']))}. Got: {getattr(pre, name)}"
                    )
                _set(pre, name, v)
    if cfg.pretrained.generator_path and asdict(cfg.generator) != asdict(d.generator):
        raise ValueError(
            "model.generator.* overrides are only used when deriving generator config and must be unset "
            "when model.pretrained.generator_path is provided."
        )
    if not cfg.from_scratch and not cfg.pretrained.generator_path:
        g = cfg.generator
        if g.hidden_size is not None or g.intermediate_size is not None or g.num_attention_heads is not None:
            raise ValueError(
                "model.from_scratch=false with derived generator weights (pretrained.generator_path unset) "
                "cannot use model.generator shape overrides."
            )
    if cfg.backbone_type == "rope":
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size"):
            if int(getattr(cfg.rope, name)) <= 0:
                raise ValueError(f"model.rope.{name} must be > 0.")
        if int(cfg.rope.hidden_size) % int(cfg.rope.num_attention_heads):
            raise ValueError("model.rope.hidden_size must be divisible by model.rope.num_attention_heads.")
    if cfg.rope.norm_arch == "post":
        if cfg.rope.keel_alpha_init is not None:
            _warn("model.rope.keel_alpha_init has no effect when model.rope.norm_arch='post'. "
                  "Set model.rope.norm_arch='keel' to use KEEL alpha scaling.")
        if cfg.rope.keel_alpha_learnable != d.rope.keel_alpha_learnable:
            _warn("model.rope.keel_alpha_learnable has no effect when model.rope.norm_arch='post'. "
                  "Set model.rope.norm_arch='keel' to use learnable KEEL alpha.")
    if cfg.rope.ffn_type == "mlp" and cfg.rope.swiglu_adjust_intermediate != d.rope.swiglu_adjust_intermediate:
        _warn("model.rope.swiglu_adjust_intermediate has no effect when model.rope.ffn_type='mlp'. "
              "The intermediate size scaling is only applied for ffn_type='swiglu'.")


def validate_data_config(cfg: DataConfig) -> None:
    src, pack = cfg.source, cfg.packing
    if src.load_from_disk:
        if src.streaming:
            raise ValueError("data.source.streaming=true is not compatible with data.source.load_from_disk. "
                             "Set data.source.streaming=false.")
        clash = [f"data.source.{n}" for n in ("dataset_name", "data_files", "dataset_config_name") if getattr(src, n)]
        if clash:
            raise ValueError("data.source.load_from_disk cannot be combined with: " + ", ".join(sorted(clash)))
    if src.dataset_config_name and not src.dataset_name:
        raise ValueError("data.source.dataset_config_name requires data.source.dataset_name.")
    if not src.load_from_disk and not src.dataset_name and not src.data_files:
        raise ValueError("No dataset source configured. Provide one of: data.source.load_from_disk, "
                         "data.source.dataset_name, or data.source.data_files.")
    if int(pack.max_seq_length) < 8:
        raise ValueError("data.packing.max_seq_length must be >= 8 for pretraining.")
    if int(src.shuffle_buffer_size) < 0:
        raise ValueError("data.source.shuffle_buffer_size must be >= 0.")
    if not src.streaming and int(src.shuffle_buffer_size) not in {0, 1}:
        raise ValueError("data.source.shuffle_buffer_size must be 0 or 1 when data.source.streaming=false "
                         "(non-streaming datasets only support shuffle off/on).")
    if not pack.enabled and pack.block_cross_document_attention:
        raise ValueError("data.packing.block_cross_document_attention=true requires data.packing.enabled=true.")
    if pack.enabled and pack.block_cross_document_attention and int(pack.max_seq_length) > _DENSE_DOC_BLOCK_WARN_SEQ_LEN:
        _warn(
            "data.packing.block_cross_document_attention builds dense O(S^2) pairwise masks in the reference "
            f"implementation. Configured data.packing.max_seq_length={int(pack.max_seq_length)} may be expensive "
            f"there (warning threshold: {_DENSE_DOC_BLOCK_WARN_SEQ_LEN}); the sm_100a attention kernels take "
            "document ids directly and skip other documents' tiles instead."
        )


def validate_train_config(cfg: TrainConfig) -> None:
    _set(cfg, "sdpa_kernel", normalize_choice("train.sdpa_kernel", cfg.sdpa_kernel))
    _set(cfg, "mixed_precision", normalize_mixed_precision(cfg.mixed_precision))
    for name in ("mode", "scope", "backend"):
        _set(cfg.compile, name, normalize_choice(f"train.compile.{name}", getattr(cfg.compile, name)))
    ck = cfg.checkpoint
    _set(ck, "resume_data_strategy", normalize_choice("train.checkpoint.resume_data_strategy", ck.resume_data_strategy))
    di = cfg.distributed
    _set(di, "parallelism", normalize_choice("train.distributed.parallelism", di.parallelism))
    _set(di, "nvls", normalize_choice("train.distributed.nvls", di.nvls))
    for name in ("comm_timeout_s", "step_deadline_s", "heartbeat_s"):
        if float(getattr(di, name)) < 0.0:
            raise ValueError(f"train.distributed.{name} must be >= 0.")
    if float(di.comm_timeout_s) == 0.0:
        raise ValueError("train.distributed.comm_timeout_s must be > 0: device-side waits are always bounded.")
    if ck.output_dir is not None and not str(ck.output_dir).strip():
        _set(ck, "output_dir", None)
    if ck.resume_from_checkpoint is not None:
        _set(ck, "resume_from_checkpoint", str(ck.resume_from_checkpoint).strip() or None)
    if ck.overwrite_output_dir and ck.resume_from_checkpoint:
        raise ValueError("train.checkpoint.overwrite_output_dir=true cannot be combined with "
                         "train.checkpoint.resume_from_checkpoint. Overwrite would delete checkpoints before resume.")
    for name, lo in (("max_steps", 1), ("per_device_train_batch_size", 1), ("gradient_accumulation_steps", 1),
                     ("dataloader.num_workers", 0), ("checkpoint.save_steps", 0), ("checkpoint.save_total_limit", 0),
                     ("checkpoint.resume_replay_max_micro_batches", 0), ("objective.mlm_max_ngram", 1)):
        if int(_nested_get(cfg, name)) < lo:
            raise ValueError(f"train.{name} must be >= {lo}.")
    if not 0.0 < float(cfg.objective.mlm_probability) < 1.0:
        raise ValueError("train.objective.mlm_probability must be in (0, 1).")
    mp, rp = float(cfg.objective.mask_token_prob), float(cfg.objective.random_token_prob)
    if mp < 0.0 or rp < 0.0 or mp + rp > 1.0:
        raise ValueError("Invalid masking probabilities: train.objective.mask_token_prob + "
                         "train.objective.random_token_prob must be <= 1.")
    if float(cfg.objective.sampling_temperature) <= 0.0:
        raise ValueError("train.objective.sampling_temperature must be > 0.")
    if not isinstance(cfg.decoupled_training, bool):
        raise ValueError("train.decoupled_training must be a boolean (true/false). "
                         f"Got {type(cfg.decoupled_training).__name__}.")
    if not cfg.compile.enabled:
        d = TrainCompileConfig()
        for name in ("mode", "scope", "backend"):
            if getattr(cfg.compile, name) != getattr(d, name):
                _warn(f"train.compile.{name} has no effect when train.compile.enabled=false. "
                      f"Current value ({getattr(cfg.compile, name)!r}) will be ignored.")


def validate_optim_config(cfg: OptimConfig) -> None:
    _set(cfg.scheduler, "type", normalize_choice("optim.scheduler.type", cfg.scheduler.type))
    if float(cfg.lr.base) <= 0.0:
        raise ValueError("optim.lr.base must be > 0.")
    for name in ("generator", "discriminator"):
        v = float(getattr(cfg.lr, name))
        if v != -1.0 and v <= 0.0:
            raise ValueError(f"optim.lr.{name} must be -1 (inherit) or > 0.")
    if float(cfg.weight_decay) < 0.0:
        raise ValueError("optim.weight_decay must be >= 0.")
    if float(cfg.max_grad_norm) < 0.0:
        raise ValueError("optim.max_grad_norm must be >= 0.")
    if int(cfg.scheduler.warmup_steps) < 0:
        raise ValueError("optim.scheduler.warmup_steps must be >= 0.")


def validate_logging_config(cfg: LoggingConfig) -> None:
    _set(cfg, "backend", normalize_choice("logging.backend", cfg.backend))
    _set(cfg.wandb, "watch", normalize_choice("logging.wandb.watch", cfg.wandb.watch))
    if not str(cfg.project_name).strip():
        raise ValueError("logging.project_name must be non-empty.")
    if cfg.output_dir is not None and not str(cfg.output_dir).strip():
        _set(cfg, "output_dir", None)
    if int(cfg.logging_steps) < 0:
        raise ValueError("logging.logging_steps must be >= 0.")
    if int(cfg.wandb.watch_log_freq) < 1:
        raise ValueError("logging.wandb.watch_log_freq must be >= 1.")
    if not cfg.wandb.enabled:
        d = LoggingWandbConfig()
        if cfg.wandb.watch != d.watch:
            _warn("logging.wandb.watch only applies when logging.wandb.enabled=true. "
                  f"Current value ({cfg.wandb.watch!r}) will be ignored.")
        if int(cfg.wandb.watch_log_freq) != d.watch_log_freq:
            _warn("logging.wandb.watch_log_freq only applies when logging.wandb.enabled=true. "
                  f"Current value ({int(cfg.wandb.watch_log_freq)}) will be ignored.")


def validate_training_workflow_options(*, data_cfg: DataConfig, train_cfg: TrainConfig,
                                       model_cfg: ModelConfig | None = None, optim_cfg: OptimConfig | None = None,
                                       logging_cfg: LoggingConfig | None = None) -> None:
    """Cross-section rules (SDPA policy × packing, doc-blocking × backbone, ES × optimiser layout)."""
    sdpa = str(train_cfg.sdpa_kernel).strip().lower()
    blocking = bool(data_cfg.packing.enabled) and bool(data_cfg.packing.block_cross_document_attention)
    if blocking and sdpa == "flash":
        raise ValueError(
            "train.sdpa_kernel=flash is not supported with data.packing.enabled=true. "
            "Packed batches may require 3D document-blocking attention masks that are incompatible "
            "with strict flash SDPA kernels. Use train.sdpa_kernel=auto|mem_efficient|math instead."
        )
    if model_cfg is None:
        return
    backbone = str(model_cfg.backbone_type).strip().lower()
    if backbone != "rope" and sdpa != "auto":
        _warn("train.sdpa_kernel has no effect when model.backbone_type='hf_deberta_v2'. "
              "The HF DeBERTa-v2 disentangled attention does not go through scaled_dot_product_attention. "
              f"Current value ({train_cfg.sdpa_kernel!r}) will be ignored.")
    if backbone == "rope" and str(model_cfg.rope.attention_implementation).lower() != "sdpa" and sdpa != "auto":
        raise ValueError(
            "train.sdpa_kernel only affects rope attention when model.rope.attention_implementation='sdpa'. "
            "Set train.sdpa_kernel=auto or switch model.rope.attention_implementation=sdpa."
        )
    if backbone != "rope" and blocking:
        raise ValueError(
            "data.packing.block_cross_document_attention=true is only supported with model.backbone_type='rope'. "
            "Use data.packing.block_cross_document_attention=false or switch to model.backbone_type='rope'."
        )
    sharing = str(model_cfg.embedding_sharing).strip().lower()
    opt = optim_cfg or OptimConfig()
    gen_lr = float(opt.lr.generator)
    if sharing == "es" and gen_lr > 0 and gen_lr != float(opt.lr.base):
        raise ValueError(
            "model.embedding_sharing='es' shares embedding parameters between generator and discriminator, "
            f"but optim.lr.generator ({gen_lr}) differs from optim.lr.base ({opt.lr.base}). "
            "Set optim.lr.generator=-1 (inherit) or match it to optim.lr.base, or switch to embedding_sharing='gdes'/'none'."
        )
    if train_cfg.decoupled_training and sharing == "es":
        raise ValueError(
            "train.decoupled_training is incompatible with model.embedding_sharing='es' because shared embedding "
            "parameters are assigned to the generator optimizer only, so discriminator-phase gradients on them "
            "would be dropped. Use embedding_sharing='gdes' or 'none' for decoupled training."
        )


def apply_profile_defaults(*, model_cfg: ModelConfig, train_cfg: TrainConfig, optim_cfg: OptimConfig | None = None) -> None:
    """Profile/backbone defaults that yield to anything the user set explicitly (file or flag)."""
    em, et, eo = _explicit_fields(model_cfg), _explicit_fields(train_cfg), _explicit_fields(optim_cfg)
    dm, dt, do = ModelConfig(), TrainConfig(), OptimConfig()

    def maybe(obj, root_default, explicit, path, value):
        if path in explicit or _nested_get(obj, path) != _nested_get(root_default, path):
            return
        parent = _nested_get(obj, path.rsplit(".", 1)[0]) if "." in path else obj
        _set(parent, path.rsplit(".", 1)[-1], value)

    if str(model_cfg.profile).strip().lower() == "deberta_v3_parity":
        maybe(model_cfg, dm, em, "backbone_type", "hf_deberta_v2")
        maybe(model_cfg, dm, em, "embedding_sharing", "gdes")
        maybe(model_cfg, dm, em, "hf.attention_kernel", "dynamic")
    if str(model_cfg.backbone_type).strip().lower() == "hf_deberta_v2":
        maybe(train_cfg, dt, et, "objective.mask_token_prob", 1.0)
        maybe(train_cfg, dt, et, "objective.random_token_prob", 0.0)
        maybe(train_cfg, dt, et, "objective.disc_loss_weight", 10.0)
        if optim_cfg is not None:
            maybe(optim_cfg, do, eo, "adam.epsilon", 1e-6)
            maybe(optim_cfg, do, eo, "scheduler.warmup_steps", 10_000)
        maybe(train_cfg, dt, et, "token_weighted_gradient_accumulation", True)


def validate_run_metadata_schema(raw: dict[str, object], *, source: str) -> None:
    if "config_schema_version" not in raw:
        raise ValueError(f"run metadata missing `config_schema_version` at {source}. "
                         "Refusing resume/export with ambiguous config schema.")
    try:
        version = int(raw["config_schema_version"])  # type: ignore[arg-type]
    except Exception as e:
        raise ValueError(f"Invalid config_schema_version in {source}: {raw['config_schema_version']!r}") from e
    if version != RUN_CONFIG_SCHEMA_VERSION:
        raise ValueError(
            f"Unsupported run metadata schema at {source}: {version}. Expected {RUN_CONFIG_SCHEMA_VERSION}. "
            "Backward resume/export compatibility is not guaranteed before stable release."
        )


def _load_snapshot(raw: dict[str, object], cls: type, source: str, name: str):
    expected = {f.name for f in fields(cls)}
    unknown, missing = sorted(set(raw) - expected), sorted(expected - set(raw))
    if unknown:
        raise ValueError(f"Unsupported {name} keys in {source}: {', '.join(unknown)}. This snapshot was produced by an "
                         "older pre-release schema; backward resume/export compatibility is not guaranteed.")
    if missing:
        raise ValueError(f"Missing required {name} keys in {source}: {', '.join(missing)}. "
                         "This snapshot does not match the current config schema.")
    try:
        return cls(**raw)
    except TypeError as e:
        raise ValueError(f"Failed to parse {name} at {source}. The persisted config schema does not match "
                         "this code version.") from e


def load_model_config_snapshot(raw, *, source: str) -> ModelConfig:
    return _load_snapshot(raw, ModelConfig, source, "model_config.json")


def load_data_config_snapshot(raw, *, source: str) -> DataConfig:
    return _load_snapshot(raw, DataConfig, source, "data_config.json")


def load_train_config_snapshot(raw, *, source: str) -> TrainConfig:
    return _load_snapshot(raw, TrainConfig, source, "train_config.json")


def load_optim_config_snapshot(raw, *, source: str) -> OptimConfig:
    return _load_snapshot(raw, OptimConfig, source, "optim_config.json")


def load_logging_config_snapshot(raw, *, source: str) -> LoggingConfig:
    return _load_snapshot(raw, LoggingConfig, source, "logging_config.json")


# ---------------------------------------------------------------------------------------------
# file loading
# ---------------------------------------------------------------------------------------------
_VAR_FULL_RE = re.compile(r"^\$variables\.([A-Za-z0-9_.-]+)$")
_VAR_INLINE_RE = re.compile(r"\{\$variables\.([A-Za-z0-9_.-]+)\}")
_VAR_BRACE_RE = re.compile(r"\$\{variables\.([A-Za-z0-9_.-]+)\}")
_VAR_SUSPICIOUS_RE = re.compile(r"\$variables\.[A-Za-z0-9_.-]+")
_SECTIONS = ("model", "data", "train", "optim", "logging")
_SECTION_CLASSES = {"model": ModelConfig, "data": DataConfig, "train": TrainConfig, "optim": OptimConfig,
                    "logging": LoggingConfig}
# flat keys of earlier schema versions and where their values live now
_MOVED_TRAIN_KEYS = {
    "project_name": "logging.project_name", "run_name": "logging.run_name",
    "report_to": "logging.wandb.enabled + logging.backend", "logging_steps": "logging.logging_steps",
    "wandb_watch": "logging.wandb.watch", "wandb_watch_log_freq": "logging.wandb.watch_log_freq",
    "debug_metrics": "logging.debug.metrics", **{k: f"optim.{v}" for k, v in OptimConfig._LEGACY.items()},
    "weight_decay": "optim.weight_decay", "max_grad_norm": "optim.max_grad_norm",
}


def _legacy_key_suggestion(section: str, key: str) -> str | None:
    """Where an unknown (older-schema) key should be written today, if we know."""
    if section in ("model", "data", "train"):
        path = _SECTION_CLASSES[section]._LEGACY.get(key)
        if path is not None:
            return f"{section}.{path}"
        if section == "model" and key.startswith("pretrained_"):
            return "model.rope.pretrained.<field>"
        if section == "train":
            return _MOVED_TRAIN_KEYS.get(key)
    if section == "root":
        return {"checkpoint": "train.checkpoint", "debug": "logging.debug"}.get(key)
    return None


def _load_raw_config_mapping(path: str | Path) -> tuple[dict[str, Any], str]:
    p = Path(path).expanduser().resolve()
    suffix = p.suffix.lower()
    if suffix not in {".yaml", ".yml", ".json"}:
        raise ValueError("Config file must end with .json, .yaml, or .yml")
    if suffix == ".json":
        return load_json_mapping(p), "JSON"
    import yaml

    raw = yaml.safe_load(p.read_text(encoding="utf-8")) or {}
    if not isinstance(raw, dict):
        raise ValueError("Config file must parse to a dict.")
    return raw, "YAML"


def _resolve_variables(data: dict[str, Any]) -> dict[str, Any]:
    """Substitute ``$variables.a.b`` (whole value, keeps type) and ``{$variables.x}`` / ``${variables.x}`` (inline)."""
    raw_vars = data.get("variables") or {}
    if not isinstance(raw_vars, dict):
        raise ValueError("variables must be a mapping if provided.")
    done: dict[str, Any] = {}
    stack: list[str] = []

    def lookup(path: str) -> Any:
        if path in done:
            return done[path]
        if path in stack:
            raise ValueError(f"Circular variable reference: {' -> '.join(stack + [path])}")
        cur: Any = raw_vars
        for part in path.split("."):
            if not isinstance(cur, dict) or part not in cur:
                raise ValueError(f"Unknown variable reference: variables.{path}")
            cur = cur[part]
        stack.append(path)
        done[path] = resolve(cur)
        stack.pop()
        return done[path]

    def resolve(value: Any) -> Any:
        if isinstance(value, dict):
            return {k: resolve(v) for k, v in value.items()}
        if isinstance(value, list):
            return [resolve(v) for v in value]
        if not isinstance(value, str):
            return value
        full = _VAR_FULL_RE.fullmatch(value)
        if full:
            return lookup(full.group(1))
        sub = lambda m: str(lookup(m.group(1)))  # noqa: E731
        out = _VAR_BRACE_RE.sub(sub, _VAR_INLINE_RE.sub(sub, value))
        left = _VAR_SUSPICIOUS_RE.findall(out)
        if left:
            warnings.warn(f"String contains unresolved variable-like patterns: {left}. "
                          "Use {$variables.name} or ${variables.name} for inline substitution.", stacklevel=2)
        return out

    for path in sorted(leaf_paths(raw_vars)):
        lookup(path)
    return {k: resolve(v) for k, v in data.items() if k != "variables"}


def _split_full_sections(raw: dict[str, Any], *, format_name: str) -> dict[str, dict[str, Any]]:
    unknown = sorted(k for k in raw if k not in _SECTIONS)
    if unknown:
        shown = [f"{k} (use {_legacy_key_suggestion('root', k)})" if _legacy_key_suggestion("root", k) else str(k)
                 for k in unknown]
        raise ValueError(f"Unknown top-level keys in nested {format_name} config "
                         f"(expected only {', '.join(sorted(_SECTIONS))}): {', '.join(shown)}")
    out = {k: (raw.get(k) or {}) for k in _SECTIONS}
    for k, v in out.items():
        if not isinstance(v, dict):
            raise ValueError(f"{format_name} config section {k!r} must be a dict.")
    return out


def _coerce_file_scalar(raw: Any, field_type: Any, path: str) -> Any:
    """Strict typing of values read from files: booleans must be booleans, numeric strings are accepted."""
    target, optional = unwrap_optional_type(field_type)
    if raw is None:
        if optional:
            return None
        raise ValueError(f"Config field {path} cannot be null.")
    if target is bool:
        if isinstance(raw, bool):
            return raw
        raise ValueError(f"Config field {path} must be a boolean true/false, got {type(raw).__name__}: {raw!r}.")
    if target in (int, float):
        word = "an integer" if target is int else "a number"
        if isinstance(raw, bool):
            raise ValueError(f"Config field {path} must be {word}, got bool: {raw!r}.")
        if isinstance(raw, int) or (target is float and isinstance(raw, float)):
            return target(raw)
        if isinstance(raw, str):
            try:
                return target(raw.strip())
            except ValueError as exc:
                raise ValueError(f"Config field {path} must be {word}, got string: {raw!r}.") from exc
        raise ValueError(f"Config field {path} must be {word}, got {type(raw).__name__}: {raw!r}.")
    if target is str:
        if isinstance(raw, bool) and path == "train.mixed_precision":
            # YAML 1.1 reads a bare ``no`` / ``yes`` as a boolean; both are documented aliases here
            return normalize_mixed_precision(raw)
        if not isinstance(raw, str):
            raise ValueError(f"Config field {path} must be a string, got {type(raw).__name__}: {raw!r}.")
        return raw
    return raw


def _from_mapping(obj: Any, mapping: dict[str, Any], *, section: str) -> Any:
    if not mapping:
        return obj
    allowed = {f.name for f in fields(obj)}
    unknown = sorted(set(mapping) - allowed)
    if unknown:
        shown = [f"{k} (use {_legacy_key_suggestion(section, k)})" if _legacy_key_suggestion(section, k) else str(k)
                 for k in unknown]
        raise ValueError(f"Unknown keys in section {section!r}: {', '.join(shown)}")
    hints = get_type_hints(type(obj))
    updates: dict[str, Any] = {}
    for key, value in mapping.items():
        cur = getattr(obj, key)
        if dataclasses.is_dataclass(cur):
            if not isinstance(value, dict):
                raise ValueError(f"Section {section}.{key} must be a mapping.")
            updates[key] = _from_mapping(cur, value, section=f"{section}.{key}")
        else:
            updates[key] = _coerce_file_scalar(value, hints.get(key, Any), f"{section}.{key}")
    return replace(obj, **updates)


def _build_config_from_section_mappings(maps: dict[str, dict[str, Any]]) -> Config:
    parts = {}
    for name, cls in _SECTION_CLASSES.items():
        parts[name] = _from_mapping(cls(), maps.get(name, {}), section=name)
        _mark_explicit_fields(parts[name], leaf_paths(maps.get(name, {})))
    cfg = Config(**parts)
    _sync_legacy_train_aliases(train_cfg=cfg.train, optim_cfg=cfg.optim, logging_cfg=cfg.logging)
    return cfg


def config_from_mapping(raw: dict[str, Any], *, format_name: str = "mapping") -> Config:
    """Build a (not yet validated) ``Config`` from a nested mapping with an optional ``variables`` block."""
    return _build_config_from_section_mappings(_split_full_sections(_resolve_variables(raw), format_name=format_name))


def apply_dotted_override(cfg: Config, override: str) -> Config:
    """Apply ``section.path=value`` to a Config; the leaf is recorded as explicitly set."""
    text = str(override).strip()
    if "=" not in text:
        raise ValueError(f"Invalid override {override!r}. Expected format like model.rope.hidden_size=768.")
    path, raw_value = (s.strip() for s in text.split("=", 1))
    parts = [p.strip() for p in path.split(".") if p.strip()]
    if len(parts) < 2:
        raise ValueError(f"Invalid override path {path!r}. Expected format section.field (for example train.max_steps).")
    root = parts[0]
    if root not in _SECTIONS:
        raise ValueError(f"Unknown override section {root!r}; expected one of {', '.join(sorted(_SECTIONS))}.")

    def apply(obj: Any, rest: list[str]) -> Any:
        key = rest[0]
        if not dataclasses.is_dataclass(obj) or key not in {f.name for f in fields(obj)}:
            raise ValueError(f"Unknown override field {path!r}.")
        if len(rest) == 1:
            if dataclasses.is_dataclass(getattr(obj, key)):
                raise ValueError(f"Override path {path!r} names a section, not a field.")
            tp = get_type_hints(type(obj)).get(key, Any)
            return replace(obj, **{key: coerce_scalar(raw_value, tp, allow_none=False, allow_bool_numeric=False)})
        return replace(obj, **{key: apply(getattr(obj, key), rest[1:])})

    old = getattr(cfg, root)
    new = apply(old, parts[1:])
    _mark_explicit_fields(new, _explicit_fields(old) | {".".join(parts[1:])})
    out = replace(cfg, **{root: new})
    _sync_legacy_train_aliases(train_cfg=out.train, optim_cfg=out.optim, logging_cfg=out.logging)
    return out


def validate_config(cfg: Config) -> Config:
    """Profile defaults + all validators + alias mirroring, in the order the CLI applies them."""
    apply_profile_defaults(model_cfg=cfg.model, train_cfg=cfg.train, optim_cfg=cfg.optim)
    validate_model_config(cfg.model)
    validate_data_config(cfg.data)
    validate_train_config(cfg.train)
    validate_optim_config(cfg.optim)
    validate_logging_config(cfg.logging)
    validate_training_workflow_options(data_cfg=cfg.data, train_cfg=cfg.train, model_cfg=cfg.model,
                                       optim_cfg=cfg.optim, logging_cfg=cfg.logging)
    _sync_legacy_train_aliases(train_cfg=cfg.train, optim_cfg=cfg.optim, logging_cfg=cfg.logging)
    return cfg


def load_config(path: str | Path, overrides: list[str] | None = None) -> Config:
    """File → variables → sections → typed dataclasses → overrides → profile defaults → validation."""
    raw, fmt = _load_raw_config_mapping(path)
    cfg = config_from_mapping(raw, format_name=fmt)
    for expr in overrides or []:
        cfg = apply_dotted_override(cfg, expr)
    return validate_config(cfg)


def iter_leaf_paths_for_dataclass(cls: type, *, prefix: str = "") -> list[tuple[str, Any]]:
    """``[(dotted.path, annotated type), …]`` for every scalar leaf under a config dataclass."""
    out: list[tuple[str, Any]] = []
    hints = get_type_hints(cls)
    for f in fields(cls):
        path = f"{prefix}.{f.name}" if prefix else f.name
        target, _ = unwrap_optional_type(hints.get(f.name, f.type))
        if dataclasses.is_dataclass(target):
            out.extend(iter_leaf_paths_for_dataclass(target, prefix=path))
        else:
            out.append((path, hints.get(f.name, f.type)))
    return out


__all__ = [
    "RUN_CONFIG_SCHEMA_VERSION", "Config", "ModelConfig", "DataConfig", "TrainConfig", "OptimConfig", "LoggingConfig",
    "apply_dotted_override", "apply_profile_defaults", "asdict_without_private", "choices_for", "config_from_mapping",
    "iter_leaf_paths_for_dataclass", "load_config", "load_data_config_snapshot", "load_logging_config_snapshot",
    "load_model_config_snapshot", "load_optim_config_snapshot", "load_train_config_snapshot", "normalize_choice",
    "normalize_mixed_precision", "resolve_effective_mixed_precision", "validate_config", "validate_data_config",
    "validate_logging_config", "validate_model_config", "validate_optim_config", "validate_run_metadata_schema",
    "validate_train_config", "validate_training_workflow_options",
]
