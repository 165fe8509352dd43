"""Backbone config/weight resolution for the generator and the discriminator.

Behaviour follows ``modeling/builder.py`` of the reference: repo-owned HF presets
(xsmall/small/base/large) for scratch ``hf_deberta_v2`` runs, synthetic
``DebertaRoPEConfig`` for scratch rope runs, ``from_pretrained`` sources otherwise; the
generator is derived from the discriminator (half depth for hf, one third for rope)
unless its own source is given; tokenizer ↔ config vocabulary and special-id contract
with optional placeholder-token growth.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from deberta_b200.config import ModelConfig, validate_model_config

from .deberta_v2 import DebertaV2Config, DebertaV2Model
from .rope_encoder import DebertaRoPEConfig, DebertaRoPEModel

__all__ = ["build_backbone_configs", "build_backbones", "resolve_backbone_sources", "HF_PRESETS"]

_SPECIAL_ID_ATTRS = ("pad_token_id", "cls_token_id", "sep_token_id", "mask_token_id", "bos_token_id", "eos_token_id")
_EXTRA_TOKEN_TEMPLATE = "<|deberta_extra_token_{idx}|>"

HF_PRESETS: dict[str, dict[str, int]] = {
    "xsmall": {"hidden_size": 384, "num_hidden_layers": 12, "num_attention_heads": 6, "intermediate_size": 1536},
    "small": {"hidden_size": 768, "num_hidden_layers": 6, "num_attention_heads": 12, "intermediate_size": 3072},
    "base": {"hidden_size": 768, "num_hidden_layers": 12, "num_attention_heads": 12, "intermediate_size": 3072},
    "large": {"hidden_size": 1024, "num_hidden_layers": 24, "num_attention_heads": 16, "intermediate_size": 4096},
}


@dataclass(frozen=True)
class ComponentSources:
    component: str
    config_source: str | None
    config_origin: str
    weight_source: str | None
    weight_origin: str
    derived_from_discriminator: bool


@dataclass(frozen=True)
class BackboneSources:
    discriminator: ComponentSources
    generator: ComponentSources


def resolve_backbone_sources(model_cfg: ModelConfig) -> BackboneSources:
    """Where each component's config and weights come from (``builder.py:185-299``)."""
    hf = (model_cfg.backbone_type or "hf_deberta_v2").lower() == "hf_deberta_v2"
    scratch = bool(model_cfg.from_scratch)
    disc_path = model_cfg.pretrained.discriminator_path or None
    gen_path = model_cfg.pretrained.generator_path or None
    if hf or not scratch:
        d_cfg = None if (hf and scratch) else disc_path
    else:
        d_cfg = None
    if d_cfg is None:
        d_origin = "repo_hf_defaults" if hf else "synthetic_from_model_cfg"
    else:
        d_origin = "pretrained_discriminator_path"
    disc = ComponentSources("discriminator", d_cfg, d_origin, None if scratch else disc_path,
                            "scratch" if scratch else "pretrained_discriminator_path", False)
    g_cfg_origin = "pretrained_generator_path" if gen_path else "derived_from_discriminator_config"
    if scratch:
        g_w, g_w_origin = None, "scratch"
    elif gen_path:
        g_w, g_w_origin = gen_path, "pretrained_generator_path"
    else:
        g_w, g_w_origin = disc_path, "derived_from_pretrained_discriminator_path"
    gen = ComponentSources("generator", gen_path, g_cfg_origin, g_w, g_w_origin, gen_path is None)
    return BackboneSources(disc, gen)


# ---- tokenizer / vocabulary contract -----------------------------------------------------------
def _tok_len(tokenizer: Any) -> int:
    try:
        return int(len(tokenizer))
    except Exception as e:
        raise ValueError("Tokenizer must support len(tokenizer) for vocab-size alignment.") from e


def _round_up(value: int, multiple: int) -> int:
    return int(value) if multiple <= 1 or value % multiple == 0 else int(value) + (multiple - value % multiple)


def _grow_tokenizer(tokenizer: Any, target: int, component: str, allow: bool) -> None:
    """Append inert placeholder tokens until ``len(tokenizer) == target``."""
    cur = _tok_len(tokenizer)
    if target <= cur:
        return
    if not allow:
        raise ValueError(
            f"{component} tokenizer vocab ({cur}) is smaller than required size ({target}), "
            "but model.tokenizer_allow_vocab_resize=false. Enable tokenizer resize or align vocab settings."
        )
    add = getattr(tokenizer, "add_tokens", None)
    if not callable(add):
        raise ValueError(f"{component} tokenizer does not support add_tokens(...), cannot grow vocab from {cur} to {target}.")
    added = int(add([_EXTRA_TOKEN_TEMPLATE.format(idx=i) for i in range(cur, target)], special_tokens=False))
    if added != target - cur or _tok_len(tokenizer) != target:
        raise RuntimeError(f"Failed to grow {component} tokenizer vocab: needed={target - cur}, added={added}, "
                           f"final_size={_tok_len(tokenizer)}, target={target}.")


def _required_vocab(current: int, model_cfg: ModelConfig, scratch: bool, component: str, cfg_vocab: int | None) -> int:
    target = model_cfg.tokenizer.vocab_target
    multiple = int(model_cfg.tokenizer.vocab_multiple)
    want = current
    if target is not None:
        if int(target) < current:
            raise ValueError(f"model.tokenizer_vocab_target ({int(target)}) is smaller than tokenizer size "
                             f"({current}) for {component}; shrinking tokenizer vocab is not supported.")
        want = max(want, int(target))
    if not scratch:
        if cfg_vocab is None:
            raise ValueError(f"{component} config vocab_size is required in pretrained mode.")
        if current > cfg_vocab:
            raise ValueError(f"Tokenizer/checkpoint vocab mismatch for {component}: tokenizer={current}, "
                             f"config={cfg_vocab}. Use a matching tokenizer or checkpoint.")
        if target is None and model_cfg.tokenizer.allow_vocab_resize:
            want = max(want, cfg_vocab)
        if want > cfg_vocab:
            raise ValueError(f"Requested tokenizer vocab for {component} ({want}) exceeds checkpoint config "
                             f"vocab_size ({cfg_vocab}).")
    want = _round_up(want, multiple)
    if not scratch and want > int(cfg_vocab):
        raise ValueError(f"model.tokenizer_vocab_multiple={multiple} rounds {component} tokenizer size to {want}, "
                         f"which exceeds checkpoint config vocab_size ({cfg_vocab}).")
    return want


def _align_tokenizer_contract(cfg: Any, tokenizer: Any, *, component: str, model_cfg: ModelConfig) -> None:
    """Scratch: config takes vocab size and special ids from the tokenizer. Pretrained: they must agree."""
    scratch = bool(model_cfg.from_scratch)
    allow = bool(model_cfg.tokenizer.allow_vocab_resize)
    if scratch:
        _grow_tokenizer(tokenizer, _required_vocab(_tok_len(tokenizer), model_cfg, True, component, None), component, allow)
        cfg.vocab_size = _tok_len(tokenizer)
        for attr in _SPECIAL_ID_ATTRS:
            tid = getattr(tokenizer, attr, None)
            if tid is not None:
                try:
                    setattr(cfg, attr, int(tid))
                except (TypeError, ValueError):
                    pass
        return
    cfg_vocab = getattr(cfg, "vocab_size", None)
    if cfg_vocab is None:
        raise ValueError(f"{component} config is missing vocab_size; cannot validate tokenizer/checkpoint compatibility.")
    _grow_tokenizer(tokenizer, _required_vocab(_tok_len(tokenizer), model_cfg, False, component, int(cfg_vocab)),
                    component, allow)
    if int(cfg_vocab) != _tok_len(tokenizer):
        raise ValueError(f"Tokenizer/checkpoint vocab mismatch for {component}: tokenizer={_tok_len(tokenizer)}, "
                         f"config={int(cfg_vocab)}. Use a matching tokenizer or checkpoint.")
    for attr in _SPECIAL_ID_ATTRS:
        tid = getattr(tokenizer, attr, None)
        if tid is None:
            continue
        have = getattr(cfg, attr, None)
        if have is None:
            setattr(cfg, attr, int(tid))
            continue
        try:
            have_i = int(have)
        except Exception as e:
            raise ValueError(f"Invalid {component} config field {attr}={have!r}; expected int-like token id.") from e
        if have_i != int(tid):
            raise ValueError(f"Tokenizer/config special-token mismatch for {component}.{attr}: tokenizer={int(tid)}, "
                             f"config={have_i}. Use a tokenizer compatible with the checkpoint.")


def _check_max_positions(cfg: Any, required: int, component: str) -> None:
    have = getattr(cfg, "max_position_embeddings", None)
    if have is not None and int(have) < int(required):
        raise ValueError(f"{component} max_position_embeddings={int(have)} is smaller than required "
                         f"sequence length {int(required)}.")


def scaled_swiglu_intermediate_size(value: int) -> int:
    """2/3 of the MLP width rounded up to a multiple of 128 (same parameter budget as the plain MLP)."""
    return _round_up(max(1, int(int(value) * (2.0 / 3.0))), 128)


def _derive_generator_config(base_cfg: Any, model_cfg: ModelConfig) -> Any:
    gen = copy.deepcopy(base_cfg)
    g = model_cfg.generator
    if getattr(gen, "num_hidden_layers", None) is not None:
        layers = int(gen.num_hidden_layers)
        default = max(1, layers // 2) if str(model_cfg.backbone_type).lower() == "hf_deberta_v2" else max(1, layers // 3)
        gen.num_hidden_layers = int(g.num_hidden_layers or default)
    if g.hidden_size is not None:
        gen.hidden_size = int(g.hidden_size)
    if g.intermediate_size is not None:
        gen.intermediate_size = int(g.intermediate_size)
    if g.num_attention_heads is not None:
        gen.num_attention_heads = int(g.num_attention_heads)
    if int(gen.hidden_size) % int(gen.num_attention_heads):
        raise ValueError("generator_hidden_size must be divisible by generator_num_attention_heads. "
                         f"Got hidden_size={gen.hidden_size}, heads={gen.num_attention_heads}.")
    return gen


def _apply_dropout(cfg: Any, model_cfg: ModelConfig) -> None:
    if model_cfg.dropout.hidden_prob is not None:
        cfg.hidden_dropout_prob = float(model_cfg.dropout.hidden_prob)
    if model_cfg.dropout.attention_probs_prob is not None:
        cfg.attention_probs_dropout_prob = float(model_cfg.dropout.attention_probs_prob)


def build_repo_hf_deberta_v2_config(model_size: str) -> DebertaV2Config:
    """DeBERTa-v3 architecture of the given size with the published hyper-parameters (``builder.py:613-673``)."""
    dims = HF_PRESETS[str(model_size).strip().lower()]
    return DebertaV2Config(
        vocab_size=128_100, hidden_act="gelu", hidden_dropout_prob=0.1, attention_probs_dropout_prob=0.1,
        initializer_range=0.02, layer_norm_eps=1e-7, legacy=True, pooler_hidden_size=dims["hidden_size"],
        pooler_hidden_act="gelu", pooler_dropout=0.0, z_steps=0, max_position_embeddings=512,
        max_relative_positions=-1, position_buckets=256, relative_attention=True, position_biased_input=False,
        share_att_key=True, norm_rel_ebd="layer_norm", pos_att_type=["p2c", "c2p"], type_vocab_size=0, **dims,
    )


_ROPE_PRETRAINED_OVERRIDES = (
    ("max_position_embeddings", int), ("rope_theta", float), ("rotary_pct", float),
    ("use_absolute_position_embeddings", bool), ("type_vocab_size", int), ("norm_arch", str), ("norm_eps", float),
    ("keel_alpha_init", float), ("keel_alpha_learnable", bool), ("ffn_type", str), ("use_bias", bool),
    ("initializer_range", float),
)


def _normalize_hf_config(cfg: Any, *, model_cfg: ModelConfig, tokenizer: Any, component: str) -> None:
    _align_tokenizer_contract(cfg, tokenizer, component=component, model_cfg=model_cfg)
    if model_cfg.hf.max_position_embeddings is not None:
        cfg.max_position_embeddings = int(model_cfg.hf.max_position_embeddings)
    _apply_dropout(cfg, model_cfg)
    cfg.hf_attention_kernel = str(model_cfg.hf.attention_kernel)
    cfg.use_rmsnorm_heads = False


def _normalize_rope_config(cfg: Any, *, model_cfg: ModelConfig, tokenizer: Any, max_position_embeddings: int,
                           component: str, explicit_source: bool, derived: bool) -> None:
    r = model_cfg.rope
    if model_cfg.from_scratch:
        if explicit_source:
            if r.max_position_embeddings is not None:
                cfg.max_position_embeddings = int(r.max_position_embeddings)
            elif getattr(cfg, "max_position_embeddings", None) is None:
                cfg.max_position_embeddings = int(max_position_embeddings)
        elif not derived:
            cfg.hidden_size, cfg.num_hidden_layers = int(r.hidden_size), int(r.num_hidden_layers)
            cfg.num_attention_heads, cfg.intermediate_size = int(r.num_attention_heads), int(r.intermediate_size)
            cfg.hidden_act = str(r.hidden_act)
            cfg.max_position_embeddings = int(r.max_position_embeddings or max_position_embeddings)
            cfg.rope_theta, cfg.rotary_pct = float(r.rope_theta), float(r.rotary_pct)
            cfg.use_absolute_position_embeddings = bool(r.use_absolute_position_embeddings)
            cfg.type_vocab_size, cfg.norm_eps, cfg.norm_arch = int(r.type_vocab_size), float(r.norm_eps), str(r.norm_arch)
            cfg.keel_alpha_init = None if r.keel_alpha_init is None else float(r.keel_alpha_init)
            cfg.keel_alpha_learnable = bool(r.keel_alpha_learnable)
            cfg.ffn_type, cfg.use_bias = str(r.ffn_type), bool(r.use_bias)
            cfg.initializer_range = float(r.initializer_range)
            if str(r.ffn_type).lower() == "swiglu" and r.swiglu_adjust_intermediate:
                cfg.intermediate_size = scaled_swiglu_intermediate_size(int(cfg.intermediate_size))
    else:
        for name, cast in _ROPE_PRETRAINED_OVERRIDES:
            val = getattr(r.pretrained, name, None)
            if val is not None:
                setattr(cfg, name, cast(val))
    cfg.attention_implementation = str(r.attention_implementation)
    cfg.use_rmsnorm_heads = True
    _apply_dropout(cfg, model_cfg)
    _align_tokenizer_contract(cfg, tokenizer, component=component, model_cfg=model_cfg)
    _check_max_positions(cfg, max_position_embeddings, component)


def _load_config(cls, source: str, component: str, origin: str):
    try:
        return cls.from_pretrained(source)
    except Exception as e:
        raise RuntimeError(f"Failed to load {component} config from source '{source}' (resolved from {origin}).") from e


def build_backbone_configs(*, model_cfg: ModelConfig, tokenizer: Any, max_position_embeddings: int) -> tuple[Any, Any]:
    """(discriminator config, generator config) for the configured backbone family."""
    validate_model_config(model_cfg)
    src = resolve_backbone_sources(model_cfg)
    if (model_cfg.backbone_type or "hf_deberta_v2").lower() == "hf_deberta_v2":
        d = src.discriminator
        disc = (build_repo_hf_deberta_v2_config(model_cfg.hf.model_size) if d.config_source is None
                else _load_config(DebertaV2Config, d.config_source, "discriminator HF", d.config_origin))
        if d.config_source is None:  # optional shape overrides of a from-scratch model (model.hf.scratch.*)
            sc = model_cfg.hf.scratch
            for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "position_buckets"):
                if getattr(sc, key) is not None:
                    setattr(disc, key, int(getattr(sc, key)))
            if sc.hidden_size is not None:
                disc.pooler_hidden_size = int(sc.hidden_size)
        g = src.generator
        if g.config_source is None:
            gen = _derive_generator_config(disc, model_cfg)
            # released DeBERTa-v3 xsmall generators run the last layer twice
            gen.z_steps = 2 if str(model_cfg.hf.model_size).strip().lower() == "xsmall" else 0
        else:
            gen = _load_config(DebertaV2Config, g.config_source, "generator HF", g.config_origin)
        _normalize_hf_config(disc, model_cfg=model_cfg, tokenizer=tokenizer, component="discriminator")
        _normalize_hf_config(gen, model_cfg=model_cfg, tokenizer=tokenizer, component="generator")
        _check_max_positions(disc, max_position_embeddings, "discriminator")
        _check_max_positions(gen, max_position_embeddings, "generator")
        return disc, gen
    r = model_cfg.rope
    d = src.discriminator
    disc = (DebertaRoPEConfig(hidden_size=r.hidden_size, num_hidden_layers=r.num_hidden_layers,
                              num_attention_heads=r.num_attention_heads, intermediate_size=r.intermediate_size,
                              hidden_act=r.hidden_act)
            if d.config_source is None else _load_config(DebertaRoPEConfig, d.config_source, "discriminator RoPE", d.config_origin))
    _normalize_rope_config(disc, model_cfg=model_cfg, tokenizer=tokenizer, max_position_embeddings=max_position_embeddings,
                           component="discriminator", explicit_source=d.config_source is not None, derived=False)
    g = src.generator
    gen = (_derive_generator_config(disc, model_cfg) if g.config_source is None
           else _load_config(DebertaRoPEConfig, g.config_source, "generator RoPE", g.config_origin))
    _normalize_rope_config(gen, model_cfg=model_cfg, tokenizer=tokenizer, max_position_embeddings=max_position_embeddings,
                           component="generator", explicit_source=g.config_source is not None,
                           derived=g.derived_from_discriminator)
    return disc, gen


def build_backbones(*, model_cfg: ModelConfig, disc_config: Any, gen_config: Any,
                    load_pretrained_weights: bool = True) -> tuple[Any, Any]:
    """Instantiate (discriminator, generator); pretrained weights only when asked and configured."""
    validate_model_config(model_cfg)
    cls = DebertaV2Model if (model_cfg.backbone_type or "hf_deberta_v2").lower() == "hf_deberta_v2" else DebertaRoPEModel
    if model_cfg.from_scratch or not load_pretrained_weights:
        return cls(disc_config), cls(gen_config)
    src = resolve_backbone_sources(model_cfg)
    out = []
    for comp, cfg in ((src.discriminator, disc_config), (src.generator, gen_config)):
        if comp.weight_source is None:
            raise RuntimeError("Resolved pretrained weight source is missing.")
        try:
            out.append(cls.from_pretrained(comp.weight_source, config=cfg))
        except Exception as e:
            raise RuntimeError(f"Failed to load {comp.component} backbone from source '{comp.weight_source}' "
                               f"(resolved from {comp.weight_origin}).") from e
    return out[0], out[1]
