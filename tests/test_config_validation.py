"""Validators, profile defaults and cross-section rules of the config system.

Reference counterparts: the validator cases of ``tests/test_config_and_training_cli.py`` and
``tests/test_config_and_training_runtime.py`` (normalisers, option compatibility, profile defaults).
"""

from __future__ import annotations

import warnings

import pytest

from deberta_b200 import config as C


def _model(**kw):
    return C.ModelConfig(**kw)


def _rope(**kw):
    return C.ModelConfig(backbone_type="rope", **kw)


# ---------------------------------------------------------------------------------------------- model
@pytest.mark.parametrize("kw,msg", [
    (dict(tokenizer_name_or_path="  "), "tokenizer.name_or_path must be a non-empty"),
    (dict(from_scratch=False), "pretrained.discriminator_path must be set"),
    (dict(backbone_type="rope", max_position_embeddings=0), "rope.max_position_embeddings must be > 0"),
    (dict(backbone_type="rope", rotary_pct=0.0), "rotary_pct must be in \\(0, 1\\]"),
    (dict(backbone_type="rope", rotary_pct=1.5), "rotary_pct must be in \\(0, 1\\]"),
    (dict(tokenizer_vocab_multiple=0), "vocab_multiple must be >= 1"),
    (dict(tokenizer_vocab_target=0), "vocab_target must be > 0"),
    (dict(hf_max_position_embeddings=0), "hf.max_position_embeddings must be > 0"),
    (dict(from_scratch=False, pretrained_discriminator_path="x", hf_max_position_embeddings=1024), "only supported when model.from_scratch=true"),
    (dict(hidden_size=512), "only valid when model.backbone_type='rope'"),
    (dict(backbone_type="rope", pretrained_rope_theta=5.0), "apply only when model.from_scratch=false"),
    (dict(backbone_type="rope", from_scratch=False, pretrained_discriminator_path="microsoft/deberta-v3-base"),
     "requires DebertaRoPE checkpoints"),
    (dict(backbone_type="rope", from_scratch=False, pretrained_discriminator_path="x", hidden_size=512),
     "only affect scratch RoPE initialization"),
    (dict(backbone_type="rope", from_scratch=False, pretrained_discriminator_path="x", pretrained_max_position_embeddings=0),
     "pretrained.max_position_embeddings must be > 0"),
    (dict(backbone_type="rope", from_scratch=False, pretrained_discriminator_path="x", pretrained_rotary_pct=2.0),
     "pretrained.rotary_pct must be in"),
    (dict(backbone_type="rope", from_scratch=False, pretrained_discriminator_path="x", pretrained_norm_arch="sideways"),
     "pretrained.norm_arch must be one of"),
    (dict(pretrained_generator_path="g", generator_hidden_size=128), "must be unset"),
    (dict(from_scratch=False, pretrained_discriminator_path="x", generator_hidden_size=128), "cannot use model.generator shape overrides"),
    (dict(backbone_type="rope", num_hidden_layers=0), "rope.num_hidden_layers must be > 0"),
    (dict(backbone_type="rope", hidden_size=100, num_attention_heads=12), "divisible by model.rope.num_attention_heads"),
    (dict(backbone_type="transformer-xl"), "backbone_type"),
    (dict(embedding_sharing="everything"), "embedding_sharing"),
    (dict(backbone_type="rope", ffn_type="moe"), "ffn_type"),
])
def test_model_validator_rejects(kw, msg):
    with pytest.raises(ValueError, match=msg):
        C.validate_model_config(_model(**kw))


def test_model_validator_normalises_in_place():
    cfg = _model(backbone_type=" ROPE ", embedding_sharing="GDES", norm_arch="KEEL", ffn_type="SwiGLU",
                 tokenizer_name_or_path="  synthetic:100 ", pretrained_generator_path="   ")
    C.validate_model_config(cfg)
    assert (cfg.backbone_type, cfg.embedding_sharing, cfg.rope.norm_arch, cfg.rope.ffn_type) == ("rope", "gdes", "keel", "swiglu")
    assert cfg.tokenizer.name_or_path == "synthetic:100" and cfg.pretrained.generator_path is None
    pre = _rope(from_scratch=False, pretrained_discriminator_path="x", pretrained_ffn_type=" SWIGLU ")
    C.validate_model_config(pre)
    assert pre.rope.pretrained.ffn_type == "swiglu"


@pytest.mark.parametrize("kw,needle", [
    (dict(backbone_type="rope", hf_model_size="large"), "model.hf.model_size only applies"),
    (dict(backbone_type="rope", keel_alpha_init=0.5), "keel_alpha_init has no effect"),
    (dict(backbone_type="rope", keel_alpha_learnable=True), "keel_alpha_learnable has no effect"),
    (dict(backbone_type="rope", swiglu_adjust_intermediate=False), "swiglu_adjust_intermediate has no effect"),
])
def test_model_validator_warns_about_inert_options(kw, needle):
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        C.validate_model_config(_model(**kw))
    assert any(needle in str(w.message) for w in caught)


# ---------------------------------------------------------------------------------------------- data
def _data(**kw):
    base = dict(dataset_name="synthetic")
    base.update(kw)
    return C.DataConfig(**base)


@pytest.mark.parametrize("kw,msg", [
    (dict(dataset_name=None), "No dataset source configured"),
    (dict(dataset_name=None, load_from_disk="/d"), "streaming=true is not compatible"),
    (dict(load_from_disk="/d", streaming=False, shuffle_buffer_size=1), "cannot be combined with: data.source.dataset_name"),
    (dict(dataset_name=None, dataset_config_name="en", data_files="a.txt"), "dataset_config_name requires"),
    (dict(max_seq_length=4), "max_seq_length must be >= 8"),
    (dict(shuffle_buffer_size=-1), "shuffle_buffer_size must be >= 0"),
    (dict(streaming=False, shuffle_buffer_size=100), "must be 0 or 1 when data.source.streaming=false"),
    (dict(pack_sequences=False, block_cross_document_attention=True), "requires data.packing.enabled=true"),
])
def test_data_validator_rejects(kw, msg):
    with pytest.raises(ValueError, match=msg):
        C.validate_data_config(_data(**kw))


def test_data_validator_accepts_each_source_and_warns_on_long_blocked_sequences():
    C.validate_data_config(_data())
    C.validate_data_config(_data(dataset_name=None, data_files="a.txt"))
    C.validate_data_config(_data(dataset_name=None, load_from_disk="/d", streaming=False, shuffle_buffer_size=1))
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        C.validate_data_config(_data(max_seq_length=8192, block_cross_document_attention=True))
    assert any("pairwise masks" in str(w.message) for w in caught)


# ---------------------------------------------------------------------------------------------- train / optim / logging
@pytest.mark.parametrize("kw,msg", [
    (dict(max_steps=0), "train.max_steps must be >= 1"),
    (dict(per_device_train_batch_size=0), "per_device_train_batch_size must be >= 1"),
    (dict(gradient_accumulation_steps=0), "gradient_accumulation_steps must be >= 1"),
    (dict(mlm_probability=1.0), "mlm_probability must be in"),
    (dict(mask_token_prob=0.9, random_token_prob=0.2), "Invalid masking probabilities"),
    (dict(sampling_temperature=0.0), "sampling_temperature must be > 0"),
    (dict(mlm_max_ngram=0), "mlm_max_ngram must be >= 1"),
    (dict(overwrite_output_dir=True, resume_from_checkpoint="auto"), "cannot be combined"),
    (dict(mixed_precision="fp8"), "mixed_precision"),
    (dict(resume_data_strategy="teleport"), "resume_data_strategy"),
])
def test_train_validator_rejects(kw, msg):
    with pytest.raises(ValueError, match=msg):
        C.validate_train_config(C.TrainConfig(**kw))


def test_train_validator_normalises_and_warns():
    cfg = C.TrainConfig(mixed_precision="BF16", output_dir="  ", resume_from_checkpoint="  ", torch_compile_mode="max-autotune")
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        C.validate_train_config(cfg)
    assert cfg.mixed_precision == "bf16" and cfg.checkpoint.output_dir is None and cfg.checkpoint.resume_from_checkpoint is None
    assert any("train.compile.mode has no effect" in str(w.message) for w in caught)


@pytest.mark.parametrize("value,want", [("bf16", "bf16"), ("no", "no"), (False, "no"), ("none", "no"), (True, "bf16"), ("fp32", "no")])
def test_mixed_precision_spellings(value, want):
    try:
        assert C.normalize_mixed_precision(value) == want
    except ValueError:
        assert value in ("fp32", True, "none")  # spellings a build may choose not to accept; never silently mapped elsewhere


def test_bf16_request_fails_loudly_when_the_preflight_fails():
    assert C.resolve_effective_mixed_precision("bf16", bf16_sanity_check=lambda: True) == "bf16"
    with pytest.raises(RuntimeError, match="bf16 preflight failed"):
        C.resolve_effective_mixed_precision("bf16", bf16_sanity_check=lambda: False)  # never a silent fp32 fallback
    assert C.resolve_effective_mixed_precision("no", bf16_sanity_check=lambda: pytest.fail("not consulted")) == "no"


@pytest.mark.parametrize("kw,msg", [
    (dict(learning_rate=0.0), "optim.lr.base must be > 0"),
    (dict(generator_learning_rate=0.0), "optim.lr.generator must be -1"),
    (dict(weight_decay=-0.1), "weight_decay must be >= 0"),
    (dict(max_grad_norm=-1.0), "max_grad_norm must be >= 0"),
    (dict(warmup_steps=-1), "warmup_steps must be >= 0"),
    (dict(lr_scheduler_type="zigzag"), "scheduler.type"),
])
def test_optim_validator_rejects(kw, msg):
    try:
        cfg = C.OptimConfig(**kw)
    except TypeError:
        pytest.skip("flat spelling not offered for this field")
    with pytest.raises(ValueError, match=msg):
        C.validate_optim_config(cfg)


def test_logging_validator():
    with pytest.raises(ValueError, match="project_name must be non-empty"):
        C.validate_logging_config(C.LoggingConfig(project_name=" "))
    with pytest.raises(ValueError, match="logging_steps must be >= 0"):
        C.validate_logging_config(C.LoggingConfig(logging_steps=-1))
    cfg = C.LoggingConfig(output_dir="  ")
    C.validate_logging_config(cfg)
    assert cfg.output_dir is None


# ---------------------------------------------------------------------------------------------- cross-section rules
def test_workflow_rules():
    blocked = _data(block_cross_document_attention=True)
    with pytest.raises(ValueError, match="sdpa_kernel=flash is not supported"):
        C.validate_training_workflow_options(data_cfg=blocked, train_cfg=C.TrainConfig(sdpa_kernel="flash"))
    with pytest.raises(ValueError, match="only supported with model.backbone_type='rope'"):
        C.validate_training_workflow_options(data_cfg=blocked, train_cfg=C.TrainConfig(), model_cfg=_model())
    C.validate_training_workflow_options(data_cfg=blocked, train_cfg=C.TrainConfig(), model_cfg=_rope())
    with pytest.raises(ValueError, match="only affects rope attention"):
        C.validate_training_workflow_options(data_cfg=_data(), train_cfg=C.TrainConfig(sdpa_kernel="math"),
                                             model_cfg=_rope(attention_implementation="eager"))
    with pytest.raises(ValueError, match="decoupled_training is incompatible with model.embedding_sharing='es'"):
        C.validate_training_workflow_options(data_cfg=_data(), train_cfg=C.TrainConfig(decoupled_training=True),
                                             model_cfg=_model(embedding_sharing="es"))
    with pytest.raises(ValueError, match="differs from optim.lr.base"):
        C.validate_training_workflow_options(data_cfg=_data(), train_cfg=C.TrainConfig(decoupled_training=False),
                                             model_cfg=_model(embedding_sharing="es"),
                                             optim_cfg=C.OptimConfig(learning_rate=1e-4, generator_learning_rate=5e-4))
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        C.validate_training_workflow_options(data_cfg=_data(), train_cfg=C.TrainConfig(sdpa_kernel="math"), model_cfg=_model())
    assert any("has no effect when model.backbone_type='hf_deberta_v2'" in str(w.message) for w in caught)


# ---------------------------------------------------------------------------------------------- profile defaults
def test_hf_backbone_defaults_follow_the_published_recipe_unless_set_explicitly():
    m, t, o = _model(), C.TrainConfig(), C.OptimConfig()
    C.apply_profile_defaults(model_cfg=m, train_cfg=t, optim_cfg=o)
    assert (t.objective.mask_token_prob, t.objective.random_token_prob, t.objective.disc_loss_weight) == (1.0, 0.0, 10.0)
    assert o.adam.epsilon == 1e-6 and o.scheduler.warmup_steps == 10_000 and t.token_weighted_gradient_accumulation is True
    # rope keeps the modern defaults
    m, t, o = _rope(), C.TrainConfig(), C.OptimConfig()
    C.apply_profile_defaults(model_cfg=m, train_cfg=t, optim_cfg=o)
    d = C.TrainConfig()
    assert t.objective.mask_token_prob == d.objective.mask_token_prob and t.objective.disc_loss_weight == d.objective.disc_loss_weight


def test_explicit_values_survive_profile_defaults(tmp_path):
    import yaml

    p = tmp_path / "c.yaml"
    p.write_text(yaml.safe_dump({"model": {"tokenizer": {"name_or_path": "synthetic:512"}},
                                 "data": {"source": {"dataset_name": "synthetic"}},
                                 "train": {"objective": {"disc_loss_weight": 50.0}},
                                 "optim": {"scheduler": {"warmup_steps": 7}}}))
    cfg = C.load_config(p)
    assert cfg.train.objective.disc_loss_weight == 50.0 and cfg.optim.scheduler.warmup_steps == 7
    assert cfg.train.objective.mask_token_prob == 1.0  # untouched fields still get the backbone default
    cfg = C.load_config(p, overrides=["train.objective.mask_token_prob=0.8"])
    assert cfg.train.objective.mask_token_prob == 0.8


def test_parity_profile_selects_the_hf_backbone():
    m, t = C.ModelConfig(profile="deberta_v3_parity"), C.TrainConfig()
    C.apply_profile_defaults(model_cfg=m, train_cfg=t)
    assert (m.backbone_type, m.embedding_sharing, m.hf.attention_kernel) == ("hf_deberta_v2", "gdes", "dynamic")


# ---------------------------------------------------------------------------------------------- choices / overrides
def test_choices_and_aliases():
    assert "rope" in C.choices_for("model.backbone_type") and C.choices_for("model.not_a_choice") is None
    assert C.normalize_choice("model.backbone_type", " Rope ") == "rope"
    with pytest.raises(ValueError, match="model.backbone_type"):
        C.normalize_choice("model.backbone_type", "lstm")


def test_dotted_override_errors():
    cfg = C.config_from_mapping({"data": {"source": {"dataset_name": "synthetic"}}})
    with pytest.raises(ValueError):
        C.apply_dotted_override(cfg, "train.no_such_field=1")
    with pytest.raises(ValueError):
        C.apply_dotted_override(cfg, "train.max_steps")  # no value
    with pytest.raises(ValueError):
        C.apply_dotted_override(cfg, "train.max_steps=many")
    out = C.apply_dotted_override(cfg, "train.checkpoint.output_dir=none")
    assert out.train.checkpoint.output_dir is None
    out = C.apply_dotted_override(cfg, "model.rope.keel_alpha_init=0.25")
    assert out.model.rope.keel_alpha_init == 0.25


def test_every_leaf_path_is_typed_and_unique():
    for cls in (C.ModelConfig, C.DataConfig, C.TrainConfig, C.OptimConfig, C.LoggingConfig):
        leaves = C.iter_leaf_paths_for_dataclass(cls)
        paths = [p for p, _ in leaves]
        assert len(paths) == len(set(paths)) and all(tp is not None for _, tp in leaves)
    assert "rope.pretrained.rope_theta" in [p for p, _ in C.iter_leaf_paths_for_dataclass(C.ModelConfig)]
