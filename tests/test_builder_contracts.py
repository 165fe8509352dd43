"""Backbone source resolution, presets, generator derivation and the tokenizer ↔ config contract.

The reference covers the same matrix in ``tests/test_builder.py`` (config/weight source matrix, presets,
vocabulary growth, special-id contract, ``z_steps``).
"""

from __future__ import annotations

import pytest
import torch

from deberta_b200.config import ModelConfig
from deberta_b200.data.synthetic import SyntheticTokenizer
from deberta_b200.models import builder as B
from deberta_b200.models.deberta_v2 import DebertaV2Config, DebertaV2Model
from deberta_b200.models.rope_encoder import DebertaRoPEConfig, DebertaRoPEModel


def _rope_cfg(**kw):
    base = dict(backbone_type="rope", hidden_size=64, num_hidden_layers=6, num_attention_heads=4, intermediate_size=128)
    base.update(kw)
    return ModelConfig(**base)


# ---------------------------------------------------------------------------------------------- sources
def test_sources_scratch_hf_uses_repo_defaults_and_no_weights():
    s = B.resolve_backbone_sources(ModelConfig())
    assert (s.discriminator.config_source, s.discriminator.config_origin) == (None, "repo_hf_defaults")
    assert s.discriminator.weight_source is None and s.discriminator.weight_origin == "scratch"
    assert s.generator.derived_from_discriminator and s.generator.config_origin == "derived_from_discriminator_config"
    assert s.generator.weight_source is None and s.generator.weight_origin == "scratch"


def test_sources_scratch_rope_is_synthetic_from_model_cfg():
    s = B.resolve_backbone_sources(_rope_cfg())
    assert s.discriminator.config_origin == "synthetic_from_model_cfg" and s.discriminator.config_source is None


def test_sources_pretrained_with_and_without_generator_path():
    cfg = ModelConfig(from_scratch=False, pretrained_discriminator_path="org/disc")
    s = B.resolve_backbone_sources(cfg)
    assert s.discriminator.config_source == s.discriminator.weight_source == "org/disc"
    assert s.generator.config_source is None and s.generator.weight_source == "org/disc"
    assert s.generator.weight_origin == "derived_from_pretrained_discriminator_path"
    cfg = ModelConfig(from_scratch=False, pretrained_discriminator_path="org/disc", pretrained_generator_path="org/gen")
    s = B.resolve_backbone_sources(cfg)
    assert s.generator.config_source == s.generator.weight_source == "org/gen"
    assert not s.generator.derived_from_discriminator and s.generator.weight_origin == "pretrained_generator_path"


def test_sources_scratch_generator_path_gives_config_only():
    s = B.resolve_backbone_sources(_rope_cfg(pretrained_generator_path="some/gen"))
    assert s.generator.config_source == "some/gen" and s.generator.weight_source is None


# ---------------------------------------------------------------------------------------------- presets
@pytest.mark.parametrize("size,dims", [("xsmall", (384, 12, 6, 1536)), ("small", (768, 6, 12, 3072)),
                                       ("base", (768, 12, 12, 3072)), ("large", (1024, 24, 16, 4096))])
def test_hf_presets_have_the_published_shapes(size, dims):
    c = B.build_repo_hf_deberta_v2_config(size)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.intermediate_size) == dims
    assert c.vocab_size == 128_100 and c.position_buckets == 256 and c.max_relative_positions == -1
    assert c.share_att_key and c.relative_attention and not c.position_biased_input
    assert list(c.pos_att_type) == ["p2c", "c2p"] and c.norm_rel_ebd == "layer_norm"
    assert c.layer_norm_eps == 1e-7 and c.type_vocab_size == 0 and c.pooler_hidden_size == dims[0]


def test_hf_scratch_configs_take_vocab_and_special_ids_from_the_tokenizer():
    tok = SyntheticTokenizer(640)
    disc, gen = B.build_backbone_configs(model_cfg=ModelConfig(hf_model_size="small"), tokenizer=tok, max_position_embeddings=128)
    assert disc.vocab_size == gen.vocab_size == 640
    assert (disc.pad_token_id, disc.cls_token_id, disc.sep_token_id, disc.mask_token_id) == (0, 1, 2, 4)
    assert disc.num_hidden_layers == 6 and gen.num_hidden_layers == 3  # half depth
    assert gen.hidden_size == disc.hidden_size and gen.z_steps == 0
    assert not disc.use_rmsnorm_heads and disc.hf_attention_kernel == "dynamic"


def test_xsmall_generator_repeats_its_last_layer():
    _d, gen = B.build_backbone_configs(model_cfg=ModelConfig(hf_model_size="xsmall"), tokenizer=SyntheticTokenizer(640),
                                       max_position_embeddings=128)
    assert gen.z_steps == 2 and gen.num_hidden_layers == 6


def test_generator_overrides_and_head_divisibility():
    cfg = ModelConfig(hf_model_size="small", generator_num_hidden_layers=2, generator_hidden_size=256,
                      generator_intermediate_size=512, generator_num_attention_heads=4)
    _d, gen = B.build_backbone_configs(model_cfg=cfg, tokenizer=SyntheticTokenizer(640), max_position_embeddings=64)
    assert (gen.num_hidden_layers, gen.hidden_size, gen.intermediate_size, gen.num_attention_heads) == (2, 256, 512, 4)
    bad = ModelConfig(hf_model_size="small", generator_hidden_size=250, generator_num_attention_heads=4)
    with pytest.raises(ValueError, match="divisible"):
        B.build_backbone_configs(model_cfg=bad, tokenizer=SyntheticTokenizer(640), max_position_embeddings=64)


def test_rope_generator_defaults_to_a_third_of_the_depth():
    disc, gen = B.build_backbone_configs(model_cfg=_rope_cfg(), tokenizer=SyntheticTokenizer(640), max_position_embeddings=256)
    assert disc.num_hidden_layers == 6 and gen.num_hidden_layers == 2
    assert disc.max_position_embeddings == 256 and disc.use_rmsnorm_heads and gen.use_rmsnorm_heads
    assert disc.norm_eps == 1e-6 and disc.vocab_size == 640


def test_rope_swiglu_width_is_rescaled_to_keep_the_parameter_budget():
    assert B.scaled_swiglu_intermediate_size(3072) == 2048
    assert B.scaled_swiglu_intermediate_size(100) == 128
    disc, _ = B.build_backbone_configs(model_cfg=_rope_cfg(ffn_type="swiglu", intermediate_size=3072),
                                       tokenizer=SyntheticTokenizer(640), max_position_embeddings=64)
    assert disc.intermediate_size == 2048
    keep, _ = B.build_backbone_configs(model_cfg=_rope_cfg(ffn_type="swiglu", intermediate_size=3072,
                                                           swiglu_adjust_intermediate=False),
                                       tokenizer=SyntheticTokenizer(640), max_position_embeddings=64)
    assert keep.intermediate_size == 3072


def test_dropout_overrides_reach_both_components():
    cfg = ModelConfig(hf_model_size="small", hidden_dropout_prob=0.05, attention_probs_dropout_prob=0.02)
    disc, gen = B.build_backbone_configs(model_cfg=cfg, tokenizer=SyntheticTokenizer(640), max_position_embeddings=64)
    for c in (disc, gen):
        assert c.hidden_dropout_prob == 0.05 and c.attention_probs_dropout_prob == 0.02


def test_sequence_length_must_fit_max_positions():
    cfg = ModelConfig(hf_model_size="small", hf_max_position_embeddings=128)
    with pytest.raises(ValueError, match="max_position_embeddings=128 is smaller than required"):
        B.build_backbone_configs(model_cfg=cfg, tokenizer=SyntheticTokenizer(640), max_position_embeddings=256)
    with pytest.raises(ValueError, match="smaller than required"):
        B.build_backbone_configs(model_cfg=_rope_cfg(max_position_embeddings=64), tokenizer=SyntheticTokenizer(640),
                                 max_position_embeddings=128)


# ---------------------------------------------------------------------------------------------- vocabulary
def test_vocab_multiple_grows_the_tokenizer_with_inert_placeholders():
    tok = SyntheticTokenizer(1001)
    cfg = _rope_cfg(tokenizer_vocab_multiple=128, tokenizer_allow_vocab_resize=True)
    disc, gen = B.build_backbone_configs(model_cfg=cfg, tokenizer=tok, max_position_embeddings=64)
    assert len(tok) == 1024 and disc.vocab_size == gen.vocab_size == 1024
    assert tok._extra[0] == "<|deberta_extra_token_1001|>" and len(tok._extra) == 23


def test_vocab_growth_needs_permission_and_never_shrinks():
    with pytest.raises(ValueError, match="tokenizer_allow_vocab_resize=false"):
        B.build_backbone_configs(model_cfg=_rope_cfg(tokenizer_vocab_multiple=128), tokenizer=SyntheticTokenizer(1001),
                                 max_position_embeddings=64)
    with pytest.raises(ValueError, match="shrinking tokenizer vocab is not supported"):
        B.build_backbone_configs(model_cfg=_rope_cfg(tokenizer_vocab_target=500, tokenizer_allow_vocab_resize=True),
                                 tokenizer=SyntheticTokenizer(1001), max_position_embeddings=64)
    tok = SyntheticTokenizer(1001)
    B.build_backbone_configs(model_cfg=_rope_cfg(tokenizer_vocab_target=1100, tokenizer_allow_vocab_resize=True),
                             tokenizer=tok, max_position_embeddings=64)
    assert len(tok) == 1100


def test_growth_requires_add_tokens_and_checks_the_result():
    class Frozen(SyntheticTokenizer):
        add_tokens = None

    with pytest.raises(ValueError, match="does not support add_tokens"):
        B._grow_tokenizer(Frozen(10), 12, "discriminator", True)

    class Lying(SyntheticTokenizer):
        def add_tokens(self, tokens, special_tokens=False):
            return 0

    with pytest.raises(RuntimeError, match="Failed to grow"):
        B._grow_tokenizer(Lying(10), 12, "discriminator", True)

    class NoLen:
        pass

    with pytest.raises(ValueError, match="len\\(tokenizer\\)"):
        B._tok_len(NoLen())


def _pretrained_cfg(**kw):
    return ModelConfig(from_scratch=False, pretrained_discriminator_path="x", **kw)


def test_pretrained_contract_vocab_rules():
    cfg = DebertaV2Config(vocab_size=640, pad_token_id=0)
    B._align_tokenizer_contract(cfg, SyntheticTokenizer(640), component="discriminator", model_cfg=_pretrained_cfg())
    assert cfg.cls_token_id == 1 and cfg.mask_token_id == 4  # missing ids are filled from the tokenizer
    with pytest.raises(ValueError, match="vocab mismatch"):
        B._align_tokenizer_contract(DebertaV2Config(vocab_size=600), SyntheticTokenizer(640), component="discriminator",
                                    model_cfg=_pretrained_cfg())
    # a smaller tokenizer is padded up to the checkpoint's vocabulary when resizing is allowed
    tok = SyntheticTokenizer(630)
    B._align_tokenizer_contract(DebertaV2Config(vocab_size=640), tok, component="discriminator",
                                model_cfg=_pretrained_cfg(tokenizer_allow_vocab_resize=True))
    assert len(tok) == 640
    with pytest.raises(ValueError, match="vocab mismatch"):
        B._align_tokenizer_contract(DebertaV2Config(vocab_size=640), SyntheticTokenizer(630), component="discriminator",
                                    model_cfg=_pretrained_cfg())
    with pytest.raises(ValueError, match="exceeds checkpoint config"):
        B._align_tokenizer_contract(DebertaV2Config(vocab_size=640), SyntheticTokenizer(630), component="discriminator",
                                    model_cfg=_pretrained_cfg(tokenizer_allow_vocab_resize=True, tokenizer_vocab_target=700))
    with pytest.raises(ValueError, match="rounds discriminator tokenizer size"):
        B._align_tokenizer_contract(DebertaV2Config(vocab_size=640), SyntheticTokenizer(630), component="discriminator",
                                    model_cfg=_pretrained_cfg(tokenizer_allow_vocab_resize=True, tokenizer_vocab_multiple=512))


def test_pretrained_contract_special_ids_must_agree():
    cfg = DebertaV2Config(vocab_size=640, pad_token_id=0)
    cfg.mask_token_id = 9
    with pytest.raises(ValueError, match="special-token mismatch for discriminator.mask_token_id"):
        B._align_tokenizer_contract(cfg, SyntheticTokenizer(640), component="discriminator", model_cfg=_pretrained_cfg())
    cfg.mask_token_id = "four"
    with pytest.raises(ValueError, match="expected int-like token id"):
        B._align_tokenizer_contract(cfg, SyntheticTokenizer(640), component="discriminator", model_cfg=_pretrained_cfg())


def test_rope_pretrained_overrides_are_applied_only_in_pretrained_mode():
    cfg = DebertaRoPEConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                            vocab_size=640, max_position_embeddings=64)
    mc = ModelConfig(backbone_type="rope", from_scratch=False, pretrained_discriminator_path="x",
                     pretrained_max_position_embeddings=512, pretrained_rope_theta=50000.0, pretrained_ffn_type="swiglu")
    B._normalize_rope_config(cfg, model_cfg=mc, tokenizer=SyntheticTokenizer(640), max_position_embeddings=256,
                             component="discriminator", explicit_source=True, derived=False)
    assert cfg.max_position_embeddings == 512 and cfg.rope_theta == 50000.0 and cfg.ffn_type == "swiglu"
    assert cfg.hidden_size == 64  # architecture stays the checkpoint's


# ---------------------------------------------------------------------------------------------- instantiation
def test_build_backbones_scratch_families_and_failure_messages(tmp_path):
    tok = SyntheticTokenizer(320)
    mc = ModelConfig(hf_model_size="xsmall", generator_num_hidden_layers=1)
    d, g = B.build_backbone_configs(model_cfg=mc, tokenizer=tok, max_position_embeddings=32)
    d.num_hidden_layers = 1
    disc, gen = B.build_backbones(model_cfg=mc, disc_config=d, gen_config=g)
    assert isinstance(disc, DebertaV2Model) and isinstance(gen, DebertaV2Model)
    rc = _rope_cfg(num_hidden_layers=3)
    d, g = B.build_backbone_configs(model_cfg=rc, tokenizer=tok, max_position_embeddings=32)
    disc, gen = B.build_backbones(model_cfg=rc, disc_config=d, gen_config=g)
    assert isinstance(disc, DebertaRoPEModel) and len(gen.encoder.layers) == 1
    out = disc(input_ids=torch.randint(5, 320, (2, 16)))
    hidden = out[0] if isinstance(out, tuple) else getattr(out, "last_hidden_state", out)
    assert tuple(hidden.shape) == (2, 16, 64)
    missing = ModelConfig(backbone_type="rope", from_scratch=False, pretrained_discriminator_path=str(tmp_path / "absent"))
    with pytest.raises(RuntimeError, match="Failed to load discriminator"):
        B.build_backbones(model_cfg=missing, disc_config=d, gen_config=g)
    # without weight loading the same configuration instantiates randomly initialised models
    disc, _ = B.build_backbones(model_cfg=missing, disc_config=d, gen_config=g, load_pretrained_weights=False)
    assert isinstance(disc, DebertaRoPEModel)


def test_pretrained_round_trip_through_save_and_load(tmp_path):
    tok = SyntheticTokenizer(320)
    rc = _rope_cfg(num_hidden_layers=3)
    d, g = B.build_backbone_configs(model_cfg=rc, tokenizer=tok, max_position_embeddings=32)
    disc, _gen = B.build_backbones(model_cfg=rc, disc_config=d, gen_config=g)
    disc.save_pretrained(tmp_path / "disc")
    mc = ModelConfig(backbone_type="rope", from_scratch=False, pretrained_discriminator_path=str(tmp_path / "disc"))
    d2, g2 = B.build_backbone_configs(model_cfg=mc, tokenizer=tok, max_position_embeddings=32)
    assert d2.hidden_size == 64 and d2.num_hidden_layers == 3 and g2.num_hidden_layers == 1
    loaded = DebertaRoPEModel.from_pretrained(str(tmp_path / "disc"), config=d2)
    for (n1, p1), (n2, p2) in zip(disc.state_dict().items(), loaded.state_dict().items()):
        assert n1 == n2 and torch.equal(p1, p2)
    with pytest.raises(RuntimeError, match="Failed to load discriminator RoPE config"):
        B._load_config(DebertaRoPEConfig, str(tmp_path / "nothing"), "discriminator RoPE", "pretrained_discriminator_path")
