"""Behaviour of the RTD pretrainer and its heads on tiny CPU models (no reference install needed).

Reference counterparts: ``tests/test_smoke.py:979-1528`` (pretrainer forward smoke, sampler forbidden ids, enhanced mask
decoder behaviour, heads) and the gradient-isolation checks of ``tools/audit_contracts.py:786-1100``.
"""

from __future__ import annotations

import copy
import math

import pytest
import torch
import torch.nn.functional as F

from deberta_b200.models.mask_utils import AttnMask, normalize_keep_mask
from deberta_b200.models.rope_encoder import DebertaRoPEConfig, DebertaRoPEModel
from deberta_b200.models.rtd import (DebertaV3RTDPretrainer, MaskedLMHead, RTDHead, attention_mask_to_active_tokens)
from deberta_b200.ops.heads import gumbel_sample, mlm_loss_and_sample_reference, rtd_loss

VOCAB = 160


def _cfg(layers=2, **kw):
    base = dict(vocab_size=VOCAB, hidden_size=32, num_hidden_layers=layers, num_attention_heads=2, intermediate_size=64,
                attention_implementation="eager", use_rmsnorm_heads=True, pad_token_id=0, max_position_embeddings=64)
    base.update(kw)
    return DebertaRoPEConfig(**base)


def _model(sharing="gdes", **kw):
    torch.manual_seed(0)
    d, g = _cfg(2), _cfg(1)
    return DebertaV3RTDPretrainer(discriminator_backbone=DebertaRoPEModel(d), generator_backbone=DebertaRoPEModel(g),
                                  disc_config=d, gen_config=g, embedding_sharing=sharing,
                                  additional_forbidden_token_ids=[0, 1, 2, 3, 4], **kw)


def _batch(pad=False, seed=5):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(5, VOCAB, (3, 24), generator=g)
    labels = torch.full_like(ids, -100)
    pick = torch.rand(3, 24, generator=g) < 0.25
    pick[:, 0] = False
    labels[pick] = ids[pick]
    ids = ids.masked_fill(pick, 4)
    mask = None
    if pad:
        mask = torch.ones_like(ids)
        mask[1, 18:] = 0
        ids[1, 18:] = 0
        labels[1, 18:] = -100
    return ids, labels, mask


# ---------------------------------------------------------------------------------------------- masks
def test_keep_masks_must_be_bool_or_integer():
    assert normalize_keep_mask(torch.tensor([[1, 0]])).dtype == torch.bool
    assert normalize_keep_mask(torch.tensor([[True, False]])).tolist() == [[True, False]]
    with pytest.raises((TypeError, ValueError)):
        normalize_keep_mask(torch.tensor([[1.0, 0.0]]))


def test_active_tokens_from_every_mask_shape():
    ids = torch.tensor([[7, 8, 9, 0]])
    assert attention_mask_to_active_tokens(input_ids=ids, attention_mask=None, pad_token_id=None).tolist() == [[True] * 4]
    assert attention_mask_to_active_tokens(input_ids=ids, attention_mask=None, pad_token_id=0).tolist() == [[True, True, True, False]]
    assert attention_mask_to_active_tokens(input_ids=ids, attention_mask=torch.tensor([[1, 1, 0, 0]]), pad_token_id=0).tolist() == \
        [[True, True, False, False]]
    pair = torch.zeros(1, 4, 4, dtype=torch.bool)
    pair[0, :2, :2] = True
    pair[0, 2, 2] = True
    # pairwise masks: a token is active when it may attend to itself, and never when it is padding
    assert attention_mask_to_active_tokens(input_ids=ids, attention_mask=pair, pad_token_id=0).tolist() == [[True, True, True, False]]
    assert attention_mask_to_active_tokens(input_ids=ids, attention_mask=pair[:, None], pad_token_id=0).tolist() == \
        [[True, True, True, False]]
    with pytest.raises(ValueError, match="attention_mask must have shape"):
        attention_mask_to_active_tokens(input_ids=ids, attention_mask=torch.ones(4), pad_token_id=0)


def test_attn_mask_from_document_ids_is_pairwise():
    doc = torch.tensor([[1, 1, 2, 2, 0]])
    m = AttnMask.from_any(None, doc)
    assert m.is_pairwise and m.token_keep().tolist() == [[True, True, True, True, False]]
    plain = AttnMask.from_any(torch.tensor([[1, 1, 1, 0, 0]]))
    assert not plain.is_pairwise and plain.token_keep().tolist() == [[True, True, True, False, False]]


# ---------------------------------------------------------------------------------------------- heads
def test_rtd_loss_is_a_masked_mean_with_counts():
    logits = torch.tensor([[2.0, -1.0, 0.5, 3.0]])
    labels = torch.tensor([[1.0, 0.0, 0.0, 1.0]])
    active = torch.tensor([[True, True, True, False]])
    st = rtd_loss(logits, labels, active)
    want = F.binary_cross_entropy_with_logits(logits[0, :3], labels[0, :3])
    assert torch.allclose(st.loss, want) and float(st.token_count) == 3.0 and float(st.positive_count) == 1.0
    assert math.isclose(float(st.accuracy), 2 / 3, rel_tol=1e-6)
    empty = rtd_loss(logits, labels, torch.zeros_like(active))
    assert float(empty.loss) == 0.0 and float(empty.token_count) == 0.0  # no division by zero


def test_rtd_head_adds_cls_context_except_under_pairwise_masks():
    torch.manual_seed(1)
    head = RTDHead(_cfg())
    h = torch.randn(2, 6, 32)
    with_cls = head(h, attention_mask=torch.ones(2, 6, dtype=torch.long))
    other_cls = h.clone()
    other_cls[:, 0] += 1.0
    assert not torch.allclose(head(other_cls, attention_mask=None)[:, 1:], with_cls[:, 1:])  # CLS reaches every token
    pair = torch.ones(2, 6, 6, dtype=torch.bool)
    a, b = head(h, attention_mask=pair), head(other_cls, attention_mask=pair)
    assert torch.allclose(a[:, 1:], b[:, 1:])  # not under a pairwise mask
    assert head._use_global_cls_context(None) and head._use_global_cls_context(torch.ones(2, 6))
    assert not head._use_global_cls_context(pair) and not head._use_global_cls_context(pair[:, None])
    assert not head._use_global_cls_context(AttnMask.from_any(None, torch.ones(2, 6, dtype=torch.long)))


def test_rtd_head_loss_stats_equal_head_then_loss():
    torch.manual_seed(2)
    head = RTDHead(_cfg())
    h = torch.randn(2, 6, 32)
    labels = (torch.rand(2, 6) < 0.3).float()
    active = torch.ones(2, 6, dtype=torch.bool)
    active[1, 4:] = False
    a = head.loss_stats(h, None, labels, active)
    b = rtd_loss(head(h), labels, active)
    assert torch.allclose(a.loss, b.loss) and torch.equal(a.accuracy, b.accuracy) and torch.equal(a.token_count, b.token_count)


def test_lm_head_ties_to_the_word_embeddings_it_is_given():
    torch.manual_seed(3)
    head = MaskedLMHead(_cfg(), tie_word_embeddings=True)
    emb = torch.randn(VOCAB, 32)
    w, b = head.projection(emb)
    assert w is emb and b.shape == (VOCAB,)
    logits = head(torch.randn(5, 32), word_embedding_weight=emb)
    assert logits.shape == (5, VOCAB)
    with pytest.raises((ValueError, RuntimeError)):
        head.projection(None)  # a tied head has no table of its own
    untied = MaskedLMHead(_cfg(), tie_word_embeddings=False)
    w2, _ = untied.projection(None)
    assert w2.shape == (VOCAB, 32)


# ---------------------------------------------------------------------------------------------- sampling
def test_gumbel_sampling_never_returns_forbidden_ids_and_follows_the_logits():
    torch.manual_seed(4)
    logits = torch.zeros(4000, 6)
    logits[:, 2] = 3.0
    forbidden = torch.tensor([True, False, False, False, False, True])
    s = gumbel_sample(logits, temperature=1.0, forbidden_vocab_mask=forbidden)
    assert not bool(((s == 0) | (s == 5)).any())
    share = float((s == 2).float().mean())
    want = math.exp(3) / (math.exp(3) + 3)
    assert abs(share - want) < 0.03
    cold = gumbel_sample(logits, temperature=0.05, forbidden_vocab_mask=None)
    assert float((cold == 2).float().mean()) > 0.999  # low temperature → arg-max
    with pytest.raises(ValueError, match="temperature must be > 0"):
        gumbel_sample(logits, temperature=0.0, forbidden_vocab_mask=None)
    with pytest.raises(ValueError, match="must match logits vocabulary"):
        gumbel_sample(logits, temperature=1.0, forbidden_vocab_mask=torch.zeros(5, dtype=torch.bool))


def test_forbidden_mask_construction():
    mask = DebertaV3RTDPretrainer._build_forbidden_token_mask(vocab_size=6, forbidden_ids={0, 5, 99, -1})
    assert mask.tolist() == [True, False, False, False, False, True]  # out-of-range ids are ignored
    assert DebertaV3RTDPretrainer._build_forbidden_token_mask(vocab_size=0, forbidden_ids={1}).numel() == 0
    with pytest.raises(ValueError, match="excludes all vocabulary ids"):
        DebertaV3RTDPretrainer._build_forbidden_token_mask(vocab_size=2, forbidden_ids={0, 1})
    m = _model()
    assert {0, 1, 2, 3, 4} <= m._forbidden_sample_token_ids
    assert "_forbidden_sample_token_mask" not in m.state_dict()  # not part of checkpoints


def test_mlm_loss_reference_is_mean_cross_entropy_over_masked_rows():
    torch.manual_seed(5)
    x, w, b = torch.randn(7, 32), torch.randn(VOCAB, 32), torch.randn(VOCAB)
    labels = torch.randint(5, VOCAB, (7,))
    loss, sampled = mlm_loss_and_sample_reference(x, w, b, labels, None, 1.0)
    assert torch.allclose(loss, F.cross_entropy(x @ w.t() + b, labels)) and sampled.shape == (7,) and sampled.dtype == torch.int64


# ---------------------------------------------------------------------------------------------- pretrainer
@pytest.mark.parametrize("pad", [False, True])
def test_generator_phase_builds_corruption_and_labels(pad):
    m = _model()
    ids, labels, mask = _batch(pad)
    torch.manual_seed(11)
    out = m.forward_generator_phase(input_ids=ids, attention_mask=mask, labels=labels)
    masked = labels.ne(-100)
    assert out.has_masked_targets and float(out.gen_token_count) == float(masked.sum())
    assert torch.equal(out.corrupted_input_ids[~masked], ids[~masked])  # only masked positions change
    sampled = out.corrupted_input_ids[masked]
    assert bool((sampled >= 5).all())  # specials are never sampled
    # a position is labelled "replaced" exactly when the sample differs from the original token
    assert torch.equal(out.disc_labels[masked], sampled.ne(labels[masked]).float())
    assert float(out.disc_labels[~masked].sum()) == 0.0
    assert not out.corrupted_input_ids.requires_grad and not out.disc_labels.requires_grad
    assert out.gen_loss_raw.requires_grad and 0 < float(out.gen_loss_raw) < 2 * math.log(VOCAB)


def test_generator_phase_without_masked_targets_is_a_differentiable_zero():
    m = _model()
    ids, labels, _ = _batch()
    out = m.forward_generator_phase(input_ids=ids, attention_mask=None, labels=torch.full_like(labels, -100))
    assert not out.has_masked_targets and float(out.gen_loss_raw) == 0.0 and float(out.gen_token_count) == 0.0
    assert torch.equal(out.corrupted_input_ids, ids) and float(out.disc_labels.sum()) == 0.0
    out.gen_loss_raw.backward()  # keeps every rank's backward graph alive
    full = m(input_ids=ids, labels=torch.full_like(labels, -100))
    assert float(full.loss) == 0.0 and float(full.disc_token_count) == 0.0


def test_combined_forward_weights_the_two_losses_and_counts_active_tokens():
    m = _model()
    ids, labels, mask = _batch(pad=True)
    torch.manual_seed(12)
    out = m(input_ids=ids, attention_mask=mask, labels=labels, gen_loss_weight=2.0, disc_loss_weight=10.0)
    assert torch.allclose(out.loss, 2.0 * out.gen_loss_raw + 10.0 * out.disc_loss_raw)
    assert float(out.disc_token_count) == float(mask.sum()) and float(out.gen_token_count) == float(labels.ne(-100).sum())
    assert 0.0 <= float(out.disc_accuracy) <= 1.0 and float(out.disc_positive_count) <= float(out.gen_token_count)
    assert not out.gen_loss.requires_grad and not out.disc_loss.requires_grad


def test_phase_argument_validation():
    m = _model()
    ids, labels, _ = _batch()
    with pytest.raises(ValueError, match="labels must be provided"):
        m(input_ids=ids, phase="generator")
    with pytest.raises(ValueError, match="labels must be provided"):
        m(input_ids=ids)
    with pytest.raises(ValueError, match="corrupted_input_ids must be provided"):
        m(input_ids=ids, phase="discriminator")
    with pytest.raises(ValueError, match="disc_labels must be provided"):
        m(input_ids=ids, phase="discriminator", corrupted_input_ids=ids)
    with pytest.raises(ValueError, match="phase must be one of"):
        m(input_ids=ids, labels=labels, phase="sideways")


def test_discriminator_loss_does_not_reach_the_generator():
    """The sampled corruption is detached: the RTD loss trains the discriminator (and, with GDES, only its deltas)."""
    m = _model("gdes")
    ids, labels, _ = _batch()
    torch.manual_seed(13)
    g = m.forward_generator_phase(input_ids=ids, labels=labels)
    d = m.forward_discriminator_phase(input_ids=ids, corrupted_input_ids=g.corrupted_input_ids, disc_labels=g.disc_labels)
    d.disc_loss_raw.backward()
    gen_params = dict(m.generator.named_parameters())
    assert all(p.grad is None or float(p.grad.abs().sum()) == 0.0 for p in gen_params.values())
    assert all(p.grad is None for p in m.generator_lm_head.parameters())
    delta = m.discriminator.embeddings.word_embeddings.bias
    assert delta.grad is not None and float(delta.grad.abs().sum()) > 0.0
    m.zero_grad(set_to_none=True)
    g.gen_loss_raw.backward()
    assert all(p.grad is None for p in m.discriminator.parameters())  # and the MLM loss stays out of the discriminator
    assert float(gen_params["embeddings.word_embeddings.weight"].grad.abs().sum()) > 0.0


@pytest.mark.parametrize("sharing", ["none", "es", "gdes"])
def test_embedding_sharing_modes(sharing):
    m = _model(sharing)
    gen_w = m.generator.embeddings.word_embeddings.weight
    disc_emb = m.discriminator.embeddings.word_embeddings
    names = set(m.state_dict())
    if sharing == "none":
        assert disc_emb.weight is not gen_w and "discriminator.embeddings.word_embeddings.weight" in names
    elif sharing == "es":
        assert disc_emb.weight is gen_w  # one table, trained by both losses
    else:
        assert "discriminator.embeddings.word_embeddings.bias" in names
        assert "discriminator.embeddings.word_embeddings.weight" not in names
        assert float(disc_emb.bias.abs().sum()) == 0.0  # deltas start at zero
        assert torch.equal(disc_emb.weight, gen_w.detach() + disc_emb.bias)
        with torch.no_grad():
            gen_w.add_(1.0)
        assert not torch.equal(disc_emb.weight, gen_w.detach() + disc_emb.bias)  # a stale copy until the next sync
        m.sync_discriminator_embeddings_from_generator()
        assert torch.equal(disc_emb.weight, gen_w.detach() + disc_emb.bias)


def test_state_dict_round_trip_reproduces_outputs():
    a, b = _model("gdes"), _model("gdes")
    with torch.no_grad():
        for p in a.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    a.sync_discriminator_embeddings_from_generator()
    b.load_state_dict(copy.deepcopy(a.state_dict()), strict=True)
    b.sync_discriminator_embeddings_from_generator()
    ids, labels, mask = _batch(pad=True)
    outs = []
    for m in (a, b):
        torch.manual_seed(21)
        outs.append(m(input_ids=ids, attention_mask=mask, labels=labels))
    assert torch.equal(outs[0].loss, outs[1].loss) and torch.equal(outs[0].disc_accuracy, outs[1].disc_accuracy)


def _hf_model(**kw):
    from deberta_b200.models.deberta_v2 import DebertaV2Model

    from ._ref import tiny_hf_config

    torch.manual_seed(0)
    d = tiny_hf_config(vocab_size=VOCAB, cls_token_id=1, sep_token_id=2, mask_token_id=4)
    g = copy.deepcopy(d)
    g.num_hidden_layers = 1
    return DebertaV3RTDPretrainer(discriminator_backbone=DebertaV2Model(d), generator_backbone=DebertaV2Model(g), disc_config=d,
                                  gen_config=g, embedding_sharing="gdes", additional_forbidden_token_ids=[0, 1, 2, 3, 4], **kw)


def test_enhanced_mask_decoder_applies_to_position_free_inputs_only():
    on, off = _hf_model(use_enhanced_mask_decoder=True), _hf_model(use_enhanced_mask_decoder=False)
    off.load_state_dict(on.state_dict())
    assert on._uses_emd() and not off._uses_emd()
    assert not _model(use_enhanced_mask_decoder=True)._uses_emd()  # rotary backbones carry positions in attention itself
    ids, labels, _ = _batch()
    torch.manual_seed(31)
    a = on.forward_generator_phase(input_ids=ids, labels=labels)
    torch.manual_seed(31)
    b = off.forward_generator_phase(input_ids=ids, labels=labels)
    assert not torch.allclose(a.gen_loss_raw, b.gen_loss_raw)  # the decoder re-runs the last layer with position queries
    assert float(a.gen_token_count) == float(b.gen_token_count)
    on.generator.z_steps = 2  # a generator that already repeats its last layer does not get the decoder on top
    assert not on._uses_emd()


def test_sampling_temperature_reaches_the_sampler():
    m = _model()
    ids, labels, _ = _batch()
    agree = []
    for temp in (1e-5, 5.0):
        torch.manual_seed(41)
        out = m.forward_generator_phase(input_ids=ids, labels=labels, sampling_temperature=temp)
        torch.manual_seed(42)
        again = m.forward_generator_phase(input_ids=ids, labels=labels, sampling_temperature=temp)
        agree.append(float((out.corrupted_input_ids == again.corrupted_input_ids).float().mean()))
    assert agree[0] == 1.0 and agree[1] < 1.0  # near-greedy samples repeat, hot samples do not
