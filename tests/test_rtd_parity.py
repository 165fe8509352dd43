"""RTD pretrainer vs the reference on CPU fp32 with copied weights and mirrored RNG."""

from __future__ import annotations

import copy

import pytest
import torch

from deberta_b200.models.deberta_v2 import DebertaV2Model
from deberta_b200.models.rope_encoder import DebertaRoPEConfig, DebertaRoPEModel
from deberta_b200.models.rtd import DebertaV3RTDPretrainer

from ._ref import import_reference, tiny_hf_config


def _build(backbone: str, sharing: str):
    import_reference()
    from deberta.modeling.rtd import DebertaV3RTDPretrainer as RefRTD

    torch.manual_seed(0)
    if backbone == "hf":
        from deberta.modeling.deberta_v2_native import DebertaV2Model as RefBackbone

        dcfg = tiny_hf_config(cls_token_id=1, sep_token_id=2, mask_token_id=3)
        gcfg = copy.deepcopy(dcfg)
        gcfg.num_hidden_layers = 1
        Ours = DebertaV2Model
    else:
        from deberta.modeling.rope_encoder import DebertaRoPEConfig as RC, DebertaRoPEModel as RefBackbone

        kw = dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=2, intermediate_size=128,
                  attention_implementation="eager", use_rmsnorm_heads=True)
        dcfg, gcfg = RC(**kw), RC(**{**kw, "num_hidden_layers": 1})
        Ours = DebertaRoPEModel
    ref = RefRTD(discriminator_backbone=RefBackbone(dcfg), generator_backbone=RefBackbone(gcfg), disc_config=dcfg,
                 gen_config=gcfg, embedding_sharing=sharing, additional_forbidden_token_ids=[0, 1, 2, 3])
    if backbone == "rope":
        dcfg, gcfg = DebertaRoPEConfig(**dcfg.to_dict()), DebertaRoPEConfig(**gcfg.to_dict())
    ours = DebertaV3RTDPretrainer(discriminator_backbone=Ours(dcfg), generator_backbone=Ours(gcfg), disc_config=dcfg,
                                  gen_config=gcfg, embedding_sharing=sharing,
                                  additional_forbidden_token_ids=[0, 1, 2, 3])
    assert list(ref.state_dict()) == list(ours.state_dict())
    ours.load_state_dict(ref.state_dict(), strict=True)
    return ref, ours


def _batch(pad=False):
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(4, 512, (3, 32), generator=g)
    labels = torch.full_like(ids, -100)
    pick = torch.rand(3, 32, generator=g) < 0.2
    labels[pick] = ids[pick]
    ids = ids.masked_fill(pick, 3)
    mask = None
    if pad:
        mask = torch.ones_like(ids)
        mask[1, 25:] = 0
        ids[1, 25:] = 0
        labels[1, 25:] = -100
    return ids, labels, mask


@pytest.mark.parametrize("backbone", ["hf", "rope"])
@pytest.mark.parametrize("sharing", ["gdes", "es", "none"])
@pytest.mark.parametrize("pad", [False, True])
def test_combined_forward_and_grads_match(backbone, sharing, pad):
    ref, ours = _build(backbone, sharing)
    ids, labels, mask = _batch(pad)
    torch.manual_seed(11)
    a = ref(input_ids=ids, attention_mask=mask, labels=labels)
    torch.manual_seed(11)
    b = ours(input_ids=ids, attention_mask=mask, labels=labels)
    for f in ("loss", "gen_loss", "disc_loss", "disc_accuracy", "gen_token_count", "disc_token_count",
              "disc_positive_count"):
        torch.testing.assert_close(getattr(b, f), getattr(a, f), atol=2e-5, rtol=1e-4)
    a.loss.backward()
    b.loss.backward()
    rg = dict(ref.named_parameters())
    for n, p in ours.named_parameters():
        if rg[n].grad is None:
            assert p.grad is None or p.grad.abs().max() == 0
        else:
            torch.testing.assert_close(p.grad, rg[n].grad, atol=1e-4, rtol=2e-3)


def test_phase_api_and_gdes_sync():
    ref, ours = _build("hf", "gdes")
    ids, labels, _ = _batch()
    torch.manual_seed(3)
    ga = ref(input_ids=ids, labels=labels, phase="generator")
    torch.manual_seed(3)
    gb = ours(input_ids=ids, labels=labels, phase="generator")
    assert torch.equal(ga.corrupted_input_ids, gb.corrupted_input_ids)
    assert torch.equal(ga.disc_labels, gb.disc_labels)
    da = ref(input_ids=ids, corrupted_input_ids=ga.corrupted_input_ids, disc_labels=ga.disc_labels, phase="discriminator")
    db = ours(input_ids=ids, corrupted_input_ids=gb.corrupted_input_ids, disc_labels=gb.disc_labels, phase="discriminator")
    torch.testing.assert_close(db.disc_loss_raw, da.disc_loss_raw, atol=1e-5, rtol=1e-4)
    with torch.no_grad():
        ours.generator.embeddings.word_embeddings.weight.add_(1.0)
    ours.sync_discriminator_embeddings_from_generator()
    assert torch.equal(ours.discriminator.embeddings.word_embeddings.base_weight,
                       ours.generator.embeddings.word_embeddings.weight)
    assert not ours.discriminator.embeddings.word_embeddings.base_weight.requires_grad


def test_no_masked_targets_and_forbidden_ids():
    _, ours = _build("hf", "gdes")
    ids, labels, _ = _batch()
    out = ours(input_ids=ids, labels=torch.full_like(labels, -100))
    assert float(out.loss) == 0.0 and float(out.disc_token_count) == 0.0
    g = ours(input_ids=ids, labels=labels, phase="generator", sampling_temperature=5.0)
    sampled = g.corrupted_input_ids[labels.ne(-100)]
    assert not torch.isin(sampled, torch.tensor([0, 1, 2, 3])).any()
