"""Our rope backbone vs the reference modules on CPU in fp32 with copied weights."""

from __future__ import annotations

import pytest
import torch

from deberta_b200.models.rope_encoder import DebertaRoPEConfig, DebertaRoPEModel

from ._ref import import_reference


def _pair(**over):
    import_reference()
    from deberta.modeling.rope_encoder import DebertaRoPEConfig as RC, DebertaRoPEModel as RM

    kw = dict(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
              max_position_embeddings=64, attention_implementation="eager")
    kw.update(over)
    torch.manual_seed(0)
    ref = RM(RC(**kw)).eval()
    ours = DebertaRoPEModel(DebertaRoPEConfig(**kw)).eval()
    ours.load_state_dict(ref.state_dict(), strict=True)
    assert list(ref.state_dict()) == list(ours.state_dict())
    return ref, ours


@pytest.mark.parametrize("over", [
    dict(ffn_type="swiglu"), dict(ffn_type="mlp", use_bias=True), dict(norm_arch="keel", keel_alpha_learnable=True),
    dict(rotary_pct=0.5, use_absolute_position_embeddings=True), dict(attention_implementation="sdpa"),
])
@pytest.mark.parametrize("mask_kind", ["none", "padding", "pairwise"])
def test_rope_forward_matches_reference(over, mask_kind):
    ref, ours = _pair(**over)
    ids = torch.randint(1, 300, (2, 32))
    mask = None
    if mask_kind == "padding":
        mask = torch.ones(2, 32, dtype=torch.long)
        mask[1, 20:] = 0
    elif mask_kind == "pairwise":
        import_reference()
        from deberta.training.compile import _build_doc_block_mask

        doc = torch.ones(2, 32, dtype=torch.long)
        doc[:, 10:] = 2
        doc[1, 28:] = 0
        mask = _build_doc_block_mask(doc)
    a = ref(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    b = ours(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    for x, y in zip(a.hidden_states, b.hidden_states):
        torch.testing.assert_close(y, x, atol=3e-5, rtol=1e-4)


def test_doc_ids_equal_dense_block_mask():
    import_reference()
    from deberta.training.compile import _build_doc_block_mask

    from deberta_b200.models.mask_utils import AttnMask

    _, ours = _pair()
    ids = torch.randint(1, 300, (2, 32))
    doc = torch.ones(2, 32, dtype=torch.long)
    doc[:, 7:] = 2
    doc[:, 19:] = 3
    doc[0, 30:] = 0
    dense = ours(input_ids=ids, attention_mask=_build_doc_block_mask(doc)).last_hidden_state
    compact = ours(input_ids=ids, attention_mask=AttnMask(doc_ids=doc)).last_hidden_state
    torch.testing.assert_close(compact, dense, atol=1e-6, rtol=1e-6)
