"""Our hf_deberta_v2 backbone vs the reference modules on CPU in fp32 with copied weights."""

from __future__ import annotations

import pytest
import torch

from deberta_b200.models.deberta_v2 import DebertaV2Model
from deberta_b200.ops.attention import log_bucket_positions, relative_position_luts, relative_positions

from ._ref import import_reference, tiny_hf_config


def _pair(**over):
    import_reference()
    from deberta.modeling.deberta_v2_native import DebertaV2Model as RefModel

    torch.manual_seed(0)
    cfg = tiny_hf_config(**over)
    ref = RefModel(cfg).eval()
    ours = DebertaV2Model(cfg).eval()
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    return ref, ours


@pytest.mark.parametrize("mask_kind", ["none", "padding", "pairwise"])
def test_forward_matches_reference(mask_kind):
    ref, ours = _pair()
    ids = torch.randint(1, 512, (3, 40))
    mask = None
    if mask_kind == "padding":
        mask = torch.ones(3, 40, dtype=torch.long)
        mask[0, 30:] = 0
        mask[2, 5:] = 0
    elif mask_kind == "pairwise":
        doc = torch.ones(3, 40, dtype=torch.long)
        doc[:, 20:] = 2
        doc[1, 35:] = 0
        active = doc.ne(0)
        keep = doc[:, :, None].eq(doc[:, None, :]) & active[:, :, None] & active[:, None, :]
        keep[:, :, 0] |= ~active
        idx = torch.arange(40)
        keep[:, idx, idx] = active
        mask = keep
    a = ref(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    b = ours(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    assert len(a.hidden_states) == len(b.hidden_states)
    for x, y in zip(a.hidden_states, b.hidden_states):
        torch.testing.assert_close(y, x, atol=2e-5, rtol=1e-4)


def test_state_dict_names_match_reference():
    ref, ours = _pair()
    assert list(ref.state_dict().keys()) == list(ours.state_dict().keys())


def test_query_states_and_grads_match_reference():
    ref, ours = _pair()
    torch.manual_seed(1)
    h = torch.randn(2, 24, 64)
    qs = torch.randn(2, 24, 64)
    rel_r = ref.encoder.get_rel_embedding()
    rel_o = ours.encoder.get_rel_embedding()
    out_r, _ = ref.encoder.layer[-1](h, None, query_states=qs, relative_pos=ref.encoder.get_rel_pos(h), rel_embeddings=rel_r)
    out_o, _ = ours.encoder.layer[-1](h, None, query_states=qs, rel_embeddings=rel_o)
    torch.testing.assert_close(out_o, out_r, atol=2e-5, rtol=1e-4)
    out_r.square().sum().backward()
    out_o.square().sum().backward()
    gr = dict(ref.named_parameters())
    for name, p in ours.named_parameters():
        if p.grad is not None:
            torch.testing.assert_close(p.grad, gr[name].grad, atol=5e-4, rtol=1e-3)


def test_z_steps_and_p2p_match_reference():
    ref, ours = _pair(z_steps=2, pos_att_type=["p2c", "c2p", "p2p"])
    ids = torch.randint(1, 512, (2, 20))
    torch.testing.assert_close(
        ours(input_ids=ids).last_hidden_state, ref(input_ids=ids).last_hidden_state, atol=2e-5, rtol=1e-4
    )


def test_log_buckets_match_reference():
    import_reference()
    from deberta.modeling.deberta_v2_native import build_relative_position

    for q, k, b, p in [(512, 512, 256, 512), (40, 40, 32, 64), (700, 700, 256, 512), (16, 24, 0, 0)]:
        want = build_relative_position(q, k, bucket_size=b, max_position=p, device=torch.device("cpu"))
        got = relative_positions(q, k, b, p)
        assert torch.equal(want, got)
    c2p, p2c = relative_position_luts(512, 512, 256, 512, 256)
    rel = build_relative_position(512, 512, bucket_size=256, max_position=512, device=torch.device("cpu")).clamp(-256, 256)
    qi, ki = torch.meshgrid(torch.arange(512), torch.arange(512), indexing="ij")
    assert torch.equal(c2p[qi - ki + 511].long(), (rel + 256).clamp(0, 511))
    assert torch.equal(p2c[qi - ki + 511].long(), (256 - rel).clamp(0, 511))
    assert log_bucket_positions(torch.tensor([-10000, 10000]), 256, 512).abs().max() <= 255
