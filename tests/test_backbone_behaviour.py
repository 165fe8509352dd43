"""Invariants of the two backbone families on tiny CPU models (no reference install needed).

Reference counterparts: the rope attention-mask edge cases of ``tests/test_smoke.py:731-943`` and the gradient-leak
checks of ``tools/audit_contracts.py`` (padding and document isolation shown through gradients).
"""

from __future__ import annotations

import math

import pytest
import torch

from deberta_b200.models.deberta_v2 import DebertaV2Model, normalize_pos_att_type
from deberta_b200.models.norm import RMSNorm
from deberta_b200.models.rope import RotaryEmbedding
from deberta_b200.models.rope_encoder import DebertaRoPEConfig, DebertaRoPEModel
from deberta_b200.ops.attention import (dense_keep_mask, log_bucket_positions, relative_position_luts, relative_positions,
                                        rotate_interleaved)

from ._ref import tiny_hf_config


def _rope(**kw):
    base = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=64,
                attention_implementation="eager", pad_token_id=0, max_position_embeddings=64)
    base.update(kw)
    torch.manual_seed(0)
    return DebertaRoPEModel(DebertaRoPEConfig(**base)).eval()


def _hf(**kw):
    torch.manual_seed(0)
    return DebertaV2Model(tiny_hf_config(vocab_size=128, **kw)).eval()


def _ids(b=2, s=12, seed=1):
    return torch.randint(5, 128, (b, s), generator=torch.Generator().manual_seed(seed))


def _hidden(out):
    return out.last_hidden_state if hasattr(out, "last_hidden_state") else out[0]


# ---------------------------------------------------------------------------------------------- relative positions
def test_log_buckets_are_odd_symmetric_monotone_and_exact_near_zero():
    rel = torch.arange(-511, 512)
    b = log_bucket_positions(rel, 256, 512)
    assert torch.equal(b, -b.flip(0))                       # bucket(-d) = -bucket(d)
    assert bool((b[1:] >= b[:-1]).all())                    # never decreasing in the distance
    near = rel.abs() <= 128
    assert torch.equal(b[near], rel[near])                  # distances up to half the bucket count are kept exactly
    assert int(b.max()) == 255 and int(b.min()) == -255     # the far end lands in the last bucket


def test_relative_position_matrix_and_lookup_tables_agree():
    S, buckets, maxpos, span = 40, 16, 64, 16
    rel = relative_positions(S, S, buckets, maxpos)
    assert rel.shape[-2:] == (S, S) and int(rel.reshape(S, S)[3, 3]) == 0
    r = rel.reshape(S, S)
    assert torch.equal(r, -r.t())
    c2p, p2c = relative_position_luts(S, S, buckets, maxpos, span)
    assert c2p.numel() == 2 * S - 1 and int(c2p.min()) >= 0 and int(c2p.max()) < 2 * span
    q, k = 7, 30
    assert int(c2p[q - k + S - 1]) == int((r[q, k] + span).clamp(0, 2 * span - 1))
    assert int(p2c[q - k + S - 1]) == int((-r[q, k] + span).clamp(0, 2 * span - 1))


def test_pos_att_type_normalisation():
    assert normalize_pos_att_type("p2c|c2p") == ["p2c", "c2p"]
    assert normalize_pos_att_type(["C2P", " p2c "]) == ["c2p", "p2c"]
    assert normalize_pos_att_type(None) == []


def test_dense_keep_mask_semantics():
    keep, live = dense_keep_mask(torch.tensor([[1, 1, 0]], dtype=torch.bool), None, None)
    assert keep.shape == (1, 1, 1, 3) and keep.flatten().tolist() == [True, True, False]  # padded keys are never attended
    assert live.flatten().tolist() == [True, True, False]
    keep, live = dense_keep_mask(None, torch.tensor([[1, 1, 2, 0]]), None)
    k = keep[0, 0]
    assert k[0].tolist() == [True, True, False, False] and k[2].tolist() == [False, False, True, False]
    assert k[3].tolist() == [True, False, False, False]  # a dead query keeps one edge so that its softmax row is defined
    assert live.flatten().tolist() == [True, True, True, False]
    assert dense_keep_mask(None, None, None) == (None, None)


# ---------------------------------------------------------------------------------------------- rotary / norm pieces
def test_rotary_is_a_rotation_and_depends_only_on_relative_offsets():
    rot = RotaryEmbedding(16)
    cos, sin = rot.get_cos_sin(32, device="cpu", dtype=torch.float32)
    x = torch.randn(1, 32, 2, 16)
    y = rotate_interleaved(x, cos[None, :, None], sin[None, :, None], 16) if cos.dim() == 2 else rotate_interleaved(x, cos, sin, 16)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)       # lengths are kept
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)                      # position 0 is the identity
    q = torch.randn(16)
    k = torch.randn(16)

    def dot(i, j):
        qq = torch.zeros(1, 32, 1, 16)
        kk = torch.zeros(1, 32, 1, 16)
        qq[0, i, 0], kk[0, j, 0] = q, k
        c, s = (cos[None, :, None], sin[None, :, None]) if cos.dim() == 2 else (cos, sin)
        return float((rotate_interleaved(qq, c, s, 16)[0, i, 0] * rotate_interleaved(kk, c, s, 16)[0, j, 0]).sum())

    assert math.isclose(dot(3, 9), dot(13, 19), rel_tol=1e-4, abs_tol=1e-5)  # same offset, same score
    assert not math.isclose(dot(3, 9), dot(3, 10), rel_tol=1e-3)


def test_partial_rotary_leaves_the_tail_dimensions_alone():
    rot = RotaryEmbedding(8, full_dim=16)
    cos, sin = rot.get_cos_sin(6, device="cpu", dtype=torch.float32)
    x = torch.randn(1, 6, 1, 16)
    c, s = (cos[None, :, None], sin[None, :, None]) if cos.dim() == 2 else (cos, sin)
    y = rotate_interleaved(x, c, s, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and not torch.allclose(y[:, 1:, :, :8], x[:, 1:, :, :8])


def test_rmsnorm_matches_its_definition_and_has_no_bias():
    n = RMSNorm(8, eps=1e-6)
    with torch.no_grad():
        n.weight.copy_(torch.arange(1.0, 9.0))
    x = torch.randn(3, 8)
    want = x / x.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt() * n.weight
    assert torch.allclose(n(x), want, atol=1e-6) and [k for k, _ in n.named_parameters()] == ["weight"]


# ---------------------------------------------------------------------------------------------- rope backbone
@pytest.mark.parametrize("kw", [dict(), dict(norm_arch="keel", keel_alpha_init=2.0), dict(ffn_type="swiglu"),
                                dict(rotary_pct=0.5), dict(use_bias=True), dict(use_absolute_position_embeddings=True)])
def test_rope_variants_run_and_respect_padding(kw):
    m = _rope(**kw)
    ids = _ids()
    mask = torch.ones_like(ids)
    mask[1, 8:] = 0
    a = _hidden(m(input_ids=ids, attention_mask=mask))
    other = ids.clone()
    other[1, 8:] = torch.randint(5, 128, (4,))
    b = _hidden(m(input_ids=other, attention_mask=mask))
    assert a.shape == (2, 12, 32) and torch.isfinite(a).all()
    assert torch.allclose(a[0], b[0], atol=1e-6) and torch.allclose(a[1, :8], b[1, :8], atol=1e-5)  # pads are invisible


def test_rope_architecture_switches_change_the_parameter_set():
    base, keel, swi, bias = (_rope(ffn_type="mlp"), _rope(ffn_type="mlp", norm_arch="keel", keel_alpha_learnable=True),
                             _rope(ffn_type="swiglu"), _rope(ffn_type="mlp", use_bias=True))
    names = lambda m: set(m.state_dict())  # noqa: E731
    assert any("alpha" in n for n in names(keel) - names(base))
    shapes = lambda m: {k: tuple(v.shape) for k, v in m.state_dict().items()}  # noqa: E731
    assert shapes(swi) != shapes(base)  # gate and up projections share one fused matrix
    assert any(n.endswith(".bias") for n in names(bias) - names(base))
    assert not any(n.endswith("dense.bias") or n.endswith("proj.bias") for n in names(base))


def test_rope_document_ids_isolate_documents_in_values_and_gradients():
    m = _rope()
    ids = _ids(1, 12)
    doc = torch.tensor([[1] * 5 + [2] * 7])
    emb = m.embeddings.word_embeddings.weight
    out = _hidden(m(input_ids=ids, doc_ids=doc)) if "doc_ids" in m.forward.__code__.co_varnames else None
    if out is None:
        from deberta_b200.models.mask_utils import AttnMask

        run = lambda x: _hidden(m(input_ids=x, attention_mask=AttnMask(doc_ids=doc)))  # noqa: E731
    else:
        run = lambda x: _hidden(m(input_ids=x, doc_ids=doc))  # noqa: E731
    a = run(ids)
    changed = ids.clone()
    changed[0, 7] = (changed[0, 7] + 1) % 123 + 5
    b = run(changed)
    assert torch.allclose(a[0, :5], b[0, :5], atol=1e-6) and not torch.allclose(a[0, 5:], b[0, 5:])
    m.zero_grad()
    run(ids)[0, :5].sum().backward()
    touched = emb.grad.abs().sum(-1).nonzero().flatten().tolist()
    assert set(touched) <= set(ids[0, :5].tolist())  # no gradient reaches tokens of the other document


def test_rope_hidden_states_and_checkpointing():
    m = _rope()
    ids = _ids()
    out = m(input_ids=ids, output_hidden_states=True, return_dict=True)
    assert len(out.hidden_states) == 3 and torch.equal(out.hidden_states[-1], out.last_hidden_state)
    m.train()
    ref = _hidden(m(input_ids=ids))
    ref.sum().backward()
    g_ref = m.encoder.layers[0].attn.qkv.weight.grad.clone()
    m.zero_grad()
    m.gradient_checkpointing_enable()
    chk = _hidden(m(input_ids=ids))
    chk.sum().backward()
    assert torch.allclose(ref, chk, atol=1e-6)
    assert torch.allclose(g_ref, m.encoder.layers[0].attn.qkv.weight.grad, atol=1e-6)
    m.gradient_checkpointing_disable()


@pytest.mark.parametrize("learnable", [False, True])
def test_rope_save_and_load_pretrained(tmp_path, learnable):
    m = _rope(ffn_type="swiglu", norm_arch="keel", keel_alpha_init=0.7, keel_alpha_learnable=learnable)
    if learnable:
        with torch.no_grad():
            m.encoder.layers[0].alpha1.alpha.fill_(0.3)  # a trained value must come back from the checkpoint
    m.save_pretrained(tmp_path)
    assert ("encoder.layers.0.alpha1.alpha" in m.state_dict()) == learnable  # a fixed alpha is not stored
    again = DebertaRoPEModel.from_pretrained(tmp_path).eval()
    assert again.config.ffn_type == "swiglu" and again.config.model_type == "deberta-rope"
    assert math.isclose(float(again.encoder.layers[0].alpha1.alpha), 0.3 if learnable else 0.7, rel_tol=1e-6)
    assert math.isclose(float(again.encoder.layers[1].alpha2.alpha), 0.7, rel_tol=1e-6)
    ids = _ids()
    assert torch.allclose(_hidden(m(input_ids=ids)), _hidden(again(input_ids=ids)), atol=1e-6)


def test_rope_rejects_sequences_beyond_max_positions_only_with_absolute_positions():
    m = _rope(max_position_embeddings=16)
    assert _hidden(m(input_ids=_ids(1, 24))).shape == (1, 24, 32)  # rotary positions extend on demand
    absolute = _rope(max_position_embeddings=16, use_absolute_position_embeddings=True)
    with pytest.raises((IndexError, ValueError, RuntimeError)):
        absolute(input_ids=_ids(1, 24))


# ---------------------------------------------------------------------------------------------- DeBERTa-v2 backbone
def test_hf_backbone_respects_padding_and_returns_all_layers():
    m = _hf()
    ids = _ids()
    mask = torch.ones_like(ids)
    mask[0, 9:] = 0
    out = m(input_ids=ids, attention_mask=mask, output_hidden_states=True, return_dict=True)
    assert len(out.hidden_states) == 3 and out.last_hidden_state.shape == (2, 12, 64)
    other = ids.clone()
    other[0, 9:] = 7
    again = m(input_ids=other, attention_mask=mask, return_dict=True).last_hidden_state
    assert torch.allclose(out.last_hidden_state[0, :9], again[0, :9], atol=1e-5)
    assert torch.allclose(out.last_hidden_state[1], again[1], atol=1e-6)


def test_hf_backbone_is_position_aware_only_through_relative_attention():
    m = _hf()
    ids = _ids(1, 10)
    base = _hidden(m(input_ids=ids))
    rolled = _hidden(m(input_ids=ids.roll(1, dims=1)))
    assert not torch.allclose(base.roll(1, dims=1), rolled, atol=1e-4)  # order matters …
    emb = m.embeddings(input_ids=ids)
    emb = emb[0] if isinstance(emb, tuple) else emb
    emb_rolled = m.embeddings(input_ids=ids.roll(1, dims=1))
    emb_rolled = emb_rolled[0] if isinstance(emb_rolled, tuple) else emb_rolled
    assert torch.allclose(emb.roll(1, dims=1), emb_rolled, atol=1e-6)   # … but the input embeddings carry no position


def test_hf_z_steps_repeat_the_last_layer():
    one, two = _hf(), _hf(z_steps=2)
    two.load_state_dict(one.state_dict())
    ids = _ids()
    a, b = _hidden(one(input_ids=ids)), _hidden(two(input_ids=ids))
    assert a.shape == b.shape and not torch.allclose(a, b)


def test_hf_state_dict_uses_the_published_parameter_names():
    names = set(_hf().state_dict())
    for want in ("embeddings.word_embeddings.weight", "embeddings.LayerNorm.weight", "encoder.rel_embeddings.weight",
                 "encoder.LayerNorm.weight", "encoder.layer.0.attention.self.query_proj.weight",
                 "encoder.layer.0.attention.output.dense.weight", "encoder.layer.1.intermediate.dense.bias",
                 "encoder.layer.1.output.LayerNorm.bias"):
        assert want in names, want
    assert "embeddings.position_embeddings.weight" in names  # kept (unused) when position_biased_input=false, as in released checkpoints


def test_hf_gradient_checkpointing_matches():
    m = _hf().train()
    ids = _ids()
    a = _hidden(m(input_ids=ids))
    m.gradient_checkpointing_enable()
    b = _hidden(m(input_ids=ids))
    b.sum().backward()
    assert torch.allclose(a, b, atol=1e-6) and m.embeddings.word_embeddings.weight.grad is not None


def test_hf_save_and_load_pretrained_restores_unsaved_buffers(tmp_path):
    m = _hf(position_biased_input=True)
    m.save_pretrained(tmp_path)
    again = DebertaV2Model.from_pretrained(tmp_path).eval()
    want = torch.arange(m.config.max_position_embeddings).unsqueeze(0)
    assert torch.equal(again.embeddings.position_ids, want)  # not stored in the checkpoint, rebuilt on load
    ids = _ids()
    assert torch.allclose(_hidden(m(input_ids=ids)), _hidden(again(input_ids=ids)), atol=1e-6)


def test_rope_load_pretrained_restores_the_rotary_table(tmp_path):
    m = _rope(ffn_type="mlp", rotary_pct=0.5)
    m.save_pretrained(tmp_path)
    assert not any("inv_freq" in k for k in m.state_dict())
    again = DebertaRoPEModel.from_pretrained(tmp_path).eval()
    assert torch.equal(again.encoder.layers[1].attn.rope.inv_freq, m.encoder.layers[1].attn.rope.inv_freq)
    ids = _ids()
    assert torch.allclose(_hidden(m(input_ids=ids)), _hidden(again(input_ids=ids)), atol=1e-6)
