"""Access to the unmodified reference package (installed under ``baseline/_ref``) for parity tests."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

REF_DIR = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


def import_reference():
    """Import and return the reference ``deberta`` package, or skip the test if it is not installed."""
    if not (REF_DIR / "deberta").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import deberta  # noqa: F401

    return deberta


def tiny_hf_config(**over):
    from transformers import DebertaV2Config

    kw = dict(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=2, intermediate_size=128,
        relative_attention=True, position_buckets=32, max_relative_positions=64, pos_att_type=["p2c", "c2p"],
        share_att_key=True, norm_rel_ebd="layer_norm", position_biased_input=False, type_vocab_size=0,
        max_position_embeddings=128, layer_norm_eps=1e-7, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
        pad_token_id=0, hidden_act="gelu",
    )
    kw.update(over)
    return DebertaV2Config(**kw)
