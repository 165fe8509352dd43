"""Packer / collator contracts, checked against the reference implementation where it is installed."""

from __future__ import annotations

import pytest
import torch

from deberta_b200.data import (DebertaV3ElectraCollator, MLMConfig, PackedStreamingConfig, PackedStreamingDataset,
                               SequentialStreamingDataset)
from deberta_b200.data.synthetic import SyntheticTextDataset, SyntheticTokenizer

from ._ref import import_reference


def _ds(n=300, mean=20):
    return SyntheticTextDataset(vocab_size=1000, mean_doc_len=mean, num_docs=n, seed=3)


def test_packer_matches_reference_blocks():
    import_reference()
    from deberta.data.streaming import PackedStreamingConfig as RC, PackedStreamingDataset as RP, SequentialStreamingDataset as RS

    tok = SyntheticTokenizer(1000)
    for ours_cls, ref_cls in ((PackedStreamingDataset, RP), (SequentialStreamingDataset, RS)):
        ours = list(ours_cls(hf_dataset=_ds(), tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=32, seed=1)))
        ref = list(ref_cls(hf_dataset=_ds(), tokenizer=tok, cfg=RC(text_column_name="text", max_seq_length=32, seed=1, shuffle_buffer_size=10000)))
        assert ours == ref and len(ours) > 10


def test_packer_structure_and_sharding():
    tok = SyntheticTokenizer(1000)
    rows = list(PackedStreamingDataset(hf_dataset=_ds(), tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=32)))
    for r in rows:
        assert len(r["input_ids"]) == 32 and r["input_ids"][0] == 1 and r["input_ids"][1] != 2
        assert r["special_tokens_mask"][0] == 1
        assert [int(t < 5) for t in r["input_ids"]] == r["special_tokens_mask"]
        assert ("attention_mask" in r) == (0 in r["input_ids"])
    assert "attention_mask" in rows[-1]
    a = list(PackedStreamingDataset(hf_dataset=_ds(), tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=32),
                                    process_index=0, num_processes=2))
    b = list(PackedStreamingDataset(hf_dataset=_ds(), tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=32),
                                    process_index=1, num_processes=2))
    assert a and b and a[0]["input_ids"] != b[0]["input_ids"]


@pytest.mark.parametrize("ngram", [1, 3])
@pytest.mark.parametrize("probs", [(1.0, 0.0), (0.8, 0.1)])
def test_collator_matches_reference(ngram, probs):
    import_reference()
    from deberta.data.collator import DebertaV3ElectraCollator as RCol, MLMConfig as RCfg

    tok = SyntheticTokenizer(1000)
    rows = list(PackedStreamingDataset(hf_dataset=_ds(), tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=64)))[:8]
    kw = dict(mlm_probability=0.15, mask_token_prob=probs[0], random_token_prob=probs[1], max_ngram=ngram)
    ours = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(**kw), packed_sequences=True)
    ref = RCol(tokenizer=tok, cfg=RCfg(**kw), packed_sequences=True)
    torch.manual_seed(9)
    a = ours([dict(r) for r in rows])
    torch.manual_seed(9)
    b = ref([dict(r) for r in rows])
    assert set(a) == set(b)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_collator_budget_and_doc_ids():
    tok = SyntheticTokenizer(1000)
    rows = list(PackedStreamingDataset(hf_dataset=_ds(2000, 60), tokenizer=tok, cfg=PackedStreamingConfig(max_seq_length=512)))[:4]
    col = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(mask_token_prob=1.0, random_token_prob=0.0),
                                   packed_sequences=True, block_cross_document_attention=True)
    out = col(rows)
    masked = out["labels"].ne(-100)
    assert masked.sum(1).tolist() == [77] * 4  # min(ceil(512*.15/10)*10, round(512*.15))
    assert bool((out["input_ids"][masked] == tok.mask_token_id).all())
    assert not bool((out["labels"][masked] < 5).any())
    doc = out["doc_ids"]
    assert doc.shape == (4, 512) and int(doc[:, 0].min()) == 1 and int(doc.max()) > 2
    assert bool((doc[:, 1:] >= doc[:, :-1]).all())
    nodoc = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(), packed_sequences=True,
                                     block_cross_document_attention=False)(rows)
    assert "doc_ids" not in nodoc and "attention_mask" not in nodoc
