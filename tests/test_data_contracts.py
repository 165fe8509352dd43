"""Behavioural contracts of the packer and the masking collator on hand-made inputs.

The reference pins the same behaviour in ``tests/test_smoke.py:39-705`` (packer edge cases, collator
document ids, masking policy, budgets and special-token handling); the cases below are written
against those contracts with their own fixtures.
"""

from __future__ import annotations

import math

import pytest
import torch

from deberta_b200.data import (DebertaV3ElectraCollator, MLMConfig, PackedStreamingConfig, PackedStreamingDataset,
                               SequentialStreamingDataset)
from deberta_b200.data.synthetic import SyntheticTextDataset, SyntheticTokenizer, load_tokenizer, parse_synthetic_spec

PAD, CLS, SEP, UNK, MASK = 0, 1, 2, 3, 4


class ListDataset:
    """Minimal stand-in for a streaming dataset: rows, ``shuffle`` and ``shard`` that record their arguments."""

    def __init__(self, rows, log=None):
        self.rows, self.log = list(rows), ([] if log is None else log)

    def shuffle(self, seed=0, buffer_size=None):
        self.log.append(("shuffle", seed, buffer_size))
        g = torch.Generator().manual_seed(int(seed))
        order = torch.randperm(len(self.rows), generator=g).tolist()
        return ListDataset([self.rows[i] for i in order], self.log)

    def shard(self, num_shards, index):
        self.log.append(("shard", num_shards, index))
        return ListDataset(self.rows[index::num_shards], self.log)

    def __iter__(self):
        return iter(self.rows)


def _words(lo, hi):
    return " ".join(f"t{i}" for i in range(lo, hi))


def _pack(rows, max_seq=10, cls=PackedStreamingDataset, **kw):
    cfg = PackedStreamingConfig(max_seq_length=max_seq, shuffle_buffer_size=0, **kw)
    return list(cls(hf_dataset=ListDataset(rows), tokenizer=SyntheticTokenizer(1000), cfg=cfg))


# ---------------------------------------------------------------------------------------------- packer
def test_packer_joins_documents_with_separators_and_wraps_blocks():
    rows = [{"text": _words(10, 13)}, {"text": _words(20, 23)}, {"text": _words(30, 34)}]
    out = _pack(rows, max_seq=10)
    assert out[0]["input_ids"] == [CLS, 10, 11, 12, SEP, 20, 21, 22, SEP, SEP]
    assert out[0]["special_tokens_mask"] == [1, 0, 0, 0, 1, 0, 0, 0, 1, 1]
    assert "attention_mask" not in out[0]
    # the remainder is flushed as a padded block with its mask
    assert out[1]["input_ids"] == [CLS, 30, 31, 32, 33, SEP, PAD, PAD, PAD, PAD]
    assert out[1]["attention_mask"] == [1] * 6 + [0] * 4
    assert out[1]["special_tokens_mask"] == [1, 0, 0, 0, 0, 1, 1, 1, 1, 1]


def test_packer_drops_leading_separators_of_a_block():
    # first doc fills the block exactly, so its separator would open the next block
    rows = [{"text": _words(10, 18)}, {"text": _words(20, 24)}]
    out = _pack(rows, max_seq=10)
    assert out[0]["input_ids"] == [CLS, *range(10, 18), SEP]
    assert out[1]["input_ids"][:2] == [CLS, 20]
    assert SEP not in out[1]["input_ids"][1:5]


def test_packer_skips_blank_documents_and_rejects_missing_column():
    out = _pack([{"text": "   "}, {"text": ""}, {"text": _words(10, 14)}], max_seq=8)
    assert len(out) == 1 and out[0]["input_ids"][:5] == [CLS, 10, 11, 12, 13]
    with pytest.raises(KeyError, match="Text column 'text' not found"):
        _pack([{"body": "t10 t11"}], max_seq=8)


def test_packer_accepts_list_valued_text_and_custom_column():
    out = _pack([{"body": ["t10 t11", "t12"]}], max_seq=8, text_column_name="body")
    assert out[0]["input_ids"][:5] == [CLS, 10, 11, 12, SEP]


def test_packer_rejects_tiny_sequence_length_and_incomplete_tokenizers():
    with pytest.raises(ValueError, match="too small"):
        _pack([{"text": "t10"}], max_seq=4)

    class NoSep(SyntheticTokenizer):
        sep_token_id = None

    with pytest.raises(ValueError, match="sep_token_id"):
        PackedStreamingDataset(hf_dataset=ListDataset([]), tokenizer=NoSep(100), cfg=PackedStreamingConfig())


def test_packer_empty_stream_yields_nothing():
    assert _pack([], max_seq=8) == []
    assert _pack([{"text": " "}], max_seq=8) == []


def test_packer_long_document_spans_blocks_without_losing_tokens():
    out = _pack([{"text": _words(10, 40)}], max_seq=10)
    body = [t for r in out for t in r["input_ids"] if t >= 5]
    assert body == list(range(10, 40))
    assert all(len(r["input_ids"]) == 10 for r in out)


def test_packer_shuffles_with_seed_plus_epoch_and_shards_by_rank():
    log = []
    ds = ListDataset([{"text": _words(10 + i, 12 + i)} for i in range(8)], log)
    cfg = PackedStreamingConfig(max_seq_length=8, seed=5, shuffle_buffer_size=64)
    p = PackedStreamingDataset(hf_dataset=ds, tokenizer=SyntheticTokenizer(1000), cfg=cfg, process_index=1, num_processes=4)
    first = list(p)
    assert ("shuffle", 5, 64) in log and ("shard", 4, 1) in log
    p.set_epoch(3)
    second = list(p)
    assert ("shuffle", 8, 64) in log
    assert first != second
    p.set_epoch(0)
    assert list(p) == first  # same epoch → same order


def test_packer_without_shuffle_buffer_keeps_source_order():
    log = []
    ds = ListDataset([{"text": _words(10, 12)}], log)
    list(PackedStreamingDataset(hf_dataset=ds, tokenizer=SyntheticTokenizer(1000),
                                cfg=PackedStreamingConfig(max_seq_length=8, shuffle_buffer_size=0)))
    assert not any(e[0] == "shuffle" for e in log)


def test_packer_set_epoch_clamps_negative_and_forwards_to_dataset():
    class Epochy(ListDataset):
        seen = None

        def set_epoch(self, e):
            Epochy.seen = e

    p = PackedStreamingDataset(hf_dataset=Epochy([]), tokenizer=SyntheticTokenizer(100), cfg=PackedStreamingConfig())
    p.set_epoch(-4)
    assert p._current_epoch() == 0 and Epochy.seen == 0
    p.set_epoch(7)
    assert p._current_epoch() == 7 and Epochy.seen == 7


def test_sequential_dataset_one_document_per_row_with_continuation():
    rows = [{"text": _words(10, 13)}, {"text": _words(20, 31)}]
    out = _pack(rows, max_seq=10, cls=SequentialStreamingDataset)
    assert out[0]["input_ids"] == [CLS, 10, 11, 12, SEP, PAD, PAD, PAD, PAD, PAD]
    assert out[1]["input_ids"] == [CLS, *range(20, 28), SEP]
    assert out[2]["input_ids"][:5] == [CLS, 28, 29, 30, SEP]
    assert all(r["input_ids"].count(SEP) == 1 for r in out)


def test_packer_works_under_a_dataloader_with_workers_sharding_by_worker():
    rows = [{"text": _words(10 + 3 * i, 13 + 3 * i)} for i in range(12)]
    ds = PackedStreamingDataset(hf_dataset=ListDataset(rows), tokenizer=SyntheticTokenizer(1000),
                                cfg=PackedStreamingConfig(max_seq_length=8, shuffle_buffer_size=0))
    single = [r["input_ids"] for r in ds]
    loader = torch.utils.data.DataLoader(ds, batch_size=None, num_workers=2)
    multi = [list(map(int, r["input_ids"])) for r in loader]
    flat = lambda rs: sorted(t for r in rs for t in r if t >= 5)  # noqa: E731
    assert flat(multi) == flat(single)  # every token delivered exactly once across the workers


# ---------------------------------------------------------------------------------------------- synthetic corpus
def test_synthetic_spec_parsing_and_tokenizer_loading():
    assert parse_synthetic_spec(None) == {} and parse_synthetic_spec("default") == {}
    spec = parse_synthetic_spec("zipf1.3-mean9-vocab321")
    assert spec["vocab_size"] == 321 and spec["mean_doc_len"] == 9 and abs(spec["zipf_s"] - 1.3) < 1e-9
    with pytest.raises(ValueError, match="Unrecognised synthetic dataset spec"):
        parse_synthetic_spec("bogus")
    tok = load_tokenizer("synthetic:777")
    assert isinstance(tok, SyntheticTokenizer) and len(tok) == 777
    assert tok("t10 t11", add_special_tokens=True)["input_ids"] == [CLS, 10, 11, SEP]
    assert 5 <= tok("zebra")["input_ids"][0] < 777  # arbitrary words hash into the ordinary range


def test_synthetic_dataset_is_deterministic_shardable_and_epoch_dependent():
    a = [r["text"] for r in SyntheticTextDataset(vocab_size=500, num_docs=40, seed=1)]
    b = [r["text"] for r in SyntheticTextDataset(vocab_size=500, num_docs=40, seed=1)]
    assert a == b and len(a) == 40
    s0 = [r["text"] for r in SyntheticTextDataset(vocab_size=500, num_docs=40, seed=1).shard(2, 0)]
    s1 = [r["text"] for r in SyntheticTextDataset(vocab_size=500, num_docs=40, seed=1).shard(2, 1)]
    assert len(s0) + len(s1) == 40 and set(s0).isdisjoint(s1) or len(set(s0) & set(s1)) < 3
    c = SyntheticTextDataset(vocab_size=500, num_docs=40, seed=2)
    assert [r["text"] for r in c] != a


def test_synthetic_tokenizer_pad_builds_masks_only_when_needed():
    tok = SyntheticTokenizer(100)
    same = tok.pad([{"input_ids": [1, 9, 2]}, {"input_ids": [1, 8, 2]}])
    assert "attention_mask" not in same
    ragged = tok.pad([{"input_ids": [1, 9, 2]}, {"input_ids": [1, 2]}])
    assert ragged["input_ids"].tolist() == [[1, 9, 2], [1, 2, 0]]
    assert ragged["attention_mask"].tolist() == [[1, 1, 1], [1, 1, 0]]


# ---------------------------------------------------------------------------------------------- collator
def _rows(n=4, seq=64):
    ds = SyntheticTextDataset(vocab_size=1000, mean_doc_len=12, num_docs=400, seed=11)
    cfg = PackedStreamingConfig(max_seq_length=seq, shuffle_buffer_size=0)
    return list(PackedStreamingDataset(hf_dataset=ds, tokenizer=SyntheticTokenizer(1000), cfg=cfg))[:n]


def _col(**kw):
    cfg_kw = {k: kw.pop(k) for k in list(kw) if k in ("mlm_probability", "mask_token_prob", "random_token_prob", "max_ngram")}
    return DebertaV3ElectraCollator(tokenizer=kw.pop("tokenizer", SyntheticTokenizer(1000)), cfg=MLMConfig(**cfg_kw), **kw)


@pytest.mark.parametrize("bad", [dict(mlm_probability=0.0), dict(mlm_probability=1.0), dict(max_ngram=0),
                                 dict(mask_token_prob=0.7, random_token_prob=0.4), dict(mask_token_prob=-0.1)])
def test_collator_rejects_invalid_masking_configuration(bad):
    with pytest.raises(ValueError):
        _col(**bad)


def test_collator_requires_a_mask_token():
    class NoMask(SyntheticTokenizer):
        mask_token_id = None

    with pytest.raises(ValueError, match="mask token"):
        _col(tokenizer=NoMask(100))


def test_collator_never_masks_special_or_padding_positions():
    rows = _rows(6, 64)
    rows[2] = {"input_ids": rows[2]["input_ids"][:20], "special_tokens_mask": rows[2]["special_tokens_mask"][:20]}
    torch.manual_seed(0)
    out = _col(packed_sequences=True)(rows)
    ids = torch.tensor([r["input_ids"] + [PAD] * (64 - len(r["input_ids"])) for r in rows])
    picked = out["labels"].ne(-100)
    assert not bool((ids[picked] < 5).any())
    assert torch.equal(out["labels"][picked], ids[picked])
    assert torch.equal(out["input_ids"][~picked], ids[~picked])  # unpicked positions are untouched
    assert out["attention_mask"][2].tolist() == [1] * 20 + [0] * 44


def test_collator_all_mask_policy_and_keep_policy():
    rows = _rows(4, 64)
    torch.manual_seed(1)
    out = _col(mask_token_prob=1.0, random_token_prob=0.0)(rows)
    picked = out["labels"].ne(-100)
    assert bool((out["input_ids"][picked] == MASK).all())
    torch.manual_seed(1)
    keep = _col(mask_token_prob=0.0, random_token_prob=0.0)(rows)
    kp = keep["labels"].ne(-100)
    assert torch.equal(keep["input_ids"][kp], keep["labels"][kp])  # selected but left as they were


def test_collator_random_replacements_are_never_special_tokens():
    rows = _rows(8, 64)
    torch.manual_seed(2)
    out = _col(mask_token_prob=0.0, random_token_prob=1.0)(rows)
    picked = out["labels"].ne(-100)
    assert int(picked.sum()) > 0
    assert bool((out["input_ids"][picked] >= 5).all())


@pytest.mark.parametrize("seq,prob", [(64, 0.15), (128, 0.15), (512, 0.15), (96, 0.3)])
def test_collator_budget_formula(seq, prob):
    col = _col(mlm_probability=prob)
    window, cap, n_pred = col._budget(seq)
    assert window == max(1, int(1.0 / prob))
    assert cap == math.ceil(seq * prob / 10) * 10
    assert n_pred == min(cap, max(1, round(seq * prob)))
    rows = _rows(3, seq)
    torch.manual_seed(3)
    out = col(rows)
    assert int(out["labels"].ne(-100).sum(1).max()) <= n_pred


def test_windowed_sampler_picks_one_candidate_per_window():
    cand = torch.arange(100, 135)
    torch.manual_seed(4)
    sel = DebertaV3ElectraCollator._sample_windowed_unigram_indices(cand, mask_window=6)
    assert sel.numel() == math.ceil(35 / 6)
    for w, s in enumerate(sel.tolist()):
        assert 100 + 6 * w <= s < min(135, 100 + 6 * (w + 1))
    assert DebertaV3ElectraCollator._sample_windowed_unigram_indices(cand[:0], mask_window=6).numel() == 0
    assert torch.equal(DebertaV3ElectraCollator._sample_windowed_unigram_indices(cand, mask_window=1), cand)


def test_collator_document_ids_follow_separators():
    row = {"input_ids": [CLS, 10, 11, SEP, 12, SEP, SEP, 13, 14, SEP, PAD, PAD],
           "special_tokens_mask": [1, 0, 0, 1, 0, 1, 1, 0, 0, 1, 1, 1], "attention_mask": [1] * 10 + [0] * 2}
    out = _col(packed_sequences=True, block_cross_document_attention=True)([row])
    # a separator belongs to the document it closes; a run of separators opens one document, not two; pads are 0
    assert out["doc_ids"].tolist() == [[1, 1, 1, 1, 2, 2, 3, 3, 3, 3, 0, 0]]
    assert out["attention_mask"].tolist() == [[1] * 10 + [0] * 2]


def test_collator_single_document_rows_get_no_document_ids():
    row = {"input_ids": [CLS, 10, 11, 12, 13, 14, 15, SEP], "special_tokens_mask": [1, 0, 0, 0, 0, 0, 0, 1]}
    out = _col(packed_sequences=True, block_cross_document_attention=True)([row, dict(row)])
    assert "doc_ids" not in out and "attention_mask" not in out


def test_collator_document_ids_only_for_packed_blocking_configurations():
    rows = _rows(2, 64)
    assert "doc_ids" in _col(packed_sequences=True, block_cross_document_attention=True)(rows)
    assert "doc_ids" not in _col(packed_sequences=True, block_cross_document_attention=False)(rows)
    assert "doc_ids" not in _col(packed_sequences=False, block_cross_document_attention=True)(rows)


def test_collator_drops_all_ones_attention_mask_but_keeps_real_padding():
    row = {"input_ids": [CLS, 10, 11, 12, 13, 14, 15, SEP], "special_tokens_mask": [1, 0, 0, 0, 0, 0, 0, 1],
           "attention_mask": [1] * 8}
    assert "attention_mask" not in _col()([row, dict(row)])
    short = {"input_ids": [CLS, 10, SEP], "special_tokens_mask": [1, 0, 1]}
    out = _col()([row, short])
    assert out["attention_mask"].tolist()[1] == [1, 1, 1, 0, 0, 0, 0, 0]


def test_collator_unions_dataset_special_mask_with_tokenizer_specials():
    # the dataset flags position 2 as special although its id is ordinary; UNK (3) is special by id only
    row = {"input_ids": [CLS, UNK, 50, 51, 52, 53, 54, SEP], "special_tokens_mask": [1, 0, 1, 0, 0, 0, 0, 1]}
    col = _col(mlm_probability=0.5, mask_token_prob=1.0, random_token_prob=0.0)
    for seed in range(20):
        torch.manual_seed(seed)
        out = col([dict(row), dict(row)])
        assert bool((out["labels"][:, [0, 1, 2, 7]] == -100).all())


def test_collator_does_not_mutate_its_input_features():
    rows = _rows(2, 64)
    before = [dict(input_ids=list(r["input_ids"]), special_tokens_mask=list(r["special_tokens_mask"])) for r in rows]
    _col()(rows)
    for r, b in zip(rows, before):
        assert r["input_ids"] == b["input_ids"] and r["special_tokens_mask"] == b["special_tokens_mask"]


class WordPieceTok(SyntheticTokenizer):
    """Ids ≥ 500 are ``##`` continuation pieces of the preceding word."""

    all_special_tokens = ["[PAD]", "[CLS]", "[SEP]", "[UNK]", "[MASK]"]

    def tokenize(self, text):
        return ["hello", "wor", "##ld"]

    def convert_ids_to_tokens(self, ids):
        names = {0: "[PAD]", 1: "[CLS]", 2: "[SEP]", 3: "[UNK]", 4: "[MASK]"}
        one = lambda i: names.get(int(i), f"##p{int(i)}" if int(i) >= 500 else f"w{int(i)}")  # noqa: E731
        return one(ids) if isinstance(ids, int) else [one(i) for i in ids]


def test_word_groups_follow_continuation_pieces_and_break_at_specials():
    col = _col(tokenizer=WordPieceTok(1000), max_ngram=2)
    assert col._word_boundary_scheme == "wordpiece"
    ids = [CLS, 10, 500, 501, 11, SEP, 502, 12, 503, SEP]
    spec = [t < 5 for t in ids]
    groups = col._build_word_groups(ids, spec)
    # a continuation piece straight after a special token starts its own group
    assert groups == [[1, 2, 3], [4], [6], [7, 8]]


@pytest.mark.parametrize("ngram", [2, 3])
def test_ngram_masking_masks_whole_words_within_budget(ngram):
    tok = WordPieceTok(1000)
    g = torch.Generator().manual_seed(5)
    rows = []
    for _ in range(4):
        body = []
        while len(body) < 62:
            body.append(int(torch.randint(5, 500, (1,), generator=g)))
            body.extend(int(x) for x in torch.randint(500, 1000, (int(torch.randint(0, 3, (1,), generator=g)),), generator=g))
        ids = [CLS, *body[:62], SEP]
        rows.append({"input_ids": ids, "special_tokens_mask": [int(t < 5) for t in ids]})
    col = _col(tokenizer=tok, max_ngram=ngram, mask_token_prob=1.0, random_token_prob=0.0)
    torch.manual_seed(6)
    out = col(rows)
    _w, cap, _n = col._budget(64)
    for b, r in enumerate(rows):
        picked = out["labels"][b].ne(-100).tolist()
        assert 0 < sum(picked) <= cap
        for grp in col._build_word_groups(r["input_ids"], [t < 5 for t in r["input_ids"]]):
            flags = {picked[i] for i in grp}
            assert len(flags) == 1  # a word is masked entirely or not at all


def test_ngram_masking_with_unknown_scheme_degrades_to_token_groups():
    col = _col(max_ngram=3, mask_token_prob=1.0, random_token_prob=0.0)  # SyntheticTokenizer has no tokenize()
    torch.manual_seed(7)
    out = col(_rows(2, 64))
    assert int(out["labels"].ne(-100).sum()) > 0


def test_collator_pad_to_multiple_of_is_forwarded_when_supported():
    seen = {}

    class Tok(SyntheticTokenizer):
        def pad(self, features, padding=True, return_tensors="pt", pad_to_multiple_of=None, **kw):
            seen["m"] = pad_to_multiple_of
            return super().pad(features, return_tensors=return_tensors)

    _col(tokenizer=Tok(1000), pad_to_multiple_of=16)(_rows(2, 64))
    assert seen["m"] == 16
