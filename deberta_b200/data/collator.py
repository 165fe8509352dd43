"""Dynamic masking collator for RTD pretraining (contract of ``data/collator.py`` of the reference).

Output batch: ``input_ids`` (masked), ``labels`` (original ids at masked positions, -100
elsewhere), ``attention_mask`` only when something is padded, ``doc_ids`` ``[B,S]``
(1-based, 0 = padding) when packed sequences should not attend across documents.

Masking is DeBERTa's *windowed* policy: maskable positions are cut into consecutive
windows of ``int(1/p)`` candidates, one position (or one whole-word n-gram, ``p(n) ∝ 1/n``)
is picked per window, and the first ``min(ceil(S·p/10)·10, max(1, round(S·p)))`` picks are
kept. The random draws are made in the same order as the reference, so both produce
identical batches from the same torch seed.
"""

from __future__ import annotations

import logging
import math
from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any

import torch

logger = logging.getLogger(__name__)

__all__ = ["MLMConfig", "DebertaV3ElectraCollator"]


@dataclass
class MLMConfig:
    mlm_probability: float = 0.15
    mask_token_prob: float = 0.8
    random_token_prob: float = 0.1
    max_ngram: int = 1


def _scheme_of(tokens: Sequence[str]) -> str:
    for marker, name in (("##", "wordpiece"), ("▁", "sentencepiece"), ("Ġ", "gpt2")):
        if any(t.startswith(marker) for t in tokens):
            return name
    return "none"


class DebertaV3ElectraCollator:
    def __init__(self, *, tokenizer: Any, cfg: MLMConfig, packed_sequences: bool = False,
                 block_cross_document_attention: bool = True, pad_to_multiple_of: int | None = None) -> None:
        self.tokenizer, self.cfg, self.pad_to_multiple_of = tokenizer, cfg, pad_to_multiple_of
        self._packed_sequences = bool(packed_sequences)
        self._block_cross_document_attention = bool(block_cross_document_attention)
        if tokenizer.mask_token_id is None:
            raise ValueError("Tokenizer must define a mask token for MLM masking.")
        if not 0.0 < float(cfg.mlm_probability) < 1.0:
            raise ValueError("mlm_probability must be in (0, 1).")
        if int(cfg.max_ngram) < 1:
            raise ValueError("max_ngram must be >= 1")
        mp, rp = float(cfg.mask_token_prob), float(cfg.random_token_prob)
        if mp < 0 or rp < 0 or mp + rp > 1.0:
            raise ValueError("Invalid masking probabilities: mask_token_prob + random_token_prob must be <= 1.")
        self._special_token_ids = self._collect_special_token_ids()
        self._special_ids_tensor = (torch.tensor(sorted(self._special_token_ids), dtype=torch.long)
                                    if self._special_token_ids else None)
        self._non_special_ids = self._build_non_special_token_ids()
        self._word_boundary_scheme = self._detect_word_boundary_scheme()
        self._word_continuation_by_id = self._build_word_continuation_lookup()
        if int(cfg.max_ngram) > 1 and self._word_boundary_scheme == "none":
            logger.warning("Tokenizer word-boundary probe returned scheme='none'; whole-word n-gram masking "
                           "will degrade to conservative token-level groups.")

    # ---- vocabulary helpers ------------------------------------------------------------------
    def _vocab_size(self) -> int:
        try:
            return int(len(self.tokenizer))
        except TypeError:
            return int(self.tokenizer.vocab_size)

    def _collect_special_token_ids(self) -> set[int]:
        out: set[int] = set()
        for sid in getattr(self.tokenizer, "all_special_ids", []) or []:
            try:
                out.add(int(sid))
            except (TypeError, ValueError):
                pass
        if getattr(self.tokenizer, "pad_token_id", None) is not None:
            out.add(int(self.tokenizer.pad_token_id))
        return out

    def _build_non_special_token_ids(self) -> torch.Tensor | None:
        if not self._special_token_ids:
            return None
        keep = torch.ones(self._vocab_size(), dtype=torch.bool)
        for sid in self._special_token_ids:
            if 0 <= sid < keep.numel():
                keep[sid] = False
        return torch.arange(keep.numel())[keep] if bool(keep.any()) else None

    def _sample_random_words(self, shape, device) -> torch.Tensor:
        """Uniform replacement ids that are never special tokens."""
        if self._non_special_ids is None:
            return torch.randint(0, self._vocab_size(), shape, device=device)
        ids = self._non_special_ids.to(device)
        return ids[torch.randint(0, int(ids.numel()), shape, device=device)]

    def _infer_special_tokens_mask(self, input_ids: torch.Tensor) -> torch.Tensor:
        if self._special_ids_tensor is not None and self._special_ids_tensor.numel():
            out = torch.isin(input_ids, self._special_ids_tensor.to(input_ids.device))
        else:
            out = torch.zeros_like(input_ids, dtype=torch.bool)
            if hasattr(self.tokenizer, "get_special_tokens_mask"):
                try:
                    rows = [self.tokenizer.get_special_tokens_mask(r, already_has_special_tokens=True)
                            for r in input_ids.tolist()]
                    out = torch.tensor(rows, dtype=torch.bool, device=input_ids.device)
                except Exception:
                    pass
        pad = getattr(self.tokenizer, "pad_token_id", None)
        return out | input_ids.eq(int(pad)) if pad is not None else out

    def _detect_word_boundary_scheme(self) -> str | None:
        tokenize = getattr(self.tokenizer, "tokenize", None)
        if not callable(tokenize):
            return None
        try:
            probe = tokenize("hello world")
        except Exception:
            return None
        return _scheme_of([str(t) for t in probe]) if isinstance(probe, list) and probe else None

    def _build_word_continuation_lookup(self) -> list[bool] | None:
        """``lookup[id]`` = token continues the previous word (one ``convert_ids_to_tokens`` call, up front)."""
        scheme = str(self._word_boundary_scheme or "").lower()
        if scheme not in {"wordpiece", "sentencepiece", "gpt2"}:
            return None
        n = self._vocab_size()
        try:
            toks = self.tokenizer.convert_ids_to_tokens(list(range(n)))
        except Exception:
            return None
        if not isinstance(toks, list) or len(toks) != n:
            return None
        special = set(getattr(self.tokenizer, "all_special_tokens", []))
        out = [False] * n
        for i, t in enumerate(toks):
            if not t or str(t) in special:
                continue
            t = str(t)
            out[i] = t.startswith("##") or (scheme == "sentencepiece" and not t.startswith("▁")) or (
                scheme == "gpt2" and not t.startswith("Ġ"))
        return out

    # ---- batch assembly ----------------------------------------------------------------------
    def __call__(self, features: list[dict[str, Any]]) -> dict[str, torch.Tensor]:
        if any("attention_mask" in f for f in features):
            features = [f if "attention_mask" in f else {**f, "attention_mask": [1] * len(f["input_ids"])}
                        for f in features]
        lengths = [len(f["input_ids"]) for f in features]
        needs_pad = len(set(lengths)) > 1 or (self.pad_to_multiple_of is not None and lengths
                                              and max(lengths) % int(self.pad_to_multiple_of))
        kw: dict[str, Any] = {"return_tensors": "pt", "pad_to_multiple_of": self.pad_to_multiple_of}
        if not needs_pad and not any("attention_mask" in f for f in features):
            kw["return_attention_mask"] = False
        try:
            batch = dict(self.tokenizer.pad(features, **kw))
        except TypeError:
            kw.pop("return_attention_mask", None)
            try:
                batch = dict(self.tokenizer.pad(features, **kw))
            except TypeError:
                kw.pop("pad_to_multiple_of", None)
                batch = dict(self.tokenizer.pad(features, **kw))
        pad_id = getattr(self.tokenizer, "pad_token_id", None)
        if "attention_mask" not in batch and pad_id is not None:
            attn = batch["input_ids"].ne(int(pad_id))
            if not bool(attn.all()):
                batch["attention_mask"] = attn.long()
        inferred = self._infer_special_tokens_mask(batch["input_ids"])
        special = batch.pop("special_tokens_mask", None)
        # datasets may flag only structural specials; the union keeps every tokenizer special unmaskable
        special = inferred if special is None else (special.bool() | inferred)
        doc_ids = None
        if self._packed_sequences and self._block_cross_document_attention:
            doc_ids = self._compute_document_ids(input_ids=batch["input_ids"], special_tokens_mask=special,
                                                 attention_mask=batch.get("attention_mask"))
        if doc_ids is not None:
            batch["doc_ids"] = doc_ids
        else:
            attn = batch.get("attention_mask")
            if attn is not None and bool(attn.bool().all()):
                batch.pop("attention_mask")  # nothing padded: the models' no-mask fast path applies
        batch["input_ids"], batch["labels"] = self._mask_tokens(batch["input_ids"], special_tokens_mask=special)
        return batch

    def _compute_document_ids(self, *, input_ids, special_tokens_mask, attention_mask) -> torch.Tensor | None:
        """1-based document index per token (0 = pad); ``None`` when no row has an internal separator."""
        sep_id = getattr(self.tokenizer, "sep_token_id", None)
        if input_ids.ndim != 2 or special_tokens_mask.shape != input_ids.shape or sep_id is None or input_ids.shape[1] < 3:
            return None
        pad_id = getattr(self.tokenizer, "pad_token_id", None)
        sep = input_ids.eq(int(sep_id)) & special_tokens_mask
        if attention_mask is not None and attention_mask.ndim == 2:
            active = attention_mask.bool()
        elif pad_id is not None:
            active = input_ids.ne(int(pad_id))
        else:
            active = torch.ones_like(input_ids, dtype=torch.bool)
        if not bool((sep[:, 1:-1] & active[:, 1:-1]).any()):
            return None
        prev = torch.zeros_like(sep)
        prev[:, 1:] = sep[:, :-1]
        boundary = (sep & ~prev).long()  # a run of separators counts once
        doc_ids = boundary.cumsum(dim=1) - boundary + 1
        cls_id = getattr(self.tokenizer, "cls_token_id", None)
        if cls_id is not None:
            doc_ids = doc_ids.masked_fill(input_ids.eq(int(cls_id)) & active, 1)
        if pad_id is not None:
            doc_ids = doc_ids.masked_fill(input_ids.eq(int(pad_id)), 0)
        return doc_ids

    # ---- masking -----------------------------------------------------------------------------
    def _mask_tokens(self, input_ids, *, special_tokens_mask):
        if int(self.cfg.max_ngram) <= 1:
            return self._mask_tokens_unigram_windowed(input_ids, special_tokens_mask=special_tokens_mask)
        return self._mask_tokens_ngram(input_ids, special_tokens_mask=special_tokens_mask, max_ngram=int(self.cfg.max_ngram))

    def _budget(self, seq_len: int) -> tuple[int, int, int]:
        """(window, per-sequence cap, number to predict) for a sequence length."""
        p = float(self.cfg.mlm_probability)
        cap = int(math.ceil(seq_len * p / 10.0) * 10)
        return max(1, int(1.0 / p)), cap, min(cap, max(1, int(round(seq_len * p))))

    @staticmethod
    def _sample_windowed_unigram_indices(maskable_idx: torch.Tensor, *, mask_window: int) -> torch.Tensor:
        """One uniformly chosen candidate out of every ``mask_window`` consecutive candidates."""
        count = int(maskable_idx.numel())
        if count <= 0:
            return maskable_idx.new_empty((0,), dtype=torch.long)
        if mask_window <= 1:
            return maskable_idx
        n = int(math.ceil(count / mask_window))
        starts = torch.arange(n, device=maskable_idx.device) * mask_window
        sizes = torch.clamp(torch.full((n,), mask_window, device=maskable_idx.device), max=count - starts)
        offs = torch.floor(torch.rand(n, device=maskable_idx.device, dtype=torch.float32) * sizes.float()).long()
        return maskable_idx.index_select(0, starts + offs)

    def _replace(self, input_ids: torch.Tensor, b: int, selected: torch.Tensor) -> None:
        """mask / random / keep roll over the selected positions of row ``b`` (in place)."""
        mp, rp = float(self.cfg.mask_token_prob), float(self.cfg.random_token_prob)
        mask_id = int(self.tokenizer.mask_token_id)
        if mp >= 1.0 and rp <= 0.0:
            input_ids[b, selected] = mask_id
            return
        keep_p = max(0.0, 1.0 - mp - rp)
        roll = torch.rand(int(selected.numel()), device=input_ids.device, dtype=torch.float32)
        m, r = roll < mp, roll >= (mp + keep_p)
        if bool(m.any()):
            input_ids[b, selected[m]] = mask_id
        if rp > 0.0 and bool(r.any()):
            input_ids[b, selected[r]] = self._sample_random_words((int(r.sum()),), input_ids.device)

    def _mask_tokens_unigram_windowed(self, input_ids, *, special_tokens_mask):
        input_ids = input_ids.long().clone()
        labels = torch.full_like(input_ids, -100)
        window, _cap, n_pred = self._budget(input_ids.shape[1])
        for b in range(input_ids.shape[0]):
            cand = torch.nonzero(~special_tokens_mask[b].bool(), as_tuple=False).squeeze(-1)
            if cand.numel() == 0:
                continue
            sel = self._sample_windowed_unigram_indices(cand, mask_window=window)[:n_pred]
            if sel.numel() == 0:
                continue
            labels[b].scatter_(0, sel, input_ids[b].index_select(0, sel))
            self._replace(input_ids, b, sel)
        return input_ids, labels

    def _mask_tokens_ngram(self, input_ids, *, special_tokens_mask, max_ngram: int):
        """Whole-word n-gram masking: per window of ``n·window`` words pick a start, mask ``n`` words."""
        if max_ngram <= 1:
            return self._mask_tokens_unigram_windowed(input_ids, special_tokens_mask=special_tokens_mask)
        input_ids = input_ids.long().clone()
        labels = torch.full_like(input_ids, -100)
        probs = torch.tensor([1.0 / n for n in range(1, max_ngram + 1)], dtype=torch.float32, device=input_ids.device)
        probs = probs / probs.sum().clamp(min=1e-12)
        window, cap, n_pred = self._budget(input_ids.shape[1])
        for b in range(input_ids.shape[0]):
            spec = special_tokens_mask[b].bool()
            if bool(spec.all()):
                continue
            groups = self._build_word_groups(input_ids[b].tolist(), spec.tolist())
            if not groups:
                continue
            chosen = [False] * len(groups)
            off = 0
            while off < len(groups):
                n = int(torch.multinomial(probs, 1).item()) + 1
                ctx = min(n * window, len(groups) - off)
                if ctx <= 0:
                    break
                m = int(torch.randint(0, ctx, (1,), device=input_ids.device).item())
                start, end = off + m, min(off + m + n, len(groups))
                off = max(off + ctx, end)
                for i in range(start, end):
                    chosen[i] = True
            picked: list[int] = []
            used = 0
            for flag, grp in zip(chosen, groups):
                if not flag:
                    continue
                if used + len(grp) > cap:
                    break
                if used + len(grp) > n_pred and used > 0:
                    continue  # never split a word to hit the budget exactly
                picked.extend(grp)
                used += len(grp)
                if used >= n_pred:
                    break
            if not picked:
                pool = [g for f, g in zip(chosen, groups) if f and len(g) <= cap] or [g for g in groups if len(g) <= cap]
                if not pool:
                    continue
                picked = list(pool[0])
            sel = torch.tensor(picked, device=input_ids.device, dtype=torch.long)
            labels[b].scatter_(0, sel, input_ids[b].index_select(0, sel))
            self._replace(input_ids, b, sel)
        return input_ids, labels

    def _build_word_groups(self, ids: Sequence[int], spec: Sequence[bool]) -> list[list[int]]:
        """Contiguous token positions that form one word; special positions are hard boundaries."""
        lookup = self._word_continuation_by_id
        if lookup is not None:
            def cont(i: int) -> bool | None:
                t = int(ids[i])
                return None if (t in self._special_token_ids or not 0 <= t < len(lookup)) else bool(lookup[t])
        else:
            toks = self.tokenizer.convert_ids_to_tokens(list(ids))
            special = set(getattr(self.tokenizer, "all_special_tokens", []))
            scheme = self._word_boundary_scheme
            if scheme is None:
                scheme = _scheme_of([t for t, s in zip(toks, spec) if not s and t and t not in special])
                self._word_boundary_scheme = scheme

            def cont(i: int) -> bool | None:
                t = toks[i]
                if not t or t in special:
                    return None
                return t.startswith("##") or (scheme == "sentencepiece" and not t.startswith("▁")) or (
                    scheme == "gpt2" and not t.startswith("Ġ"))
        groups: list[list[int]] = []
        prev: int | None = None
        for i, is_spec in enumerate(spec):
            c = None if is_spec else cont(i)
            if c is None:
                prev = None
                continue
            if groups and prev is not None and i == prev + 1 and c:
                groups[-1].append(i)
            else:
                groups.append([i])
            prev = i
        return groups
