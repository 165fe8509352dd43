"""Offline synthetic corpus and tokenizer.

The benchmark configurations are defined on synthetic data: token ids drawn from a
Zipf(s) law over the non-special vocabulary, grouped into documents whose lengths are
geometric with a given mean. ``SyntheticTextDataset`` renders such documents as text of
the form ``"t123 t45 …"`` so they flow through the same packer / collator path as real
text, and ``SyntheticTokenizer`` maps that text back to ids without any downloaded files.
Both shard and shuffle deterministically from a seed.
"""

from __future__ import annotations

import re
from collections.abc import Iterator
from typing import Any

import numpy as np
import torch

SYNTHETIC_DATASET_NAME = "synthetic"
SYNTHETIC_TOKENIZER_NAME = "synthetic"
_SPEC_RE = re.compile(r"^zipf(?P<s>[0-9.]+)-mean(?P<mean>[0-9]+)(?:-vocab(?P<vocab>[0-9]+))?(?:-docs(?P<docs>[0-9]+))?$")


def parse_synthetic_spec(spec: str | None) -> dict[str, Any]:
    """``"zipf1.1-mean60[-vocab128100][-docs100000]"`` → keyword arguments of ``SyntheticTextDataset``."""
    if not spec or str(spec).strip().lower() in {"default", "none"}:
        return {}
    m = _SPEC_RE.match(str(spec).strip().lower())
    if not m:
        raise ValueError(f"Unrecognised synthetic dataset spec {spec!r}; expected e.g. 'zipf1.1-mean60-vocab128100'.")
    out: dict[str, Any] = {"zipf_s": float(m["s"]), "mean_doc_len": int(m["mean"])}
    if m["vocab"]:
        out["vocab_size"] = int(m["vocab"])
    if m["docs"]:
        out["num_docs"] = int(m["docs"])
    return out


class ZipfSampler:
    """Inverse-CDF sampler of Zipf(s) ranks over ``[first_id, vocab_size)``."""

    def __init__(self, vocab_size: int, zipf_s: float = 1.1, first_id: int = 5) -> None:
        n = int(vocab_size) - int(first_id)
        if n <= 0:
            raise ValueError("vocab_size must exceed the number of reserved special ids")
        w = 1.0 / np.power(np.arange(1, n + 1, dtype=np.float64), float(zipf_s))
        self.cdf = np.cumsum(w / w.sum())
        self.first_id = int(first_id)

    def sample(self, rng: np.random.Generator, n: int) -> np.ndarray:
        return np.searchsorted(self.cdf, rng.random(n), side="left").astype(np.int64) + self.first_id


class SyntheticTextDataset:
    """Iterable of ``{"text": "t17 t5 …"}`` documents with ``shuffle`` / ``shard`` / ``set_epoch`` like HF datasets."""

    def __init__(self, *, vocab_size: int = 128_100, zipf_s: float = 1.1, mean_doc_len: int = 60,
                 num_docs: int | None = None, seed: int = 0, text_column_name: str = "text",
                 _shard: tuple[int, int] = (1, 0)) -> None:
        self.vocab_size, self.zipf_s, self.mean_doc_len = int(vocab_size), float(zipf_s), int(mean_doc_len)
        self.num_docs, self.seed, self.text_column_name = num_docs, int(seed), str(text_column_name)
        self._num_shards, self._shard_index = _shard
        self._epoch = 0
        self._sampler = ZipfSampler(self.vocab_size, self.zipf_s)

    def _clone(self, **kw: Any) -> "SyntheticTextDataset":
        base = dict(vocab_size=self.vocab_size, zipf_s=self.zipf_s, mean_doc_len=self.mean_doc_len,
                    num_docs=self.num_docs, seed=self.seed, text_column_name=self.text_column_name,
                    _shard=(self._num_shards, self._shard_index))
        base.update(kw)
        out = SyntheticTextDataset(**base)
        out._epoch = self._epoch
        return out

    def shuffle(self, seed: int = 0, buffer_size: int | None = None) -> "SyntheticTextDataset":
        return self._clone(seed=int(seed))

    def shard(self, num_shards: int, index: int) -> "SyntheticTextDataset":
        return self._clone(_shard=(self._num_shards * int(num_shards), self._shard_index * int(num_shards) + int(index)))

    def set_epoch(self, epoch: int) -> None:
        self._epoch = int(epoch)

    def iter_token_docs(self) -> Iterator[np.ndarray]:
        """Documents as id arrays (skips the text round trip; used by the fast synthetic batch source)."""
        rng = np.random.default_rng([self.seed, self._epoch, self._num_shards, self._shard_index])
        p = 1.0 / max(1, self.mean_doc_len)
        produced = 0
        limit = None if self.num_docs is None else max(0, (self.num_docs - self._shard_index + self._num_shards - 1) // self._num_shards)
        while limit is None or produced < limit:
            lengths = rng.geometric(p, size=256)
            toks = self._sampler.sample(rng, int(lengths.sum()))
            pos = 0
            for n in lengths:
                if limit is not None and produced >= limit:
                    return
                yield toks[pos : pos + n]
                pos += n
                produced += 1

    def __iter__(self) -> Iterator[dict[str, str]]:
        for doc in self.iter_token_docs():
            yield {self.text_column_name: " ".join(f"t{int(t)}" for t in doc)}


class SyntheticTokenizer:
    """Whitespace tokenizer over ``t<id>`` words with DeBERTa-like special ids; no files needed.

    ``[PAD]=0 [CLS]=1 [SEP]=2 [UNK]=3 [MASK]=4``; words that are not ``t<id>`` hash into the
    ordinary id range so arbitrary text still tokenizes deterministically.
    """

    pad_token, cls_token, sep_token, unk_token, mask_token = "[PAD]", "[CLS]", "[SEP]", "[UNK]", "[MASK]"
    pad_token_id, cls_token_id, sep_token_id, unk_token_id, mask_token_id = 0, 1, 2, 3, 4
    bos_token_id = eos_token_id = None
    is_fast = True

    def __init__(self, vocab_size: int = 128_100) -> None:
        self.vocab_size = int(vocab_size)
        self._extra: list[str] = []
        self.name_or_path = SYNTHETIC_TOKENIZER_NAME

    def __len__(self) -> int:
        return self.vocab_size + len(self._extra)

    @property
    def all_special_ids(self) -> list[int]:
        return [0, 1, 2, 3, 4]

    def add_tokens(self, tokens: list[str], special_tokens: bool = False) -> int:
        self._extra.extend(tokens)
        return len(tokens)

    def get_special_tokens_mask(self, ids: list[int], already_has_special_tokens: bool = True) -> list[int]:
        return [1 if int(t) < 5 else 0 for t in ids]

    def convert_ids_to_tokens(self, ids):
        names = {0: "[PAD]", 1: "[CLS]", 2: "[SEP]", 3: "[UNK]", 4: "[MASK]"}
        one = lambda i: names.get(int(i), f"▁t{int(i)}")  # noqa: E731
        return one(ids) if isinstance(ids, int) else [one(i) for i in ids]

    def _word_id(self, w: str) -> int:
        if len(w) > 1 and w[0] == "t" and w[1:].isdigit():
            i = int(w[1:])
            if 5 <= i < self.vocab_size:
                return i
        h = 0
        for ch in w.encode("utf-8"):
            h = (h * 131 + ch) % 2_147_483_647
        return 5 + h % (self.vocab_size - 5)

    def __call__(self, text, add_special_tokens: bool = False, **_: Any) -> dict[str, Any]:
        def enc(t: str) -> list[int]:
            ids = [self._word_id(w) for w in t.split()]
            return [1] + ids + [2] if add_special_tokens else ids
        if isinstance(text, str):
            return {"input_ids": enc(text)}
        return {"input_ids": [enc(t) for t in text]}

    def pad(self, features: list[dict[str, Any]], padding: bool = True, return_tensors: str | None = "pt", **_: Any):
        """Right-pad a list of feature dicts to the longest ``input_ids`` (pads get attention 0, special 1)."""
        width = max(len(f["input_ids"]) for f in features)
        fill = {"input_ids": self.pad_token_id, "attention_mask": 0, "special_tokens_mask": 1, "token_type_ids": 0}
        need_mask = any(len(f["input_ids"]) != width for f in features) or any("attention_mask" in f for f in features)
        out: dict[str, list] = {}
        for key in {k for f in features for k in f}:
            if key not in fill:
                continue
            out[key] = [list(f.get(key, [1] * len(f["input_ids"]))) + [fill[key]] * (width - len(f["input_ids"]))
                        for f in features]
        if need_mask and "attention_mask" not in out:
            out["attention_mask"] = [[1] * len(f["input_ids"]) + [0] * (width - len(f["input_ids"])) for f in features]
        return {k: torch.tensor(v, dtype=torch.long) for k, v in out.items()} if return_tensors == "pt" else out

    def save_pretrained(self, path: str) -> None:
        import json
        from pathlib import Path

        Path(path).mkdir(parents=True, exist_ok=True)
        (Path(path) / "synthetic_tokenizer.json").write_text(json.dumps({"vocab_size": self.vocab_size, "extra": self._extra}))


def load_tokenizer(name_or_path: str, *, vocab_size: int = 128_100) -> Any:
    """``"synthetic"`` / ``"synthetic:<vocab>"`` → ``SyntheticTokenizer``; anything else → ``AutoTokenizer``."""
    key = str(name_or_path).strip()
    if key.lower().split(":")[0] == SYNTHETIC_TOKENIZER_NAME:
        parts = key.split(":")
        return SyntheticTokenizer(int(parts[1]) if len(parts) > 1 else vocab_size)
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(key, use_fast=True)
