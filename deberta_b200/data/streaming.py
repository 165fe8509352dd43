"""Streaming datasets that turn documents into fixed-length token blocks.

Contract (``data/streaming.py`` of the reference): documents are tokenized without special
tokens, a ``[SEP]`` is appended after every document, the concatenated stream is cut into
blocks of ``max_seq_length - 2`` tokens and wrapped as ``[CLS] block [SEP]``; leading
separators of a block are dropped; the tail is flushed (minus trailing separators) with
padding and an ``attention_mask``; ``special_tokens_mask`` marks CLS / every SEP / PAD.
Each (rank, dataloader worker) pair reads a disjoint shard and the shuffle seed is
``seed + epoch``.
"""

from __future__ import annotations

import multiprocessing as mp
from collections.abc import Iterator
from dataclasses import dataclass
from typing import Any

import torch

__all__ = ["PackedStreamingConfig", "PackedStreamingDataset", "SequentialStreamingDataset"]


@dataclass
class PackedStreamingConfig:
    text_column_name: str = "text"
    max_seq_length: int = 512
    seed: int = 42
    shuffle_buffer_size: int = 10_000


class _TokenStream:
    """Rolling token buffer with O(1) amortised pops from the left."""

    def __init__(self) -> None:
        self.buf: list[int] = []
        self.start = 0

    def __len__(self) -> int:
        return len(self.buf) - self.start

    def extend(self, ids: list[int]) -> None:
        self.buf.extend(ids)

    def take(self, n: int) -> list[int]:
        out = self.buf[self.start : self.start + n]
        self.start += len(out)
        if self.start >= 65536 or self.start * 2 >= len(self.buf):
            self.buf = self.buf[self.start :]
            self.start = 0
        return out

    def rest(self) -> list[int]:
        return self.buf[self.start :]


class PackedStreamingDataset(torch.utils.data.IterableDataset):
    """Packs a (streaming) text dataset into ``[CLS] … [SEP]`` blocks of ``max_seq_length`` ids."""

    def __init__(self, *, hf_dataset: Any, tokenizer: Any, cfg: PackedStreamingConfig, process_index: int = 0,
                 num_processes: int = 1) -> None:
        super().__init__()
        self.hf_dataset, self.tokenizer, self.cfg = hf_dataset, tokenizer, cfg
        self.process_index, self.num_processes = int(process_index), int(num_processes)
        for name in ("cls_token_id", "sep_token_id", "pad_token_id"):
            if getattr(tokenizer, name, None) is None:
                raise ValueError(f"Tokenizer must define {name}.")
        try:  # shared so that persistent dataloader workers observe set_epoch()
            self._epoch: Any = mp.Value("i", 0)
        except Exception:
            self._epoch = None
        self._epoch_local = 0

    def set_epoch(self, epoch: int) -> None:
        e = int(max(0, epoch))
        if self._epoch is not None:
            with self._epoch.get_lock():
                self._epoch.value = e
        self._epoch_local = e
        if hasattr(self.hf_dataset, "set_epoch"):
            try:
                self.hf_dataset.set_epoch(e)
            except Exception:
                pass

    def _current_epoch(self) -> int:
        return int(self._epoch.value) if self._epoch is not None else int(self._epoch_local)

    def _iter_examples(self) -> Iterator[dict[str, Any]]:
        ds = self.hf_dataset
        seed = int(self.cfg.seed) + self._current_epoch()
        if self.cfg.shuffle_buffer_size and self.cfg.shuffle_buffer_size > 0 and hasattr(ds, "shuffle"):
            try:
                ds = ds.shuffle(buffer_size=self.cfg.shuffle_buffer_size, seed=seed)
            except TypeError:
                ds = ds.shuffle(seed=seed)
        info = torch.utils.data.get_worker_info()
        workers, wid = (1, 0) if info is None else (int(info.num_workers), int(info.id))
        if hasattr(ds, "shard"):
            ds = ds.shard(num_shards=self.num_processes * workers, index=self.process_index * workers + wid)
        return iter(ds)

    def _token_ids(self, example: dict[str, Any]) -> list[int]:
        key = self.cfg.text_column_name
        raw = example.get(key)
        if raw is None:
            raise KeyError(f"Text column '{key}' not found. Available keys: {list(example.keys())}")
        text = "\n".join(str(x) for x in raw) if isinstance(raw, (list, tuple)) else str(raw)
        if not text.strip():
            return []
        enc = self.tokenizer(text, add_special_tokens=False, return_attention_mask=False, return_token_type_ids=False)
        return [int(t) for t in enc.get("input_ids", [])]

    def _wrap(self, chunk: list[int], max_seq: int) -> dict[str, Any]:
        cls_id, sep_id, pad_id = (int(self.tokenizer.cls_token_id), int(self.tokenizer.sep_token_id),
                                  int(self.tokenizer.pad_token_id))
        pad = max_seq - len(chunk) - 2
        special = {cls_id, sep_id, pad_id}
        out: dict[str, Any] = {
            "input_ids": [cls_id, *chunk, sep_id, *([pad_id] * pad)],
            "special_tokens_mask": [1, *(1 if t in special else 0 for t in chunk), 1, *([1] * pad)],
        }
        if pad > 0:
            out["attention_mask"] = [1] * (max_seq - pad) + [0] * pad
        return out

    def __iter__(self) -> Iterator[dict[str, Any]]:
        max_seq = int(self.cfg.max_seq_length)
        if max_seq < 8:
            raise ValueError("max_seq_length is too small for pretraining.")
        sep_id, block = int(self.tokenizer.sep_token_id), max_seq - 2
        stream = _TokenStream()
        for ex in self._iter_examples():
            ids = self._token_ids(ex)
            if not ids:
                continue
            stream.extend(ids)
            stream.extend([sep_id])
            while len(stream) >= block:
                chunk = stream.take(block)
                lead = 0
                while lead < len(chunk) and chunk[lead] == sep_id:
                    lead += 1
                if lead < len(chunk):
                    yield self._wrap(chunk[lead:], max_seq)
        tail = stream.rest()
        while tail and tail[-1] == sep_id:
            tail.pop()
        tail = tail[:block]
        lead = 0
        while lead < len(tail) and tail[lead] == sep_id:
            lead += 1
        if lead < len(tail):
            yield self._wrap(tail[lead:], max_seq)


class SequentialStreamingDataset(PackedStreamingDataset):
    """One document per sequence; documents longer than a block continue in the next sequence."""

    def __iter__(self) -> Iterator[dict[str, Any]]:
        max_seq = int(self.cfg.max_seq_length)
        if max_seq < 8:
            raise ValueError("max_seq_length is too small for pretraining.")
        block = max_seq - 2
        for ex in self._iter_examples():
            ids = self._token_ids(ex)
            for i in range(0, len(ids), block):
                yield self._wrap(ids[i : i + block], max_seq)
