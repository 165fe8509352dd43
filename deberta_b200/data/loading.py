"""Dataset source resolution (``data/loading.py`` of the reference) plus the built-in synthetic source.

``data.source.dataset_name = "synthetic"`` (optionally ``dataset_config_name =
"zipf1.1-mean60"`` etc.) selects the offline generator of ``data/synthetic.py`` instead of
the Hugging Face hub; every other value goes through ``datasets`` exactly as in the reference.
"""

from __future__ import annotations

from typing import Any

from deberta_b200.config import DataConfig

from .synthetic import SYNTHETIC_DATASET_NAME, SyntheticTextDataset, parse_synthetic_spec


def load_hf_dataset(*, cfg: DataConfig, split: str | None = None, streaming: bool | None = None) -> Any:
    """Open the configured dataset: ``load_from_disk`` | hub name (+config, +data_files) | local text files."""
    src = cfg.source
    split = split or src.train_split
    streaming = bool(src.streaming if streaming is None else streaming)
    if src.dataset_name and str(src.dataset_name).strip().lower() == SYNTHETIC_DATASET_NAME:
        return SyntheticTextDataset(**parse_synthetic_spec(src.dataset_config_name), text_column_name=src.text_column_name)
    import datasets

    if src.load_from_disk:
        ds = datasets.load_from_disk(src.load_from_disk)
        if isinstance(ds, datasets.DatasetDict):
            if split not in ds:
                raise ValueError(f"Split {split!r} not found in dataset at {src.load_from_disk}: {list(ds.keys())}")
            ds = ds[split]
        return ds
    files = [f.strip() for f in str(src.data_files).split(",") if f.strip()] if src.data_files else None
    if src.dataset_name:
        kw: dict[str, Any] = {"split": split, "streaming": streaming}
        if src.dataset_config_name:
            kw["name"] = src.dataset_config_name
        if files:
            kw["data_files"] = files
        return datasets.load_dataset(src.dataset_name, **kw)
    if files:
        return datasets.load_dataset("text", data_files=files, split=split, streaming=streaming)
    raise ValueError("No dataset source configured. Provide one of: data.source.load_from_disk, "
                     "data.source.dataset_name, or data.source.data_files.")
