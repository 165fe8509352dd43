"""Data pipeline: dataset sources, streaming packer, masking collator."""

from .collator import DebertaV3ElectraCollator, MLMConfig
from .loading import load_hf_dataset
from .streaming import PackedStreamingConfig, PackedStreamingDataset, SequentialStreamingDataset

__all__ = ["DebertaV3ElectraCollator", "MLMConfig", "load_hf_dataset", "PackedStreamingConfig",
           "PackedStreamingDataset", "SequentialStreamingDataset"]
