"""Backbones, the RTD pretraining wrapper and their builders."""

from .builder import build_backbone_configs, build_backbones
from .deberta_v2 import DebertaV2Config, DebertaV2Model
from .rope_encoder import DebertaRoPEConfig, DebertaRoPEModel
from .rtd import DebertaV3RTDPretrainer

__all__ = ["build_backbone_configs", "build_backbones", "DebertaV2Config", "DebertaV2Model", "DebertaRoPEConfig",
           "DebertaRoPEModel", "DebertaV3RTDPretrainer"]
