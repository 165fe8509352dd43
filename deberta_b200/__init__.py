"""deberta_b200: Blackwell-native DeBERTa-v3 replaced-token-detection pretraining.

Same capabilities as the ``deberta`` package of pszemraj/deberta (config schema, CLI,
backbones, RTD objective, data pipeline, checkpoints, export), with hot operations
implemented as hand-written sm_100a kernels.
"""

__version__ = "0.1.0"

__all__ = ["__version__"]
