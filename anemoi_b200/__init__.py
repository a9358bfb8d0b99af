"""B200-native sparse mixed-precision attention behind ``anemoi_attention``."""

from .api import NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention

__all__ = ["NVFP4Calibration", "QuantConfig", "SparseConfig", "VisualLayout", "anemoi_attention"]
