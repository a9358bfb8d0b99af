"""B200-native sparse mixed-precision attention behind ``anemoi_attention``."""

from .api import NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention
from .host import HostAttention

__all__ = ["HostAttention", "NVFP4Calibration", "QuantConfig", "SparseConfig", "VisualLayout",
           "anemoi_attention"]
