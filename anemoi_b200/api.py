"""Public Q/K/V attention entry point for B200 (sm_100a).

Mirrors the reference's stable interface (anemoi/layers/attention/api.py:10-194):
the same four frozen configuration dataclasses with the same validation errors,
and ``anemoi_attention(query, key, value, *, layout, layer, sparse_config,
quant_config, calibration)`` with the same fixed semantics (no mask, no dropout,
non-causal, ``scale`` either ``None`` or ``1/sqrt(head_dim)``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch


def _is_real(value) -> bool:
    return not isinstance(value, bool) and isinstance(value, (int, float))


def _finite_in(value, low: float, high: float, *, closed_high: bool) -> bool:
    if not _is_real(value) or not math.isfinite(float(value)):
        return False
    v = float(value)
    return low <= v <= high if closed_high else low <= v < high


@dataclass(frozen=True)
class VisualLayout:
    """Video tokens of shape (frames, height, width) after an optional packed prefix."""

    video_shape: tuple[int, int, int]
    prefix_tokens: int = 0

    def __post_init__(self) -> None:
        shape = self.video_shape
        if (
            not isinstance(shape, tuple)
            or len(shape) != 3
            or any(type(v) is not int or v <= 0 for v in shape)
        ):
            raise ValueError("video_shape must contain three positive integers")
        if type(self.prefix_tokens) is not int or self.prefix_tokens < 0:
            raise ValueError("prefix_tokens must be a nonnegative integer")

    @property
    def video_tokens(self) -> int:
        return math.prod(self.video_shape)

    @property
    def sequence_tokens(self) -> int:
        return self.prefix_tokens + self.video_tokens


@dataclass(frozen=True)
class SparseConfig:
    """Query block size and the per-layer block-drop schedule.

    ``layer_sparsity_bands`` holds ``(first, last, ratio)`` triples over zero-based
    half-open layer ranges; the first matching band overrides ``sparsity_ratio``.
    """

    query_block_size: int = 64
    sparsity_ratio: float = 0.80
    layer_sparsity_bands: tuple[tuple[int, int, float], ...] = ()
    maxpool_weight: float = 0.0

    def __post_init__(self) -> None:
        if type(self.query_block_size) is not int or self.query_block_size not in (64, 128):
            raise ValueError("query_block_size must be 64 or 128")
        if not _finite_in(self.sparsity_ratio, 0.0, 1.0, closed_high=False):
            raise ValueError("sparsity_ratio must be finite and in [0, 1)")
        if not _is_real(self.maxpool_weight):
            raise TypeError("maxpool_weight must be a real number")
        if not _finite_in(self.maxpool_weight, 0.0, 1.0, closed_high=True):
            raise ValueError("maxpool_weight must be finite and in [0, 1]")
        cursor = 0
        for band in self.layer_sparsity_bands:
            if not isinstance(band, tuple) or len(band) != 3:
                raise TypeError("layer bands must be (first, last, sparsity)")
            first, last, ratio = band
            if (
                type(first) is not int
                or type(last) is not int
                or not 0 <= first < last
                or first < cursor
            ):
                raise ValueError("layer bands must be sorted, disjoint, and nonnegative")
            if not _finite_in(ratio, 0.0, 1.0, closed_high=False):
                raise ValueError("layer sparsities must be finite and in [0, 1)")
            cursor = last

    def sparsity_for_layer(self, layer: int) -> float:
        for first, last, ratio in self.layer_sparsity_bands:
            if first <= layer < last:
                return ratio
        return self.sparsity_ratio


@dataclass(frozen=True)
class QuantConfig:
    """Shares of the retained blocks per precision cell, and the prefix precisions."""

    nvfp4_ratio: float = 0.0
    int8_ratio: float = 1.0
    fp16_ratio: float = 0.0
    prefix_kv_precision: str = "int8"
    prefix_query_precision: str = "int8"

    def __post_init__(self) -> None:
        shares = (self.nvfp4_ratio, self.int8_ratio, self.fp16_ratio)
        bad = any(
            not _is_real(v) or not math.isfinite(float(v)) or float(v) < 0.0 for v in shares
        )
        if bad or not math.isclose(sum(map(float, shares)), 1.0, abs_tol=1.0e-6):
            raise ValueError("NVFP4/INT8/FP16 ratios must be nonnegative and sum to one")
        if self.prefix_kv_precision not in ("nvfp4", "int8", "fp16"):
            raise ValueError("prefix_kv_precision must be nvfp4, int8, or fp16")
        if self.prefix_query_precision not in ("int8", "fp16"):
            raise ValueError("prefix_query_precision must be int8 or fp16")


@dataclass(frozen=True)
class NVFP4Calibration:
    """Tensor-level global scales of Q, K and V for the NVFP4 cell."""

    q_scale: float = 1.0
    k_scale: float = 1.0
    v_scale: float = 1.0

    def __post_init__(self) -> None:
        for v in (self.q_scale, self.k_scale, self.v_scale):
            if not _is_real(v) or not math.isfinite(float(v)) or float(v) <= 0.0:
                raise ValueError("NVFP4 calibration scales must be finite and positive")

    @property
    def scales(self) -> tuple[float, float, float]:
        return (float(self.q_scale), float(self.k_scale), float(self.v_scale))


def anemoi_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: torch.Tensor | None = None,
    *,
    layout: VisualLayout,
    layer: int,
    sparse_config: SparseConfig | None = None,
    quant_config: QuantConfig | None = None,
    calibration: NVFP4Calibration | None = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    scale: float | None = None,
) -> torch.Tensor:
    """Block-sparse mixed-precision attention over ``[1, S, H, D]`` Q/K/V on one B200."""
    if attn_mask is not None:
        raise ValueError("attn_mask is not supported")
    if dropout_p != 0.0:
        raise ValueError("dropout_p must be 0.0")
    if is_causal:
        raise ValueError("is_causal must be False")
    if not isinstance(layout, VisualLayout):
        raise TypeError("layout must be VisualLayout")
    if type(layer) is not int or layer < 0:
        raise ValueError("layer must be a nonnegative integer")
    if query.ndim != 4 or query.size(1) != layout.sequence_tokens:
        raise ValueError("Q sequence length must match layout.sequence_tokens")
    if scale is not None and not math.isclose(scale, 1.0 / math.sqrt(query.size(-1))):
        raise ValueError("scale must be None or 1/sqrt(head_dim)")
    sparse = sparse_config if sparse_config else SparseConfig()
    quant = quant_config if quant_config else QuantConfig()
    calib = NVFP4Calibration() if calibration is None else calibration
    if not isinstance(calib, NVFP4Calibration):
        raise TypeError("calibration must be NVFP4Calibration")

    from .executor import execute_ragged_attention

    return execute_ragged_attention(
        query,
        key,
        value,
        prefix_tokens=layout.prefix_tokens,
        video_shape=layout.video_shape,
        layer=layer,
        query_block_size=sparse.query_block_size,
        sparsity_ratio=sparse.sparsity_for_layer(layer),
        nvfp4_ratio=quant.nvfp4_ratio,
        int8_ratio=quant.int8_ratio,
        fp16_ratio=quant.fp16_ratio,
        prefix_kv_precision=quant.prefix_kv_precision,
        prefix_query_precision=quant.prefix_query_precision,
        maxpool_weight=float(sparse.maxpool_weight),
        nvfp4_scales=calib.scales,
    )


__all__ = [
    "NVFP4Calibration",
    "QuantConfig",
    "SparseConfig",
    "VisualLayout",
    "anemoi_attention",
]
