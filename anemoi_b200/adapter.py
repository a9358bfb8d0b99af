"""MiniMax-H3 adapter: drives the sparse attention like the reference's denoising loop.

Mirrors ``anemoi/models/minimax_h3/mpa_attention.py`` of the reference
(``H3MPAConfig`` :72-350, ``H3MPAAttention`` :385-636, ``install_layout_observer`` :639-656):
a callable that sits behind the model's (post-Ulysses) attention call, runs dense attention
for the first denoising steps of a request and the first layers of every step, and the
sparse mixed-precision path everywhere else, with per-layer sparsity bands, per-layer
precision bands and per-layer NVFP4 global scales.  Request and step boundaries are inferred
by an observer hooked in front of the transformer (one call per denoising step; a timestep
that reverses direction starts a new request).

Only what the sm_100a path implements is accepted: the experimental knobs of the reference
(FP8/MXFP8 phases, K-tail draft maps, diag-Jensen, anchors, smooth-K) must stay at their
"off" values, as they are on the reference's public path (mpa/executor.py:1262-1273).
The per-layer NVFP4 scales are supplied by the caller (a mapping or a JSON file with the
keys ``q_tensor_scale``, ``k_tensor_scale``, ``v_tensor_scale`` under ``scales``); the
reference ships its own calibration file for its checkpoint.
"""

from __future__ import annotations

import json
import math
import warnings
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Mapping

import torch
import torch.nn.functional as F

from .api import NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention

_SCALE_KEYS = ("q_tensor_scale", "k_tensor_scale", "v_tensor_scale")


def _is_real(value) -> bool:
    return not isinstance(value, bool) and isinstance(value, (int, float)) and math.isfinite(float(value))


def _check_bands(bands, layers: int, width: tuple[int, ...], what: str) -> None:
    """Bands are ``(first, last, ...)`` tuples, sorted, disjoint, inside ``[0, layers]``."""
    end = 0
    for band in bands:
        if not isinstance(band, tuple) or len(band) not in width:
            raise TypeError(f"{what} bands must be tuples of {' or '.join(map(str, width))} entries")
        first, last = band[0], band[1]
        if type(first) is not int or type(last) is not int or not 0 <= first < last <= layers or first < end:
            raise ValueError(f"{what} bands must be sorted, disjoint, and in range")
        end = last


@dataclass(frozen=True)
class H3MPAConfig:
    """Geometry, dense-first schedule and precision phases of one request."""

    video_shape: tuple[int, int, int] = (37, 24, 42)
    prefix_tokens: int = 951
    sparsity_ratio: float = 0.8
    query_block_size: int = 64
    prefix_kv_precision: str = "int8"
    prefix_query_precision: str = "int8"
    fp8_ratio: float = 0.0
    nvfp4_ratio: float = 0.0
    int8_ratio: float = 1.0
    mxfp8_ratio: float = 0.0
    fp16_ratio: float = 0.0
    dense_first_steps: int = 10
    dense_first_layers: int = 2
    layers_per_step: int = 50
    layer_sparsity_bands: tuple[tuple[int, int, float], ...] = ()
    layer_precision_bands: tuple[tuple[float | int, ...], ...] = ()
    draftmap_proxy: str = "mean"
    layer_draftmap_bands: tuple[tuple[int, int, str], ...] = ()
    diag_jensen: bool = False
    enable_anchors: bool = False
    strict: bool = True
    maxpool_weight: float = 0.0
    smooth_k: bool = False

    def __post_init__(self) -> None:
        shape = self.video_shape
        if not isinstance(shape, tuple) or len(shape) != 3 or any(type(n) is not int or n <= 0 for n in shape):
            raise ValueError("video_shape must contain three positive integers")
        if type(self.prefix_tokens) is not int or self.prefix_tokens <= 0:
            raise ValueError("prefix_tokens must be a positive integer")
        if type(self.layers_per_step) is not int or self.layers_per_step <= 0:
            raise ValueError("layers_per_step must be a positive integer")
        if type(self.query_block_size) is not int or self.query_block_size not in (64, 128):
            raise ValueError("query_block_size must be 64 or 128")
        for name in ("diag_jensen", "enable_anchors", "strict", "smooth_k"):
            if type(getattr(self, name)) is not bool:
                raise TypeError(f"{name} must be a boolean")
        if self.prefix_kv_precision not in ("nvfp4", "int8", "fp16"):
            raise ValueError("prefix_kv_precision must be nvfp4, int8, or fp16 on sm_100a")
        if self.prefix_query_precision not in ("int8", "fp16"):
            raise ValueError("prefix_query_precision must be int8 or fp16 on sm_100a")
        for name in ("dense_first_steps", "dense_first_layers"):
            value = getattr(self, name)
            if type(value) is not int or value < 0:
                raise ValueError("dense guards must be nonnegative integers")
        if self.dense_first_layers > self.layers_per_step:
            raise ValueError("dense_first_layers exceeds layers_per_step")
        if not _is_real(self.sparsity_ratio) or not 0.0 <= float(self.sparsity_ratio) < 1.0:
            raise ValueError("sparsity_ratio must be finite and in [0, 1)")
        if isinstance(self.maxpool_weight, bool) or not isinstance(self.maxpool_weight, (int, float)):
            raise TypeError("maxpool_weight must be a real number")
        if not math.isfinite(float(self.maxpool_weight)) or not 0.0 <= float(self.maxpool_weight) <= 1.0:
            raise ValueError("maxpool_weight must be finite and in [0, 1]")
        # knobs that have no sm_100a implementation stay off, as on the reference's public path
        if (float(self.fp8_ratio) != 0.0 or float(self.mxfp8_ratio) != 0.0 or self.draftmap_proxy != "mean"
                or self.layer_draftmap_bands or self.smooth_k):
            raise ValueError("fp8/mxfp8 phases, K-tail draft maps and smooth_k are not available on sm_100a")
        if self.diag_jensen and float(self.maxpool_weight) != 0.0:
            raise ValueError("maxpool_weight cannot be combined with diag_jensen")
        ratios = (float(self.nvfp4_ratio), float(self.int8_ratio), float(self.fp16_ratio))
        if any(not math.isfinite(r) or r < 0.0 for r in ratios) or not math.isclose(sum(ratios), 1.0, abs_tol=1.0e-6):
            raise ValueError("native phases require nonnegative NVFP4/INT8/FP16 ratios summing to one")
        _check_bands(self.layer_sparsity_bands, self.layers_per_step, (3,), "layer sparsity")
        for _, _, sparsity in self.layer_sparsity_bands:
            if not _is_real(sparsity) or not 0.0 <= float(sparsity) < 1.0:
                raise ValueError("layer sparsities must be finite and in [0, 1)")
        _check_bands(self.layer_precision_bands, self.layers_per_step, (5, 6), "layer precision")
        for band in self.layer_precision_bands:
            values = tuple(float(x) for x in band[2:])
            if any(not math.isfinite(x) or x < 0.0 for x in values) or not math.isclose(sum(values), 1.0, abs_tol=1.0e-6):
                raise ValueError("layer precision ratios must be nonnegative and sum to one")
            if len(values) == 4 and values[2] != 0.0:
                raise ValueError("the MXFP8 middle phase is not available on sm_100a")

    @property
    def video_tokens(self) -> int:
        return math.prod(self.video_shape)

    @property
    def sequence_tokens(self) -> int:
        return self.prefix_tokens + self.video_tokens

    def to_dict(self) -> dict[str, Any]:
        out = asdict(self)
        out.update(video_tokens=self.video_tokens, sequence_tokens=self.sequence_tokens)
        return out

    def _layer(self, layer: int) -> int:
        if type(layer) is not int or not 0 <= layer < self.layers_per_step:
            raise ValueError("layer is outside the configured transformer stack")
        return layer

    def precision(self, layer: int) -> tuple[float, float, float, float]:
        """``(nvfp4, int8, mxfp8, fp16)`` of a layer (mxfp8 is always 0 here)."""
        layer = self._layer(layer)
        for band in self.layer_precision_bands:
            if band[0] <= layer < band[1]:
                values = tuple(float(x) for x in band[2:])
                return (values[0], values[1], 0.0, values[-1])
        return (float(self.nvfp4_ratio), float(self.int8_ratio), 0.0, float(self.fp16_ratio))

    def sparsity(self, layer: int) -> float:
        layer = self._layer(layer)
        for first, last, value in self.layer_sparsity_bands:
            if first <= layer < last:
                return float(value)
        return float(self.sparsity_ratio)


def load_nvfp4_scales(source: Mapping | str | Path) -> dict[str, tuple[float, ...]]:
    """Per-layer NVFP4 global scales from a mapping or a JSON file (``{"scales": {...}}`` or the
    three lists at top level)."""
    table = json.loads(Path(source).read_text()) if isinstance(source, (str, Path)) else source
    table = table.get("scales", table)
    out = {key: tuple(float(x) for x in table[key]) for key in _SCALE_KEYS}
    if len({len(v) for v in out.values()}) != 1 or any(not (x > 0.0 and math.isfinite(x)) for v in out.values() for x in v):
        raise ValueError("NVFP4 scale lists must have one positive finite entry per layer")
    return out


def _first_video_position(video_indices: torch.Tensor, sequence_length: int) -> int:
    """Packed position where the target video starts: the first index of the last run of
    consecutive entries (mpa_attention.py:371-382 of the reference)."""
    if not isinstance(video_indices, torch.Tensor) or video_indices.ndim != 1:
        raise ValueError("video_indices must be rank one")
    if video_indices.numel() == 0:
        return sequence_length
    if video_indices.dtype not in (torch.int32, torch.int64):
        raise TypeError("video_indices must have integer dtype")
    jumps = (video_indices.diff() != 1).nonzero()
    start = int(jumps[-1]) + 1 if jumps.numel() else 0
    return int(video_indices[start])


class H3MPAAttention:
    """Post-Ulysses attention callable with the reference's dense-first schedule."""

    def __init__(self, config: H3MPAConfig, nvfp4_scales: Mapping | str | Path | None = None):
        if not isinstance(config, H3MPAConfig):
            raise TypeError("config must be H3MPAConfig")
        self.config = config
        self._scales = None if nvfp4_scales is None else load_nvfp4_scales(nvfp4_scales)
        self._layout = VisualLayout(config.video_shape, config.prefix_tokens)
        self.request, self.step, self.layer = -1, -1, 0
        self.dense_calls = self.mpa_calls = 0
        self.last_request_mpa_calls: int | None = None
        self._timestep: float | None = None
        self._direction = 0
        self._sequence_seen: int | None = None
        self._mpa_before_request = 0
        self._closed = -1
        self._device: torch.device | None = None      # where the sparse path last ran

    # ---- request / step tracking -------------------------------------------------------
    def observe(self, *, timestep: torch.Tensor | None, video_indices: torch.Tensor | None,
                position_ids: torch.Tensor) -> None:
        """Called once per transformer forward (one denoising step)."""
        sequence = int(position_ids.shape[0])
        self._sequence_seen = sequence
        if sequence != self.config.sequence_tokens:
            raise ValueError(f"observed {sequence} tokens, expected {self.config.sequence_tokens}")
        if video_indices is not None:
            prefix = _first_video_position(video_indices, sequence)
            if prefix != self.config.prefix_tokens:
                raise ValueError(f"observed prefix {prefix}, expected {self.config.prefix_tokens}")
        now = None if timestep is None else float(timestep.detach().float().max().item())
        before, self._timestep = self._timestep, now
        turned = False
        if before is not None and now is not None and abs(now - before) > 1.0e-6:
            sign = 1 if now > before else -1
            if self._direction == 0:
                self._direction = sign
            else:
                turned = sign != self._direction
        if self.step < 0 or turned:
            self.close_request()
            self.request += 1
            self.step, self._direction = 0, 0
        else:
            self.step += 1
        self.layer = 0

    def close_request(self) -> None:
        if self.request < 0 or self.request == self._closed:
            return
        self.last_request_mpa_calls = self.mpa_calls - self._mpa_before_request
        self._mpa_before_request = self.mpa_calls
        self._closed = self.request
        if self.last_request_mpa_calls > 0 and self._device is not None:
            # The end of a request is a synchronisation point anyway: read the device's sticky
            # status word there.  Non-zero means a bounded wait inside one of this device's
            # kernels gave up during the request; the outputs of that call are not valid.
            from . import executor

            status = executor.last_status(self._device)
            if status != 0:
                raise RuntimeError(
                    f"a kernel on {self._device} gave up a bounded wait during request {self.request} "
                    f"(status {status}); its results are invalid. Call executor.reset_status() after "
                    "handling the failure")
        if self.step + 1 <= self.config.dense_first_steps or self.last_request_mpa_calls > 0:
            return
        message = "request passed the dense-first schedule without an MPA call"
        if self.config.strict:
            raise RuntimeError(message)
        warnings.warn(message, RuntimeWarning, stacklevel=2)

    # ---- the two attention paths -------------------------------------------------------
    @staticmethod
    def _check(q, k, v) -> None:
        if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
            raise TypeError("Q/K/V must be tensors")
        if q.ndim != 3 or q.shape != k.shape or q.shape != v.shape:
            raise ValueError("Q/K/V must share [sequence,heads,D]")
        if (q.device.type != "cuda" or k.device != q.device or v.device != q.device
                or q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype
                or q.shape[-1] not in (64, 128) or any(t.stride(-1) != 1 for t in (q, k, v))):
            raise ValueError("Q/K/V must be same-dtype CUDA tensors with head_dim 64 or 128")

    @staticmethod
    def dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Dense attention of ``[S, H, D]`` tensors through torch's library kernel."""
        H3MPAAttention._check(q, k, v)
        out = F.scaled_dot_product_attention(*(t.transpose(0, 1).unsqueeze(0) for t in (q, k, v)),
                                             dropout_p=0.0, is_causal=False)
        return out.squeeze(0).transpose(0, 1)

    def calibration(self, layer: int) -> NVFP4Calibration | None:
        nvfp4 = self.config.precision(layer)[0]
        if nvfp4 <= 0.0 and self.config.prefix_kv_precision != "nvfp4":
            return None
        if self._scales is None:
            raise RuntimeError("an NVFP4 phase needs per-layer scales (nvfp4_scales=...)")
        if not 0 <= layer < len(self._scales[_SCALE_KEYS[0]]):
            raise ValueError("layer is outside the NVFP4 calibration")
        return NVFP4Calibration(*(self._scales[key][layer] for key in _SCALE_KEYS))

    def mpa(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, layer: int) -> torch.Tensor:
        """Sparse mixed-precision attention of one layer (strided ``[S, H, D]`` views are fine)."""
        self._check(q, k, v)
        self._device = q.device
        cfg = self.config
        if q.shape[0] != cfg.sequence_tokens:
            raise ValueError("packed sequence length does not match the H3 request")
        nvfp4, int8, _, fp16 = cfg.precision(layer)
        if cfg.diag_jensen or cfg.enable_anchors:
            # the experimental routing variants are not part of the public call; as in the
            # reference's adapter (mpa_attention.py:584-600) the executor is called directly
            from . import executor

            calib = self.calibration(layer)
            return executor.sm100_ragged_attention(
                q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), prefix_tokens=cfg.prefix_tokens,
                sparsity_ratio=cfg.sparsity(layer), retained_nvfp4_ratio=nvfp4, retained_int8_ratio=int8,
                retained_fp16_ratio=fp16, video_shape=cfg.video_shape, layer=layer,
                query_block_size=cfg.query_block_size, prefix_kv_precision=cfg.prefix_kv_precision,
                prefix_query_precision=cfg.prefix_query_precision, maxpool_weight=float(cfg.maxpool_weight),
                nvfp4_scales=(1.0, 1.0, 1.0) if calib is None else (calib.q_scale, calib.k_scale,
                                                                     calib.v_scale),
                diag_jensen=cfg.diag_jensen, enable_anchors=cfg.enable_anchors).squeeze(0)
        out = anemoi_attention(
            q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), layout=self._layout, layer=layer,
            sparse_config=SparseConfig(cfg.query_block_size, cfg.sparsity(layer), (), float(cfg.maxpool_weight)),
            quant_config=QuantConfig(nvfp4, int8, fp16, cfg.prefix_kv_precision, cfg.prefix_query_precision),
            calibration=self.calibration(layer))
        return out.squeeze(0)

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if self.config.strict and self.request < 0:
            raise RuntimeError("the H3 layout observer did not run")
        layer, self.layer = self.layer, self.layer + 1
        if self.step < self.config.dense_first_steps or layer < self.config.dense_first_layers:
            self.dense_calls += 1
            return self.dense(q, k, v)
        self.mpa_calls += 1
        return self.mpa(q, k, v, layer=layer)

    def stats(self) -> dict[str, Any]:
        total = self.dense_calls + self.mpa_calls
        return {"config": self.config.to_dict(), "routing_block_size": self.config.query_block_size,
                "request": self.request, "step": self.step, "layer": self.layer,
                "observed_sequence": self._sequence_seen, "dense_calls": self.dense_calls,
                "mpa_calls": self.mpa_calls, "mpa_calls_measured_request": self.last_request_mpa_calls,
                "mpa_fraction": self.mpa_calls / total if total else None}


def install_layout_observer(transformer: torch.nn.Module, attention: H3MPAAttention):
    """Hooks ``attention.observe`` in front of ``transformer.forward`` (keyword arguments
    ``position_ids``, ``timestep``, ``video_indices``); returns the hook handle."""
    if not isinstance(attention, H3MPAAttention):
        raise TypeError("attention must be H3MPAAttention")

    def before_forward(_module, _args, kwargs):
        ids = kwargs.get("position_ids")
        if ids is not None:
            attention.observe(timestep=kwargs.get("timestep"), video_indices=kwargs.get("video_indices"),
                              position_ids=ids)

    return transformer.register_forward_pre_hook(before_forward, with_kwargs=True)


__all__ = ["H3MPAAttention", "H3MPAConfig", "install_layout_observer", "load_nvfp4_scales"]
