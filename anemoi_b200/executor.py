"""Orchestration of one ``anemoi_attention`` call on a B200.

Follows the reference's executor (anemoi/layers/attention/mpa/executor.py):
``execute_ragged_attention`` (:1227-1295) dispatches on the device capability -
here only (10, 0) is accepted - and ``sm100_ragged_attention`` walks the same
steps as ``sm120_ragged_h3_attention`` (:876-1224): validate, resolve phases,
slot tables (cached), prepare operands, draft probability, route, attention
phases, prefix rows on a side stream, assembly.  No host synchronisation happens
on the path.  The public path pins the same options as the reference: mean-pool
draft map, no diag-Jensen term, no anchors, no MXFP8 cell.
"""

from __future__ import annotations

import math
from functools import lru_cache

import torch
import torch.nn.functional as F

from . import native
from .layout import materialize_ragged_2d_layout
from .routing import PHASE_ORDER, resolve_phases, route_counts, video_phases

_STATUS: dict = {}
_STAGE_EVENTS: list | None = None


def collect_stage_events(enable: bool) -> None:
    """Start (or stop) recording CUDA events around each native stage of later calls."""
    global _STAGE_EVENTS
    _STAGE_EVENTS = [] if enable else None


def stage_times_ms() -> dict:
    """Per-stage device time summed over the calls recorded so far (synchronises)."""
    torch.cuda.synchronize()
    out: dict = {}
    for name, start, end in _STAGE_EVENTS or []:
        out[name] = out.get(name, 0.0) + start.elapsed_time(end)
    return out


_PROFILE_NVTX = False
_PAIR_Q64 = True      # Q64 query blocks run two per CTA; False keeps one (padded) block per CTA


def set_profile_nvtx(enabled: bool) -> None:
    """Process-wide switch for the NVTX ranges of every call (the per-call ``profile_nvtx``
    argument turns them on for one call).  The ranges carry the reference's names
    (anemoi/layers/attention/mpa/executor.py:901-902, 983-990, 1102, 1179, 1207):
    ``anemoi.complete`` around the call and inside it ``anemoi.peripheral.prepare``,
    ``anemoi.dense_prefix``, ``anemoi.peripheral.draft_route_materialize``, ``anemoi.mpa_mainloop``
    and ``anemoi.peripheral.assembly``, so a timeline taken from either implementation reads
    the same."""
    global _PROFILE_NVTX
    if type(enabled) is not bool:
        raise TypeError("enabled must be a bool")
    _PROFILE_NVTX = enabled


class _Range:
    """An NVTX range on the calling thread (host-side marker around the launches)."""

    def __init__(self, name: str, enabled: bool):
        self.name, self.enabled = name, enabled

    def __enter__(self):
        if self.enabled:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.enabled:
            torch.cuda.nvtx.range_pop()
        return False


class _Stage:
    """Brackets one native stage with CUDA events on the current stream when enabled."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _STAGE_EVENTS is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if _STAGE_EVENTS is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _STAGE_EVENTS.append((self.name, self.start, end))
        return False


@lru_cache(maxsize=8)
def _prefix_stream(device: torch.device) -> torch.cuda.Stream:
    return torch.cuda.Stream(device=device)


@lru_cache(maxsize=64)
def _valid_k(device: torch.device, prefix_tokens: int, query_block: int, counts_key) -> torch.Tensor:
    """Real keys per 64-key stage (executor.py:334-342,1052-1067 of the reference)."""
    counts = torch.tensor(counts_key, dtype=torch.int32)
    p = math.ceil(prefix_tokens / 64)
    pre = torch.clamp(prefix_tokens - torch.arange(p, dtype=torch.int32) * 64, 0, 64)
    if query_block == 128:
        vid = torch.stack((counts.clamp_max(64), (counts - 64).clamp_min(0)), dim=-1).reshape(-1)
    else:
        vid = counts
    return torch.cat((pre, vid)).to(torch.int32).to(device).contiguous()


def make_shape(q: torch.Tensor, *, prefix_tokens: int, video_blocks: int, query_block_size: int,
               active: tuple[str, ...], native_prefix: bool, has_maxpool: bool,
               nvfp4_scales=(1.0, 1.0, 1.0)) -> native.Shape:
    return native.Shape(
        heads=q.size(2), head_dim=q.size(3), query_block=query_block_size, seq_tokens=q.size(1),
        prefix_tokens=prefix_tokens, video_blocks=video_blocks,
        has_nvfp4=int("nvfp4" in active), has_int8=int("int8" in active),
        has_fp16=int("fp16" in active), has_prefix_query_int8=int(native_prefix),
        has_maxpool=int(has_maxpool), input_is_bf16=int(q.dtype == torch.bfloat16),
        q_global_scale=nvfp4_scales[0], k_global_scale=nvfp4_scales[1],
        v_global_scale=nvfp4_scales[2],
    )


def sm100_ragged_attention(
    q_bshd: torch.Tensor,
    k_bshd: torch.Tensor,
    v_bshd: torch.Tensor,
    *,
    prefix_tokens: int,
    sparsity_ratio: float,
    retained_nvfp4_ratio: float,
    retained_int8_ratio: float,
    retained_fp16_ratio: float,
    video_shape: tuple[int, int, int],
    layer: int,
    query_block_size: int = 128,
    prefix_kv_precision: str = "int8",
    prefix_query_precision: str = "int8",
    maxpool_weight: float = 0.0,
    nvfp4_scales: tuple[float, float, float] = (1.0, 1.0, 1.0),
    return_parts: bool = False,
    profile_nvtx: bool = False,
    diag_jensen: bool = False,
    enable_anchors: bool = False,
):
    """Per-frame ragged Q64/Q128 routing and mixed-precision attention on sm_100a.

    ``enable_anchors`` selects the reference's experimental anchored routing: every pair of
    same-frame neighbouring blocks is kept, at the lowest active precision if the ranking dropped
    it (anemoi/layers/attention/mpa/executor.py:1151-1158, routing.py:190-203).

    ``diag_jensen`` selects the reference's experimental diag-Jensen draft map (second moments of
    the blocks added to the pooled logits, anemoi/layers/attention/mpa/executor.py:1105-1126); as
    there, it cannot be combined with the max-pool blend."""
    if any(type(flag) is not bool for flag in (profile_nvtx, diag_jensen, enable_anchors)):
        raise TypeError("profile_nvtx, diag_jensen and enable_anchors must be bool")
    if diag_jensen and maxpool_weight != 0.0:
        raise ValueError("maxpool_weight cannot be combined with diag_jensen")
    with _Range("anemoi.complete", profile_nvtx or _PROFILE_NVTX):
        return _ragged_attention(
            q_bshd, k_bshd, v_bshd, prefix_tokens=prefix_tokens, sparsity_ratio=sparsity_ratio,
            retained_nvfp4_ratio=retained_nvfp4_ratio, retained_int8_ratio=retained_int8_ratio,
            retained_fp16_ratio=retained_fp16_ratio, video_shape=video_shape, layer=layer,
            query_block_size=query_block_size, prefix_kv_precision=prefix_kv_precision,
            prefix_query_precision=prefix_query_precision, maxpool_weight=maxpool_weight,
            nvfp4_scales=nvfp4_scales, return_parts=return_parts,
            nvtx=profile_nvtx or _PROFILE_NVTX, diag_jensen=diag_jensen, enable_anchors=enable_anchors)


def _ragged_attention(q_bshd, k_bshd, v_bshd, *, prefix_tokens, sparsity_ratio, retained_nvfp4_ratio,
                      retained_int8_ratio, retained_fp16_ratio, video_shape, layer, query_block_size,
                      prefix_kv_precision, prefix_query_precision, maxpool_weight, nvfp4_scales,
                      return_parts, nvtx, diag_jensen=False, enable_anchors=False):
    if q_bshd.shape != k_bshd.shape or q_bshd.shape != v_bshd.shape:
        raise ValueError("Q/K/V must share [1,S,H,D], D in {64,128}")
    if (
        q_bshd.ndim != 4
        or q_bshd.size(0) != 1
        or q_bshd.size(-1) not in (64, 128)
        or q_bshd.dtype not in (torch.float16, torch.bfloat16)
        or k_bshd.dtype != q_bshd.dtype
        or v_bshd.dtype != q_bshd.dtype
        or q_bshd.device.type != "cuda"
        or k_bshd.device != q_bshd.device
        or v_bshd.device != q_bshd.device
    ):
        raise ValueError("Q/K/V must be same-dtype CUDA [1,S,H,D], D in {64,128}")
    if any(t.stride(3) != 1 or t.stride(1) % 8 or t.stride(2) % 8 or t.data_ptr() % 16
           for t in (q_bshd, k_bshd, v_bshd)):
        raise ValueError("Q/K/V need a contiguous head dimension and 16-byte aligned rows")
    if query_block_size not in (64, 128):
        raise ValueError("query_block_size must be 64 or 128")
    if isinstance(maxpool_weight, bool) or not isinstance(maxpool_weight, (int, float)):
        raise TypeError("maxpool_weight must be a real number")
    if not math.isfinite(float(maxpool_weight)) or not 0.0 <= float(maxpool_weight) <= 1.0:
        raise ValueError("maxpool_weight must be finite and in [0, 1]")
    if type(prefix_tokens) is not int or not 0 <= prefix_tokens < q_bshd.size(1):
        raise ValueError("prefix_tokens must be nonnegative and precede the video tokens")
    if (
        not isinstance(video_shape, tuple)
        or len(video_shape) != 3
        or any(type(v) is not int or v <= 0 for v in video_shape)
        or math.prod(video_shape) != q_bshd.size(1) - prefix_tokens
    ):
        raise ValueError("video_shape must match the post-prefix token count")

    device = q_bshd.device
    video = video_phases(retained_nvfp4_ratio, retained_int8_ratio, retained_fp16_ratio)
    if prefix_query_precision not in ("int8", "fp16"):
        raise ValueError("prefix_query_precision must be int8 or fp16")
    native_prefix = prefix_tokens > 0 and prefix_query_precision == "int8" and "int8" in video
    active, prefix_phase = resolve_phases(video, prefix_tokens, prefix_kv_precision)

    frames, height, width = video_shape
    current = torch.cuda.current_stream(device)
    side = _prefix_stream(device)
    prefix_out = None
    if prefix_tokens and not native_prefix:
        # dense attention of the prefix rows on the caller's tensors, as the reference does
        side.wait_stream(current)
        with torch.cuda.stream(side), _Range("anemoi.dense_prefix", nvtx):
            prefix_out = F.scaled_dot_product_attention(
                q_bshd[:, :prefix_tokens].permute(0, 2, 1, 3),
                k_bshd.permute(0, 2, 1, 3),
                v_bshd.permute(0, 2, 1, 3),
                dropout_p=0.0,
                is_causal=False,
            )[0].contiguous()

    layout = materialize_ragged_2d_layout(device, frames=frames, height=height, width=width,
                                          logical_block=query_block_size, enable_anchors=enable_anchors)
    blocks = layout.video_blocks
    shape = make_shape(q_bshd, prefix_tokens=prefix_tokens, video_blocks=blocks,
                       query_block_size=query_block_size, active=active,
                       native_prefix=native_prefix, has_maxpool=2 if diag_jensen else maxpool_weight != 0.0,
                       nvfp4_scales=nvfp4_scales)
    store = native.allocate_operands(shape, device)
    with _Stage("prepare"), _Range("anemoi.peripheral.prepare", nvtx):
        native.prepare(shape, q_bshd, k_bshd, v_bshd, layout.indices, layout.counts, store)
    valid_k = _valid_k(device, prefix_tokens, query_block_size, _counts_key(layout))
    status = _status_word(device)

    if native_prefix:
        side.wait_stream(current)
        with torch.cuda.stream(side):
            with _Stage("prefix_attention"), _Range("anemoi.dense_prefix", nvtx):
                prefix_out = native.prefix_attention(shape, store, valid_k, status)
            for t in store.buffers.values():
                if t is not None:
                    t.record_stream(side)
            valid_k.record_stream(side)
            status.record_stream(side)

    with _Range("anemoi.peripheral.draft_route_materialize", nvtx):
        with _Stage("draft"):
            prob = (native.draft_probability_jensen(shape, store) if diag_jensen
                    else native.draft_probability(shape, store, float(maxpool_weight)))
        n16, n8, n4 = route_counts(blocks * blocks, sparsity_ratio=float(sparsity_ratio),
                                   nvfp4_ratio=float(retained_nvfp4_ratio),
                                   int8_ratio=float(retained_int8_ratio),
                                   fp16_ratio=float(retained_fp16_ratio))
        phase_index = -1 if prefix_phase is None else PHASE_ORDER.index(prefix_phase)
        with _Stage("route"):
            lists = (native.route_anchored(shape, prob, n16, n8, n4, phase_index, layout.anchors, layout.anchor_ids)
                     if enable_anchors else native.route(shape, prob, n16, n8, n4, phase_index))
    with _Stage("attention"), _Range("anemoi.mpa_mainloop", nvtx):
        # Q64: two query blocks per CTA fill the 128-row MMA shape and walk the union of their lists
        pairs = native.pair_lists(shape, lists) if query_block_size == 64 and _PAIR_Q64 else None
        packed = native.attention(shape, store, lists, valid_k, status, pairs)

    current.wait_stream(side)
    if prefix_out is not None:
        prefix_out.record_stream(current)
    with _Stage("assemble"), _Range("anemoi.peripheral.assembly", nvtx):
        out = native.assemble(shape, prefix_out, packed, layout.inverse, lists.row_counts,
                              q_bshd.dtype)
    if return_parts:
        return out, dict(shape=shape, store=store, prob=prob, lists=lists, packed=packed,
                         prefix_out=prefix_out, valid_k=valid_k, budgets=(n16, n8, n4),
                         layout=layout, status=status)
    return out


def _counts_key(layout) -> tuple:
    key = getattr(layout, "_counts_key", None)
    if key is None:
        key = tuple(int(c) for c in layout.counts.cpu().tolist())
        object.__setattr__(layout, "_counts_key", key)
    return key


def _status_word(device: torch.device) -> torch.Tensor:
    """The device's sticky status word: allocated once, never cleared by a call, so the first
    give-up of a bounded wait stays on record until ``reset_status``."""
    device = torch.device(device)
    word = _STATUS.get(device)
    if word is None:
        word = _STATUS[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def last_status(device=None) -> int:
    """Synchronise and return the device's status word (0 = clean).

    A non-zero value means a bounded wait inside an attention kernel gave up in some call on
    this device since the last ``reset_status``; that call's output is not valid.  Callers that
    synchronise anyway (end of a request, end of a benchmark step) check it there.
    """
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _STATUS.get(torch.device(device))
    return 0 if word is None else int(word.item())


def reset_status(device=None) -> None:
    """Clear the device's status word (after a reported give-up has been handled)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _STATUS.get(torch.device(device))
    if word is not None:
        word.zero_()


def execute_ragged_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    prefix_tokens: int,
    video_shape: tuple[int, int, int],
    layer: int,
    query_block_size: int,
    sparsity_ratio: float,
    nvfp4_ratio: float,
    int8_ratio: float,
    fp16_ratio: float,
    prefix_kv_precision: str,
    prefix_query_precision: str,
    maxpool_weight: float = 0.0,
    nvfp4_scales: tuple[float, float, float] = (1.0, 1.0, 1.0),
) -> torch.Tensor:
    """Dispatch the stable routing configuration to the sm_100a backend."""
    if query.device.type != "cuda":
        raise RuntimeError("Anemoi attention requires an SM100 (B200) CUDA device")
    capability = tuple(torch.cuda.get_device_capability(query.device))
    if capability != (10, 0):
        raise RuntimeError("Anemoi attention requires SM100 (B200)")
    phases = video_phases(nvfp4_ratio, int8_ratio, fp16_ratio)
    if prefix_tokens and prefix_query_precision == "int8" and "int8" not in phases:
        raise RuntimeError("prefix-query INT8 requires an active INT8 phase")
    return sm100_ragged_attention(
        query,
        key,
        value,
        prefix_tokens=prefix_tokens,
        sparsity_ratio=sparsity_ratio,
        retained_nvfp4_ratio=nvfp4_ratio,
        retained_int8_ratio=int8_ratio,
        retained_fp16_ratio=fp16_ratio,
        video_shape=video_shape,
        layer=layer,
        query_block_size=query_block_size,
        prefix_kv_precision=prefix_kv_precision,
        prefix_query_precision=prefix_query_precision,
        maxpool_weight=maxpool_weight,
        nvfp4_scales=nvfp4_scales,
    )


__all__ = ["execute_ragged_attention", "sm100_ragged_attention", "last_status", "reset_status",
           "set_profile_nvtx"]
