"""TEST INFRASTRUCTURE - CPU restatement of gather / pool / quantise (one head at a time).

Follows the reference's fused preparation kernels
(csrc/attention/cuda/sm120/q128_microscaling_preparation.cu):
  * narrow + pack, zero padding ........ :220-232, :362-394
  * mean / max pools ................... :375-381, :511-520
  * INT8 Q/K (scale = amax/127 + 1e-7,
    round half away from zero) ......... :442-509
  * V as E4M3 with a per-(head, channel)
    scale amax/2.25 .................... :686-803
  * NVFP4 Q/K rows and V token groups .. :396-425, :605-640
Division is IEEE fp32 (the reference compiles with fast-math; its own tests pin
the codes with IEEE division, tests/test_sm120_d64_cuda.py:187-193).

All results are in natural order: packed rows (block-major slots) x channels.
Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import formats as F


@dataclass
class Geometry:
    """Slot tables of a video layout (same contents as the product's RaggedLayout)."""

    indices: np.ndarray      # [R*QB] raster token per slot (0 for padding)
    slot_valid: np.ndarray   # [R*QB] bool
    counts: np.ndarray       # [R]
    inverse: np.ndarray      # [video tokens] -> slot
    query_block: int
    prefix_tokens: int

    @property
    def video_blocks(self) -> int:
        return int(self.counts.shape[0])

    @property
    def prefix_stages(self) -> int:
        return math.ceil(self.prefix_tokens / 64)

    @property
    def stages(self) -> int:
        return self.prefix_stages + self.video_blocks * (self.query_block // 64)

    def valid_k(self) -> np.ndarray:
        """Real keys per 64-key stage (executor.py:334-342,1052-1067)."""
        p = self.prefix_stages
        pre = np.clip(self.prefix_tokens - 64 * np.arange(p), 0, 64)
        c = self.counts.astype(np.int64)
        if self.query_block == 128:
            vid = np.stack((np.minimum(c, 64), np.maximum(c - 64, 0)), axis=-1).reshape(-1)
        else:
            vid = c
        return np.concatenate((pre, vid)).astype(np.int32)


def make_geometry(blocks, frames: int, height: int, width: int, query_block: int,
                  prefix_tokens: int) -> Geometry:
    """Build slot tables from per-frame blocks (layout.py:37-67 of the reference)."""
    per_frame = len(blocks)
    frame_tokens = height * width
    local = np.zeros((per_frame, query_block), dtype=np.int64)
    valid = np.zeros((per_frame, query_block), dtype=bool)
    for b, block in enumerate(blocks):
        local[b, : len(block)] = block
        valid[b, : len(block)] = True
    offsets = (np.arange(frames, dtype=np.int64) * frame_tokens)[:, None, None]
    indices = ((local[None] + offsets) * valid[None]).reshape(-1)
    slot_valid = np.broadcast_to(valid[None], (frames, per_frame, query_block)).reshape(-1)
    counts = np.tile(np.array([len(b) for b in blocks], dtype=np.int32), frames)
    inverse = np.empty(frames * frame_tokens, dtype=np.int64)
    inverse[indices[slot_valid]] = np.arange(indices.size)[slot_valid]
    return Geometry(indices, slot_valid.copy(), counts, inverse, query_block, prefix_tokens)


def pack_rows(x16: np.ndarray, geo: Geometry, with_prefix: bool) -> np.ndarray:
    """[S, D] fp16 of one head -> packed rows. Prefix rows (padded to 64) come first."""
    p = geo.prefix_tokens
    video = np.where(geo.slot_valid[:, None], x16[p:][geo.indices], np.float16(0))
    if not with_prefix:
        return video
    cap = geo.prefix_stages * 64
    pre = np.zeros((cap, x16.shape[1]), dtype=np.float16)
    pre[:p] = x16[:p]
    return np.concatenate((pre, video), axis=0)


def pack_prefix_queries(x16: np.ndarray, geo: Geometry) -> np.ndarray:
    """Prefix query rows padded with zeros to a multiple of the query block."""
    qb = geo.query_block
    cap = math.ceil(geo.prefix_tokens / qb) * qb
    out = np.zeros((cap, x16.shape[1]), dtype=np.float16)
    out[: geo.prefix_tokens] = x16[: geo.prefix_tokens]
    return out


def mean_pool(video_rows: np.ndarray, geo: Geometry) -> np.ndarray:
    """fp16( (sum over the block's slots in slot order, fp32) / real count )."""
    qb = geo.query_block
    blocks = video_rows.reshape(-1, qb, video_rows.shape[-1]).astype(np.float32)
    acc = np.zeros((blocks.shape[0], blocks.shape[2]), dtype=np.float32)
    for s in range(qb):
        acc = acc + blocks[:, s]
    return (acc / geo.counts.astype(np.float32)[:, None]).astype(np.float16)


def max_pool(video_rows: np.ndarray, geo: Geometry) -> np.ndarray:
    qb = geo.query_block
    blocks = video_rows.reshape(-1, qb, video_rows.shape[-1]).astype(np.float32)
    valid = np.arange(qb)[None, :, None] < geo.counts[:, None, None]
    return np.where(valid, blocks, -np.inf).max(axis=1).astype(np.float16)


def second_moment_pool(video_rows: np.ndarray, geo: Geometry) -> np.ndarray:
    """fp16( (sum of squares over the block's slots in slot order, one FMA per slot, fp32) / real
    count ): the per-channel second moments of the diag-Jensen draft map (reference:
    anemoi/layers/attention/mpa/executor.py:1105-1124)."""
    qb = geo.query_block
    blocks = video_rows.reshape(-1, qb, video_rows.shape[-1]).astype(np.float64)
    acc = np.zeros((blocks.shape[0], blocks.shape[2]), dtype=np.float32)
    for s in range(qb):
        # fma(x, x, acc): the square of an fp16 value is exact in fp64, one rounding to fp32
        acc = (acc.astype(np.float64) + blocks[:, s] * blocks[:, s]).astype(np.float32)
    return (acc / geo.counts.astype(np.float32)[:, None]).astype(np.float16)


def int8_quantise(rows: np.ndarray, group_rows: int):
    """Symmetric INT8 per group of ``group_rows`` rows x all channels."""
    x = rows.astype(np.float32).reshape(-1, group_rows, rows.shape[-1])
    amax = np.abs(x).max(axis=(1, 2))
    scale = (amax / np.float32(127.0) + np.float32(1.0e-7)).astype(np.float32)
    t = (x / scale[:, None, None]).astype(np.float32)
    t = t + np.where(t >= 0, np.float32(0.5), np.float32(-0.5))
    codes = np.trunc(t).astype(np.int32).astype(np.int8)
    return codes.reshape(rows.shape), scale


def v_e4m3_quantise(v_rows: np.ndarray):
    """Per-channel E4M3 of V: code = e4m3(v * (2.25/amax)), scale = amax/2.25."""
    v = v_rows.astype(np.float32)
    amax = np.abs(v).max(axis=0)
    with np.errstate(divide="ignore"):
        recip = np.where(amax == 0, np.float32(0), np.float32(2.25) / amax).astype(np.float32)
    codes = F.e4m3_encode((v * recip[None, :]).astype(np.float32))
    codes = np.where(recip[None, :] == 0, 0, codes).astype(np.uint8)
    scale = (amax / np.float32(2.25)).astype(np.float32)
    return codes, scale


@dataclass
class HeadOperands:
    """Everything the attention phases of one head consume, in natural order."""

    q16: np.ndarray; k16: np.ndarray; v16: np.ndarray            # packed fp16 rows
    q_pool: np.ndarray; k_pool: np.ndarray
    q_max: np.ndarray | None; k_max: np.ndarray | None
    q_i8: np.ndarray | None = None; q_i8_scale: np.ndarray | None = None
    k_i8: np.ndarray | None = None; k_i8_scale: np.ndarray | None = None
    v_e4m3: np.ndarray | None = None; v_e4m3_scale: np.ndarray | None = None
    pq_i8: np.ndarray | None = None; pq_i8_scale: np.ndarray | None = None
    q4: np.ndarray | None = None; q4_sf: np.ndarray | None = None
    k4: np.ndarray | None = None; k4_sf: np.ndarray | None = None
    v4: np.ndarray | None = None; v4_sf: np.ndarray | None = None   # v4_sf: [Kp/16, D]


def prepare_head(q, k, v, geo: Geometry, *, has_nvfp4: bool, has_int8: bool,
                 has_prefix_query_int8: bool, has_maxpool: bool,
                 global_scales=(1.0, 1.0, 1.0), second_moments: bool = False) -> HeadOperands:
    """``q, k, v``: [S, D] of one head (any float dtype; narrowed to fp16 first)."""
    q16, k16, v16 = (F.narrow_to_fp16(t) for t in (q, k, v))
    qp = pack_rows(q16, geo, with_prefix=False)
    kp = pack_rows(k16, geo, with_prefix=True)
    vp = pack_rows(v16, geo, with_prefix=True)
    cap = geo.prefix_stages * 64
    ops = HeadOperands(
        q16=qp, k16=kp, v16=vp,
        q_pool=mean_pool(qp, geo), k_pool=mean_pool(kp[cap:], geo),
        q_max=max_pool(qp, geo) if has_maxpool else None,
        k_max=max_pool(kp[cap:], geo) if has_maxpool else None,
    )
    if second_moments:      # they travel in the max-pool slots (the two modes exclude each other)
        ops.q_max = second_moment_pool(qp, geo)
        ops.k_max = second_moment_pool(kp[cap:], geo)
    if has_int8:
        ops.q_i8, ops.q_i8_scale = int8_quantise(qp, geo.query_block)
        ops.k_i8, ops.k_i8_scale = int8_quantise(kp, 64)
        ops.v_e4m3, ops.v_e4m3_scale = v_e4m3_quantise(vp)
        if has_prefix_query_int8 and geo.prefix_tokens:
            ops.pq_i8, ops.pq_i8_scale = int8_quantise(pack_prefix_queries(q16, geo),
                                                       geo.query_block)
    if has_nvfp4:
        gq, gk, gv = global_scales
        ops.q4, ops.q4_sf = F.nvfp4_quantise(qp, gq, axis=-1)
        ops.k4, ops.k4_sf = F.nvfp4_quantise(kp, gk, axis=-1)
        ops.v4, ops.v4_sf = F.nvfp4_quantise(vp, gv, axis=0)   # groups of 16 tokens
    return ops
