"""TEST INFRASTRUCTURE - CPU restatement of the block-sparse mixed-precision attention.

One head at a time.  For every query block the 64-key stages of its list are
visited in the order NVFP4 -> INT8 -> FP16 with one shared online-softmax state
(base 2, running maximum ``m``, denominator ``d``, output ``O``), following
csrc/attention/cuda/sm120/q64_attention_phase_composer.inl:1-146 (NVFP4),
:506-932 (INT8) and :934-1331 (FP16) and the helpers in
csrc/attention/cuda/sm120/primitives/qattn/attn_utils.cuh:363-389 (key mask),
:470-561 (running maximum / rescale), :598-625 (denominator from unquantised P).

Quantisation points that are modelled exactly:
  NVFP4  scores from e2m1 codes x ue4m3 scales, score scale sigma*q_gs*k_gs;
         P -> e2m1(6 P) (q64_attention.cuh:581-636); V codes x scales x v_gs.
  INT8   exact integer scores, scale sigma*q_scale*k_scale[stage];
         P -> e4m3(P * 2**8.807) (attn_utils.cuh:28-30,581-596); V as E4M3 with
         a per-channel scale.
  FP16   fp16 operands, P -> fp16.
Accumulation is fp32 throughout (the reference uses fp16 accumulators inside a
stage for the INT8 and FP16 cells; that difference is inside the stated
output tolerance).  ``exp2`` is exact here, ``ex2.approx`` there.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package.
"""

from __future__ import annotations

import math

import numpy as np

from . import formats as F
from .prep import Geometry, HeadOperands

FP8_OFFSET = np.float32(8.807)
LOG2E = 1.4426950408889634


def _online_update(state, s_scaled, mask_cols, offset=np.float32(0.0)):
    """Advance (m, d, O-rescale) by one stage; returns P (with offset applied) and alpha."""
    m, d = state
    s_scaled = np.where(mask_cols[None, :], np.float32(-np.inf), s_scaled)
    m_new = np.maximum(m, s_scaled.max(axis=1))
    alpha = np.exp2(m - m_new).astype(np.float32)
    p = np.exp2(s_scaled - m_new[:, None] + offset).astype(np.float32)
    d_new = d * alpha + p.sum(axis=1, dtype=np.float32) * np.exp2(-offset)
    return (m_new, d_new.astype(np.float32)), p, alpha


def attention_rows(ops: HeadOperands, geo: Geometry, q_rows: slice, lists, *, head_dim: int,
                   q_scale_index: int | None, global_scales=(1.0, 1.0, 1.0),
                   prefix_query: bool = False) -> np.ndarray | None:
    """Attention output (fp16, [rows, D]) of one query block, or None for an empty list.

    ``lists`` = (nvfp4 stages, int8 stages, fp16 stages).  ``prefix_query`` selects
    the INT8 prefix-query operands (``ops.pq_i8``) instead of the video queries.
    """
    nv, i8, hi = lists
    if len(nv) + len(i8) + len(hi) == 0:
        return None
    valid_k = geo.valid_k()
    sigma = np.float32((1.0 / math.sqrt(head_dim)) * LOG2E)
    rows = q_rows.stop - q_rows.start
    m = np.full(rows, -5.0e6, dtype=np.float32)
    d = np.zeros(rows, dtype=np.float32)
    out = np.zeros((rows, head_dim), dtype=np.float32)
    cols = np.arange(64)
    gq, gk, gv = (np.float32(g) for g in global_scales)

    if len(nv):
        q = F.e2m1_decode(ops.q4[q_rows]).reshape(rows, -1, 16) * F.e4m3_decode(ops.q4_sf[q_rows])[..., None]
        q = q.reshape(rows, head_dim).astype(np.float32)
        c = np.float32(sigma * gq * gk)
        for st in nv:
            ks = slice(int(st) * 64, int(st) * 64 + 64)
            k = (F.e2m1_decode(ops.k4[ks]).reshape(64, -1, 16) * F.e4m3_decode(ops.k4_sf[ks])[..., None]).reshape(64, head_dim)
            s = (q @ k.T).astype(np.float32) * c
            (m, d), p, alpha = _online_update((m, d), s, cols >= valid_k[st])
            p_hat = F.e2m1_decode(F.e2m1_encode(p * np.float32(6.0))) / np.float32(6.0)
            vsf = F.e4m3_decode(ops.v4_sf[int(st) * 4 : int(st) * 4 + 4])          # [4, D]
            v = F.e2m1_decode(ops.v4[ks]).reshape(4, 16, head_dim) * vsf[:, None, :] * gv
            out = out * alpha[:, None] + (p_hat @ v.reshape(64, head_dim)).astype(np.float32)

    if len(i8):
        if prefix_query:
            q = ops.pq_i8[q_rows].astype(np.float32)
            qs = ops.pq_i8_scale[q_scale_index]
        else:
            q = ops.q_i8[q_rows].astype(np.float32)
            qs = ops.q_i8_scale[q_scale_index]
        for st in i8:
            ks = slice(int(st) * 64, int(st) * 64 + 64)
            s_int = (q @ ops.k_i8[ks].astype(np.float32).T).astype(np.float32)      # exact
            c = np.float32(sigma * np.float32(qs * ops.k_i8_scale[st]))
            (m, d), p, alpha = _online_update((m, d), s_int * c, cols >= valid_k[st], FP8_OFFSET)
            p_hat = F.e4m3_decode(F.e4m3_encode(p)) * np.exp2(-FP8_OFFSET)
            v = F.e4m3_decode(ops.v_e4m3[ks]) * ops.v_e4m3_scale[None, :]
            out = out * alpha[:, None] + (p_hat.astype(np.float32) @ v.astype(np.float32))

    if len(hi):
        q = ops.q16[q_rows].astype(np.float32)
        for st in hi:
            ks = slice(int(st) * 64, int(st) * 64 + 64)
            s = (q @ ops.k16[ks].astype(np.float32).T).astype(np.float32) * sigma
            (m, d), p, alpha = _online_update((m, d), s, cols >= valid_k[st])
            p_hat = p.astype(np.float16).astype(np.float32)
            out = out * alpha[:, None] + (p_hat @ ops.v16[ks].astype(np.float32))

    return (out / d[:, None]).astype(np.float32).astype(np.float16)


def dense_reference(q, k, v) -> np.ndarray:
    """softmax(Q K^T / sqrt(D)) V in float64 on [S, D] arrays of one head."""
    q, k, v = (np.asarray(t, dtype=np.float64) for t in (q, k, v))
    s = q @ k.T / math.sqrt(q.shape[-1])
    s = np.exp(s - s.max(axis=1, keepdims=True))
    return (s / s.sum(axis=1, keepdims=True)) @ v
