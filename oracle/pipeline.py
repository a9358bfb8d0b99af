"""TEST INFRASTRUCTURE - the whole ``anemoi_attention`` call restated on the CPU.

Order of work per head (anemoi/layers/attention/mpa/executor.py:876-1224 of the
reference): slot tables -> gather / pool / quantise -> draft probability ->
budgets and global top-k -> stage lists with the prefix splice -> phases per
query block -> prefix rows -> inverse scatter into ``[1, S, H, D]``
(csrc/attention/cuda/sm89/output_assembly.cu:219-305: rows whose three counts
are all zero become +0).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package.
"""

from __future__ import annotations

import math

import numpy as np

from . import attention as A
from . import prep as P
from . import route as R

PHASES = ("nvfp4", "int8", "fp16")


def resolve(nvfp4_ratio, int8_ratio, fp16_ratio, prefix_tokens, prefix_kv_precision):
    video = tuple(n for n, r in zip(PHASES, (nvfp4_ratio, int8_ratio, fp16_ratio)) if r > 0.0)
    if not prefix_tokens:
        return video, video, None
    active = tuple(n for n in PHASES if n in video or n == prefix_kv_precision)
    return video, active, prefix_kv_precision


def head_attention(q, k, v, geo: P.Geometry, *, sparsity, ratios, prefix_kv_precision="int8",
                   prefix_query_precision="int8", maxpool_weight=0.0,
                   global_scales=(1.0, 1.0, 1.0), return_parts=False, diag_jensen=False):
    """One head: ``q, k, v`` [S, D] -> fp16 [S, D] in raster order."""
    r4, r8, r16 = ratios
    d = q.shape[-1]
    video, active, prefix_phase = resolve(r4, r8, r16, geo.prefix_tokens, prefix_kv_precision)
    native_prefix = geo.prefix_tokens > 0 and prefix_query_precision == "int8" and "int8" in video
    ops = P.prepare_head(q, k, v, geo, has_nvfp4="nvfp4" in active, has_int8="int8" in active,
                         has_prefix_query_int8=native_prefix, has_maxpool=maxpool_weight != 0.0,
                         global_scales=global_scales, second_moments=diag_jensen)
    if diag_jensen:
        prob = R.draft_probability_jensen(ops.q_pool, ops.k_pool, ops.q_max, ops.k_max)
    else:
        prob = R.draft_probability(ops.q_pool, ops.k_pool, ops.q_max, ops.k_max, maxpool_weight)
    rr = geo.video_blocks
    n16, n8, n4 = R.budgets(rr * rr, sparsity, r4, r8, r16)
    ids, low, mid, high = R.route(prob, n16, n8, n4)
    lists = R.stage_lists(ids, low, mid, high, query_block=geo.query_block,
                          prefix_stages=geo.prefix_stages, prefix_phase=prefix_phase)
    qb = geo.query_block
    s_total = geo.prefix_tokens + geo.inverse.shape[0]
    packed = np.zeros((rr * qb, d), dtype=np.float16)
    for i in range(rr):
        o = A.attention_rows(ops, geo, slice(i * qb, (i + 1) * qb), lists[i], head_dim=d,
                             q_scale_index=i, global_scales=global_scales)
        if o is not None:
            packed[i * qb : (i + 1) * qb] = o
    out = np.zeros((s_total, d), dtype=np.float16)
    out[geo.prefix_tokens :] = packed[geo.inverse]
    if geo.prefix_tokens:
        if native_prefix:
            every = np.arange(geo.stages, dtype=np.int32)
            for t in range(math.ceil(geo.prefix_tokens / qb)):
                o = A.attention_rows(ops, geo, slice(t * qb, (t + 1) * qb), ((), every, ()),
                                     head_dim=d, q_scale_index=t, prefix_query=True)
                lo, hi = t * qb, min((t + 1) * qb, geo.prefix_tokens)
                out[lo:hi] = o[: hi - lo]
        else:
            qf = np.asarray(q, dtype=np.float32) if not hasattr(q, "detach") else q.detach().float().numpy()
            kf = np.asarray(k, dtype=np.float32) if not hasattr(k, "detach") else k.detach().float().numpy()
            vf = np.asarray(v, dtype=np.float32) if not hasattr(v, "detach") else v.detach().float().numpy()
            out[: geo.prefix_tokens] = A.dense_reference(qf[: geo.prefix_tokens], kf, vf).astype(np.float16)
    if return_parts:
        return out, dict(ops=ops, prob=prob, ids=ids, low=low, mid=mid, high=high, lists=lists,
                         packed=packed, budgets=(n16, n8, n4))
    return out
