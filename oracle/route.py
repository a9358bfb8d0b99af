"""TEST INFRASTRUCTURE - CPU restatement of Draft-Attention scoring and routing.

* ``draft_probability`` - pooled-QK row softmax, fp16 logits, optional mean/max
  blend (csrc/attention/cuda/sm120/h3_draft_probability.cu:131-222,427-465).  The
  reference leaves the accumulation order of the pooled product to cuBLAS and uses
  a fast-math ``expf``; here the arithmetic is fixed (sequential fp32 dot product,
  a fixed polynomial ``exp2`` evaluated with separately rounded multiplies and
  adds, a 32-lane strided row sum folded by an xor butterfly, IEEE division) so
  that the CUDA kernel can reproduce it bit for bit.  ``draft_probability_plain``
  is the unconstrained fp32 version the reference's tests compare against with
  ``atol=5e-4`` (tests/test_sm120_maxpool_cuda.py:106-127).
* ``route`` - stable global top-k per head, precision by rank, per-row lists
  ``[NVFP4 ids, INT8 ids, FP16 ids]`` each ascending
  (anemoi/layers/attention/mpa/routing.py:106-235,
  csrc/attention/cuda/sm120/h3_route_precision.cu:111-158,222-296).
* ``stage_lists`` - logical ids -> 64-key stage ids with the prefix stages
  spliced in front of the prefix phase (h3_route_precision.cu:298-369,
  anemoi/layers/attention/mpa/executor.py:233-297).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package.
"""

from __future__ import annotations

import math

import numpy as np

_LN2 = math.log(2.0)
EXP2_COEFFS = tuple(np.float32(_LN2 ** k / math.factorial(k)) for k in range(8))
LOG2E = np.float32(1.4426950408889634)


def exp_canonical(t: np.ndarray) -> np.ndarray:
    """e**t for t <= 0 in fp32 with a fixed operation sequence."""
    t = np.asarray(t, dtype=np.float32)
    y = np.maximum((t * LOG2E).astype(np.float32), np.float32(-125.0))
    n = np.rint(y).astype(np.float32)
    f = (y - n).astype(np.float32)
    p = np.full_like(f, EXP2_COEFFS[7])
    for c in EXP2_COEFFS[6::-1]:
        p = ((p * f).astype(np.float32) + c).astype(np.float32)
    return np.ldexp(p, n.astype(np.int32)).astype(np.float32)


def _logits16(qp: np.ndarray, kp: np.ndarray) -> np.ndarray:
    d = qp.shape[-1]
    q = qp.astype(np.float32)
    k = kp.astype(np.float32)
    acc = np.zeros((q.shape[0], k.shape[0]), dtype=np.float32)
    for c in range(d):
        acc = acc + (q[:, c : c + 1] * k[None, :, c]).astype(np.float32)
    scale = np.float32(1.0 / math.sqrt(d))
    return (acc * scale).astype(np.float32).astype(np.float16)


def _row_sum32(e: np.ndarray) -> np.ndarray:
    rows, cols = e.shape
    padded = np.zeros((rows, (cols + 31) // 32 * 32), dtype=np.float32)
    padded[:, :cols] = e
    lanes = padded.reshape(rows, -1, 32)
    part = np.zeros((rows, 32), dtype=np.float32)
    for c in range(lanes.shape[1]):
        part = part + lanes[:, c]
    lane = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        part = part + part[:, lane ^ off]
    return part[:, 0]


def _softmax_canonical(logit16: np.ndarray) -> np.ndarray:
    x = logit16.astype(np.float32)
    m = x.max(axis=1, keepdims=True)
    e = exp_canonical(x - m)
    inv = (np.float32(1.0) / _row_sum32(e)).astype(np.float32)
    return (e * inv[:, None]).astype(np.float32)


def draft_probability(q_pool, k_pool, q_max=None, k_max=None, maxpool_weight: float = 0.0):
    """[R, D] fp16 pools of one head -> [R, R] fp16 probability (canonical arithmetic)."""
    w = float(maxpool_weight)
    if w == 0.0 or q_max is None:
        return _softmax_canonical(_logits16(q_pool, k_pool)).astype(np.float16)
    if w == 1.0:
        return _softmax_canonical(_logits16(q_max, k_max)).astype(np.float16)
    pm = _softmax_canonical(_logits16(q_pool, k_pool))
    px = _softmax_canonical(_logits16(q_max, k_max))
    w32 = np.float32(w)
    a = ((np.float32(1.0) - w32) * pm).astype(np.float32)
    b = (w32 * px).astype(np.float32)
    return (a + b).astype(np.float32).astype(np.float16)


def _dots32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """fp32 FMA chain over the channels in ascending order (a, b fp32 [rows, D] / [cols, D])."""
    acc = np.zeros((a.shape[0], b.shape[0]), dtype=np.float32)
    for c in range(a.shape[1]):
        acc = (acc.astype(np.float64) + a[:, c : c + 1].astype(np.float64) * b[None, :, c].astype(np.float64)
               ).astype(np.float32)
    return acc


def draft_probability_jensen(q_pool, k_pool, q_second, k_second):
    """Diag-Jensen draft map of one head (reference: anemoi/layers/attention/mpa/routing.py:87-103):
    logits = q.k/sqrt(D) + 0.5 * max((q2.k2 - (q*q).(k*k)) / D, 0) in fp32 (not rounded to fp16),
    row softmax, fp16.  Canonical arithmetic: every dot product is an FMA chain over ascending
    channels (the inputs of the third one are the fp32 squares of the pools), the logit is
    fma(0.5, max((v - w) * (1/D), 0), round(qk * (1/sqrt(D)))), the softmax the canonical one."""
    d = q_pool.shape[-1]
    q, k = q_pool.astype(np.float32), k_pool.astype(np.float32)
    base = (_dots32(q, k) * np.float32(1.0 / math.sqrt(d))).astype(np.float32)
    v = _dots32(q_second.astype(np.float32), k_second.astype(np.float32))
    w = _dots32((q * q).astype(np.float32), (k * k).astype(np.float32))
    t = np.maximum(((v - w).astype(np.float32) * np.float32(1.0 / d)).astype(np.float32), np.float32(0.0))
    logits = (base.astype(np.float64) + 0.5 * t.astype(np.float64)).astype(np.float32)
    m = logits.max(axis=1, keepdims=True)
    e = exp_canonical((logits - m).astype(np.float32))
    inv = (np.float32(1.0) / _row_sum32(e)).astype(np.float32)
    return (e * inv[:, None]).astype(np.float32).astype(np.float16)


def draft_probability_plain(q_pool, k_pool, q_max=None, k_max=None, maxpool_weight: float = 0.0):
    """Reference-style arithmetic: fp32 matmul, fp16 logits, fp32 softmax, fp16 result."""
    def soft(a, b):
        z = (a.astype(np.float32) @ b.astype(np.float32).T) * np.float32(1.0 / math.sqrt(a.shape[-1]))
        z = z.astype(np.float16).astype(np.float32)
        z = np.exp(z - z.max(axis=1, keepdims=True))
        return z / z.sum(axis=1, keepdims=True)
    w = float(maxpool_weight)
    if w == 0.0 or q_max is None:
        return soft(q_pool, k_pool).astype(np.float16)
    if w == 1.0:
        return soft(q_max, k_max).astype(np.float16)
    return ((1.0 - w) * soft(q_pool, k_pool) + w * soft(q_max, k_max)).astype(np.float16)


def budgets(items: int, sparsity: float, r4: float, r8: float, r16: float):
    """(fp16, int8, nvfp4) retained pairs per head (routing.py:53-61 of the reference)."""
    kept = min(items, max(1, math.floor((1.0 - sparsity) * items + 0.5)))
    ideal = (kept * r16, kept * r8, kept * r4)
    share = [math.floor(v) for v in ideal]
    order = sorted(range(3), key=lambda i: (-(ideal[i] - share[i]), i))
    for i in order[: kept - sum(share)]:
        share[i] += 1
    return tuple(share)


def route(prob16: np.ndarray, n16: int, n8: int, n4: int, anchors: np.ndarray | None = None):
    """One head: [R, R] fp16 -> (ids [R, R] int32, low, middle, high counts [R] int32).

    Pairs are ranked by descending probability, ties by ascending flat index
    ``row * R + col``; ranks ``< n16`` are FP16 (code 3), the next ``n8`` INT8
    (code 2), the next ``n4`` NVFP4 (code 1).  Row lists hold the NVFP4 columns,
    then INT8, then FP16, each ascending; unused tail entries are 0.

    ``anchors`` ([R, R] bool, the reference's experimental anchor variant,
    anemoi/layers/attention/mpa/routing.py:190-203): anchor pairs the ranking dropped are
    forced into the lowest active precision, and as many of the lowest-ranked pairs of that
    precision that are not anchors are dropped instead.
    """
    r = prob16.shape[0]
    key = (prob16.astype(np.float16).view(np.uint16).astype(np.int64) & 0x7FFF).reshape(-1)
    order = np.argsort(-key, kind="stable")
    code = np.zeros(r * r, dtype=np.uint8)
    code[order[:n16]] = 3
    code[order[n16 : n16 + n8]] = 2
    code[order[n16 + n8 : n16 + n8 + n4]] = 1
    if anchors is not None:
        lowest_code, lowest_count = (1, n4) if n4 else ((2, n8) if n8 else (3, n16))
        retained = n16 + n8 + n4
        mask = np.asarray(anchors, dtype=bool).reshape(-1)
        missing = mask & (code == 0)
        low_ids = order[retained - lowest_count : retained]
        ordinary_reversed = ~mask[low_ids][::-1]
        evict = (ordinary_reversed & (np.cumsum(ordinary_reversed) <= int(missing.sum())))[::-1]
        code[low_ids[evict]] = 0
        code[missing] = lowest_code
    code = code.reshape(r, r)
    ids = np.zeros((r, r), dtype=np.int32)
    counts = np.zeros((3, r), dtype=np.int32)
    for i in range(r):
        parts = [np.nonzero(code[i] == c)[0] for c in (1, 2, 3)]
        row = np.concatenate(parts)
        ids[i, : row.size] = row
        counts[:, i] = [p.size for p in parts]
    return ids, counts[0], counts[1], counts[2]


def stage_lists(ids, low, mid, high, *, query_block: int, prefix_stages: int,
                prefix_phase: str | None):
    """Per row: list of 64-key stage ids per phase, in execution order.

    Returns ``[(nvfp4 stages, int8 stages, fp16 stages)]`` per row.  A logical
    block ``c`` maps to stages ``p + c*f .. p + c*f + f-1`` (``f = query_block/64``);
    the prefix stages ``0..p-1`` are placed at the front of ``prefix_phase``.
    """
    f = query_block // 64
    rows = []
    for i in range(ids.shape[0]):
        a, b, c = int(low[i]), int(mid[i]), int(high[i])
        seg = [ids[i, :a], ids[i, a : a + b], ids[i, a + b : a + b + c]]
        out = []
        for name, logical in zip(("nvfp4", "int8", "fp16"), seg):
            st = (prefix_stages + logical.astype(np.int64)[:, None] * f + np.arange(f)[None, :]).reshape(-1)
            if prefix_phase == name:
                st = np.concatenate((np.arange(prefix_stages, dtype=np.int64), st))
            out.append(st.astype(np.int32))
        rows.append(tuple(out))
    return rows
