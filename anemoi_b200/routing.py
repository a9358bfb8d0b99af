"""Host-side routing arithmetic: retained-block budgets and phase resolution.

* ``route_counts`` - how many block pairs of a head are kept and how they split
  between the FP16, INT8 and NVFP4 cells (largest-remainder apportionment, ties
  to FP16, then INT8, then NVFP4).  Follows the reference's ``_route_counts``
  (anemoi/layers/attention/mpa/routing.py:23-61).
* ``resolve_phases`` - which precision phases a call executes and which phase
  carries the prefix keys.  Follows anemoi/layers/attention/mpa/executor.py:144-176
  and :958-975 for the three public cells (the MXFP8 cell is never public).
"""

from __future__ import annotations

import math

PHASE_ORDER = ("nvfp4", "int8", "fp16")


def route_counts(items: int, *, sparsity_ratio: float, nvfp4_ratio: float, int8_ratio: float,
                 fp16_ratio: float) -> tuple[int, int, int]:
    """Return the per-head budgets ``(fp16, int8, nvfp4)`` out of ``items`` block pairs."""
    if type(items) is not int or items <= 0:
        raise ValueError("items must be a positive integer")
    given = (sparsity_ratio, nvfp4_ratio, int8_ratio, fp16_ratio)
    for v in given:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
            raise TypeError("route ratios must be finite real scalars")
    drop, r4, r8, r16 = (float(v) for v in given)
    if not 0.0 <= drop < 1.0:
        raise ValueError("sparsity_ratio must be in [0, 1)")
    if min(r4, r8, r16) < 0.0:
        raise ValueError("precision ratios must be nonnegative")
    if not math.isclose(r4 + r8 + r16, 1.0, rel_tol=0.0, abs_tol=1.0e-6):
        raise ValueError("NVFP4/INT8/FP16 ratios must sum to one")
    kept = min(items, max(1, math.floor((1.0 - drop) * items + 0.5)))
    ideal = (kept * r16, kept * r8, kept * r4)
    share = [math.floor(v) for v in ideal]
    by_remainder = sorted(range(3), key=lambda i: (-(ideal[i] - share[i]), i))
    for i in by_remainder[: kept - sum(share)]:
        share[i] += 1
    return share[0], share[1], share[2]


def video_phases(nvfp4_ratio: float, int8_ratio: float, fp16_ratio: float) -> tuple[str, ...]:
    shares = (float(nvfp4_ratio), float(int8_ratio), float(fp16_ratio))
    if any(not math.isfinite(v) or v < 0.0 for v in shares) or not math.isclose(
        sum(shares), 1.0, abs_tol=1.0e-6
    ):
        raise ValueError("phase ratios must be nonnegative and sum to one")
    return tuple(name for name, v in zip(PHASE_ORDER, shares) if v > 0.0)


def resolve_phases(video: tuple[str, ...], prefix_tokens: int, prefix_kv_precision: str
                   ) -> tuple[tuple[str, ...], str | None]:
    """Return ``(active phases in execution order, prefix phase or None)``."""
    if not prefix_tokens:
        return video, None
    if prefix_kv_precision not in PHASE_ORDER:
        raise ValueError("prefix_kv_precision must be nvfp4, int8, or fp16")
    active = tuple(p for p in PHASE_ORDER if p in video or p == prefix_kv_precision)
    return active, prefix_kv_precision


__all__ = ["PHASE_ORDER", "route_counts", "video_phases", "resolve_phases"]
