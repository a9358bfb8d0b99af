"""Producer-side fusions in front of ``anemoi_attention``.

``fused_qknorm_rope`` keeps the name, arguments and in-place behaviour of the reference's
Triton-backed function
(anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/fusions.py:243-274): RMS norm per
head, then rotary embedding of the leading ``rotary_dim`` channels, for ``(B, seq, heads, D)``.
It runs as one CUDA kernel of this library (``anemoi_sm100_qknorm_rope``); there is no eager
fallback.
"""

from __future__ import annotations

import torch

from . import native


def fused_qknorm_rope(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                      eps: float) -> torch.Tensor:
    """RMSNorm per head then partial rotary, in place, for ``(B, seq, heads, head_dim)``.

    ``cos``/``sin``: ``(seq, rotary_dim)`` (or ``(B, seq, rotary_dim)``), consumed in float32 at the
    precision they arrive in, as the reference's fused kernel does."""
    if x.ndim != 4:
        raise ValueError("x must be (B, seq, heads, head_dim)")
    batch, seq, heads, head_dim = x.shape
    rotary_dim = cos.shape[-1]
    if rotary_dim > head_dim or rotary_dim % 2 != 0:
        raise ValueError(f"fused qknorm+rope needs an even rotary_dim no wider than head_dim, "
                         f"got rotary_dim={rotary_dim}, head_dim={head_dim}")
    if rotary_dim % 16 != 0:
        raise ValueError("the sm_100a kernel pairs whole 8-channel vectors: rotary_dim must be a multiple of 16")
    for b in range(batch):
        c = cos[b] if cos.ndim == 3 else cos
        s = sin[b] if sin.ndim == 3 else sin
        native.qknorm_rope_(x[b], weight, c.reshape(seq, rotary_dim), s.reshape(seq, rotary_dim), eps)
    return x


__all__ = ["fused_qknorm_rope"]
