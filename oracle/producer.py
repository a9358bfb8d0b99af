"""CPU restatement of the producer fusion (per-head RMS norm + partial rotary) in the canonical
arithmetic of ``csrc/producer.cu`` -- test infrastructure only.

Formula of the reference's fused kernel
(anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/fusions.py:208-274); the
summation order (8-channel sequential FMA chain per lane, xor butterfly over the D/8 lanes),
the IEEE reciprocal square root and the single FMA of the rotation are this library's choices,
restated here step by step in float32 so that the GPU result can be compared bit for bit.
"""

from __future__ import annotations

import numpy as np
import torch

F32 = np.float32


def _fma(a, b, c):
    """float32 fused multiply-add: exact product and sum in float64, one rounding."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(F32)


def qknorm_rope(x: torch.Tensor, weight: torch.Tensor, cos: np.ndarray, sin: np.ndarray, eps: float) -> torch.Tensor:
    """``x`` [tokens, heads, D] fp16/bf16, ``weight`` [D] same dtype, ``cos/sin`` [tokens, rotary] float32."""
    tokens, heads, d = x.shape
    rotary = cos.shape[-1]
    half = rotary // 2
    v = x.float().numpy().astype(F32)
    w = weight.float().numpy().astype(F32)
    lanes = d // 8
    part = np.zeros((tokens, heads, lanes), dtype=F32)
    for i in range(8):
        vi = v.reshape(tokens, heads, lanes, 8)[..., i]
        part = _fma(vi, vi, part)
    off = lanes // 2
    idx = np.arange(lanes)
    while off > 0:
        part = (part + part[..., idx ^ off]).astype(F32)
        off //= 2
    total = part[..., 0]
    r = (F32(1.0) / np.sqrt(((total / F32(d)).astype(F32) + F32(eps)).astype(F32)).astype(F32)).astype(F32)
    n = ((v * r[..., None]).astype(F32) * w).astype(F32)
    out = n.copy()
    if rotary:
        c = cos.astype(F32)[:, None, :]
        s = sin.astype(F32)[:, None, :]
        first, second = n[..., :half], n[..., half:rotary]
        rot = np.concatenate((-second, first), axis=-1)
        out[..., :rotary] = _fma(rot, np.broadcast_to(s, rot.shape), (n[..., :rotary] * c).astype(F32))
    return torch.from_numpy(out).to(x.dtype)


def eager_reference(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, eps: float):
    """Plain float32 statement of the same formula (no fixed summation order), for tolerance checks."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    rotary = cos.shape[-1]
    a, b = n[..., : rotary // 2], n[..., rotary // 2 : rotary]
    rot = torch.cat((-b, a), dim=-1)
    out = n.clone()
    out[..., :rotary] = n[..., :rotary] * cos[:, None, :].float() + rot * sin[:, None, :].float()
    return out
