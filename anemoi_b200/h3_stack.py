"""A random-init stand-in for the MiniMax-H3 DiT block stack: the harness that drives the sparse
attention path and its Ulysses exchange the way the reference's launcher does for one denoising
step.  It is NOT a reproduction of the real model (whose definition, config and checkpoint are
external to the reference repository); only what the reference fixes is used:

  * 56 heads of 128 channels (attention width 7,168), residual width 5,376, 50 blocks,
    separate ``to_q / to_k / to_v`` projections, RMS qk-norm with a weight, partial rotary
    embedding, ``to_out``, a SwiGLU feed-forward and 6-way adaLN modulation
    (anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/ulysses_custom.py:217-277,
    fusions.py:1-23, README.md:132);
  * sequence-sharded everywhere except the attention, which is head-sharded between one packed
    QKV all-to-all and one output all-to-all (ulysses_custom.py:107-165);
  * the attention callable is ``H3MPAAttention`` (dense for the first layers of a step, sparse
    mixed-precision elsewhere, anemoi/models/minimax_h3/mpa_attention.py:611-620).
Assumed, because the reference does not state them: feed-forward width 14,336 and 64 rotary
channels.  The projections are plain library GEMMs (model glue); the producer fusion, the
exchange relayouts and the attention are this library's kernels.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import ulysses


@dataclass(frozen=True)
class H3StackConfig:
    width: int = 5376
    heads: int = 56
    head_dim: int = 128
    ffn_width: int = 14336
    rotary_dim: int = 64
    layers: int = 50
    eps: float = 1e-6

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim


class H3BlockStack:
    """Weights of ``layers`` blocks on one device and the forward of one denoising step over a
    sequence shard ``x`` ``[rows, width]``."""

    def __init__(self, config: H3StackConfig, device, dtype=torch.bfloat16, seed: int = 0,
                 shared_weights: bool = False):
        self.config = config
        c = config
        gen = torch.Generator(device=device).manual_seed(seed)

        def weight(rows, cols):
            return (torch.randn(rows, cols, generator=gen, device=device) * rows ** -0.5).to(dtype)

        def block():
            return dict(wq=weight(c.width, c.inner), wk=weight(c.width, c.inner), wv=weight(c.width, c.inner),
                        wo=weight(c.inner, c.width), w1=weight(c.width, c.ffn_width),
                        w3=weight(c.width, c.ffn_width), w2=weight(c.ffn_width, c.width),
                        qn=torch.ones(c.head_dim, device=device, dtype=dtype),
                        kn=torch.ones(c.head_dim, device=device, dtype=dtype),
                        mod=(torch.randn(6, c.width, generator=gen, device=device) * 0.1).to(dtype))

        first = block()
        self.blocks = [first if shared_weights else (first if i == 0 else block()) for i in range(c.layers)]

    @staticmethod
    def _norm(x: torch.Tensor, eps: float) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)

    def step(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, attention_fn, *, norm_rope,
             group=None, pack=None, merge=None, on_attention=None, exchange=None,
             fuse_producer: bool = False) -> torch.Tensor:
        """One denoising step: every block in turn.  ``attention_fn(q, k, v)`` takes the
        head-sharded ``[S, h, D]`` tensors of a layer; ``norm_rope(x, weight, cos, sin, eps)`` is the
        producer fusion (in place, ``[1, rows, heads, D]``); ``on_attention(begin)`` is called with
        True / False around the exchange + attention of each layer (timing hook); ``exchange`` is an
        optional ``ulysses.PeerExchange`` (stores into the peers' memory instead of all-to-alls);
        with ``fuse_producer`` the producer fusion is folded into that exchange's stores."""
        c = self.config
        rows = x.size(0)
        kw = {}
        if pack is not None:
            kw.update(pack=pack, merge=merge)
        if exchange is not None:
            kw.update(exchange=exchange)
        for blk in self.blocks:
            shift1, scale1, gate1, shift2, scale2, gate2 = blk["mod"]
            h = self._norm(x, c.eps) * (1 + scale1) + shift1
            q = (h @ blk["wq"]).view(1, rows, c.heads, c.head_dim)
            k = (h @ blk["wk"]).view(1, rows, c.heads, c.head_dim)
            v = (h @ blk["wv"]).view(1, rows, c.heads, c.head_dim)
            producer = {}
            if exchange is not None and fuse_producer:
                # qk-norm + rotary ride on the exchange's stores: no in-place pass over q and k
                producer = dict(producer=(blk["qn"], blk["kn"], cos, sin, c.eps))
            else:
                norm_rope(q, blk["qn"], cos, sin, c.eps)
                norm_rope(k, blk["kn"], cos, sin, c.eps)
            if on_attention is not None:
                on_attention(True)
            attn = ulysses.ulysses_attention(
                q, k, v, lambda qh, kh, vh: attention_fn(qh[0], kh[0], vh[0]).unsqueeze(0), group, **kw,
                **producer)
            if on_attention is not None:
                on_attention(False)
            x = x + gate1 * (attn.reshape(rows, c.inner) @ blk["wo"])
            h = self._norm(x, c.eps) * (1 + scale2) + shift2
            x = x + gate2 * ((F.silu(h @ blk["w1"]) * (h @ blk["w3"])) @ blk["w2"])
        return x


__all__ = ["H3BlockStack", "H3StackConfig"]
