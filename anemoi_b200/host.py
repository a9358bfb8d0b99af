"""``anemoi_attention`` for callers whose Q/K/V live in pinned host memory.

The reference's operator takes CUDA tensors (anemoi/layers/attention/api.py:134-194); a caller
that holds its activations on the host pays the copies in front of and behind it, one after
the other.  Heads are independent on this path (pools, routing budget, lists and attention are
all per head), so this entry walks the heads in groups on three streams: while group ``g`` runs
the layer, group ``g+1`` is copied in and group ``g-1`` is copied out.  Each group and tensor is
ONE strided copy.  The result is bit-identical to a single call on all heads.

With ``sharded=True`` (several GPUs of one node, one process each) every rank holds its rows of
the sequence on its host; each head group is copied in, exchanged to head-sharded form by stores
into the peers' memory (``ulysses.PeerExchange``), attended, exchanged back and copied out, so
the host copies of one group also run under the exchange and attention of another.
"""

from __future__ import annotations

import torch

from . import native
from .api import NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention


class HostAttention:
    """Reusable state of the pipelined host-input call on one device: two sets of device
    input buffers for a head group and the two copy streams."""

    def __init__(self, device, *, group_heads: int = 4, sharded: bool = False, process_group=None):
        self.device = torch.device(device)
        self.group_heads = int(group_heads)
        if self.group_heads <= 0:
            raise ValueError("group_heads must be positive")
        self.process_group = process_group
        self.world = 1
        if sharded:
            import torch.distributed as dist

            self.world = dist.get_world_size(process_group)
            if self.group_heads % self.world:
                raise ValueError("a head group must divide evenly over the ranks")
        self._exchanges: dict = {}
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self._buffers: dict = {}

    def _slot(self, slot: int, shape, dtype):
        key = (slot, tuple(shape), dtype)
        got = self._buffers.get(key)
        if got is None:
            got = tuple(torch.empty(shape, dtype=dtype, device=self.device) for _ in range(3))
            self._buffers[key] = got
        return got

    def _exchange(self, rows: int, heads: int, dim: int, dtype):
        """The peer exchange for head groups of ``heads`` heads (built on first use; collective)."""
        from .ulysses import PeerExchange

        key = (rows, heads, dim, dtype)
        got = self._exchanges.get(key)
        if got is None:
            got = self._exchanges[key] = PeerExchange(rows, heads, dim, dtype, self.device, self.process_group)
        return got

    def close(self) -> None:
        """Collective: releases the exchange regions of the sharded mode."""
        for exchange in self._exchanges.values():
            exchange.close()
        self._exchanges.clear()

    def __call__(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, out: torch.Tensor,
                 *, layout: VisualLayout, layer: int, sparse_config: SparseConfig | None = None,
                 quant_config: QuantConfig | None = None,
                 calibration: NVFP4Calibration | None = None) -> torch.Tensor:
        """``query, key, value, out``: pinned host ``[1, S, H, D]`` tensors; returns ``out``
        after queueing everything (synchronise the current stream, or ``self.copy_out``,
        before reading it)."""
        for t in (query, key, value, out):
            if t.device.type != "cpu" or not t.is_pinned() or t.ndim != 4 or not t.is_contiguous():
                raise ValueError("host attention needs contiguous pinned host [1, S, H, D] tensors")
        if not (query.shape == key.shape == value.shape == out.shape):
            raise ValueError("Q, K, V and the output must share their shape")
        heads = query.size(2)
        compute = torch.cuda.current_stream(self.device)
        groups = [(h, min(h + self.group_heads, heads)) for h in range(0, heads, self.group_heads)]
        if self.world > 1 and any((h1 - h0) % self.world for h0, h1 in groups):
            raise ValueError("every head group must divide evenly over the ranks")
        ready, done, copied = {}, {}, {}
        self.copy_in.wait_stream(compute)

        def load(i):
            h0, h1 = groups[i]
            shape = (1, query.size(1), h1 - h0, query.size(3))
            dq, dk, dv = self._slot(i & 1, shape, query.dtype)
            with torch.cuda.stream(self.copy_in):
                # the slot's previous tenant (group i-2) must have finished computing
                if i >= 2:
                    self.copy_in.wait_event(done[i - 2])
                for dst, src in ((dq, query), (dk, key), (dv, value)):
                    native.copy_head_group(dst, src[:, :, h0:h1], self.copy_in)
                ready[i] = self.copy_in.record_event()

        load(0)
        for i, (h0, h1) in enumerate(groups):
            if i + 1 < len(groups):
                load(i + 1)
            shape = (1, query.size(1), h1 - h0, query.size(3))
            dq, dk, dv = self._slot(i & 1, shape, query.dtype)
            compute.wait_event(ready[i])
            if self.world == 1:
                result = anemoi_attention(dq, dk, dv, layout=layout, layer=layer, sparse_config=sparse_config,
                                          quant_config=quant_config, calibration=calibration)
            else:
                from .ulysses import ulysses_anemoi_attention

                # the peers store group i's output into the slot that held group i-2's: that
                # group must have left for the host before this rank lets group i start anywhere
                if i >= 2:
                    compute.wait_event(copied[i - 2])
                exchange = self._exchange(query.size(1), h1 - h0, query.size(3), query.dtype)
                result = ulysses_anemoi_attention(dq, dk, dv, layout=layout, layer=layer,
                                                  sparse_config=sparse_config, quant_config=quant_config,
                                                  calibration=calibration, group=self.process_group,
                                                  exchange=exchange)
            done[i] = compute.record_event()
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done[i])
                native.copy_head_group(out[:, :, h0:h1], result, self.copy_out)
                copied[i] = self.copy_out.record_event()
            if self.world == 1:
                result.record_stream(self.copy_out)
        compute.wait_stream(self.copy_out)
        return out


__all__ = ["HostAttention"]
