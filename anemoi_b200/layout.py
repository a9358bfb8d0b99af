"""Slot tables that tie the raster video tokens to the packed block order.

``indices[slot]`` is the raster token stored in a packed slot (0 for padding),
``slot_valid[slot]`` says whether the slot holds a real token, ``counts[block]``
is the number of real tokens of a block and ``inverse[token]`` is the slot of a
raster token.  Blocks are frame-major; inside a frame they follow the order of
``make_ragged_2d_partition`` and tokens inside a block ascend in raster order.

Same contents as the reference's ``materialize_ragged_2d_layout``
(anemoi/layers/attention/mpa/layout.py:25-109); tensors are int32 here because
the kernels index with 32-bit integers, and any torch device is accepted so the
CPU tests can build them.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import torch

from .partition import make_ragged_2d_partition


@dataclass(frozen=True)
class RaggedLayout:
    indices: torch.Tensor      # int32 [R * block]
    slot_valid: torch.Tensor   # bool  [R * block]
    counts: torch.Tensor       # int32 [R]
    inverse: torch.Tensor      # int32 [frames * height * width]
    blocks_per_frame: int
    logical_block: int
    frames: int

    @property
    def video_blocks(self) -> int:
        return self.blocks_per_frame * self.frames


@lru_cache(maxsize=64)
def _build(device_type: str, device_index: int | None, frames: int, height: int, width: int,
           logical_block: int) -> RaggedLayout:
    part = make_ragged_2d_partition(height, width, logical_block, include_adjacency=False)
    per_frame = part.block_count
    frame_tokens = height * width
    local = torch.zeros((per_frame, logical_block), dtype=torch.int64)
    valid = torch.zeros((per_frame, logical_block), dtype=torch.bool)
    for b, block in enumerate(part.blocks):
        local[b, : len(block)] = torch.tensor(block, dtype=torch.int64)
        valid[b, : len(block)] = True
    offsets = (torch.arange(frames, dtype=torch.int64) * frame_tokens).view(frames, 1, 1)
    indices = (local.unsqueeze(0) + offsets) * valid.unsqueeze(0)
    slot_valid = valid.unsqueeze(0).expand(frames, -1, -1).reshape(-1)
    indices = indices.reshape(-1)
    counts = torch.tensor(part.counts, dtype=torch.int32).repeat(frames)
    inverse = torch.empty(frames * frame_tokens, dtype=torch.int64)
    slots = torch.arange(indices.numel(), dtype=torch.int64)
    inverse[indices[slot_valid]] = slots[slot_valid]
    device = torch.device(device_type, device_index)
    return RaggedLayout(
        indices=indices.to(torch.int32).to(device).contiguous(),
        slot_valid=slot_valid.to(device).contiguous(),
        counts=counts.to(device).contiguous(),
        inverse=inverse.to(torch.int32).to(device).contiguous(),
        blocks_per_frame=per_frame,
        logical_block=logical_block,
        frames=frames,
    )


def materialize_ragged_2d_layout(device, *, frames: int, height: int, width: int,
                                 logical_block: int) -> RaggedLayout:
    """Return the cached slot tables of a ``frames x height x width`` video."""
    if logical_block not in (64, 128):
        raise ValueError("logical_block must be 64 or 128")
    if any(type(v) is not int or v <= 0 for v in (frames, height, width)):
        raise ValueError("video dimensions must be positive integers")
    resolved = torch.device(device)
    index = resolved.index
    if resolved.type == "cuda" and index is None:
        index = torch.cuda.current_device()
    return _build(resolved.type, index, frames, height, width, logical_block)


__all__ = ["RaggedLayout", "materialize_ragged_2d_layout"]
