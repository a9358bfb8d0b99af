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
    anchors: torch.Tensor | None = None      # bool [R, R]: same-frame neighbours (enable_anchors)
    anchor_ids: torch.Tensor | None = None   # int32: flat indices of the set entries, frame-major
    anchor_count: int = 0

    @property
    def video_blocks(self) -> int:
        return self.blocks_per_frame * self.frames


@lru_cache(maxsize=64)
def _build(device_type: str, device_index: int | None, frames: int, height: int, width: int,
           logical_block: int, enable_anchors: bool = False) -> RaggedLayout:
    part = make_ragged_2d_partition(height, width, logical_block, include_adjacency=enable_anchors)
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
    anchors = anchor_ids = None
    anchor_count = 0
    if enable_anchors:
        # every (source, target) pair of neighbouring blocks of one frame, for every frame
        # (reference: anemoi/layers/attention/mpa/layout.py:72-98)
        total = frames * per_frame
        pairs = torch.tensor([(a, b) for a, row in enumerate(part.adjacency) for b, near in enumerate(row) if near],
                             dtype=torch.int64)
        base = (torch.arange(frames, dtype=torch.int64) * per_frame).view(-1, 1)
        ids = ((base + pairs[:, 0]) * total + base + pairs[:, 1]).reshape(-1)
        mask = torch.zeros(total * total, dtype=torch.bool)
        mask[ids] = True
        anchors = mask.view(total, total).to(device).contiguous()
        anchor_ids = ids.to(torch.int32).to(device).contiguous()
        anchor_count = int(ids.numel())
    return RaggedLayout(
        indices=indices.to(torch.int32).to(device).contiguous(),
        slot_valid=slot_valid.to(device).contiguous(),
        counts=counts.to(device).contiguous(),
        inverse=inverse.to(torch.int32).to(device).contiguous(),
        blocks_per_frame=per_frame,
        logical_block=logical_block,
        frames=frames,
        anchors=anchors,
        anchor_ids=anchor_ids,
        anchor_count=anchor_count,
    )


def materialize_ragged_2d_layout(device, *, frames: int, height: int, width: int,
                                 logical_block: int, enable_anchors: bool = False) -> RaggedLayout:
    """Return the cached slot tables of a ``frames x height x width`` video (with the anchor mask
    of the experimental anchored routing when ``enable_anchors``)."""
    if type(enable_anchors) is not bool:
        raise TypeError("enable_anchors must be a built-in bool")
    if logical_block not in (64, 128):
        raise ValueError("logical_block must be 64 or 128")
    if any(type(v) is not int or v <= 0 for v in (frames, height, width)):
        raise ValueError("video dimensions must be positive integers")
    resolved = torch.device(device)
    index = resolved.index
    if resolved.type == "cuda" and index is None:
        index = torch.cuda.current_device()
    return _build(resolved.type, index, frames, height, width, logical_block, enable_anchors)


__all__ = ["RaggedLayout", "materialize_ragged_2d_layout"]
