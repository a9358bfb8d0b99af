"""Generates ``tests/golden/reference_anchors.npz``: the reference's own routing with anchors.

Test infrastructure.  ``route_probability`` of the reference
(anemoi/layers/attention/mpa/routing.py:106-235) is plain torch and runs on CPU; the anchors are the
same-frame adjacency pairs its layout builds (mpa/layout.py:69-98).  Inputs are rebuilt from the
seeds by ``tests/test_anchors.py``; the row lists and counts are stored.

Run where the reference checkout is present:  python tests/golden/make_anchor_golden.py
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

# name: frames, height, width, block, drop, (nvfp4, int8, fp16) ratios, seed
CASES = {
    "mixed": (2, 32, 48, 64, 0.5, (0.4, 0.4, 0.2), 0),
    "int8_fp16": (2, 40, 56, 128, 0.4, (0.0, 0.5, 0.5), 1),
    "fp16": (2, 32, 32, 64, 0.5, (0.0, 0.0, 1.0), 2),
}


def case_inputs(name: str):
    """A seeded fp16 probability map [R, R] with ties across rows and columns, and the geometry."""
    from anemoi_b200.partition import make_ragged_2d_partition

    frames, height, width, block, drop, ratios, seed = CASES[name]
    part = make_ragged_2d_partition(height, width, block, include_adjacency=True)
    blocks = frames * part.block_count
    gen = torch.Generator().manual_seed(seed)
    prob = torch.softmax(torch.randn(blocks, blocks, generator=gen) * 2.5, dim=-1).half()
    prob[1, :7] = prob[0, 0]
    prob[blocks // 2, 3:9] = prob[0, 0]
    return prob, part, frames, blocks


def anchor_matrix(part, frames: int) -> np.ndarray:
    """Same-frame adjacency as one [R, R] bool matrix (block-diagonal over the frames)."""
    per = part.block_count
    adj = np.asarray(part.adjacency, dtype=bool)
    out = np.zeros((frames * per, frames * per), dtype=bool)
    for f in range(frames):
        out[f * per : (f + 1) * per, f * per : (f + 1) * per] = adj
    return out


def main() -> None:
    root = Path(os.environ.get("ANEMOI_REFERENCE_ROOT", ROOT.parent / "reference"))
    sys.path.insert(0, str(root))
    from anemoi.layers.attention.mpa.routing import route_probability

    out = {}
    for name, (frames, height, width, block, drop, ratios, seed) in CASES.items():
        prob, part, frames, blocks = case_inputs(name)
        anchors = torch.from_numpy(anchor_matrix(part, frames))
        plan = route_probability(prob[None, None], anchors, anchor_count=int(anchors.sum()), prefix_blocks=0,
                                 sparsity_ratio=drop, nvfp4_ratio=ratios[0], fp8_ratio=ratios[1],
                                 fp16_ratio=ratios[2])
        out[name + "_ids"] = plan.block_ids[0, 0].numpy().astype(np.int32)
        out[name + "_counts"] = np.stack([plan.nvfp4_counts[0, 0].numpy(), plan.fp8_counts[0, 0].numpy(),
                                          plan.fp16_counts[0, 0].numpy()]).astype(np.int32)
    path = ROOT / "tests" / "golden" / "reference_anchors.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
