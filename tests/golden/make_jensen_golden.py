"""Generates ``tests/golden/reference_jensen.npz``: the reference's own diag-Jensen draft map.

Test infrastructure.  ``draft_probability(q_pool, k_pool, q_second=, k_second=)`` of the reference
(anemoi/layers/attention/mpa/routing.py:64-103) is plain torch and runs on CPU; the second
moments are formed as its executor forms them (mpa/executor.py:1105-1124: mean of the squares of
the packed fp16 rows over the block's real tokens, rounded to fp16).  Inputs are rebuilt from the
seeds by ``tests/test_jensen.py``; only the maps are stored.

Run where the reference checkout is present:  python tests/golden/make_jensen_golden.py
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

# name: blocks, tokens per block, D, seed
CASES = {"d64": (40, 64, 64, 0), "d128": (77, 128, 128, 1), "ragged": (33, 64, 128, 2)}


def case_inputs(name: str):
    """Packed fp16 rows of one head, [blocks, slots, D], and the real token count per block."""
    blocks, slots, dim, seed = CASES[name]
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(blocks, slots, dim, generator=gen) * 0.6).half()
    k = (torch.randn(blocks, slots, dim, generator=gen) * 0.6 + 0.2).half()
    counts = torch.full((blocks,), slots, dtype=torch.int64)
    if name == "ragged":
        counts = torch.randint(slots // 2, slots + 1, (blocks,), generator=gen)
        mask = torch.arange(slots)[None, :, None] < counts[:, None, None]
        q, k = q * mask, k * mask
    return q, k, counts


def pools(x: torch.Tensor, counts: torch.Tensor):
    den = counts.to(torch.float32).view(-1, 1)
    mean = (x.float().sum(dim=1) / den).half()
    second = (x.float().square().sum(dim=1) / den).half()
    return mean, second


def main() -> None:
    root = Path(os.environ.get("ANEMOI_REFERENCE_ROOT", ROOT.parent / "reference"))
    sys.path.insert(0, str(root))
    from anemoi.layers.attention.mpa.routing import draft_probability

    out = {}
    for name in CASES:
        q, k, counts = case_inputs(name)
        (qm, q2), (km, k2) = pools(q, counts), pools(k, counts)
        prob = draft_probability(qm[None, None], km[None, None], q_second=q2[None, None], k_second=k2[None, None])
        out[name] = prob[0, 0].numpy().view(np.uint16)
    path = ROOT / "tests" / "golden" / "reference_jensen.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
