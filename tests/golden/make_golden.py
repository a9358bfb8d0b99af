"""Generates tests/golden/reference_vectors.json by running the reference's own
CPU-runnable functions (imported from a checkout of anemoi-project/anemoi).

    python tests/golden/make_golden.py /path/to/anemoi

The file is committed; tests never import the reference.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import base64

import numpy as np
import torch


def pack(t: torch.Tensor) -> dict:
    """Tensor -> {dtype, shape, base64 of the raw bytes}."""
    a = t.contiguous().numpy()
    return {"dtype": str(a.dtype), "shape": list(a.shape), "b64": base64.b64encode(a.tobytes()).decode()}


def sha(blocks) -> str:
    return hashlib.sha256(json.dumps(blocks, separators=(",", ":")).encode()).hexdigest()


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from anemoi.layers.attention.mpa import executor as E
    from anemoi.layers.attention.mpa.ragged_2d import make_ragged_2d_partition
    from anemoi.layers.attention.mpa.routing import _route_counts, draft_probability, route_probability

    out: dict = {}
    geometries = [(8, 8, 64), (16, 16, 64), (24, 40, 64), (16, 16, 128), (12, 32, 64), (24, 42, 128),
                  (24, 42, 64), (30, 52, 128), (30, 52, 64), (48, 84, 128), (48, 84, 64), (7, 20, 64),
                  (17, 30, 64), (5, 5, 64), (1, 100, 64), (100, 1, 64), (3, 50, 128), (17, 23, 64),
                  (12, 20, 128), (10, 14, 64), (12, 12, 128), (9, 9, 128), (31, 53, 64), (2, 2, 64)]
    out["partition"] = []
    for h, w, c in geometries:
        p = make_ragged_2d_partition(h, w, c, include_adjacency=False)
        out["partition"].append({"geometry": [h, w, c], "sha256": sha(p.blocks), "counts": list(p.counts)})

    out["route_counts"] = []
    for items in (1, 4, 16, 256, 74529, 451584, 1750329):
        for drop in (0.0, 0.5, 0.8, 0.9, 0.999):
            for r4, r8, r16 in ((0, 1, 0), (0, 0.5, 0.5), (0.4, 0.4, 0.2), (1 / 3, 1 / 3, 1 / 3), (1, 0, 0), (0.25, 0.25, 0.5)):
                n = _route_counts(items, sparsity_ratio=drop, nvfp4_ratio=r4, fp8_ratio=r8, fp16_ratio=r16)
                out["route_counts"].append({"items": items, "drop": drop, "ratios": [r4, r8, r16], "n": list(n)})

    gen = torch.Generator().manual_seed(7)
    out["route"] = []
    for r, drop, ratios in ((12, 0.5, (0.4, 0.4, 0.2)), (9, 0.8, (0.0, 1.0, 0.0)), (16, 0.3, (0.5, 0.0, 0.5)), (6, 0.0, (0.2, 0.3, 0.5))):
        logits = torch.randn(1, 2, r, r, generator=gen)
        prob = torch.softmax(logits, -1).to(torch.float16)
        prob[0, 0, 1, :4] = prob[0, 0, 0, 0]          # exact ties across rows and columns
        prob[0, 1, :, 2] = prob[0, 1, 0, 2]
        plan = route_probability(prob, None, anchor_count=0, prefix_blocks=0, sparsity_ratio=drop,
                                 nvfp4_ratio=ratios[0], fp8_ratio=ratios[1], fp16_ratio=ratios[2])
        entry = {"r": r, "drop": drop, "ratios": list(ratios),
                 "prob_bits": pack(prob.view(torch.int16)),
                 "ids": pack(plan.block_ids), "low": pack(plan.nvfp4_counts),
                 "mid": pack(plan.fp8_counts), "high": pack(plan.fp16_counts), "compose": []}
        for qb, pblocks, pphase, active in ((64, 0, "int8", ("nvfp4", "int8", "fp16")), (128, 2, "int8", ("nvfp4", "int8", "fp16")),
                                            (128, 3, "fp16", ("nvfp4", "int8", "fp16")), (64, 1, "nvfp4", ("nvfp4", "int8", "fp16"))):
            if pphase not in active:
                continue
            ids, nv, mid, hi = E._compose_sm120_phase_route(
                plan.block_ids, plan.nvfp4_counts, plan.fp8_counts, plan.fp16_counts,
                query_block_size=qb, prefix_blocks=pblocks, prefix_phase=pphase, active_phases=active)
            entry["compose"].append({"qb": qb, "prefix_blocks": pblocks, "prefix_phase": pphase,
                                     "ids": pack(ids), "nv": pack(nv), "mid": pack(mid), "high": pack(hi)})
        out["route"].append(entry)

    out["pool"] = []
    for block, dim in ((64, 64), (128, 128)):
        x = torch.randn(1, 1, 3 * block, dim, generator=gen).to(torch.float16)
        counts = torch.tensor([[block, block - 7, block - 1]], dtype=torch.int32)
        valid = torch.arange(block).view(1, 1, 1, block, 1) < counts.view(1, 1, 3, 1, 1)
        x = (x.view(1, 1, 3, block, dim) * valid).view(1, 1, 3 * block, dim)
        mean = E._pool_query(x, counts, block)
        mx = E._pool_query(x, counts, block, maximum=True)
        prob = draft_probability(mean, mx)
        out["pool"].append({"block": block, "dim": dim, "x_bits": pack(x.view(torch.int16)),
                            "counts": counts.tolist(), "mean_bits": pack(mean.view(torch.int16)),
                            "max_bits": pack(mx.view(torch.int16)),
                            "prob_bits": pack(prob.view(torch.int16))})

    pre = torch.tensor([[64, 36]], dtype=torch.int32)
    vid = torch.tensor([[126, 120, 64, 3]], dtype=torch.int32)
    out["valid_k_q128"] = {"prefix": pre.tolist(), "video": vid.tolist(),
                           "expanded": E._expand_q128_valid_k(pre, vid).tolist()}
    path = Path(__file__).resolve().parent / "reference_vectors.json"
    path.write_text(json.dumps(out, separators=(",", ":")))
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
