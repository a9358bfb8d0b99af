"""Generates tests/golden/adapter_trace.json by driving the reference's own H3MPAAttention
(anemoi/models/minimax_h3/mpa_attention.py) with its two attention paths stubbed out, so the
schedule it follows (dense-first steps and layers, request detection, band lookups) is pinned.

    python tests/golden/make_adapter_golden.py /path/to/anemoi

The file is committed; tests never import the reference.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

SCENARIOS = [
    {"name": "two_requests",
     "config": {"video_shape": [2, 4, 4], "prefix_tokens": 5, "dense_first_steps": 2, "dense_first_layers": 1,
                "layers_per_step": 4},
     "timesteps": [1.0, 0.9, 0.8, 0.7, 1.0, 0.9, 0.5]},
    {"name": "rising_then_falling",
     "config": {"video_shape": [1, 3, 3], "prefix_tokens": 2, "dense_first_steps": 1, "dense_first_layers": 0,
                "layers_per_step": 3, "query_block_size": 128},
     "timesteps": [0.1, 0.2, 0.3, 0.3, 0.25, 0.2, None, 0.1]},
    {"name": "bands",
     "config": {"video_shape": [2, 2, 2], "prefix_tokens": 3, "dense_first_steps": 0, "dense_first_layers": 2,
                "layers_per_step": 6, "sparsity_ratio": 0.75, "nvfp4_ratio": 0.4, "int8_ratio": 0.4,
                "fp16_ratio": 0.2, "layer_sparsity_bands": [[0, 2, 0.5], [4, 6, 0.9]],
                "layer_precision_bands": [[1, 3, 0.0, 0.5, 0.5], [3, 4, 0.25, 0.25, 0.0, 0.5]]},
     "timesteps": [1.0, 0.5]},
]
VIDEO_INDEX_CASES = [[0, 1, 2, 10, 11, 12, 13], [5, 6, 7, 8], [], [3], [0, 2, 4, 5, 6], [9, 3, 4, 5]]


def build_config(cls, spec: dict):
    kw = dict(spec)
    kw["video_shape"] = tuple(kw["video_shape"])
    for key in ("layer_sparsity_bands", "layer_precision_bands"):
        if key in kw:
            kw[key] = tuple(tuple(b) for b in kw[key])
    return cls(**kw)


def drive(attention_cls, config, timesteps) -> dict:
    att = attention_cls(config)
    log = []
    att.dense = lambda q, k, v: log.append(["dense"]) or q
    att.mpa = lambda q, k, v, layer: log.append(["mpa", layer]) or q
    pos = torch.zeros(config.sequence_tokens)
    x = torch.zeros(1)
    for t in timesteps:
        att.observe(timestep=None if t is None else torch.tensor([t]), video_indices=None, position_ids=pos)
        for _ in range(config.layers_per_step):
            att(x, x, x)
        log.append(["step", att.request, att.step])
    att.close_request()
    stats = att.stats()
    stats.pop("config")
    return {"log": log, "stats": stats}


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from anemoi.models.minimax_h3 import mpa_attention as M

    out = {"scenarios": [], "video_start": []}
    for sc in SCENARIOS:
        cfg = build_config(M.H3MPAConfig, sc["config"])
        entry = dict(sc)
        entry.update(drive(M.H3MPAAttention, cfg, sc["timesteps"]))
        entry["precision"] = [list(cfg.precision(layer)) for layer in range(cfg.layers_per_step)]
        probe = M.H3MPAAttention(cfg)
        entry["sparsity"] = [probe._sparsity(layer) for layer in range(cfg.layers_per_step)]
        entry["sequence_tokens"] = cfg.sequence_tokens
        out["scenarios"].append(entry)
    for case in VIDEO_INDEX_CASES:
        out["video_start"].append({"indices": case,
                                   "start": M._target_video_start(torch.tensor(case, dtype=torch.int64), 99)})
    path = Path(__file__).resolve().parent / "adapter_trace.json"
    path.write_text(json.dumps(out, separators=(",", ":")))
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_adapter_golden.py <path of the reference checkout>")
    main(sys.argv[1])
