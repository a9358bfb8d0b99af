"""Generates ``tests/golden/reference_kernels_*.npz``: outputs of the reference's OWN CUDA kernels.

Test infrastructure.  The reference's SM120 extension is built for sm_100a, unchanged, by
``oracle/ref_build/build.py`` (output ``oracle/_ref/_ref_sm120.so``); importing that module
registers ``torch.ops.mixed_attention.*`` exactly as the reference's build does.  This script
drives those operators the way the reference's executor does
(anemoi/layers/attention/mpa/executor.py:1013-1199: prepare -> draft probability -> route ->
materialise -> attention phases; prefix rows: backends/sm120_q128.py:97-115) on two small seeded
cases and stores what they return.  ``tests/test_reference_kernels_cpu.py`` then holds the CPU
oracle to these fixtures, which pins the oracle - and through it the CUDA path of this
repository - to the reference's kernels rather than to a reading of their source.

The block-scaled NVFP4 attention phase does not assemble for sm_100a, so only its operands
(codes and scales) are pinned here, not its attention output.

Run on a B200:  python tests/golden/make_kernel_golden.py
"""

from __future__ import annotations

import hashlib
import importlib.util
import math
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from anemoi_b200.partition import make_ragged_2d_partition  # noqa: E402
from oracle import prep as P  # noqa: E402
from oracle import route as R  # noqa: E402
from tests.helpers import smooth_fields  # noqa: E402

CASES = {
    # name: video shape, prefix, heads, D, QB, dtype, outlier channels, max-pool weight, drop
    "q128": ((2, 12, 20), 70, 2, 128, 128, torch.bfloat16, (17, 93), 0.5, 0.5),
    "q64": ((2, 10, 14), 0, 2, 64, 64, torch.float16, (), 0.0, 0.5),
}


def load_reference_ops():
    path = ROOT / "oracle" / "_ref" / "_ref_sm120.so"
    if not path.exists():
        raise SystemExit(f"{path} is missing: run python oracle/ref_build/build.py first")
    spec = importlib.util.spec_from_file_location("_ref_sm120", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return torch.ops.mixed_attention


def u16(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def raw(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype in (torch.float8_e4m3fn,):
        t = t.view(torch.uint8)
    return t.cpu().numpy()


def digest(array: np.ndarray) -> np.ndarray:
    """SHA-256 of the array's bytes: the packed fp16 rows are compared by digest (the oracle
    reproduces them bit for bit), which keeps the fixtures small."""
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(array).tobytes()).digest(), dtype=np.uint8)


def run_case(ops, name: str) -> dict:
    video, prefix, heads, dim, qb, dtype, outliers, weight, drop = CASES[name]
    frames, height, width = video
    q, k, v = smooth_fields(frames, height, width, heads, dim, prefix, seed=0, outliers=outliers, dtype=dtype)
    scales = tuple(float(t.float().abs().max()) / (6 * 448) for t in (q, k, v))
    dev = torch.device("cuda")
    qd, kd, vd = (t.to(dev) for t in (q, k, v))
    part = make_ragged_2d_partition(height, width, qb, include_adjacency=False)
    geo = P.make_geometry(part.blocks, frames, height, width, qb, prefix)
    indices = torch.from_numpy(geo.indices.astype(np.int64)).to(dev)
    slot_valid = torch.from_numpy(geo.slot_valid.astype(bool)).to(dev)
    counts = torch.from_numpy(geo.counts.astype(np.int32)).to(dev)
    gs = tuple(torch.tensor(s, device=dev, dtype=torch.float32) for s in scales)
    native_prefix = prefix > 0

    # executor.py:1009-1039: the raw tensors are handed over as BHSD views of the BSHD storage
    prepared = ops.prepare_h3_sm120_operands(
        qd.permute(0, 2, 1, 3), kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), indices, slot_valid,
        counts, prefix, qb, True, True, False, True, native_prefix, True, *gs)
    out = {"scales": np.asarray(scales, dtype=np.float64)}
    names = ("q_pool", "k_pool", "q16", "k16", "v16", "q4", "q4_scale", "k4", "k4_scale", "v4",
             "v4_scale")
    for i, nm in enumerate(names):
        t = prepared[i]
        out[nm] = u16(t) if t.dtype == torch.float16 else raw(t)
    for nm in ("q16", "k16", "v16"):
        full = out.pop(nm)                      # [1, H, rows, D]
        out[nm + "_sha256"] = np.stack([digest(full[0, h]) for h in range(full.shape[1])])
    for i, nm in zip(range(17, 27), ("q8", "q8_scale", "k8", "k8_scale", "v8", "v8_scale", "pq8",
                                     "pq8_scale", "q_max", "k_max")):
        t = prepared[i]
        out[nm] = u16(t) if t.dtype == torch.float16 else raw(t)
    q_pool, k_pool, q16, k16, v16 = prepared[0:5]
    q8, q8_scale, k8, k8_scale, v8, v8_scale = prepared[17:23]
    pq8, pq8_scale = prepared[23:25]
    q_max, k_max = prepared[25], prepared[26]

    # draft probability, with and without the max-pool blend (executor.py:1141-1150)
    prob_mean = ops.sm120_h3_draft_probability(q_pool, k_pool)
    out["prob_mean"] = u16(prob_mean)
    prob = prob_mean
    if weight:
        prob = ops.sm120_h3_draft_probability(q_pool, k_pool, q_max, k_max, weight)
        out["prob_blend"] = u16(prob)
        out["blend_weight"] = np.float64(weight)

    blocks = int(counts.numel())
    prefix_blocks = math.ceil(prefix / 64)
    pre = torch.clamp(prefix - torch.arange(prefix_blocks, device=dev, dtype=torch.int32) * 64, 0, 64)
    if qb == 128:
        vid = torch.stack((counts.clamp_max(64), (counts - 64).clamp_min(0)), dim=-1).reshape(-1)
    else:
        vid = counts
    valid_k = torch.cat((pre, vid)).to(torch.int32).view(1, -1).contiguous()
    out["valid_k"] = raw(valid_k)
    scale = 1.0 / math.sqrt(dim)

    cells = {"int8": (0.0, 1.0, 0.0), "int8_fp16": (0.0, 0.5, 0.5)}
    if prefix == 0:
        cells["fp16"] = (0.0, 0.0, 1.0)
    for cell, ratios in cells.items():
        n16, n8, n4 = R.budgets(blocks * blocks, drop, *ratios)
        ids, low, mid, high = ops.sm120_h3_route_precision(prob, n16, n8, n4, None, None, 0)
        out[f"{cell}_budgets"] = np.asarray((n16, n8, n4))
        out[f"{cell}_route_ids"] = raw(ids)
        out[f"{cell}_route_counts"] = np.stack([raw(low), raw(mid), raw(high)])
        phases = tuple(n for n, r in zip(("nvfp4", "int8", "fp16"), ratios) if r > 0)
        prefix_phase = None if prefix == 0 else "int8"
        phase_index = {"nvfp4": 0, "int8": 1, "fp16": 2}[prefix_phase or phases[0]]
        has_fp16 = "fp16" in phases
        mids, nv_c, mid_c, hi_c = ops.sm120_h3_materialize_route(
            ids, low, mid, high, qb, prefix_blocks, phase_index,
            prefix_phase is None or prefix_phase == phases[0], has_fp16)
        out[f"{cell}_stage_ids"] = raw(mids)
        # a phase that is not active comes back as an empty tensor
        for nm, t in (("nv", nv_c), ("mid", mid_c), ("hi", hi_c)):
            out[f"{cell}_stage_counts_{nm}"] = raw(t)
        if cell == "fp16":
            fn = ops.sm120_q64_fp16_attention_forward if qb == 64 else ops.sm120_q128_fp16_attention_forward
            video_out, _ = fn(q16, k16, v16, mids, hi_c, valid_k, scale)
        else:
            fn = ops.sm120_q64_int8_attention_forward if qb == 64 else ops.sm120_q128_int8_attention_forward
            video_out, _ = fn(q8, k8, v8, q16, k16, v16, mids, mid_c, hi_c, q8_scale, k8_scale,
                              v8_scale, valid_k, 0, scale, has_fp16)
        out[f"{cell}_video_out"] = u16(video_out)
    if native_prefix:
        fn = (ops.sm120_q64_prefix_int8_attention_forward if qb == 64
              else ops.sm120_q128_prefix_int8_attention_forward)
        prefix_out = fn(pq8, k8, v8, pq8_scale, k8_scale, v8_scale, valid_k, prefix, scale)
        out["prefix_out"] = u16(prefix_out)
    torch.cuda.synchronize()
    return out


def main() -> None:
    ops = load_reference_ops()
    target = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden"
    target.mkdir(parents=True, exist_ok=True)
    for name in CASES:
        data = run_case(ops, name)
        path = target / f"reference_kernels_{name}.npz"
        np.savez_compressed(path, **data)
        print(f"wrote {path} ({path.stat().st_size} bytes, {len(data)} arrays)")


if __name__ == "__main__":
    main()
