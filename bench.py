"""Benchmark of the sparse mixed-precision attention layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the third benchmark configuration, the one the metric is quoted on):
512-token prefix + 21x48x84 video tokens (S = 85,184), 56 heads, D = 128, bf16,
Q128 query blocks, 80 % of block pairs dropped, retained pairs split NVFP4 / INT8 /
FP16 = 40 / 40 / 20, NVFP4 global scales amax/(6*448).  Inputs are seeded synthetic
tensors with the smooth-field statistics of the reference's captured Q/K/V.

One "step" is one whole ``anemoi_attention`` layer call.  ``value`` is the
dense-equivalent throughput 4*S^2*D*H / time with inputs resident in HBM; ``e2e``
is the same metric through the public API with pinned-host inputs copied to the
device and the result copied back inside the timed region.  With N > 1 the heads
are sharded over N GPUs by a Ulysses sequence<->head all-to-all (strong scaling).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "sparse-attn layer ms & dense-equiv TFLOPS @84,672 tok, 1/2/4/8 B200"
WORKLOAD = dict(prefix=512, video=(21, 48, 84), heads=56, dim=128, query_block=128, drop=0.8,
                ratios=(0.4, 0.4, 0.2), maxpool=0.0, outliers=(17, 93))
# Small case for profiler captures only (never a bench line): same cells and block shapes,
# 8 heads of the 832x480 geometry - about 0.5 GB on the device, inputs still larger than L2.
PROFILE_WORKLOAD = dict(WORKLOAD, video=(21, 30, 52), heads=8)


def dense_equivalent_flops(s: int, d: int, h: int) -> float:
    return 4.0 * s * s * d * h


def executed_flops(w, kept_pairs: int, blocks: int) -> float:
    """FLOPs the attention kernels execute per layer: retained pairs + prefix columns + prefix rows."""
    qb, d, h = w["query_block"], w["dim"], w["heads"]
    p = math.ceil(w["prefix"] / 64)
    kp = 64 * p + blocks * qb
    rows_prefix = math.ceil(w["prefix"] / qb) * qb
    return 4.0 * d * h * (kept_pairs * qb * qb + blocks * qb * 64 * p + rows_prefix * kp)


def synth_qkv(w, heads: int, device, seed: int, rows: slice | None = None, dtype=torch.bfloat16):
    """Seeded smooth-field Q/K/V ``[1, S, heads, D]`` (see module docstring)."""
    f, hh, ww = w["video"]
    d, prefix = w["dim"], w["prefix"]
    gen = torch.Generator(device=device).manual_seed(seed)
    radius = 6
    taps = torch.exp(-0.5 * (torch.arange(-radius, radius + 1, dtype=torch.float32, device=device) / 2.0) ** 2)
    taps = taps / taps.sum()

    def field():
        out = torch.empty(prefix + f * hh * ww, heads, d, dtype=dtype, device=device)
        out[:prefix] = torch.randn(prefix, heads, d, generator=gen, device=device).to(dtype)
        for h in range(heads):
            x = torch.randn(f, d, hh, ww, generator=gen, device=device)
            x = torch.nn.functional.pad(x, (0, 0, radius, radius), mode="reflect")
            x = torch.nn.functional.conv2d(x, taps.view(1, 1, -1, 1).expand(d, 1, -1, 1), groups=d)
            x = torch.nn.functional.pad(x, (radius, radius, 0, 0), mode="reflect")
            x = torch.nn.functional.conv2d(x, taps.view(1, 1, 1, -1).expand(d, 1, 1, -1), groups=d)
            x = x + 0.5 * torch.randn(x.shape, generator=gen, device=device)
            for ch in w["outliers"]:
                x[:, ch] *= 8.0
            out[prefix:, h] = x.permute(0, 2, 3, 1).reshape(f * hh * ww, d).to(dtype)
        return out.unsqueeze(0)

    q, k = field(), field()
    v = torch.randn(1, prefix + f * hh * ww, heads, d, generator=gen, device=device).to(dtype)
    if rows is not None:
        q, k, v = (t[:, rows].contiguous() for t in (q, k, v))
    return q, k, v


class ClockSampler:
    """Samples the GPU's SM clock and throttle reasons while the timed region runs: NVML queries
    from a thread of this process every 10 ms (read-only; a sample is also taken on entry and on
    exit, so that a region of a few milliseconds still has some), or `nvidia-smi -lms` when the
    NVML binding is missing."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows: list[list[str]] = []
        self.proc = None
        self.nvml = None
        self.handle = None
        self.stop = threading.Event()

    def _open_nvml(self) -> bool:
        try:
            import pynvml

            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml = pynvml
            return True
        except Exception:
            self.nvml = None
            return False

    def _sample_nvml(self) -> None:
        n = self.nvml
        try:
            sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
            mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(
                n, "nvmlDeviceGetCurrentClocksEventReasons") else n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        except Exception:
            return
        bits = (0x8, 0x40, 0x20, 0x4)    # hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        self.rows.append([str(sm), str(mx)] + ["Active" if mask & b else "Not Active" for b in bits])

    def __enter__(self):
        if self._open_nvml():
            self._sample_nvml()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _poll(self):
        while not self.stop.wait(0.01):
            self._sample_nvml()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.nvml is not None:
            self.stop.set()
            self.thread.join(timeout=2)
            self._sample_nvml()
            try:
                self.nvml.nvmlShutdown()
            except Exception:
                pass
        elif self.proc is not None:
            self.proc.terminate()
            self.proc.wait(timeout=5)
            self.thread.join(timeout=2)
        return False

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 6:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvml" if self.nvml is not None else "nvidia-smi"}


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle restatement of the reference's algorithm on the host cores
# ------------------------------------------------------------------------------------------
def cpu_sample(w, query_blocks: int, seed: int = 1) -> dict:
    """Time one head of the workload on the CPU with ``query_blocks`` query blocks of attention
    and extrapolate to the whole layer (heads and query blocks are independent)."""
    import numpy as np

    from anemoi_b200.partition import make_ragged_2d_partition
    from oracle import attention as A, prep as P, route as R
    from oracle.pipeline import resolve

    f, hh, ww = w["video"]
    q, k, v = synth_qkv(w, 1, torch.device("cpu"), seed)
    amax = [float(t.float().abs().max()) / (6 * 448) for t in (q, k, v)]
    t0 = time.perf_counter()
    part = make_ragged_2d_partition(hh, ww, w["query_block"], include_adjacency=False)
    t_partition = time.perf_counter() - t0
    geo = P.make_geometry(part.blocks, f, hh, ww, w["query_block"], w["prefix"])
    r4, r8, r16 = w["ratios"]
    _, active, prefix_phase = resolve(r4, r8, r16, w["prefix"], "int8")
    t0 = time.perf_counter()
    ops = P.prepare_head(q[0, :, 0], k[0, :, 0], v[0, :, 0], geo, has_nvfp4="nvfp4" in active,
                         has_int8="int8" in active, has_prefix_query_int8=True,
                         has_maxpool=w["maxpool"] != 0.0, global_scales=tuple(amax))
    t_prep = time.perf_counter() - t0
    t0 = time.perf_counter()
    prob = R.draft_probability(ops.q_pool, ops.k_pool, ops.q_max, ops.k_max, w["maxpool"])
    rr = geo.video_blocks
    n16, n8, n4 = R.budgets(rr * rr, w["drop"], r4, r8, r16)
    ids, low, mid, high = R.route(prob, n16, n8, n4)
    lists = R.stage_lists(ids, low, mid, high, query_block=geo.query_block,
                          prefix_stages=geo.prefix_stages, prefix_phase=prefix_phase)
    t_route = time.perf_counter() - t0
    qb = geo.query_block
    pick = np.linspace(0, rr - 1, query_blocks).astype(int)
    t0 = time.perf_counter()
    stages_done = 0
    for i in pick:
        A.attention_rows(ops, geo, slice(i * qb, (i + 1) * qb), lists[i], head_dim=w["dim"],
                         q_scale_index=int(i), global_scales=tuple(amax))
        stages_done += sum(len(x) for x in lists[i])
    t_attn = time.perf_counter() - t0
    stages_all = sum(sum(len(x) for x in row) for row in lists)
    prefix_stage_work = math.ceil(w["prefix"] / qb) * geo.stages
    t_head = t_prep + t_route + t_attn * (stages_all + prefix_stage_work) / max(stages_done, 1)
    layer_s = t_head * w["heads"]
    s = w["prefix"] + f * hh * ww
    return {
        "layer_seconds": layer_s,
        "tflops": dense_equivalent_flops(s, w["dim"], w["heads"]) / layer_s / 1e12,
        "sample": (f"one head of the workload: gather/quantise {t_prep:.2f}s + draft/route {t_route:.2f}s "
                   f"+ {query_blocks} of {rr} query blocks of attention {t_attn:.2f}s, scaled by stages "
                   f"and x{w['heads']} heads (partition search {t_partition:.2f}s, once per geometry, not counted)"),
        "cores": os.cpu_count(),
        "sample_seconds": t_prep + t_route + t_attn,
    }


def reference_kernels_same_gpu(heads: int = 56, repeats: int = 5) -> dict:
    """The reference's OWN kernels (its SM120 extension built unchanged for sm_100a,
    oracle/ref_build) beside this library's on the same B200, stage by stage, on the second
    benchmark configuration (prefix 512 + 21x30x52, Q128, max-pool 0.5, INT8/FP16 50/50): the
    largest configuration whose cells the reference's kernels can run on sm_100a (its NVFP4
    phase does not assemble for this architecture).  Driven as the reference's executor drives
    them (anemoi/layers/attention/mpa/executor.py:1013-1199)."""
    import numpy as np

    from anemoi_b200 import executor
    from anemoi_b200.layout import materialize_ragged_2d_layout
    from anemoi_b200.routing import route_counts
    from tests.golden.make_kernel_golden import load_reference_ops

    ops = load_reference_ops()
    w = dict(WORKLOAD, video=(21, 30, 52), heads=heads, ratios=(0.0, 0.5, 0.5), maxpool=0.5)
    device = torch.device("cuda", 0)
    q, k, v = synth_qkv(w, heads, device, seed=0)
    prefix, qb, dim, video = w["prefix"], w["query_block"], w["dim"], w["video"]
    lay = materialize_ragged_2d_layout(device, frames=video[0], height=video[1], width=video[2],
                                       logical_block=qb)
    counts = lay.counts
    valid = torch.arange(qb, device=device).view(1, -1) < counts.view(-1, 1)
    indices, slot_valid = lay.indices.to(torch.int64), valid.reshape(-1)
    blocks, pb = counts.numel(), math.ceil(prefix / 64)
    pre = torch.clamp(prefix - torch.arange(pb, device=device, dtype=torch.int32) * 64, 0, 64)
    vid = torch.stack((counts.clamp_max(64), (counts - 64).clamp_min(0)), dim=-1).reshape(-1)
    valid_k = torch.cat((pre, vid)).to(torch.int32).view(1, -1).contiguous()
    n16, n8, n4 = route_counts(blocks * blocks, sparsity_ratio=w["drop"], nvfp4_ratio=0.0,
                               int8_ratio=0.5, fp16_ratio=0.5)
    scale = 1.0 / math.sqrt(dim)

    def mark():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def reference_layer(book):
        t = [mark()]
        p = ops.prepare_h3_sm120_operands(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                          indices, slot_valid, counts, prefix, qb, False, True, False, True,
                                          True, True, None, None, None)
        t.append(mark())
        prob = ops.sm120_h3_draft_probability(p[0], p[1], p[25], p[26], 0.5)
        ids, low, mid, high = ops.sm120_h3_route_precision(prob, n16, n8, n4, None, None, 0)
        mids, _, mid_c, hi_c = ops.sm120_h3_materialize_route(ids, low, mid, high, qb, pb, 1, True, True)
        t.append(mark())
        ops.sm120_q128_int8_attention_forward(p[17], p[19], p[21], p[2], p[3], p[4], mids, mid_c, hi_c,
                                              p[18], p[20], p[22], valid_k, 0, scale, True)
        t.append(mark())
        ops.sm120_q128_prefix_int8_attention_forward(p[23], p[19], p[21], p[24], p[20], p[22], valid_k,
                                                     prefix, scale)
        t.append(mark())
        book.append(t)

    for _ in range(2):
        reference_layer([])
    torch.cuda.synchronize()
    book = []
    for _ in range(repeats):
        reference_layer(book)
    torch.cuda.synchronize()
    names = ("prepare", "draft+route+materialise", "attention int8+fp16", "prefix rows int8")
    ref = {n: float(np.median([t[i].elapsed_time(t[i + 1]) for t in book])) for i, n in enumerate(names)}
    kw = dict(prefix_tokens=prefix, sparsity_ratio=w["drop"], retained_nvfp4_ratio=0.0,
              retained_int8_ratio=0.5, retained_fp16_ratio=0.5, video_shape=video, layer=0,
              query_block_size=qb, maxpool_weight=0.5)
    for _ in range(2):
        executor.sm100_ragged_attention(q, k, v, **kw)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    executor.collect_stage_events(True)
    start.record()
    for _ in range(repeats):
        executor.sm100_ragged_attention(q, k, v, **kw)
    end.record()
    mine = {kk: vv / repeats for kk, vv in executor.stage_times_ms().items()}
    executor.collect_stage_events(False)
    return {"workload": "configs[1]: prefix 512 + video 21x30x52 (S=33272), H=56, D=128, bf16, Q128, 80% drop, "
                        "max-pool 0.5, INT8/FP16 50/50",
            "reference_kernels_ms": {**{kk: round(vv, 3) for kk, vv in ref.items()},
                                     "sum (no output assembly)": round(sum(ref.values()), 3)},
            "this_library_ms": {**{kk: round(vv, 3) for kk, vv in mine.items()},
                                "whole layer": round(start.elapsed_time(end) / repeats, 3)},
            "note": "reference = its mma.sync kernels recompiled for sm_100a; stage times by CUDA events; this "
                    "library's prefix rows run on a side stream beside draft and route"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    last = None
    # every step is a bounded sample (one head, some query blocks); with many steps the samples get
    # fewer query blocks each, so that the whole run stays within a few minutes
    total_steps = args.warmup + args.steps
    blocks = args.cpu_query_blocks if total_steps <= 5 else max(8, min(args.cpu_query_blocks, 160 // total_steps))
    for i in range(total_steps):
        last = cpu_sample(WORKLOAD, query_blocks=blocks, seed=1 + i)
        if i >= args.warmup:
            times.append(last["layer_seconds"])
    mean_s = sum(times) / len(times)
    w = WORKLOAD
    s = w["prefix"] + math.prod(w["video"])
    value = dense_equivalent_flops(s, w["dim"], w["heads"]) / mean_s / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s dense-equivalent",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s dense-equivalent", "cores": last["cores"],
                         "kind": "port", "extrapolated": True, "sample": last["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s dense-equivalent", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    # Beside the CPU port: the reference's own CUDA kernels on this GPU, where they were built.
    if torch.cuda.is_available() and (ROOT / "oracle" / "_ref" / "_ref_sm120.so").exists():
        try:
            line["reference_kernels_b200"] = reference_kernels_same_gpu()
        except Exception as exc:  # the comparison is extra information, never a reason to fail the arm
            line["reference_kernels_b200"] = {"unavailable": str(exc).splitlines()[0][:160]}
    print(json.dumps(line))


def workload_config(n_gpus: int) -> dict:
    w = WORKLOAD
    return {"workload": "configs[2]: prefix 512 + video 21x48x84 (S=85184), H=56, D=128, bf16, "
                        "Q128, 80% block drop, NVFP4/INT8/FP16 = 40/40/20, prefix K/V and prefix queries INT8",
            "parallelism": f"ulysses{n_gpus}" if n_gpus > 1 else "single",
            "heads_per_gpu": w["heads"] // n_gpus,
            "l2": "inputs (3.66 GB of Q/K/V) exceed the 126 MB L2; no explicit flush"}


def profiled_traffic(heads_local: int, s_total: int):
    """DRAM bytes of one video-attention launch from profiles/attention_kernel_small_case.md
    (a line ``dram_bytes_small_case: <read> <written> heads=<h> tokens=<s>``), scaled by heads x tokens."""
    path = ROOT / "profiles" / "attention_kernel_small_case.md"
    try:
        for text in path.read_text().splitlines():
            if text.startswith("dram_bytes_small_case:"):
                fields = text.split()
                read, written = float(fields[1]), float(fields[2])
                meta = dict(f.split("=") for f in fields[3:])
                scale = heads_local * s_total / (int(meta["heads"]) * int(meta["tokens"]))
                return (read + written) * scale, (
                    f"ncu dram__bytes of the small case in {path.name} ({meta['heads']} heads, "
                    f"{meta['tokens']} tokens), scaled by heads x tokens")
    except (OSError, ValueError, KeyError, IndexError):
        pass
    return None, "no ncu figure in profiles/attention_kernel_small_case.md"


def error_versus_dense(q, k, v, out, head: int = 0, rows: int = 2048) -> dict:
    """Error of the sparse mixed-precision layer against dense fp32 attention of the same inputs
    on `rows` evenly spaced query rows of one head (sparsity and quantisation error together)."""
    s_total, d = q.shape[1], q.shape[3]
    pick = torch.linspace(0, s_total - 1, rows, device=q.device).long()
    qf = q[0, pick, head].float()
    kf, vf = k[0, :, head].float(), v[0, :, head].float()
    dense = torch.softmax(qf @ kf.T / math.sqrt(d), dim=-1) @ vf
    got = out[0, pick, head].float()
    diff = got - dense
    return {"head": head, "rows": rows, "max_abs": float(diff.abs().max()),
            "relative_l2": float(diff.norm() / dense.norm()),
            "cosine": float(torch.nn.functional.cosine_similarity(got.flatten(), dense.flatten(), dim=0)),
            "note": "error of the ALGORITHM at 80% block drop on this synthetic data (Q and K are independent "
                    "random fields, so block-mean routing finds little of the attention mass); the CUDA path "
                    "matches the CPU oracle on the same inputs within 2e-2 / cosine 0.999 (tests)"}


def dense_flash_sample(q, k, v, heads: int = 8) -> dict:
    """Dense bf16 attention of the same sequence through torch's library kernel, for context.

    Timed on `heads` heads (the cost is linear in heads) and scaled to all of them.  It is a
    comparison figure only: nothing of the sparse layer runs through it.
    """
    import torch.nn.functional as F

    h_all = q.shape[2]
    heads = min(heads, h_all)
    qq, kk, vv = (x[:, :, :heads].transpose(1, 2).contiguous() for x in (q, k, v))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        F.scaled_dot_product_attention(qq, kk, vv)
        torch.cuda.synchronize()
        start.record()
        for _ in range(2):
            F.scaled_dot_product_attention(qq, kk, vv)
        end.record()
        torch.cuda.synchronize()
    except RuntimeError as exc:  # out of memory or no kernel for this shape
        return {"unavailable": str(exc).splitlines()[0][:120]}
    ms = start.elapsed_time(end) / 2 * (h_all / heads)
    s_total, d = q.shape[1], q.shape[3]
    return {"ms_per_layer": ms, "tflops": dense_equivalent_flops(s_total, d, h_all) / (ms * 1e-3) / 1e12,
            "impl": f"torch scaled_dot_product_attention (library kernel), {heads} of {h_all} heads timed, scaled"}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch.distributed as dist

    from anemoi_b200 import NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention
    from anemoi_b200 import executor
    from anemoi_b200.build import build
    from anemoi_b200.routing import route_counts

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if rank == 0:
        build()
    if world > 1:
        dist.barrier()

    w = WORKLOAD
    s_total = w["prefix"] + math.prod(w["video"])
    layout = VisualLayout(w["video"], w["prefix"])
    sparse = SparseConfig(w["query_block"], w["drop"], (), w["maxpool"])
    quant = QuantConfig(*w["ratios"], "int8", "int8")

    if world == 1:
        q, k, v = synth_qkv(w, w["heads"], device, seed=0)
    else:
        from anemoi_b200 import ulysses

        rows = ulysses.shard_rows(s_total, world)
        lo = sum(rows[:rank])
        # every rank draws the same seeded tensors head by head and keeps its sequence shard
        q, k, v = synth_qkv(w, w["heads"], device, seed=0, rows=slice(lo, lo + rows[rank]))
    amax = torch.stack([t.float().abs().max() for t in (q, k, v)])
    if world > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    calib = NVFP4Calibration(*[float(a) / (6 * 448) for a in amax.tolist()])

    exchange, exchange_kind = open_exchange(args, world, rows[rank] if world > 1 else 0, w["heads"], w["dim"],
                                            q.dtype, device)

    def layer(qq, kk, vv):
        if world == 1:
            return anemoi_attention(qq, kk, vv, layout=layout, layer=0, sparse_config=sparse,
                                    quant_config=quant, calibration=calib)
        return ulysses.ulysses_anemoi_attention(qq, kk, vv, layout=layout, layer=0, sparse_config=sparse,
                                                quant_config=quant, calibration=calib,
                                                pipeline_groups=args.pipeline_groups, exchange=exchange)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        out = layer(q, k, v)
    barrier()
    if executor.last_status(device) != 0:
        raise SystemExit("attention kernel reported an aborted wait")

    # ---- timed: inputs resident in HBM ----
    from anemoi_b200 import native

    executor.collect_stage_events(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = native.launches_total()
    with ClockSampler(local) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            out = layer(q, k, v)
        end.record()
        barrier()
    ms = start.elapsed_time(end) / args.steps
    launches = (native.launches_total() - launches_before) // args.steps
    stages = {kk: vv / args.steps for kk, vv in executor.stage_times_ms().items()}
    executor.collect_stage_events(False)
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    # ---- timed: end to end from pinned host memory ----
    hq, hk, hv = (torch.empty(x.shape, dtype=x.dtype, pin_memory=True).copy_(x) for x in (q, k, v))
    hout = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
    host_call = None
    if world == 1 or exchange is not None:
        # the library's host-input entry: head groups on three streams, so that the copy of one
        # group runs under the layer of another (heads are independent; same result bit for bit).
        # With N > 1 every rank holds its rows on its host and each head group goes through the
        # peer-store exchange.
        from anemoi_b200 import HostAttention

        # sharded: at least two heads per rank and group (a group's prefix rows are one long CTA per tile)
        group_heads = (args.e2e_group_heads if world == 1
                       else max(-(-args.e2e_group_heads // world) * world, 2 * world))
        host_call = HostAttention(device, group_heads=group_heads, sharded=world > 1)

        def e2e_step():
            host_call(hq, hk, hv, hout, layout=layout, layer=0, sparse_config=sparse,
                      quant_config=quant, calibration=calib)
    else:
        def e2e_step():
            dq, dk, dv = (x.to(device, non_blocking=True) for x in (hq, hk, hv))
            hout.copy_(layer(dq, dk, dv), non_blocking=True)

    for _ in range(min(args.warmup, 2)):
        e2e_step()
    barrier()
    e2e_steps = max(1, min(args.steps, 5))
    start.record()
    for _ in range(e2e_steps):
        e2e_step()
    end.record()
    barrier()
    te = torch.tensor([start.elapsed_time(end) / e2e_steps], device=device)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item())
    e2e_matches = bool(torch.equal(hout.to(device), out)) if host_call is not None else None
    if host_call is not None:
        host_call.close()

    # ---- N > 1: the sharded result against an unsharded run of one head (outside the timing) ----
    sharded_ok = None
    if world > 1:
        head = 0
        parts = [torch.empty(r, w["dim"], dtype=q.dtype, device=device) for r in rows]
        full = []
        for t in (q, k, v):
            dist.all_gather(parts, t[0, :, head].contiguous())
            full.append(torch.cat(parts).view(1, s_total, 1, w["dim"]).clone())
        if rank == 0:
            single = anemoi_attention(*full, layout=layout, layer=0, sparse_config=sparse,
                                      quant_config=quant, calibration=calib)
            sharded_ok = bool(torch.equal(single[0, lo : lo + rows[rank], 0], out[0, :, head]))
        del full, parts

    if rank == 0:
        from anemoi_b200.layout import materialize_ragged_2d_layout

        blocks = materialize_ragged_2d_layout("cpu", frames=w["video"][0], height=w["video"][1],
                                              width=w["video"][2], logical_block=w["query_block"]).video_blocks
        n16, n8, n4 = route_counts(blocks * blocks, sparsity_ratio=w["drop"], nvfp4_ratio=w["ratios"][0],
                                   int8_ratio=w["ratios"][1], fp16_ratio=w["ratios"][2])
        flops = dense_equivalent_flops(s_total, w["dim"], w["heads"])
        peaks, peak_kind = measured_peaks()
        bf16 = float(peaks["bf16_tflops"])
        qb, d, p = w["query_block"], w["dim"], math.ceil(w["prefix"] / 64)
        per_head = 4.0 * d
        f4 = per_head * n4 * qb * qb
        f8 = per_head * (n8 * qb * qb + blocks * qb * 64 * p)
        f16 = per_head * n16 * qb * qb
        heads_local = w["heads"] // world
        video_flops = heads_local * (f4 + f8 + f16)
        # per-dtype tensor peaks relative to the measured bf16 GEMM: 8-bit kinds 2x, NVFP4 4x (nominal ratios)
        mixed_peak = (f4 + f8 + f16) / (f4 / (4 * bf16) + f8 / (2 * bf16) + f16 / bf16)
        attn_ms = stages.get("attention", float("nan"))
        achieved = video_flops / (attn_ms * 1e-3) / 1e12 if attn_ms == attn_ms else None
        # DRAM traffic of one video-attention launch: read from the committed ncu summary of the
        # small profiling case (8 heads of 33,272 tokens) and scaled by heads x tokens; the
        # operands of a head stay L2-resident in both cases, so the traffic is the compulsory
        # read of the records and the write of O.  None when the summary does not carry it.
        traffic, traffic_source = profiled_traffic(heads_local, s_total)
        line = {
            "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s dense-equivalent",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4+int8/e4m3+fp16 (fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world),
            "clocks": clocks.summary(),
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s dense-equivalent",
                    "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(sum(x.numel() * x.element_size() for x in (q, k, v))),
                    "d2h_bytes_per_step": int(out.numel() * out.element_size()),
                    "path": (f"HostAttention: head groups of {args.e2e_group_heads} on three streams, one strided "
                             "copy per group and tensor" if world == 1 else
                             "HostAttention, sharded: per rank and head group, copy in its rows, peer-store exchange, "
                             "layer, exchange back, copy out, on three streams" if host_call is not None else
                             "per rank: copy in its sequence shard, Ulysses layer, copy out"),
                    "equals_device_resident_result": e2e_matches},
            # kernels of this library launched per step, counted by the ctypes layer as it calls them
            # (v_amax, prepare, prefix attention, draft, hist, threshold, rowstat, headscan, emit,
            # attention, assemble; with N > 1 also pack and merge)
            "gpu_launches": launches,
            "stage_ms": stages,
            "roofline": {"bound": "tensor", "kernel": "attention_kernel<128> (video query blocks)",
                         "achieved": achieved, "peak": mixed_peak, "unit": "TFLOP/s",
                         "frac": (achieved / mixed_peak) if achieved else None, "traffic": traffic,
                         "traffic_source": traffic_source,
                         "peak_source": f"{peak_kind} bf16 GEMM {bf16} TFLOP/s x (1, 2, 4) for fp16, 8-bit, NVFP4 "
                                        "cells, weighted by executed FLOPs"},
        }
        # The HBM-side stages against the measured copy bandwidth (and the nominal 8 TB/s): algorithmic
        # bytes / CUDA-event time.  Preparation: Q, K, V read once, V once more for its per-channel
        # amax, every operand record written once.  Routing (draft + route): the pools read, the fp16
        # map written once and read three times (histogram, row counts, lists), the lists written.
        # Draft and route run beside the prefix rows' launch of the side stream, so their event
        # times include the SMs they share with it.
        hbm = float(peaks["hbm_gbs"])
        d_, r_ = w["dim"], blocks
        stages_all = math.ceil(w["prefix"] / 64) + r_ * (qb // 64)
        rec_bytes = heads_local * (r_ * qb * d_ * 2 + stages_all * 2 * 64 * d_ * 2                       # fp16
                                   + (r_ + math.ceil(w["prefix"] / qb)) * qb * d_ + stages_all * 2 * 64 * d_  # int8
                                   + r_ * (qb * d_ // 2 + (d_ // 64) * 512) + stages_all * (64 * d_ + (d_ // 64) * 512 + 512)
                                   + 2 * r_ * d_ * 2)
        in_bytes = heads_local * s_total * d_ * 2 * 4
        route_bytes = heads_local * (4 * r_ * r_ * 2 + 2 * r_ * d_ * 2) + heads_local * 4 * (
            (n16 + n8 + n4) * (qb // 64) + r_ * p)
        prep_ms, rt_ms = stages.get("prepare"), (stages.get("draft", 0.0) + stages.get("route", 0.0))
        if prep_ms and rt_ms:
            line["hbm_stages"] = {
                "prepare": {"bytes": in_bytes + rec_bytes, "GBs": (in_bytes + rec_bytes) / (prep_ms * 1e-3) / 1e9,
                            "frac_of_measured": (in_bytes + rec_bytes) / (prep_ms * 1e-3) / 1e9 / hbm,
                            "frac_of_nominal_8TBs": (in_bytes + rec_bytes) / (prep_ms * 1e-3) / 1e9 / 8000.0},
                "draft_route": {"bytes": route_bytes, "GBs": route_bytes / (rt_ms * 1e-3) / 1e9,
                                "frac_of_measured": route_bytes / (rt_ms * 1e-3) / 1e9 / hbm,
                                "frac_of_nominal_8TBs": route_bytes / (rt_ms * 1e-3) / 1e9 / 8000.0,
                                "note": "the 50.6 MB map stays in L2; the stage is launch- and latency-bound"},
                "peak_source": f"{peak_kind} copy bandwidth {hbm} GB/s"}
        if world == 1:
            from anemoi_b200 import native

            # the library's own tcgen05 probe per MMA kind (128x128 tiles, no-swizzle operands)
            kinds = {k: native.tensor_peak(k, device) for k in native.TENSOR_KINDS}
            measured_mixed = (f4 + f8 + f16) / (f4 / kinds["nvfp4"] + f8 * 0.5 / kinds["i8"] +
                                                f8 * 0.5 / kinds["f8"] + f16 / kinds["f16"])
            line["roofline"]["tcgen05_measured"] = {
                **{k: round(v, 1) for k, v in kinds.items()}, "mixed": round(measured_mixed, 1),
                "frac_of_mixed": (achieved / measured_mixed) if achieved else None,
                "note": "TFLOP/s of the library's tensor-pipe probe per kind; mixed = executed FLOPs weighted "
                        "(QK of the 8-bit cell is kind::i8, its PV kind::f8f6f4)"}
        if world > 1:
            line["sharded_equals_single"] = sharded_ok
            line["config"]["exchange"] = exchange_kind
        if world == 1 and not args.no_dense:
            line["dense_bf16"] = dense_flash_sample(q, k, v)
            line["error_vs_dense_fp32"] = error_versus_dense(q, k, v, out)
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_sample(w, query_blocks=args.cpu_query_blocks)
            line["cpu_baseline"] = {"value": cpu["tflops"], "unit": "TFLOP/s dense-equivalent",
                                    "cores": cpu["cores"], "kind": "port", "extrapolated": True,
                                    "sample": cpu["sample"]}
        print(json.dumps(line))
    if exchange is not None:
        exchange.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def open_exchange(args, world, rows_local, heads, dim, dtype, device):
    """The transport of the Ulysses exchange at N > 1: stores into the peers' memory
    (`--exchange peer`, and `auto` when the set-up succeeds on every rank) or NCCL
    all_to_all_single (`--exchange nccl`, and `auto` otherwise); the JSON line names which."""
    if world == 1:
        return None, "none"
    if args.exchange == "nccl":
        return None, "nccl all_to_all_single + pack/merge kernels"
    from anemoi_b200 import ulysses

    try:
        return (ulysses.PeerExchange(rows_local, heads, dim, dtype, device),
                "stores into the peers' memory (CUDA IPC), flag hand-over, no collective call")
    except RuntimeError as exc:
        if args.exchange == "peer":
            raise
        return None, f"nccl all_to_all_single + pack/merge kernels ({exc})"


# ------------------------------------------------------------------------------------------
# one denoising step of a random-init MiniMax-H3-shaped block stack (the fifth configuration)
# ------------------------------------------------------------------------------------------
def run_dit_step(args) -> None:
    """`--config dit-step`: one denoising step of the stand-in block stack
    (anemoi_b200/h3_stack.py: 50 blocks, width 5,376, 56 x 128 heads) on the 512 + 21x48x84-token
    sequence, sequence-sharded over N GPUs with the Ulysses exchange around every attention and
    `H3MPAAttention` behind it (dense for the first two layers, NVFP4/INT8/FP16 40/40/20 at 80 %
    drop elsewhere).  One JSON line: step time, time inside exchange + attention, its share.
    Not the headline line: `metric` names the step."""
    import torch.distributed as dist

    from anemoi_b200 import ulysses
    from anemoi_b200.adapter import H3MPAAttention, H3MPAConfig
    from anemoi_b200.build import build
    from anemoi_b200.h3_stack import H3BlockStack, H3StackConfig
    from anemoi_b200.producer import fused_qknorm_rope

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if rank == 0:
        build()
    if world > 1:
        dist.barrier()

    w = WORKLOAD
    cfg = H3StackConfig(layers=args.dit_layers)
    s_total = w["prefix"] + math.prod(w["video"])
    rows = ulysses.shard_rows(s_total, world)
    lo = sum(rows[:rank])
    stack = H3BlockStack(cfg, device, seed=0)
    gen = torch.Generator(device=device).manual_seed(100 + rank)
    x = torch.randn(rows[rank], cfg.width, generator=gen, device=device).to(torch.bfloat16)
    pos = torch.arange(lo, lo + rows[rank], device=device, dtype=torch.float32)
    freq = torch.exp(-torch.arange(cfg.rotary_dim // 2, device=device, dtype=torch.float32) * (8.0 / cfg.rotary_dim))
    ang = torch.cat((pos[:, None] * freq[None], pos[:, None] * freq[None]), dim=-1)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    # per-layer NVFP4 tensor scales = amax / (6 * 448) of the layer's Q, K, V, from a calibration
    # pass whose attention just returns V (the activations of the real step differ slightly)
    amax = torch.zeros(cfg.layers, 3, device=device)
    layer_box = [0]

    def calibrate(q, k, v):
        amax[layer_box[0]] = torch.stack([t.float().abs().max() for t in (q, k, v)])
        layer_box[0] += 1
        return v

    stack.step(x, cos, sin, calibrate, norm_rope=fused_qknorm_rope)
    if world > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    scales = (amax / (6 * 448)).clamp_min(1e-8).cpu().tolist()
    attention = H3MPAAttention(
        H3MPAConfig(video_shape=w["video"], prefix_tokens=w["prefix"], sparsity_ratio=w["drop"],
                    query_block_size=w["query_block"], nvfp4_ratio=w["ratios"][0], int8_ratio=w["ratios"][1],
                    fp16_ratio=w["ratios"][2], dense_first_steps=0, dense_first_layers=args.dit_dense_layers,
                    layers_per_step=cfg.layers),
        nvfp4_scales={"scales": {"q_tensor_scale": [r[0] for r in scales],
                                 "k_tensor_scale": [r[1] for r in scales],
                                 "v_tensor_scale": [r[2] for r in scales]}})
    position_ids = torch.empty(s_total, device="meta")
    marks = []

    def on_attention(begin):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        marks.append(e)

    exchange, exchange_kind = open_exchange(args, world, rows[rank], cfg.heads, cfg.head_dim, x.dtype, device)

    def one_step(timestep: float):
        attention.observe(timestep=torch.tensor(timestep), video_indices=None, position_ids=position_ids)
        return stack.step(x, cos, sin, attention, norm_rope=fused_qknorm_rope, on_attention=on_attention,
                          exchange=exchange, fuse_producer=exchange is not None and not args.no_fused_producer)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from anemoi_b200 import executor

    t = 1.0
    for _ in range(args.warmup):
        one_step(t)
        t -= 0.02
    barrier()
    marks.clear()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            out = one_step(t)
            t -= 0.02
        end.record()
        barrier()
    if executor.last_status(device) != 0:
        raise SystemExit("attention kernel reported an aborted wait")
    step_ms = start.elapsed_time(end) / args.steps
    attn_ms = sum(a.elapsed_time(b) for a, b in zip(marks[0::2], marks[1::2])) / args.steps
    both = torch.tensor([step_ms, attn_ms], device=device)
    if world > 1:
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
    if rank == 0:
        stats = attention.stats()
        print(json.dumps({
            "metric": "one denoising step of a random-init MiniMax-H3-shaped block stack, ms", "value": float(both[0]),
            "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": False,
            "scaling": "strong", "data": "synthetic", "dtype": "bf16 GEMMs; nvfp4+int8/e4m3+fp16 attention",
            "attention_and_exchange_ms": float(both[1]), "attention_share": float(both[1] / both[0]),
            "finite": bool(torch.isfinite(out).all()),
            "config": {"workload": "configs[4] stand-in: 512-token prefix + 21x48x84 video tokens, "
                                   f"{cfg.layers} blocks (width {cfg.width}, {cfg.heads}x{cfg.head_dim} heads, "
                                   f"SwiGLU {cfg.ffn_width} assumed, {cfg.rotary_dim} rotary channels assumed), "
                                   f"dense attention in the first {args.dit_dense_layers} layers, sparse "
                                   "NVFP4/INT8/FP16 40/40/20 at 80% drop elsewhere",
                       "parallelism": f"ulysses{world}" if world > 1 else "single", "exchange": exchange_kind,
                       "producer": "inside the exchange's stores" if exchange is not None and not args.no_fused_producer
                                   else "in-place kernel before the exchange",
                       "dense_calls": stats["dense_calls"], "mpa_calls": stats["mpa_calls"]},
            "clocks": clocks.summary()}))
    if exchange is not None:
        exchange.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# kernel sweep (the fourth benchmark configuration): not a bench line, a table
# ------------------------------------------------------------------------------------------
SWEEP_CELLS = {"nvfp4": (1.0, 0.0, 0.0), "int8": (0.0, 1.0, 0.0), "fp16": (0.0, 0.0, 1.0),
               "nvfp4+int8": (0.5, 0.5, 0.0), "nvfp4+fp16": (0.5, 0.0, 0.5),
               "int8+fp16": (0.0, 0.5, 0.5), "nvfp4+int8+fp16": (0.4, 0.4, 0.2)}


def run_sweep(args) -> None:
    """Visual-only 21x48x84 layer over D x query block x drop ratio x cells (x maxpool weight for
    the mixed cell), `--sweep-heads` heads per point.  One JSON line per point: stage times,
    preparation and routing GB/s (algorithmic bytes / CUDA-event time) and the attention
    kernel's executed FLOPs against the mixed tensor peak.  Writes `--sweep-out` as well."""
    from anemoi_b200 import executor
    from anemoi_b200.build import build
    from anemoi_b200.layout import materialize_ragged_2d_layout
    from anemoi_b200.routing import route_counts

    build()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    bf16 = float(peaks["bf16_tflops"])
    video, heads = (21, 48, 84), args.sweep_heads
    s_total = math.prod(video)
    rows = []
    for d in (64, 128):
        w = dict(WORKLOAD, prefix=0, video=video, dim=d, outliers=(17, 53) if d == 64 else (17, 93))
        q, k, v = synth_qkv(w, heads, device, seed=0)
        scales = tuple(float(t.float().abs().max()) / (6 * 448) for t in (q, k, v))
        for qb in (64, 128):
            blocks = materialize_ragged_2d_layout("cpu", frames=video[0], height=video[1], width=video[2],
                                                  logical_block=qb).video_blocks
            for drop in (0.5, 0.8, 0.9):
                for cell, ratios in SWEEP_CELLS.items():
                    for weight in ((0.0, 0.5, 1.0) if cell == "nvfp4+int8+fp16" else (0.0,)):
                        def call():
                            return executor.sm100_ragged_attention(
                                q, k, v, prefix_tokens=0, sparsity_ratio=drop,
                                retained_nvfp4_ratio=ratios[0], retained_int8_ratio=ratios[1],
                                retained_fp16_ratio=ratios[2], video_shape=video, layer=0,
                                query_block_size=qb, maxpool_weight=weight,
                                nvfp4_scales=scales if ratios[0] > 0 else (1.0, 1.0, 1.0),
                                return_parts=True)
                        call()
                        executor.collect_stage_events(True)
                        out, parts = call()
                        st = executor.stage_times_ms()
                        executor.collect_stage_events(False)
                        if executor.last_status(device) != 0 or not bool(torch.isfinite(out).all()):
                            raise SystemExit(f"sweep point failed: D={d} Q={qb} drop={drop} {cell}")
                        n16, n8, n4 = route_counts(blocks * blocks, sparsity_ratio=drop, nvfp4_ratio=ratios[0],
                                                   int8_ratio=ratios[1], fp16_ratio=ratios[2])
                        f4, f8, f16 = (4.0 * d * heads * n * qb * qb for n in (n4, n8, n16))
                        mixed = (f4 + f8 + f16) / (f4 / (4 * bf16) + f8 / (2 * bf16) + f16 / bf16)
                        store = parts["store"].buffers
                        rec_bytes = sum(t.numel() * t.element_size() for t in store.values() if t is not None)
                        in_bytes = 3 * q.numel() * q.element_size() + (v.numel() * 2 if ratios[1] > 0 else 0)
                        route_bytes = (4 * heads * blocks * blocks * 2 + 2 * heads * blocks * d * 2 * (2 if weight else 1)
                                       + parts["lists"].stage_ids.numel() * 4)
                        row = {"D": d, "Q": qb, "drop": drop, "cell": cell, "maxpool": weight, "heads": heads,
                               "stage_ms": {kk: round(vv, 4) for kk, vv in st.items()},
                               "prepare_GBs": round((in_bytes + rec_bytes) / (st["prepare"] * 1e-3) / 1e9, 1),
                               "routing_GBs": round(route_bytes / ((st["draft"] + st["route"]) * 1e-3) / 1e9, 1),
                               "attention_TFLOPs": round((f4 + f8 + f16) / (st["attention"] * 1e-3) / 1e12, 1),
                               "attention_frac_of_mixed_peak": round((f4 + f8 + f16) / (st["attention"] * 1e-3) / 1e12 / mixed, 3)}
                        rows.append(row)
                        print(json.dumps(row), flush=True)
    if args.sweep_out:
        with open(args.sweep_out, "w") as fh:
            fh.write(f"# kernel sweep, visual-only 21x48x84 (S={s_total}), {heads} heads per point, "
                     f"peak = {peak_kind} bf16 {bf16} TFLOP/s x (1,2,4)\n\n")
            fh.write("| D | Q | drop | cell | maxpool | prepare ms | prepare GB/s | draft+route ms | routing GB/s | "
                     "attention ms | executed TFLOP/s | frac of mixed peak |\n|---|---|---|---|---|---|---|---|---|---|---|---|\n")
            for r in rows:
                t = r["stage_ms"]
                fh.write(f"| {r['D']} | {r['Q']} | {r['drop']} | {r['cell']} | {r['maxpool']} | {t['prepare']:.3f} | "
                         f"{r['prepare_GBs']} | {t['draft'] + t['route']:.3f} | {r['routing_GBs']} | {t['attention']:.3f} | "
                         f"{r['attention_TFLOPs']} | {r['attention_frac_of_mixed_peak']} |\n")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-query-blocks", type=int, default=32,
                    help="query blocks of attention timed per CPU sample (evenly spaced over the video)")
    ap.add_argument("--no-dense", action="store_true",
                    help="skip the dense bf16 library attention timed beside the sparse layer")
    ap.add_argument("--e2e-group-heads", type=int, default=4,
                    help="heads per group of the pipelined host-input call (end-to-end number)")
    ap.add_argument("--exchange", choices=("auto", "peer", "nccl"), default="auto",
                    help="N > 1: Ulysses exchange by stores into the peers' memory, by NCCL all-to-all, or "
                         "the first if its set-up succeeds on every rank")
    ap.add_argument("--no-fused-producer", action="store_true",
                    help="dit-step with the peer exchange: run qk-norm + rotary as its own in-place kernel "
                         "instead of inside the exchange's stores")
    ap.add_argument("--pipeline-groups", type=int, default=1,
                    help="head groups whose exchange is pipelined under the attention (N > 1)")
    ap.add_argument("--config", choices=("layer", "dit-step"), default="layer",
                    help="layer: the headline attention-layer benchmark; dit-step: one denoising step of the "
                         "random-init block stack with Ulysses (not the headline line)")
    ap.add_argument("--dit-layers", type=int, default=50)
    ap.add_argument("--dit-dense-layers", type=int, default=2)
    ap.add_argument("--sweep", action="store_true", help="run the kernel sweep instead of the benchmark")
    ap.add_argument("--sweep-heads", type=int, default=4)
    ap.add_argument("--sweep-out", default="")
    ap.add_argument("--profile-case", action="store_true",
                    help="run the small profiling case instead of the benchmark workload")
    args = ap.parse_args()
    if args.profile_case:
        WORKLOAD.update(PROFILE_WORKLOAD)
    if args.sweep:
        run_sweep(args)
    elif args.config == "dit-step":
        run_dit_step(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
