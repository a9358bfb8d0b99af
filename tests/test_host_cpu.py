"""CPU tests: host logic and the oracle against the reference's own known answers.

Known-answer sources inside the reference repository:
  * partition SHA-256 vectors ........ tests/test_mpa_ragged_2d.py:85-146
  * route examples and tie-break ..... tests/test_mpa_ragged_2d.py:156-234
  * E2M1 midpoints, INT8 rounding .... tests/test_sm120_d64_cuda.py:165-193
plus tests/golden/reference_vectors.json, produced by tests/golden/make_golden.py
from the reference's CPU-runnable functions.
"""

import base64
import hashlib
import json
import math
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from anemoi_b200 import (NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout,
                         anemoi_attention)
from anemoi_b200.layout import materialize_ragged_2d_layout
from anemoi_b200.partition import make_ragged_2d_partition
from anemoi_b200.routing import resolve_phases, route_counts, video_phases
from oracle import formats as F
from oracle import prep as P
from oracle import route as R

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = json.loads((ROOT / "tests" / "golden" / "reference_vectors.json").read_text())


def unpack(entry) -> np.ndarray:
    raw = base64.b64decode(entry["b64"])
    return np.frombuffer(raw, dtype=np.dtype(entry["dtype"])).reshape(entry["shape"]).copy()


def sha(blocks) -> str:
    return hashlib.sha256(json.dumps(blocks, separators=(",", ":")).encode()).hexdigest()


# ---- partition ---------------------------------------------------------------------------
REFERENCE_PINNED = {
    (8, 8, 64): "bed7ce3a87c88a80e42bebb28d80ea1d414684177870eda040e6e4af9d9e60f2",
    (16, 16, 64): "797b760414bab5e0ddef088fcc536d6fd86433f0cbc0d08bb51bb86978fcfc4b",
    (24, 40, 64): "465b75da839dd0166793796a4e2ed9a950d3007a55e31b94a8df32e093c8152f",
    (16, 16, 128): "8bfd7ff9cd7ea1baf4c07eb514da757932cea8bcc84d3a4893d34325efef4090",
    (12, 32, 64): "47f7df182539bdfb7175d06d75b67dfeb79d48def654d974304d27627bcc3060",
    (24, 42, 128): "b63bf0e8091a0504cd92d1d8eff2e7f50830fee60d22a78876a521da242ebdd8",
}


@pytest.mark.parametrize("geometry,digest", sorted(REFERENCE_PINNED.items()))
def test_partition_matches_reference_pinned_hashes(geometry, digest):
    part = make_ragged_2d_partition(*geometry, include_adjacency=False)
    assert sha(part.blocks) == digest


def test_partition_matches_reference_outputs():
    for entry in GOLDEN["partition"]:
        h, w, c = entry["geometry"]
        part = make_ragged_2d_partition(h, w, c, include_adjacency=False)
        assert sha(part.blocks) == entry["sha256"], entry["geometry"]
        assert list(part.counts) == entry["counts"]


@pytest.mark.parametrize("geometry", [(7, 20, 64), (24, 42, 64), (13, 29, 128), (1, 77, 64), (40, 3, 64)])
def test_partition_is_exact_balanced_connected_cover(geometry):
    h, w, c = geometry
    part = make_ragged_2d_partition(h, w, c)
    n = math.ceil(h * w / c)
    assert part.block_count == n
    q, r = divmod(h * w, n)
    assert sorted(part.counts) == sorted([q + 1] * r + [q] * (n - r))
    seen = sorted(t for b in part.blocks for t in b)
    assert seen == list(range(h * w))
    for block in part.blocks:
        cells = set(block)
        stack = [block[0]]
        cells.remove(block[0])
        while stack:
            t = stack.pop()
            y, x = divmod(t, w)
            for o in ((y - 1, x), (y + 1, x), (y, x - 1), (y, x + 1)):
                if 0 <= o[0] < h and 0 <= o[1] < w and o[0] * w + o[1] in cells:
                    cells.remove(o[0] * w + o[1])
                    stack.append(o[0] * w + o[1])
        assert not cells
    assert part.adjacency is not None and all(part.adjacency[i][i] for i in range(n))


def test_partition_rejects_bad_arguments():
    with pytest.raises(ValueError):
        make_ragged_2d_partition(0, 4, 64)
    with pytest.raises(ValueError):
        make_ragged_2d_partition(4, 4, 0)
    with pytest.raises(TypeError):
        make_ragged_2d_partition(4, 4, 64, include_adjacency=1)


def test_layout_tables_on_cpu():
    lay = materialize_ragged_2d_layout("cpu", frames=3, height=10, width=14, logical_block=64)
    part = make_ragged_2d_partition(10, 14, 64, include_adjacency=False)
    geo = P.make_geometry(part.blocks, 3, 10, 14, 64, 0)
    assert np.array_equal(lay.indices.numpy(), geo.indices)
    assert np.array_equal(lay.slot_valid.numpy(), geo.slot_valid)
    assert np.array_equal(lay.counts.numpy(), geo.counts)
    assert np.array_equal(lay.inverse.numpy(), geo.inverse)
    # every token owns exactly one valid slot
    assert np.array_equal(geo.indices[geo.inverse], np.arange(3 * 140))
    with pytest.raises(ValueError):
        materialize_ragged_2d_layout("cpu", frames=1, height=4, width=4, logical_block=32)


def test_valid_k_matches_reference_expansion():
    g = GOLDEN["valid_k_q128"]
    geo = P.Geometry(indices=np.zeros(4 * 128, dtype=np.int64), slot_valid=np.ones(4 * 128, dtype=bool),
                     counts=np.array(g["video"][0], dtype=np.int32), inverse=np.zeros(1, dtype=np.int64),
                     query_block=128, prefix_tokens=100)
    assert geo.valid_k().tolist() == g["expanded"][0]


# ---- budgets and phases ------------------------------------------------------------------
def test_route_counts_match_reference():
    for e in GOLDEN["route_counts"]:
        r4, r8, r16 = e["ratios"]
        got = route_counts(e["items"], sparsity_ratio=e["drop"], nvfp4_ratio=r4, int8_ratio=r8, fp16_ratio=r16)
        assert list(got) == e["n"], e
        assert list(R.budgets(e["items"], e["drop"], r4, r8, r16)) == e["n"]


def test_route_counts_validation():
    with pytest.raises(ValueError):
        route_counts(0, sparsity_ratio=0.5, nvfp4_ratio=0, int8_ratio=1, fp16_ratio=0)
    with pytest.raises(ValueError):
        route_counts(4, sparsity_ratio=1.0, nvfp4_ratio=0, int8_ratio=1, fp16_ratio=0)
    with pytest.raises(ValueError):
        route_counts(4, sparsity_ratio=0.5, nvfp4_ratio=0.5, int8_ratio=1, fp16_ratio=0)
    with pytest.raises(TypeError):
        route_counts(4, sparsity_ratio=True, nvfp4_ratio=0, int8_ratio=1, fp16_ratio=0)


def test_phase_resolution():
    assert video_phases(0.4, 0.4, 0.2) == ("nvfp4", "int8", "fp16")
    assert video_phases(0.0, 1.0, 0.0) == ("int8",)
    assert resolve_phases(("nvfp4", "fp16"), 512, "int8") == (("nvfp4", "int8", "fp16"), "int8")
    assert resolve_phases(("int8",), 0, "int8") == (("int8",), None)
    with pytest.raises(ValueError):
        resolve_phases(("int8",), 4, "auto")


# ---- routing oracle against the reference ---------------------------------------------------
def test_route_reference_examples():
    prob = np.zeros((4, 4), dtype=np.float16)
    prob[0] = (7.0, 5.0, 6.0, 4.0)
    n16, n8, n4 = R.budgets(16, 0.75, 0.25, 0.25, 0.50)
    ids, low, mid, high = R.route(prob, n16, n8, n4)
    assert ids[0, :4].tolist() == [3, 1, 0, 2]
    assert (int(low[0]), int(mid[0]), int(high[0])) == (1, 1, 2)
    # all-zero map: ties resolve by row-major index, best rank goes to FP16
    zero = np.zeros((2, 2), dtype=np.float16)
    n16, n8, n4 = R.budgets(4, 0.5, 0.0, 0.5, 0.5)
    ids, low, mid, high = R.route(zero, n16, n8, n4)
    assert (mid.tolist(), high.tolist()) == ([1, 0], [1, 0])
    assert ids[0, :2].tolist() == [1, 0]   # INT8 column 1, then FP16 column 0


def test_route_and_stage_lists_match_reference_outputs():
    for e in GOLDEN["route"]:
        prob = unpack(e["prob_bits"]).view(np.float16)
        ref_ids, ref_low, ref_mid, ref_high = (unpack(e[k]) for k in ("ids", "low", "mid", "high"))
        r = e["r"]
        n16, n8, n4 = R.budgets(r * r, e["drop"], *e["ratios"])
        for h in range(prob.shape[1]):
            ids, low, mid, high = R.route(prob[0, h], n16, n8, n4)
            assert np.array_equal(low, ref_low[0, h]) and np.array_equal(mid, ref_mid[0, h])
            assert np.array_equal(high, ref_high[0, h])
            for i in range(r):
                n = int(low[i] + mid[i] + high[i])
                assert np.array_equal(ids[i, :n], ref_ids[0, h, i, :n])
            for comp in e["compose"]:
                cids, cnv, cmid, chigh = (unpack(comp[k]) for k in ("ids", "nv", "mid", "high"))
                lists = R.stage_lists(ids, low, mid, high, query_block=comp["qb"],
                                      prefix_stages=comp["prefix_blocks"], prefix_phase=comp["prefix_phase"])
                for i, (a, b, c) in enumerate(lists):
                    assert (len(a), len(b), len(c)) == (int(cnv[0, h, i]), int(cmid[0, h, i]), int(chigh[0, h, i]))
                    got = np.concatenate((a, b, c))
                    want = cids[0, h, i, : got.size]
                    if comp["prefix_phase"] == "fp16" and comp["prefix_blocks"]:
                        # The reference stores FP16-phase prefix stages at the tail of the row but
                        # its kernel executes them first (q64_attention_phase_composer.inl:1050-1054);
                        # the lists here are in execution order.
                        p = comp["prefix_blocks"]
                        head = want[: len(a) + len(b)]
                        want = np.concatenate((head, want[-p:], want[len(head) : -p]))
                    assert np.array_equal(got, want)


def test_pools_and_probability_against_reference():
    for e in GOLDEN["pool"]:
        block, dim = e["block"], e["dim"]
        x = unpack(e["x_bits"]).view(np.float16)[0, 0]
        counts = np.array(e["counts"][0], dtype=np.int32)
        geo = P.Geometry(indices=np.zeros(1, dtype=np.int64), slot_valid=np.ones(1, dtype=bool), counts=counts,
                         inverse=np.zeros(1, dtype=np.int64), query_block=block, prefix_tokens=0)
        mean = P.mean_pool(x, geo)
        mx = P.max_pool(x, geo)
        ref_mean = unpack(e["mean_bits"]).view(np.float16)[0, 0]
        ref_max = unpack(e["max_bits"]).view(np.float16)[0, 0]
        assert np.array_equal(mx.view(np.uint16), ref_max.view(np.uint16))
        assert np.abs(mean.astype(np.float32) - ref_mean.astype(np.float32)).max() <= 2e-3
        ref_prob = unpack(e["prob_bits"]).view(np.float16)[0, 0].astype(np.float32)
        got = R.draft_probability(ref_mean, ref_max).astype(np.float32)
        assert np.abs(got - ref_prob).max() <= 5e-4
        plain = R.draft_probability_plain(ref_mean, ref_max).astype(np.float32)
        assert np.abs(plain - ref_prob).max() <= 5e-4


def test_canonical_exp_is_accurate():
    t = -np.abs(np.random.default_rng(1).standard_normal(4096).astype(np.float32)) * 20
    got = R.exp_canonical(t).astype(np.float64)
    want = np.exp(t.astype(np.float64))
    assert np.max(np.abs(got - want) / want) < 1e-5   # argument rounding dominates for |t| ~ 70
    assert R.exp_canonical(np.float32(0.0)) == np.float32(1.0)


# ---- number formats ---------------------------------------------------------------------------
def test_e2m1_midpoints_tie_to_even_code():
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    assert F.e2m1_encode(mids).tolist() == [0, 2, 2, 4, 4, 6, 6]
    assert F.e2m1_encode(-mids).tolist() == [8, 10, 10, 12, 12, 14, 14]
    assert F.e2m1_encode(np.array([100.0, -100.0], dtype=np.float32)).tolist() == [7, 15]
    assert np.array_equal(F.e2m1_decode(np.arange(8, dtype=np.uint8)), F.E2M1_MAGNITUDES)


def test_e4m3_matches_torch_and_saturates():
    x = torch.randn(50000, generator=torch.Generator().manual_seed(3)) * 60
    want = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(F.e4m3_encode(x.numpy()), want)
    assert F.e4m3_encode(np.array([1e9, -1e9, 464.1], dtype=np.float32)).tolist() == [0x7E, 0xFE, 0x7E]
    every = np.arange(256, dtype=np.uint8)
    keep = (every & 0x7F) != 0x7F
    assert np.array_equal(F.e4m3_encode(F.e4m3_decode(every[keep])), every[keep] & np.where(F.e4m3_decode(every[keep]) == 0, 0x80 | 0, 0xFF))


def test_int8_rounds_half_away_from_zero():
    rows = np.zeros((64, 64), dtype=np.float16)
    rows[0, 0] = 127.0
    rows[0, 1] = 0.5
    rows[0, 2] = -0.5
    rows[0, 3] = 1.49
    codes, scale = P.int8_quantise(rows, 64)
    assert scale[0] == np.float32(127.0) / np.float32(127.0) + np.float32(1e-7)
    assert codes[0, :4].tolist() == [127, 0, 0, 1]   # 0.5/scale is just below 0.5


def test_nvfp4_quantise_roundtrip_and_zero_groups():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((8, 64)).astype(np.float16)
    x[3] = 0
    codes, sf = F.nvfp4_quantise(x, 0.01, axis=-1)
    assert codes.shape == (8, 64) and sf.shape == (8, 4)
    assert not codes[3].any() and not sf[3].any()
    back = F.nvfp4_dequantise(codes, sf, 0.01)
    assert np.abs(back - x.astype(np.float32)).max() < 0.6
    cv, sv = F.nvfp4_quantise(x.T.copy(), 0.01, axis=0)
    assert np.array_equal(cv.T, codes) and np.array_equal(sv.T, sf)


# ---- public API contract ---------------------------------------------------------------------------
def test_api_validation_errors():
    q = torch.zeros(1, 16, 2, 64, dtype=torch.float16)
    lay = VisualLayout((1, 4, 4))
    with pytest.raises(ValueError):
        anemoi_attention(q, q, q, torch.zeros(1), layout=lay, layer=0)
    with pytest.raises(ValueError):
        anemoi_attention(q, q, q, layout=lay, layer=0, dropout_p=0.1)
    with pytest.raises(ValueError):
        anemoi_attention(q, q, q, layout=lay, layer=0, is_causal=True)
    with pytest.raises(TypeError):
        anemoi_attention(q, q, q, layout=(1, 4, 4), layer=0)
    with pytest.raises(ValueError):
        anemoi_attention(q, q, q, layout=lay, layer=-1)
    with pytest.raises(ValueError):
        anemoi_attention(q, q, q, layout=VisualLayout((1, 4, 5)), layer=0)
    with pytest.raises(ValueError):
        anemoi_attention(q, q, q, layout=lay, layer=0, scale=0.3)
    with pytest.raises(TypeError):
        anemoi_attention(q, q, q, layout=lay, layer=0, calibration=(1.0, 1.0, 1.0))
    with pytest.raises(RuntimeError):   # CPU tensors: no fallback path exists
        anemoi_attention(q, q, q, layout=lay, layer=0)


def test_config_dataclasses_validate_like_the_reference():
    with pytest.raises(ValueError):
        VisualLayout((4, 4))
    with pytest.raises(ValueError):
        VisualLayout((1, 4, 4), prefix_tokens=-1)
    assert VisualLayout((2, 3, 4), 5).sequence_tokens == 29
    with pytest.raises(ValueError):
        SparseConfig(query_block_size=32)
    with pytest.raises(ValueError):
        SparseConfig(sparsity_ratio=1.0)
    with pytest.raises(TypeError):
        SparseConfig(maxpool_weight=True)
    with pytest.raises(ValueError):
        SparseConfig(maxpool_weight=1.5)
    with pytest.raises(TypeError):
        SparseConfig(layer_sparsity_bands=((0, 2),))
    with pytest.raises(ValueError):
        SparseConfig(layer_sparsity_bands=((0, 4, 0.5), (3, 6, 0.5)))
    cfg = SparseConfig(layer_sparsity_bands=((0, 2, 0.5), (4, 6, 0.9)))
    assert [cfg.sparsity_for_layer(i) for i in (0, 1, 2, 4, 5, 6)] == [0.5, 0.5, 0.8, 0.9, 0.9, 0.8]
    with pytest.raises(ValueError):
        QuantConfig(nvfp4_ratio=0.5, int8_ratio=0.6)
    with pytest.raises(ValueError):
        QuantConfig(prefix_kv_precision="auto")
    with pytest.raises(ValueError):
        QuantConfig(prefix_query_precision="nvfp4")
    with pytest.raises(ValueError):
        NVFP4Calibration(q_scale=0.0)
    assert NVFP4Calibration(2, 3, 4).scales == (2.0, 3.0, 4.0)


# ---- C ABI ---------------------------------------------------------------------------
def test_library_exports_every_declared_symbol(native_library):
    header = (ROOT / "include" / "anemoi_sm100.h").read_text()
    declared = sorted(set(re.findall(r"\b(anemoi_sm100_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(native_library, name), name
    from anemoi_b200 import native

    assert sorted(native.EXPORTED) == declared
    assert native_library.anemoi_sm100_arch() == 100


def test_operand_sizes_and_argument_checks(native_library):
    import ctypes as C

    from anemoi_b200 import native

    s = native.Shape(heads=2, head_dim=128, query_block=128, seq_tokens=512 + 1008, prefix_tokens=512,
                     video_blocks=8, has_nvfp4=1, has_int8=1, has_fp16=1, has_prefix_query_int8=1,
                     has_maxpool=0, input_is_bf16=1, q_global_scale=1.0, k_global_scale=1.0, v_global_scale=1.0)
    stages = 8 + 16
    size = lambda which: native_library.anemoi_sm100_operand_bytes(C.byref(s), which)
    assert size(native.BUF_Q_FP16) == 2 * 8 * 128 * 128 * 2
    assert size(native.BUF_KV_FP16) == 2 * stages * 2 * 64 * 128 * 2
    assert size(native.BUF_Q_INT8) == 2 * (8 + 4) * 128 * 128
    assert size(native.BUF_KV_NVFP4) == 2 * stages * (64 * 128 + 2 * 512 + 512)
    assert size(native.BUF_POOL) == 2 * 8 * 128 * 2
    s.head_dim = 96
    assert size(native.BUF_Q_FP16) < 0
    s.head_dim = 128
    # null pointers are rejected before any launch
    assert native_library.anemoi_sm100_prepare(C.byref(s), None, None, None, None, None, None, None, None) == -1
    assert native_library.anemoi_sm100_route(C.byref(s), None, 1, 1, 1, 0, None, 0, None, None, None, 0, None) == -1
    assert native_library.anemoi_sm100_merge_heads(None, None, 4, 2, 2, 128, None) == -1


def test_nvtx_switch_takes_only_bools():
    from anemoi_b200 import executor

    with pytest.raises(TypeError):
        executor.set_profile_nvtx("yes")
    executor.set_profile_nvtx(False)
