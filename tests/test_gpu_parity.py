"""GPU parity: every stage of the sm_100a path against the CPU oracle, through the C ABI."""

import math

import numpy as np
import pytest
import torch

from tests.helpers import Records, compare_metrics, smooth_fields

pytestmark = pytest.mark.gpu

CASES = [
    # name, video_shape, prefix, H, D, QB, dtype, ratios(nv,i8,f16), drop, w, pkv, pq
    ("cfg1", (4, 16, 16), 0, 4, 64, 64, torch.float16, (0.0, 1.0, 0.0), 0.8, 0.0, "int8", "int8"),
    ("q128_i8f16_prefix", (3, 12, 20), 100, 3, 128, 128, torch.bfloat16, (0.0, 0.5, 0.5), 0.8, 0.5, "int8", "int8"),
    ("q128_mixed_prefix", (3, 12, 20), 70, 2, 128, 128, torch.bfloat16, (0.4, 0.4, 0.2), 0.7, 0.0, "int8", "int8"),
    ("q64_mixed", (2, 10, 14), 0, 2, 64, 64, torch.float16, (0.4, 0.4, 0.2), 0.5, 1.0, "int8", "int8"),
    ("q64_d128_nv", (2, 10, 14), 33, 2, 128, 64, torch.bfloat16, (1.0, 0.0, 0.0), 0.6, 0.0, "nvfp4", "fp16"),
    ("q128_d64_f16", (2, 12, 12), 64, 2, 64, 128, torch.float16, (0.0, 0.0, 1.0), 0.5, 0.0, "fp16", "fp16"),
    ("q128_nv_f16_pint8", (2, 12, 12), 40, 2, 128, 128, torch.bfloat16, (0.5, 0.0, 0.5), 0.5, 0.25, "int8", "fp16"),
    # the NVFP4+INT8 cell (no FP16 phase), prefixed and visual-only, both query blocks and head dims
    ("q128_nv_i8_prefix", (3, 12, 20), 70, 2, 128, 128, torch.bfloat16, (0.5, 0.5, 0.0), 0.7, 0.0, "int8", "int8"),
    ("q64_d64_nv_i8", (2, 10, 14), 0, 2, 64, 64, torch.float16, (0.5, 0.5, 0.0), 0.5, 0.0, "int8", "int8"),
    # the NVFP4 phase holds nothing but the prefix stages
    ("q128_i8_prefix_nvfp4", (2, 12, 12), 40, 2, 128, 128, torch.bfloat16, (0.0, 1.0, 0.0), 0.5, 0.0, "nvfp4", "int8"),
    # Q128 blocks of 64 real keys: every second stage of a block is fully masked (valid_k == 0)
    ("q128_half_blocks", (5, 8, 8), 20, 2, 128, 128, torch.bfloat16, (0.3, 0.4, 0.3), 0.4, 0.0, "int8", "int8"),
    # rest of the cell x head-dim x query-block matrix
    ("q128_d64_nv", (2, 12, 12), 0, 2, 64, 128, torch.float16, (1.0, 0.0, 0.0), 0.5, 0.0, "int8", "int8"),
    ("q64_d128_i8_prefix", (2, 10, 14), 50, 2, 128, 64, torch.bfloat16, (0.0, 1.0, 0.0), 0.6, 0.0, "int8", "int8"),
    ("q64_d128_f16", (2, 10, 14), 0, 2, 128, 64, torch.bfloat16, (0.0, 0.0, 1.0), 0.6, 0.0, "int8", "int8"),
    ("q64_d64_nv_f16_prefix", (2, 10, 14), 30, 2, 64, 64, torch.float16, (0.5, 0.0, 0.5), 0.5, 0.0, "fp16", "fp16"),
    ("q64_d64_i8_f16", (2, 10, 14), 0, 2, 64, 64, torch.float16, (0.0, 0.5, 0.5), 0.5, 0.5, "int8", "int8"),
    ("q64_d128_mixed_prefix", (2, 10, 14), 90, 2, 128, 64, torch.bfloat16, (0.4, 0.4, 0.2), 0.5, 0.0, "int8", "int8"),
    ("q128_d64_mixed", (3, 12, 20), 0, 2, 64, 128, torch.float16, (0.4, 0.4, 0.2), 0.6, 0.0, "int8", "int8"),
    ("q128_d64_i8_prefix", (2, 12, 12), 130, 2, 64, 128, torch.float16, (0.0, 1.0, 0.0), 0.5, 0.0, "int8", "int8"),
    # 99 % of the block pairs dropped: the global budget of a head (3 of 256 pairs) leaves most
    # query blocks with an empty list
    ("q64_empty_rows", (4, 16, 16), 0, 2, 64, 64, torch.float16, (0.0, 0.5, 0.5), 0.99, 0.0, "int8", "int8"),
]


def _run(case):
    from anemoi_b200.executor import sm100_ragged_attention
    from anemoi_b200.partition import make_ragged_2d_partition
    from oracle import pipeline as PL, prep as P

    name, vs, prefix, H, D, QB, dtype, ratios, drop, w, pkv, pq = case
    f, hh, ww = vs
    outl = (17, 53) if D == 64 else (17, 93)
    q, k, v = smooth_fields(f, hh, ww, H, D, prefix, seed=0, outliers=outl if dtype == torch.bfloat16 else (), dtype=dtype)
    amax = [float(t.float().abs().max()) / (6 * 448) for t in (q, k, v)]
    scales = tuple(amax) if ratios[0] > 0 or pkv == "nvfp4" else (1.0, 1.0, 1.0)
    qd, kd, vd = (t.cuda() for t in (q, k, v))
    out, parts = sm100_ragged_attention(
        qd, kd, vd, prefix_tokens=prefix, sparsity_ratio=drop, retained_nvfp4_ratio=ratios[0],
        retained_int8_ratio=ratios[1], retained_fp16_ratio=ratios[2], video_shape=vs, layer=0,
        query_block_size=QB, prefix_kv_precision=pkv, prefix_query_precision=pq, maxpool_weight=w,
        nvfp4_scales=scales, return_parts=True)
    torch.cuda.synchronize()
    assert int(parts["status"].item()) == 0, "a bounded wait inside the attention kernel gave up"
    part = make_ragged_2d_partition(hh, ww, QB, include_adjacency=False)
    geo = P.make_geometry(part.blocks, f, hh, ww, QB, prefix)
    oracle = []
    for h in range(H):
        o, pr = PL.head_attention(q[0, :, h], k[0, :, h], v[0, :, h], geo, sparsity=drop, ratios=ratios,
                                  prefix_kv_precision=pkv, prefix_query_precision=pq, maxpool_weight=w,
                                  global_scales=scales, return_parts=True)
        oracle.append((o, pr))
    return out, parts, oracle, geo


@pytest.fixture(scope="module", params=CASES, ids=[c[0] for c in CASES])
def run(request, native_library):
    return request.param, _run(request.param)


def test_layout_tables(run):
    case, (out, parts, oracle, geo) = run
    lay = parts["layout"]
    assert np.array_equal(lay.indices.cpu().numpy(), geo.indices)
    assert np.array_equal(lay.counts.cpu().numpy(), geo.counts)
    assert np.array_equal(lay.inverse.cpu().numpy(), geo.inverse)
    assert np.array_equal(parts["valid_k"].cpu().numpy(), geo.valid_k())


def test_prepare_bit_exact(run):
    case, (out, parts, oracle, geo) = run
    shape, store = parts["shape"], parts["store"]
    for h in range(shape.heads):
        ops = oracle[h][1]["ops"]
        rec = Records(store, shape, h)
        assert np.array_equal(rec.b["q_pool"][h].view(np.uint16), ops.q_pool.view(np.uint16))
        assert np.array_equal(rec.b["k_pool"][h].view(np.uint16), ops.k_pool.view(np.uint16))
        if shape.has_maxpool:
            assert np.array_equal(rec.b["q_max_pool"][h].view(np.uint16), ops.q_max.view(np.uint16))
            assert np.array_equal(rec.b["k_max_pool"][h].view(np.uint16), ops.k_max.view(np.uint16))
        if shape.has_fp16:
            kk, vv = rec.kv_fp16()
            assert np.array_equal(rec.q_fp16().view(np.uint16), ops.q16.view(np.uint16))
            assert np.array_equal(kk.view(np.uint16), ops.k16.view(np.uint16))
            assert np.array_equal(vv.view(np.uint16), ops.v16.view(np.uint16))
        if shape.has_int8:
            qc, qs = rec.q_int8()
            kc, ks, vc, vsc = rec.kv_int8()
            assert np.array_equal(qs, ops.q_i8_scale) and np.array_equal(qc, ops.q_i8)
            assert np.array_equal(ks, ops.k_i8_scale) and np.array_equal(kc, ops.k_i8)
            assert np.array_equal(vsc, ops.v_e4m3_scale) and np.array_equal(vc, ops.v_e4m3)
            if shape.has_prefix_query_int8:
                pc, ps = rec.q_int8(prefix=True)
                assert np.array_equal(ps, ops.pq_i8_scale) and np.array_equal(pc, ops.pq_i8)
        if shape.has_nvfp4:
            qc, qsf = rec.q_nvfp4()
            kc, ksf, vc, vsf = rec.kv_nvfp4()
            assert np.array_equal(qsf, ops.q4_sf) and np.array_equal(qc, ops.q4)
            assert np.array_equal(ksf, ops.k4_sf) and np.array_equal(kc, ops.k4)
            assert np.array_equal(vsf, ops.v4_sf) and np.array_equal(vc, ops.v4)


def test_probability_bit_exact(run):
    from oracle import route as R

    case, (out, parts, oracle, geo) = run
    prob = parts["prob"].cpu().numpy()
    w = case[9]
    for h in range(prob.shape[0]):
        assert np.array_equal(prob[h].view(np.uint16), oracle[h][1]["prob"].view(np.uint16))
        ops = oracle[h][1]["ops"]
        plain = R.draft_probability_plain(ops.q_pool, ops.k_pool, ops.q_max, ops.k_max, w)
        assert np.abs(prob[h].astype(np.float32) - plain.astype(np.float32)).max() <= 5e-4


def test_route_lists_bit_exact(run):
    case, (out, parts, oracle, geo) = run
    lists = parts["lists"]
    off = lists.row_offset.cpu().numpy()
    cnt = lists.row_counts.cpu().numpy()
    ids = lists.stage_ids.cpu().numpy()
    for h in range(off.shape[0]):
        expect = oracle[h][1]["lists"]
        assert parts["budgets"] == oracle[h][1]["budgets"]
        for i, (nv, i8, hi) in enumerate(expect):
            assert tuple(cnt[h, i, :3]) == (len(nv), len(i8), len(hi)), (h, i)
            got = ids[h, off[h, i] : off[h, i] + cnt[h, i, :3].sum()]
            assert np.array_equal(got, np.concatenate((nv, i8, hi))), (h, i)


def test_launch_order_is_longest_first(run):
    """The fourth entry of row_counts lists a head's query blocks (1-based) by descending list
    length, ties by block index: the order in which the attention kernel launches them."""
    case, (out, parts, oracle, geo) = run
    cnt = parts["lists"].row_counts.cpu().numpy()
    for h in range(cnt.shape[0]):
        total = cnt[h, :, :3].sum(axis=1)
        want = sorted(range(len(total)), key=lambda i: (-int(total[i]), i))
        assert (cnt[h, :, 3] - 1).tolist() == want


def test_attention_within_tolerance(run):
    case, (out, parts, oracle, geo) = run
    packed = parts["packed"].cpu().numpy()
    cnt = parts["lists"].row_counts.cpu().numpy()
    QB = parts["shape"].query_block
    worst = (0.0, 1.0)
    for h in range(packed.shape[0]):
        want = oracle[h][1]["packed"]
        for i in range(cnt.shape[1]):
            if cnt[h, i, :3].sum() == 0:
                continue
            rows = slice(i * QB, i * QB + int(geo.counts[i]))
            ma, cos, _ = compare_metrics(packed[h, rows], want[rows])
            worst = (max(worst[0], ma), min(worst[1], cos))
    assert worst[0] <= 2e-2 and worst[1] >= 0.999, worst


def test_empty_lists_give_positive_zero(run):
    """Query blocks whose three counts are all zero are never touched by the attention kernel;
    the assembly writes +0 for their tokens (reference: csrc/attention/cuda/sm89/
    output_assembly.cu:272-291, tests/test_sm120_d64_cuda.py:236-258): no NaN, sign bit clear."""
    case, (out, parts, oracle, geo) = run
    cnt = parts["lists"].row_counts.cpu().numpy()
    QB = parts["shape"].query_block
    prefix = case[2]
    bits = out[0].view(torch.int16).cpu().numpy()
    empty_blocks = 0
    for h in range(cnt.shape[0]):
        for i in range(cnt.shape[1]):
            if cnt[h, i, :3].sum() != 0:
                continue
            empty_blocks += 1
            tokens = geo.indices[i * QB : i * QB + int(geo.counts[i])]
            assert (bits[prefix + tokens, h] == 0).all(), (h, i)
    if case[0] == "q64_empty_rows":
        assert empty_blocks >= 10


def test_output_within_tolerance(run):
    case, (out, parts, oracle, geo) = run
    got = out[0].float().cpu().numpy()
    for h in range(got.shape[1]):
        want = oracle[h][0].astype(np.float32)
        ma, cos, rel = compare_metrics(got[:, h], want)
        assert ma <= 2e-2 and cos >= 0.999, (h, ma, cos, rel)
    assert not np.isnan(got).any()


def test_error_versus_dense_attention_is_reported(run, record_property):
    """Error of the sparse mixed-precision result against dense fp64 attention of the same
    inputs: reported per case, and the GPU path must be as far from dense as the oracle is
    (the sparsity and quantisation error belong to the algorithm, not to the implementation)."""
    from oracle.attention import dense_reference

    case, (out, parts, oracle, geo) = run
    name, vs, prefix, H, D, QB, dtype, ratios, drop, w, pkv, pq = case
    f, hh, ww = vs
    outl = (17, 53) if D == 64 else (17, 93)
    q, k, v = smooth_fields(f, hh, ww, H, D, prefix, seed=0, outliers=outl if dtype == torch.bfloat16 else (), dtype=dtype)
    got = out[0].float().cpu().numpy()
    h = 0
    dense = dense_reference(q[0, :, h].float().numpy(), k[0, :, h].float().numpy(), v[0, :, h].float().numpy())
    ma_g, cos_g, rel_g = compare_metrics(got[:, h], dense)
    ma_o, cos_o, rel_o = compare_metrics(oracle[h][0].astype(np.float32), dense)
    record_property("dense_error", {"case": name, "gpu": (ma_g, cos_g, rel_g), "oracle": (ma_o, cos_o, rel_o)})
    print(f"[{name}] vs dense fp64: gpu max_abs={ma_g:.4f} cos={cos_g:.5f} rel={rel_g:.4f} | "
          f"oracle max_abs={ma_o:.4f} cos={cos_o:.5f} rel={rel_o:.4f}")
    assert abs(rel_g - rel_o) <= 5e-3 and abs(cos_g - cos_o) <= 1e-3


def test_public_api_matches_executor(run):
    from anemoi_b200 import (NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout,
                             anemoi_attention)

    case, (out, parts, oracle, geo) = run
    name, vs, prefix, H, D, QB, dtype, ratios, drop, w, pkv, pq = case
    if pq == "int8" and ratios[1] == 0.0 and prefix:
        pytest.skip("prefix-query INT8 without an INT8 phase is rejected by the API")
    f, hh, ww = vs
    outl = (17, 53) if D == 64 else (17, 93)
    q, k, v = smooth_fields(f, hh, ww, H, D, prefix, seed=0, outliers=outl if dtype == torch.bfloat16 else (), dtype=dtype)
    s = parts["shape"]
    calib = NVFP4Calibration(s.q_global_scale, s.k_global_scale, s.v_global_scale)
    again = anemoi_attention(
        q.cuda(), k.cuda(), v.cuda(), layout=VisualLayout(vs, prefix), layer=3,
        sparse_config=SparseConfig(QB, drop, (), w),
        quant_config=QuantConfig(ratios[0], ratios[1], ratios[2], pkv, pq), calibration=calib)
    assert torch.equal(again, out)


@pytest.mark.parametrize("index", [1, 2])
def test_repeated_calls_are_bit_identical(native_library, index):
    """Run-to-run determinism (40 calls): a lost barrier phase would show up here as a changed
    warp of output rows."""
    from anemoi_b200.executor import last_status, sm100_ragged_attention

    name, vs, prefix, H, D, QB, dtype, ratios, drop, w, pkv, pq = CASES[index]
    f, hh, ww = vs
    q, k, v = smooth_fields(f, hh, ww, H, D, prefix, seed=1, outliers=(17, 93), dtype=dtype)
    qd, kd, vd = (t.cuda() for t in (q, k, v))
    first = None
    for _ in range(40):
        out = sm100_ragged_attention(
            qd, kd, vd, prefix_tokens=prefix, sparsity_ratio=drop, retained_nvfp4_ratio=ratios[0],
            retained_int8_ratio=ratios[1], retained_fp16_ratio=ratios[2], video_shape=vs, layer=0,
            query_block_size=QB, prefix_kv_precision=pkv, prefix_query_precision=pq,
            maxpool_weight=w, nvfp4_scales=(0.01, 0.01, 0.002))
        if first is None:
            first = out.clone()
        else:
            assert torch.equal(out, first)
    assert last_status() == 0
