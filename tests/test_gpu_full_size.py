"""GPU parity at the full sequence lengths of the two large configurations, two heads each:
prefix 512 + video 21x48x84 (D = 128, Q128, NVFP4/INT8/FP16 40/40/20, 80 % drop) and prefix 512 +
video 21x30x52 (Q128, max-pool weight 0.5, INT8/FP16 50/50).  The whole probability map and every
routing list of one head are bit-exact against the oracle; 16 query blocks spread over the video
and all prefix rows of that head are within tolerance; the size-independent properties hold
(budgets, sortedness, head independence, repeatability)."""

import numpy as np
import pytest
import torch

from tests.helpers import compare_metrics, smooth_fields

pytestmark = pytest.mark.gpu

PREFIX, HEADS, D, QB, DROP = 512, 2, 128, 128, 0.8
CONFIGS = {
    # name: video shape, ratios (nvfp4, int8, fp16), max-pool weight
    "1344x768": ((21, 48, 84), (0.4, 0.4, 0.2), 0.0),
    "832x480": ((21, 30, 52), (0.0, 0.5, 0.5), 0.5),
}


@pytest.fixture(scope="module", params=list(CONFIGS), ids=list(CONFIGS))
def full(request, native_library):
    from anemoi_b200.executor import sm100_ragged_attention

    video, ratios, weight = CONFIGS[request.param]
    q, k, v = smooth_fields(*video, HEADS, D, PREFIX, seed=11, outliers=(17, 93), dtype=torch.bfloat16)
    scales = tuple(float(t.float().abs().max()) / (6 * 448) for t in (q, k, v)) if ratios[0] else (1.0, 1.0, 1.0)
    kw = dict(prefix_tokens=PREFIX, sparsity_ratio=DROP, retained_nvfp4_ratio=ratios[0],
              retained_int8_ratio=ratios[1], retained_fp16_ratio=ratios[2], video_shape=video, layer=0,
              query_block_size=QB, nvfp4_scales=scales, maxpool_weight=weight)
    qd, kd, vd = (t.cuda() for t in (q, k, v))
    out, parts = sm100_ragged_attention(qd, kd, vd, return_parts=True, **kw)
    torch.cuda.synchronize()
    assert int(parts["status"].item()) == 0
    return dict(q=q, k=k, v=v, scales=scales, kw=kw, out=out, parts=parts, dev=(qd, kd, vd),
                video=video, ratios=ratios, weight=weight)


def test_lists_meet_the_budgets_and_are_sorted(full):
    parts = full["parts"]
    n16, n8, n4 = parts["budgets"]
    lists = parts["lists"]
    off, cnt, ids = (t.cpu().numpy() for t in (lists.row_offset, lists.row_counts, lists.stage_ids))
    blocks, stages = cnt.shape[1], 8 + 2 * cnt.shape[1]
    for h in range(cnt.shape[0]):
        # every retained 128-key block is two stages; the 8 prefix stages ride in the INT8 phase
        assert cnt[h, :, 0].sum() == 2 * n4 and cnt[h, :, 2].sum() == 2 * n16
        assert cnt[h, :, 1].sum() == 2 * n8 + 8 * blocks
        for i in range(0, blocks, 37):
            a = off[h, i]
            for c in cnt[h, i, :3]:
                seg = ids[h, a : a + c]
                assert (np.diff(seg) > 0).all() and (seg >= 0).all() and (seg < stages).all()
                a += c
    assert torch.isfinite(full["out"]).all()


def test_head_zero_matches_the_oracle(full):
    from anemoi_b200.partition import make_ragged_2d_partition
    from oracle import attention as A, prep as P, route as R
    from oracle.pipeline import resolve

    q, k, v, parts = full["q"], full["k"], full["v"], full["parts"]
    video, ratios, weight = full["video"], full["ratios"], full["weight"]
    part = make_ragged_2d_partition(video[1], video[2], QB, include_adjacency=False)
    geo = P.make_geometry(part.blocks, *video, QB, PREFIX)
    _, active, prefix_phase = resolve(*ratios, PREFIX, "int8")
    ops = P.prepare_head(q[0, :, 0], k[0, :, 0], v[0, :, 0], geo, has_nvfp4="nvfp4" in active,
                         has_int8=True, has_prefix_query_int8=True, has_maxpool=weight != 0.0,
                         global_scales=full["scales"])
    prob = R.draft_probability(ops.q_pool, ops.k_pool, ops.q_max, ops.k_max, weight)
    got_prob = parts["prob"][0].cpu().numpy()
    assert np.array_equal(got_prob.view(np.uint16), prob.view(np.uint16))        # whole R x R map
    rr = geo.video_blocks
    n16, n8, n4 = R.budgets(rr * rr, DROP, *ratios)
    assert (n16, n8, n4) == tuple(parts["budgets"])
    ids, low, mid, high = R.route(prob, n16, n8, n4)
    want = R.stage_lists(ids, low, mid, high, query_block=QB, prefix_stages=geo.prefix_stages,
                         prefix_phase=prefix_phase)
    lists = parts["lists"]
    off, cnt, sid = (t.cpu().numpy() for t in (lists.row_offset, lists.row_counts, lists.stage_ids))
    for i, (nv, i8, hi) in enumerate(want):                                       # every row
        assert tuple(cnt[0, i, :3]) == (len(nv), len(i8), len(hi)), i
        assert np.array_equal(sid[0, off[0, i] : off[0, i] + cnt[0, i, :3].sum()], np.concatenate((nv, i8, hi))), i
    packed = parts["packed"][0].cpu().numpy()
    worst = (0.0, 1.0)
    for i in np.linspace(0, rr - 1, 16).astype(int):                              # 16 spread blocks
        ref = A.attention_rows(ops, geo, slice(i * QB, (i + 1) * QB), want[i], head_dim=D,
                               q_scale_index=i, global_scales=full["scales"])
        rows = slice(i * QB, i * QB + int(geo.counts[i]))
        ma, cos, _ = compare_metrics(packed[rows], ref[: int(geo.counts[i])])
        worst = (max(worst[0], ma), min(worst[1], cos))
    assert worst[0] <= 2e-2 and worst[1] >= 0.999, worst
    # the prefix rows: INT8 cell over every stage of the head (the longest lists of the workload)
    every = np.arange(geo.stages, dtype=np.int32)
    got = full["out"][0, :PREFIX, 0].float().cpu().numpy()
    for t in range(PREFIX // QB):
        ref = A.attention_rows(ops, geo, slice(t * QB, (t + 1) * QB), ((), every, ()), head_dim=D,
                               q_scale_index=t, prefix_query=True)
        ma, cos, _ = compare_metrics(got[t * QB : (t + 1) * QB], ref.astype(np.float32))
        assert ma <= 2e-2 and cos >= 0.999, (t, ma, cos)


def test_heads_are_independent_and_runs_repeat(full):
    from anemoi_b200.executor import sm100_ragged_attention

    qd, kd, vd = full["dev"]
    alone = sm100_ragged_attention(qd[:, :, 1:2], kd[:, :, 1:2], vd[:, :, 1:2], **full["kw"])
    assert torch.equal(alone[:, :, 0], full["out"][:, :, 1])
    again = sm100_ragged_attention(qd, kd, vd, **full["kw"])
    assert torch.equal(again, full["out"])
