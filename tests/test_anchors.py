"""Routing with anchors (an experimental variant of the reference): the CPU restatement against
the reference's own ``route_probability``, the layout's anchor mask against the same fixtures'
geometry, and the CUDA kernels (selection with a fourth boundary over the non-anchor pairs)
against the restatement (which follows the reference's sort-and-evict formulation)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from tests.golden.make_anchor_golden import CASES, anchor_matrix, case_inputs


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_the_reference_function(name):
    from oracle import route as R

    golden = np.load(Path(__file__).parent / "golden" / "reference_anchors.npz")
    frames, height, width, block, drop, ratios, seed = CASES[name]
    prob, part, frames, blocks = case_inputs(name)
    n16, n8, n4 = R.budgets(blocks * blocks, drop, *ratios)
    ids, low, mid, high = R.route(prob.numpy(), n16, n8, n4, anchor_matrix(part, frames))
    assert np.array_equal(np.stack([low, mid, high]), golden[name + "_counts"])
    for i in range(blocks):
        n = int(low[i] + mid[i] + high[i])
        assert np.array_equal(ids[i, :n], golden[name + "_ids"][i, :n]), i
    # every anchor pair is kept, and the budget is unchanged
    kept = np.zeros((blocks, blocks), dtype=bool)
    for i in range(blocks):
        kept[i, ids[i, : int(low[i] + mid[i] + high[i])]] = True
    assert kept[anchor_matrix(part, frames)].all()
    assert int(kept.sum()) == n16 + n8 + n4


@pytest.mark.parametrize("name", list(CASES))
def test_layout_builds_the_reference_anchor_mask(name):
    from anemoi_b200.layout import materialize_ragged_2d_layout

    frames, height, width, block, *_ = CASES[name]
    _, part, _, blocks = case_inputs(name)
    layout = materialize_ragged_2d_layout("cpu", frames=frames, height=height, width=width, logical_block=block,
                                          enable_anchors=True)
    want = anchor_matrix(part, frames)
    assert np.array_equal(layout.anchors.numpy(), want)
    assert layout.anchor_count == int(want.sum())
    ids = layout.anchor_ids.numpy().astype(np.int64)
    assert want.reshape(-1)[ids].all() and len(set(ids.tolist())) == ids.size
    plain = materialize_ragged_2d_layout("cpu", frames=frames, height=height, width=width, logical_block=block)
    assert plain.anchors is None and plain.anchor_count == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("prefix", [0, 100])
def test_kernels_match_the_oracle(native_library, name, prefix):
    from anemoi_b200 import native
    from anemoi_b200.layout import materialize_ragged_2d_layout
    from oracle import route as R

    frames, height, width, block, drop, ratios, seed = CASES[name]
    prob, part, frames, blocks = case_inputs(name)
    heads = 3
    gen = torch.Generator().manual_seed(seed + 10)
    probs = torch.stack([prob] + [torch.softmax(torch.randn(blocks, blocks, generator=gen) * 2.5, -1).half()
                                  for _ in range(heads - 1)])
    probs[2, 5, :] = probs[2, 4, 0]                       # a long run of ties in another head
    layout = materialize_ragged_2d_layout("cuda", frames=frames, height=height, width=width, logical_block=block,
                                          enable_anchors=True)
    n16, n8, n4 = R.budgets(blocks * blocks, drop, *ratios)
    phase = -1 if not prefix else (1 if n8 else 2)
    shape = native.Shape(heads=heads, head_dim=128, query_block=block, seq_tokens=prefix + blocks * block,
                         prefix_tokens=prefix, video_blocks=blocks, has_nvfp4=int(n4 > 0), has_int8=int(n8 > 0),
                         has_fp16=1, has_prefix_query_int8=0, has_maxpool=0, input_is_bf16=1, q_global_scale=1.0,
                         k_global_scale=1.0, v_global_scale=1.0)
    lists = native.route_anchored(shape, probs.cuda(), n16, n8, n4, phase, layout.anchors, layout.anchor_ids)
    torch.cuda.synchronize()
    off = lists.row_offset.cpu().numpy()
    cnt = lists.row_counts.cpu().numpy()
    ids = lists.stage_ids.cpu().numpy()
    pstages = (prefix + 63) // 64
    anchors = anchor_matrix(part, frames)
    for h in range(heads):
        o_ids, low, mid, high = R.route(probs[h].numpy(), n16, n8, n4, anchors)
        want = R.stage_lists(o_ids, low, mid, high, query_block=block, prefix_stages=pstages,
                             prefix_phase=None if phase < 0 else ("nvfp4", "int8", "fp16")[phase])
        expect = 0
        for i in range(blocks):
            assert off[h, i] == expect, (h, i)
            flat = np.concatenate(want[i])
            assert [len(w) for w in want[i]] == cnt[h, i, :3].tolist(), (h, i)
            assert np.array_equal(ids[h, off[h, i] : off[h, i] + flat.size], flat), (h, i)
            expect += flat.size


@pytest.mark.gpu
def test_layer_with_anchors_runs_and_keeps_every_neighbour(native_library):
    from anemoi_b200 import executor
    from tests.helpers import smooth_fields

    vs, prefix = (2, 32, 48), 0
    q, k, v = (t.cuda() for t in smooth_fields(*vs, 2, 128, prefix, seed=3, dtype=torch.bfloat16))
    kw = dict(prefix_tokens=prefix, sparsity_ratio=0.5, retained_nvfp4_ratio=0.4, retained_int8_ratio=0.4,
              retained_fp16_ratio=0.2, video_shape=vs, layer=0, query_block_size=64,
              nvfp4_scales=(0.01, 0.01, 0.002), return_parts=True)
    out, parts = executor.sm100_ragged_attention(q, k, v, enable_anchors=True, **kw)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and executor.last_status() == 0
    lists, layout = parts["lists"], parts["layout"]
    blocks = parts["shape"].video_blocks
    off, cnt, ids = (t.cpu().numpy() for t in (lists.row_offset, lists.row_counts, lists.stage_ids))
    anchors = layout.anchors.cpu().numpy()
    for h in range(2):
        for i in range(blocks):
            n = int(cnt[h, i, :3].sum())
            assert set(np.nonzero(anchors[i])[0].tolist()) <= set(ids[h, off[h, i] : off[h, i] + n].tolist())
    with pytest.raises(ValueError, match="lowest-precision budget"):
        executor.sm100_ragged_attention(q, k, v, enable_anchors=True, **{**kw, "sparsity_ratio": 0.99})
