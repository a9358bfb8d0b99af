"""The diag-Jensen draft map (an experimental routing variant of the reference): the CPU
restatement against the reference's own function, and the CUDA kernels against the restatement."""

from pathlib import Path

import numpy as np
import pytest
import torch

from tests.golden.make_jensen_golden import CASES, case_inputs


def _oracle_pools(x: torch.Tensor, counts: torch.Tensor):
    from oracle import prep as P

    blocks, slots, dim = x.shape
    geo = type("G", (), {"query_block": slots, "counts": counts.numpy()})()
    rows = x.reshape(blocks * slots, dim).numpy()
    return P.mean_pool(rows, geo), P.second_moment_pool(rows, geo)


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_the_reference_function(name):
    """Fixtures: the reference's `draft_probability(..., q_second=, k_second=)` on pools formed the
    way its executor forms them (tests/golden/make_jensen_golden.py).  The restatement fixes the
    summation order, so single values may differ in the last bit of the fp16 result."""
    from oracle import route as R

    golden = np.load(Path(__file__).parent / "golden" / "reference_jensen.npz")
    q, k, counts = case_inputs(name)
    (qm, q2), (km, k2) = _oracle_pools(q, counts), _oracle_pools(k, counts)
    mine = R.draft_probability_jensen(qm, km, q2, k2)
    ref = golden[name].view(np.float16)
    assert np.abs(mine.astype(np.float32) - ref.astype(np.float32)).max() <= 5e-4
    assert (mine.view(np.uint16) == ref.view(np.uint16)).mean() >= 0.98


def test_jensen_excludes_the_max_pool_blend():
    from anemoi_b200.executor import sm100_ragged_attention

    x = torch.zeros(1, 64, 1, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="diag_jensen"):
        sm100_ragged_attention(x, x, x, prefix_tokens=0, sparsity_ratio=0.5, retained_nvfp4_ratio=0.0,
                               retained_int8_ratio=1.0, retained_fp16_ratio=0.0, video_shape=(1, 8, 8), layer=0,
                               query_block_size=64, maxpool_weight=0.5, diag_jensen=True)


@pytest.mark.gpu
@pytest.mark.parametrize("vs,dim,qb,prefix", [((2, 10, 14), 64, 64, 0), ((2, 12, 20), 128, 128, 37)])
def test_kernels_match_the_oracle(native_library, vs, dim, qb, prefix):
    """Second-moment pools and the Jensen map bit for bit against the restatement; the lists that
    follow differ from the plain map's, and the layer runs clean."""
    from anemoi_b200 import executor
    from anemoi_b200.partition import make_ragged_2d_partition
    from oracle import prep as P, route as R
    from tests.helpers import smooth_fields

    q, k, v = smooth_fields(*vs, 2, dim, prefix, seed=4, outliers=(5, 41), dtype=torch.bfloat16)
    kw = dict(prefix_tokens=prefix, sparsity_ratio=0.6, retained_nvfp4_ratio=0.0, retained_int8_ratio=0.5,
              retained_fp16_ratio=0.5, video_shape=vs, layer=0, query_block_size=qb, return_parts=True)
    out, parts = executor.sm100_ragged_attention(q.cuda(), k.cuda(), v.cuda(), diag_jensen=True, **kw)
    _, plain = executor.sm100_ragged_attention(q.cuda(), k.cuda(), v.cuda(), **kw)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and executor.last_status() == 0
    part = make_ragged_2d_partition(vs[1], vs[2], qb, include_adjacency=False)
    geo = P.make_geometry(part.blocks, *vs, qb, prefix)
    store = parts["store"].buffers
    for head in range(2):
        ops = P.prepare_head(q[0, :, head].float().numpy(), k[0, :, head].float().numpy(),
                             v[0, :, head].float().numpy(), geo, has_nvfp4=False, has_int8=True,
                             has_prefix_query_int8=prefix > 0, has_maxpool=False, second_moments=True)
        assert np.array_equal(store["q_max_pool"][head].cpu().numpy().view(np.uint16), ops.q_max.view(np.uint16))
        assert np.array_equal(store["k_max_pool"][head].cpu().numpy().view(np.uint16), ops.k_max.view(np.uint16))
        want = R.draft_probability_jensen(ops.q_pool, ops.k_pool, ops.q_max, ops.k_max)
        got = parts["prob"][head].cpu().numpy()
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), head
    assert not torch.equal(parts["prob"], plain["prob"])
