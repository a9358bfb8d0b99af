"""GPU lifecycle checks of the sm_100a path: results do not depend on what earlier tenants left
in recycled device memory, replays are bit-stable, and the give-up path of the kernels' bounded
waits reports and returns (reference models: tests/test_sm120_lifecycle_cuda.py and
tests/test_sm120_d64_cuda.py:236-258 of the reference)."""

import pytest
import torch

from tests.helpers import smooth_fields

pytestmark = pytest.mark.gpu


def _call(q, k, v, vs, prefix, ratios, drop, qb):
    from anemoi_b200.executor import sm100_ragged_attention

    return sm100_ragged_attention(
        q, k, v, prefix_tokens=prefix, sparsity_ratio=drop, retained_nvfp4_ratio=ratios[0],
        retained_int8_ratio=ratios[1], retained_fp16_ratio=ratios[2], video_shape=vs, layer=0,
        query_block_size=qb, nvfp4_scales=(0.01, 0.01, 0.002))


@pytest.mark.parametrize("cell", [(0.4, 0.4, 0.2), (0.0, 1.0, 0.0)], ids=["mixed", "int8"])
def test_nan_poisoned_allocator_churn_and_replays(native_library, cell):
    """Every scratch and output buffer of a call comes from the caching allocator.  Between calls
    the freed blocks are filled with NaN; a kernel that read a byte it had not written, or left
    an output row unwritten, would show it.  The case drops 97 % of the block pairs so that some
    query blocks have empty lists (their rows must be +0), and is replayed 128 times."""
    from anemoi_b200.executor import last_status

    vs, prefix, qb = (4, 16, 16), 0, 64
    q, k, v = (t.cuda() for t in smooth_fields(*vs, 2, 128, prefix, seed=5, outliers=(17, 93),
                                               dtype=torch.bfloat16))
    first = _call(q, k, v, vs, prefix, cell, 0.97, qb).clone()
    assert torch.isfinite(first).all()
    assert (first[0].view(torch.int16) == 0).all(dim=-1).any(), "expected some empty query blocks"
    for rep in range(128):
        if rep % 8 == 0:
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            poison = [torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
                      for n in (1 << 22, 1 << 20, 3 << 18, 1 << 16, 1 << 12)]
            del poison
        out = _call(q, k, v, vs, prefix, cell, 0.97, qb)
        assert torch.equal(out, first), rep
    assert last_status() == 0


def test_bounded_wait_gives_up_and_the_next_call_is_clean(native_library):
    """A wait that nothing can satisfy (a barrier nobody arrives on, no copy or MMA in flight)
    returns after its limit with the status word set; the context stays usable and the next
    attention call is clean."""
    from anemoi_b200 import native
    from anemoi_b200.executor import last_status

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    native.wait_selftest(200_000, status)          # 0.2 ms
    torch.cuda.synchronize()
    assert int(status.item()) == 99
    vs = (2, 10, 14)
    q, k, v = (t.cuda() for t in smooth_fields(*vs, 2, 128, 0, seed=2, dtype=torch.bfloat16))
    out = _call(q, k, v, vs, 0, (0.4, 0.4, 0.2), 0.5, 64)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert last_status() == 0


def test_route_runs_on_every_visible_device(native_library):
    """Function attributes are per device: routing on a second GPU of the same process must
    not fail its launch (one GPU: the loop runs once)."""
    from anemoi_b200.executor import last_status

    vs = (2, 10, 14)
    q, k, v = smooth_fields(*vs, 2, 128, 0, seed=2, dtype=torch.bfloat16)
    outs = []
    for dev in range(min(torch.cuda.device_count(), 2)):
        with torch.cuda.device(dev):
            out = _call(q.cuda(dev), k.cuda(dev), v.cuda(dev), vs, 0, (0.0, 1.0, 0.0), 0.5, 64)
            torch.cuda.synchronize(dev)
            assert last_status(torch.device("cuda", dev)) == 0
            outs.append(out.cpu())
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


def test_pipelined_host_input_equals_the_single_call(native_library):
    """Q/K/V in pinned host memory, walked in head groups on three streams (copy in, layer, copy
    out): heads are independent, so the result equals one call on all heads bit for bit."""
    from anemoi_b200 import HostAttention, NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention

    vs, prefix, heads = (2, 12, 20), 37, 5
    q, k, v = smooth_fields(*vs, heads, 128, prefix, seed=4, outliers=(17, 93), dtype=torch.bfloat16)
    kw = dict(layout=VisualLayout(vs, prefix), layer=0, sparse_config=SparseConfig(128, 0.6, (), 0.5),
              quant_config=QuantConfig(0.4, 0.4, 0.2), calibration=NVFP4Calibration(0.01, 0.01, 0.002))
    want = anemoi_attention(q.cuda(), k.cuda(), v.cuda(), **kw).cpu()
    hq, hk, hv = (t.contiguous().pin_memory() for t in (q, k, v))
    hout = torch.empty_like(hq).pin_memory()
    runner = HostAttention("cuda", group_heads=2)       # groups of 2, 2 and 1 heads
    for _ in range(2):                                   # second pass reuses the device buffers
        hout.fill_(float("nan"))
        runner(hq, hk, hv, hout, **kw)
        torch.cuda.synchronize()
        assert torch.equal(hout, want)


def test_nvtx_ranges_do_not_change_the_result(native_library):
    """The opt-in NVTX ranges (the reference's names) only mark the host timeline."""
    from anemoi_b200 import executor

    vs = (2, 10, 14)
    q, k, v = (t.cuda() for t in smooth_fields(*vs, 2, 128, 37, seed=2, dtype=torch.bfloat16))
    kw = dict(prefix_tokens=37, sparsity_ratio=0.5, retained_nvfp4_ratio=0.4, retained_int8_ratio=0.4,
              retained_fp16_ratio=0.2, video_shape=vs, layer=0, query_block_size=64,
              nvfp4_scales=(0.01, 0.01, 0.002))
    plain = executor.sm100_ragged_attention(q, k, v, **kw)
    marked = executor.sm100_ragged_attention(q, k, v, profile_nvtx=True, **kw)
    executor.set_profile_nvtx(True)
    try:
        switched = executor.sm100_ragged_attention(q, k, v, **kw)
    finally:
        executor.set_profile_nvtx(False)
    assert torch.equal(plain, marked) and torch.equal(plain, switched)
    with pytest.raises(TypeError):
        executor.sm100_ragged_attention(q, k, v, profile_nvtx=1, **kw)


@pytest.mark.parametrize("vs,dim,prefix,cell,drop", [
    ((2, 10, 14), 64, 0, (0.4, 0.4, 0.2), 0.5),        # 6 blocks
    ((3, 9, 21), 128, 37, (0.4, 0.4, 0.2), 0.6),       # 9 blocks: the last pair has one block
    ((4, 16, 16), 64, 0, (0.0, 1.0, 0.0), 0.8),
    ((3, 9, 21), 128, 70, (1.0, 0.0, 0.0), 0.5),
    ((4, 16, 16), 128, 0, (0.5, 0.0, 0.5), 0.97),      # blocks with empty lists inside pairs
])
def test_q64_pairs_equal_one_block_per_cta(native_library, vs, dim, prefix, cell, drop):
    """Two Q64 query blocks per CTA walking the union of their lists give, bit for bit, what one
    (padded) block per CTA gives: every row meets exactly its own stages in its own order."""
    from anemoi_b200 import executor

    q, k, v = (t.cuda() for t in smooth_fields(*vs, 3, dim, prefix, seed=7, outliers=(5, 41),
                                               dtype=torch.bfloat16))
    paired = _call(q, k, v, vs, prefix, cell, drop, 64)
    executor._PAIR_Q64 = False
    try:
        single = _call(q, k, v, vs, prefix, cell, drop, 64)
    finally:
        executor._PAIR_Q64 = True
    torch.cuda.synchronize()
    assert torch.isfinite(paired).all()
    assert torch.equal(paired, single)
    assert executor.last_status() == 0
