"""Host logic of the Ulysses exchange on two CPU ranks (gloo): uneven shards, row-count cache,
and equality with the unsharded computation.  The CUDA relayout kernels are replaced by the
torch permutes they are defined to equal (relayout.py:110-119,143-149 of the reference)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from anemoi_b200 import ulysses


def torch_pack(q, k, v, world, begin=0, count=None):
    rows, heads, d = q.shape
    hl = heads // world
    count = hl - begin if count is None else count
    out = torch.empty((world, rows, count, 3 * d), dtype=q.dtype)
    for i, t in enumerate((q, k, v)):
        out[..., i * d : (i + 1) * d] = t.reshape(rows, world, hl, d)[:, :, begin : begin + count].permute(1, 0, 2, 3)
    return out


def torch_merge(x, out=None, begin=0):
    world, rows, hc, d = x.shape
    if out is None:
        out = torch.empty((rows, world * hc, d), dtype=x.dtype)
    per_rank = out.size(1) // world
    out.view(rows, world, per_rank, d)[:, :, begin : begin + hc] = x.permute(1, 0, 2, 3)
    return out


def toy_attention(q, k, v):
    # per-head dense attention: any head-independent function exercises the exchange
    qh, kh, vh = (t[0].permute(1, 0, 2).float() for t in (q, k, v))
    p = torch.softmax(qh @ kh.transpose(1, 2) / q.size(-1) ** 0.5, dim=-1)
    return (p @ vh).permute(1, 0, 2).unsqueeze(0).to(q.dtype)


def _worker(rank, world, port, total_rows, heads, d, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)
        full = [torch.randn(1, total_rows, heads, d, generator=gen).to(torch.bfloat16) for _ in range(3)]
        rows = ulysses.shard_rows(total_rows, world)
        lo = sum(rows[:rank])
        mine = [t[:, lo : lo + rows[rank]].contiguous() for t in full]
        want = toy_attention(*full)[:, lo : lo + rows[rank]]
        ok = True
        for groups in (1, 2, 3):  # one exchange, pipelined head groups, more groups than heads
            got = ulysses.ulysses_attention(*mine, toy_attention, pack=torch_pack, merge=torch_merge,
                                            pipeline_groups=groups)
            ok = ok and torch.equal(got, want)
        counts = ulysses.row_counts(rows[rank])
        # a changed local length without a reset must fail loudly, not desynchronise
        raised = False
        try:
            ulysses.row_counts(rows[rank] + 1)
        except RuntimeError:
            raised = True
        results[rank] = (ok, counts == rows, raised)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("total_rows", [37, 40])
def test_two_rank_exchange_matches_unsharded(total_rows):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), total_rows, 4, 16, results), nprocs=world, join=True)
    assert dict(results) == {0: (True, True, True), 1: (True, True, True)}


def test_shard_rows_matches_tensor_split():
    for total, world in ((38247, 4), (85184, 8), (7, 8), (33272, 8)):
        want = [t.numel() for t in torch.tensor_split(torch.arange(total), world)]
        assert ulysses.shard_rows(total, world) == want


def test_head_groups_cover_the_local_heads():
    assert ulysses.head_groups(7, 2) == [(0, 4), (4, 3)]
    assert ulysses.head_groups(28, 2) == [(0, 14), (14, 14)]
    assert ulysses.head_groups(1, 2) == [(0, 1)]
    assert ulysses.head_groups(5, 1) == [(0, 5)]
    for heads, groups in ((7, 3), (56, 4), (2, 8)):
        parts = ulysses.head_groups(heads, groups)
        assert parts[0][0] == 0 and sum(c for _, c in parts) == heads
        assert all(parts[i][0] + parts[i][1] == parts[i + 1][0] for i in range(len(parts) - 1))


def _stack_worker(rank, world, port, results):
    """The stand-in block stack on two CPU ranks: sequence-sharded with the exchange around the
    attention equals the unsharded stack (fp32, tiny widths, eager stand-ins for the CUDA kernels)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from anemoi_b200.h3_stack import H3BlockStack, H3StackConfig
        from oracle.producer import eager_reference

        cfg = H3StackConfig(width=48, heads=4, head_dim=16, ffn_width=64, rotary_dim=16, layers=3)
        stack = H3BlockStack(cfg, "cpu", dtype=torch.float32, seed=3)
        total = 37
        gen = torch.Generator().manual_seed(9)
        x = torch.randn(total, cfg.width, generator=gen)
        ang = torch.randn(total, cfg.rotary_dim, generator=gen)
        cos, sin = ang.cos(), ang.sin()

        def norm_rope(t, weight, c, s_, eps):
            t.copy_(eager_reference(t[0], weight, c, s_, eps).unsqueeze(0))
            return t

        def attention(q, k, v):      # [S, h, D] per-head dense attention
            p = torch.softmax(torch.einsum("shd,thd->hst", q, k) / q.size(-1) ** 0.5, dim=-1)
            return torch.einsum("hst,thd->shd", p, v)

        rows = ulysses.shard_rows(total, world)
        lo = sum(rows[:rank])
        sl = slice(lo, lo + rows[rank])
        ulysses.reset_row_counts()
        got = stack.step(x[sl], cos[sl], sin[sl], attention, norm_rope=norm_rope, pack=torch_pack, merge=torch_merge)
        # unsharded: same code with a one-rank "exchange"
        want = _single_rank_step(stack, x, cos, sin, attention, norm_rope)
        results[rank] = bool(torch.allclose(got, want[sl], atol=1e-5, rtol=1e-5))
    finally:
        dist.destroy_process_group()


def _single_rank_step(stack, x, cos, sin, attention, norm_rope):
    import unittest.mock as mock

    with mock.patch.object(dist, "is_initialized", lambda: False):
        return stack.step(x, cos, sin, attention, norm_rope=norm_rope)


def test_block_stack_sharded_equals_unsharded():
    world = 2
    port = _free_port()
    results = mp.Manager().dict()
    mp.spawn(_stack_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_exchange_region_layout_is_aligned_and_disjoint():
    from anemoi_b200.ulysses import exchange_region_layout

    lay = exchange_region_layout([301, 300, 300], 6, 128)
    assert lay["recv"] % 256 == 0 and lay["out0"] % 256 == 0 and lay["out1"] % 256 == 0
    assert lay["recv"] + lay["recv_bytes"] <= lay["out0"]
    assert lay["out0"] + lay["out_bytes"] <= lay["out1"] <= lay["bytes"] - lay["out_bytes"]
