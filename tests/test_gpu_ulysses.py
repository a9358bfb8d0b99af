"""GPU (2 or more devices): the head-sharded Ulysses run equals the single-GPU run bit for bit,
through the all-to-all exchange and through the stores into the peers' memory."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from anemoi_b200 import (NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout,
                                 anemoi_attention, ulysses)
        from tests.helpers import smooth_fields

        heads, prefix, vs = 4 * world, 37, (2, 12, 20)
        q, k, v = smooth_fields(*vs, heads, 128, prefix, seed=3, outliers=(17, 93), dtype=torch.bfloat16)
        kw = dict(layout=VisualLayout(vs, prefix), layer=0, sparse_config=SparseConfig(128, 0.6, (), 0.5),
                  quant_config=QuantConfig(0.4, 0.4, 0.2), calibration=NVFP4Calibration(0.01, 0.01, 0.002))
        full = anemoi_attention(q.cuda(), k.cuda(), v.cuda(), **kw)
        rows = ulysses.shard_rows(q.size(1), world)      # uneven: 517 tokens
        lo = sum(rows[:rank])
        mine = [t[:, lo : lo + rows[rank]].contiguous().cuda() for t in (q, k, v)]
        got = ulysses.ulysses_anemoi_attention(*mine, **kw)
        torch.cuda.synchronize()
        ok = bool(torch.equal(got, full[:, lo : lo + rows[rank]]))
        # the same through stores into the peers' memory, three layers in a row (buffer reuse)
        from anemoi_b200.executor import last_status

        peer = ulysses.PeerExchange(rows[rank], heads, 128, torch.bfloat16, torch.device("cuda", rank))
        try:
            for _ in range(3):
                got = ulysses.ulysses_anemoi_attention(*mine, exchange=peer, **kw)
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(got, full[:, lo : lo + rows[rank]]))
            ok = ok and last_status(torch.device("cuda", rank)) == 0
            # the producer step folded into the exchange equals the in-place kernel before it
            from anemoi_b200.producer import fused_qknorm_rope

            gen = torch.Generator().manual_seed(9)
            wq, wk = ((1 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16).cuda() for _ in range(2))
            angle = torch.rand(q.size(1), 64, generator=gen) * 6.2832
            cos, sin = (f(angle)[lo : lo + rows[rank]].contiguous().cuda() for f in (torch.cos, torch.sin))
            qn, kn = mine[0].clone(), mine[1].clone()
            fused_qknorm_rope(qn, wq, cos, sin, 1e-6)
            fused_qknorm_rope(kn, wk, cos, sin, 1e-6)
            want = ulysses.ulysses_anemoi_attention(qn, kn, mine[2], exchange=peer, **kw)
            want = want.clone()
            local = lambda a, b, c: anemoi_attention(a, b, c, **kw)          # noqa: E731
            got = ulysses.ulysses_attention(*mine, local, exchange=peer, producer=(wq, wk, cos, sin, 1e-6))
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(got, want))
            # the host-input entry in its sharded mode: this rank's rows from pinned host memory,
            # head groups of two (one head per rank and group), two passes (buffer reuse)
            from anemoi_b200 import HostAttention

            hq, hk, hv = (t.cpu().contiguous().pin_memory() for t in mine)
            hout = torch.empty_like(hq).pin_memory()
            # groups of `world` heads, and groups of 3 * world with a shorter last group (two
            # exchanges of different sizes alive at once)
            for group_heads in (world, 3 * world):
                runner = HostAttention(torch.device("cuda", rank), group_heads=group_heads, sharded=True)
                try:
                    for _ in range(2):
                        hout.fill_(float("nan"))
                        runner(hq, hk, hv, hout, **kw)
                        torch.cuda.synchronize()
                        ok = ok and bool(torch.equal(hout, full[:, lo : lo + rows[rank]].cpu()))
                finally:
                    runner.close()
        finally:
            peer.close()
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_sharded_run_equals_single_gpu(native_library):
    world = min(torch.cuda.device_count(), 2)
    if world < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {r: True for r in range(world)}
