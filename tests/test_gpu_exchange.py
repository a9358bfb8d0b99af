"""GPU (one device): the store kernels of the peer exchange against index arithmetic in torch.

The ranks of a node are emulated on one device: every "rank" has its own receive, output and flag
buffers there and the pushes run one after the other, so no launch ever waits for a later one
(the waits are issued only after every push they depend on).  Row counts are uneven and one
rank may hold no rows, as ``tensor_split`` produces for short sequences.  The same exchange
across two real devices is covered by tests/test_gpu_ulysses.py."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("counts,heads,dim", [((5, 4), 4, 128), ((3, 3, 2, 2), 8, 64), ((7, 0, 1), 6, 128),
                                              ((300, 299, 299, 299, 299, 299, 299, 299), 8, 128)])
def test_push_kernels_match_the_all_to_all_layout(native_library, counts, heads, dim):
    from anemoi_b200 import native
    from anemoi_b200.ulysses import first_rows

    world, first = len(counts), first_rows(list(counts))
    total, h_local = first[-1], heads // len(counts)
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(1)
    # strided inputs: q, k, v are column slices of one wider projection output
    wide = [torch.randn(c, heads, 3 * dim, generator=gen, device=dev).to(torch.bfloat16) for c in counts]
    qkv = [[w[..., i * dim:(i + 1) * dim] for i in range(3)] for w in wide]
    recv = [torch.full((total, h_local, 3 * dim), float("nan"), dtype=torch.bfloat16, device=dev)
            for _ in range(world)]
    out = [torch.full((c, heads, dim), float("nan"), dtype=torch.bfloat16, device=dev) for c in counts]
    flags_in = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
    flags_out = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ptrs = lambda ts: [t.data_ptr() for t in ts]          # noqa: E731

    for epoch in (1, 2):
        for r in range(world):
            native.push_qkv(*qkv[r], ptrs(recv), ptrs(flags_in), first, r, epoch, done)
        for r in range(world):
            native.wait_flags(flags_in[r].data_ptr(), world, epoch, 1_000_000_000, status, dev)
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and int(done.item()) == 0
        for d in range(world):
            for r in range(world):
                for i in range(3):
                    want = qkv[r][i][:, d * h_local:(d + 1) * h_local]
                    got = recv[d][first[r]:first[r + 1], :, i * dim:(i + 1) * dim]
                    assert torch.equal(got, want), (epoch, d, r, i)

    heads_out = [torch.randn(total, h_local, dim, generator=gen, device=dev).to(torch.bfloat16)
                 for _ in range(world)]
    for r in range(world):
        native.push_out(heads_out[r], ptrs(out), ptrs(flags_out), first, r, 1, done)
    for r in range(world):
        native.wait_flags(flags_out[r].data_ptr(), world, 1, 1_000_000_000, status, dev)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for o in range(world):
        want = torch.cat([h[first[o]:first[o + 1]] for h in heads_out], dim=1)
        assert torch.equal(out[o], want), o


def test_flag_wait_gives_up_with_the_late_rank_in_the_status_word(native_library):
    """Nothing publishes epoch 5 for rank 1: the wait returns after its limit, records 71, and a
    later wait on the same stream returns at once because the status word is already set."""
    from anemoi_b200 import native

    dev = torch.device("cuda")
    flags = torch.tensor([5, 4, 5, 0, 0, 0, 0, 0], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    native.wait_flags(flags.data_ptr(), 3, 5, 300_000, status, dev)       # 0.3 ms
    native.wait_flags(flags.data_ptr(), 3, 5, 300_000, status, dev)
    torch.cuda.synchronize()
    assert int(status.item()) == 71
    # epochs compare modulo 2^32: a flag that wrapped past the epoch counts as reached
    flags = torch.tensor([2, 1, 0, 0, 0, 0, 0, 0], dtype=torch.int32, device=dev)
    status.zero_()
    native.wait_flags(flags.data_ptr(), 2, 0xFFFFFFFF, 300_000, status, dev)
    torch.cuda.synchronize()
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,heads,dim,rotary", [((37, 36), 4, 128, 64), ((9, 8, 8, 8), 8, 64, 32),
                                                     ((5, 0, 4), 3, 128, 128)])
def test_push_with_the_producer_step_equals_producer_then_push(native_library, counts, heads, dim, rotary, dtype):
    """qk-norm + partial rotary folded into the exchange's stores give, bit for bit, what the
    in-place producer kernel followed by the plain push gives; v passes through, and the caller's
    q and k are left as the projections wrote them."""
    from anemoi_b200 import native
    from anemoi_b200.producer import fused_qknorm_rope
    from anemoi_b200.ulysses import first_rows

    world, first = len(counts), first_rows(list(counts))
    total, h_local = first[-1], heads // len(counts)
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(3)
    wide = [torch.randn(c, heads, 3 * dim, generator=gen, device=dev).to(dtype) for c in counts]
    qkv = [[w[..., i * dim:(i + 1) * dim] for i in range(3)] for w in wide]
    wq = (1 + 0.1 * torch.randn(dim, generator=gen, device=dev)).to(dtype)
    wk = (1 + 0.1 * torch.randn(dim, generator=gen, device=dev)).to(dtype)
    angle = [torch.rand(c, rotary, generator=gen, device=dev) * 6.2832 for c in counts]
    cos, sin = [a.cos().contiguous() for a in angle], [a.sin().contiguous() for a in angle]
    ptrs = lambda ts: [t.data_ptr() for t in ts]          # noqa: E731

    def run(fused: bool):
        recv = [torch.full((total, h_local, 3 * dim), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
        flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
        done = torch.zeros(1, dtype=torch.int32, device=dev)
        for r in range(world):
            q, k, v = qkv[r]
            if fused:
                before = wide[r].clone()
                native.push_qkv(q, k, v, ptrs(recv), ptrs(flags), first, r, 1, done,
                                (wq, wk, cos[r], sin[r], 1e-6))
                assert torch.equal(wide[r], before)
            else:
                q, k = q.contiguous(), k.contiguous()
                if counts[r]:
                    fused_qknorm_rope(q[None], wq, cos[r], sin[r], 1e-6)
                    fused_qknorm_rope(k[None], wk, cos[r], sin[r], 1e-6)
                native.push_qkv(q, k, v, ptrs(recv), ptrs(flags), first, r, 1, done)
        torch.cuda.synchronize()
        assert all(int(f[:world].min()) == 1 for f in flags)
        return recv

    for a, b in zip(run(True), run(False)):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
