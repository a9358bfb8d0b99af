"""GPU: Ulysses relayout kernels are bit-equal to the torch permutes they replace
(the reference checks its Triton kernels the same way, relayout.py:165-198), and the
preparation kernel consumes the strided head-sharded receive buffer in place."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pack_and_merge_equal_torch_permutes(native_library):
    from anemoi_b200 import native
    from tests.test_ulysses_cpu import torch_merge, torch_pack

    gen = torch.Generator().manual_seed(2)
    for rows, heads, d, world in ((37, 8, 128, 4), (5, 56, 128, 8), (64, 4, 64, 2), (0, 8, 64, 2)):
        fused = torch.randn(rows, heads, 3 * d, generator=gen).to(torch.bfloat16).cuda()
        q, k, v = (fused[..., i * d : (i + 1) * d] for i in range(3))     # strided views
        got = native.pack_qkv_destination_major(q, k, v, world)
        want = torch_pack(q.cpu(), k.cpu(), v.cpu(), world)
        assert torch.equal(got.cpu(), want)
        x = torch.randn(world, rows, heads // world, d, generator=gen).to(torch.float16).cuda()
        assert torch.equal(native.merge_heads(x).cpu(), torch_merge(x.cpu()))
        # a sub-range of every rank's heads (head-group pipelining of the exchange)
        hl = heads // world
        if hl >= 2 and rows:
            begin, count = 1, hl - 1
            got = native.pack_qkv_destination_major(q, k, v, world, begin, count)
            assert torch.equal(got.cpu(), torch_pack(q.cpu(), k.cpu(), v.cpu(), world, begin, count))
            part = torch.randn(world, rows, count, d, generator=gen).to(torch.float16).cuda()
            out = torch.zeros(rows, heads, d, dtype=torch.float16, device="cuda")
            native.merge_heads(part, out, begin)
            assert torch.equal(out.cpu(), torch_merge(part.cpu(), torch.zeros(rows, heads, d, dtype=torch.float16), begin))
    with pytest.raises(ValueError):
        native.pack_qkv_destination_major(q, k, v, 3)


def test_strided_qkv_views_give_the_same_output(native_library):
    from anemoi_b200 import QuantConfig, SparseConfig, VisualLayout, anemoi_attention
    from tests.helpers import smooth_fields

    q, k, v = smooth_fields(2, 10, 14, 2, 128, 24, seed=4, dtype=torch.bfloat16)
    lay = VisualLayout((2, 10, 14), 24)
    kw = dict(layout=lay, layer=0, sparse_config=SparseConfig(64, 0.5),
              quant_config=QuantConfig(0.3, 0.4, 0.3))
    want = anemoi_attention(q.cuda(), k.cuda(), v.cuda(), **kw)
    fused = torch.cat((q, k, v), dim=-1).cuda()                      # [1, S, H, 3D]
    views = [fused[..., i * 128 : (i + 1) * 128] for i in range(3)]
    assert not views[0].is_contiguous()
    assert torch.equal(anemoi_attention(*views, **kw), want)
