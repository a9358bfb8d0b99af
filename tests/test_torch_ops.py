"""The ``torch.ops.anemoi_sm100`` registration over the C ABI: schemas on CPU, results on the GPU
equal to the ctypes layer's."""

import pytest
import torch


def test_operators_are_registered():
    from anemoi_b200 import torch_ops

    torch_ops.load()
    for name, pieces in (("draft_probability", ("Tensor q_pool", "float maxpool_weight", "-> Tensor")),
                         ("route", ("int n16", "int prefix_phase", "-> (Tensor, Tensor, Tensor)")),
                         ("qknorm_rope_", ("Tensor(a!) x", "-> Tensor(a!)"))):
        schema = str(getattr(torch.ops.anemoi_sm100, name).default._schema)
        assert all(p in schema for p in pieces), schema


@pytest.mark.gpu
def test_operators_equal_the_ctypes_layer(native_library):
    from anemoi_b200 import native, torch_ops
    from anemoi_b200.producer import fused_qknorm_rope
    from anemoi_b200.routing import route_counts

    torch_ops.load()
    heads, blocks, dim, qb, prefix = 3, 45, 128, 128, 100
    gen = torch.Generator().manual_seed(0)
    qp, kp = ((torch.randn(heads, blocks, dim, generator=gen) * 0.5).half().cuda() for _ in range(2))
    shape = native.Shape(heads=heads, head_dim=dim, query_block=qb, seq_tokens=prefix + blocks * qb,
                         prefix_tokens=prefix, video_blocks=blocks, has_nvfp4=0, has_int8=1, has_fp16=1,
                         has_prefix_query_int8=0, has_maxpool=0, input_is_bf16=1, q_global_scale=1.0,
                         k_global_scale=1.0, v_global_scale=1.0)
    prob = torch.ops.anemoi_sm100.draft_probability(qp, kp, None, None, 0.0, qb)
    store = native.OperandStore(shape=shape, struct=native.Operands(),
                                buffers={"q_pool": qp, "k_pool": kp, "q_max_pool": None, "k_max_pool": None})
    assert torch.equal(prob, native.draft_probability(shape, store, 0.0))
    n16, n8, n4 = route_counts(blocks * blocks, sparsity_ratio=0.7, nvfp4_ratio=0.0, int8_ratio=0.5, fp16_ratio=0.5)
    off, cnt, ids = torch.ops.anemoi_sm100.route(prob, n16, n8, n4, 1, qb, prefix, dim)
    want = native.route(shape, prob, n16, n8, n4, 1)
    assert torch.equal(off, want.row_offset) and torch.equal(cnt, want.row_counts)
    used = int((want.row_offset[0, -1] + want.row_counts[0, -1, :3].sum()).item())
    assert torch.equal(ids[:, :used], want.stage_ids[:, :used])
    x = torch.randn(1, 37, 4, dim, generator=gen).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(dim, generator=gen)).to(torch.bfloat16).cuda()
    angle = (torch.rand(37, 64, generator=gen) * 6.28).cuda()
    a = torch.ops.anemoi_sm100.qknorm_rope_(x.clone(), w, angle.cos(), angle.sin(), 1e-6)
    b = fused_qknorm_rope(x.clone(), w, angle.cos().contiguous(), angle.sin().contiguous(), 1e-6)
    assert torch.equal(a, b)
