"""GPU: the routing entry point that uses the library's own scratch array.

Hosts that cannot allocate on their request path call ``anemoi_sm100_route_static``; it must
give exactly the lists of ``anemoi_sm100_route`` (row counts and every row's stage list,
bit for bit) - here on two calls in a row, because the shared array keeps the previous
call's contents.  Collected last so that a failure here cannot hide any other test.
"""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rows(lists):
    off = lists.row_offset.cpu().numpy()
    cnt = lists.row_counts.cpu().numpy()
    ids = lists.stage_ids.cpu().numpy()
    out = []
    for h in range(off.shape[0]):
        for i in range(off.shape[1]):
            n = int(cnt[h, i, :3].sum())
            out.append(ids[h, off[h, i] : off[h, i] + n].copy())
    return cnt, out


def test_static_scratch_route_matches_route(native_library):
    from anemoi_b200 import native
    from anemoi_b200.routing import route_counts

    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(11)
    for call, (heads, blocks, qb, prefix, phase) in enumerate(((5, 96, 128, 100, 1), (3, 70, 64, 0, -1))):
        shape = native.Shape(heads=heads, head_dim=128, query_block=qb, seq_tokens=prefix + blocks * qb,
                             prefix_tokens=prefix, video_blocks=blocks, has_nvfp4=1, has_int8=1, has_fp16=1,
                             has_prefix_query_int8=0, has_maxpool=0, input_is_bf16=1, q_global_scale=1.0,
                             k_global_scale=1.0, v_global_scale=1.0)
        prob = torch.softmax(torch.randn(heads, blocks, blocks, generator=gen) * 3, -1).to(torch.float16)
        prob[0, 1, :9] = prob[0, 0, 0]            # ties across rows and columns
        prob = prob.to(dev)
        n16, n8, n4 = route_counts(blocks * blocks, sparsity_ratio=0.7, nvfp4_ratio=0.4, int8_ratio=0.4,
                                   fp16_ratio=0.2)
        want = native.route(shape, prob, n16, n8, n4, phase)
        got = native.RouteLists(row_offset=torch.full_like(want.row_offset, -1),
                                row_counts=torch.full_like(want.row_counts, -1),
                                stage_ids=torch.full_like(want.stage_ids, -1), capacity=want.capacity)
        native.route_static(shape, prob, n16, n8, n4, phase, got)
        torch.cuda.synchronize()
        wc, wr = _rows(want)
        gc, gr = _rows(got)
        assert np.array_equal(gc, wc), f"call {call}: row counts differ"
        assert all(np.array_equal(a, b) for a, b in zip(gr, wr)), f"call {call}: stage lists differ"


def test_static_scratch_route_refuses_oversized_shapes(native_library):
    from anemoi_b200 import native

    limit = native_library.anemoi_sm100_route_static_max_bytes()
    assert limit == 8 * 1024 * 1024
    heads, blocks = 64, 2048          # 64 * (32777 + 8192) * 4 bytes > 8 MiB
    shape = native.Shape(heads=heads, head_dim=128, query_block=64, seq_tokens=blocks * 64, prefix_tokens=0,
                         video_blocks=blocks, has_nvfp4=0, has_int8=1, has_fp16=0, has_prefix_query_int8=0,
                         has_maxpool=0, input_is_bf16=1, q_global_scale=1.0, k_global_scale=1.0,
                         v_global_scale=1.0)
    one = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = native_library.anemoi_sm100_route_static(C.byref(shape), C.c_void_p(one.data_ptr()), 1, 1, 1, -1,
                                                  C.c_void_p(one.data_ptr()), C.c_void_p(one.data_ptr()),
                                                  C.c_void_p(one.data_ptr()), 1, None)
    assert rc == -3
