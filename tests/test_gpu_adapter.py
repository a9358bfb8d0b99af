"""GPU: the MiniMax-H3 adapter routes calls to dense attention or to the sparse path as its
schedule says, and its sparse calls equal ``anemoi_attention`` with the layer's settings."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_adapter_calls_equal_the_public_api(native_library):
    from anemoi_b200 import (NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout,
                             anemoi_attention)
    from anemoi_b200.adapter import H3MPAAttention, H3MPAConfig
    from tests.helpers import smooth_fields

    vs, prefix, heads, d = (2, 10, 14), 24, 2, 128
    q, k, v = (t[0].cuda() for t in smooth_fields(*vs, heads, d, prefix, seed=3, dtype=torch.bfloat16))
    scales = {"q_tensor_scale": [0.02] * 3, "k_tensor_scale": [0.02] * 3, "v_tensor_scale": [0.004] * 3}
    cfg = H3MPAConfig(video_shape=vs, prefix_tokens=prefix, sparsity_ratio=0.5, query_block_size=64,
                      nvfp4_ratio=0.3, int8_ratio=0.4, fp16_ratio=0.3, dense_first_steps=1,
                      dense_first_layers=1, layers_per_step=3,
                      layer_sparsity_bands=((2, 3, 0.25),), layer_precision_bands=((2, 3, 0.0, 0.5, 0.5),))
    att = H3MPAAttention(cfg, nvfp4_scales=scales)
    pos = torch.zeros(cfg.sequence_tokens)
    dense = torch.nn.functional.scaled_dot_product_attention(
        *(t.transpose(0, 1).unsqueeze(0) for t in (q, k, v))).squeeze(0).transpose(0, 1)

    att.observe(timestep=torch.tensor([1.0]), video_indices=None, position_ids=pos)
    for _ in range(3):                                   # step 0 is dense in every layer
        assert torch.equal(att(q, k, v), dense)
    att.observe(timestep=torch.tensor([0.9]), video_indices=None, position_ids=pos)
    assert torch.equal(att(q, k, v), dense)              # layer 0 stays dense
    layout = VisualLayout(vs, prefix)
    want1 = anemoi_attention(q[None], k[None], v[None], layout=layout, layer=1,
                             sparse_config=SparseConfig(64, 0.5), quant_config=QuantConfig(0.3, 0.4, 0.3),
                             calibration=NVFP4Calibration(0.02, 0.02, 0.004))[0]
    assert torch.equal(att(q, k, v), want1)
    want2 = anemoi_attention(q[None], k[None], v[None], layout=layout, layer=2,
                             sparse_config=SparseConfig(64, 0.25), quant_config=QuantConfig(0.0, 0.5, 0.5))[0]
    assert torch.equal(att(q, k, v), want2)
    assert att.stats()["dense_calls"] == 4 and att.stats()["mpa_calls"] == 2
    assert not torch.equal(want1, dense)

    fused = torch.cat((q, k, v), dim=-1)                 # strided [S, H, D] views, as after a fused projection
    views = [fused[..., i * d : (i + 1) * d] for i in range(3)]
    assert torch.equal(att.mpa(*views, layer=1), want1)
    with pytest.raises(ValueError):
        att.mpa(q[:-1], k[:-1], v[:-1], layer=1)
