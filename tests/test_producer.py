"""Producer fusion (per-head RMS norm + partial rotary): the CPU restatement against the plain
formula, and the CUDA kernel against the restatement bit for bit."""

from pathlib import Path

import pytest
import torch


def _case(tokens, heads, d, rotary, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn(tokens, heads, d, generator=gen) * (1 + torch.arange(d) % 5)).to(dtype)
    w = (1 + 0.1 * torch.randn(d, generator=gen)).to(dtype)
    angle = torch.rand(tokens, rotary, generator=gen) * 6.2832
    return x, w, torch.cos(angle), torch.sin(angle)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d, rotary", [(128, 64), (128, 128), (64, 32), (64, 0)])
def test_oracle_follows_the_formula(dtype, d, rotary):
    from oracle.producer import eager_reference, qknorm_rope

    x, w, cos, sin = _case(29, 3, d, rotary, dtype, seed=d + rotary)
    got = qknorm_rope(x, w, cos.numpy(), sin.numpy(), 1e-6).float()
    want = eager_reference(x, w, cos, sin, 1e-6)
    # one rounding to the 16-bit type separates them (bf16: 2^-8 relative, fp16: 2^-11)
    tol = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    assert ((got - want).abs() <= tol * want.abs() + 1e-6).all()
    # rows are independent and the transform keeps the head norm up to the weight
    assert got.shape == x.shape


def test_oracle_matches_the_reference_function():
    """Fixtures made by running the reference's own fused kernel under Triton's CPU interpreter
    (tests/golden/make_producer_golden.py; float32 results before the final rounding).  Rounded to
    the caller's type they equal the restatement bit for bit except where the float32 results
    differ in their last bits across a rounding boundary (different summation order of the
    squares): at most 1 value in 5,000, and then by one unit in the last place."""
    import numpy as np

    from oracle.producer import qknorm_rope
    from tests.golden.make_producer_golden import CASES, EPS

    golden = np.load(Path(__file__).parent / "golden" / "reference_producer.npz")
    for name, (tokens, heads, d, rotary, dtype) in CASES.items():
        x, w, cos, sin = _case(tokens, heads, d, rotary, dtype, seed=tokens + heads)
        mine = qknorm_rope(x, w, cos.numpy(), sin.numpy(), EPS)
        ref = torch.from_numpy(golden[name]).to(dtype)
        equal = mine.view(torch.int16) == ref.view(torch.int16)
        assert equal.float().mean().item() >= 1 - 2e-4, name
        step = (mine.view(torch.int16).int() - ref.view(torch.int16).int()).abs()
        assert int(step.max()) <= 1, name


def test_api_validation_needs_no_gpu():
    from anemoi_b200.producer import fused_qknorm_rope

    x = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16)
    w = torch.ones(128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="even rotary_dim"):
        fused_qknorm_rope(x, w, torch.zeros(4, 130), torch.zeros(4, 130), 1e-6)
    with pytest.raises(ValueError, match="multiple of 16"):
        fused_qknorm_rope(x, w, torch.zeros(4, 24), torch.zeros(4, 24), 1e-6)
    with pytest.raises(ValueError):
        fused_qknorm_rope(x[0], w, torch.zeros(4, 64), torch.zeros(4, 64), 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens, heads, d, rotary", [(37, 3, 128, 64), (5, 56, 128, 128), (64, 2, 64, 32),
                                                      (1, 1, 64, 0), (300, 7, 128, 16)])
def test_kernel_is_bit_exact_against_the_oracle(native_library, dtype, tokens, heads, d, rotary):
    from anemoi_b200.producer import fused_qknorm_rope
    from oracle.producer import qknorm_rope

    x, w, cos, sin = _case(tokens, heads, d, rotary, dtype, seed=tokens + heads)
    want = qknorm_rope(x, w, cos.numpy(), sin.numpy(), 1e-6)
    dev = x.cuda()[None].clone()
    out = fused_qknorm_rope(dev, w.cuda(), cos.cuda(), sin.cuda(), 1e-6)
    assert out.data_ptr() == dev.data_ptr()                       # in place
    assert torch.equal(out[0].cpu().view(torch.int16), want.view(torch.int16))
    # strided view: q inside a fused [tokens, heads, 3*D] projection output; k and v untouched
    fused = torch.randn(tokens, heads, 3 * d).to(dtype).cuda()
    fused[..., :d] = x.cuda()
    before = fused.clone()
    fused_qknorm_rope(fused[None, ..., :d], w.cuda(), cos.cuda(), sin.cuda(), 1e-6)
    assert torch.equal(fused[..., :d].cpu().view(torch.int16), want.view(torch.int16))
    assert torch.equal(fused[..., d:], before[..., d:])
