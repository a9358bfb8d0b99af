"""The tensor-pipe probe behind the roofline denominators runs clean and orders the kinds."""

import pytest

pytestmark = pytest.mark.gpu


def test_tensor_peak_per_kind(native_library):
    from anemoi_b200 import native

    rate = {kind: native.tensor_peak(kind, iterations=1024, repeats=2) for kind in native.TENSOR_KINDS}
    print("tcgen05 measured, TFLOP/s:", {k: round(v, 1) for k, v in rate.items()})
    # a B200 delivers hundreds of TFLOP/s in every kind; narrower operands are not slower
    assert all(v > 100.0 for v in rate.values()), rate
    assert rate["f8"] >= 0.9 * rate["f16"] and rate["i8"] >= 0.9 * rate["f16"], rate
    assert rate["nvfp4"] >= 0.9 * rate["f8"], rate


def test_tensor_peak_rejects_bad_arguments(native_library):
    import ctypes as C

    import torch

    from anemoi_b200 import native

    lib = native.library()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flops = C.c_double(0.0)
    assert lib.anemoi_sm100_tensor_peak(7, 16, C.c_void_p(status.data_ptr()), C.byref(flops), None) == -1
    assert lib.anemoi_sm100_tensor_peak(0, 0, C.c_void_p(status.data_ptr()), C.byref(flops), None) == -1
