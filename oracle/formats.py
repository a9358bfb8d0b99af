"""TEST INFRASTRUCTURE - CPU restatement of the number formats on the path.

Encoders/decoders for FP8 E4M3 (round to nearest even, saturate to +-448) and
FP4 E2M1 (round to nearest even, saturate to +-6), and the bf16 -> fp16
narrowing step.  These restate the conversions the reference performs with
``__nv_cvt_float_to_fp8(.., __NV_SATFINITE, __NV_E4M3)`` and
``__nv_cvt_float2_to_fp4x2(.., __NV_E2M1, cudaRoundNearest)``
(csrc/attention/cuda/sm120/q128_microscaling_preparation.cu:43-62) and the
torch restatement in the reference's own tests (tests/test_sm120_d64_cuda.py:165-186:
E2M1 midpoints .25 .75 1.25 1.75 2.5 3.5 5 with ties to the even code).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package; the product never does.
"""

from __future__ import annotations

import numpy as np

E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def narrow_to_fp16(x) -> np.ndarray:
    """bf16/fp16/fp32 torch tensor or array -> fp16 array via fp32, round to nearest even."""
    if hasattr(x, "detach"):
        x = x.detach().float().cpu().numpy()
    return np.asarray(x, dtype=np.float32).astype(np.float16)


def _round_to_grid(mag: np.ndarray, min_exp: int, mant_bits: int, max_value: float) -> np.ndarray:
    """Round non-negative float64 ``mag`` to the nearest-even representable value."""
    mag = np.minimum(mag, max_value)
    _, ex = np.frexp(mag)                      # mag = m * 2**ex, m in [0.5, 1)
    e = np.maximum(ex - 1, min_exp)            # unbiased exponent, clamped to subnormal range
    quantum = np.ldexp(1.0, e - mant_bits)
    return np.rint(mag / quantum) * quantum


def e4m3_encode(x) -> np.ndarray:
    """float array -> E4M3 bit patterns (uint8); RN-even, finite saturation, NaN -> 0x7f."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    nan = np.isnan(mag)
    mag = np.where(nan, 0.0, mag)
    val = _round_to_grid(mag, -6, 3, 448.0)
    m, ex = np.frexp(val)
    e = ex - 1
    normal = (val > 0) & (e >= -6)
    expfield = np.where(normal, e + 7, 0).astype(np.int64)
    mant = np.where(normal, np.rint((m * 2.0 - 1.0) * 8.0), np.rint(val * 512.0)).astype(np.int64)
    bits = (expfield << 3) | mant
    bits = np.where(val == 0, 0, bits)
    bits = bits | (np.signbit(x).astype(np.int64) << 7)
    bits = np.where(nan, 0x7F, bits)
    return bits.astype(np.uint8)


def e4m3_decode(bits) -> np.ndarray:
    bits = np.asarray(bits, dtype=np.uint8).astype(np.int64)
    expfield = (bits >> 3) & 0xF
    mant = bits & 0x7
    val = np.where(
        expfield == 0,
        mant * 2.0 ** -9,
        (1.0 + mant / 8.0) * np.exp2((expfield - 7).astype(np.float64)),
    )
    val = np.where((bits & 0x7F) == 0x7F, np.nan, val)
    return np.where(bits & 0x80, -val, val).astype(np.float32)


def e2m1_encode(x) -> np.ndarray:
    """float array -> E2M1 codes 0..15 (bit 3 = sign); RN-even, saturate at 6."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    mag = np.where(np.isnan(mag), 0.0, mag)
    val = _round_to_grid(mag, 0, 1, 6.0)
    code = np.searchsorted(E2M1_MAGNITUDES.astype(np.float64), val).astype(np.int64)
    code = code | (np.signbit(x).astype(np.int64) << 3)
    return code.astype(np.uint8)


def e2m1_decode(code) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    val = E2M1_MAGNITUDES[code & 7]
    return np.where(code & 8, -val, val).astype(np.float32)


def nvfp4_scale_bits(amax: np.ndarray, global_scale: float) -> np.ndarray:
    """E4M3 scale byte of one 16-element group: e4m3((amax / 6) / global_scale)."""
    amax = np.asarray(amax, dtype=np.float32)
    return e4m3_encode((amax / np.float32(6.0)) / np.float32(global_scale))


def nvfp4_quantise(x16: np.ndarray, global_scale: float, axis: int = -1):
    """Quantise fp16 values in groups of 16 along ``axis``.

    Returns ``(codes uint8 same shape, scale bytes with the axis reduced by 16)``.
    ``scale = e4m3((amax/6)/gs)``; ``dq = e4m3_value(scale) * gs``;
    ``code = e2m1(x / dq)``, all zero when ``dq == 0``
    (q128_microscaling_preparation.cu:43-62,396-425).
    """
    x = np.moveaxis(np.asarray(x16, dtype=np.float16).astype(np.float32), axis, -1)
    shape = x.shape
    g = x.reshape(*shape[:-1], shape[-1] // 16, 16)
    amax = np.abs(g).max(axis=-1)
    sbits = nvfp4_scale_bits(amax, global_scale)
    dq = (e4m3_decode(sbits) * np.float32(global_scale)).astype(np.float32)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = np.where(dq == 0, np.float32(0), g / np.where(dq == 0, np.float32(1), dq))
    codes = np.where(dq == 0, 0, e2m1_encode(ratio.astype(np.float32))).astype(np.uint8)
    codes = np.moveaxis(codes.reshape(shape), -1, axis)
    sbits = np.moveaxis(sbits, -1, axis)
    return codes, sbits


def nvfp4_dequantise(codes: np.ndarray, sbits: np.ndarray, global_scale: float, axis: int = -1):
    c = np.moveaxis(e2m1_decode(codes), axis, -1)
    s = np.moveaxis(e4m3_decode(sbits), axis, -1)
    out = c.reshape(*s.shape, 16) * s[..., None] * np.float32(global_scale)
    return np.moveaxis(out.reshape(c.shape), -1, axis).astype(np.float32)
