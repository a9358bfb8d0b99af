// Per-head RMS norm with weight + partial rotary embedding of one row, 8 channels per thread,
// D/8 consecutive lanes per row (shared by the stand-alone producer kernel and by the gather of
// the preparation kernel).  Formula and canonical arithmetic: see producer.cu.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace nr {

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__half>(__half v) {
  return __half2float(v);
}
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// `raw`: the thread's 8 channels (lane * 8 ...) of the row, zeros for a row that is not live.
// Every lane of the warp must call this (it shuffles inside groups of D/8 lanes).  `cos_row` /
// `sin_row` point at the row's token in the fp32 tables ([rotary_dim] entries); they are only
// read by live lanes inside the rotary span.  Returns the 8 results rounded to T.
template <typename T, int D>
__device__ __forceinline__ uint4 norm_rope8(uint4 raw, const T* weight, const float* cos_row,
                                            const float* sin_row, int rotary_dim, float eps, int lane,
                                            bool live) {
  constexpr int kLanes = D / 8;
  const T* e = reinterpret_cast<const T*>(&raw);
  float v[8];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = to_float<T>(e[i]);
    sum = __fmaf_rn(v[i], v[i], sum);
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, off));
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)D), eps)));
  const uint4 wraw = *reinterpret_cast<const uint4*>(weight + lane * 8);
  const T* w = reinterpret_cast<const T*>(&wraw);
  float n[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) n[i] = __fmul_rn(__fmul_rn(v[i], r), to_float<T>(w[i]));

  // partner channels live half/8 lanes away (rotary_dim is a multiple of 16)
  const int half = rotary_dim / 2;
  const int c0 = lane * 8;
  const bool rotary = c0 < rotary_dim;
  const bool first = c0 < half;
  const int partner_lane = first ? lane + half / 8 : lane - half / 8;
  float cs[8], sn[8];
  if (rotary && live) {
    // 8 consecutive table entries of this token: two 16-byte loads each
    const float4* ct = reinterpret_cast<const float4*>(cos_row + c0);
    const float4* st = reinterpret_cast<const float4*>(sin_row + c0);
    *reinterpret_cast<float4*>(cs) = __ldg(ct);
    *reinterpret_cast<float4*>(cs + 4) = __ldg(ct + 1);
    *reinterpret_cast<float4*>(sn) = __ldg(st);
    *reinterpret_cast<float4*>(sn + 4) = __ldg(st + 1);
  }
  uint4 packed;
  T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // every lane takes part in the shuffle; lanes outside the span read themselves
    const float pn = __shfl_sync(0xffffffffu, n[i], rotary ? partner_lane : lane, kLanes);
    float out = n[i];
    if (rotary && live) out = __fmaf_rn(first ? -pn : pn, sn[i], __fmul_rn(n[i], cs[i]));
    o[i] = from_float<T>(out);
  }
  return packed;
}

}  // namespace nr
