// Producer-side fusion in front of the attention path: per-head RMS norm with weight, then
// partial rotary embedding, in place on Q or K ([tokens][heads][D], 16-bit).  One pass over HBM
// (read + write) instead of the six of an eager implementation.
//
// Follows the reference's fused kernel
// (anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/fusions.py:208-274):
//   variance = sum_j x_j^2 / D;  r = 1/sqrt(variance + eps);  n_j = (x_j * r) * w_j
//   inside the rotary span [0, rotary_dim), half = rotary_dim/2, channel j pairs with j +- half:
//     out_j = n_j * cos_j + rot_j * sin_j,  rot_j = -n_{j+half} (j < half), +n_{j-half} (j >= half)
//   outside it out_j = n_j; cos/sin are fp32 tables [tokens][rotary_dim] shared by the heads.
// The reference leaves the summation order and the contraction of the last line to its
// compiler; here they are fixed so that a CPU restatement reproduces every bit: each thread
// sums its 8 channels with a sequential FMA chain, the D/8 threads of a row combine with an
// xor butterfly (largest offset first), r is an IEEE division by an IEEE square root, and
// out_j = fma(rot_j, sin_j, round(n_j * cos_j)).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/anemoi_sm100.h"

namespace {

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

// One row (token, head) per group of D/8 consecutive lanes, 8 channels per thread; every thread
// walks kRows rows (a block covers kRows consecutive slabs of rows) with all of their 16-byte
// loads issued before the first use, so that enough bytes are in flight per SM.
constexpr int kRows = 1;

template <typename T, int D>
__global__ void __launch_bounds__(256) qknorm_rope_kernel(T* x, const T* weight, const float* cos_table,
                                                          const float* sin_table, int64_t rows,
                                                          int heads, int rotary_dim, float eps,
                                                          int64_t token_stride, int64_t head_stride) {
  constexpr int kLanes = D / 8;
  constexpr int kSlab = 256 / kLanes;  // rows per block and pass
  const int lane = threadIdx.x % kLanes;
  const int64_t row0 = (int64_t)blockIdx.x * (kSlab * kRows) + threadIdx.x / kLanes;

  T* ptr[kRows];
  int64_t token[kRows];
  bool live[kRows];
  uint4 raw[kRows];
#pragma unroll
  for (int k = 0; k < kRows; ++k) {
    const int64_t row = row0 + (int64_t)k * kSlab;
    live[k] = row < rows;
    // rows < 2^31 (checked by the launcher): 32-bit division
    const uint32_t r32 = live[k] ? (uint32_t)row : 0u;
    token[k] = r32 / (uint32_t)heads;
    const int head = (int)(r32 - (uint32_t)token[k] * (uint32_t)heads);
    ptr[k] = x + token[k] * token_stride + (int64_t)head * head_stride + lane * 8;
    raw[k] = make_uint4(0, 0, 0, 0);
    if (live[k]) raw[k] = *reinterpret_cast<const uint4*>(ptr[k]);
  }
  const uint4 wraw = *reinterpret_cast<const uint4*>(weight + lane * 8);
  const T* w = reinterpret_cast<const T*>(&wraw);
  // partner channels live half/8 lanes away (rotary_dim is a multiple of 16)
  const int half = rotary_dim / 2;
  const int c0 = lane * 8;
  const bool rotary = c0 < rotary_dim;
  const bool first = c0 < half;
  const int partner_lane = first ? lane + half / 8 : lane - half / 8;

#pragma unroll
  for (int k = 0; k < kRows; ++k) {
    const T* e = reinterpret_cast<const T*>(&raw[k]);
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
    float n[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) n[i] = __fmul_rn(__fmul_rn(v[i], r), to_float<T>(w[i]));

    float out[8];
    float cs[8], sn[8];
    if (rotary && live[k]) {
      // 8 consecutive table entries of this token: two 16-byte loads each (rotary_dim % 16 == 0)
      const float4* ct = reinterpret_cast<const float4*>(cos_table + token[k] * rotary_dim + c0);
      const float4* st = reinterpret_cast<const float4*>(sin_table + token[k] * rotary_dim + c0);
      *reinterpret_cast<float4*>(cs) = __ldg(ct);
      *reinterpret_cast<float4*>(cs + 4) = __ldg(ct + 1);
      *reinterpret_cast<float4*>(sn) = __ldg(st);
      *reinterpret_cast<float4*>(sn + 4) = __ldg(st + 1);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // every lane takes part in the shuffle; lanes outside the span read themselves
      const float pn = __shfl_sync(0xffffffffu, n[i], rotary ? partner_lane : lane, kLanes);
      out[i] = n[i];
      if (rotary && live[k]) out[i] = __fmaf_rn(first ? -pn : pn, sn[i], __fmul_rn(n[i], cs[i]));
    }
    if (live[k]) {
      uint4 packed;
      T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = from_float<T>(out[i]);
      *reinterpret_cast<uint4*>(ptr[k]) = packed;
    }
  }
}

template <typename T>
int launch(void* x, const void* weight, const float* c, const float* s, int64_t tokens, int heads, int d,
           int rotary, float eps, const int64_t* strides, cudaStream_t st) {
  const int64_t rows = tokens * heads;
  const int64_t rows_per_block = (256 / (d / 8)) * kRows;
  const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  if (blocks > 0x7fffffffLL || rows > 0x7fffffffLL) return ANEMOI_SM100_ELIMIT;
  if (d == 64) {
    qknorm_rope_kernel<T, 64><<<(unsigned)blocks, 256, 0, st>>>(static_cast<T*>(x), static_cast<const T*>(weight),
                                                                c, s, rows, heads, rotary, eps, strides[0], strides[1]);
  } else {
    qknorm_rope_kernel<T, 128><<<(unsigned)blocks, 256, 0, st>>>(static_cast<T*>(x), static_cast<const T*>(weight),
                                                                 c, s, rows, heads, rotary, eps, strides[0], strides[1]);
  }
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

}  // namespace

extern "C" int anemoi_sm100_qknorm_rope(void* x, const void* weight, const float* cos_table,
                                        const float* sin_table, int64_t tokens, int32_t heads,
                                        int32_t head_dim, int32_t rotary_dim, float eps, int32_t is_bf16,
                                        const int64_t* strides, void* stream) {
  if (!x || !weight || !strides || tokens < 0 || heads <= 0) return ANEMOI_SM100_EINVAL;
  if (rotary_dim > 0 && (!cos_table || !sin_table)) return ANEMOI_SM100_EINVAL;
  if (head_dim != 64 && head_dim != 128) return ANEMOI_SM100_EINVAL;
  // the pairing j <-> j + rotary_dim/2 must move whole 8-channel vectors
  if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 16) return ANEMOI_SM100_EINVAL;
  if (strides[0] % 8 || strides[1] % 8 || !(eps >= 0.0f)) return ANEMOI_SM100_EINVAL;
  if (tokens == 0) return ANEMOI_SM100_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return is_bf16 ? launch<__nv_bfloat16>(x, weight, cos_table, sin_table, tokens, heads, head_dim, rotary_dim,
                                         eps, strides, st)
                 : launch<__half>(x, weight, cos_table, sin_table, tokens, heads, head_dim, rotary_dim, eps,
                                  strides, st);
}
