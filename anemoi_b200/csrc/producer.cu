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
#include "norm_rope.cuh"

namespace {

// One row (token, head) per group of D/8 consecutive lanes; 8 channels per thread.
template <typename T, int D>
__global__ void __launch_bounds__(256) qknorm_rope_kernel(T* x, const T* weight, const float* cos_table,
                                                          const float* sin_table, int64_t rows,
                                                          int heads, int rotary_dim, float eps,
                                                          int64_t token_stride, int64_t head_stride) {
  constexpr int kLanes = D / 8;
  const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) / kLanes;
  const int lane = threadIdx.x % kLanes;
  const bool live = row < rows;
  // rows < 2^31 (checked by the launcher): 32-bit division
  const uint32_t r32 = live ? (uint32_t)row : 0u;
  const int64_t token = r32 / (uint32_t)heads;
  const int head = (int)(r32 - (uint32_t)token * (uint32_t)heads);
  T* p = x + token * token_stride + (int64_t)head * head_stride + lane * 8;
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (live) raw = *reinterpret_cast<const uint4*>(p);
  const uint4 out = nr::norm_rope8<T, D>(raw, weight, cos_table + token * rotary_dim,
                                         sin_table + token * rotary_dim, rotary_dim, eps, lane, live);
  if (live) *reinterpret_cast<uint4*>(p) = out;
}

template <typename T>
int launch(void* x, const void* weight, const float* c, const float* s, int64_t tokens, int heads, int d,
           int rotary, float eps, const int64_t* strides, cudaStream_t st) {
  const int64_t rows = tokens * heads;
  const int64_t rows_per_block = 256 / (d / 8);
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
