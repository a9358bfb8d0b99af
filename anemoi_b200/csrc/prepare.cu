// Gather + narrow + pool + quantise: one pass over raw Q/K/V that fills the
// operand store (tile records) every later kernel consumes.  HBM-bandwidth bound.
//
// One CTA = one (task, head).  A task is a video query tile, a video key/value
// block (QB rows = QB/64 stages), a prefix key/value stage, or a prefix query
// tile.  The CTA gathers the tile's rows with 16-byte loads into shared memory
// (narrowed to fp16), derives pools / amax / scales from shared memory, and
// streams the tile records out with 16-byte coalesced stores.
//
// Numeric contract (reference: csrc/attention/cuda/sm120/q128_microscaling_preparation.cu):
//   narrow  bf16 -> f32 -> f16 rn (:227-232); invalid slots and prefix padding are +0 (:369-374)
//   mean    f16( sum_slots f32 in slot order / count ), IEEE division (:375-377,511-517)
//   max     over valid slots (:378-381)
//   INT8    scale = amax/127 + 1e-7; code = trunc(x/scale +- 0.5) (:458,503-506)
//   V E4M3  code = e4m3_satfinite(v * (2.25/amax_channel)); scale = amax/2.25 (:744-748,784-794)
//   NVFP4   scale = e4m3_satfinite((amax16/6)/gs); code = e2m1_rn(x/(e4m3(scale)*gs)) (:43-62)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "records.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kPad = 8;  // halves of padding per shared-memory row

struct PrepParams {
  anemoi_sm100_shape s;
  anemoi_sm100_operands o;
  const void* q;
  const void* k;
  const void* v;
  const int32_t* indices;
  const int32_t* counts;
  int prefix_stages, stages, prefix_q_tiles;
  int64_t stride[6];  // token and head stride (elements) of q, k, v
};

template <typename InT>
__device__ __forceinline__ uint4 load_narrow8(const InT* p);
// 8 raw 16-bit elements -> 8 fp16 (bf16 through fp32, round to nearest even; fp16 unchanged)
template <typename InT>
__device__ __forceinline__ uint4 narrow8(uint4 raw);
template <>
__device__ __forceinline__ uint4 narrow8<__half>(uint4 raw) {
  return raw;
}
template <>
__device__ __forceinline__ uint4 narrow8<__nv_bfloat16>(uint4 raw) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
  uint4 out;
  __half2* h = reinterpret_cast<__half2*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(b[i]);
    h[i] = __floats2half2_rn(f.x, f.y);
  }
  return out;
}

template <>
__device__ __forceinline__ uint4 load_narrow8<__half>(const __half* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
template <>
__device__ __forceinline__ uint4 load_narrow8<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
  uint4 out;
  __half2* h = reinterpret_cast<__half2*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(b[i]);
    h[i] = __floats2half2_rn(f.x, f.y);
  }
  return out;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) r = fmaxf(r, red[w]);
  return r;
}

__device__ __forceinline__ uint8_t nv_scale_byte(float amax, float gs) {
  return __nv_cvt_float_to_fp8(__fdiv_rn(__fdiv_rn(amax, 6.0f), gs), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t bits) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(bits, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// Correctly rounded x / y from the correctly rounded reciprocal `inv` = 1/y shared by a
// whole group: q0 = x*inv, residual r = x - q0*y (exact in an FMA), q = q0 + r*inv.  For the
// normal-range operands here this equals IEEE division bit for bit at a third of its cost.
__device__ __forceinline__ float div_rn(float x, float y, float inv) {
  const float q0 = __fmul_rn(x, inv);
  const float r = __fmaf_rn(-q0, y, x);
  return __fmaf_rn(r, inv, q0);
}
__device__ __forceinline__ uint8_t e2m1_pair(float lo, float hi, float dq, float inv_dq) {
  if (dq == 0.0f) return 0;
  return __nv_cvt_float2_to_fp4x2(make_float2(div_rn(lo, dq, inv_dq), div_rn(hi, dq, inv_dq)),
                                  __NV_E2M1, cudaRoundNearest);
}
__device__ __forceinline__ int8_t int8_code(float x, float scale, float inv_scale) {
  float t = div_rn(x, scale, inv_scale);
  t = __fadd_rn(t, t >= 0.0f ? 0.5f : -0.5f);
  return static_cast<int8_t>(__float2int_rz(t));
}

// Gathers ROWS rows into `tile` ([ROWS][D + kPad] halves), zero for invalid slots.  The trip
// count is a compile-time constant and the loop is split into a load pass and a store pass, so
// every thread has all of its 16-byte loads (and the slot-index loads before them) in flight at
// once: the kernel is bound by memory latency per CTA, not by arithmetic.
template <typename InT, int D, int ROWS>
__device__ __forceinline__ void gather_tile(__half* tile, const InT* src, const PrepParams& p,
                                            int head, bool video, int first_slot, int first_token,
                                            int valid_rows, int64_t token_stride,
                                            int64_t head_stride) {
  constexpr int kVec = D / 8;
  constexpr int kIter = ROWS * kVec / kThreads;
  static_assert(ROWS * kVec % kThreads == 0, "tile must be a multiple of the CTA's vector width");
  int64_t token[kIter];
#pragma unroll
  for (int i = 0; i < kIter; ++i) {
    const int r = (threadIdx.x + i * kThreads) / kVec;
    token[i] = r < valid_rows
                   ? (video ? (int64_t)p.s.prefix_tokens + __ldg(p.indices + first_slot + r)
                            : (int64_t)first_token + r)
                   : -1;
  }
  uint4 raw[kIter];
#pragma unroll
  for (int i = 0; i < kIter; ++i) {
    const int c8 = (threadIdx.x + i * kThreads) % kVec;
    raw[i] = make_uint4(0, 0, 0, 0);
    if (token[i] >= 0)
      raw[i] = __ldg(reinterpret_cast<const uint4*>(src + token[i] * token_stride +
                                                    (int64_t)head * head_stride + c8 * 8));
  }
#pragma unroll
  for (int i = 0; i < kIter; ++i) {
    const int idx = threadIdx.x + i * kThreads;
    const int r = idx / kVec, c8 = idx % kVec;
    *reinterpret_cast<uint4*>(tile + r * (D + kPad) + c8 * 8) = narrow8<InT>(raw[i]);
  }
}

// fp16 tile record (K-major image of `rows` x D; also used for the MN-major V tile).
template <int D>
__device__ __forceinline__ void write_fp16_tile(uint8_t* dst, const __half* tile, int row0,
                                                int rows) {
  constexpr int kChunks = D / 8;
  for (int idx = threadIdx.x; idx < rows * kChunks; idx += kThreads) {
    const int r = (idx / (8 * kChunks)) * 8 + (idx & 7), j = (idx >> 3) % kChunks;
    *reinterpret_cast<uint4*>(dst + (size_t)idx * 16) =
        *reinterpret_cast<const uint4*>(tile + (row0 + r) * (D + kPad) + j * 8);
  }
}

template <int D>
__device__ __forceinline__ float tile_amax(const __half* tile, int row0, int rows, float* red) {
  constexpr int kVec = D / 8;
  float m = 0.0f;
  for (int idx = threadIdx.x; idx < rows * kVec; idx += kThreads) {
    const int r = idx / kVec, c8 = idx % kVec;
    uint4 raw = *reinterpret_cast<const uint4*>(tile + (row0 + r) * (D + kPad) + c8 * 8);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  return block_max(m, red);
}

template <int D>
__device__ __forceinline__ void write_int8_tile(uint8_t* dst, const __half* tile, int row0,
                                                int rows, float scale) {
  constexpr int kChunks = D / 16;
  const float inv_scale = __frcp_rn(scale);
  for (int idx = threadIdx.x; idx < rows * kChunks; idx += kThreads) {
    const int r = (idx / (8 * kChunks)) * 8 + (idx & 7), j = (idx >> 3) % kChunks;
    const __half* src = tile + (row0 + r) * (D + kPad) + j * 16;
    uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 8);
    const __half* ha = reinterpret_cast<const __half*>(&a);
    const __half* hb = reinterpret_cast<const __half*>(&b);
    uint4 out;
    int8_t* c = reinterpret_cast<int8_t*>(&out);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      c[i] = int8_code(__half2float(ha[i]), scale, inv_scale);
      c[8 + i] = int8_code(__half2float(hb[i]), scale, inv_scale);
    }
    *reinterpret_cast<uint4*>(dst + (size_t)idx * 16) = out;
  }
}

// NVFP4 K-major tile (rows x D, groups of 16 channels) + scale blocks.
template <int D>
__device__ __forceinline__ void write_nvfp4_rows(uint8_t* codes, uint8_t* sf, const __half* tile,
                                                 int row0, int rows, float gs) {
  constexpr int kChunks = D / 32;
  for (int idx = threadIdx.x; idx < rows * kChunks; idx += kThreads) {
    const int r = (idx / (8 * kChunks)) * 8 + (idx & 7), j = (idx >> 3) % kChunks;
    const __half* src = tile + (row0 + r) * (D + kPad) + j * 32;
    uint4 out;
    uint8_t* c = reinterpret_cast<uint8_t*>(&out);
    uint8_t sb[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      uint4 a = *reinterpret_cast<const uint4*>(src + g * 16);
      uint4 b = *reinterpret_cast<const uint4*>(src + g * 16 + 8);
      float x[16];
      const __half* ha = reinterpret_cast<const __half*>(&a);
      const __half* hb = reinterpret_cast<const __half*>(&b);
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] = __half2float(ha[i]);
        x[8 + i] = __half2float(hb[i]);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
      sb[g] = nv_scale_byte(amax, gs);
      const float dq = __fmul_rn(e4m3_to_float(sb[g]), gs);
      const float inv_dq = __frcp_rn(dq);
#pragma unroll
      for (int i = 0; i < 8; ++i) c[g * 8 + i] = e2m1_pair(x[2 * i], x[2 * i + 1], dq, inv_dq);
    }
    *reinterpret_cast<uint4*>(codes + (size_t)idx * 16) = out;
    uint8_t* s = sf + (j >> 1) * 512 + rec::sf_offset(r, (j & 1) * 2);
    *reinterpret_cast<uint16_t*>(s) = (uint16_t)sb[0] | ((uint16_t)sb[1] << 8);
  }
}

// V^T tiles of one 64-key stage: channels x keys, keys contiguous.
template <int D>
__device__ __forceinline__ void write_v_e4m3(uint8_t* dst, const __half* tile, int row0,
                                             const float* recip) {
  for (int idx = threadIdx.x; idx < D * 4; idx += kThreads) {
    const int c = (idx >> 5) * 8 + (idx & 7), jj = (idx >> 3) & 3;
    const float rc = recip[c];
    uint4 out;
    uint8_t* o = reinterpret_cast<uint8_t*>(&out);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float v = __half2float(tile[(row0 + jj * 16 + i) * (D + kPad) + c]);
      o[i] = rc == 0.0f ? (uint8_t)0
                        : (uint8_t)__nv_cvt_float_to_fp8(__fmul_rn(v, rc), __NV_SATFINITE, __NV_E4M3);
    }
    *reinterpret_cast<uint4*>(dst + (size_t)idx * 16) = out;
  }
}

template <int D>
__device__ __forceinline__ void write_v_nvfp4(uint8_t* codes, uint8_t* sf, const __half* tile,
                                              int row0, float gs) {
  for (int idx = threadIdx.x; idx < D * 2; idx += kThreads) {
    const int c = (idx >> 4) * 8 + (idx & 7), jj = (idx >> 3) & 1;
    uint4 out;
    uint8_t* o = reinterpret_cast<uint8_t*>(&out);
    uint8_t sb[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float x[16];
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        x[i] = __half2float(tile[(row0 + jj * 32 + g * 16 + i) * (D + kPad) + c]);
        amax = fmaxf(amax, fabsf(x[i]));
      }
      sb[g] = nv_scale_byte(amax, gs);
      const float dq = __fmul_rn(e4m3_to_float(sb[g]), gs);
      const float inv_dq = __frcp_rn(dq);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[g * 8 + i] = e2m1_pair(x[2 * i], x[2 * i + 1], dq, inv_dq);
    }
    *reinterpret_cast<uint4*>(codes + (size_t)idx * 16) = out;
    uint8_t* s = sf + rec::sf_offset(c, jj * 2);
    *reinterpret_cast<uint16_t*>(s) = (uint16_t)sb[0] | ((uint16_t)sb[1] << 8);
  }
}

template <int D>
// `second`: the extra pool holds the second moments (mean of the squares, one FMA per row in
// row order; padding rows are zero) instead of the maxima - the diag-Jensen draft map's input.
__device__ __forceinline__ void write_pools(const __half* tile, int rows, int count, __half* mean,
                                            __half* maxp, bool second) {
  if (threadIdx.x < D) {
    const int c = threadIdx.x;
    float sum = 0.0f, mx = -INFINITY, sq = 0.0f;
#pragma unroll 8
    for (int r = 0; r < rows; ++r) {
      const float x = __half2float(tile[r * (D + kPad) + c]);
      sum = __fadd_rn(sum, x);
      sq = __fmaf_rn(x, x, sq);
      if (r < count) mx = fmaxf(mx, x);
    }
    mean[c] = __float2half_rn(__fdiv_rn(sum, (float)count));
    if (maxp != nullptr) maxp[c] = __float2half_rn(second ? __fdiv_rn(sq, (float)count) : mx);
  }
}

template <typename InT, int QB, int D>
__global__ void __launch_bounds__(kThreads) prepare_kernel(PrepParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* tile = reinterpret_cast<__half*>(smem_raw);
  __shared__ float red[kThreads / 32];
  __shared__ float recip[D];

  const int R = p.s.video_blocks;
  // heads vary fastest across concurrently running CTAs: neighbours read adjacent 2*D-byte
  // pieces of the same token rows
  const int head = blockIdx.x;
  const int task = blockIdx.y;
  constexpr int kF = QB / 64;
  const InT* q = static_cast<const InT*>(p.q);
  const InT* k = static_cast<const InT*>(p.k);
  const InT* v = static_cast<const InT*>(p.v);
  const int64_t qtiles_i8 = R + p.prefix_q_tiles;

  if (task < R || task >= 2 * R + p.prefix_stages) {
    // ---------------- query tile (video or prefix) ----------------
    const bool video = task < R;
    const int t = video ? task : task - (2 * R + p.prefix_stages);
    const int valid = video ? p.counts[t] : min(QB, p.s.prefix_tokens - t * QB);
    gather_tile<InT, D, QB>(tile, q, p, head, video, t * QB, t * QB, valid, p.stride[0],
                            p.stride[1]);
    __syncthreads();
    if (video) {
      __half* mean = static_cast<__half*>(p.o.q_pool) + ((int64_t)head * R + t) * D;
      __half* mx = p.s.has_maxpool
                       ? static_cast<__half*>(p.o.q_max_pool) + ((int64_t)head * R + t) * D
                       : nullptr;
      write_pools<D>(tile, QB, valid, mean, mx, p.s.has_maxpool == 2);
      if (p.s.has_fp16) {
        write_fp16_tile<D>(static_cast<uint8_t*>(p.o.q_fp16) +
                               ((int64_t)head * R + t) * rec::q_fp16_bytes(QB, D),
                           tile, 0, QB);
      }
      if (p.s.has_nvfp4) {
        uint8_t* r4 = static_cast<uint8_t*>(p.o.q_nvfp4) +
                      ((int64_t)head * R + t) * rec::q_nvfp4_bytes(QB, D);
        write_nvfp4_rows<D>(r4, r4 + QB * D / 2, tile, 0, QB, p.s.q_global_scale);
      }
    }
    if (p.s.has_int8) {
      const int64_t slot = (int64_t)head * qtiles_i8 + (video ? t : R + t);
      const float amax = tile_amax<D>(tile, 0, QB, red);
      const float scale = __fadd_rn(__fdiv_rn(amax, 127.0f), 1.0e-7f);
      if (threadIdx.x == 0) p.o.q_int8_scale[slot] = scale;
      write_int8_tile<D>(static_cast<uint8_t*>(p.o.q_int8) + slot * rec::q_int8_bytes(QB, D), tile,
                         0, QB, scale);
    }
    return;
  }

  // ---------------- key/value block (video) or stage (prefix) ----------------
  const bool video = task < 2 * R;
  const int b = video ? task - R : task - 2 * R;
  const int nst = video ? kF : 1;
  const int stage0 = video ? p.prefix_stages + b * kF : b;
  const int valid = video ? p.counts[b] : min(64, p.s.prefix_tokens - b * 64);
  const int64_t rec0 = (int64_t)head * p.stages + stage0;

  if (video) {
    gather_tile<InT, D, QB>(tile, k, p, head, true, b * QB, 0, valid, p.stride[2], p.stride[3]);
  } else {
    gather_tile<InT, D, 64>(tile, k, p, head, false, 0, b * 64, valid, p.stride[2], p.stride[3]);
  }
  __syncthreads();
  if (video) {
    __half* mean = static_cast<__half*>(p.o.k_pool) + ((int64_t)head * R + b) * D;
    __half* mx = p.s.has_maxpool
                     ? static_cast<__half*>(p.o.k_max_pool) + ((int64_t)head * R + b) * D
                     : nullptr;
    write_pools<D>(tile, QB, valid, mean, mx, p.s.has_maxpool == 2);
  }
  for (int g = 0; g < nst; ++g) {
    if (p.s.has_fp16) {
      write_fp16_tile<D>(static_cast<uint8_t*>(p.o.kv_fp16) + (rec0 + g) * rec::kv_fp16_bytes(D),
                         tile, g * 64, 64);
    }
    if (p.s.has_int8) {
      const float amax = tile_amax<D>(tile, g * 64, 64, red);
      const float scale = __fadd_rn(__fdiv_rn(amax, 127.0f), 1.0e-7f);
      if (threadIdx.x == 0) p.o.k_int8_scale[rec0 + g] = scale;
      write_int8_tile<D>(static_cast<uint8_t*>(p.o.kv_int8) + (rec0 + g) * rec::kv_int8_bytes(D),
                         tile, g * 64, 64, scale);
    }
    if (p.s.has_nvfp4) {
      uint8_t* r4 = static_cast<uint8_t*>(p.o.kv_nvfp4) + (rec0 + g) * rec::kv_nvfp4_bytes(D);
      write_nvfp4_rows<D>(r4, r4 + rec::kv_nvfp4_ksf_offset(D), tile, g * 64, 64,
                          p.s.k_global_scale);
    }
  }
  __syncthreads();

  // ---- values of the same rows ----
  if (video) {
    gather_tile<InT, D, QB>(tile, v, p, head, true, b * QB, 0, valid, p.stride[4], p.stride[5]);
  } else {
    gather_tile<InT, D, 64>(tile, v, p, head, false, 0, b * 64, valid, p.stride[4], p.stride[5]);
  }
  if (p.s.has_int8 && threadIdx.x < D) {
    const float amax =
        __half2float(__float2half_rn(p.o.v_amax[(int64_t)head * D + threadIdx.x]));
    recip[threadIdx.x] = amax == 0.0f ? 0.0f : __fdiv_rn(2.25f, amax);
    if (task == R) p.o.v_e4m3_scale[(int64_t)head * D + threadIdx.x] = __fdiv_rn(amax, 2.25f);
  }
  __syncthreads();
  for (int g = 0; g < nst; ++g) {
    if (p.s.has_fp16) {
      write_fp16_tile<D>(static_cast<uint8_t*>(p.o.kv_fp16) + (rec0 + g) * rec::kv_fp16_bytes(D) +
                             64 * D * 2,
                         tile, g * 64, 64);
    }
    if (p.s.has_int8) {
      write_v_e4m3<D>(static_cast<uint8_t*>(p.o.kv_int8) + (rec0 + g) * rec::kv_int8_bytes(D) +
                          64 * D,
                      tile, g * 64, recip);
    }
    if (p.s.has_nvfp4) {
      uint8_t* r4 = static_cast<uint8_t*>(p.o.kv_nvfp4) + (rec0 + g) * rec::kv_nvfp4_bytes(D);
      write_v_nvfp4<D>(r4 + rec::kv_nvfp4_v_offset(D), r4 + rec::kv_nvfp4_vsf_offset(D), tile,
                       g * 64, p.s.v_global_scale);
    }
  }
}

// max |v| per (head, channel) over every token, as the bit pattern of a
// non-negative float (integer max == float max).  `out` must be zeroed first.
template <typename InT>
__global__ void __launch_bounds__(256) v_amax_kernel(const InT* v, int* out, int64_t tokens,
                                                     int heads, int d8, int64_t token_stride,
                                                     int64_t head_stride, int tokens_per_block) {
  const int col8 = blockIdx.x * 256 + threadIdx.x;
  if (col8 >= heads * d8) return;
  const int head = col8 / d8, c8 = col8 % d8;
  const int64_t t0 = (int64_t)blockIdx.y * tokens_per_block;
  const int64_t t1 = min(tokens, t0 + tokens_per_block);
  float m[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t t = t0; t < t1; ++t) {
    uint4 raw = load_narrow8<InT>(v + t * token_stride + head * head_stride + c8 * 8);
    const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = fmaxf(m[i], fabsf(__half2float(h[i])));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) atomicMax(out + col8 * 8 + i, __float_as_int(m[i]));
}

template <typename InT, int QB, int D>
int launch(const PrepParams& p, cudaStream_t stream) {
  const size_t smem = (size_t)QB * (D + kPad) * sizeof(__half);
  auto kernel = prepare_kernel<InT, QB, D>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  if (p.s.has_int8) {
    if (cudaMemsetAsync(p.o.v_amax, 0, sizeof(float) * p.s.heads * D, stream) != cudaSuccess)
      return ANEMOI_SM100_ELAUNCH;
    const int cols = p.s.heads * D / 8;
    const int tokens_per_block = 128;
    dim3 grid((cols + 255) / 256, (p.s.seq_tokens + tokens_per_block - 1) / tokens_per_block);
    v_amax_kernel<InT><<<grid, 256, 0, stream>>>(
        static_cast<const InT*>(p.v), reinterpret_cast<int*>(p.o.v_amax), p.s.seq_tokens,
        p.s.heads, D / 8, p.stride[4], p.stride[5], tokens_per_block);
  }
  const int tasks = 2 * p.s.video_blocks + p.prefix_stages + p.prefix_q_tiles;
  if (tasks > 65535) return ANEMOI_SM100_ELIMIT;
  dim3 grid(p.s.heads, tasks);
  kernel<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

}  // namespace

extern "C" int anemoi_sm100_arch(void) { return 100; }

extern "C" int64_t anemoi_sm100_operand_bytes(const anemoi_sm100_shape* s, int which) {
  if (rec::validate_shape(s) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  const int64_t H = s->heads, D = s->head_dim, QB = s->query_block, R = s->video_blocks;
  const int64_t NS = rec::stages(*s), PQ = rec::prefix_query_tiles(*s);
  switch (which) {
    case ANEMOI_SM100_BUF_Q_FP16: return s->has_fp16 ? H * R * rec::q_fp16_bytes(QB, D) : 0;
    case ANEMOI_SM100_BUF_KV_FP16: return s->has_fp16 ? H * NS * rec::kv_fp16_bytes(D) : 0;
    case ANEMOI_SM100_BUF_Q_INT8: return s->has_int8 ? H * (R + PQ) * rec::q_int8_bytes(QB, D) : 0;
    case ANEMOI_SM100_BUF_KV_INT8: return s->has_int8 ? H * NS * rec::kv_int8_bytes(D) : 0;
    case ANEMOI_SM100_BUF_Q_NVFP4: return s->has_nvfp4 ? H * R * rec::q_nvfp4_bytes(QB, D) : 0;
    case ANEMOI_SM100_BUF_KV_NVFP4: return s->has_nvfp4 ? H * NS * rec::kv_nvfp4_bytes(D) : 0;
    case ANEMOI_SM100_BUF_Q_INT8_SCALE: return s->has_int8 ? H * (R + PQ) * 4 : 0;
    case ANEMOI_SM100_BUF_K_INT8_SCALE: return s->has_int8 ? H * NS * 4 : 0;
    case ANEMOI_SM100_BUF_V_E4M3_SCALE: return s->has_int8 ? H * D * 4 : 0;
    case ANEMOI_SM100_BUF_V_AMAX: return s->has_int8 ? H * D * 4 : 0;
    case ANEMOI_SM100_BUF_POOL: return H * R * D * 2;
    default: return ANEMOI_SM100_EINVAL;
  }
}

extern "C" int anemoi_sm100_prepare(const anemoi_sm100_shape* shape, const void* q, const void* k,
                                    const void* v, const int64_t* strides, const int32_t* indices,
                                    const int32_t* counts, const anemoi_sm100_operands* out,
                                    void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !q || !k || !v || !indices || !counts || !out)
    return ANEMOI_SM100_EINVAL;
  const anemoi_sm100_shape& s = *shape;
  if (!out->q_pool || !out->k_pool) return ANEMOI_SM100_EINVAL;
  if (s.has_maxpool && (!out->q_max_pool || !out->k_max_pool)) return ANEMOI_SM100_EINVAL;
  if (s.has_fp16 && (!out->q_fp16 || !out->kv_fp16)) return ANEMOI_SM100_EINVAL;
  if (s.has_int8 && (!out->q_int8 || !out->kv_int8 || !out->q_int8_scale || !out->k_int8_scale ||
                     !out->v_e4m3_scale || !out->v_amax))
    return ANEMOI_SM100_EINVAL;
  if (s.has_nvfp4 && (!out->q_nvfp4 || !out->kv_nvfp4)) return ANEMOI_SM100_EINVAL;
  PrepParams p;
  p.s = s;
  p.o = *out;
  p.q = q;
  p.k = k;
  p.v = v;
  p.indices = indices;
  p.counts = counts;
  for (int i = 0; i < 6; ++i) {
    p.stride[i] = strides ? strides[i] : (i & 1 ? (int64_t)s.head_dim : (int64_t)s.heads * s.head_dim);
    if (p.stride[i] <= 0 || p.stride[i] % 8) return ANEMOI_SM100_EINVAL;
  }
  p.prefix_stages = rec::prefix_stages(s);
  p.stages = rec::stages(s);
  p.prefix_q_tiles = rec::prefix_query_tiles(s);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define ANEMOI_DISPATCH(T)                                                        \
  (s.query_block == 64 ? (s.head_dim == 64 ? launch<T, 64, 64>(p, st) : launch<T, 64, 128>(p, st)) \
                       : (s.head_dim == 64 ? launch<T, 128, 64>(p, st) : launch<T, 128, 128>(p, st)))
  return s.input_is_bf16 ? ANEMOI_DISPATCH(__nv_bfloat16) : ANEMOI_DISPATCH(__half);
#undef ANEMOI_DISPATCH
}
