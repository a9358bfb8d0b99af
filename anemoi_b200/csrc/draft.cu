// Draft probability: pooled-QK logits (fp32 accumulate, rounded to fp16), row
// softmax in fp32, optional mean/max blend, fp16 result [H][R][R].
//
// Reference: csrc/attention/cuda/sm120/h3_draft_probability.cu:131-222 (softmax
// and blend) and :427-465 (cuBLAS pooled GEMM, fp16 logits).  The reference
// leaves the accumulation order to cuBLAS and uses a fast-math expf, so its own
// map is only reproducible to ~5e-4; the routing that follows ranks these values
// globally, so here every operation is fixed and individually rounded:
//   dot     acc = fma(q[c], k[c], acc) for c = 0..D-1 (products of fp16 values are
//           exact in fp32, so this equals a separately rounded add)
//   logit   f16_rn(acc * f32(1/sqrt(D)))
//   exp     y = max(t*log2e, -125); n = rint(y); f = y - n;
//           p = Horner degree 7 of 2^f with rounded multiplies and adds; e = p * 2^n
//   sum     lane l adds columns l, l+32, ... ascending; lanes are folded with an
//           xor butterfly 16, 8, 4, 2, 1
//   prob    f16_rn(e * (1/sum)), IEEE reciprocal; blend f16_rn((1-w)*pm + w*px)
// A CPU restatement with the same sequence reproduces the map bit for bit.
#include <cuda_fp16.h>

#include "records.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kChunk = 128;                   // key blocks per pass: 4 per lane
constexpr int kPitch = kChunk + 4;            // floats per channel row of the key tile
constexpr int kSlab = 64;                     // channels of the key tile held at a time
constexpr int kMaxBlocks = 4096;              // rows per head the shared-memory buffers allow

__device__ __forceinline__ float exp_canonical(float t) {
  const float y = fmaxf(__fmul_rn(t, __int_as_float(0x3fb8aa3b)), -125.0f);
  const float n = rintf(y);
  const float f = __fsub_rn(y, n);
  float p = __int_as_float(0x377fe5fe);
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x39218489));
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3aaec3ff));
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3c1d955b));
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3d635847));
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3e75fdf0));
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3f317218));
  p = __fadd_rn(__fmul_rn(p, f), 1.0f);
  return __fmul_rn(p, __int_as_float((static_cast<int>(n) + 127) << 23));
}

// fp16 logits of kWarps * RPW query blocks against every key block of the head.  Each warp owns
// RPW (2 or 4) rows, each lane four key columns of the 128-column pass: per channel one 16-byte
// load of keys (four shared-memory wavefronts per warp) and one broadcast load of the warp's
// query values feed 4 * RPW FMAs, so with four rows the FMA pipe rather than shared memory
// sets the pace.  Every logit is still the plain channel-ordered FMA chain (the canonical
// order).
template <int D, int RPW>
__device__ __forceinline__ void row_logits(const __half* q_pool, const __half* k_pool, int head,
                                           int R, int row0, float* kc, float* qs, __half* lg,
                                           int lg_stride) {
  constexpr int kRows = kWarps * RPW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = D == 64 ? 0.125f : __int_as_float(0x3db504f3);
  // query pools as floats, the rows of a warp interleaved: qs[warp][channel][RPW]
  for (int idx = threadIdx.x; idx < kRows * D; idx += kWarps * 32) {
    const int r = idx / D, c = idx % D;
    const int row = row0 + r;
    qs[((r / RPW) * D + c) * RPW + (r % RPW)] =
        row < R ? __half2float(q_pool[((int64_t)head * R + row) * D + c]) : 0.0f;
  }
  for (int c0 = 0; c0 < R; c0 += kChunk) {
    float acc[RPW][4];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[r][j] = 0.0f;
    const float* qw = qs + warp * D * RPW;
    // the key tile is staged kSlab channels at a time; the chain still runs over c = 0..D-1
    for (int s0 = 0; s0 < D; s0 += kSlab) {
      __syncthreads();
      // key pools of columns [c0, c0 + kChunk), channels [s0, s0 + kSlab), as [channel][column] floats
      for (int idx = threadIdx.x; idx < kChunk * (kSlab / 8); idx += kWarps * 32) {
        const int col = idx % kChunk, c8 = idx / kChunk;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (c0 + col < R)
          raw = __ldg(reinterpret_cast<const uint4*>(k_pool + ((int64_t)head * R + c0 + col) * D + s0) + c8);
        const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) kc[(c8 * 8 + i) * kPitch + col] = __half2float(h[i]);
      }
      __syncthreads();
#pragma unroll 4
      for (int c = 0; c < kSlab; ++c) {
        float qv[RPW];
        if (RPW == 4) {
          const float4 t = *reinterpret_cast<const float4*>(qw + (s0 + c) * 4);
          qv[0] = t.x;
          qv[1] = t.y;
          qv[RPW - 2] = t.z;
          qv[RPW - 1] = t.w;
        } else {
          const float2 t = *reinterpret_cast<const float2*>(qw + (s0 + c) * 2);
          qv[0] = t.x;
          qv[1] = t.y;
        }
        const float4 kv = *reinterpret_cast<const float4*>(kc + c * kPitch + lane * 4);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          acc[r][0] = __fmaf_rn(qv[r], kv.x, acc[r][0]);
          acc[r][1] = __fmaf_rn(qv[r], kv.y, acc[r][1]);
          acc[r][2] = __fmaf_rn(qv[r], kv.z, acc[r][2]);
          acc[r][3] = __fmaf_rn(qv[r], kv.w, acc[r][3]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = c0 + lane * 4 + j;
        if (col < R)
          lg[(warp * RPW + r) * lg_stride + col] = __float2half_rn(__fmul_rn(acc[r][j], scale));
      }
  }
  __syncwarp();
}

// max and 1/sum of one row held in shared memory (warp-collective).
__device__ __forceinline__ void row_stats(const __half* lg, int R, float& mx, float& inv) {
  const int lane = threadIdx.x & 31;
  float m = -INFINITY;
  for (int j = lane; j < R; j += 32) m = fmaxf(m, __half2float(lg[j]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  float s = 0.0f;
  for (int j = lane; j < R; j += 32) s = __fadd_rn(s, exp_canonical(__fsub_rn(__half2float(lg[j]), m)));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
  mx = m;
  inv = __fdiv_rn(1.0f, s);
}

// ---- diag-Jensen variant (an experimental routing proxy of the reference,
// anemoi/layers/attention/mpa/routing.py:87-103) -------------------------------------------
//   logit = q.k/sqrt(D) + 0.5 * max((q2.k2 - (q*q).(k*k)) / D, 0)   in fp32, not rounded to fp16
// q2, k2: per-channel second moments of the blocks.  Three dot products per pair, each the same
// channel-ordered FMA chain as above (two rows per warp, four key columns per lane); the third
// one's inputs are the fp32 squares of the pools.  kStep 0: base = round(acc * scale) stored;
// 1: v = acc stored in the second buffer; 2: logit = fma(0.5, max((v - acc) / D, 0), base).
template <int D, int kStep>
__device__ __forceinline__ void jensen_pass(const __half* q_src, const __half* k_src, int head, int R,
                                            int row0, float* kc, float* qs, float* lg, float* var,
                                            int stride) {
  constexpr int kRows = kWarps * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = D == 64 ? 0.125f : __int_as_float(0x3db504f3);
  __syncthreads();
  for (int idx = threadIdx.x; idx < kRows * D; idx += kWarps * 32) {
    const int r = idx / D, c = idx % D;
    const int row = row0 + r;
    float x = row < R ? __half2float(q_src[((int64_t)head * R + row) * D + c]) : 0.0f;
    if (kStep == 2) x = __fmul_rn(x, x);
    qs[((r >> 1) * D + c) * 2 + (r & 1)] = x;
  }
  for (int c0 = 0; c0 < R; c0 += kChunk) {
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const float* qw = qs + warp * D * 2;
    for (int s0 = 0; s0 < D; s0 += kSlab) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < kChunk * (kSlab / 8); idx += kWarps * 32) {
        const int col = idx % kChunk, c8 = idx / kChunk;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (c0 + col < R)
          raw = __ldg(reinterpret_cast<const uint4*>(k_src + ((int64_t)head * R + c0 + col) * D + s0) + c8);
        const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float x = __half2float(h[i]);
          if (kStep == 2) x = __fmul_rn(x, x);
          kc[(c8 * 8 + i) * kPitch + col] = x;
        }
      }
      __syncthreads();
#pragma unroll 4
      for (int c = 0; c < kSlab; ++c) {
        const float2 qv = *reinterpret_cast<const float2*>(qw + (s0 + c) * 2);
        const float4 kv = *reinterpret_cast<const float4*>(kc + c * kPitch + lane * 4);
        acc[0][0] = __fmaf_rn(qv.x, kv.x, acc[0][0]);
        acc[0][1] = __fmaf_rn(qv.x, kv.y, acc[0][1]);
        acc[0][2] = __fmaf_rn(qv.x, kv.z, acc[0][2]);
        acc[0][3] = __fmaf_rn(qv.x, kv.w, acc[0][3]);
        acc[1][0] = __fmaf_rn(qv.y, kv.x, acc[1][0]);
        acc[1][1] = __fmaf_rn(qv.y, kv.y, acc[1][1]);
        acc[1][2] = __fmaf_rn(qv.y, kv.z, acc[1][2]);
        acc[1][3] = __fmaf_rn(qv.y, kv.w, acc[1][3]);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = c0 + lane * 4 + j;
        if (col >= R) continue;
        const int at = (warp * 2 + r) * stride + col;
        if (kStep == 0) {
          lg[at] = __fmul_rn(acc[r][j], scale);
        } else if (kStep == 1) {
          var[at] = acc[r][j];
        } else {
          const float t = fmaxf(__fmul_rn(__fsub_rn(var[at], acc[r][j]), 1.0f / D), 0.0f);
          lg[at] = __fmaf_rn(0.5f, t, lg[at]);
        }
      }
  }
  __syncwarp();
}

template <int D>
__global__ void __launch_bounds__(kWarps * 32) draft_jensen_kernel(const __half* q_pool,
                                                                   const __half* k_pool,
                                                                   const __half* q_second,
                                                                   const __half* k_second, int R,
                                                                   __half* prob) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr int kRows = kWarps * 2;
  const int stride = (R + 3) & ~3;
  float* kc = reinterpret_cast<float*>(smem_raw);  // [kSlab][kPitch]
  float* qs = kc + kSlab * kPitch;                 // [kWarps][D][2]
  float* lg = qs + kRows * D;                      // [kRows][stride] fp32 logits
  float* var = lg + kRows * stride;                // [kRows][stride]
  const int head = blockIdx.y, row0 = blockIdx.x * kRows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  jensen_pass<D, 0>(q_pool, k_pool, head, R, row0, kc, qs, lg, var, stride);
  jensen_pass<D, 1>(q_second, k_second, head, R, row0, kc, qs, lg, var, stride);
  jensen_pass<D, 2>(q_pool, k_pool, head, R, row0, kc, qs, lg, var, stride);
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + warp * 2 + r;
    if (row >= R) break;
    const float* mine = lg + (warp * 2 + r) * stride;
    float m = -INFINITY;
    for (int j = lane; j < R; j += 32) m = fmaxf(m, mine[j]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float sum = 0.0f;
    for (int j = lane; j < R; j += 32) sum = __fadd_rn(sum, exp_canonical(__fsub_rn(mine[j], m)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, off));
    const float inv = __fdiv_rn(1.0f, sum);
    __half* out = prob + ((int64_t)head * R + row) * R;
    for (int j = lane; j < R; j += 32)
      out[j] = __float2half_rn(__fmul_rn(exp_canonical(__fsub_rn(mine[j], m)), inv));
  }
}

template <int D, bool kBlend, int RPW>
__global__ void __launch_bounds__(kWarps * 32) draft_kernel(const __half* q_pool,
                                                            const __half* k_pool,
                                                            const __half* q_max, const __half* k_max,
                                                            float w, int R, __half* prob) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr int kRows = kWarps * RPW;
  const int lg_stride = (R + 7) & ~7;
  float* kc = reinterpret_cast<float*>(smem_raw);                   // [kSlab][kPitch]
  float* qs = kc + kSlab * kPitch;                                      // [kWarps][D][2]
  __half* lg = reinterpret_cast<__half*>(qs + kRows * D);           // [kRows][lg_stride]
  __half* lgx = lg + kRows * lg_stride;                             // blend only
  const int head = blockIdx.y, row0 = blockIdx.x * kRows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  row_logits<D, RPW>(q_pool, k_pool, head, R, row0, kc, qs, lg, lg_stride);
  if (kBlend) {
    __syncthreads();
    row_logits<D, RPW>(q_max, k_max, head, R, row0, kc, qs, lgx, lg_stride);
  }
  for (int r = 0; r < RPW; ++r) {
    const int row = row0 + warp * RPW + r;
    if (row >= R) break;
    const __half* mine = lg + (warp * RPW + r) * lg_stride;
    float m, inv;
    row_stats(mine, R, m, inv);
    __half* out = prob + ((int64_t)head * R + row) * R;
    if (!kBlend) {
      for (int j = lane; j < R; j += 32)
        out[j] = __float2half_rn(__fmul_rn(exp_canonical(__fsub_rn(__half2float(mine[j]), m)), inv));
    } else {
      const __half* minex = lgx + (warp * RPW + r) * lg_stride;
      float mxx, invx;
      row_stats(minex, R, mxx, invx);
      const float wm = __fsub_rn(1.0f, w);
      for (int j = lane; j < R; j += 32) {
        const float pm = __fmul_rn(exp_canonical(__fsub_rn(__half2float(mine[j]), m)), inv);
        const float px = __fmul_rn(exp_canonical(__fsub_rn(__half2float(minex[j]), mxx)), invx);
        out[j] = __float2half_rn(__fadd_rn(__fmul_rn(wm, pm), __fmul_rn(w, px)));
      }
    }
  }
}

// Shared memory of one CTA: key tile, query rows, the logits of its rows (twice when blending).
template <int D, bool kBlend, int RPW>
constexpr size_t smem_bytes(int R) {
  return (size_t)kSlab * kPitch * 4 + (size_t)kWarps * RPW * D * 4 +
         (size_t)kWarps * RPW * ((R + 7) & ~7) * 2 * (kBlend ? 2 : 1);
}

template <int D, bool kBlend, int RPW>
int launch_rows(const __half* qp, const __half* kp, const __half* qx, const __half* kx, float w, int R,
                int H, __half* prob, cudaStream_t st) {
  const size_t smem = smem_bytes<D, kBlend, RPW>(R);
  auto kernel = draft_kernel<D, kBlend, RPW>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  constexpr int kRows = kWarps * RPW;
  dim3 grid((R + kRows - 1) / kRows, H);
  kernel<<<grid, kWarps * 32, smem, st>>>(qp, kp, qx, kx, w, R, prob);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

// Four rows per warp while two CTAs still fit an SM's shared memory, else two rows per warp.
template <int D, bool kBlend>
int launch(const __half* qp, const __half* kp, const __half* qx, const __half* kx, float w, int R,
           int H, __half* prob, cudaStream_t st) {
  if (smem_bytes<D, kBlend, 4>(R) <= 113 * 1024)
    return launch_rows<D, kBlend, 4>(qp, kp, qx, kx, w, R, H, prob, st);
  return launch_rows<D, kBlend, 2>(qp, kp, qx, kx, w, R, H, prob, st);
}

}  // namespace

extern "C" int anemoi_sm100_draft_probability(const anemoi_sm100_shape* shape, const void* q_pool,
                                              const void* k_pool, const void* q_max_pool,
                                              const void* k_max_pool, float maxpool_weight,
                                              void* probability, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !q_pool || !k_pool || !probability)
    return ANEMOI_SM100_EINVAL;
  if (!(maxpool_weight >= 0.0f && maxpool_weight <= 1.0f)) return ANEMOI_SM100_EINVAL;
  if (maxpool_weight != 0.0f && (!q_max_pool || !k_max_pool)) return ANEMOI_SM100_EINVAL;
  const int R = shape->video_blocks, H = shape->heads, D = shape->head_dim;
  if (R > kMaxBlocks || (maxpool_weight != 0.0f && maxpool_weight != 1.0f && R > 2400))
    return ANEMOI_SM100_ELIMIT;  // shared-memory row buffers
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* qp = static_cast<const __half*>(q_pool);
  const __half* kp = static_cast<const __half*>(k_pool);
  const __half* qx = static_cast<const __half*>(q_max_pool);
  const __half* kx = static_cast<const __half*>(k_max_pool);
  __half* prob = static_cast<__half*>(probability);
  if (maxpool_weight == 1.0f) {  // max pools only
    qp = qx;
    kp = kx;
    maxpool_weight = 0.0f;
  }
  const bool blend = maxpool_weight != 0.0f;
  if (D == 64)
    return blend ? launch<64, true>(qp, kp, qx, kx, maxpool_weight, R, H, prob, st)
                 : launch<64, false>(qp, kp, qx, kx, maxpool_weight, R, H, prob, st);
  return blend ? launch<128, true>(qp, kp, qx, kx, maxpool_weight, R, H, prob, st)
               : launch<128, false>(qp, kp, qx, kx, maxpool_weight, R, H, prob, st);
}

extern "C" int anemoi_sm100_draft_probability_jensen(const anemoi_sm100_shape* shape,
                                                     const void* q_pool, const void* k_pool,
                                                     const void* q_second, const void* k_second,
                                                     void* probability, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !q_pool || !k_pool || !q_second || !k_second ||
      !probability)
    return ANEMOI_SM100_EINVAL;
  const int R = shape->video_blocks, H = shape->heads, D = shape->head_dim;
  const size_t smem = (size_t)kSlab * kPitch * 4 + (size_t)kWarps * 2 * D * 4 +
                      (size_t)kWarps * 2 * ((R + 3) & ~3) * 4 * 2;
  if (smem > 227 * 1024) return ANEMOI_SM100_ELIMIT;  // two fp32 row buffers: R up to about 1,400
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((R + kWarps * 2 - 1) / (kWarps * 2), H);
  const __half* qp = static_cast<const __half*>(q_pool);
  const __half* kp = static_cast<const __half*>(k_pool);
  const __half* q2 = static_cast<const __half*>(q_second);
  const __half* k2 = static_cast<const __half*>(k_second);
  __half* prob = static_cast<__half*>(probability);
  if (D == 64) {
    if (cudaFuncSetAttribute(draft_jensen_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return ANEMOI_SM100_ELAUNCH;
    draft_jensen_kernel<64><<<grid, kWarps * 32, smem, st>>>(qp, kp, q2, k2, R, prob);
  } else {
    if (cudaFuncSetAttribute(draft_jensen_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return ANEMOI_SM100_ELAUNCH;
    draft_jensen_kernel<128><<<grid, kWarps * 32, smem, st>>>(qp, kp, q2, k2, R, prob);
  }
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}
