// Output assembly: inverse scatter of the packed video rows, prefix rows in front,
// cast to the caller's dtype, [1, S, H, D] contiguous.
//
// Reference: csrc/attention/cuda/sm89/output_assembly.cu:219-305 - video token s
// takes packed row inverse[s - prefix]; a query block whose three stage counts are
// all zero was never written by the attention kernel and yields +0; fp16 -> bf16
// goes through fp32 with round to nearest.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "records.cuh"

namespace {

template <typename OutT>
__device__ __forceinline__ uint4 convert8(uint4 raw);
template <>
__device__ __forceinline__ uint4 convert8<__half>(uint4 raw) { return raw; }
template <>
__device__ __forceinline__ uint4 convert8<__nv_bfloat16>(uint4 raw) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
  uint4 out;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __float22bfloat162_rn(__half22float2(h[i]));
  return out;
}

template <typename OutT, int D>
__global__ void __launch_bounds__(256) assemble_kernel(
    const void* prefix_out, int64_t prefix_rows, int prefix_is_caller_dtype, const __half* packed,
    const int32_t* inverse, const int32_t* row_counts, OutT* out, int S, int H, int prefix, int QB,
    int R) {
  constexpr int kVec = D / 8;
  const int64_t total = (int64_t)S * H * kVec;
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * 256) {
    const int c8 = (int)(idx % kVec);
    const int64_t sh = idx / kVec;
    const int h = (int)(sh % H);
    const int s = (int)(sh / H);
    uint4 val;
    if (s < prefix) {
      const int64_t off = ((int64_t)h * prefix_rows + s) * D + c8 * 8;
      if (prefix_is_caller_dtype) {
        val = __ldg(reinterpret_cast<const uint4*>(static_cast<const OutT*>(prefix_out) + off));
      } else {
        val = convert8<OutT>(
            __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(prefix_out) + off)));
      }
    } else {
      const int slot = inverse[s - prefix];
      const int32_t* rc = row_counts + ((int64_t)h * R + slot / QB) * 4;
      if (rc[0] + rc[1] + rc[2] == 0) {
        val = make_uint4(0, 0, 0, 0);
      } else {
        val = convert8<OutT>(__ldg(reinterpret_cast<const uint4*>(
            packed + ((int64_t)h * R * QB + slot) * D + c8 * 8)));
      }
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = val;
  }
}

template <typename OutT, int D>
int launch(const anemoi_sm100_shape& s, const void* prefix_out, int64_t prefix_rows, int caller,
           const void* packed, const int32_t* inverse, const int32_t* row_counts, void* out,
           cudaStream_t st) {
  const int64_t total = (int64_t)s.seq_tokens * s.heads * (D / 8);
  const int blocks = (int)min((total + 255) / 256, (int64_t)(148 * 16));
  assemble_kernel<OutT, D><<<blocks, 256, 0, st>>>(
      prefix_out, prefix_rows, caller, static_cast<const __half*>(packed), inverse, row_counts,
      static_cast<OutT*>(out), s.seq_tokens, s.heads, s.prefix_tokens, s.query_block,
      s.video_blocks);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

// ---- Ulysses relayouts: pure 16-byte copies --------------------------------------------
// q,k,v [rows][heads][D] (row / head strides in elements) -> send [ranks][rows][heads_local][3*D],
// where destination rank r receives its heads r*heads_per_rank + head_begin + (0..heads_local)
__global__ void __launch_bounds__(256) pack_qkv_kernel(const uint16_t* q, const uint16_t* k,
                                                       const uint16_t* v, uint16_t* send,
                                                       int64_t rows, int heads_local,
                                                       int heads_per_rank, int head_begin, int d8,
                                                       int64_t total, int64_t qs_row,
                                                       int64_t qs_head, int64_t ks_row,
                                                       int64_t ks_head, int64_t vs_row,
                                                       int64_t vs_head) {
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * 256) {
    const int c8 = (int)(idx % d8);
    int64_t t = idx / d8;
    const int which = (int)(t % 3);
    t /= 3;
    const int lh = (int)(t % heads_local);
    t /= heads_local;
    const int64_t row = t % rows;
    const int dest = (int)(t / rows);
    const int gh = dest * heads_per_rank + head_begin + lh;
    const uint16_t* src = which == 0 ? q + row * qs_row + gh * qs_head
                        : which == 1 ? k + row * ks_row + gh * ks_head
                                     : v + row * vs_row + gh * vs_head;
    *reinterpret_cast<uint4*>(send + idx * 8) = __ldg(reinterpret_cast<const uint4*>(src) + c8);
  }
}

// recv [ranks][rows][inner] -> out [rows][ranks][outer] at element offset `begin8` of every
// (row, rank) slot; inner = heads_local * D, outer = heads_per_rank * D (all in 16-byte units)
__global__ void __launch_bounds__(256) merge_heads_kernel(const uint16_t* recv, uint16_t* out,
                                                          int64_t rows, int ranks, int inner8,
                                                          int outer8, int begin8, int64_t total) {
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * 256) {
    const int tail = (int)(idx % inner8);
    const int64_t slot = idx / inner8;
    const int source = (int)(slot % ranks);
    const int64_t row = slot / ranks;
    *reinterpret_cast<uint4*>(out + (slot * outer8 + begin8 + tail) * 8) =
        __ldg(reinterpret_cast<const uint4*>(recv) + ((int64_t)source * rows + row) * inner8 + tail);
  }
}

}  // namespace

extern "C" int anemoi_sm100_assemble(const anemoi_sm100_shape* shape, const void* prefix_out,
                                     int64_t prefix_rows, int prefix_is_caller_dtype,
                                     const void* out_packed, const int32_t* inverse,
                                     const int32_t* row_counts, void* output, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !out_packed || !inverse || !row_counts ||
      !output)
    return ANEMOI_SM100_EINVAL;
  if (shape->prefix_tokens > 0 && (!prefix_out || prefix_rows < shape->prefix_tokens))
    return ANEMOI_SM100_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const anemoi_sm100_shape& s = *shape;
  if (s.input_is_bf16) {
    return s.head_dim == 64
               ? launch<__nv_bfloat16, 64>(s, prefix_out, prefix_rows, prefix_is_caller_dtype,
                                           out_packed, inverse, row_counts, output, st)
               : launch<__nv_bfloat16, 128>(s, prefix_out, prefix_rows, prefix_is_caller_dtype,
                                            out_packed, inverse, row_counts, output, st);
  }
  return s.head_dim == 64 ? launch<__half, 64>(s, prefix_out, prefix_rows, prefix_is_caller_dtype,
                                               out_packed, inverse, row_counts, output, st)
                          : launch<__half, 128>(s, prefix_out, prefix_rows, prefix_is_caller_dtype,
                                                out_packed, inverse, row_counts, output, st);
}

extern "C" int anemoi_sm100_pack_qkv_heads(const void* q, const void* k, const void* v, void* send,
                                           int64_t rows, int32_t heads, int32_t head_dim,
                                           int32_t ranks, int32_t head_begin, int32_t head_count,
                                           const int64_t* strides, void* stream) {
  if (!q || !k || !v || !send || !strides || rows < 0 || heads <= 0 || ranks <= 0 ||
      heads % ranks || head_dim % 8 || head_begin < 0 || head_count <= 0 ||
      head_begin + head_count > heads / ranks)
    return ANEMOI_SM100_EINVAL;
  for (int i = 0; i < 6; ++i)
    if (strides[i] % 8) return ANEMOI_SM100_EINVAL;
  const int64_t total = rows * ranks * head_count * 3 * (head_dim / 8);
  if (total == 0) return ANEMOI_SM100_OK;
  const int blocks = (int)min((total + 255) / 256, (int64_t)(148 * 16));
  pack_qkv_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(k),
      static_cast<const uint16_t*>(v), static_cast<uint16_t*>(send), rows, head_count,
      heads / ranks, head_begin, head_dim / 8, total, strides[0], strides[1], strides[2],
      strides[3], strides[4], strides[5]);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_pack_qkv(const void* q, const void* k, const void* v, void* send,
                                     int64_t rows, int32_t heads, int32_t head_dim, int32_t ranks,
                                     const int64_t* strides, void* stream) {
  if (ranks <= 0 || heads <= 0 || heads % ranks) return ANEMOI_SM100_EINVAL;
  return anemoi_sm100_pack_qkv_heads(q, k, v, send, rows, heads, head_dim, ranks, 0, heads / ranks,
                                     strides, stream);
}

extern "C" int anemoi_sm100_merge_heads_into(const void* recv, void* out, int64_t rows,
                                             int32_t ranks, int32_t head_count, int32_t head_dim,
                                             int32_t heads_per_rank, int32_t head_begin,
                                             void* stream) {
  if (!recv || !out || rows < 0 || ranks <= 0 || head_count <= 0 || head_dim % 8 ||
      head_begin < 0 || head_begin + head_count > heads_per_rank)
    return ANEMOI_SM100_EINVAL;
  const int inner8 = head_count * head_dim / 8;
  const int64_t total = rows * ranks * inner8;
  if (total == 0) return ANEMOI_SM100_OK;
  const int blocks = (int)min((total + 255) / 256, (int64_t)(148 * 16));
  merge_heads_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(recv), static_cast<uint16_t*>(out), rows, ranks, inner8,
      heads_per_rank * head_dim / 8, head_begin * head_dim / 8, total);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_merge_heads(const void* recv, void* out, int64_t rows, int32_t ranks,
                                        int32_t heads_per_rank, int32_t head_dim, void* stream) {
  return anemoi_sm100_merge_heads_into(recv, out, rows, ranks, heads_per_rank, head_dim,
                                       heads_per_rank, 0, stream);
}

// One strided copy between pinned host memory and the device: `height` rows of `width` bytes,
// rows `src_pitch` / `dst_pitch` bytes apart (cudaMemcpy2DAsync).  With it a group of heads of
// a host tensor [1, S, H, D] moves to or from a contiguous device tensor [1, S, heads, D] in one
// call, so that the copies of one head group can run under the attention of another.
extern "C" int anemoi_sm100_copy_rows(void* dst, int64_t dst_pitch, const void* src,
                                      int64_t src_pitch, int64_t width, int64_t height,
                                      int32_t to_device, void* stream) {
  if (!dst || !src || width <= 0 || height <= 0 || dst_pitch < width || src_pitch < width)
    return ANEMOI_SM100_EINVAL;
  const cudaError_t err = cudaMemcpy2DAsync(
      dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width, (size_t)height,
      to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  return err == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}
