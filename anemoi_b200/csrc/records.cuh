// Byte layout of the operand records shared by the preparation kernels (writers)
// and the attention kernels (readers).
//
// A tile is stored as core matrices of 8 rows x 16 bytes (128 contiguous bytes):
//   K-major tile  [rows][row_bytes]:  offset(r, chunk j) = ((r/8)*chunks + j)*128 + (r%8)*16
// with chunks = row_bytes / 16.  The fp16 V tile (keys x channels, channels
// contiguous) uses the same formula and is consumed as an MN-major operand.
// Scale bytes of a block-scaled operand with up to 128 rows are stored per
// 64-element K step as 512 bytes: offset(row, group g) = (row%32)*16 + (row/32)*4 + g.
#pragma once

#include <stdint.h>

#include "../../include/anemoi_sm100.h"

namespace rec {

__host__ __device__ inline int prefix_stages(const anemoi_sm100_shape& s) {
  return (s.prefix_tokens + 63) / 64;
}
__host__ __device__ inline int stages(const anemoi_sm100_shape& s) {
  return prefix_stages(s) + s.video_blocks * (s.query_block / 64);
}
__host__ __device__ inline int prefix_query_tiles(const anemoi_sm100_shape& s) {
  return s.has_prefix_query_int8 ? (s.prefix_tokens + s.query_block - 1) / s.query_block : 0;
}

inline int validate_shape(const anemoi_sm100_shape* s) {
  if (s == nullptr) return ANEMOI_SM100_EINVAL;
  if (s->heads <= 0 || s->heads > 65535) return ANEMOI_SM100_EINVAL;
  if (s->head_dim != 64 && s->head_dim != 128) return ANEMOI_SM100_EINVAL;
  if (s->query_block != 64 && s->query_block != 128) return ANEMOI_SM100_EINVAL;
  if (s->video_blocks <= 0 || s->prefix_tokens < 0 || s->seq_tokens <= s->prefix_tokens)
    return ANEMOI_SM100_EINVAL;
  if (!(s->has_nvfp4 || s->has_int8 || s->has_fp16)) return ANEMOI_SM100_EINVAL;
  if (s->has_prefix_query_int8 && !s->has_int8) return ANEMOI_SM100_EINVAL;
  if (s->has_nvfp4 && !(s->q_global_scale > 0.f && s->k_global_scale > 0.f && s->v_global_scale > 0.f))
    return ANEMOI_SM100_EINVAL;
  return ANEMOI_SM100_OK;
}


// ---- record sizes (bytes) ---------------------------------------------------
__host__ __device__ inline int64_t q_fp16_bytes(int qb, int d) { return (int64_t)qb * d * 2; }
__host__ __device__ inline int64_t kv_fp16_bytes(int d) { return 2 * 64 * (int64_t)d * 2; }
__host__ __device__ inline int64_t q_int8_bytes(int qb, int d) { return (int64_t)qb * d; }
__host__ __device__ inline int64_t kv_int8_bytes(int d) { return 2 * 64 * (int64_t)d; }
// nvfp4 query record: codes (qb*d/2) then d/64 scale blocks of 512 bytes
__host__ __device__ inline int64_t q_nvfp4_bytes(int qb, int d) {
  return (int64_t)qb * d / 2 + (d / 64) * 512;
}
// nvfp4 key/value record: K codes (32*d) | V^T codes (32*d) | K scales (d/64*512) | V scales (512)
__host__ __device__ inline int64_t kv_nvfp4_bytes(int d) {
  return 64 * (int64_t)d + (d / 64) * 512 + 512;
}
__host__ __device__ inline int kv_nvfp4_v_offset(int d) { return 32 * d; }
__host__ __device__ inline int kv_nvfp4_ksf_offset(int d) { return 64 * d; }
__host__ __device__ inline int kv_nvfp4_vsf_offset(int d) { return 64 * d + (d / 64) * 512; }

// ---- offsets inside a tile --------------------------------------------------
__host__ __device__ inline int tile_offset(int row, int chunk, int chunks) {
  return (((row >> 3) * chunks + chunk) << 7) + ((row & 7) << 4);
}
__host__ __device__ inline int sf_offset(int row, int group) {
  return ((row & 31) << 4) + ((row >> 5) << 2) + group;
}

}  // namespace rec
