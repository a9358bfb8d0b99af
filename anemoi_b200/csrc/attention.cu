// Block-sparse mixed-precision flash attention for sm_100a.
//
// One CTA owns one query tile (QB rows of one head, padded to the 128-row MMA
// shape) and walks that tile's ragged list of 64-key stages in the order
// NVFP4 -> INT8 -> FP16 with one online-softmax state.
//
// Warp roles (256 threads = two warpgroups; the second one gives most of its registers to the
// first with setmaxnreg, so a softmax thread may use 192 registers at two CTAs per SM):
//   warps 0-3  softmax: warp w owns TMEM lanes 32*w.. (query rows); one thread per row holds
//              the row's 64 scores of a stage in registers (few threads with long unrolled
//              instruction streams: the per-stage fixed cost is paid once per row)
//   warp 4     loader: one lane issues 1-D bulk copies (TMA engine) of the Q record of
//              each phase and of one K|V record per stage into a ring of shared-memory
//              slots, completion counted on mbarriers
//   warp 5     MMA: allocates TMEM; one lane issues tcgen05.mma
//                S[128x64]  = Q K^T   kind::mxf4nvf4 / kind::i8 / kind::f16
//                O[128xD]  += P V     kind::mxf4nvf4 / kind::f8f6f4 / kind::f16
//              and tcgen05.commit to mbarriers
//   warps 6-7  idle (they complete the second warpgroup)
// TMEM columns: S0 [0,64), O [64,64+D), and [192,256) holds the NVFP4 scale factors in the
// NVFP4 phase and a second score buffer S1 in the INT8 / FP16 phases (QK of stage g+1 runs
// while the softmax threads still read the scores of stage g).
// O stays in TMEM across all stages; it is rescaled (read-modify-write by the
// softmax threads) only when some row's running maximum moved, and at a phase
// change, where it is also converted between the phases' value domains.  P is
// double-buffered in shared memory for the 4- and 8-bit cells, so the softmax
// threads only wait for the previous PV when they have to rescale O.
//
// Numerics follow the reference's phases
// (csrc/attention/cuda/sm120/q64_attention_phase_composer.inl:1-146, 506-932,
// 934-1331; primitives/qattn/attn_utils.cuh:363-389, 470-625):
//   base-2 online softmax, sigma = log2(e)/sqrt(D), m0 = -5e6, keys >= valid_k masked,
//   denominator accumulated from the unquantised P,
//   NVFP4: score scale sigma*q_gs*k_gs, P -> e2m1(6P) with a constant 448 block scale,
//          O_true = O * v_gs/(6*448)
//   INT8 : exact s32 scores, scale sigma*q_scale*k_scale[stage], P -> e4m3(P*2^8.807),
//          O_true[c] = O[c] * v_scale[c] * 2^-8.807
//   FP16 : P -> f16
// Accumulation is fp32 in TMEM (the reference accumulates a stage in fp16 for the
// INT8 and FP16 cells).
#include <climits>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "bounded_wait.cuh"
#include "records.cuh"
#include "sm100_primitives.cuh"

namespace {

using namespace sm100;

constexpr int kThreads = 256;         // two warpgroups: softmax | loader, MMA and two idle warps
constexpr int kSoftmaxRegs = 192;     // 128 * 192 + 128 * 64 == 256 * 128 (two CTAs per SM)
constexpr int kOtherRegs = 64;
constexpr int kSoftmaxThreads = 128;
constexpr int kLoaderWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kTmemCols = 256;
constexpr int kColS = 0;
constexpr int kColS1 = 192;  // second score buffer; aliases the scale-factor columns
constexpr int kColO = 64;
constexpr int kColSfaQ = 192;  // 2 k-steps x 4 columns
constexpr int kColSfbK = 200;  // 2 k-steps x 4 columns
constexpr int kColSfaP = 208;
constexpr int kColSfbV = 212;
constexpr int kMaxSlots = 8;
constexpr float kFp8Offset = 8.807f;

enum Cell : int { kNv = 0, kI8 = 1, kF16 = 2 };

struct AttnParams {
  anemoi_sm100_shape s;
  anemoi_sm100_operands o;
  const int32_t* row_offset;
  const int32_t* row_counts;
  const int32_t* stage_ids;
  int64_t capacity;
  const int32_t* valid_k;
  // Q64 pairs: query blocks 2t and 2t+1 of a head share one CTA (rows 0-63 and 64-127 of the
  // 128-row MMA shape) and walk the union of their lists; bits 30 / 31 of a list entry say which
  // of the two blocks the stage belongs to.  Null: one query block per CTA.
  const int32_t* pair_counts;  // [H][ceil(R/2)][4]
  const int32_t* pair_ids;     // [H][capacity], a pair's list starts at row_offset of block 2t
  __half* out;       // [H][tiles*QB][D]
  int32_t* status;
  uint64_t wait_ns;  // limit of every mbarrier wait
  int dense_prefix;  // 1: prefix query tiles, INT8 cell over every stage
  int stages;        // 64-key stages per head
  int q_tiles_int8;  // records per head in q_int8 (R + prefix query tiles)
  int out_rows;      // rows per head in `out`
  int ring_bytes;    // key/value ring; re-partitioned into equal slots at every phase
  int q_region;      // bytes
  int p_region;      // bytes
};

struct Barriers {
  uint64_t kv_full[kMaxSlots];
  uint64_t kv_free[kMaxSlots];
  uint64_t q_full, q_free;
  uint64_t s_full[2];  // scores ready, per score buffer
  uint64_t s_free;     // scores read by the softmax warps (NVFP4 phase: single buffer)
  uint64_t all_done;  // every MMA of the tile complete (epilogue)
  // Two P barriers used alternately: a warp that skips the wait for the previous PV may run one stage
  // ahead, and its arrival must not be counted into the previous stage's phase.
  uint64_t p_full[2];
  WaitContext wc;
  uint32_t tmem_base;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Packed two-wide fp32 arithmetic (one instruction for two elements).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(v),
               "r"(v), "r"(v), "r"(v)
               : "memory");
}

template <int D>
struct CellInfo {
  // bytes per stage record and per Q record, chunk counts (16-byte chunks per row)
  __device__ static int kv_bytes(int cell) {
    return cell == kNv ? (int)rec::kv_nvfp4_bytes(D)
                       : (cell == kI8 ? (int)rec::kv_int8_bytes(D) : (int)rec::kv_fp16_bytes(D));
  }
  __device__ static int q_bytes(int cell, int qb) {
    return cell == kNv ? (int)rec::q_nvfp4_bytes(qb, D)
                       : (cell == kI8 ? (int)rec::q_int8_bytes(qb, D) : (int)rec::q_fp16_bytes(qb, D));
  }
};

// ------------------------------------------------------------------------------------------
// softmax side
// ------------------------------------------------------------------------------------------
struct RowState {
  float m, d;
};

// O[row][c] *= alpha (* colf[c] when kColf) for all D columns of the thread's row, 64 columns
// (two TMEM loads in flight) per step.
template <int D, bool kColf>
__device__ __forceinline__ void rescale_o(uint32_t tmem_row, float alpha, const float* colf) {
  const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll 1
  for (int c0 = 0; c0 < D; c0 += 64) {
    uint32_t r[64];
    tmem_ld32(tmem_row + kColO + c0, *reinterpret_cast<uint32_t(*)[32]>(r));
    tmem_ld32(tmem_row + kColO + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
    tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 64; j += 2) {
      float2 v = fmul2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), alpha2);
      if (kColf) v = fmul2(v, *reinterpret_cast<const float2*>(colf + c0 + j));
      r[j] = __float_as_uint(v.x);
      r[j + 1] = __float_as_uint(v.y);
    }
    tmem_st32(tmem_row + kColO + c0, *reinterpret_cast<uint32_t(*)[32]>(r));
    tmem_st32(tmem_row + kColO + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
  }
  tmem_wait_st();
}

// Writes the thread's 64 probabilities (one query row of the stage) into the K-major P tile
// in shared memory.
template <int CELL>
__device__ __forceinline__ void write_p(uint8_t* p_tile, int row, const float (&p)[64]) {
  if (CELL == kF16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 v;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(p[j * 8 + 2 * i], p[j * 8 + 2 * i + 1]);
      *reinterpret_cast<uint4*>(p_tile + rec::tile_offset(row, j, 8)) = v;
    }
  } else if (CELL == kI8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 v;
      uint16_t* h = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        h[i] = __nv_cvt_float2_to_fp8x2(make_float2(p[j * 16 + 2 * i], p[j * 16 + 2 * i + 1]),
                                        __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint4*>(p_tile + rec::tile_offset(row, j, 4)) = v;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint4 v;
      uint8_t* h = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        h[i] = __nv_cvt_float2_to_fp4x2(make_float2(p[j * 32 + 2 * i], p[j * 32 + 2 * i + 1]),
                                        __NV_E2M1, cudaRoundNearest);  // p already holds 6 P
      *reinterpret_cast<uint4*>(p_tile + rec::tile_offset(row, j, 2)) = v;
    }
  }
}

// A row of zeros in the P tile (a stage that does not belong to this row's query block).
__device__ __forceinline__ void write_zero_p(uint8_t* p_tile, int row, int cell) {
  const int chunks = cell == kF16 ? 8 : (cell == kI8 ? 4 : 2);
  for (int j = 0; j < chunks; ++j)
    *reinterpret_cast<uint4*>(p_tile + rec::tile_offset(row, j, chunks)) = make_uint4(0, 0, 0, 0);
}

// Bytes of one P tile (128 rows x 64 keys) per cell, and which of the two buffers stage g uses.
__device__ __forceinline__ int p_tile_bytes(int cell) {
  return cell == kNv ? 128 * 32 : (cell == kI8 ? 128 * 64 : 128 * 128);
}
__device__ __forceinline__ int p_buffer(int cell, int g) { return cell == kF16 ? 0 : (g & 1); }
// Score buffer of stage g: the NVFP4 phase has a single one (the other holds its scale factors).
__device__ __forceinline__ int s_buffer(int cell, int g) { return cell == kNv ? 0 : (g & 1); }
__device__ __forceinline__ uint32_t s_column(int sb) { return sb ? kColS1 : kColS; }

// One stage of one phase for the thread's row.  A single copy of this code serves the three
// cells (the cell is a run-time value): the kernel's hot code has to stay well inside the
// instruction cache, and three unrolled copies did not.
template <int D>
__device__ __forceinline__ void softmax_stage(Barriers* b, const AttnParams& p, uint8_t* p_smem,
                                              const float* colf, uint32_t tmem_row, int row,
                                              int cell, int g, bool phase_first,
                                              float score_scale, int valid, bool live_warp,
                                              bool member, int sb, uint32_t s_parity,
                                              uint64_t* prev_pv_bar, uint32_t prev_pv_parity,
                                              RowState& st) {
  wait(&b->wc, &b->s_full[sb], s_parity, 10 + cell);
  tc_fence_after_sync();
  // Barrier arrivals are one per warp (lane 0 after a warp sync).
  const bool lead = (row & 31) == 0;
  if (!live_warp) {
    // padding rows of a 64-row tile: keep the barrier protocol, skip the math
    if (lead) {
      if (cell == kNv) mbar_arrive(&b->s_free);
      mbar_arrive(&b->p_full[g & 1]);
    }
    return;
  }
  if (!member) {
    // A stage of the other query block of the pair (warp-uniform: a warp's rows belong to one
    // block).  These rows contribute nothing: P = 0, running maximum and denominator untouched.
    // O still has to change its value domain at the first stage of a phase.
    if (cell == kNv) {
      __syncwarp();
      if (lead) mbar_arrive(&b->s_free);
    }
    if (g > 0 && (phase_first || cell == kF16)) {
      wait(&b->wc, prev_pv_bar, prev_pv_parity, 20 + cell);
      tc_fence_after_sync();
      if (phase_first) rescale_o<D, true>(tmem_row, 1.0f, colf);
    }
    write_zero_p(p_smem + p_buffer(cell, g) * p_tile_bytes(cell), row, cell);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncwarp();
    if (lead) mbar_arrive(&b->p_full[g & 1]);
    return;
  }
  float s[64];
  {
    uint32_t r[64];
    tmem_ld32(tmem_row + s_column(sb), *reinterpret_cast<uint32_t(*)[32]>(r));
    tmem_ld32(tmem_row + s_column(sb) + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
    tmem_wait_ld();
    if (cell == kNv) {
      // Only the NVFP4 phase has a single score buffer, whose release the MMA warp must see
      // before the next QK.  With two buffers, QK of stage g+2 is issued after the MMA warp has
      // waited for P of stage g, which every softmax thread writes after this load.
      tc_fence_before_sync();
      __syncwarp();
      if (lead) mbar_arrive(&b->s_free);
    }
    if (cell == kI8) {
      // Scores are s32; as_float(i + 0x4B400000) == 12582912 + i exactly for |i| < 2^22, so
      // the conversion is an integer add and a float subtract (no conversion instruction).
      const float2 magic2 = make_float2(-12582912.0f, -12582912.0f);
#pragma unroll
      for (int j = 0; j < 64; j += 2) {
        const float2 v = fadd2(make_float2(__int_as_float((int)r[j] + 0x4B400000),
                                           __int_as_float((int)r[j + 1] + 0x4B400000)),
                               magic2);
        s[j] = v.x;
        s[j + 1] = v.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) s[j] = __uint_as_float(r[j]);
    }
  }
  if (valid < 64) {
    // ragged blocks usually lose only a few keys: the common case touches the last 8 columns
    if (valid >= 56) {
#pragma unroll
      for (int j = 56; j < 64; ++j) s[j] = j < valid ? s[j] : -INFINITY;
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) s[j] = j < valid ? s[j] : -INFINITY;
    }
  }
  float mx;
  {
    float m0 = max3(s[0], s[1], s[2]), m1 = max3(s[3], s[4], s[5]);
    float m2 = max3(s[6], s[7], s[8]), m3 = max3(s[9], s[10], s[11]);
#pragma unroll
    for (int j = 12; j < 60; j += 8) {
      m0 = max3(m0, s[j], s[j + 1]);
      m1 = max3(m1, s[j + 2], s[j + 3]);
      m2 = max3(m2, s[j + 4], s[j + 5]);
      m3 = max3(m3, s[j + 6], s[j + 7]);
    }
    m0 = max3(m0, s[60], s[61]);
    m1 = max3(m1, s[62], s[63]);
    mx = fmaxf(max3(m0, m1, m2), m3);
  }

  const float m_new = fmaxf(st.m, mx * score_scale);
  const float alpha = ex2(st.m - m_new);
  // exponent = s * scale + bias; the NVFP4 cell produces 6 P directly (e2m1 input range),
  // the INT8 cell P * 2^8.807 (e4m3 input range); the sums are scaled back.
  const float bias = cell == kI8 ? kFp8Offset - m_new
                                 : (cell == kNv ? 2.5849625007f - m_new : -m_new);
  const float sum_scale = cell == kI8 ? 0.0022326917f : (cell == kNv ? 0.16666667f : 1.0f);
  const float2 scale2 = make_float2(score_scale, score_scale);
  const float2 bias2 = make_float2(bias, bias);
  float2 acc0 = make_float2(0.0f, 0.0f), acc1 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int j = 0; j < 64; j += 4) {
    const float2 a0 = ffma2(make_float2(s[j], s[j + 1]), scale2, bias2);
    const float2 a1 = ffma2(make_float2(s[j + 2], s[j + 3]), scale2, bias2);
    const float e0 = ex2(a0.x), e1 = ex2(a0.y), e2 = ex2(a1.x), e3 = ex2(a1.y);
    s[j] = e0;
    s[j + 1] = e1;
    s[j + 2] = e2;
    s[j + 3] = e3;
    acc0 = fadd2(acc0, make_float2(e0, e1));
    acc1 = fadd2(acc1, make_float2(e2, e3));
  }
  const float sum = ((acc0.x + acc0.y) + (acc1.x + acc1.y)) * sum_scale;
  st.d = st.d * alpha + sum;
  st.m = m_new;

  if (g > 0) {
    const bool need = phase_first || __any_sync(0xffffffffu, alpha != 1.0f);
    // O may only be touched once the previous PV is complete.  The single FP16 P
    // buffer also needs that; the double-buffered 4/8-bit P tiles are free as soon as
    // this stage's scores arrived (QK of stage g is issued after PV of stage g-2).
    if (need || cell == kF16) {
      // the previous stage's PV signals the release of its key/value slot
      wait(&b->wc, prev_pv_bar, prev_pv_parity, 20 + cell);
      tc_fence_after_sync();
    }
    if (need) {
      if (phase_first) {
        rescale_o<D, true>(tmem_row, alpha, colf);
      } else {
        rescale_o<D, false>(tmem_row, alpha, nullptr);
      }
    }
  }
  uint8_t* p_tile = p_smem + p_buffer(cell, g) * p_tile_bytes(cell);
  if (cell == kNv) {
    write_p<kNv>(p_tile, row, s);
  } else if (cell == kI8) {
    write_p<kI8>(p_tile, row, s);
  } else {
    write_p<kF16>(p_tile, row, s);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncwarp();
  if (lead) mbar_arrive(&b->p_full[g & 1]);
}

// ------------------------------------------------------------------------------------------
// MMA side
// ------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void issue_qk(int cell, uint32_t tmem_s, uint32_t tmem, uint32_t q_addr,
                                         uint32_t k_addr, uint32_t kv_slot_addr, uint32_t issue) {
  if (cell == kF16) {
    constexpr uint32_t chunks = D / 8;
    const uint32_t idesc = instr_desc(kFmtF16, kFmtF16, kAccF32, 128, 64, 0, 0);
#pragma unroll
    for (int k = 0; k < D / 16; ++k)
      mma_f16_ss(tmem_s, smem_desc(q_addr + k * 256, 128, chunks * 128),
                 smem_desc(k_addr + k * 256, 128, chunks * 128), idesc, k > 0, issue);
  } else if (cell == kI8) {
    constexpr uint32_t chunks = D / 16;
    const uint32_t idesc = instr_desc(kFmtS8, kFmtS8, kAccS32, 128, 64, 0, 0);
#pragma unroll
    for (int k = 0; k < D / 32; ++k)
      mma_i8_ss(tmem_s, smem_desc(q_addr + k * 256, 128, chunks * 128),
                smem_desc(k_addr + k * 256, 128, chunks * 128), idesc, k > 0, issue);
  } else {
    constexpr uint32_t chunks = D / 32;
    const uint32_t idesc = instr_desc_nvf4(128, 64);
    const uint32_t ksf = kv_slot_addr + rec::kv_nvfp4_ksf_offset(D);
#pragma unroll
    for (int k = 0; k < D / 64; ++k)
      tmem_cp_32x128b_warpx4(tmem + kColSfbK + 4 * k, smem_desc(ksf + 512 * k, 128, 128), issue);
#pragma unroll
    for (int k = 0; k < D / 64; ++k)
      mma_nvf4_ss(tmem_s, smem_desc(q_addr + k * 256, 128, chunks * 128),
                  smem_desc(k_addr + k * 256, 128, chunks * 128), idesc, k > 0,
                  tmem + kColSfaQ + 4 * k, tmem + kColSfbK + 4 * k, issue);
  }
}

template <int D>
__device__ __forceinline__ void issue_pv(int cell, uint32_t tmem, uint32_t p_addr,
                                         uint32_t kv_slot_addr, uint32_t accumulate,
                                         uint32_t issue) {
  if (cell == kF16) {
    const uint32_t v_addr = kv_slot_addr + 64 * D * 2;
    const uint32_t idesc = instr_desc(kFmtF16, kFmtF16, kAccF32, 128, D, 0, 1);
    constexpr uint32_t v_lbo = (D / 8) * 128;  // between 8-key groups
#pragma unroll
    for (int k = 0; k < 4; ++k)
      mma_f16_ss(tmem + kColO, smem_desc(p_addr + k * 256, 128, 8 * 128),
                 smem_desc(v_addr + k * 2 * v_lbo, v_lbo, 128), idesc, accumulate | (k > 0), issue);
  } else if (cell == kI8) {
    const uint32_t v_addr = kv_slot_addr + 64 * D;
    const uint32_t idesc = instr_desc(kFmtE4M3, kFmtE4M3, kAccF32, 128, D, 0, 0);
#pragma unroll
    for (int k = 0; k < 2; ++k)
      mma_f8_ss(tmem + kColO, smem_desc(p_addr + k * 256, 128, 4 * 128),
                smem_desc(v_addr + k * 256, 128, 4 * 128), idesc, accumulate | (k > 0), issue);
  } else {
    const uint32_t v_addr = kv_slot_addr + rec::kv_nvfp4_v_offset(D);
    const uint32_t vsf = kv_slot_addr + rec::kv_nvfp4_vsf_offset(D);
    const uint32_t idesc = instr_desc_nvf4(128, D);
    tmem_cp_32x128b_warpx4(tmem + kColSfbV, smem_desc(vsf, 128, 128), issue);
    mma_nvf4_ss(tmem + kColO, smem_desc(p_addr, 128, 2 * 128), smem_desc(v_addr, 128, 2 * 128),
                idesc, accumulate, tmem + kColSfaP, tmem + kColSfbV, issue);
  }
}

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads, 2) attention_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int QB = p.s.query_block;
  const int head = blockIdx.y;
  // launch order of the head's query blocks (longest list first) as written by the routing
  // stage; 0 = no order given
  int tile = blockIdx.x;
  const bool pairs = p.pair_counts != nullptr;
  const int pair_tiles = (p.s.video_blocks + 1) / 2;
  if (!p.dense_prefix) {
    const int ordered =
        pairs ? p.pair_counts[((int64_t)head * pair_tiles + blockIdx.x) * 4 + 3]
              : p.row_counts[((int64_t)head * p.s.video_blocks + blockIdx.x) * 4 + 3];
    if (ordered > 0) tile = ordered - 1;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // query blocks of this CTA (two for a complete pair) and the first one's index
  const int tile_blocks = pairs && 2 * tile + 1 < p.s.video_blocks ? 2 : 1;
  const int block0 = pairs ? 2 * tile : tile;

  // ---- this tile's work list ----
  int cnt[3];
  int first_of[3] = {0, 0, 0};  // where each phase starts inside the list
  const int32_t* list;
  if (p.dense_prefix) {
    cnt[0] = 0;
    cnt[1] = p.stages;
    cnt[2] = 0;
    list = nullptr;
  } else if (pairs) {
    const int32_t* pc = p.pair_counts + ((int64_t)head * pair_tiles + tile) * 4;
    cnt[0] = pc[0];
    cnt[1] = pc[1];
    cnt[2] = pc[2];
    // phase c of the union sits where the two blocks' phases before it would end
    const int32_t* ra = p.row_counts + ((int64_t)head * p.s.video_blocks + block0) * 4;
    int before = 0;
    for (int c = 0; c < 3; ++c) {
      first_of[c] = before;
      before += ra[c] + (tile_blocks == 2 ? ra[4 + c] : 0);
    }
    list = p.pair_ids + (int64_t)head * p.capacity +
           p.row_offset[(int64_t)head * p.s.video_blocks + block0];
  } else {
    const int32_t* rc = p.row_counts + ((int64_t)head * p.s.video_blocks + tile) * 4;
    cnt[0] = rc[0];
    cnt[1] = rc[1];
    cnt[2] = rc[2];
    list = p.stage_ids + (int64_t)head * p.capacity +
           p.row_offset[(int64_t)head * p.s.video_blocks + tile];
    first_of[1] = cnt[0];
    first_of[2] = cnt[0] + cnt[1];
  }
  const int total = cnt[0] + cnt[1] + cnt[2];
  if (total == 0) return;
  // After a give-up anywhere on this device the status word stays set: later CTAs (of this and
  // of later launches, until the host clears the word) return at once instead of each running
  // into its own wait limit.
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;

  uint8_t* q_smem = smem;
  uint8_t* p_smem = smem + p.q_region;
  uint8_t* slots = p_smem + p.p_region;
  float* colf = reinterpret_cast<float*>(slots + (size_t)p.ring_bytes);
  Barriers* b = reinterpret_cast<Barriers*>(colf + D);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxSlots; ++i) {
      mbar_init(&b->kv_full[i], 1);
      mbar_init(&b->kv_free[i], 1);
    }
    mbar_init(&b->q_full, 1);
    mbar_init(&b->q_free, 1);
    mbar_init(&b->s_full[0], 1);
    mbar_init(&b->s_full[1], 1);
    mbar_init(&b->s_free, kSoftmaxThreads / 32);
    mbar_init(&b->p_full[0], kSoftmaxThreads / 32);
    mbar_init(&b->p_full[1], kSoftmaxThreads / 32);
    mbar_init(&b->all_done, 1);
    b->wc.abort = 0;
    b->wc.status = p.status;
    b->wc.limit_ns = p.wait_ns;
    mbar_init_fence();
  }
  // Query rows beyond QB (64-row tiles padded to the 128-row MMA shape) are never
  // initialised: rows are independent, their results stay in TMEM lanes nobody reads.
  if (warp == kMmaWarp) {
    tmem_alloc(&b->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = b->tmem_base;

  const int q_index_fp = head * p.s.video_blocks + block0;  // q_fp16 / q_nvfp4 record
  const int64_t q_index_i8 =
      (int64_t)head * p.q_tiles_int8 + (p.dense_prefix ? p.s.video_blocks + tile : block0);
  const float sigma = (D == 64 ? 0.125f : 0.08838834764831845f) * 1.4426950408889634f;

  // The second warpgroup (loader, MMA and two idle warps) hands most of its registers to the
  // softmax warpgroup.  All four warps of a warpgroup execute the same setmaxnreg instruction,
  // and each sits at the top of the branch whose code runs under the new register count.
  if (warp >= kLoaderWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
  if (warp == kLoaderWarp) {
    // =============================== loader ===============================
    // The whole warp walks the list with uniform control flow; one lane issues.
    const uint32_t lead = lane == 0;
    int phase_ord = 0;
    uint32_t filled = 0, fillpar = 0;  // per slot: ever filled / parity of the fill count
    for (int cell = 0; cell < 3; ++cell) {
      if (cnt[cell] == 0) continue;
      if (phase_ord > 0) wait<kPark>(&b->wc, &b->q_free, (phase_ord - 1) & 1, 1);
      const int qbytes = CellInfo<D>::q_bytes(cell, QB);
      const uint8_t* qsrc =
          cell == kNv ? static_cast<const uint8_t*>(p.o.q_nvfp4) + (int64_t)q_index_fp * qbytes
          : cell == kI8 ? static_cast<const uint8_t*>(p.o.q_int8) + q_index_i8 * qbytes
                        : static_cast<const uint8_t*>(p.o.q_fp16) + (int64_t)q_index_fp * qbytes;
      mbar_arrive_expect_tx(&b->q_full, qbytes * tile_blocks, lead);
      if (cell == kNv && QB == 64) {
        // codes fill the first half of the 128-row tile; scale blocks follow the full tile.
        // A pair's second record: codes into the second half of the tile, scale blocks behind
        // the first record's (the MMA warp folds them into one block before it copies them).
        const int codes = QB * D / 2;
        bulk_g2s(q_smem, qsrc, codes, &b->q_full, lead);
        bulk_g2s(q_smem + 128 * D / 2, qsrc + codes, qbytes - codes, &b->q_full, lead);
        if (tile_blocks == 2) {
          bulk_g2s(q_smem + codes, qsrc + qbytes, codes, &b->q_full, lead);
          bulk_g2s(q_smem + 128 * D / 2 + (qbytes - codes), qsrc + qbytes + codes, qbytes - codes,
                   &b->q_full, lead);
        }
      } else {
        // records of consecutive query blocks follow one another: two make a 128-row tile
        bulk_g2s(q_smem, qsrc, qbytes * tile_blocks, &b->q_full, lead);
      }
      const int kvbytes = CellInfo<D>::kv_bytes(cell);
      const uint8_t* kvbase =
          (cell == kNv ? static_cast<const uint8_t*>(p.o.kv_nvfp4)
           : cell == kI8 ? static_cast<const uint8_t*>(p.o.kv_int8)
                         : static_cast<const uint8_t*>(p.o.kv_fp16)) +
          (int64_t)head * p.stages * kvbytes;
      const int first = first_of[cell];
      // The ring is cut into equal slots of this phase's record size; slots of the
      // previous phase must all be released before the new geometry is written.
      const int slot_bytes = (kvbytes + 127) & ~127;
      const int nslot = min(kMaxSlots, p.ring_bytes / slot_bytes);
      for (int sl = 0; sl < kMaxSlots; ++sl)
        if ((filled >> sl) & 1u)
          wait<kPark>(&b->wc, &b->kv_free[sl], ((fillpar >> sl) & 1u) ^ 1u, 2);
      int stage_l = 0;  // list entries, 32 at a time, one per lane
      int slot = -1;
      for (int i = 0; i < cnt[cell]; ++i) {
        if ((i & 31) == 0 && list != nullptr && i + lane < cnt[cell])
          stage_l = list[first + i + lane];
        const int stage = list ? (__shfl_sync(0xffffffffu, stage_l, i & 31) & 0x3fffffff) : i;
        slot = slot + 1 == nslot ? 0 : slot + 1;
        if ((filled >> slot) & 1u)
          wait<kPark>(&b->wc, &b->kv_free[slot], ((fillpar >> slot) & 1u) ^ 1u, 2);
        mbar_arrive_expect_tx(&b->kv_full[slot], kvbytes, lead);
        bulk_g2s(slots + (size_t)slot * slot_bytes, kvbase + (int64_t)stage * kvbytes, kvbytes,
                 &b->kv_full[slot], lead);
        filled |= 1u << slot;
        fillpar ^= 1u << slot;
      }
      ++phase_ord;
    }
  } else if (warp == kMmaWarp) {
    // =============================== MMA issue ===============================
    // Uniform control flow for the whole warp (descriptors stay warp-uniform values);
    // only the tcgen05 instructions themselves are predicated on one lane.
    const uint32_t lead = lane == 0;
    int g = 0, phase_ord = 0;
    uint32_t usepar = 0;  // per slot: parity of the number of fills consumed
    const uint32_t q_addr = smem_u32(q_smem), p_addr = smem_u32(p_smem);
    for (int cell = 0; cell < 3; ++cell) {
      if (cnt[cell] == 0) continue;
      wait<kPark>(&b->wc, &b->q_full, phase_ord & 1, 3);
      tc_fence_after_sync();
      if (cell == kNv) {
        if (tile_blocks == 2) {
          // Scale bytes of rows 0-63 sit in the low eight bytes of every 16-byte chunk, those of
          // rows 64-127 in the high eight.  Both records hold their 64 rows in the low halves:
          // the second record's move up into the first record's empty high halves.
          uint8_t* sfa = q_smem + 128 * D / 2;
          const uint8_t* sfb = sfa + (D / 64) * 512;
          for (int c = lane; c < (D / 64) * 32; c += 32) {
            const uint2 lo = *reinterpret_cast<const uint2*>(sfb + c * 16);
            *reinterpret_cast<uint2*>(sfa + c * 16 + 8) = lo;
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        const uint32_t qsf = q_addr + 128 * D / 2;
#pragma unroll
        for (int k = 0; k < D / 64; ++k)
          tmem_cp_32x128b_warpx4(tmem + kColSfaQ + 4 * k, smem_desc(qsf + 512 * k, 128, 128),
                                 lead);
      }
      const int n = cnt[cell];
      const int slot_bytes = (CellInfo<D>::kv_bytes(cell) + 127) & ~127;
      const int nslot = min(kMaxSlots, p.ring_bytes / slot_bytes);
      const uint32_t ring_addr = smem_u32(slots);
      // software pipeline: QK of stage i+1 is issued before PV of stage i
      int qk_slot = 0, pv_slot = 0;
      for (int i = 0; i <= n; ++i) {
        if (i < n) {
          const int gi = g + i;
          const int slot = qk_slot;
          qk_slot = qk_slot + 1 == nslot ? 0 : qk_slot + 1;
          wait<kPark>(&b->wc, &b->kv_full[slot], (usepar >> slot) & 1u, 4);
          usepar ^= 1u << slot;
          const int sb = s_buffer(cell, gi);
          // single score buffer of the NVFP4 phase (always the first phase: gi == i)
          if (cell == kNv && i > 0) wait<kPark>(&b->wc, &b->s_free, (uint32_t)(i - 1) & 1u, 5);
          tc_fence_after_sync();
          const uint32_t slot_addr = ring_addr + slot * slot_bytes;
          issue_qk<D>(cell, tmem + s_column(sb), tmem, q_addr, slot_addr, slot_addr, lead);
          mma_commit(&b->s_full[sb], lead);
          if (i == n - 1) mma_commit(&b->q_free, lead);
        }
        if (i > 0) {
          const int gj = g + i - 1;
          const int slot = pv_slot;
          pv_slot = pv_slot + 1 == nslot ? 0 : pv_slot + 1;
          wait<kPark>(&b->wc, &b->p_full[gj & 1], (gj >> 1) & 1, 6);
          tc_fence_after_sync();
          const uint32_t slot_addr = ring_addr + slot * slot_bytes;
          issue_pv<D>(cell, tmem, p_addr + p_buffer(cell, gj) * p_tile_bytes(cell), slot_addr,
                      gj > 0, lead);
          mma_commit(&b->kv_free[slot], lead);  // also tells the softmax warps this PV is done
        }
      }
      g += n;
      ++phase_ord;
    }
    // The end of the tile is signalled on a barrier of its own.
    mma_commit(&b->all_done, lead);
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    // =============================== softmax rows ===============================
    const int row = warp * 32 + lane;            // query row == TMEM lane
    const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);
    RowState st{-5.0e6f, 0.0f};
    int s_use0 = 0, s_use1 = 0;  // stages consumed from each score buffer so far
    uint32_t pvpar = 0;         // per slot: parity of the number of PVs that used it
    int prev_slot = 0;
    uint32_t prev_slot_parity = 0;
    int g = 0;
    int prev_cell = -1;
    const float nv_dom = p.s.v_global_scale * (1.0f / (6.0f * 448.0f));
    const float* vscale = p.o.v_e4m3_scale ? p.o.v_e4m3_scale + (int64_t)head * D : nullptr;
    const bool live_warp = warp * 32 < QB * tile_blocks;
    const int my_block = warp * 32 >= QB && tile_blocks == 2 ? 1 : 0;  // which block of a pair
    if (cnt[kNv] > 0) {
      tmem_st4(tmem_row + kColSfaP, 0x7e7e7e7eu);  // constant 448 block scale of P
      tmem_wait_st();
    }
    for (int cell = 0; cell < 3; ++cell) {
      if (cnt[cell] == 0) continue;
      if (prev_cell >= 0) {
        // per-channel factor that moves O from the previous phase's domain into this one's
        asm volatile("bar.sync 5, 128;" ::: "memory");
        for (int c = threadIdx.x; c < D; c += kSoftmaxThreads) {
          const float from = prev_cell == kNv ? nv_dom
                                              : (prev_cell == kI8 ? vscale[c] * 0.0022326917f : 1.0f);
          const float to = cell == kI8 ? vscale[c] * 0.0022326917f : 1.0f;
          colf[c] = to == 0.0f ? 0.0f : from / to;
        }
        asm volatile("bar.sync 5, 128;" ::: "memory");
      }
      const int first = first_of[cell];
      const float q_scale =
          cell == kI8 ? p.o.q_int8_scale[q_index_i8 + my_block] : 1.0f;
      const float base_scale =
          cell == kNv ? sigma * p.s.q_global_scale * p.s.k_global_scale : sigma;
      // Per-stage metadata (stage id -> real keys, key scale) is fetched 32 stages at a
      // time, one stage per lane, and handed out with shuffles: no dependent global
      // loads sit on the per-stage critical path.
      int meta_valid = 64;
      int meta_member = 1;
      float meta_scale = 1.0f;
      const int nslot = min(kMaxSlots, p.ring_bytes / ((CellInfo<D>::kv_bytes(cell) + 127) & ~127));
      const float* kscale = cell == kI8 ? p.o.k_int8_scale + (int64_t)head * p.stages : nullptr;
      int slot = 0;
      for (int i = 0; i < cnt[cell]; ++i, ++g) {
        if ((i & 31) == 0) {
          const int mine = i + lane;
          if (mine < cnt[cell]) {
            const int entry = list ? list[first + mine] : mine;
            const int stage = entry & 0x3fffffff;
            if (pairs) meta_member = (entry >> (30 + my_block)) & 1;
            meta_valid = p.valid_k[stage];
            if (cell == kI8) meta_scale = sigma * (q_scale * kscale[stage]);
          }
        }
        const int valid = __shfl_sync(0xffffffffu, meta_valid, i & 31);
        const bool member = !pairs || __shfl_sync(0xffffffffu, meta_member, i & 31) != 0;
        const bool phase_first = i == 0 && prev_cell >= 0;
        const int sb = s_buffer(cell, g);
        const uint32_t s_parity = (sb ? s_use1 : s_use0) & 1;
        s_use0 += sb ? 0 : 1;
        s_use1 += sb ? 1 : 0;
        // barrier that the PV of the previous stage completes (its key/value slot release)
        uint64_t* pv_bar = &b->kv_free[prev_slot];
        const uint32_t pv_parity = prev_slot_parity;
        prev_slot = slot;
        prev_slot_parity = (pvpar >> slot) & 1u;
        pvpar ^= 1u << slot;
        slot = slot + 1 == nslot ? 0 : slot + 1;
        const float sc =
            cell == kI8 ? __shfl_sync(0xffffffffu, meta_scale, i & 31) : base_scale;
        softmax_stage<D>(b, p, p_smem, colf, tmem_row, row, cell, g, phase_first, sc, valid,
                         live_warp, member, sb, s_parity, pv_bar, pv_parity, st);
      }
      prev_cell = cell;
    }
    // ---- epilogue: O_true / d -> fp16, packed row order ----
    wait(&b->wc, &b->all_done, 0, 7);
    if (live_warp) {
      tc_fence_after_sync();
      // a block of a pair may have an empty list of its own: its rows are never read
      const float inv = st.d > 0.0f ? 1.0f / st.d : 0.0f;
      const bool live = row < QB * tile_blocks;
      __half* dst = p.out + ((int64_t)head * p.out_rows + (int64_t)block0 * QB + row) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_row + kColO + c0, r);
        tmem_wait_ld();
        if (live) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float a = __uint_as_float(r[j + 2 * i]), c = __uint_as_float(r[j + 2 * i + 1]);
              if (prev_cell == kNv) {
                a *= nv_dom;
                c *= nv_dom;
              } else if (prev_cell == kI8) {
                a *= vscale[c0 + j + 2 * i] * 0.0022326917f;
                c *= vscale[c0 + j + 2 * i + 1] * 0.0022326917f;
              }
              h[i] = __floats2half2_rn(a * inv, c * inv);
            }
            *reinterpret_cast<uint4*>(dst + c0 + j) = v;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemCols);
}

template <int D>
int launch(AttnParams& p, int tiles, cudaStream_t st) {
  const int QB = p.s.query_block;
  int q_region = 0, p_region = 0, slot = 0;
  const bool nv = p.s.has_nvfp4 && !p.dense_prefix, f16 = p.s.has_fp16 && !p.dense_prefix;
  if (nv) {
    // a pair of Q64 blocks brings a second set of scale blocks
    q_region = max(q_region, 128 * D / 2 + (D / 64) * 512 * (p.pair_counts ? 2 : 1));
    p_region = max(p_region, 2 * 128 * 32);
    slot = max(slot, (int)rec::kv_nvfp4_bytes(D));
  }
  if (p.s.has_int8) {
    q_region = max(q_region, 128 * D);
    p_region = max(p_region, 2 * 128 * 64);
    slot = max(slot, (int)rec::kv_int8_bytes(D));
  }
  if (f16) {
    q_region = max(q_region, 128 * D * 2);
    p_region = max(p_region, 128 * 128);
    slot = max(slot, (int)rec::kv_fp16_bytes(D));
  }
  (void)QB;
  q_region = (q_region + 1023) & ~1023;
  const int fixed = q_region + p_region + D * 4 + (int)sizeof(Barriers);
  // two CTAs per SM: measured limit is 115,528 bytes of dynamic shared memory per CTA
  const int budget = 115528;
  int ring = ((budget - fixed) / 128) * 128;
  ring = max(ring, 2 * ((slot + 127) & ~127));
  ring = min(ring, kMaxSlots * ((slot + 127) & ~127));
  p.ring_bytes = ring;
  p.q_region = q_region;
  p.p_region = p_region;
  const size_t smem = (size_t)fixed + (size_t)ring;
  auto kernel = attention_kernel<D>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  kernel<<<dim3(tiles, p.s.heads), kThreads, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

int check_ops(const anemoi_sm100_shape& s, const anemoi_sm100_operands& o, bool dense_prefix) {
  if (s.has_int8 && (!o.q_int8 || !o.kv_int8 || !o.q_int8_scale || !o.k_int8_scale || !o.v_e4m3_scale))
    return ANEMOI_SM100_EINVAL;
  if (dense_prefix) return s.has_int8 ? ANEMOI_SM100_OK : ANEMOI_SM100_EINVAL;
  if (s.has_fp16 && (!o.q_fp16 || !o.kv_fp16)) return ANEMOI_SM100_EINVAL;
  if (s.has_nvfp4 && (!o.q_nvfp4 || !o.kv_nvfp4)) return ANEMOI_SM100_EINVAL;
  return ANEMOI_SM100_OK;
}

uint64_t g_wait_limit_ns = 2000000000ull;

// A one-CTA kernel whose single wait can never be satisfied: nothing arrives on the barrier
// and no copy or MMA is in flight.  It exercises the give-up path of the bounded waits.
__global__ void wait_selftest_kernel(uint64_t limit_ns, int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ WaitContext wc;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    wc.abort = 0;
    wc.status = status;
    wc.limit_ns = limit_ns;
    mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) wait(&wc, &bar, 0, 99);
  __syncthreads();
  // every other thread's wait must now return at once
  if (threadIdx.x != 0) wait(&wc, &bar, 0, 98);
}

}  // namespace

extern "C" int anemoi_sm100_set_wait_limit_ns(uint64_t limit_ns) {
  if (limit_ns == 0) return ANEMOI_SM100_EINVAL;
  g_wait_limit_ns = limit_ns;
  return ANEMOI_SM100_OK;
}

extern "C" int anemoi_sm100_wait_selftest(uint64_t limit_ns, int32_t* status, void* stream) {
  if (limit_ns == 0 || limit_ns > 100000000ull || status == nullptr) return ANEMOI_SM100_EINVAL;
  wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

namespace {
int video_attention(const anemoi_sm100_shape* shape, const anemoi_sm100_operands* ops,
                    const int32_t* row_offset, const int32_t* row_counts, const int32_t* stage_ids,
                    const int32_t* pair_counts, const int32_t* pair_ids, int64_t list_capacity,
                    const int32_t* valid_k, void* out_packed, int32_t* status, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !ops || !row_offset || !row_counts ||
      !valid_k || !out_packed || !status || list_capacity <= 0)
    return ANEMOI_SM100_EINVAL;
  if (check_ops(*shape, *ops, false) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  AttnParams p{};
  p.s = *shape;
  p.o = *ops;
  p.row_offset = row_offset;
  p.row_counts = row_counts;
  p.stage_ids = stage_ids;
  p.pair_counts = pair_counts;
  p.pair_ids = pair_ids;
  p.capacity = list_capacity;
  p.valid_k = valid_k;
  p.out = static_cast<__half*>(out_packed);
  p.status = status;
  p.wait_ns = g_wait_limit_ns;
  p.dense_prefix = 0;
  p.stages = rec::stages(*shape);
  p.q_tiles_int8 = shape->video_blocks + rec::prefix_query_tiles(*shape);
  p.out_rows = shape->video_blocks * shape->query_block;
  const int tiles = pair_counts ? (shape->video_blocks + 1) / 2 : shape->video_blocks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return shape->head_dim == 64 ? launch<64>(p, tiles, st) : launch<128>(p, tiles, st);
}
}  // namespace

extern "C" int anemoi_sm100_attention(const anemoi_sm100_shape* shape,
                                      const anemoi_sm100_operands* ops, const int32_t* row_offset,
                                      const int32_t* row_counts, const int32_t* stage_ids,
                                      int64_t list_capacity, const int32_t* valid_k,
                                      void* out_packed, int32_t* status, void* stream) {
  if (!stage_ids) return ANEMOI_SM100_EINVAL;
  return video_attention(shape, ops, row_offset, row_counts, stage_ids, nullptr, nullptr,
                         list_capacity, valid_k, out_packed, status, stream);
}

extern "C" int anemoi_sm100_attention_pairs(const anemoi_sm100_shape* shape,
                                            const anemoi_sm100_operands* ops,
                                            const int32_t* row_offset, const int32_t* row_counts,
                                            const int32_t* pair_counts, const int32_t* pair_ids,
                                            int64_t list_capacity, const int32_t* valid_k,
                                            void* out_packed, int32_t* status, void* stream) {
  if (!pair_counts || !pair_ids || !shape || shape->query_block != 64) return ANEMOI_SM100_EINVAL;
  return video_attention(shape, ops, row_offset, row_counts, nullptr, pair_counts, pair_ids,
                         list_capacity, valid_k, out_packed, status, stream);
}

extern "C" int anemoi_sm100_prefix_attention(const anemoi_sm100_shape* shape,
                                             const anemoi_sm100_operands* ops,
                                             const int32_t* valid_k, void* out_prefix,
                                             int32_t* status, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !ops || !valid_k || !out_prefix || !status)
    return ANEMOI_SM100_EINVAL;
  if (!shape->has_prefix_query_int8 || shape->prefix_tokens == 0) return ANEMOI_SM100_EINVAL;
  if (check_ops(*shape, *ops, true) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  AttnParams p{};
  p.s = *shape;
  p.o = *ops;
  p.valid_k = valid_k;
  p.out = static_cast<__half*>(out_prefix);
  p.status = status;
  p.wait_ns = g_wait_limit_ns;
  p.dense_prefix = 1;
  p.stages = rec::stages(*shape);
  const int tiles = rec::prefix_query_tiles(*shape);
  p.q_tiles_int8 = shape->video_blocks + tiles;
  p.out_rows = tiles * shape->query_block;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return shape->head_dim == 64 ? launch<64>(p, tiles, st) : launch<128>(p, tiles, st);
}
