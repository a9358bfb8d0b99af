// Block-sparse mixed-precision flash attention for sm_100a.
//
// One CTA (640 threads, one per SM) owns one query tile: QB rows of one head, padded to the
// 128-row MMA shape.  It walks the tile's ragged list of 64-key stages in the order
// NVFP4 -> INT8 -> FP16.  Stage g runs in pipeline g % 3 (its own score buffer S in tensor
// memory and its own probability tile P in shared memory) and accumulates into output
// accumulator g % 2, so three stages are in flight: while one pipeline does its exponentials,
// the tensor core computes QK^T and PV for the others.  The running row maximum is still ONE
// sequence over all stages (each pipeline hands its new maximum to the next through shared
// memory), so every probability is quantised against exactly the maximum a strictly
// sequential walk would use; only the fp32 accumulation is split over two accumulators and
// merged in the epilogue.
//
// Warp roles (five warpgroups, registers moved between them with setmaxnreg):
//   warps 0-11  softmax of pipelines 0..2 (four warps each): thread = query row = TMEM lane;
//               loads the row's 64 scores, releases S, finds the maximum, computes
//               P = 2^(s*scale - m), its sum, converts P to the cell's operand format
//   warps 12-15 correction: rescale an accumulator when the maximum moved since the stage
//               that last touched it (and convert it between the value domains of the
//               phases), off the softmax warps' path
//   warp 16     loader: 1-D bulk copies (TMA engine) of the Q records and of the key and value
//               parts of each stage record into two rings of shared-memory units
//   warps 17-19 MMA of pipelines 0..2: one lane each issues tcgen05.mma (QK^T into S, PV into
//               O) and tcgen05.commit to mbarriers
// TMEM (512 columns): O accumulators at [0,D) and [128,128+D); S of pipeline p at
// [256+64p, +64); scale factors of the NVFP4 phase at [448,512).
//
// Numerics follow the reference's phases
// (csrc/attention/cuda/sm120/q64_attention_phase_composer.inl:1-146, 506-932, 934-1331;
// primitives/qattn/attn_utils.cuh:363-389, 470-625):
//   base-2 online softmax, sigma = log2(e)/sqrt(D), m0 = -5e6, keys >= valid_k masked,
//   denominator accumulated from the unquantised P,
//   NVFP4: score scale sigma*q_gs*k_gs, P -> e2m1(6P) with a constant 448 block scale,
//          O_true = O * v_gs/(6*448)
//   INT8 : exact s32 scores, scale sigma*q_scale*k_scale[stage], P -> e4m3(P*2^8.807),
//          O_true[c] = O[c] * v_scale[c] * 2^-8.807
//   FP16 : P -> f16
// Accumulation is fp32 in TMEM (the reference accumulates a stage in fp16 for the INT8 and
// FP16 cells).
#include <climits>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "bounded_wait.cuh"
#include "records.cuh"
#include "sm100_primitives.cuh"

namespace {

using namespace sm100;

constexpr int kPipes = 3;
constexpr int kThreads = 640;
// setmaxnreg moves registers inside the CTA's own pool, which is what the CTA was launched
// with: 640 threads x 96 registers (the most the launch bound allows).  An increase that the
// decreases of the same CTA cannot cover would wait forever.
constexpr int kLaunchRegs = 96;
constexpr int kSoftmaxRegs = 128;
constexpr int kCorrectionRegs = 48;
constexpr int kOtherRegs = 48;
static_assert(kPipes * 128 * kSoftmaxRegs + 128 * kCorrectionRegs + 128 * kOtherRegs <=
                  kThreads * kLaunchRegs,
              "register budget of the warpgroups exceeds the CTA's pool");
constexpr int kSoftmaxThreads = kPipes * 128;
constexpr int kCorrectionWarp0 = 12;
constexpr int kLoaderWarp = 16;
constexpr int kMmaWarp0 = 17;
constexpr int kTmemCols = 512;
constexpr int kColO = 0;       // + 128 * accumulator
constexpr int kColS = 256;     // + 64 * pipeline
constexpr int kColSf = 448;    // + 20 * pipeline: K scales (8), V scales (4), Q scales (8)
constexpr int kSfbK = 0, kSfbV = 8, kSfaQ = 12;
constexpr int kColSfaP = 508;  // constant 448 block scale of P, shared by the pipelines
constexpr int kMaxUnits = 2 * kPipes;
constexpr int kPBytes = 16384;      // P tile of one pipeline (128 x 64 f16 is the largest)
constexpr int kSmemLimit = 232448;  // dynamic shared memory a CTA may opt into
constexpr float kFp8Offset = 8.807f;
constexpr float kFp8OffsetInv = 0.0022326917f;  // 2^-8.807

enum Cell : int { kNv = 0, kI8 = 1, kF16 = 2 };

#ifdef ATTN_PROFILE
// Debug build only: cycles spent per wait site, summed over all CTAs (lane 0 of each warp).
__device__ unsigned long long g_prof[64];
#define PROF_BEGIN() const long long prof_t0_ = clock64()
#define PROF_END(i) \
  if ((threadIdx.x & 31) == 0) atomicAdd(&g_prof[i], (unsigned long long)(clock64() - prof_t0_))
#else
#define PROF_BEGIN()
#define PROF_END(i)
#endif

struct AttnParams {
  anemoi_sm100_shape s;
  anemoi_sm100_operands o;
  const int32_t* row_offset;
  const int32_t* row_counts;
  const int32_t* stage_ids;
  int64_t capacity;
  const int32_t* valid_k;
  __half* out;       // [H][tiles*QB][D]
  int32_t* status;
  uint64_t wait_ns;  // limit of every mbarrier wait
  int dense_prefix;  // 1: prefix query tiles, INT8 cell over every stage
  int stages;        // 64-key stages per head
  int q_tiles_int8;  // records per head in q_int8 (R + prefix query tiles)
  int out_rows;      // rows per head in `out`
  int q_off[3];      // byte offsets of the three Q records in shared memory
  int p_off;         // three P tiles
  int k_off, k_unit, k_units;  // ring of key units
  int v_off, v_unit, v_units;  // ring of value units
  int misc_off;      // Scratch, then Barriers
};

struct Barriers {
  uint64_t k_full[kMaxUnits], k_free[kMaxUnits];  // key part of a stage landed / QK complete
  uint64_t v_full[kMaxUnits], v_free[kMaxUnits];  // value part landed / PV complete
  uint64_t q_full;
  uint64_t s_full[kPipes];   // scores of the pipeline's stage ready
  uint64_t s_free[kPipes];   // ... and read into registers by its four softmax warps
  uint64_t p_full[kPipes];   // P written
  uint64_t p_free[kPipes];   // ... and read by its PV
  uint64_t o_ok[kPipes];     // the stage's accumulator is in the state its PV may add onto
  uint64_t pv_done[2];       // PV into the accumulator complete
  uint64_t m_ready[kPipes][4];  // new running maximum published, per warp
  uint64_t c_req[kPipes][4];    // rescale request to the correction warp of the same rows
  uint64_t c_ack[kPipes][4];    // ... read by it
  uint64_t all_done;
  WaitContext wc;
  uint32_t tmem_base;
};

struct Scratch {
  float m[kPipes][128];      // running maximum after the pipeline's latest stage
  float alpha[kPipes][128];  // factor for the accumulator of the pipeline's current stage
  float fin_m[kPipes][128];  // final maximum / partial denominator of each pipeline
  float fin_d[kPipes][128];
  float colf[3][128];        // per-channel domain change NVFP4->INT8, NVFP4->FP16, INT8->FP16
  float dom_i8[128];         // v_scale[c] * 2^-8.807
  int flag[kPipes][4];       // request word: bit 0 rescale, cells in bits 4.. (from), 8.. (to)
};

struct Plan {
  int c0, c01, n;  // stages: [0,c0) NVFP4, [c0,c01) INT8, [c01,n) FP16
};
__device__ __forceinline__ int cell_of(const Plan& pl, int g) {
  return g < pl.c0 ? kNv : (g < pl.c01 ? kI8 : kF16);
}

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


// bytes of the key part / value part of a stage record, and where they sit in the record
template <int D>
__device__ __host__ __forceinline__ int k_bytes(int cell) {
  return cell == kNv ? 32 * D + (D / 64) * 512 : (cell == kI8 ? 64 * D : 128 * D);
}
template <int D>
__device__ __host__ __forceinline__ int v_bytes(int cell) {
  return cell == kNv ? 32 * D + 512 : (cell == kI8 ? 64 * D : 128 * D);
}
template <int D>
__device__ __forceinline__ int rec_bytes(int cell) {
  return cell == kNv ? (int)rec::kv_nvfp4_bytes(D)
                     : (cell == kI8 ? (int)rec::kv_int8_bytes(D) : (int)rec::kv_fp16_bytes(D));
}

// ------------------------------------------------------------------------------------------
// softmax side
// ------------------------------------------------------------------------------------------
// 64 scores of one stage: s32 -> f32 for the INT8 cell, masking of the padded keys, row maximum.
__device__ __forceinline__ float stage_max(uint32_t (&r)[64], bool is_i8, int valid) {
  if (is_i8) {
    // as_float(i + 0x4B400000) == 12582912 + i exactly for |i| < 2^22, so the conversion is an
    // integer add and a float subtract (no conversion instruction)
    const float2 magic2 = make_float2(-12582912.0f, -12582912.0f);
#pragma unroll
    for (int j = 0; j < 64; j += 2) {
      const float2 v = fadd2(make_float2(__int_as_float((int)r[j] + 0x4B400000),
                                         __int_as_float((int)r[j + 1] + 0x4B400000)),
                             magic2);
      r[j] = __float_as_uint(v.x);
      r[j + 1] = __float_as_uint(v.y);
    }
  }
  if (valid < 64) {
    // ragged blocks usually lose only a few keys: the common case touches the last 8 columns
    if (valid >= 56) {
#pragma unroll
      for (int j = 56; j < 64; ++j) r[j] = j < valid ? r[j] : 0xff800000u;
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = j < valid ? r[j] : 0xff800000u;
    }
  }
#define S_(j) __uint_as_float(r[(j)])
  float m0 = max3(S_(0), S_(1), S_(2)), m1 = max3(S_(3), S_(4), S_(5));
  float m2 = max3(S_(6), S_(7), S_(8)), m3 = max3(S_(9), S_(10), S_(11));
#pragma unroll
  for (int j = 12; j < 60; j += 8) {
    m0 = max3(m0, S_(j), S_(j + 1));
    m1 = max3(m1, S_(j + 2), S_(j + 3));
    m2 = max3(m2, S_(j + 4), S_(j + 5));
    m3 = max3(m3, S_(j + 6), S_(j + 7));
  }
  m0 = max3(m0, S_(60), S_(61));
  m1 = max3(m1, S_(62), S_(63));
#undef S_
  return fmaxf(max3(m0, m1, m2), m3);
}

// P = 2^(s*scale + bias) in place for 64 scores; returns their sum.
__device__ __forceinline__ float stage_exp(uint32_t (&r)[64], float scale, float bias) {
  const float2 scale2 = make_float2(scale, scale);
  const float2 bias2 = make_float2(bias, bias);
  float2 acc0 = make_float2(0.0f, 0.0f), acc1 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int j = 0; j < 64; j += 4) {
    const float2 a0 = ffma2(
        make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), scale2, bias2);
    const float2 a1 = ffma2(
        make_float2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), scale2, bias2);
    const float e0 = ex2(a0.x), e1 = ex2(a0.y), e2 = ex2(a1.x), e3 = ex2(a1.y);
    r[j] = __float_as_uint(e0);
    r[j + 1] = __float_as_uint(e1);
    r[j + 2] = __float_as_uint(e2);
    r[j + 3] = __float_as_uint(e3);
    acc0 = fadd2(acc0, make_float2(e0, e1));
    acc1 = fadd2(acc1, make_float2(e2, e3));
  }
  return (acc0.x + acc0.y) + (acc1.x + acc1.y);
}

// Writes 64 probabilities of the thread's row into a K-major P tile (128 rows x 64 keys).
template <int CELL>
__device__ __forceinline__ void write_p(uint8_t* p_tile, int row, const uint32_t (&r)[64]) {
#define P_(j) __uint_as_float(r[(j)])
  if (CELL == kF16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 v;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(P_(j * 8 + 2 * i), P_(j * 8 + 2 * i + 1));
      *reinterpret_cast<uint4*>(p_tile + rec::tile_offset(row, j, 8)) = v;
    }
  } else if (CELL == kI8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 v;
      uint16_t* h = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        h[i] = __nv_cvt_float2_to_fp8x2(make_float2(P_(j * 16 + 2 * i), P_(j * 16 + 2 * i + 1)),
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
        h[i] = __nv_cvt_float2_to_fp4x2(make_float2(P_(j * 32 + 2 * i), P_(j * 32 + 2 * i + 1)),
                                        __NV_E2M1, cudaRoundNearest);  // r already holds 6 P
      *reinterpret_cast<uint4*>(p_tile + rec::tile_offset(row, j, 2)) = v;
    }
  }
#undef P_
}

// O[row][c] *= alpha (* colf[c]) for all D columns of the thread's row.
template <int D>
__device__ __forceinline__ void rescale_o(uint32_t tmem_o_row, float alpha, const float* colf) {
  const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll 1
  for (int c0 = 0; c0 < D; c0 += 32) {
    uint32_t r[32];
    tmem_ld32(tmem_o_row + c0, r);
    tmem_wait_ld();
    if (colf != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float2 v = fmul2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), alpha2);
        v = fmul2(v, *reinterpret_cast<const float2*>(colf + c0 + j));
        r[j] = __float_as_uint(v.x);
        r[j + 1] = __float_as_uint(v.y);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float2 v = fmul2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), alpha2);
        r[j] = __float_as_uint(v.x);
        r[j + 1] = __float_as_uint(v.y);
      }
    }
    tmem_st32(tmem_o_row + c0, r);
  }
  tmem_wait_st();
}

// ------------------------------------------------------------------------------------------
// MMA side
// ------------------------------------------------------------------------------------------
// S[128 x 64] = Q K^T for the key unit at `k_addr`; `tmem_sf` = the pipeline's scale columns.
template <int D>
__device__ __forceinline__ void issue_qk(int cell, uint32_t tmem_s, uint32_t tmem_sf,
                                         uint32_t q_addr, uint32_t k_addr) {
  if (cell == kF16) {
    constexpr uint32_t chunks = D / 8;
    const uint32_t idesc = instr_desc(kFmtF16, kFmtF16, kAccF32, 128, 64, 0, 0);
#pragma unroll
    for (int k = 0; k < D / 16; ++k)
      mma_f16_ss(tmem_s, smem_desc(q_addr + k * 256, 128, chunks * 128),
                 smem_desc(k_addr + k * 256, 128, chunks * 128), idesc, k > 0);
  } else if (cell == kI8) {
    constexpr uint32_t chunks = D / 16;
    const uint32_t idesc = instr_desc(kFmtS8, kFmtS8, kAccS32, 128, 64, 0, 0);
#pragma unroll
    for (int k = 0; k < D / 32; ++k)
      mma_i8_ss(tmem_s, smem_desc(q_addr + k * 256, 128, chunks * 128),
                smem_desc(k_addr + k * 256, 128, chunks * 128), idesc, k > 0);
  } else {
    constexpr uint32_t chunks = D / 32;
    const uint32_t idesc = instr_desc_nvf4(128, 64);
    const uint32_t ksf = k_addr + 32 * D;  // scale blocks follow the codes in the unit
#pragma unroll
    for (int k = 0; k < D / 64; ++k)
      tmem_cp_32x128b_warpx4(tmem_sf + kSfbK + 4 * k, smem_desc(ksf + 512 * k, 128, 128));
#pragma unroll
    for (int k = 0; k < D / 64; ++k)
      mma_nvf4_ss(tmem_s, smem_desc(q_addr + k * 256, 128, chunks * 128),
                  smem_desc(k_addr + k * 256, 128, chunks * 128), idesc, k > 0,
                  tmem_sf + kSfaQ + 4 * k, tmem_sf + kSfbK + 4 * k);
  }
}

// O[128 x D] (+)= P[128 x 64] V for the value unit at `v_addr`.
template <int D>
__device__ __forceinline__ void issue_pv(int cell, uint32_t tmem_o, uint32_t tmem_sf,
                                         uint32_t tmem_sfa_p, uint32_t p_addr, uint32_t v_addr,
                                         uint32_t accumulate) {
  if (cell == kF16) {
    const uint32_t idesc = instr_desc(kFmtF16, kFmtF16, kAccF32, 128, D, 0, 1);
    constexpr uint32_t v_lbo = (D / 8) * 128;  // between 8-key groups
#pragma unroll
    for (int k = 0; k < 4; ++k)
      mma_f16_ss(tmem_o, smem_desc(p_addr + k * 256, 128, 8 * 128),
                 smem_desc(v_addr + k * 2 * v_lbo, v_lbo, 128), idesc, accumulate | (k > 0));
  } else if (cell == kI8) {
    const uint32_t idesc = instr_desc(kFmtE4M3, kFmtE4M3, kAccF32, 128, D, 0, 0);
#pragma unroll
    for (int k = 0; k < 2; ++k)
      mma_f8_ss(tmem_o, smem_desc(p_addr + k * 256, 128, 4 * 128),
                smem_desc(v_addr + k * 256, 128, 4 * 128), idesc, accumulate | (k > 0));
  } else {
    const uint32_t vsf = v_addr + 32 * D;  // the scale block follows the codes in the unit
    const uint32_t idesc = instr_desc_nvf4(128, D);
    tmem_cp_32x128b_warpx4(tmem_sf + kSfbV, smem_desc(vsf, 128, 128));
    mma_nvf4_ss(tmem_o, smem_desc(p_addr, 128, 2 * 128), smem_desc(v_addr, 128, 2 * 128), idesc,
                accumulate, tmem_sfa_p, tmem_sf + kSfbV);
  }
}

// position of stage g in a ring of `units` (units >= 3), advanced by the pipeline stride
struct RingPos {
  int slot;
  uint32_t par;
  __device__ __forceinline__ void advance(int by, int units) {
    slot += by;
    if (slot >= units) {
      slot -= units;
      par ^= 1u;
    }
  }
};

// Real keys and score scale of the pipeline's k-th stage (kept out of line: it runs once per
// 32 stages and must not hold registers in the softmax loop).
template <int D>
__device__ __noinline__ void fetch_stage_meta(const AttnParams& p, const Plan& pl,
                                              const int32_t* list, int head, int64_t q_index_i8,
                                              int pi, int k, int& valid, float& scale) {
  const int g = kPipes * k + pi;
  valid = 0;
  scale = 0.0f;
  if (g >= pl.n) return;
  const float sigma = (D == 64 ? 0.125f : 0.08838834764831845f) * 1.4426950408889634f;
  const int cell = cell_of(pl, g);
  const int st = list ? list[g] : g;
  valid = p.valid_k[st];
  if (cell == kI8) {
    scale = sigma * (p.o.q_int8_scale[q_index_i8] * p.o.k_int8_scale[(int64_t)head * p.stages + st]);
  } else {
    scale = cell == kNv ? sigma * p.s.q_global_scale * p.s.k_global_scale : sigma;
  }
}

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads, 1) attention_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int QB = p.s.query_block;
  const int head = blockIdx.y;
  // launch order of the head's query blocks (longest list first) as written by the routing
  // stage; 0 = no order given
  int tile = blockIdx.x;
  if (!p.dense_prefix) {
    const int ordered = p.row_counts[((int64_t)head * p.s.video_blocks + blockIdx.x) * 4 + 3];
    if (ordered > 0) tile = ordered - 1;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ATTN_PROFILE
  const long long prof_start = clock64();
#endif

  // ---- this tile's work list ----
  Plan pl;
  const int32_t* list;
  if (p.dense_prefix) {
    pl.c0 = 0;
    pl.c01 = p.stages;
    pl.n = p.stages;
    list = nullptr;
  } else {
    const int32_t* rc = p.row_counts + ((int64_t)head * p.s.video_blocks + tile) * 4;
    pl.c0 = rc[0];
    pl.c01 = pl.c0 + rc[1];
    pl.n = pl.c01 + rc[2];
    list = p.stage_ids + (int64_t)head * p.capacity +
           p.row_offset[(int64_t)head * p.s.video_blocks + tile];
  }
  if (pl.n == 0) return;
  // After a give-up anywhere on this device the status word stays set: later CTAs (of this and
  // of later launches, until the host clears the word) return at once instead of each running
  // into its own wait limit.
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  const int n = pl.n;

  uint8_t* q_smem = smem;
  uint8_t* p_smem = smem + p.p_off;
  uint8_t* k_ring = smem + p.k_off;
  uint8_t* v_ring = smem + p.v_off;
  Scratch* sc = reinterpret_cast<Scratch*>(smem + p.misc_off);
  Barriers* b = reinterpret_cast<Barriers*>(smem + p.misc_off + sizeof(Scratch));

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxUnits; ++i) {
      mbar_init(&b->k_full[i], 1);
      mbar_init(&b->k_free[i], 1);
      mbar_init(&b->v_full[i], 1);
      mbar_init(&b->v_free[i], 1);
    }
    mbar_init(&b->q_full, 1);
    for (int i = 0; i < kPipes; ++i) {
      mbar_init(&b->s_full[i], 1);
      mbar_init(&b->s_free[i], 4);
      mbar_init(&b->p_full[i], 4);
      mbar_init(&b->p_free[i], 1);
      for (int w = 0; w < 4; ++w) {
        mbar_init(&b->m_ready[i][w], 1);
        mbar_init(&b->c_req[i][w], 1);
        mbar_init(&b->c_ack[i][w], 1);
      }
    }
    for (int i = 0; i < kPipes; ++i) mbar_init(&b->o_ok[i], 4);
    for (int i = 0; i < 2; ++i) mbar_init(&b->pv_done[i], 1);
    mbar_init(&b->all_done, kPipes);
    b->wc.abort = 0;
    b->wc.status = p.status;
    b->wc.limit_ns = p.wait_ns;
    mbar_init_fence();
  }
  // Query rows beyond QB (64-row tiles padded to the 128-row MMA shape) are never
  // initialised: rows are independent, their results stay in TMEM lanes nobody reads.
  if (warp == kMmaWarp0) {
    tmem_alloc(&b->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = b->tmem_base;
  WaitContext* const wc = &b->wc;

  const int q_index_fp = head * p.s.video_blocks + tile;  // q_fp16 / q_nvfp4 record
  const int64_t q_index_i8 =
      (int64_t)head * p.q_tiles_int8 + (p.dense_prefix ? p.s.video_blocks + tile : tile);
  const float sigma = (D == 64 ? 0.125f : 0.08838834764831845f) * 1.4426950408889634f;
  const float nv_dom = p.s.v_global_scale * (1.0f / (6.0f * 448.0f));
  const float* vscale = p.o.v_e4m3_scale ? p.o.v_e4m3_scale + (int64_t)head * D : nullptr;

  // All four warps of a warpgroup execute the same setmaxnreg instruction, and each sits at the
  // top of the branch whose code runs under the new register count.
  if (warp >= kLoaderWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    if (warp == kLoaderWarp) {
      // =============================== loader ===============================
      // The whole warp runs the loop with uniform control flow (list entries are fetched 32 at
      // a time, one per lane); one lane issues the copies.  The key parts and the value parts
      // of the stage records go to two rings with cursors of their own: a key unit is free as
      // soon as its QK has run, a value unit only after its PV.
      const uint32_t lead = lane == 0;
      {
        uint32_t total = 0;
        if (pl.c0 > 0) total += (uint32_t)rec::q_nvfp4_bytes(QB, D);
        if (pl.c01 > pl.c0) total += (uint32_t)rec::q_int8_bytes(QB, D);
        if (pl.n > pl.c01) total += (uint32_t)rec::q_fp16_bytes(QB, D);
        mbar_arrive_expect_tx(&b->q_full, total, lead);
        if (pl.c0 > 0) {
          const int qbytes = (int)rec::q_nvfp4_bytes(QB, D);
          const uint8_t* src = static_cast<const uint8_t*>(p.o.q_nvfp4) + (int64_t)q_index_fp * qbytes;
          uint8_t* dst = q_smem + p.q_off[kNv];
          if (QB == 64) {
            // codes fill the first half of the 128-row tile; scale blocks follow the full tile
            const int codes = QB * D / 2;
            bulk_g2s(dst, src, codes, &b->q_full, lead);
            bulk_g2s(dst + 128 * D / 2, src + codes, qbytes - codes, &b->q_full, lead);
          } else {
            bulk_g2s(dst, src, qbytes, &b->q_full, lead);
          }
        }
        if (pl.c01 > pl.c0) {
          const int qbytes = (int)rec::q_int8_bytes(QB, D);
          bulk_g2s(q_smem + p.q_off[kI8],
                   static_cast<const uint8_t*>(p.o.q_int8) + q_index_i8 * qbytes, qbytes, &b->q_full,
                   lead);
        }
        if (pl.n > pl.c01) {
          const int qbytes = (int)rec::q_fp16_bytes(QB, D);
          bulk_g2s(q_smem + p.q_off[kF16],
                   static_cast<const uint8_t*>(p.o.q_fp16) + (int64_t)q_index_fp * qbytes, qbytes,
                   &b->q_full, lead);
        }
      }
      int win0 = -64, stage_l = 0;  // window of 32 list entries held one per lane
      int cur[2] = {0, 0};          // next stage whose key (0) / value (1) part is to be loaded
      int slot[2] = {0, 0};
      uint32_t fills[2] = {0, 0};   // per unit: parity of the number of fills so far
      uint64_t t0 = 0;
      int idle = 0;
      while (cur[0] < n || cur[1] < n) {
        bool progress = false;
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          const int g = cur[part];
          if (g >= n) continue;
          const int units = part ? p.v_units : p.k_units;
          uint64_t* full = part ? b->v_full : b->k_full;
          uint64_t* free_bar = part ? b->v_free : b->k_free;
          const int u = slot[part];
          // fill f of a unit may start once the MMA that read fill f-1 is complete
          int ok = g < units || mbar_test_wait(&free_bar[u], ((fills[part] >> u) & 1u) ^ 1u);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) continue;
          if (list != nullptr && (g < win0 || g >= win0 + 32)) {
            win0 = g;
            stage_l = win0 + lane < n ? list[win0 + lane] : 0;
          }
          const int cell = cell_of(pl, g);
          const int stage = list ? __shfl_sync(0xffffffffu, stage_l, (g - win0) & 31) : g;
          const int rb = rec_bytes<D>(cell);
          const uint8_t* src =
              (cell == kNv ? static_cast<const uint8_t*>(p.o.kv_nvfp4)
               : cell == kI8 ? static_cast<const uint8_t*>(p.o.kv_int8)
                             : static_cast<const uint8_t*>(p.o.kv_fp16)) +
              ((int64_t)head * p.stages + stage) * rb;
          uint8_t* dst = part ? v_ring + u * p.v_unit : k_ring + u * p.k_unit;
          const int bytes = part ? v_bytes<D>(cell) : k_bytes<D>(cell);
          mbar_arrive_expect_tx(&full[u], (uint32_t)bytes, lead);
          if (cell == kNv) {
            // codes, then the scale blocks behind them
            const int sf = part ? 512 : (D / 64) * 512;
            bulk_g2s(dst, src + (part ? rec::kv_nvfp4_v_offset(D) : 0), 32 * D, &full[u], lead);
            bulk_g2s(dst + 32 * D,
                     src + (part ? rec::kv_nvfp4_vsf_offset(D) : rec::kv_nvfp4_ksf_offset(D)), sf,
                     &full[u], lead);
          } else {
            bulk_g2s(dst, src + (part ? (rb >> 1) : 0), bytes, &full[u], lead);
          }
          fills[part] ^= 1u << u;
          slot[part] = u + 1 == units ? 0 : u + 1;
          cur[part] = g + 1;
          progress = true;
        }
        if (progress) {
          idle = 0;
          t0 = 0;
        } else {
          asm volatile("nanosleep.u32 100;");
          if (++idle >= 32) {
            idle = 0;
            if (b->wc.abort) break;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > p.wait_ns) {
              b->wc.abort = 1;
              atomicCAS(p.status, 0, 1);
              break;
            }
          }
        }
      }
      // Unwinding after a give-up: copies already issued must land before the CTA returns
      // its shared memory (on the normal path the MMA warps have consumed every one of them).
      if (b->wc.abort) {
        for (int u = 0; u < kMaxUnits; ++u) {
          if (u < p.k_units && u < cur[0]) drain_wait(&b->k_full[u], ((fills[0] >> u) & 1u) ^ 1u, 1000000ull);
          if (u < p.v_units && u < cur[1]) drain_wait(&b->v_full[u], ((fills[1] >> u) & 1u) ^ 1u, 1000000ull);
        }
        drain_wait(&b->q_full, 0, 1000000ull);
      }
    } else {
      // =============================== MMA issue (one warp per pipeline) =====================
      const int pi = warp - kMmaWarp0;
      if (lane == 0) {
        const uint32_t q_base = smem_u32(q_smem);
        const uint32_t p_addr = smem_u32(p_smem) + pi * kPBytes;
        const uint32_t k_base = smem_u32(k_ring), v_base = smem_u32(v_ring);
        const uint32_t tmem_s = tmem + kColS + 64 * pi;
        const uint32_t tmem_sf = tmem + kColSf + 20 * pi;
        wait<100>(wc, &b->q_full, 0, 3);
        tc_fence_after_sync();
        if (pl.c0 > 0) {
          const uint32_t qsf = q_base + p.q_off[kNv] + 128 * D / 2;
#pragma unroll
          for (int k = 0; k < D / 64; ++k)
            tmem_cp_32x128b_warpx4(tmem_sf + kSfaQ + 4 * k, smem_desc(qsf + 512 * k, 128, 128));
        }
        // QK of the pipeline's next stage is issued as soon as the softmax warps have read the
        // scores of the current one, PV of the current one when its P is written and its
        // accumulator corrected: in this order, which is the order the events happen in.
        RingPos kq{pi % p.k_units, 0}, vq{pi % p.v_units, 0};
        if (pi < n) {
          wait<50>(wc, &b->k_full[kq.slot], kq.par, 4);
          tc_fence_after_sync();
          const int cell = cell_of(pl, pi);
          issue_qk<D>(cell, tmem_s, tmem_sf, q_base + p.q_off[cell], k_base + kq.slot * p.k_unit);
          mma_commit(&b->s_full[pi]);
          mma_commit(&b->k_free[kq.slot]);
        }
        int k = 0;
        for (int g = pi; g < n; g += kPipes, ++k) {
          const int gn = g + kPipes;
          if (gn < n) {
            kq.advance(kPipes, p.k_units);
            wait<50>(wc, &b->k_full[kq.slot], kq.par, 4);
            wait<20>(wc, &b->s_free[pi], k & 1, 5);
            tc_fence_after_sync();
            const int cell = cell_of(pl, gn);
            issue_qk<D>(cell, tmem_s, tmem_sf, q_base + p.q_off[cell], k_base + kq.slot * p.k_unit);
            mma_commit(&b->s_full[pi]);
            mma_commit(&b->k_free[kq.slot]);
          }
          const int acc = g & 1;
          wait<50>(wc, &b->v_full[vq.slot], vq.par, 6);
          wait<20>(wc, &b->p_full[pi], k & 1, 7);
          wait<20>(wc, &b->o_ok[pi], k & 1, 8);
          tc_fence_after_sync();
          issue_pv<D>(cell_of(pl, g), tmem + kColO + 128 * acc, tmem_sf, tmem + kColSfaP, p_addr,
                      v_base + vq.slot * p.v_unit, g >= 2);
          mma_commit(&b->pv_done[acc]);
          mma_commit(&b->p_free[pi]);
          mma_commit(&b->v_free[vq.slot]);
          vq.advance(kPipes, p.v_units);
        }
        // The end of the tile is signalled on a barrier of its own (one arrival per MMA warp);
        // each MMA lane also waits for it, so that no MMA is in flight when tensor memory is
        // given back.
        mma_commit(&b->all_done);
        if (!drain_wait(&b->all_done, 0, p.wait_ns)) {
          b->wc.abort = 1;
          atomicCAS(p.status, 0, 9);
        }
      }
      __syncwarp();
    }
  } else if (warp >= kCorrectionWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kCorrectionRegs));
    // =============================== correction ===============================
    const int cw = warp - kCorrectionWarp0;
    const int row = cw * 32 + lane;
    const uint32_t lane_base = (uint32_t)(cw * 32) << 16;
    // per-channel factors that move O from one phase's value domain into the next one's
    for (int c = threadIdx.x - kCorrectionWarp0 * 32; c < D; c += 128) {
      const float i8 = vscale != nullptr ? vscale[c] * kFp8OffsetInv : 0.0f;
      sc->dom_i8[c] = i8;
      sc->colf[0][c] = i8 == 0.0f ? 0.0f : nv_dom / i8;
      sc->colf[1][c] = nv_dom;
      sc->colf[2][c] = i8;
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    int pi = 0, k = 0;  // stage g = 3 k + pi
    for (int g = 0; g < n; ++g) {
      const int acc = g & 1;
      wait<20>(wc, &b->c_req[pi][cw], k & 1, 30);
      const int flag = sc->flag[pi][cw];
      const float alpha = (flag & 1) ? sc->alpha[pi][row] : 1.0f;
      __syncwarp();
      if (lane == 0) mbar_arrive(&b->c_ack[pi][cw]);
      // The previous PV into this accumulator must be complete before it is touched.  The wait
      // is made even when nothing is rescaled: a barrier's phase may only complete after its
      // waiter has seen the phase before it, and o_ok of stage g+3 (same pipeline, same MMA
      // warp) is then signalled after stage g+2 waited here for PV of stage g, which that MMA
      // warp issued after it saw o_ok of stage g.
      if (g >= 2) wait<20>(wc, &b->pv_done[acc], ((g >> 1) - 1) & 1, 31);
      if (flag & 1) {
        tc_fence_after_sync();
        const int from = (flag >> 4) & 3, to = (flag >> 8) & 3;
        const float* colf =
            from == to ? nullptr : sc->colf[from == kNv ? (to == kI8 ? 0 : 1) : 2];
        rescale_o<D>(tmem + lane_base + kColO + 128 * acc, alpha, colf);
        tc_fence_before_sync();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&b->o_ok[pi]);
      if (++pi == kPipes) {
        pi = 0;
        ++k;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    // =============================== softmax rows ===============================
    const int pi = warp >> 2;                    // pipeline
    const int w = warp & 3;                      // warp of the pipeline = TMEM lane quarter
    const int row = w * 32 + lane;               // query row == TMEM lane
    const uint32_t lane_base = (uint32_t)(w * 32) << 16;
    const uint32_t tmem_s = tmem + lane_base + kColS + 64 * pi;
    const bool live_warp = w * 32 < QB;
    const bool lead = lane == 0;
    const int prev_pi = pi == 0 ? kPipes - 1 : pi - 1;   // pipeline of stage g-1
    const int prev2_pi = pi == kPipes - 1 ? 0 : pi + 1;  // pipeline of stage g-2
    uint8_t* p_tile = p_smem + pi * kPBytes;
    if (pl.c0 > 0) {
      tmem_st4(tmem + lane_base + kColSfaP, 0x7e7e7e7eu);  // constant 448 block scale of P
      tmem_wait_st();
    }
    float m_own = -5.0e6f, d = 0.0f;
    // Metadata of 32 of the pipeline's stages (real keys and score scale), one stage per lane,
    // fetched one batch ahead of its use.
    int nx_valid = 0, cu_valid = 0;
    float nx_scale = 0.0f, cu_scale = 0.0f;
    auto fetch_meta = [&](int k0) { fetch_stage_meta<D>(p, pl, list, head, q_index_i8, pi, k0 + lane, nx_valid, nx_scale); };
    fetch_meta(0);
    int k = 0;
    for (int g = pi; g < n; g += kPipes, ++k) {
      if ((k & 31) == 0) {
        cu_valid = nx_valid;
        cu_scale = nx_scale;
        fetch_meta(k + 32);
      }
      const int cell = cell_of(pl, g);
      const int valid = __shfl_sync(0xffffffffu, cu_valid, k & 31);
      const float scale = __shfl_sync(0xffffffffu, cu_scale, k & 31);
      {
        PROF_BEGIN();
        wait(wc, &b->s_full[pi], k & 1, 10 + cell);
        PROF_END(0 + cell);
      }
      PROF_BEGIN();
      tc_fence_after_sync();
      if (!live_warp) {
        // padding rows of a 64-row tile: keep the barrier protocol, skip the math
        if (k > 0) wait(wc, &b->c_ack[pi][w], (k - 1) & 1, 14);
        if (lead) {
          mbar_arrive(&b->s_free[pi]);
          sc->flag[pi][w] = 0;
          mbar_arrive(&b->c_req[pi][w]);
        }
        if (k > 0) wait(wc, &b->p_free[pi], (k - 1) & 1, 15);
        if (lead) mbar_arrive(&b->p_full[pi]);
        continue;
      }
      uint32_t r[64];
      tmem_ld32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(r));
      tmem_ld32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
      tmem_wait_ld();
      // the scores are in registers: the MMA warp may overwrite the buffer (QK of stage g+3)
      tc_fence_before_sync();
      __syncwarp();
      if (lead) mbar_arrive(&b->s_free[pi]);

      const float m_loc = stage_max(r, cell == kI8, valid) * scale;

      // one running maximum for all pipelines: take the latest (stage g-1), publish ours
      float m_prev = -5.0e6f, m_prev2 = -5.0e6f;
      if (g > 0) {
        PROF_END(9);
        {
          PROF_BEGIN();
          wait(wc, &b->m_ready[prev_pi][w], (pi == 0 ? k - 1 : k) & 1, 16);
          PROF_END(4);
        }
        m_prev = sc->m[prev_pi][row];
        if (g > 1) m_prev2 = sc->m[prev2_pi][row];  // after stage g-2: what the accumulator refers to
      }
      const float m_new = fmaxf(m_prev, m_loc);
      sc->m[pi][row] = m_new;
      __syncwarp();
      if (lead) mbar_arrive(&b->m_ready[pi][w]);

      // the accumulator of this stage was last touched by stage g-2
      const float alpha_acc = ex2(m_prev2 - m_new);
      const int cell2 = g > 1 ? cell_of(pl, g - 2) : cell;
      const bool need = g > 1 && (cell != cell2 || __any_sync(0xffffffffu, alpha_acc != 1.0f));
      if (k > 0) {
        PROF_BEGIN();
        wait(wc, &b->c_ack[pi][w], (k - 1) & 1, 17);  // previous request has been read
        PROF_END(5);
      }
      if (need) sc->alpha[pi][row] = alpha_acc;
      if (lead) sc->flag[pi][w] = need ? (1 | (cell2 << 4) | (cell << 8)) : 0;
      __syncwarp();
      if (lead) mbar_arrive(&b->c_req[pi][w]);

      // exponent = s * scale + bias; the NVFP4 cell produces 6 P directly (e2m1 input range),
      // the INT8 cell P * 2^8.807 (e4m3 input range); the sums are scaled back.
      const float bias = cell == kI8 ? kFp8Offset - m_new
                                     : (cell == kNv ? 2.5849625007f - m_new : -m_new);
      const float sum_scale = cell == kI8 ? kFp8OffsetInv : (cell == kNv ? 0.16666667f : 1.0f);
      const float sum = stage_exp(r, scale, bias);
      d = d * ex2(m_own - m_new) + sum * sum_scale;  // this pipeline's share of the denominator
      m_own = m_new;

      // the P tile is free once the pipeline's previous PV has read it
      if (k > 0) {
        PROF_BEGIN();
        wait(wc, &b->p_free[pi], (k - 1) & 1, 20 + cell);
        PROF_END(6);
      }
      if (cell == kNv) {
        write_p<kNv>(p_tile, row, r);
      } else if (cell == kI8) {
        write_p<kI8>(p_tile, row, r);
      } else {
        write_p<kF16>(p_tile, row, r);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lead) mbar_arrive(&b->p_full[pi]);
      PROF_END(7);
#ifdef ATTN_PROFILE
      if (lead) atomicAdd(&g_prof[8], 1ull);
#endif
    }
    // ---- epilogue: merge the accumulators, O_true / d -> fp16, packed row order ----
    sc->fin_m[pi][row] = m_own;
    sc->fin_d[pi][row] = d;
    asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
    wait(wc, &b->all_done, 0, 40);
    if (live_warp) {
      tc_fence_after_sync();
      const int last_pi = (n - 1) % kPipes;
      const float mf = sc->m[last_pi][row];  // maximum after the last stage
      float dsum = 0.0f;
#pragma unroll
      for (int q = 0; q < kPipes; ++q)
        if (q < n) dsum += sc->fin_d[q][row] * ex2(sc->fin_m[q][row] - mf);
      const float inv = 1.0f / dsum;
      // accumulator of the last stage refers to mf; the other one to the maximum after stage n-2
      const int acc1 = (n - 1) & 1;
      const bool has2 = n > 1;
      const int cell1 = cell_of(pl, n - 1), cell2 = has2 ? cell_of(pl, n - 2) : 0;
      const float g1 = inv;
      const float g2 = has2 ? ex2(sc->m[last_pi == 0 ? kPipes - 1 : last_pi - 1][row] - mf) * inv : 0.0f;
      const bool live = row < QB;
      __half* dst = p.out + ((int64_t)head * p.out_rows + (int64_t)tile * QB + row) * D;
      // the pipelines' warpgroups share the channels in chunks of 32
#pragma unroll 1
      for (int c0 = 32 * pi; c0 < D; c0 += 32 * kPipes) {
        uint32_t a[32], bb[32];
        tmem_ld32(tmem + lane_base + kColO + 128 * acc1 + c0, a);
        if (has2) tmem_ld32(tmem + lane_base + kColO + 128 * (acc1 ^ 1) + c0, bb);
        tmem_wait_ld();
        if (live) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float o[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int c = c0 + j + 2 * i + e;
                const float d1 = cell1 == kNv ? nv_dom : (cell1 == kI8 ? sc->dom_i8[c] : 1.0f);
                float accv = __uint_as_float(a[j + 2 * i + e]) * d1 * g1;
                if (has2) {
                  const float d2 = cell2 == kNv ? nv_dom : (cell2 == kI8 ? sc->dom_i8[c] : 1.0f);
                  accv += __uint_as_float(bb[j + 2 * i + e]) * d2 * g2;
                }
                o[e] = accv;
              }
              h[i] = __floats2half2_rn(o[0], o[1]);
            }
            *reinterpret_cast<uint4*>(dst + c0 + j) = v;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp0) tmem_dealloc(tmem, kTmemCols);
#ifdef ATTN_PROFILE
  if (threadIdx.x == 0) {
    atomicAdd(&g_prof[21], (unsigned long long)(clock64() - prof_start));
    atomicAdd(&g_prof[22], 1ull);
    atomicAdd(&g_prof[23], (unsigned long long)n);
  }
#endif
}

template <int D>
int launch(AttnParams& p, int tiles, cudaStream_t st) {
  const bool nv = p.s.has_nvfp4 && !p.dense_prefix, f16 = p.s.has_fp16 && !p.dense_prefix;
  int off = 0, ku = 0, vu = 0;
  p.q_off[kNv] = p.q_off[kI8] = p.q_off[kF16] = 0;
  if (nv) {
    p.q_off[kNv] = off;
    off += (128 * D / 2 + (D / 64) * 512 + 1023) & ~1023;
    ku = max(ku, k_bytes<D>(kNv));
    vu = max(vu, v_bytes<D>(kNv));
  }
  if (p.s.has_int8) {
    p.q_off[kI8] = off;
    off += 128 * D;
    ku = max(ku, k_bytes<D>(kI8));
    vu = max(vu, v_bytes<D>(kI8));
  }
  if (f16) {
    p.q_off[kF16] = off;
    off += 128 * D * 2;
    ku = max(ku, k_bytes<D>(kF16));
    vu = max(vu, v_bytes<D>(kF16));
  }
  ku = (ku + 127) & ~127;
  vu = (vu + 127) & ~127;
  p.p_off = off;
  off += kPipes * kPBytes;
  const int misc = (int)((sizeof(Scratch) + sizeof(Barriers) + 127) & ~127);
  const int ring = kSmemLimit - off - misc;
  // Every barrier is waited on phase by phase by one waiter: a pipeline's MMA warp must meet
  // the same units again and again, so both rings hold a multiple of kPipes units (stage g
  // uses unit g % units, pipeline g % kPipes).  Key units turn over quickly (free after QK),
  // value units are held until PV.
  p.k_unit = ku;
  p.v_unit = vu;
  p.k_units = p.v_units = kPipes;
  if (ring < kPipes * (ku + vu)) return ANEMOI_SM100_ELAUNCH;
  if (ring >= kPipes * (ku + 2 * vu)) p.v_units = 2 * kPipes;
  if (ring >= 2 * kPipes * (ku + vu)) p.k_units = 2 * kPipes;
  p.k_off = off;
  p.v_off = off + p.k_units * ku;
  p.misc_off = p.v_off + p.v_units * vu;
  const size_t smem = (size_t)p.misc_off + misc;
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
  if (threadIdx.x == 0) wait<50>(&wc, &bar, 0, 99);
  __syncthreads();
  // every other thread's wait must now return at once
  if (threadIdx.x != 0) wait(&wc, &bar, 0, 98);
}

}  // namespace

#ifdef ATTN_PROFILE
extern "C" int anemoi_sm100_debug_profile(unsigned long long* host64, int reset) {
  if (cudaMemcpyFromSymbol(host64, g_prof, sizeof(g_prof)) != cudaSuccess) return -2;
  if (reset) {
    static unsigned long long zeros[64];
    if (cudaMemcpyToSymbol(g_prof, zeros, sizeof(zeros)) != cudaSuccess) return -2;
  }
  return 0;
}
#endif

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

extern "C" int anemoi_sm100_attention(const anemoi_sm100_shape* shape,
                                      const anemoi_sm100_operands* ops, const int32_t* row_offset,
                                      const int32_t* row_counts, const int32_t* stage_ids,
                                      int64_t list_capacity, const int32_t* valid_k,
                                      void* out_packed, int32_t* status, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !ops || !row_offset || !row_counts ||
      !stage_ids || !valid_k || !out_packed || !status || list_capacity <= 0)
    return ANEMOI_SM100_EINVAL;
  if (check_ops(*shape, *ops, false) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  AttnParams p{};
  p.s = *shape;
  p.o = *ops;
  p.row_offset = row_offset;
  p.row_counts = row_counts;
  p.stage_ids = stage_ids;
  p.capacity = list_capacity;
  p.valid_k = valid_k;
  p.out = static_cast<__half*>(out_packed);
  p.status = status;
  p.wait_ns = g_wait_limit_ns;
  p.dense_prefix = 0;
  p.stages = rec::stages(*shape);
  p.q_tiles_int8 = shape->video_blocks + rec::prefix_query_tiles(*shape);
  p.out_rows = shape->video_blocks * shape->query_block;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return shape->head_dim == 64 ? launch<64>(p, shape->video_blocks, st)
                               : launch<128>(p, shape->video_blocks, st);
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
