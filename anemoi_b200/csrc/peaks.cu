// tcgen05 tensor-pipe throughput probe: the denominator of the attention kernel's roofline,
// measured per MMA kind with the same instruction forms, operand layout (K-major core
// matrices, no swizzle) and tile shape (M = 128, N = 128, one 32-byte k-step per instruction)
// the attention kernel issues.  Two CTAs per SM, one issuing lane each; operands stay in
// shared memory and every instruction accumulates into the same TMEM tile, so nothing but the
// tensor pipe and its operand fetch is exercised.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/anemoi_sm100.h"
#include "sm100_primitives.cuh"

namespace {

using namespace sm100;

constexpr int kThreads = 128;
constexpr int kTileBytes = 128 * 256;  // 128 rows x 8 k-steps of 32 bytes
constexpr int kColSfa = 128, kColSfb = 132;

struct PeakShared {
  uint64_t done;
  uint32_t tmem_base;
};

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(kThreads, 2) tensor_peak_kernel(int kind, int iters, int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* a_tile = smem;
  uint8_t* b_tile = smem + kTileBytes;
  PeakShared* sh = reinterpret_cast<PeakShared*>(smem + 2 * kTileBytes);
  const int warp = threadIdx.x >> 5;

  // small finite values in every format: fp16 0x2C2C = 0.0652, e4m3 0x2C = 0.1875, s8 44, e2m1 pairs
  for (int i = threadIdx.x; i < 2 * kTileBytes / 16; i += kThreads)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0x2C2C2C2Cu, 0x2C2C2C2Cu, 0x2C2C2C2Cu, 0x2C2C2C2Cu);
  if (threadIdx.x == 0) {
    mbar_init(&sh->done, 1);
    mbar_init_fence();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(&sh->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;
  {
    // unit block scales (ue4m3 0x38 = 1.0) for the block-scaled kind, all lanes
    const uint32_t row = tmem + ((uint32_t)(warp * 32) << 16);
    const uint32_t one = 0x38383838u;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%1,%1,%1};" ::"r"(row + kColSfa), "r"(one)
                 : "memory");
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%1,%1,%1};" ::"r"(row + kColSfb), "r"(one)
                 : "memory");
    tmem_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  if (threadIdx.x == 0) {
    const uint32_t a_addr = smem_u32(a_tile), b_addr = smem_u32(b_tile);
    const uint32_t id_f16 = instr_desc(kFmtF16, kFmtF16, kAccF32, 128, 128, 0, 0);
    const uint32_t id_i8 = instr_desc(kFmtS8, kFmtS8, kAccS32, 128, 128, 0, 0);
    const uint32_t id_f8 = instr_desc(kFmtE4M3, kFmtE4M3, kAccF32, 128, 128, 0, 0);
    const uint32_t id_nv = instr_desc_nvf4(128, 128);
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t ad = smem_desc(a_addr + k * 256, 128, 16 * 128);
        const uint64_t bd = smem_desc(b_addr + k * 256, 128, 16 * 128);
        const uint32_t acc = (it | k) != 0;
        if (kind == ANEMOI_SM100_KIND_F16) {
          mma_f16_ss(tmem, ad, bd, id_f16, acc);
        } else if (kind == ANEMOI_SM100_KIND_I8) {
          mma_i8_ss(tmem, ad, bd, id_i8, acc);
        } else if (kind == ANEMOI_SM100_KIND_F8) {
          mma_f8_ss(tmem, ad, bd, id_f8, acc);
        } else {
          mma_nvf4_ss(tmem, ad, bd, id_nv, acc, tmem + kColSfa, tmem + kColSfb);
        }
      }
    }
    mma_commit(&sh->done);
    // bounded wait (2 s): a give-up is reported, never spun on
    const uint64_t t0 = timer_ns();
    bool ok = false;
    while (!(ok = mbar_try_wait(&sh->done, 0))) {
      if (timer_ns() - t0 > 2000000000ull) break;
    }
    if (!ok) atomicCAS(status, 0, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

extern "C" int anemoi_sm100_tensor_peak(int32_t kind, int32_t iterations, int32_t* status, double* flops,
                                        void* stream) {
  if (kind < ANEMOI_SM100_KIND_F16 || kind > ANEMOI_SM100_KIND_NVFP4 || iterations <= 0 ||
      iterations > (1 << 20) || status == nullptr || flops == nullptr)
    return ANEMOI_SM100_EINVAL;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  const int ctas = 2 * sms;
  const size_t smem = 2 * kTileBytes + sizeof(PeakShared);
  if (cudaFuncSetAttribute(tensor_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  // elements per 32-byte k-step: 16 fp16, 32 8-bit, 64 4-bit
  const double k_step = kind == ANEMOI_SM100_KIND_F16 ? 16.0 : (kind == ANEMOI_SM100_KIND_NVFP4 ? 64.0 : 32.0);
  *flops = 2.0 * 128.0 * 128.0 * k_step * 8.0 * iterations * ctas;
  tensor_peak_kernel<<<ctas, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(kind, iterations, status);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}
