// Routing: global per-head top-k over the [R][R] fp16 probability map with
// precision assigned by rank, emitted as compact ragged lists of 64-key stages
// per query block.
//
// Reference behaviour (csrc/attention/cuda/sm120/h3_route_precision.cu:111-158,
// 222-369 and anemoi/layers/attention/mpa/routing.py:158-235): pairs are ranked
// by descending probability, ties by ascending flat index row*R+col (the
// reference sorts all pairs with a stable radix sort on the 15-bit magnitude);
// ranks < n16 run in FP16, the next n8 in INT8, the next n4 in NVFP4.  Per row
// the list holds the NVFP4 columns, then INT8, then FP16, each ascending; every
// logical block expands to QB/64 consecutive stages and the prefix stages are
// placed at the front of the phase that carries them.
//
// Here the sort is replaced by selection.  A 32768-bin histogram of the keys of
// a head gives, for each of the three rank boundaries, the key that straddles it
// and how many items of that key fall above it; only items whose key equals a
// straddling key need their position inside the bin, which is their count in
// earlier rows (a per-row tally) plus their count earlier in the same row.
#include <cuda_fp16.h>

#include "records.cuh"

namespace {

constexpr int kBins = 32768;
constexpr int kHistThreads = 512;
constexpr int kRowThreads = 256;

struct RouteScratch {
  int* hist;    // [H][kBins]
  int* thr;     // [H][8]: key0, quota0, key1, quota1, key2, quota2, -, -
  int* eq;      // [H][R][4]: items per row equal to straddling key 0,1,2
  int* cursor;  // [H]
};

__host__ __device__ inline int64_t scratch_ints(int H, int R) {
  return (int64_t)H * (kBins + 8 + 4 * (int64_t)R + 1);
}

__global__ void __launch_bounds__(kHistThreads) hist_kernel(const unsigned short* prob,
                                                            int64_t items, int chunks,
                                                            int* hist) {
  extern __shared__ int local[];
  for (int i = threadIdx.x; i < kBins; i += kHistThreads) local[i] = 0;
  __syncthreads();
  const int head = blockIdx.y;
  const int64_t per = (items + chunks - 1) / chunks;
  const int64_t lo = (int64_t)blockIdx.x * per, hi = min(items, lo + per);
  const unsigned short* src = prob + (int64_t)head * items;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kHistThreads)
    atomicAdd(&local[__ldg(src + i) & 0x7fff], 1);
  __syncthreads();
  int* out = hist + (int64_t)head * kBins;
  for (int i = threadIdx.x; i < kBins; i += kHistThreads)
    if (local[i]) atomicAdd(out + i, local[i]);
}

// One CTA per head: walks the histogram from the largest key down and records,
// for each boundary B, the key whose bin contains rank B and B's offset in it.
__global__ void __launch_bounds__(1024) threshold_kernel(const int* hist, int* thr, int64_t b0,
                                                         int64_t b1, int64_t b2) {
  __shared__ int64_t warp_sum[32];
  __shared__ int result[8];
  const int head = blockIdx.x;
  const int* h = hist + (int64_t)head * kBins;
  // thread t owns keys [hi_key - 31, hi_key], hi_key = kBins - 1 - 32 t
  const int hi_key = kBins - 1 - 32 * threadIdx.x;
  int mine[32];
  int64_t total = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    mine[i] = h[hi_key - i];
    total += mine[i];
  }
  // exclusive prefix over threads (descending keys)
  int64_t incl = total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    int64_t n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  if (lane == 31) warp_sum[warp] = incl;
  if (threadIdx.x < 8) result[threadIdx.x] = threadIdx.x & 1 ? 0 : -1;
  __syncthreads();
  int64_t base = 0;
  for (int w = 0; w < warp; ++w) base += warp_sum[w];
  int64_t above = base + incl - total;
  const int64_t bound[3] = {b0, b1, b2};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int64_t next = above + mine[i];
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      if (mine[i] > 0 && above <= bound[b] && bound[b] < next) {
        result[2 * b] = hi_key - i;
        result[2 * b + 1] = (int)(bound[b] - above);
      }
    }
    above = next;
  }
  __syncthreads();
  if (threadIdx.x < 8) thr[head * 8 + threadIdx.x] = result[threadIdx.x];
}

__global__ void __launch_bounds__(kRowThreads) tally_kernel(const unsigned short* prob, int R,
                                                            const int* thr, int* eq) {
  __shared__ int acc[3];
  const int row = blockIdx.x, head = blockIdx.y;
  if (threadIdx.x < 3) acc[threadIdx.x] = 0;
  __syncthreads();
  const int k0 = thr[head * 8], k1 = thr[head * 8 + 2], k2 = thr[head * 8 + 4];
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;
  int c0 = 0, c1 = 0, c2 = 0;
  for (int j = threadIdx.x; j < R; j += kRowThreads) {
    const int key = __ldg(src + j) & 0x7fff;
    c0 += key == k0;
    c1 += key == k1;
    c2 += key == k2;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    c0 += __shfl_xor_sync(0xffffffffu, c0, off);
    c1 += __shfl_xor_sync(0xffffffffu, c1, off);
    c2 += __shfl_xor_sync(0xffffffffu, c2, off);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&acc[0], c0);
    atomicAdd(&acc[1], c1);
    atomicAdd(&acc[2], c2);
  }
  __syncthreads();
  if (threadIdx.x < 3) eq[((int64_t)head * R + row) * 4 + threadIdx.x] = acc[threadIdx.x];
}

// Ordered rank of a flagged thread inside the CTA: flagged threads of lower
// thread index in this call + `running`; `running` is advanced by the total.
__device__ __forceinline__ int ordered_rank(bool flag, int& running, int* warp_tot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned ballot = __ballot_sync(0xffffffffu, flag);
  __syncthreads();
  if (lane == 0) warp_tot[warp] = __popc(ballot);
  __syncthreads();
  int before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kRowThreads / 32; ++w) {
    const int t = warp_tot[w];
    before += w < warp ? t : 0;
    total += t;
  }
  const int rank = running + before + __popc(ballot & ((1u << lane) - 1u));
  running += total;
  return rank;
}

__global__ void __launch_bounds__(kRowThreads) emit_kernel(
    const unsigned short* prob, int R, const int* thr, const int* eq, int* cursor, int factor,
    int prefix_stages, int prefix_phase, int64_t capacity, int32_t* row_offset,
    int32_t* row_counts, int32_t* stage_ids) {
  extern __shared__ uint8_t code[];  // [R] precision code per column
  __shared__ int warp_tot[kRowThreads / 32];
  __shared__ int pre[3];
  __shared__ int base_s;
  const int row = blockIdx.x, head = blockIdx.y;
  int key_b[3], quota_b[3];
#pragma unroll
  for (int b = 0; b < 3; ++b) {
    key_b[b] = thr[head * 8 + 2 * b];
    quota_b[b] = thr[head * 8 + 2 * b + 1];
  }
  // items of each straddling key in earlier rows
  if (threadIdx.x < 3) pre[threadIdx.x] = 0;
  __syncthreads();
  {
    int s0 = 0, s1 = 0, s2 = 0;
    const int* e = eq + (int64_t)head * R * 4;
    for (int r = threadIdx.x; r < row; r += kRowThreads) {
      s0 += e[r * 4];
      s1 += e[r * 4 + 1];
      s2 += e[r * 4 + 2];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      s0 += __shfl_xor_sync(0xffffffffu, s0, off);
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
      s2 += __shfl_xor_sync(0xffffffffu, s2, off);
    }
    if ((threadIdx.x & 31) == 0) {
      atomicAdd(&pre[0], s0);
      atomicAdd(&pre[1], s1);
      atomicAdd(&pre[2], s2);
    }
  }
  __syncthreads();
  int run[3] = {pre[0], pre[1], pre[2]};
  int count[3] = {0, 0, 0};  // per category 1,2,3 (uniform across the CTA)
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;

  for (int j0 = 0; j0 < R; j0 += kRowThreads) {
    const int j = j0 + threadIdx.x;
    const bool in = j < R;
    const int key = in ? (__ldg(src + j) & 0x7fff) : -2;
    int t[3];
#pragma unroll
    for (int b = 0; b < 3; ++b) t[b] = ordered_rank(in && key == key_b[b], run[b], warp_tot);
    // rank < boundary b  <=>  key above the straddling key, or inside its bin before the quota
    bool below[3];
#pragma unroll
    for (int b = 0; b < 3; ++b) below[b] = key > key_b[b] || (key == key_b[b] && t[b] < quota_b[b]);
    const int c = !in ? 0 : (below[0] ? 3 : (below[1] ? 2 : (below[2] ? 1 : 0)));
    if (in) code[j] = (uint8_t)c;
#pragma unroll
    for (int k = 1; k <= 3; ++k) {
      int dummy = 0;
      (void)ordered_rank(c == k, dummy, warp_tot);
      count[k - 1] += dummy;
    }
  }
  __syncthreads();
  const int p = prefix_phase >= 0 ? prefix_stages : 0;
  const int total = (count[0] + count[1] + count[2]) * factor + p;
  if (threadIdx.x == 0) {
    const int off = total ? atomicAdd(cursor + head, total) : 0;
    base_s = off;
    row_offset[(int64_t)head * R + row] = off;
    int32_t* rc = row_counts + ((int64_t)head * R + row) * 4;
    rc[0] = count[0] * factor + (prefix_phase == 0 ? p : 0);
    rc[1] = count[1] * factor + (prefix_phase == 1 ? p : 0);
    rc[2] = count[2] * factor + (prefix_phase == 2 ? p : 0);
    rc[3] = 0;
  }
  __syncthreads();
  if (total == 0) return;
  if ((int64_t)base_s + total > capacity) return;  // cannot happen with exact budgets
  int32_t* list = stage_ids + (int64_t)head * capacity + base_s;
  // segment starts (in stages) of the three phases
  int seg[3];
  seg[0] = 0;
  seg[1] = count[0] * factor + (prefix_phase == 0 ? p : 0);
  seg[2] = seg[1] + count[1] * factor + (prefix_phase == 1 ? p : 0);
  if (prefix_phase >= 0)
    for (int s = threadIdx.x; s < p; s += kRowThreads) list[seg[prefix_phase] + s] = s;
  int placed[3] = {0, 0, 0};
  for (int j0 = 0; j0 < R; j0 += kRowThreads) {
    const int j = j0 + threadIdx.x;
    const int c = j < R ? code[j] : 0;
#pragma unroll
    for (int k = 1; k <= 3; ++k) {
      const int pos = ordered_rank(c == k, placed[k - 1], warp_tot);
      if (c == k) {
        const int at = seg[k - 1] + (prefix_phase == k - 1 ? p : 0) + pos * factor;
        for (int e = 0; e < factor; ++e) list[at + e] = prefix_stages + j * factor + e;
      }
    }
  }
}

// Launch order of a head's query blocks for the attention kernel: longest list first (ties by
// block index), written as block + 1 into the fourth entry of row_counts, slot = position.
// The last CTAs of a launch are then the short ones, which shortens the tail during which SMs
// run out of work.  Blocks are ranked by counting (R^2 / threads comparisons per thread).
constexpr int kOrderMaxBlocks = 4096;
__global__ void __launch_bounds__(1024) order_kernel(int R, int32_t* row_counts) {
  extern __shared__ int total[];
  const int head = blockIdx.x;
  int32_t* rc = row_counts + (int64_t)head * R * 4;
  for (int i = threadIdx.x; i < R; i += blockDim.x) total[i] = rc[i * 4] + rc[i * 4 + 1] + rc[i * 4 + 2];
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int mine = total[i];
    int rank = 0;
    for (int j = 0; j < R; ++j) rank += (total[j] > mine) || (total[j] == mine && j < i);
    rc[rank * 4 + 3] = i + 1;
  }
}

}  // namespace

extern "C" int64_t anemoi_sm100_route_scratch_bytes(const anemoi_sm100_shape* shape) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  return scratch_ints(shape->heads, shape->video_blocks) * 4;
}

extern "C" int64_t anemoi_sm100_route_list_capacity(const anemoi_sm100_shape* shape, int64_t n16,
                                                    int64_t n8, int64_t n4, int prefix_phase) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  const int64_t f = shape->query_block / 64;
  const int64_t p = prefix_phase >= 0 ? rec::prefix_stages(*shape) : 0;
  return (n16 + n8 + n4) * f + (int64_t)shape->video_blocks * p;
}

extern "C" int anemoi_sm100_route(const anemoi_sm100_shape* shape, const void* probability,
                                  int64_t n16, int64_t n8, int64_t n4, int prefix_phase,
                                  void* scratch, int64_t scratch_bytes, int32_t* row_offset,
                                  int32_t* row_counts, int32_t* stage_ids, int64_t list_capacity,
                                  void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !probability || !scratch || !row_offset ||
      !row_counts || !stage_ids)
    return ANEMOI_SM100_EINVAL;
  const int H = shape->heads, R = shape->video_blocks;
  const int64_t items = (int64_t)R * R;
  if (n16 < 0 || n8 < 0 || n4 < 0 || n16 + n8 + n4 > items || n16 + n8 + n4 <= 0)
    return ANEMOI_SM100_EINVAL;
  if (prefix_phase < -1 || prefix_phase > 2) return ANEMOI_SM100_EINVAL;
  if (prefix_phase >= 0 && shape->prefix_tokens == 0) prefix_phase = -1;
  if (scratch_bytes < scratch_ints(H, R) * 4) return ANEMOI_SM100_EINVAL;
  if (list_capacity < anemoi_sm100_route_list_capacity(shape, n16, n8, n4, prefix_phase))
    return ANEMOI_SM100_EINVAL;
  if (R > 65535 || items * H >= (1ll << 40)) return ANEMOI_SM100_ELIMIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RouteScratch sc;
  sc.hist = static_cast<int*>(scratch);
  sc.thr = sc.hist + (int64_t)H * kBins;
  sc.eq = sc.thr + (int64_t)H * 8;
  sc.cursor = sc.eq + (int64_t)H * R * 4;
  if (cudaMemsetAsync(sc.hist, 0, (size_t)H * kBins * 4, st) != cudaSuccess ||
      cudaMemsetAsync(sc.cursor, 0, (size_t)H * 4, st) != cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  const unsigned short* prob = static_cast<const unsigned short*>(probability);
  // Function attributes belong to a device: they are set at every call (two cheap host-side
  // driver calls), so a process that routes on several GPUs, or from several host threads,
  // never launches these kernels without the opt-in for their dynamic shared memory.
  if (cudaFuncSetAttribute(hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBins * 4) !=
          cudaSuccess ||
      cudaFuncSetAttribute(emit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536) !=
          cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  const int chunks = (int)max((int64_t)1, min((int64_t)16, items / 32768));
  hist_kernel<<<dim3(chunks, H), kHistThreads, kBins * 4, st>>>(prob, items, chunks, sc.hist);
  threshold_kernel<<<H, 1024, 0, st>>>(sc.hist, sc.thr, n16, n16 + n8, n16 + n8 + n4);
  tally_kernel<<<dim3(R, H), kRowThreads, 0, st>>>(prob, R, sc.thr, sc.eq);
  emit_kernel<<<dim3(R, H), kRowThreads, (size_t)((R + 15) & ~15), st>>>(
      prob, R, sc.thr, sc.eq, sc.cursor, shape->query_block / 64, rec::prefix_stages(*shape),
      prefix_phase, list_capacity, row_offset, row_counts, stage_ids);
  // very large block counts keep the identity order (the fourth entries stay 0)
  if (R <= kOrderMaxBlocks) order_kernel<<<H, 1024, (size_t)R * 4, st>>>(R, row_counts);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

// ------------------------------------------------------------------------------------------
// Routing without any allocation by the caller
// ------------------------------------------------------------------------------------------
// Some hosts of this library cannot hand it scratch memory: a serving loop whose memory
// pool is frozen after start-up, or code that must not call cudaMalloc because it runs
// between other streams' work and cannot afford the implicit device synchronisation.
// For them the scratch of anemoi_sm100_route lives in this file-scope device array.
// Every GPU that loads the library holds these 8 MiB until the process exits.
constexpr int64_t kStaticScratchInts = 2 * 1024 * 1024;  // 8 MiB of int32
static __device__ __align__(256) int g_route_scratch[kStaticScratchInts];

namespace {
constexpr int kMaxDevices = 64;
int* g_route_scratch_address[kMaxDevices];  // device address of the array, per device ordinal
}  // namespace

extern "C" int64_t anemoi_sm100_route_static_max_bytes(void) { return kStaticScratchInts * 4; }

extern "C" int anemoi_sm100_route_static(const anemoi_sm100_shape* shape, const void* probability,
                                         int64_t n16, int64_t n8, int64_t n4, int prefix_phase,
                                         int32_t* row_offset, int32_t* row_counts,
                                         int32_t* stage_ids, int64_t list_capacity,
                                         void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  const int64_t need = scratch_ints(shape->heads, shape->video_blocks);
  if (need > kStaticScratchInts) return ANEMOI_SM100_ELIMIT;  // heads*(32777 + 4*blocks) ints
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return ANEMOI_SM100_ELAUNCH;
  // In host code the array's name is only a stand-in for the symbol, not a device address.
  // The address is looked up once per device, with that device current (the first call on
  // a device does it, so make that call before any stream capture), and then reused.
  int* scratch = g_route_scratch_address[device];
  if (scratch == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_route_scratch) != cudaSuccess ||
        scratch == nullptr)
      return ANEMOI_SM100_ELAUNCH;
    g_route_scratch_address[device] = scratch;
  }
  // Same kernels as anemoi_sm100_route; the bins and cursors that must start at zero are
  // cleared there on `stream` at every call, the rest is overwritten before it is read.
  return anemoi_sm100_route(shape, probability, n16, n8, n4, prefix_phase, scratch, need * 4,
                            row_offset, row_counts, stage_ids, list_capacity, stream);
}
