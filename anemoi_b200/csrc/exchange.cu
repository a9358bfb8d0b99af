// Ulysses sequence<->head exchange by direct stores into the peers' memory (one node, <= 8 ranks).
//
// Every rank owns one exchange region (cudaMalloc, exported with a CUDA IPC handle and mapped by
// the other ranks of the node).  The relayout kernels store each 16-byte vector straight where
// an all-to-all would have delivered it - over NVLink for the other ranks, locally for the own
// part - so the collective, its send buffer and the merge pass disappear.  When the last block
// of a push has stored its part, it writes the call's epoch into a flag word of every
// destination; the destination's next kernel in stream order is a one-warp wait on those flags.
// Only plain st.global / ld.acquire touch peer memory: no bulk or tensor copy, no multicast.
//
// Every wait has a limit (%globaltimer); a wait that runs out records 70 + the late rank in
// the device status word and returns, so the stream drains and the host can read the failure.
//
// This replaces pack_qkv_destination_major + all_to_all_single and all_to_all_single +
// merge_heads of the reference's custom Ulysses path
// (anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/ulysses_custom.py:107-165,
// relayout.py:83-162).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/anemoi_sm100.h"
#include "norm_rope.cuh"

namespace {

constexpr int kMaxRanks = 8;

struct PeerTable {
  uint16_t* data[kMaxRanks];   // per rank: the destination buffer as mapped into this process
  uint32_t* flags[kMaxRanks];  // per rank: its flag words (one per source rank)
  int64_t first[kMaxRanks + 1];  // first row of every rank's sequence shard; [ranks] = all rows
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Called by every thread after its stores.  The last block to finish publishes the epoch to
// every destination; the fences make all blocks' stores visible, system-wide, before the flag.
__device__ __forceinline__ void publish(const PeerTable& peers, int self, int ranks, uint32_t epoch,
                                        unsigned int* blocks_done) {
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = atomicAdd(blocks_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence_system();
  if (threadIdx.x < ranks) {
    uint32_t* flag = peers.flags[threadIdx.x] + self;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
  }
  if (threadIdx.x == 0) *blocks_done = 0;   // ready for the next launch on this stream
}

// q,k,v [rows][heads][D] of this rank's rows -> on rank `dest`: recv [all rows][heads_local][3*D]
// at rows first[self] + row.  Consecutive threads store consecutive 16-byte vectors of one row.
__global__ void __launch_bounds__(256) push_qkv_kernel(const uint16_t* q, const uint16_t* k,
                                                       const uint16_t* v, PeerTable peers, int self,
                                                       int ranks, int64_t rows, int heads_local, int d8,
                                                       int64_t total, int64_t qs_row, int64_t qs_head,
                                                       int64_t ks_row, int64_t ks_head,
                                                       int64_t vs_row, int64_t vs_head,
                                                       uint32_t epoch, unsigned int* blocks_done) {
  const int64_t row0 = peers.first[self];
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * 256) {
    const int c8 = (int)(idx % d8);
    int64_t t = idx / d8;
    const int which = (int)(t % 3);
    t /= 3;
    const int lh = (int)(t % heads_local);
    t /= heads_local;
    const int64_t row = t % rows;
    // destinations in the order self+1, self+2, ..., self: at any moment the ranks of the node
    // store to different destinations, instead of all into rank 0 first
    int dest = self + 1 + (int)(t / rows);
    dest -= dest >= ranks ? ranks : 0;
    const int gh = dest * heads_local + lh;
    const uint16_t* src = which == 0 ? q + row * qs_row + gh * qs_head
                        : which == 1 ? k + row * ks_row + gh * ks_head
                                     : v + row * vs_row + gh * vs_head;
    uint16_t* dst = peers.data[dest] +
                    ((((row0 + row) * heads_local + lh) * 3 + which) * (int64_t)d8 + c8) * 8;
    *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src) + c8);
  }
  publish(peers, self, ranks, epoch, blocks_done);
}

// The same exchange with the producer step in it: q and k get the per-head RMS norm with weight
// and the partial rotary embedding (norm_rope.cuh: the arithmetic of the stand-alone producer
// kernel, bit for bit) on their way from the projection output to the peers, v passes through.
// The normalised q and k are never written to this rank's memory: the in-place producer pass
// (one read and one write of q and k) disappears.  The D/8 lanes of a (row, head) are
// consecutive threads; whole warps stay in the loop because the lanes of a row shuffle.
template <typename T, int D>
__global__ void __launch_bounds__(256) push_qkv_norm_kernel(
    const uint16_t* q, const uint16_t* k, const uint16_t* v, const T* q_weight, const T* k_weight,
    const float* cos_table, const float* sin_table, int rotary_dim, float eps, PeerTable peers,
    int self, int ranks, int64_t rows, int heads_local, int64_t total, int64_t qs_row,
    int64_t qs_head, int64_t ks_row, int64_t ks_head, int64_t vs_row, int64_t vs_head,
    uint32_t epoch, unsigned int* blocks_done) {
  constexpr int d8 = D / 8;
  const int64_t row0 = peers.first[self];
  const int lane_in_warp = threadIdx.x & 31;
  for (int64_t base = (int64_t)blockIdx.x * 256 + (threadIdx.x - lane_in_warp); base < total;
       base += (int64_t)gridDim.x * 256) {
    const int64_t idx = base + lane_in_warp;
    const bool live = idx < total;
    const int c8 = (int)(idx % d8);
    int64_t t = idx / d8;
    const int which = (int)(t % 3);
    t /= 3;
    const int lh = (int)(t % heads_local);
    t /= heads_local;
    const int64_t row = live ? t % rows : 0;
    int dest = self + 1 + (live ? (int)(t / rows) : 0);
    dest -= dest >= ranks ? ranks : 0;
    const int gh = dest * heads_local + lh;
    const uint16_t* src = which == 0 ? q + row * qs_row + gh * qs_head
                        : which == 1 ? k + row * ks_row + gh * ks_head
                                     : v + row * vs_row + gh * vs_head;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = __ldg(reinterpret_cast<const uint4*>(src) + c8);
    // q and k rows go through the producer arithmetic (every lane calls: the row's lanes shuffle)
    const uint4 done = nr::norm_rope8<T, D>(raw, which == 1 ? k_weight : q_weight,
                                            cos_table + row * rotary_dim, sin_table + row * rotary_dim,
                                            rotary_dim, eps, c8, live && which < 2);
    if (live) {
      uint16_t* dst = peers.data[dest] +
                      ((((row0 + row) * heads_local + lh) * 3 + which) * (int64_t)d8 + c8) * 8;
      *reinterpret_cast<uint4*>(dst) = which < 2 ? done : raw;
    }
  }
  publish(peers, self, ranks, epoch, blocks_done);
}

// out_heads [all rows][heads_local][D] (this rank's heads, every row) -> on the rank that owns
// a row: out [its rows][ranks*heads_local][D] at heads self*heads_local + (0..heads_local)
__global__ void __launch_bounds__(256) push_out_kernel(const uint16_t* out_heads, PeerTable peers,
                                                       int self, int ranks, int heads_local, int d8,
                                                       int64_t total, uint32_t epoch,
                                                       unsigned int* blocks_done) {
  const int inner8 = heads_local * d8;
  const int64_t total_rows = peers.first[ranks];
  const int64_t row_shift = self + 1 < ranks ? peers.first[self + 1] : 0;
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * 256) {
    const int tail = (int)(idx % inner8);
    // rows starting with the next rank's shard (and wrapping), for the same reason
    int64_t row = idx / inner8 + row_shift;
    row -= row >= total_rows ? total_rows : 0;
    int owner = 0;
#pragma unroll
    for (int r = 1; r < kMaxRanks; ++r) owner += (r < ranks && row >= peers.first[r]) ? 1 : 0;
    uint16_t* dst = peers.data[owner] +
                    (((row - peers.first[owner]) * ranks + self) * (int64_t)inner8 + tail) * 8;
    *reinterpret_cast<uint4*>(dst) =
        __ldg(reinterpret_cast<const uint4*>(out_heads) + row * inner8 + tail);
  }
  publish(peers, self, ranks, epoch, blocks_done);
}

// One warp; lane r waits until rank r's flag has reached the epoch.
__global__ void wait_flags_kernel(const uint32_t* flags, int ranks, uint32_t epoch, uint64_t limit_ns,
                                  int32_t* status) {
  const int r = threadIdx.x;
  if (r >= ranks) return;
  if (status && *(volatile int32_t*)status != 0) return;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
    if ((int32_t)(seen - epoch) >= 0) return;
    if (globaltimer_ns() - t0 > limit_ns) break;
    __nanosleep(200);
  }
  if (status) atomicCAS(status, 0, 70 + r);
}

// `own_rows`: the buffers hold only their rank's rows, so a rank without rows may have none
int fill(PeerTable& t, void* const* data, void* const* flags, const int64_t* first, int ranks,
         bool own_rows) {
  for (int r = 0; r < ranks; ++r) {
    if (!flags[r] || first[r + 1] < first[r]) return ANEMOI_SM100_EINVAL;
    if (!data[r] && !(own_rows && first[r + 1] == first[r])) return ANEMOI_SM100_EINVAL;
    t.data[r] = static_cast<uint16_t*>(data[r]);
    t.flags[r] = static_cast<uint32_t*>(flags[r]);
    t.first[r] = first[r];
  }
  t.first[ranks] = first[ranks];
  return ANEMOI_SM100_OK;
}

}  // namespace

extern "C" int anemoi_sm100_peer_alloc(int64_t bytes, void** ptr, void* handle64) {
  if (bytes <= 0 || !ptr || !handle64) return ANEMOI_SM100_EINVAL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return ANEMOI_SM100_ELAUNCH;
  if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess ||
      cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p) != cudaSuccess) {
    cudaFree(p);
    cudaGetLastError();
    return ANEMOI_SM100_ELAUNCH;
  }
  cudaDeviceSynchronize();
  *ptr = p;
  return ANEMOI_SM100_OK;
}

extern "C" int anemoi_sm100_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return ANEMOI_SM100_EINVAL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof h);
  if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return ANEMOI_SM100_ELAUNCH;
  }
  return ANEMOI_SM100_OK;
}

extern "C" int anemoi_sm100_peer_close(void* ptr) {
  if (!ptr) return ANEMOI_SM100_EINVAL;
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_peer_free(void* ptr) {
  if (!ptr) return ANEMOI_SM100_EINVAL;
  return cudaFree(ptr) == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_push_qkv(const void* q, const void* k, const void* v,
                                     void* const* peer_recv, void* const* peer_flags,
                                     const int64_t* first_rows, int32_t self, int32_t ranks,
                                     int32_t heads, int32_t head_dim, const int64_t* strides,
                                     uint32_t epoch, void* blocks_done, void* stream) {
  if (!peer_recv || !peer_flags || !first_rows || !strides || !blocks_done || ranks <= 0 || ranks > kMaxRanks || self < 0 || self >= ranks || heads <= 0 || heads % ranks ||
      head_dim <= 0 || head_dim % 8)
    return ANEMOI_SM100_EINVAL;
  for (int i = 0; i < 6; ++i)
    if (strides[i] % 8) return ANEMOI_SM100_EINVAL;
  PeerTable t{};
  if (int rc = fill(t, peer_recv, peer_flags, first_rows, ranks, false)) return rc;
  const int64_t rows = first_rows[self + 1] - first_rows[self];
  if (rows > 0 && (!q || !k || !v)) return ANEMOI_SM100_EINVAL;   // a rank without rows has no tensors
  const int heads_local = heads / ranks, d8 = head_dim / 8;
  const int64_t total = (int64_t)ranks * rows * heads_local * 3 * d8;
  // a rank without rows still has to publish its epoch: one block, no stores
  const int blocks = (int)max((int64_t)1, min((total + 255) / 256, (int64_t)(148 * 16)));
  push_qkv_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(k),
      static_cast<const uint16_t*>(v), t, self, ranks, max(rows, (int64_t)1), heads_local, d8, total,
      strides[0], strides[1], strides[2], strides[3], strides[4], strides[5], epoch,
      static_cast<unsigned int*>(blocks_done));
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_push_out(const void* out_heads, void* const* peer_out,
                                     void* const* peer_flags, const int64_t* first_rows,
                                     int32_t self, int32_t ranks, int32_t heads_local,
                                     int32_t head_dim, uint32_t epoch, void* blocks_done,
                                     void* stream) {
  if (!out_heads || !peer_out || !peer_flags || !first_rows || !blocks_done || ranks <= 0 ||
      ranks > kMaxRanks || self < 0 || self >= ranks || heads_local <= 0 || head_dim <= 0 ||
      head_dim % 8)
    return ANEMOI_SM100_EINVAL;
  PeerTable t{};
  if (int rc = fill(t, peer_out, peer_flags, first_rows, ranks, true)) return rc;
  const int d8 = head_dim / 8;
  const int64_t total = first_rows[ranks] * heads_local * d8;
  const int blocks = (int)max((int64_t)1, min((total + 255) / 256, (int64_t)(148 * 16)));
  push_out_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(out_heads), t, self, ranks, heads_local, d8, total, epoch,
      static_cast<unsigned int*>(blocks_done));
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_wait_flags(const void* flags, int32_t ranks, uint32_t epoch,
                                       uint64_t limit_ns, int32_t* status, void* stream) {
  if (!flags || ranks <= 0 || ranks > kMaxRanks || limit_ns == 0 || limit_ns > 10000000000ull)
    return ANEMOI_SM100_EINVAL;
  wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(flags), ranks, epoch, limit_ns, status);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

namespace {
template <typename T, int D>
void launch_norm(const void* q, const void* k, const void* v, const void* qw, const void* kw,
                 const float* c, const float* sn, int rotary, float eps, const PeerTable& t, int self,
                 int ranks, int64_t rows, int heads_local, int64_t total, const int64_t* strides,
                 uint32_t epoch, void* blocks_done, cudaStream_t st) {
  const int blocks = (int)max((int64_t)1, min((total + 255) / 256, (int64_t)(148 * 16)));
  push_qkv_norm_kernel<T, D><<<blocks, 256, 0, st>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(k), static_cast<const uint16_t*>(v),
      static_cast<const T*>(qw), static_cast<const T*>(kw), c, sn, rotary, eps, t, self, ranks,
      max(rows, (int64_t)1), heads_local, total, strides[0], strides[1], strides[2], strides[3],
      strides[4], strides[5], epoch, static_cast<unsigned int*>(blocks_done));
}
}  // namespace

extern "C" int anemoi_sm100_push_qkv_norm(const void* q, const void* k, const void* v,
                                          const void* q_weight, const void* k_weight,
                                          const float* cos_table, const float* sin_table,
                                          int32_t rotary_dim, float eps, int32_t is_bf16,
                                          void* const* peer_recv, void* const* peer_flags,
                                          const int64_t* first_rows, int32_t self, int32_t ranks,
                                          int32_t heads, int32_t head_dim, const int64_t* strides,
                                          uint32_t epoch, void* blocks_done, void* stream) {
  if (!peer_recv || !peer_flags || !first_rows || !strides || !blocks_done || !q_weight ||
      !k_weight || ranks <= 0 || ranks > kMaxRanks || self < 0 || self >= ranks || heads <= 0 ||
      heads % ranks || (head_dim != 64 && head_dim != 128))
    return ANEMOI_SM100_EINVAL;
  if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 16 || !(eps >= 0.0f))
    return ANEMOI_SM100_EINVAL;
  for (int i = 0; i < 6; ++i)
    if (strides[i] % 8) return ANEMOI_SM100_EINVAL;
  PeerTable t{};
  if (int rc = fill(t, peer_recv, peer_flags, first_rows, ranks, false)) return rc;
  const int64_t rows = first_rows[self + 1] - first_rows[self];
  // a rank without rows has no tensors and no table rows
  if (rows > 0 && (!q || !k || !v)) return ANEMOI_SM100_EINVAL;
  if (rows > 0 && rotary_dim > 0 && (!cos_table || !sin_table)) return ANEMOI_SM100_EINVAL;
  const int heads_local = heads / ranks;
  const int64_t total = (int64_t)ranks * rows * heads_local * 3 * (head_dim / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define ANEMOI_LAUNCH_NORM(T, D)                                                                  \
  launch_norm<T, D>(q, k, v, q_weight, k_weight, cos_table, sin_table, rotary_dim, eps, t, self,  \
                    ranks, rows, heads_local, total, strides, epoch, blocks_done, st)
  if (is_bf16) {
    if (head_dim == 64) ANEMOI_LAUNCH_NORM(__nv_bfloat16, 64); else ANEMOI_LAUNCH_NORM(__nv_bfloat16, 128);
  } else {
    if (head_dim == 64) ANEMOI_LAUNCH_NORM(__half, 64); else ANEMOI_LAUNCH_NORM(__half, 128);
  }
#undef ANEMOI_LAUNCH_NORM
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}
