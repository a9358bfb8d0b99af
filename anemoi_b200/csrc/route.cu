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
// and how many items of that key fall above it (the quota).  One pass per row then
// counts the keys above and equal to each straddling key; a per-head scan over the
// rows turns the equal-counts into each row's position inside the straddling bins,
// from which the row's stages per phase, its list offset (an exclusive scan: the
// layout is the same at every call) and the launch order follow without touching
// the map again; a last pass per row writes the lists.  The per-row passes use one
// warp per row: ranks inside a row come from ballots, no block-wide barrier.
#include <climits>
#include <cuda_fp16.h>

#include "records.cuh"

namespace {

constexpr int kBins = 32768;
constexpr int kHistThreads = 512;
constexpr int kRowWarps = 8;  // rows per CTA in the per-row passes, one warp each
constexpr int kStat = 6;      // ints per row: keys above boundary 0,1,2; keys equal to its key 0,1,2

struct RouteScratch {
  int* hist;  // [H][kBins]
  int* thr;   // [H][8]: key0, quota0, key1, quota1, key2, quota2, -, -
  int* stat;  // [H][R][kStat]; the equal-counts become exclusive prefixes over the rows
};

__host__ __device__ inline int64_t scratch_ints(int H, int R) {
  return (int64_t)H * (kBins + 8 + kStat * (int64_t)R);
}

// A CTA counts the keys of one half of the key range (blockIdx.z) in its chunk of a head: 64 KB of
// shared-memory bins, so that it fits on an SM beside one CTA of the prefix rows' attention launch,
// which runs on a side stream at the same time (with all 128 KB of bins in one CTA the histogram
// waited for those long CTAs to retire).  The map is L2-resident; reading it twice costs little.
constexpr int kHalfBins = kBins / 2;
__global__ void __launch_bounds__(kHistThreads) hist_kernel(const unsigned short* prob,
                                                            int64_t items, int chunks,
                                                            int* hist) {
  extern __shared__ int local[];
  for (int i = threadIdx.x; i < kHalfBins; i += kHistThreads) local[i] = 0;
  __syncthreads();
  const int head = blockIdx.y, half = blockIdx.z;
  const int64_t per = (items + chunks - 1) / chunks;
  const int64_t lo = (int64_t)blockIdx.x * per, hi = min(items, lo + per);
  const unsigned short* src = prob + (int64_t)head * items;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kHistThreads) {
    const int key = __ldg(src + i) & 0x7fff;
    if ((key >> 14) == half) atomicAdd(&local[key & (kHalfBins - 1)], 1);
  }
  __syncthreads();
  int* out = hist + (int64_t)head * kBins + half * kHalfBins;
  for (int i = threadIdx.x; i < kHalfBins; i += kHistThreads)
    if (local[i]) atomicAdd(out + i, local[i]);
}

// Exclusive prefix of `v` over the threads of a 1024-thread CTA; `total` gets the sum.
// `warp_sum` is shared scratch of 32 entries; the call ends with the scratch free again.
__device__ __forceinline__ long long block_exclusive(long long v, long long* warp_sum,
                                                     long long& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const long long n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  if (lane == 31) warp_sum[warp] = incl;
  __syncthreads();
  long long base = 0, all = 0;
#pragma unroll
  for (int w = 0; w < 32; ++w) {
    const long long t = warp_sum[w];
    base += w < warp ? t : 0;
    all += t;
  }
  __syncthreads();
  total = all;
  return base + incl - v;
}

// One CTA per head: finds, for each boundary B, the key whose bin contains rank B (keys
// ranked from the largest down) and B's offset inside that bin.  Two levels: sums of 32-bin
// blocks (coalesced reads, one warp reduction each), a scan over the 1024 blocks, then one
// warp per boundary resolves the bin inside the block that straddles it.
// `sub` (optional): a second histogram that is subtracted bin by bin (the anchored variant ranks
// the items that are not anchors).  The results go to thr[head * thr_stride + thr_first ..].
__global__ void __launch_bounds__(1024) threshold_kernel(const int* hist, const int* sub, int* thr,
                                                         int thr_stride, int thr_first, int64_t b0,
                                                         int64_t b1, int64_t b2) {
  __shared__ long long warp_sum[32];
  __shared__ int block_sum[1024];
  __shared__ int hit_block[3];
  __shared__ long long hit_off[3];
  const int head = blockIdx.x;
  const int* h = hist + (int64_t)head * kBins;
  const int* hs = sub ? sub + (int64_t)head * kBins : nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int mine = 0;
#pragma unroll 4
  for (int i = 0; i < 32; ++i) {
    const int bin = (warp * 32 + i) * 32 + lane;
    const int sum = __reduce_add_sync(0xffffffffu, h[bin] - (hs ? hs[bin] : 0));
    if (lane == i) mine = sum;
  }
  block_sum[threadIdx.x] = mine;
  if (threadIdx.x < 3) hit_block[threadIdx.x] = -1;
  __syncthreads();
  // thread t owns block 1023 - t: blocks in descending key order
  const int blk = 1023 - threadIdx.x;
  const long long total = block_sum[blk];
  long long all;
  const long long above = block_exclusive(total, warp_sum, all);
  const long long bound[3] = {b0, b1, b2};
#pragma unroll
  for (int b = 0; b < 3; ++b)
    if (total > 0 && above <= bound[b] && bound[b] < above + total) {
      hit_block[b] = blk;
      hit_off[b] = bound[b] - above;
    }
  __syncthreads();
  if (warp < 3) {
    int key = -1, quota = 0;  // boundary at or past the last item: every key lies above it
    const int hb = hit_block[warp];
    if (hb >= 0) {
      const int bin = hb * 32 + 31 - lane;  // descending inside the block
      const int n = h[bin] - (hs ? hs[bin] : 0);
      int incl = n;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int m = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += m;
      }
      const long long off = hit_off[warp];
      const bool here = n > 0 && incl - n <= off && off < incl;
      const unsigned who = __ballot_sync(0xffffffffu, here);
      const int src = __ffs(who) - 1;
      key = __shfl_sync(0xffffffffu, bin, src);
      quota = __shfl_sync(0xffffffffu, (int)(off - (incl - n)), src);
    }
    if (lane == 0) {
      thr[head * thr_stride + thr_first + 2 * warp] = key;
      thr[head * thr_stride + thr_first + 2 * warp + 1] = quota;
    }
  }
}

// One warp per row: keys above each straddling key, keys equal to it.
__global__ void __launch_bounds__(kRowWarps * 32) rowstat_kernel(const unsigned short* prob, int R,
                                                                 const int* thr, int* stat) {
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5), head = blockIdx.y;
  if (row >= R) return;
  const int lane = threadIdx.x & 31;
  const int k0 = thr[head * 8], k1 = thr[head * 8 + 2], k2 = thr[head * 8 + 4];
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;
  int g0 = 0, g1 = 0, g2 = 0, e0 = 0, e1 = 0, e2 = 0;
  for (int j = lane; j < R; j += 32) {
    const int key = __ldg(src + j) & 0x7fff;
    g0 += key > k0;
    g1 += key > k1;
    g2 += key > k2;
    e0 += key == k0;
    e1 += key == k1;
    e2 += key == k2;
  }
  g0 = __reduce_add_sync(0xffffffffu, g0);
  g1 = __reduce_add_sync(0xffffffffu, g1);
  g2 = __reduce_add_sync(0xffffffffu, g2);
  e0 = __reduce_add_sync(0xffffffffu, e0);
  e1 = __reduce_add_sync(0xffffffffu, e1);
  e2 = __reduce_add_sync(0xffffffffu, e2);
  if (lane < kStat) {
    const int v = lane == 0 ? g0 : lane == 1 ? g1 : lane == 2 ? g2 : lane == 3 ? e0 : lane == 4 ? e1 : e2;
    stat[((int64_t)head * R + row) * kStat + lane] = v;
  }
}

// One CTA per head, rows in chunks of 1024: position of every row inside the straddling bins
// (exclusive scan of the equal-counts), hence its stages per phase, and its list offset
// (exclusive scan of the totals).  Then the launch order of the head's query blocks for the
// attention kernel: longest list first (ties by block index), written as block + 1 into the
// fourth entry of row_counts, slot = position; the last CTAs of a launch are then the short
// ones, which shortens the tail during which SMs run out of work.  Blocks are ranked by
// counting (R^2 / threads comparisons per thread); very large block counts keep the identity
// order (the fourth entries stay 0).
constexpr int kOrderMaxBlocks = 4096;
__global__ void __launch_bounds__(1024) headscan_kernel(int R, const int* thr, int* stat, int factor,
                                                        int prefix_stages, int prefix_phase,
                                                        int32_t* row_offset, int32_t* row_counts) {
  __shared__ long long warp_sum[32];
  __shared__ int total_s[kOrderMaxBlocks];
  const int head = blockIdx.x;
  int quota[3];
#pragma unroll
  for (int b = 0; b < 3; ++b) quota[b] = thr[head * 8 + 2 * b + 1];
  const int p = prefix_phase >= 0 ? prefix_stages : 0;
  long long carry[4] = {0, 0, 0, 0};  // equal-counts of earlier rows (3), stages of earlier rows
  for (int r0 = 0; r0 < R; r0 += 1024) {
    const int row = r0 + threadIdx.x;
    const bool in = row < R;
    int* st = stat + ((int64_t)head * R + row) * kStat;
    int below[3];
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      const int eq = in ? st[3 + b] : 0;
      long long all;
      const long long pre = carry[b] + block_exclusive(eq, warp_sum, all);
      carry[b] += all;
      // items of the straddling key in this row that still fall above the boundary
      const long long room = (long long)quota[b] - pre;
      const int take = (int)max(0ll, min((long long)eq, room));
      below[b] = in ? st[b] + take : 0;
      if (in) st[3 + b] = (int)pre;
    }
    int n[3];
    n[0] = (below[2] - below[1]) * factor + (prefix_phase == 0 ? p : 0);  // NVFP4
    n[1] = (below[1] - below[0]) * factor + (prefix_phase == 1 ? p : 0);  // INT8
    n[2] = below[0] * factor + (prefix_phase == 2 ? p : 0);               // FP16
    const int total = in ? n[0] + n[1] + n[2] : 0;
    long long all;
    const long long off = carry[3] + block_exclusive(total, warp_sum, all);
    carry[3] += all;
    if (in) {
      row_offset[(int64_t)head * R + row] = (int32_t)off;
      int32_t* rc = row_counts + ((int64_t)head * R + row) * 4;
      rc[0] = n[0];
      rc[1] = n[1];
      rc[2] = n[2];
      rc[3] = 0;
      if (row < kOrderMaxBlocks) total_s[row] = total;
    }
  }
  if (R > kOrderMaxBlocks) return;
  __syncthreads();
  int32_t* rc = row_counts + (int64_t)head * R * 4;
  for (int i = threadIdx.x; i < R; i += 1024) {
    const int mine = total_s[i];
    int rank = 0;
    for (int j = 0; j < R; ++j) rank += (total_s[j] > mine) || (total_s[j] == mine && j < i);
    rc[rank * 4 + 3] = i + 1;
  }
}

// One warp per row writes the row's list: NVFP4 columns, INT8 columns, FP16 columns, each
// ascending, every logical block expanded to `factor` stages, prefix stages at the front of
// the phase that carries them.
__global__ void __launch_bounds__(kRowWarps * 32) emit_kernel(
    const unsigned short* prob, int R, const int* thr, const int* stat, int factor,
    int prefix_stages, int prefix_phase, int64_t capacity, const int32_t* row_offset,
    const int32_t* row_counts, int32_t* stage_ids) {
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5), head = blockIdx.y;
  if (row >= R) return;
  const int lane = threadIdx.x & 31;
  const unsigned lower = (1u << lane) - 1u;
  int key_b[3], quota_b[3], run[3];
  const int* st = stat + ((int64_t)head * R + row) * kStat;
#pragma unroll
  for (int b = 0; b < 3; ++b) {
    key_b[b] = thr[head * 8 + 2 * b];
    quota_b[b] = thr[head * 8 + 2 * b + 1];
    run[b] = st[3 + b];  // items of the straddling key in earlier rows
  }
  const int32_t* rc = row_counts + ((int64_t)head * R + row) * 4;
  const int n0 = rc[0], n1 = rc[1], n2 = rc[2];
  const int total = n0 + n1 + n2;
  if (total == 0) return;
  const int64_t base = row_offset[(int64_t)head * R + row];
  if (base + total > capacity) return;  // cannot happen with exact budgets
  int32_t* list = stage_ids + (int64_t)head * capacity + base;
  const int p = prefix_phase >= 0 ? prefix_stages : 0;
  // where the video stages of each phase start
  int at[3] = {prefix_phase == 0 ? p : 0, n0 + (prefix_phase == 1 ? p : 0),
               n0 + n1 + (prefix_phase == 2 ? p : 0)};
  if (prefix_phase >= 0) {
    const int seg = prefix_phase == 0 ? 0 : (prefix_phase == 1 ? n0 : n0 + n1);
    for (int s = lane; s < p; s += 32) list[seg + s] = s;
  }
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;
  for (int j0 = 0; j0 < R; j0 += 32) {
    const int j = j0 + lane;
    const bool in = j < R;
    const int key = in ? (__ldg(src + j) & 0x7fff) : -2;
    // rank < boundary b  <=>  key above the straddling key, or inside its bin before the quota
    bool below[3];
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      const bool tie = in && key == key_b[b];
      const unsigned ties = __ballot_sync(0xffffffffu, tie);
      below[b] = key > key_b[b] || (tie && run[b] + __popc(ties & lower) < quota_b[b]);
      run[b] += __popc(ties);
    }
    const int c = !in ? 0 : (below[0] ? 3 : (below[1] ? 2 : (below[2] ? 1 : 0)));
#pragma unroll
    for (int k = 1; k <= 3; ++k) {
      const unsigned members = __ballot_sync(0xffffffffu, c == k);
      if (c == k) {
        int32_t* dst = list + at[k - 1] + __popc(members & lower) * factor;
        for (int e = 0; e < factor; ++e) dst[e] = prefix_stages + j * factor + e;
      }
      at[k - 1] += __popc(members) * factor;
    }
  }
}

// ---- routing with anchors (an experimental variant of the reference,
// anemoi/layers/attention/mpa/routing.py:190-203, sm120/h3_route_precision.cu:160-220) -------------
// Anchor pairs (a fixed [R][R] mask shared by the heads: the same-frame neighbours of a block) that
// the ranking dropped are forced into the lowest active precision, and as many of the
// lowest-ranked pairs of that precision that are not anchors are dropped instead.  Restated as
// selection: every anchor is kept (at the precision of its rank, or the lowest one), and of
// the other pairs exactly the retained - anchor_count best ranked are kept, at the precision
// of their rank among all pairs.  So a fourth boundary is taken in the ranking of the pairs
// that are not anchors (their histogram is the full one minus the anchors').  A pair's
// precision then depends on the anchor mask, and the per-row counts are taken by a pass of
// their own before the offsets are scanned.
constexpr int kAnchorStat = 4;  // ints per row: items equal to straddling key 0,1,2; non-anchors equal to key 3

__global__ void __launch_bounds__(256) anchor_hist_kernel(const unsigned short* prob, int64_t items,
                                                          const int32_t* anchor_ids, int count,
                                                          int* hist_anchor) {
  const int i = blockIdx.x * 256 + threadIdx.x, head = blockIdx.y;
  if (i >= count) return;
  const int key = __ldg(prob + (int64_t)head * items + anchor_ids[i]) & 0x7fff;
  atomicAdd(hist_anchor + (int64_t)head * kBins + key, 1);
}

struct AnchorRow {
  int key_b[4], quota_b[4], run[4];
};

__device__ __forceinline__ AnchorRow anchor_row(const int* thr, const int* stat, int head, int R,
                                                int row) {
  AnchorRow a;
  const int* st = stat + ((int64_t)head * R + row) * kAnchorStat;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    a.key_b[b] = thr[head * 16 + (b < 3 ? 2 * b : 8)];
    a.quota_b[b] = thr[head * 16 + (b < 3 ? 2 * b + 1 : 9)];
    a.run[b] = st[b];
  }
  return a;
}

// Precision code of the lane's column (0 = dropped); advances the row's tie counters.
__device__ __forceinline__ int anchor_code(AnchorRow& a, int key, bool in, bool anchor, unsigned lower,
                                           int lowest_code) {
  bool below[3];
#pragma unroll
  for (int b = 0; b < 3; ++b) {
    const bool tie = in && key == a.key_b[b];
    const unsigned ties = __ballot_sync(0xffffffffu, tie);
    below[b] = key > a.key_b[b] || (tie && a.run[b] + __popc(ties & lower) < a.quota_b[b]);
    a.run[b] += __popc(ties);
  }
  const bool tie = in && !anchor && key == a.key_b[3];
  const unsigned ties = __ballot_sync(0xffffffffu, tie);
  const bool kept = key > a.key_b[3] || (tie && a.run[3] + __popc(ties & lower) < a.quota_b[3]);
  a.run[3] += __popc(ties);
  const int ranked = below[0] ? 3 : (below[1] ? 2 : (below[2] ? 1 : 0));
  if (!in) return 0;
  if (anchor) return ranked ? ranked : lowest_code;
  return kept ? ranked : 0;
}

// One warp per row: items equal to each straddling key (the fourth among the non-anchors only).
__global__ void __launch_bounds__(kRowWarps * 32) anchor_rowstat_kernel(const unsigned short* prob,
                                                                        const uint8_t* anchors, int R,
                                                                        const int* thr, int* stat) {
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5), head = blockIdx.y;
  if (row >= R) return;
  const int lane = threadIdx.x & 31;
  const int k0 = thr[head * 16], k1 = thr[head * 16 + 2], k2 = thr[head * 16 + 4],
            k3 = thr[head * 16 + 8];
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;
  const uint8_t* an = anchors + (int64_t)row * R;
  int e0 = 0, e1 = 0, e2 = 0, e3 = 0;
  for (int j = lane; j < R; j += 32) {
    const int key = __ldg(src + j) & 0x7fff;
    e0 += key == k0;
    e1 += key == k1;
    e2 += key == k2;
    e3 += key == k3 && !an[j];
  }
  e0 = __reduce_add_sync(0xffffffffu, e0);
  e1 = __reduce_add_sync(0xffffffffu, e1);
  e2 = __reduce_add_sync(0xffffffffu, e2);
  e3 = __reduce_add_sync(0xffffffffu, e3);
  if (lane < 4)
    stat[((int64_t)head * R + row) * kAnchorStat + lane] = lane == 0 ? e0 : lane == 1 ? e1 : lane == 2 ? e2 : e3;
}

// One CTA per head: the equal-counts become exclusive prefixes over the rows.
__global__ void __launch_bounds__(1024) anchor_tiescan_kernel(int R, int* stat) {
  __shared__ long long warp_sum[32];
  const int head = blockIdx.x;
  long long carry[4] = {0, 0, 0, 0};
  for (int r0 = 0; r0 < R; r0 += 1024) {
    const int row = r0 + threadIdx.x;
    const bool in = row < R;
    int* st = stat + ((int64_t)head * R + row) * kAnchorStat;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int eq = in ? st[b] : 0;
      long long all;
      const long long pre = carry[b] + block_exclusive(eq, warp_sum, all);
      carry[b] += all;
      if (in) st[b] = (int)pre;
    }
  }
}

// One warp per row: pairs per precision (entries 0..2 of the row's counts, in logical blocks).
__global__ void __launch_bounds__(kRowWarps * 32) anchor_count_kernel(const unsigned short* prob,
                                                                      const uint8_t* anchors, int R,
                                                                      const int* thr, const int* stat,
                                                                      int lowest_code, int32_t* row_counts) {
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5), head = blockIdx.y;
  if (row >= R) return;
  const int lane = threadIdx.x & 31;
  const unsigned lower = (1u << lane) - 1u;
  AnchorRow a = anchor_row(thr, stat, head, R, row);
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;
  const uint8_t* an = anchors + (int64_t)row * R;
  int n[3] = {0, 0, 0};
  for (int j0 = 0; j0 < R; j0 += 32) {
    const int j = j0 + lane;
    const bool in = j < R;
    const int key = in ? (__ldg(src + j) & 0x7fff) : -2;
    const int c = anchor_code(a, key, in, in && an[j] != 0, lower, lowest_code);
#pragma unroll
    for (int k = 1; k <= 3; ++k) n[k - 1] += __popc(__ballot_sync(0xffffffffu, c == k));
  }
  if (lane < 3) row_counts[((int64_t)head * R + row) * 4 + lane] = n[lane];
}

// One CTA per head: stages per phase from the pair counts, list offsets in row order, launch order.
__global__ void __launch_bounds__(1024) anchor_offsets_kernel(int R, int factor, int prefix_stages,
                                                              int prefix_phase, int32_t* row_offset,
                                                              int32_t* row_counts) {
  __shared__ long long warp_sum[32];
  __shared__ int total_s[kOrderMaxBlocks];
  const int head = blockIdx.x;
  const int p = prefix_phase >= 0 ? prefix_stages : 0;
  long long carry = 0;
  for (int r0 = 0; r0 < R; r0 += 1024) {
    const int row = r0 + threadIdx.x;
    const bool in = row < R;
    int32_t* rc = row_counts + ((int64_t)head * R + row) * 4;
    int n[3] = {0, 0, 0};
    if (in)
      for (int c = 0; c < 3; ++c) n[c] = rc[c] * factor + (prefix_phase == c ? p : 0);
    const int total = n[0] + n[1] + n[2];
    long long all;
    const long long off = carry + block_exclusive(total, warp_sum, all);
    carry += all;
    if (in) {
      row_offset[(int64_t)head * R + row] = (int32_t)off;
      rc[0] = n[0];
      rc[1] = n[1];
      rc[2] = n[2];
      rc[3] = 0;
      if (row < kOrderMaxBlocks) total_s[row] = total;
    }
  }
  if (R > kOrderMaxBlocks) return;
  __syncthreads();
  int32_t* rc = row_counts + (int64_t)head * R * 4;
  for (int i = threadIdx.x; i < R; i += 1024) {
    const int mine = total_s[i];
    int rank = 0;
    for (int j = 0; j < R; ++j) rank += (total_s[j] > mine) || (total_s[j] == mine && j < i);
    rc[rank * 4 + 3] = i + 1;
  }
}

// One warp per row writes the row's list (as emit_kernel, with the anchored codes).
__global__ void __launch_bounds__(kRowWarps * 32) anchor_emit_kernel(
    const unsigned short* prob, const uint8_t* anchors, int R, const int* thr, const int* stat,
    int lowest_code, int factor, int prefix_stages, int prefix_phase, int64_t capacity,
    const int32_t* row_offset, const int32_t* row_counts, int32_t* stage_ids) {
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5), head = blockIdx.y;
  if (row >= R) return;
  const int lane = threadIdx.x & 31;
  const unsigned lower = (1u << lane) - 1u;
  AnchorRow a = anchor_row(thr, stat, head, R, row);
  const int32_t* rc = row_counts + ((int64_t)head * R + row) * 4;
  const int n0 = rc[0], n1 = rc[1], n2 = rc[2];
  const int total = n0 + n1 + n2;
  if (total == 0) return;
  const int64_t base = row_offset[(int64_t)head * R + row];
  if (base + total > capacity) return;
  int32_t* list = stage_ids + (int64_t)head * capacity + base;
  const int p = prefix_phase >= 0 ? prefix_stages : 0;
  int at[3] = {prefix_phase == 0 ? p : 0, n0 + (prefix_phase == 1 ? p : 0),
               n0 + n1 + (prefix_phase == 2 ? p : 0)};
  if (prefix_phase >= 0) {
    const int seg = prefix_phase == 0 ? 0 : (prefix_phase == 1 ? n0 : n0 + n1);
    for (int s = lane; s < p; s += 32) list[seg + s] = s;
  }
  const unsigned short* src = prob + ((int64_t)head * R + row) * R;
  const uint8_t* an = anchors + (int64_t)row * R;
  for (int j0 = 0; j0 < R; j0 += 32) {
    const int j = j0 + lane;
    const bool in = j < R;
    const int key = in ? (__ldg(src + j) & 0x7fff) : -2;
    const int c = anchor_code(a, key, in, in && an[j] != 0, lower, lowest_code);
#pragma unroll
    for (int k = 1; k <= 3; ++k) {
      const unsigned members = __ballot_sync(0xffffffffu, c == k);
      if (c == k) {
        int32_t* dst = list + at[k - 1] + __popc(members & lower) * factor;
        for (int e = 0; e < factor; ++e) dst[e] = prefix_stages + j * factor + e;
      }
      at[k - 1] += __popc(members) * factor;
    }
  }
}

// Q64 query blocks 2t and 2t+1 of a head run as one CTA of the attention kernel (rows 0-63 and
// 64-127 of the 128-row MMA shape).  That CTA walks, phase by phase, the union of the two
// blocks' lists; bits 30 and 31 of an entry say which of the two blocks the stage belongs to.
// One warp per pair, one lane per phase (a two-pointer merge of two ascending lists).  The union
// of phase c is written where the two blocks' phases before c would end, inside the space the two
// lists occupy in the stage list (a buffer of the same capacity), so no offsets are scanned.
// The pairs of a head are then ranked longest first, like the blocks.
__global__ void __launch_bounds__(kRowWarps * 32) pair_kernel(int R, int64_t capacity,
                                                              const int32_t* row_offset,
                                                              const int32_t* row_counts,
                                                              const int32_t* stage_ids,
                                                              int32_t* pair_counts,
                                                              int32_t* pair_ids) {
  const int pairs = (R + 1) / 2;
  const int pair = blockIdx.x * kRowWarps + (threadIdx.x >> 5), head = blockIdx.y;
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const int a = 2 * pair;
  const bool has_b = a + 1 < R;
  const int32_t* ca = row_counts + ((int64_t)head * R + a) * 4;
  const int64_t base = row_offset[(int64_t)head * R + a];
  const int32_t* la = stage_ids + (int64_t)head * capacity + base;
  const int32_t* lb = la + (ca[0] + ca[1] + ca[2]);  // lists follow one another in row order
  int32_t* out = pair_ids + (int64_t)head * capacity + base;
  int n = 0;
  if (lane < 3) {
    int sa = 0, sb = 0, so = 0;  // starts of this lane's phase in A, in B and in the union
    for (int c = 0; c < lane; ++c) {
      sa += ca[c];
      sb += has_b ? ca[4 + c] : 0;
    }
    so = sa + sb;
    const int na = ca[lane], nb = has_b ? ca[4 + lane] : 0;
    int i = 0, j = 0;
    while (i < na || j < nb) {
      const int x = i < na ? la[sa + i] : INT_MAX;
      const int y = j < nb ? lb[sb + j] : INT_MAX;
      const int v = min(x, y);
      out[so + n++] = v | (x == v ? 1 << 30 : 0) | (y == v ? (int)(1u << 31) : 0);
      i += x == v;
      j += y == v;
    }
  }
  if (lane < 4) pair_counts[((int64_t)head * pairs + pair) * 4 + lane] = lane < 3 ? n : 0;
}

// Launch order of a head's pairs: longest union first (ties by pair index), as for the blocks.
__global__ void __launch_bounds__(1024) pair_order_kernel(int pairs, int32_t* pair_counts) {
  __shared__ int total_s[kOrderMaxBlocks];
  const int head = blockIdx.x;
  int32_t* pc = pair_counts + (int64_t)head * pairs * 4;
  for (int i = threadIdx.x; i < pairs; i += 1024) total_s[i] = pc[i * 4] + pc[i * 4 + 1] + pc[i * 4 + 2];
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += 1024) {
    const int mine = total_s[i];
    int rank = 0;
    for (int j = 0; j < pairs; ++j) rank += (total_s[j] > mine) || (total_s[j] == mine && j < i);
    pc[rank * 4 + 3] = i + 1;
  }
}

}  // namespace

extern "C" int64_t anemoi_sm100_route_anchored_scratch_bytes(const anemoi_sm100_shape* shape) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK) return ANEMOI_SM100_EINVAL;
  return (int64_t)shape->heads * (2 * kBins + 16 + kAnchorStat * (int64_t)shape->video_blocks) * 4;
}

extern "C" int anemoi_sm100_route_anchored(const anemoi_sm100_shape* shape, const void* probability,
                                           int64_t n16, int64_t n8, int64_t n4, int prefix_phase,
                                           const uint8_t* anchors, const int32_t* anchor_ids,
                                           int32_t anchor_count, void* scratch, int64_t scratch_bytes,
                                           int32_t* row_offset, int32_t* row_counts,
                                           int32_t* stage_ids, int64_t list_capacity, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !probability || !scratch || !row_offset ||
      !row_counts || !stage_ids || !anchors || !anchor_ids || anchor_count <= 0)
    return ANEMOI_SM100_EINVAL;
  const int H = shape->heads, R = shape->video_blocks;
  const int64_t items = (int64_t)R * R, retained = n16 + n8 + n4;
  if (n16 < 0 || n8 < 0 || n4 < 0 || retained > items || retained <= 0) return ANEMOI_SM100_EINVAL;
  // as the reference: the anchors must fit into the lowest active precision
  const int64_t lowest = n4 ? n4 : (n8 ? n8 : n16);
  if (anchor_count > lowest) return ANEMOI_SM100_EINVAL;
  if (prefix_phase < -1 || prefix_phase > 2) return ANEMOI_SM100_EINVAL;
  if (prefix_phase >= 0 && shape->prefix_tokens == 0) prefix_phase = -1;
  if (scratch_bytes < anemoi_sm100_route_anchored_scratch_bytes(shape)) return ANEMOI_SM100_EINVAL;
  if (list_capacity < anemoi_sm100_route_list_capacity(shape, n16, n8, n4, prefix_phase))
    return ANEMOI_SM100_EINVAL;
  if (R > 65535 || items * H >= (1ll << 40)) return ANEMOI_SM100_ELIMIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* hist = static_cast<int*>(scratch);
  int* hist_anchor = hist + (int64_t)H * kBins;
  int* thr = hist_anchor + (int64_t)H * kBins;
  int* stat = thr + (int64_t)H * 16;
  if (cudaMemsetAsync(hist, 0, (size_t)H * kBins * 8, st) != cudaSuccess) return ANEMOI_SM100_ELAUNCH;
  if (cudaFuncSetAttribute(hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHalfBins * 4) !=
      cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  const unsigned short* prob = static_cast<const unsigned short*>(probability);
  const int chunks = (int)max((int64_t)1, min(min((int64_t)16, items / 8192), (int64_t)((296 + H / 2) / H)));
  const int factor = shape->query_block / 64, prefix_stages = rec::prefix_stages(*shape);
  const int lowest_code = n4 ? 1 : (n8 ? 2 : 3);
  const dim3 rows((R + kRowWarps - 1) / kRowWarps, H);
  hist_kernel<<<dim3(chunks, H, 2), kHistThreads, kHalfBins * 4, st>>>(prob, items, chunks, hist);
  anchor_hist_kernel<<<dim3((anchor_count + 255) / 256, H), 256, 0, st>>>(prob, items, anchor_ids,
                                                                           anchor_count, hist_anchor);
  threshold_kernel<<<H, 1024, 0, st>>>(hist, nullptr, thr, 16, 0, n16, n16 + n8, retained);
  const int64_t others = retained - anchor_count;  // pairs kept that are not anchors
  threshold_kernel<<<H, 1024, 0, st>>>(hist, hist_anchor, thr, 16, 8, others, others, others);
  anchor_rowstat_kernel<<<rows, kRowWarps * 32, 0, st>>>(prob, anchors, R, thr, stat);
  anchor_tiescan_kernel<<<H, 1024, 0, st>>>(R, stat);
  anchor_count_kernel<<<rows, kRowWarps * 32, 0, st>>>(prob, anchors, R, thr, stat, lowest_code,
                                                       row_counts);
  anchor_offsets_kernel<<<H, 1024, 0, st>>>(R, factor, prefix_stages, prefix_phase, row_offset,
                                            row_counts);
  anchor_emit_kernel<<<rows, kRowWarps * 32, 0, st>>>(prob, anchors, R, thr, stat, lowest_code, factor,
                                                      prefix_stages, prefix_phase, list_capacity,
                                                      row_offset, row_counts, stage_ids);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

extern "C" int anemoi_sm100_pair_lists(const anemoi_sm100_shape* shape, const int32_t* row_offset,
                                       const int32_t* row_counts, const int32_t* stage_ids,
                                       int64_t list_capacity, int32_t* pair_counts,
                                       int32_t* pair_ids, void* stream) {
  if (rec::validate_shape(shape) != ANEMOI_SM100_OK || !row_offset || !row_counts || !stage_ids ||
      !pair_counts || !pair_ids || list_capacity <= 0 || shape->query_block != 64)
    return ANEMOI_SM100_EINVAL;
  if (rec::stages(*shape) >= (1 << 30)) return ANEMOI_SM100_ELIMIT;  // two flag bits per entry
  const int R = shape->video_blocks, H = shape->heads, pairs = (R + 1) / 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  pair_kernel<<<dim3((pairs + kRowWarps - 1) / kRowWarps, H), kRowWarps * 32, 0, st>>>(
      R, list_capacity, row_offset, row_counts, stage_ids, pair_counts, pair_ids);
  if (pairs <= kOrderMaxBlocks) pair_order_kernel<<<H, 1024, 0, st>>>(pairs, pair_counts);
  return cudaGetLastError() == cudaSuccess ? ANEMOI_SM100_OK : ANEMOI_SM100_ELAUNCH;
}

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
  sc.stat = sc.thr + (int64_t)H * 8;
  if (cudaMemsetAsync(sc.hist, 0, (size_t)H * kBins * 4, st) != cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  const unsigned short* prob = static_cast<const unsigned short*>(probability);
  // Function attributes belong to a device: the opt-in is made at every call (a cheap host-side
  // driver call), so a process that routes on several GPUs, or from several host threads,
  // never launches the kernel without the opt-in for its dynamic shared memory.
  if (cudaFuncSetAttribute(hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHalfBins * 4) !=
      cudaSuccess)
    return ANEMOI_SM100_ELAUNCH;
  // about two waves of histogram CTAs per key-range half, each with at least 8192 items
  const int chunks = (int)max((int64_t)1, min(min((int64_t)16, items / 8192), (int64_t)((296 + H / 2) / H)));
  const int factor = shape->query_block / 64, prefix_stages = rec::prefix_stages(*shape);
  const dim3 rows((R + kRowWarps - 1) / kRowWarps, H);
  hist_kernel<<<dim3(chunks, H, 2), kHistThreads, kHalfBins * 4, st>>>(prob, items, chunks, sc.hist);
  threshold_kernel<<<H, 1024, 0, st>>>(sc.hist, nullptr, sc.thr, 8, 0, n16, n16 + n8, n16 + n8 + n4);
  rowstat_kernel<<<rows, kRowWarps * 32, 0, st>>>(prob, R, sc.thr, sc.stat);
  headscan_kernel<<<H, 1024, 0, st>>>(R, sc.thr, sc.stat, factor, prefix_stages, prefix_phase,
                                      row_offset, row_counts);
  emit_kernel<<<rows, kRowWarps * 32, 0, st>>>(prob, R, sc.thr, sc.stat, factor, prefix_stages,
                                               prefix_phase, list_capacity, row_offset, row_counts,
                                               stage_ids);
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
  if (need > kStaticScratchInts) return ANEMOI_SM100_ELIMIT;  // heads*(32776 + 6*blocks) ints
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
  // Same kernels as anemoi_sm100_route; the bins that must start at zero are cleared there on
  // `stream` at every call, the rest is overwritten before it is read.
  return anemoi_sm100_route(shape, probability, n16, n8, n4, prefix_phase, scratch, need * 4,
                            row_offset, row_counts, stage_ids, list_capacity, stream);
}
