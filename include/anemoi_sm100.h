/* C ABI of the B200 (sm_100a) sparse mixed-precision attention path.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every
 * entry point is asynchronous on `stream` (a cudaStream_t passed as void*),
 * allocates nothing unless stated, never synchronises the host, and returns 0
 * or a negative ANEMOI_SM100_E* code before anything is launched.  All device
 * pointers must belong to the current device.  Batch size is 1, as in the
 * reference (anemoi/layers/attention/mpa/executor.py:903-919).
 *
 * The functions replace, one for one or fused, the custom operators the
 * reference registers in csrc/attention/cuda/sm120/bindings.cpp:9-176 and
 * csrc/attention/cuda/sm89/bindings.cpp (shared pack / assemble operators).
 */
#ifndef ANEMOI_SM100_H_
#define ANEMOI_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  ANEMOI_SM100_OK = 0,
  ANEMOI_SM100_EINVAL = -1,   /* bad shape, flag or null pointer */
  ANEMOI_SM100_ELAUNCH = -2,  /* the CUDA runtime refused a launch */
  ANEMOI_SM100_ELIMIT = -3    /* size beyond a documented maximum */
};

/* Geometry and active precision cells of one call. */
typedef struct anemoi_sm100_shape {
  int32_t heads;            /* H (heads held by this GPU) */
  int32_t head_dim;         /* D: 64 or 128 */
  int32_t query_block;      /* QB: 64 or 128 (also the logical key block) */
  int32_t seq_tokens;       /* S = prefix_tokens + video tokens */
  int32_t prefix_tokens;
  int32_t video_blocks;     /* R = frames * blocks per frame */
  int32_t has_nvfp4;        /* cells that need operands (video phases + prefix phase) */
  int32_t has_int8;
  int32_t has_fp16;
  int32_t has_prefix_query_int8; /* prefix queries run through the INT8 cell */
  int32_t has_maxpool;          /* 1: max pools in the extra pool slots; 2: second moments (diag-Jensen) */
  int32_t input_is_bf16;    /* raw Q/K/V dtype: 1 bf16, 0 fp16 */
  float q_global_scale;     /* NVFP4 tensor-level scales (NVFP4Calibration) */
  float k_global_scale;
  float v_global_scale;
} anemoi_sm100_shape;

/* Operand store filled by anemoi_sm100_prepare and read by the attention
 * kernels.  Tiles are kept in the order the tensor core reads them from shared
 * memory (8 rows x 16 bytes core matrices, no swizzle), one contiguous record
 * per (head, query tile) or (head, 64-key stage), so a single bulk copy lands a
 * ready operand.  Pointers of inactive cells may be null.  Sizes in bytes come
 * from anemoi_sm100_operand_bytes(). */
typedef struct anemoi_sm100_operands {
  void* q_fp16;     /* [H][R] records: Q tile QBxD fp16 */
  void* kv_fp16;    /* [H][stages] records: K tile 64xD fp16 | V tile 64xD fp16 */
  void* q_int8;     /* [H][R + prefix query tiles] records: Q tile QBxD s8 */
  void* kv_int8;    /* [H][stages] records: K tile 64xD s8 | V tile Dx64 e4m3 */
  void* q_nvfp4;    /* [H][R] records: Q tile QBxD e2m1 | scale bytes */
  void* kv_nvfp4;   /* [H][stages] records: K e2m1 | V^T e2m1 | K scales | V scales */
  float* q_int8_scale;   /* [H][R + prefix query tiles] */
  float* k_int8_scale;   /* [H][stages] */
  float* v_e4m3_scale;   /* [H][D] = amax/2.25 */
  float* v_amax;         /* [H][D] scratch of the V amax pre-pass (int8 cell) */
  void* q_pool;          /* [H][R][D] fp16 mean pools */
  void* k_pool;
  void* q_max_pool;      /* [H][R][D] fp16 max pools (has_maxpool) */
  void* k_max_pool;
} anemoi_sm100_operands;

enum {
  ANEMOI_SM100_BUF_Q_FP16 = 0, ANEMOI_SM100_BUF_KV_FP16, ANEMOI_SM100_BUF_Q_INT8,
  ANEMOI_SM100_BUF_KV_INT8, ANEMOI_SM100_BUF_Q_NVFP4, ANEMOI_SM100_BUF_KV_NVFP4,
  ANEMOI_SM100_BUF_Q_INT8_SCALE, ANEMOI_SM100_BUF_K_INT8_SCALE, ANEMOI_SM100_BUF_V_E4M3_SCALE,
  ANEMOI_SM100_BUF_V_AMAX, ANEMOI_SM100_BUF_POOL, ANEMOI_SM100_BUF_COUNT
};

/* Library identity: returns 100 (the sm_ architecture this build targets). */
int anemoi_sm100_arch(void);

/* Bytes of buffer `which` (ANEMOI_SM100_BUF_*) for `shape`; 0 if the cell is
 * inactive; negative on a bad shape. */
int64_t anemoi_sm100_operand_bytes(const anemoi_sm100_shape* shape, int which);

/* Gather + narrow + pool + quantise in one pass over raw Q/K/V (logical
 * [1,S,H,D], bf16 or fp16, D contiguous).  `strides` = token and head stride in
 * elements of q, k, v (6 values, multiples of 8), or null for contiguous
 * [1,S,H,D]; strided views let the head-sharded buffer of a Ulysses exchange be
 * consumed in place (the reference accepts its BSHD-strided view the same way,
 * csrc/common/raw_bhsd_layout.h:15-28).  `indices` int32 [R*QB] (slot -> video
 * token), `counts` int32 [R] (real tokens per block).
 * Replaces prepare_h3_sm120_operands (sm120/bindings.cpp, kernels in
 * sm120/q128_microscaling_preparation.cu:245-803) and, for the pure FP16 cell,
 * pack_h3_k64_qkv_fp16 + the torch pools (mpa/executor.py:83-108). */
int anemoi_sm100_prepare(const anemoi_sm100_shape* shape, const void* q, const void* k,
                         const void* v, const int64_t* strides, const int32_t* indices,
                         const int32_t* counts, const anemoi_sm100_operands* out, void* stream);

/* Pooled-QK row softmax -> fp16 probability [H][R][R]; with 0 < w < 1 the mean
 * and max maps are blended, w == 1 uses the max pools only.
 * Replaces sm120_h3_draft_probability (sm120/h3_draft_probability.cu:531-670). */
int anemoi_sm100_draft_probability(const anemoi_sm100_shape* shape, const void* q_pool,
                                   const void* k_pool, const void* q_max_pool,
                                   const void* k_max_pool, float maxpool_weight,
                                   void* probability, void* stream);

/* The diag-Jensen draft map, an experimental routing proxy of the reference
 * (mpa/routing.py:87-103, enabled by `diag_jensen` in mpa/executor.py:1105-1126; never combined
 * with the max-pool blend): logits q.k/sqrt(D) + 0.5 * max((q2.k2 - (q*q).(k*k)) / D, 0) in fp32,
 * row softmax, fp16 [H][R][R].  `q_second`, `k_second` [H][R][D] fp16 are the per-channel second
 * moments of the blocks; anemoi_sm100_prepare writes them into the max-pool slots of the operands
 * when shape.has_maxpool == 2.  The reference computes this map with torch matmuls. */
int anemoi_sm100_draft_probability_jensen(const anemoi_sm100_shape* shape, const void* q_pool,
                                          const void* k_pool, const void* q_second,
                                          const void* k_second, void* probability, void* stream);

/* Bytes of scratch anemoi_sm100_route needs for `shape`. */
int64_t anemoi_sm100_route_scratch_bytes(const anemoi_sm100_shape* shape);

/* Entries per head of the compact stage list: (n16+n8+n4)*QB/64 + R*prefix stages
 * (prefix stages are spliced only when prefix_phase >= 0). */
int64_t anemoi_sm100_route_list_capacity(const anemoi_sm100_shape* shape, int64_t n16,
                                         int64_t n8, int64_t n4, int prefix_phase);

/* Global per-head top-k with precision by rank, compacted per query block into
 * ragged 64-key stage lists.
 *   probability  fp16 [H][R][R]
 *   n16,n8,n4    per-head budgets (FP16, INT8, NVFP4)
 *   prefix_phase -1 none, 0 nvfp4, 1 int8, 2 fp16: phase that carries the prefix stages
 *   row_offset   int32 [H][R]   start of the row's list inside the head's segment (the lists
 *                follow one another in row order: the same layout at every call)
 *   row_counts   int32 [H][R][4] stages per phase (nvfp4, int8, fp16), prefix included; the
 *                fourth entry of slot i is 1 + the query block the attention kernel should run
 *                as its i-th CTA of the head (longest list first), or 0 for "block i"
 *   stage_ids    int32 [H][capacity] lists: nvfp4 stages, int8 stages, fp16 stages;
 *                logical columns ascend inside a phase, prefix stages lead their phase
 * Ties are broken by ascending flat index row*R+col.
 * Replaces sm120_h3_route_precision + sm120_h3_materialize_route
 * (sm120/h3_route_precision.cu:373-647); anchors are not supported (the public
 * path never enables them, mpa/executor.py:1272). */
int anemoi_sm100_route(const anemoi_sm100_shape* shape, const void* probability, int64_t n16,
                       int64_t n8, int64_t n4, int prefix_phase, void* scratch,
                       int64_t scratch_bytes, int32_t* row_offset, int32_t* row_counts,
                       int32_t* stage_ids, int64_t list_capacity, void* stream);

/* Routing with anchors, an experimental variant of the reference (mpa/routing.py:190-203,
 * sm120/h3_route_precision.cu:160-220; off in the public path, enabled by `enable_anchors` in
 * mpa/executor.py:1151-1158).  `anchors` is a [R][R] byte mask shared by the heads (the
 * same-frame neighbours of every block, mpa/layout.py:69-98), `anchor_ids` its `anchor_count`
 * set flat indices.  Anchor pairs the ranking dropped are forced into the lowest active
 * precision and as many of the lowest-ranked other pairs of that precision are dropped
 * instead; `anchor_count` must not exceed that precision's budget.  Same outputs as
 * anemoi_sm100_route; scratch from anemoi_sm100_route_anchored_scratch_bytes. */
int64_t anemoi_sm100_route_anchored_scratch_bytes(const anemoi_sm100_shape* shape);
int anemoi_sm100_route_anchored(const anemoi_sm100_shape* shape, const void* probability,
                                int64_t n16, int64_t n8, int64_t n4, int prefix_phase,
                                const uint8_t* anchors, const int32_t* anchor_ids,
                                int32_t anchor_count, void* scratch, int64_t scratch_bytes,
                                int32_t* row_offset, int32_t* row_counts, int32_t* stage_ids,
                                int64_t list_capacity, void* stream);

/* Routing for callers that cannot provide scratch memory.  It has no counterpart in the
 * reference.  A host whose memory pool is fixed once it starts serving, or that must avoid
 * cudaMalloc / cudaFree on its request path (they synchronise the whole device), cannot
 * size and pass the scratch buffer anemoi_sm100_route needs.  This variant does the same
 * work with the same arguments and results, but its scratch is an 8 MiB array that is part
 * of the library image (held on every GPU that loads the library until the process ends);
 * it calls no allocating routine of any kind.  Shapes that need more scratch than that -
 * heads * (32776 + 6 * video_blocks) * 4 bytes > anemoi_sm100_route_static_max_bytes() -
 * are refused with ANEMOI_SM100_ELIMIT.  The first call on a device looks up the array's
 * device address; make that call outside any stream capture.  All calls on a device share
 * the one array (it keeps the last call's contents; what must start at zero is cleared on
 * `stream` at every call), so two calls whose kernels may overlap on the GPU race: issue
 * them on one stream or order them with events. */
int64_t anemoi_sm100_route_static_max_bytes(void);
int anemoi_sm100_route_static(const anemoi_sm100_shape* shape, const void* probability,
                              int64_t n16, int64_t n8, int64_t n4, int prefix_phase,
                              int32_t* row_offset, int32_t* row_counts, int32_t* stage_ids,
                              int64_t list_capacity, void* stream);

/* Block-sparse mixed-precision flash attention of the video query blocks.
 *   valid_k      int32 [stages] real keys per stage
 *   out_packed   fp16 [H][R*QB][D] packed row order; rows of empty lists are not written
 *   status       int32 [1] device word, set non-zero (first give-up wins, never cleared by
 *                the library) if a bounded wait gave up; the output is then invalid
 * Replaces sm120_q{64,128}_{fp16,int8_fp16,nvfp4_fp16,nv_int8_fp16}_attention_forward
 * (sm120/bindings.cpp, sm120/q64_attention_host.cu). */
int anemoi_sm100_attention(const anemoi_sm100_shape* shape, const anemoi_sm100_operands* ops,
                           const int32_t* row_offset, const int32_t* row_counts,
                           const int32_t* stage_ids, int64_t list_capacity,
                           const int32_t* valid_k, void* out_packed, int32_t* status,
                           void* stream);

/* Limit, in nanoseconds, of every bounded wait inside the attention kernels launched after
 * this call (default 2 s; process-wide).  No reference counterpart: the reference's kernels
 * have no waits that another warp must satisfy. */
int anemoi_sm100_set_wait_limit_ns(uint64_t limit_ns);

/* Self-test of the give-up path of the bounded waits (no reference counterpart): one CTA
 * waits, for at most `limit_ns` (<= 100 ms), on a barrier nothing ever arrives on, with no
 * copy or MMA in flight; *status (device int32, zeroed by the caller) becomes 99 and the
 * kernel returns normally. */
int anemoi_sm100_wait_selftest(uint64_t limit_ns, int32_t* status, void* stream);

/* Q64 only: query blocks 2t and 2t+1 of a head as one CTA (rows 0-63 and 64-127 of the 128-row MMA
 * shape), walking phase by phase the union of their two lists.  pair_lists merges the lists:
 *   pair_counts  int32 [H][ceil(R/2)][4]  stages per phase of the union; fourth entry = launch order
 *   pair_ids     int32 [H][capacity]      stage id, bit 30: belongs to block 2t, bit 31: to 2t+1;
 *                a pair's list starts at row_offset of block 2t, phase c of the union where the
 *                two blocks' phases before c would end
 * attention_pairs is anemoi_sm100_attention over those lists; rows of a block ignore the stages
 * of the other one (zero probabilities, running maximum and denominator untouched), so every
 * row sees exactly its own stages in its own order and the result is that of anemoi_sm100_attention.
 * The reference runs one 64-row block per CTA with 16 rows per warp
 * (sm120/q64_attention.cuh:1109-1390); the pairing exists because the tcgen05 shape is 128 rows. */
int anemoi_sm100_pair_lists(const anemoi_sm100_shape* shape, const int32_t* row_offset,
                            const int32_t* row_counts, const int32_t* stage_ids,
                            int64_t list_capacity, int32_t* pair_counts, int32_t* pair_ids,
                            void* stream);
int anemoi_sm100_attention_pairs(const anemoi_sm100_shape* shape, const anemoi_sm100_operands* ops,
                                 const int32_t* row_offset, const int32_t* row_counts,
                                 const int32_t* pair_counts, const int32_t* pair_ids,
                                 int64_t list_capacity, const int32_t* valid_k, void* out_packed,
                                 int32_t* status, void* stream);

/* Dense INT8-cell attention of the prefix query rows over every stage.
 *   out_prefix   fp16 [H][prefix query tiles * QB][D]
 * Replaces sm120_q{64,128}_prefix_int8_attention_forward
 * (sm120/q64_attention_host.cu:410-544). */
int anemoi_sm100_prefix_attention(const anemoi_sm100_shape* shape,
                                  const anemoi_sm100_operands* ops, const int32_t* valid_k,
                                  void* out_prefix, int32_t* status, void* stream);

/* Inverse scatter into [1,S,H,D] of the caller's dtype: prefix rows from
 * `prefix_out` ([H][rows][D], fp16 if prefix_is_caller_dtype == 0 else the
 * caller dtype, row stride `prefix_rows`), video rows from out_packed through
 * `inverse` (int32 [video tokens] -> slot); query blocks whose three counts are
 * all zero yield +0.  Replaces assemble_h3_k64_output
 * (sm89/output_assembly.cu:219-305). */
int anemoi_sm100_assemble(const anemoi_sm100_shape* shape, const void* prefix_out,
                          int64_t prefix_rows, int prefix_is_caller_dtype,
                          const void* out_packed, const int32_t* inverse,
                          const int32_t* row_counts, void* output, void* stream);

/* Ulysses relayout helpers (sequence-sharded <-> head-sharded); 16-bit elements,
 * moved unchanged with 16-byte copies.
 * pack : q,k,v [rows][heads][D] strided views (strides[6] = row and head stride
 *        of q, k, v in elements, each a multiple of 8; D contiguous)
 *        -> send [ranks][rows][heads/ranks][3*D] contiguous (destination-major)
 * merge: recv [ranks][rows][heads_per_rank][D] -> out [rows][ranks*heads_per_rank][D]
 * Replace the Triton kernels _pack_qkv_kernel / _merge_heads_kernel of
 * anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/relayout.py:37-162. */
int anemoi_sm100_pack_qkv(const void* q, const void* k, const void* v, void* send, int64_t rows,
                          int32_t heads, int32_t head_dim, int32_t ranks, const int64_t* strides,
                          void* stream);
int anemoi_sm100_merge_heads(const void* recv, void* out, int64_t rows, int32_t ranks,
                             int32_t heads_per_rank, int32_t head_dim, void* stream);
/* The same relayouts for a sub-range of every rank's heads, so that the exchange of one group of
 * heads can overlap the attention of another (head-group pipelining; the reference exchanges all
 * heads at once, ulysses_custom.py:107-165):
 * pack : send [ranks][rows][head_count][3*D] takes, for destination rank r, the heads
 *        r*(heads/ranks) + head_begin + (0..head_count)
 * merge: recv [ranks][rows][head_count][D] lands in out [rows][ranks*heads_per_rank][D] at heads
 *        r*heads_per_rank + head_begin + (0..head_count) */
int anemoi_sm100_pack_qkv_heads(const void* q, const void* k, const void* v, void* send,
                                int64_t rows, int32_t heads, int32_t head_dim, int32_t ranks,
                                int32_t head_begin, int32_t head_count, const int64_t* strides,
                                void* stream);
int anemoi_sm100_merge_heads_into(const void* recv, void* out, int64_t rows, int32_t ranks,
                                  int32_t head_count, int32_t head_dim, int32_t heads_per_rank,
                                  int32_t head_begin, void* stream);

/* The Ulysses exchange by direct stores into the peers' memory (one node, at most 8 ranks), in
 * place of pack + all-to-all and all-to-all + merge: fused with the collective between them,
 * they replace pack_qkv_destination_major + all_to_all_single and all_to_all_single +
 * merge_heads of the reference (optimized/ulysses_custom.py:107-165, relayout.py:83-162).
 *
 * Set-up (not on the hot path): every rank allocates one exchange region with peer_alloc
 * (cudaMalloc, zero-filled, exported as a 64-byte CUDA IPC handle), passes the handle to the other
 * processes of the node by any host channel, and maps theirs with peer_open; peer_close unmaps,
 * peer_free releases the own region.
 *
 * Per layer: `peer_*[r]` is rank r's buffer / flag words as mapped into this process (`[self]`
 * the local ones); `first_rows[ranks+1]` the first row of every rank's sequence shard.
 *   push_qkv : this rank's rows of q,k,v [rows][heads][D] (strides as in pack_qkv)
 *              -> on rank r: recv [all rows][heads/ranks][3*D], rows first_rows[self]..
 *   push_out : out_heads [all rows][heads_local][D] (this rank's heads, every row)
 *              -> on the owner of a row: out [its rows][ranks*heads_local][D]
 * Plain 16-byte stores over NVLink.  The last block of a push writes `epoch` into word [self] of
 * every destination's flags (release, system scope); `blocks_done` is a zeroed device word of
 * the caller, private to the stream.  wait_flags (one warp, next in stream order on the
 * destination) returns when the first `ranks` words of `flags` have all reached `epoch`, or
 * after `limit_ns` (at most 10 s) with 70 + the late rank in the sticky status word.  Epochs
 * grow by one per call and compare modulo 2^32.  Ordering that makes buffer reuse safe: a rank
 * pushes q,k,v of call e only after its wait on the outputs of call e-1, and pushes outputs
 * of call e only after its wait on the inputs of call e. */
int anemoi_sm100_peer_alloc(int64_t bytes, void** ptr, void* handle64);
int anemoi_sm100_peer_open(const void* handle64, void** ptr);
int anemoi_sm100_peer_close(void* ptr);
int anemoi_sm100_peer_free(void* ptr);
int anemoi_sm100_push_qkv(const void* q, const void* k, const void* v, void* const* peer_recv,
                          void* const* peer_flags, const int64_t* first_rows, int32_t self,
                          int32_t ranks, int32_t heads, int32_t head_dim, const int64_t* strides,
                          uint32_t epoch, void* blocks_done, void* stream);
/* push_qkv with the producer step in it: q and k get the per-head RMS norm with weight and the
 * partial rotary embedding of anemoi_sm100_qknorm_rope (same arithmetic, bit for bit; `cos_table`,
 * `sin_table` fp32 [rows][rotary_dim] for this rank's rows) on their way to the peers, v passes
 * through; q and k of the caller stay as the projection wrote them.  Replaces, fused with the
 * collective, fused_qknorm_rope + pack + all_to_all_single of the reference
 * (optimized/ulysses_custom.py:237-249 and :107-135). */
int anemoi_sm100_push_qkv_norm(const void* q, const void* k, const void* v, const void* q_weight,
                               const void* k_weight, const float* cos_table, const float* sin_table,
                               int32_t rotary_dim, float eps, int32_t is_bf16,
                               void* const* peer_recv, void* const* peer_flags,
                               const int64_t* first_rows, int32_t self, int32_t ranks, int32_t heads,
                               int32_t head_dim, const int64_t* strides, uint32_t epoch,
                               void* blocks_done, void* stream);
int anemoi_sm100_push_out(const void* out_heads, void* const* peer_out, void* const* peer_flags,
                          const int64_t* first_rows, int32_t self, int32_t ranks,
                          int32_t heads_local, int32_t head_dim, uint32_t epoch, void* blocks_done,
                          void* stream);
int anemoi_sm100_wait_flags(const void* flags, int32_t ranks, uint32_t epoch, uint64_t limit_ns,
                            int32_t* status, void* stream);

/* One strided copy between pinned host memory and the device (rows of `width` bytes, `height`
 * of them, pitches in bytes): a group of heads of a host [1,S,H,D] tensor to or from a
 * contiguous device [1,S,heads,D] tensor.  Used by the host-input entry of the Python layer to
 * overlap the copies of one head group with the attention of another; the reference has no
 * host-input path (its tensors are CUDA tensors, anemoi/layers/attention/api.py:134-194). */
int anemoi_sm100_copy_rows(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                           int64_t width, int64_t height, int32_t to_device, void* stream);

/* Producer fusion in front of the attention path: per-head RMS norm with weight, then partial
 * rotary embedding, in place on Q or K.  x [tokens][heads][head_dim] 16-bit (strides[2] = token and
 * head stride in elements, multiples of 8; head_dim contiguous), weight [head_dim] in x's type,
 * cos/sin fp32 [tokens][rotary_dim]; rotary_dim a multiple of 16, at most head_dim (0: norm only).
 * Replaces the Triton kernel _qknorm_partial_rope_kernel / fused_qknorm_rope of
 * anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/fusions.py:208-274. */
int anemoi_sm100_qknorm_rope(void* x, const void* weight, const float* cos_table,
                             const float* sin_table, int64_t tokens, int32_t heads, int32_t head_dim,
                             int32_t rotary_dim, float eps, int32_t is_bf16, const int64_t* strides,
                             void* stream);

/* Measurement helper (no reference counterpart): throughput of the tcgen05 tensor pipe for one
 * MMA kind, with the instruction forms, shared-memory operand layout and 128x128 tile of the
 * attention kernel.  Launches 2 CTAs per SM that each issue 8*iterations MMAs; the caller times
 * the launch with events on `stream`.  *flops = floating-point (or integer) operations the launch
 * performs; *status (device int32, zeroed by the caller) becomes non-zero if a bounded wait gave
 * up.  It gives the per-kind denominators of the attention roofline. */
#define ANEMOI_SM100_KIND_F16 0
#define ANEMOI_SM100_KIND_I8 1
#define ANEMOI_SM100_KIND_F8 2
#define ANEMOI_SM100_KIND_NVFP4 3
int anemoi_sm100_tensor_peak(int32_t kind, int32_t iterations, int32_t* status, double* flops,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ANEMOI_SM100_H_ */
