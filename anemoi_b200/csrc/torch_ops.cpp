// Torch operator registration over the C ABI: the binding a maintainer of the reference adds so
// that its Python side can keep calling `torch.ops.<namespace>.<op>` (the form of the
// reference's own extension, csrc/attention/cuda/sm120/bindings.cpp:9-237).  Three operators
// are registered here, one per kind of call (an allocating op, an op with several outputs, an
// in-place op); the others follow the same pattern: read sizes and strides from the tensors
// into anemoi_sm100_shape, allocate outputs with at::empty, pass at::cuda's current stream,
// TORCH_CHECK the return code.  Host code only; the kernels are in libanemoi_sm100.so.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <tuple>

#include "../../include/anemoi_sm100.h"

namespace {

void* current_stream(const at::Tensor& t) {
  return c10::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

anemoi_sm100_shape pooled_shape(const at::Tensor& pool, int64_t query_block, int64_t prefix_tokens) {
  TORCH_CHECK(pool.is_cuda() && pool.dim() == 3 && pool.scalar_type() == at::kHalf && pool.is_contiguous(),
              "pools must be contiguous CUDA fp16 [heads, blocks, head_dim]");
  anemoi_sm100_shape s{};
  s.heads = (int32_t)pool.size(0);
  s.video_blocks = (int32_t)pool.size(1);
  s.head_dim = (int32_t)pool.size(2);
  s.query_block = (int32_t)query_block;
  s.prefix_tokens = (int32_t)prefix_tokens;
  s.seq_tokens = (int32_t)(prefix_tokens + pool.size(1) * query_block);
  s.has_int8 = 1;  // the routing stages do not depend on the active cells
  s.q_global_scale = s.k_global_scale = s.v_global_scale = 1.0f;
  return s;
}

// sm120_h3_draft_probability of the reference
at::Tensor draft_probability(const at::Tensor& q_pool, const at::Tensor& k_pool,
                             const c10::optional<at::Tensor>& q_max_pool,
                             const c10::optional<at::Tensor>& k_max_pool, double maxpool_weight,
                             int64_t query_block) {
  c10::cuda::CUDAGuard guard(q_pool.device());
  anemoi_sm100_shape s = pooled_shape(q_pool, query_block, 0);
  TORCH_CHECK(k_pool.sizes() == q_pool.sizes() && k_pool.is_contiguous() && k_pool.scalar_type() == at::kHalf,
              "k_pool must match q_pool");
  const bool blend = maxpool_weight != 0.0;
  TORCH_CHECK(!blend || (q_max_pool.has_value() && k_max_pool.has_value()), "max pools are required");
  s.has_maxpool = blend;
  at::Tensor prob = at::empty({q_pool.size(0), q_pool.size(1), q_pool.size(1)}, q_pool.options());
  const int rc = anemoi_sm100_draft_probability(
      &s, q_pool.data_ptr(), k_pool.data_ptr(), blend ? q_max_pool->data_ptr() : nullptr,
      blend ? k_max_pool->data_ptr() : nullptr, (float)maxpool_weight, prob.data_ptr(), current_stream(q_pool));
  TORCH_CHECK(rc == 0, "anemoi_sm100_draft_probability failed: ", rc);
  return prob;
}

// sm120_h3_route_precision + sm120_h3_materialize_route of the reference
std::tuple<at::Tensor, at::Tensor, at::Tensor> route(const at::Tensor& probability, int64_t n16, int64_t n8,
                                                     int64_t n4, int64_t prefix_phase, int64_t query_block,
                                                     int64_t prefix_tokens, int64_t head_dim) {
  c10::cuda::CUDAGuard guard(probability.device());
  TORCH_CHECK(probability.is_cuda() && probability.dim() == 3 && probability.size(1) == probability.size(2) &&
                  probability.scalar_type() == at::kHalf && probability.is_contiguous(),
              "probability must be contiguous CUDA fp16 [heads, blocks, blocks]");
  anemoi_sm100_shape s{};
  s.heads = (int32_t)probability.size(0);
  s.video_blocks = (int32_t)probability.size(1);
  s.head_dim = (int32_t)head_dim;
  s.query_block = (int32_t)query_block;
  s.prefix_tokens = (int32_t)prefix_tokens;
  s.seq_tokens = (int32_t)(prefix_tokens + probability.size(1) * query_block);
  s.has_int8 = 1;
  s.q_global_scale = s.k_global_scale = s.v_global_scale = 1.0f;
  if (prefix_tokens == 0) prefix_phase = -1;
  const int64_t scratch_bytes = anemoi_sm100_route_scratch_bytes(&s);
  const int64_t capacity = anemoi_sm100_route_list_capacity(&s, n16, n8, n4, (int)prefix_phase);
  TORCH_CHECK(scratch_bytes > 0 && capacity > 0, "invalid routing shape or budgets");
  const auto ints = probability.options().dtype(at::kInt);
  at::Tensor scratch = at::empty({scratch_bytes}, probability.options().dtype(at::kByte));
  at::Tensor row_offset = at::empty({s.heads, s.video_blocks}, ints);
  at::Tensor row_counts = at::empty({s.heads, s.video_blocks, 4}, ints);
  at::Tensor stage_ids = at::empty({s.heads, capacity}, ints);
  const int rc = anemoi_sm100_route(&s, probability.data_ptr(), n16, n8, n4, (int)prefix_phase, scratch.data_ptr(),
                                    scratch_bytes, row_offset.data_ptr<int32_t>(), row_counts.data_ptr<int32_t>(),
                                    stage_ids.data_ptr<int32_t>(), capacity, current_stream(probability));
  TORCH_CHECK(rc == 0, "anemoi_sm100_route failed: ", rc);
  return {row_offset, row_counts, stage_ids};
}

// fused_qknorm_rope of the reference (in place)
at::Tensor& qknorm_rope_(at::Tensor& x, const at::Tensor& weight, const at::Tensor& cos, const at::Tensor& sin,
                         double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.size(0) == 1 && x.stride(3) == 1 &&
                  (x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16),
              "x must be CUDA fp16/bf16 [1, tokens, heads, head_dim] with contiguous channels");
  TORCH_CHECK(weight.scalar_type() == x.scalar_type() && weight.is_contiguous() && weight.numel() == x.size(3),
              "weight must be [head_dim] of x's dtype");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() &&
                  sin.is_contiguous() && cos.dim() == 2 && cos.size(0) == x.size(1) && sin.sizes() == cos.sizes(),
              "cos / sin must be contiguous fp32 [tokens, rotary_dim]");
  const int64_t strides[2] = {x.stride(1), x.stride(2)};
  const int rc = anemoi_sm100_qknorm_rope(x.data_ptr(), weight.data_ptr(), cos.data_ptr<float>(),
                                          sin.data_ptr<float>(), x.size(1), (int32_t)x.size(2), (int32_t)x.size(3),
                                          (int32_t)cos.size(1), (float)eps, x.scalar_type() == at::kBFloat16,
                                          strides, current_stream(x));
  TORCH_CHECK(rc == 0, "anemoi_sm100_qknorm_rope failed: ", rc);
  return x;
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(anemoi_sm100, m) {
  m.def("draft_probability(Tensor q_pool, Tensor k_pool, Tensor? q_max_pool, Tensor? k_max_pool, "
        "float maxpool_weight, int query_block) -> Tensor");
  m.def("route(Tensor probability, int n16, int n8, int n4, int prefix_phase, int query_block, "
        "int prefix_tokens, int head_dim) -> (Tensor, Tensor, Tensor)");
  m.def("qknorm_rope_(Tensor(a!) x, Tensor weight, Tensor cos, Tensor sin, float eps) -> Tensor(a!)");
}

TORCH_LIBRARY_IMPL(anemoi_sm100, CUDA, m) {
  m.impl("draft_probability", &draft_probability);
  m.impl("route", &route);
  m.impl("qknorm_rope_", &qknorm_rope_);
}
