// The whole MoE layer as one C-ABI call: the six steps that fused_experts of the reference's
// layers/moe/fused_moe.py:170-293 performs (router, token alignment, row gather, the two grouped
// GEMMs, combine), issued back to back on the caller's stream by the entry points of this library.
// A Python host saves the overhead of six bindings per call (measured: 60 us of host time per
// layer call become 27), and a C host gets the layer without re-implementing the call order.
#include "common.cuh"

namespace b200moe {
namespace {
constexpr int kLayerBlockM = 128;
}
}  // namespace b200moe

extern "C" size_t b200moe_fused_experts_rows(int64_t num_tokens, int top_k, int num_experts) {
  if (num_tokens < 0 || top_k < 1 || num_experts < 1) return 0;
  return static_cast<size_t>(num_tokens * top_k +
                             static_cast<int64_t>(num_experts) * (b200moe::kLayerBlockM - 1));
}

extern "C" int b200moe_fused_experts(const void* hidden_states, const void* gating_output,
                                     int logits_dtype, const void* w13, const void* w2, void* output,
                                     int64_t num_tokens, int num_experts, int top_k, int64_t hidden,
                                     int64_t inter, int renormalize, float* topk_weights,
                                     int32_t* topk_ids, int32_t* sorted_token_ids,
                                     int32_t* expert_ids, int32_t* num_tokens_post_pad,
                                     void* align_workspace, size_t align_workspace_bytes,
                                     void* a_sorted, void* act, void* pair_rows,
                                     b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "fused_experts";
  if (num_tokens < 0 || num_experts < 1 || hidden <= 0 || inter <= 0)
    return fail(B200MOE_ERR_SHAPE, "%s: num_tokens=%lld num_experts=%d hidden=%lld inter=%lld", name,
                (long long)num_tokens, num_experts, (long long)hidden, (long long)inter);
  if (top_k != 2)
    return fail(B200MOE_ERR_SHAPE, "%s: the combine step is written for top_k=2, got %d", name, top_k);
  if (num_tokens == 0) return B200MOE_OK;
  if (!hidden_states || !gating_output || !w13 || !w2 || !output || !topk_weights || !topk_ids ||
      !sorted_token_ids || !expert_ids || !num_tokens_post_pad || !a_sorted || !act || !pair_rows)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  const int64_t pairs = num_tokens * top_k;
  const int64_t capacity = static_cast<int64_t>(b200moe_fused_experts_rows(num_tokens, top_k, num_experts));
  const int64_t blocks = (capacity + kLayerBlockM - 1) / kLayerBlockM;
  if (int rc = b200moe_topk_softmax(topk_weights, topk_ids, gating_output, logits_dtype, num_tokens,
                                    num_experts, top_k, renormalize, stream))
    return rc;
  if (int rc = b200moe_align_block_size(topk_ids, B200MOE_I32, pairs, num_experts, kLayerBlockM,
                                        sorted_token_ids, capacity, expert_ids, blocks,
                                        num_tokens_post_pad, nullptr, /*fill_pads=*/1,
                                        align_workspace, align_workspace_bytes, stream))
    return rc;
  if (int rc = b200moe_gather_rows(hidden_states, a_sorted, sorted_token_ids, num_tokens_post_pad,
                                   capacity, num_tokens, hidden, top_k, stream))
    return rc;
  if (int rc = b200moe_grouped_gemm_w13_swiglu(a_sorted, w13, act, expert_ids, num_tokens_post_pad,
                                               capacity, num_experts, hidden, inter, kLayerBlockM,
                                               stream))
    return rc;
  if (int rc = b200moe_grouped_gemm_w2_scale(act, w2, pair_rows, topk_weights, sorted_token_ids,
                                             expert_ids, num_tokens_post_pad, capacity, pairs,
                                             num_experts, hidden, inter, kLayerBlockM, stream))
    return rc;
  return b200moe_moe_sum(pair_rows, output, B200MOE_BF16, num_tokens, hidden, top_k, /*layout=*/0,
                         stream);
}
