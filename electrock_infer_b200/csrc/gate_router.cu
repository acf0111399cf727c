// Gate projection fused with the router: logits = x @ Wg^T for 8 experts, then softmax + top-2,
// in one pass over the activations.
//
// In the reference the gate is a separate bf16 linear layer (ReplicatedLinear, layers/linear.py:32-54,
// called at models/mixtral.py:59) whose [T, 8] bf16 output is fed to the router
// (layers/moe/fused_moe.py:130-164).  Here a CTA owns 16 token rows and its eight warps split the
// hidden dimension; every warp multiplies its slice with mma.sync m16n8k16 (16 tokens x 8 experts,
// fp32 accumulate: N = 8 is exactly the expert count), the partial sums meet in shared memory and
// 16 threads route the rows.  The kernel is HBM-bound on the activations (2*H bytes per token), so
// the warp-level MMA is all the tensor-core work this needs.
//
// Operand mapping.  A lane loads 16 bytes (8 consecutive columns) of token rows g and g+8 and of
// gate row g (g = lane / 4): a dot product does not care about the order of its terms, so the
// lane's eight columns are fed to two MMAs as "its" k positions (2t, 2t+1, 2t+8, 2t+9 of the
// fragment layout) for A and B alike, which keeps every global load 16 bytes wide.
//
// Logits are accumulated in fp32.  With round_logits_bf16 they are rounded to bf16 before the
// softmax, which is what the reference's bf16 linear layer hands to its router; without it the
// fp32 values are used (no rounding ties).
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kExperts = 8;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRowsPerCta = 16;
constexpr int kChunk = kWarps * 32;  // hidden must split into 8 warp slices of whole 32-column steps

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kThreads)
gate_topk_softmax_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w,
                         float* __restrict__ weights, int32_t* __restrict__ indices,
                         float* __restrict__ logits_out, int64_t num_tokens, int hidden,
                         int renormalize, int round_logits_bf16) {
  __shared__ float s_part[kWarps][kRowsPerCta][kExperts];
  __shared__ float s_logit[kRowsPerCta][kExperts];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta;
  const bool valid0 = row0 + g < num_tokens, valid1 = row0 + g + 8 < num_tokens;
  const __nv_bfloat16* xr0 = x + (row0 + g) * hidden;
  const __nv_bfloat16* xr1 = x + (row0 + g + 8) * hidden;
  const __nv_bfloat16* wr = gate_w + static_cast<int64_t>(g) * hidden;
  const int slice = hidden / kWarps;
  const int kbeg = warp * slice + t * 8, kend = (warp + 1) * slice;

  float c[4] = {0.f, 0.f, 0.f, 0.f};
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 4
  for (int k = kbeg; k < kend; k += 32) {
    const uint4 a = valid0 ? ld_stream_16(xr0 + k) : zero;
    const uint4 b = valid1 ? ld_stream_16(xr1 + k) : zero;
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(wr + k));
    mma_bf16_16x8x16(c, a.x, b.x, a.y, b.y, w.x, w.y);
    mma_bf16_16x8x16(c, a.z, b.z, a.w, b.w, w.z, w.w);
  }
  // Accumulator layout: c0,c1 = row g, experts 2t,2t+1; c2,c3 = row g+8.
  s_part[warp][g][2 * t] = c[0];
  s_part[warp][g][2 * t + 1] = c[1];
  s_part[warp][g + 8][2 * t] = c[2];
  s_part[warp][g + 8][2 * t + 1] = c[3];
  __syncthreads();
  if (threadIdx.x < kRowsPerCta * kExperts) {
    const int r = threadIdx.x / kExperts, e = threadIdx.x % kExperts;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += s_part[w][r][e];
    s_logit[r][e] = round_logits_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
  }
  __syncthreads();
  const int64_t row = row0 + threadIdx.x;
  if (threadIdx.x < kRowsPerCta && row < num_tokens) {
    float l[kExperts];
#pragma unroll
    for (int e = 0; e < kExperts; ++e) l[e] = s_logit[threadIdx.x][e];
    // Ascending scan with strict '>' => the lower index wins a tie
    // (src/topk_softmax_kernels.cu:39,47 of the reference).
    float v1 = l[0], v2 = -INFINITY;
    int i1 = 0, i2 = -1;
#pragma unroll
    for (int e = 1; e < kExperts; ++e) {
      if (l[e] > v1) { v2 = v1; i2 = i1; v1 = l[e]; i1 = e; }
      else if (l[e] > v2) { v2 = l[e]; i2 = e; }
    }
    if (i2 < 0) i2 = (i1 == 0) ? 1 : 0;
    const float e2 = __expf(v2 - v1);
    float p1, p2;
    if (renormalize) {
      const float inv = 1.0f / (1.0f + e2);
      p1 = inv;
      p2 = e2 * inv;
    } else {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < kExperts; ++e) s += __expf(l[e] - v1);
      const float inv = 1.0f / s;
      p1 = inv;
      p2 = e2 * inv;
    }
    reinterpret_cast<float2*>(weights)[row] = make_float2(p1, p2);
    reinterpret_cast<int2*>(indices)[row] = make_int2(i1, i2);
    if (logits_out) {
      float4* o = reinterpret_cast<float4*>(logits_out + row * kExperts);
      o[0] = make_float4(l[0], l[1], l[2], l[3]);
      o[1] = make_float4(l[4], l[5], l[6], l[7]);
    }
  }
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_gate_topk_softmax(const void* hidden_states, const void* gate_weight,
                                         float* topk_weights, int32_t* topk_indices,
                                         float* logits_out, int64_t num_tokens, int64_t hidden,
                                         int num_experts, int topk, int renormalize,
                                         int round_logits_bf16, b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "gate_topk_softmax";
  if (num_experts != kExperts)
    return fail(B200MOE_ERR_SHAPE, "%s: compiled for num_experts=8, got %d", name, num_experts);
  if (topk != 2) return fail(B200MOE_ERR_SHAPE, "%s: assumes top_k=2, got %d", name, topk);
  if (hidden <= 0 || hidden % kChunk != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld must be a positive multiple of %d", name,
                (long long)hidden, kChunk);
  if (num_tokens < 0) return fail(B200MOE_ERR_SHAPE, "%s: num_tokens=%lld", name, (long long)num_tokens);
  if (num_tokens == 0) return B200MOE_OK;
  if (!hidden_states || !gate_weight || !topk_weights || !topk_indices)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(hidden_states, 16) || !aligned_to(gate_weight, 16) || !aligned_to(topk_weights, 8) ||
      !aligned_to(topk_indices, 8) || (logits_out && !aligned_to(logits_out, 16)))
    return fail(B200MOE_ERR_ALIGN, "%s: pointer alignment", name);
  const int64_t grid = ceil_div64(num_tokens, kRowsPerCta);
  if (grid > 0x7fffffffLL) return fail(B200MOE_ERR_SHAPE, "%s: num_tokens too large", name);
  launch_pdl(gate_topk_softmax_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(hidden_states),
             static_cast<const __nv_bfloat16*>(gate_weight), topk_weights, topk_indices, logits_out,
             num_tokens, static_cast<int>(hidden), renormalize, round_logits_bf16);
  return check_launch(name);
}
