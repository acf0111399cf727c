// Gate projection fused with the router: logits = x @ Wg^T for 8 experts, then softmax + top-2,
// in one pass over the activations.
//
// In the reference the gate is a separate bf16 linear layer (ReplicatedLinear, layers/linear.py:32-54,
// called at models/mixtral.py:59) whose [T, 8] bf16 output is fed to the router
// (layers/moe/fused_moe.py:130-164).  Here a warp reads four token rows at a time, multiplies them
// against the gate weight held in shared memory (each weight load is reused for the four rows),
// reduces the 4 x 8 partial sums with shuffles and routes the four rows.  The kernel is HBM-bound
// on the activations: 2*H bytes in per token, 16 (+32 with logits) bytes out.
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
constexpr int kRowsPerWarp = 4;
constexpr int kChunk = 32 * 8;  // columns covered by one 16-byte load per lane

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(kThreads)
gate_topk_softmax_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w,
                         float* __restrict__ weights, int32_t* __restrict__ indices,
                         float* __restrict__ logits_out, int64_t num_tokens, int hidden,
                         int renormalize, int round_logits_bf16) {
  extern __shared__ uint4 s_w[];  // [kExperts][hidden / 8] as 16-byte vectors
  pdl_wait();
  pdl_launch_dependents();
  const int vec_per_row = hidden / 8;
  for (int i = threadIdx.x; i < kExperts * vec_per_row; i += kThreads)
    s_w[i] = __ldg(reinterpret_cast<const uint4*>(gate_w) + i);
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t groups = ceil_div64(num_tokens, kRowsPerWarp);
  for (int64_t grp = static_cast<int64_t>(blockIdx.x) * kWarps + warp; grp < groups;
       grp += static_cast<int64_t>(gridDim.x) * kWarps) {
    const int64_t row0 = grp * kRowsPerWarp;
    float acc[kRowsPerWarp][kExperts];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int e = 0; e < kExperts; ++e) acc[r][e] = 0.f;

    for (int c = lane; c < vec_per_row; c += 32) {
      float xv[kRowsPerWarp][8];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row0 + r < num_tokens)
          v = ld_stream_16(reinterpret_cast<const uint4*>(x + (row0 + r) * hidden) + c);
        unpack8(v, xv[r]);
      }
#pragma unroll
      for (int e = 0; e < kExperts; ++e) {
        float wv[8];
        unpack8(s_w[e * vec_per_row + c], wv);
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[r][e] = fmaf(xv[r][j], wv[j], acc[r][e]);
      }
    }
    // Sum over lanes; every lane ends up with all 32 totals.
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int e = 0; e < kExperts; ++e)
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) acc[r][e] += __shfl_xor_sync(0xffffffffu, acc[r][e], d);

    // Lane r (r < 4) routes row r.  The select keeps acc in registers.
    float l[kExperts];
#pragma unroll
    for (int e = 0; e < kExperts; ++e) {
      float v = acc[0][e];
#pragma unroll
      for (int r = 1; r < kRowsPerWarp; ++r) v = (lane == r) ? acc[r][e] : v;
      l[e] = round_logits_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
    }
    const int64_t row = row0 + lane;
    if (lane < kRowsPerWarp && row < num_tokens) {
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
  const size_t smem = static_cast<size_t>(kExperts) * hidden * 2;
  if (smem > 200 * 1024)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld: the gate weight (%zu bytes) does not fit in shared memory",
                name, (long long)hidden, smem);
  if (num_tokens < 0) return fail(B200MOE_ERR_SHAPE, "%s: num_tokens=%lld", name, (long long)num_tokens);
  if (num_tokens == 0) return B200MOE_OK;
  if (!hidden_states || !gate_weight || !topk_weights || !topk_indices)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(hidden_states, 16) || !aligned_to(gate_weight, 16) || !aligned_to(topk_weights, 8) ||
      !aligned_to(topk_indices, 8) || (logits_out && !aligned_to(logits_out, 16)))
    return fail(B200MOE_ERR_ALIGN, "%s: pointer alignment", name);
  const cudaError_t attr = cudaFuncSetAttribute(gate_topk_softmax_kernel,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(smem));
  if (attr != cudaSuccess)
    return fail(B200MOE_ERR_CUDA, "%s: cannot reserve %zu bytes of shared memory: %s", name, smem,
                cudaGetErrorString(attr));
  const int64_t groups = ceil_div64(num_tokens, kRowsPerWarp);
  int64_t grid = ceil_div64(groups, kWarps);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 3;  // 3 CTAs of 64 KiB smem fit per SM
  if (grid > cap) grid = cap;
  launch_pdl(gate_topk_softmax_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), smem,
             static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(hidden_states),
             static_cast<const __nv_bfloat16*>(gate_weight), topk_weights, topk_indices, logits_out,
             num_tokens, static_cast<int>(hidden), renormalize, round_logits_bf16);
  return check_launch(name);
}
