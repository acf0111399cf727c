// Top-2 softmax router for 8 experts.
//
// Two lanes share a token: each loads half of the row with one vector load (fully coalesced,
// 16 bytes per lane for fp32 logits), finds its local best two, and the halves are merged with
// a single butterfly shuffle.  A lane pair handles several rows per pass so that enough loads
// are in flight to cover HBM latency.  Semantics follow src/topk_softmax_kernels.cu:8-63 of the
// reference (strict '>' while scanning upward => the lower index wins a tie; probabilities are
// softmax values, not renormalised) with the optional renormalisation of
// layers/moe/fused_moe.py:161-162.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kExperts = 8;
constexpr int kThreads = 256;
constexpr int kPairs = kThreads / 2;
constexpr int kRowsPerPair = 4;
constexpr int kRowsPerCta = kPairs * kRowsPerPair;

struct Cand {
  float v;
  int i;
};

// a is preferred over b when larger, or equal with the smaller expert index.
__device__ __forceinline__ bool better(const Cand& a, const Cand& b) {
  return a.v > b.v || (a.v == b.v && a.i < b.i);
}

template <typename T>
__device__ __forceinline__ void load_half_row(const T* row_ptr, int half, float (&v)[4]);

template <>
__device__ __forceinline__ void load_half_row<float>(const float* row_ptr, int half,
                                                      float (&v)[4]) {
  const float4 x = __ldg(reinterpret_cast<const float4*>(row_ptr) + half);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}

template <>
__device__ __forceinline__ void load_half_row<__nv_bfloat16>(const __nv_bfloat16* row_ptr,
                                                              int half, float (&v)[4]) {
  const uint2 x = __ldg(reinterpret_cast<const uint2*>(row_ptr) + half);
  v[0] = __uint_as_float(x.x << 16);
  v[1] = __uint_as_float(x.x & 0xffff0000u);
  v[2] = __uint_as_float(x.y << 16);
  v[3] = __uint_as_float(x.y & 0xffff0000u);
}

template <>
__device__ __forceinline__ void load_half_row<__half>(const __half* row_ptr, int half,
                                                       float (&v)[4]) {
  const uint2 x = __ldg(reinterpret_cast<const uint2*>(row_ptr) + half);
  const __half2 a = *reinterpret_cast<const __half2*>(&x.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&x.y);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  v[0] = fa.x; v[1] = fa.y; v[2] = fb.x; v[3] = fb.y;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
topk_softmax_kernel(const T* __restrict__ logits, float* __restrict__ weights,
                    int32_t* __restrict__ indices, int64_t num_tokens, int renormalize) {
  pdl_wait();
  pdl_launch_dependents();
  const int half = threadIdx.x & 1;
  const int pair = threadIdx.x >> 1;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + pair;

  float v[kRowsPerPair][4];
#pragma unroll
  for (int r = 0; r < kRowsPerPair; ++r) {
    const int64_t row = row0 + static_cast<int64_t>(r) * kPairs;
    if (row < num_tokens) {
      load_half_row<T>(logits + row * kExperts, half, v[r]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[r][j] = 0.f;
    }
  }

#pragma unroll
  for (int r = 0; r < kRowsPerPair; ++r) {
    const int64_t row = row0 + static_cast<int64_t>(r) * kPairs;
    // Local best two of this lane's four logits (ascending scan, strict '>').
    Cand t1{v[r][0], half * 4}, t2{-INFINITY, -1};
#pragma unroll
    for (int j = 1; j < 4; ++j) {
      const Cand c{v[r][j], half * 4 + j};
      if (c.v > t1.v) { t2 = t1; t1 = c; }
      else if (c.v > t2.v) { t2 = c; }
    }
    // Merge with the partner lane.
    Cand o1, o2;
    o1.v = __shfl_xor_sync(0xffffffffu, t1.v, 1);
    o1.i = __shfl_xor_sync(0xffffffffu, t1.i, 1);
    o2.v = __shfl_xor_sync(0xffffffffu, t2.v, 1);
    o2.i = __shfl_xor_sync(0xffffffffu, t2.i, 1);
    Cand m1, m2;
    if (better(t1, o1)) { m1 = t1; m2 = better(t2, o1) ? t2 : o1; }
    else                { m1 = o1; m2 = better(o2, t1) ? o2 : t1; }
    // A candidate with index -1 is the "none yet" sentinel of a half row; it only survives the
    // merge when NaNs are present.  Keep indices in range.
    if (m2.i < 0) m2.i = (m1.i == 0) ? 1 : 0;

    // Probabilities.  exp(l1 - max) is exactly 1, so only the runner-up needs an exponential.
    // The fast exponential (ex2.approx after a multiply) is accurate to a few 1e-7 here, well
    // inside the 1e-6 the routing weights are held to.
    const float e2 = __expf(m2.v - m1.v);
    float p1, p2;
    if (renormalize) {
      // p1 / (p1 + p2) with the common softmax denominator cancelled: no row sum is needed.
      const float inv = 1.0f / (1.0f + e2);
      p1 = inv;
      p2 = e2 * inv;
    } else {
      // Softmax denominator: each half summed in index order, low half first on both lanes.
      const float mx = m1.v;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) s += __expf(v[r][j] - mx);
      const float so = __shfl_xor_sync(0xffffffffu, s, 1);
      const float inv = 1.0f / (half ? (so + s) : (s + so));
      p1 = inv;
      p2 = e2 * inv;
    }
    if (row < num_tokens) {
      if (half == 0) {
        reinterpret_cast<float2*>(weights)[row] = make_float2(p1, p2);
      } else {
        reinterpret_cast<int2*>(indices)[row] = make_int2(m1.i, m2.i);
      }
    }
  }
}

template <typename T>
int launch(const void* logits, float* w, int32_t* ids, int64_t T_, int renorm, cudaStream_t st) {
  const int64_t grid = ceil_div64(T_, kRowsPerCta);
  launch_pdl(topk_softmax_kernel<T>, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, st,
             static_cast<const T*>(logits), w, ids, T_, renorm);
  return check_launch("topk_softmax");
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_topk_softmax(float* topk_weights, int32_t* topk_indices,
                                    const void* gating_output, int logits_dtype,
                                    int64_t num_tokens, int num_experts, int topk, int renormalize,
                                    b200moe_stream_t stream) {
  using namespace b200moe;
  if (num_experts != kExperts)
    return fail(B200MOE_ERR_SHAPE, "topk_softmax: compiled for num_experts=8, got %d", num_experts);
  if (topk != 2) return fail(B200MOE_ERR_SHAPE, "topk_softmax: assumes top_k=2, got %d", topk);
  if (num_tokens < 0) return fail(B200MOE_ERR_SHAPE, "topk_softmax: num_tokens=%lld", (long long)num_tokens);
  if (num_tokens == 0) return B200MOE_OK;
  if (num_tokens > (int64_t)kRowsPerCta * 0x7fffffffLL)
    return fail(B200MOE_ERR_SHAPE, "topk_softmax: num_tokens too large");
  if (!topk_weights || !topk_indices || !gating_output)
    return fail(B200MOE_ERR_NULL, "topk_softmax: null pointer");
  if (!aligned_to(topk_weights, 8) || !aligned_to(topk_indices, 8))
    return fail(B200MOE_ERR_ALIGN, "topk_softmax: outputs must be 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (logits_dtype) {
    case B200MOE_F32:
      if (!aligned_to(gating_output, 16))
        return fail(B200MOE_ERR_ALIGN, "topk_softmax: fp32 logits must be 16-byte aligned");
      return launch<float>(gating_output, topk_weights, topk_indices, num_tokens, renormalize, st);
    case B200MOE_BF16:
      if (!aligned_to(gating_output, 8))
        return fail(B200MOE_ERR_ALIGN, "topk_softmax: bf16 logits must be 8-byte aligned");
      return launch<__nv_bfloat16>(gating_output, topk_weights, topk_indices, num_tokens,
                                   renormalize, st);
    case B200MOE_F16:
      if (!aligned_to(gating_output, 8))
        return fail(B200MOE_ERR_ALIGN, "topk_softmax: fp16 logits must be 8-byte aligned");
      return launch<__half>(gating_output, topk_weights, topk_indices, num_tokens, renormalize, st);
    default:
      return fail(B200MOE_ERR_DTYPE, "topk_softmax: unsupported logits dtype %d", logits_dtype);
  }
}
