// Combine (moe_sum): out[t, :] = in[t, 0, :] + in[t, 1, :].
//
// Arithmetic follows the reference: src/moe_sum.cu:27-43 starts from x = 0 and adds the two
// expert rows in the element type (each 16-bit add is an fp32 add rounded once), so the result
// is round(round(0 + a) + b); starting from +0 matters only for the sign of a zero result.
// src/moe_sum_efficient.cu:23-48 adds the two adjacent values of an interleaved
// [tokens, hidden, 2] layout directly.
//
// Both layouts are pure streaming: 16-byte loads that bypass L1, several independent loads per
// thread in flight, 16-byte streaming stores.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // independent 16-byte output vectors per thread per step

template <typename T> struct Sum;

template <> struct Sum<float> {
  static constexpr int kVec = 4;
  __device__ static float add0(float a, float b) { return (0.0f + a) + b; }
  __device__ static float add(float a, float b) { return a + b; }
};
template <> struct Sum<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static __nv_bfloat16 add0(__nv_bfloat16 a, __nv_bfloat16 b) {
    const __nv_bfloat16 x = __float2bfloat16_rn(0.0f + __bfloat162float(a));
    return __float2bfloat16_rn(__bfloat162float(x) + __bfloat162float(b));
  }
  __device__ static __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b) {
    return __float2bfloat16_rn(__bfloat162float(a) + __bfloat162float(b));
  }
};
template <> struct Sum<__half> {
  static constexpr int kVec = 8;
  __device__ static __half add0(__half a, __half b) {
    const __half x = __float2half_rn(0.0f + __half2float(a));
    return __float2half_rn(__half2float(x) + __half2float(b));
  }
  __device__ static __half add(__half a, __half b) {
    return __float2half_rn(__half2float(a) + __half2float(b));
  }
};

template <typename T>
__device__ __forceinline__ uint4 add_vec(uint4 a, uint4 b) {
  constexpr int kVec = Sum<T>::kVec;
  uint4 o;
  const T* pa = reinterpret_cast<const T*>(&a);
  const T* pb = reinterpret_cast<const T*>(&b);
  T* po = reinterpret_cast<T*>(&o);
#pragma unroll
  for (int j = 0; j < kVec; ++j) po[j] = Sum<T>::add0(pa[j], pb[j]);
  return o;
}

// Layout [tokens, 2, hidden]; hidden % kVec == 0.  Work item = one 16-byte output vector.
template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_sum_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t tokens, int64_t hidden) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int kVec = Sum<T>::kVec;
  const int64_t vec_per_row = hidden / kVec;
  const int64_t total = tokens * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < total; i += kUnroll * stride) {
    uint4 a[kUnroll], b[kUnroll];
    int64_t o[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t v = i + u * stride;
      const int64_t t = v / vec_per_row, c = v - t * vec_per_row;
      const T* p = in + (t * 2) * hidden + c * kVec;
      a[u] = ld_stream_16(p);
      b[u] = ld_stream_16(p + hidden);
      o[u] = t * hidden + c * kVec;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) st_stream_16(out + o[u], add_vec<T>(a[u], b[u]));
  }
  for (; i < total; i += stride) {
    const int64_t t = i / vec_per_row, c = i - t * vec_per_row;
    const T* p = in + (t * 2) * hidden + c * kVec;
    const uint4 a = ld_stream_16(p), b = ld_stream_16(p + hidden);
    st_stream_16(out + t * hidden + c * kVec, add_vec<T>(a, b));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_sum_scalar_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t tokens,
                      int64_t hidden) {
  const int64_t total = tokens * hidden;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += stride) {
    const int64_t t = i / hidden, c = i - t * hidden;
    out[i] = Sum<T>::add0(in[(t * 2) * hidden + c], in[(t * 2 + 1) * hidden + c]);
  }
}

// Interleaved layout [tokens, hidden, 2]: output element i is in[2i] + in[2i+1].  A thread reads
// two 16-byte vectors (2*kVec inputs) and writes kVec outputs... one 16-byte vector when the
// element count allows it.
template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_sum_interleaved_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t total_vec) {
  constexpr int kVec = Sum<T>::kVec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total_vec;
       i += stride) {
    const uint4 a = ld_stream_16(in + i * 2 * kVec);
    const uint4 b = ld_stream_16(in + i * 2 * kVec + kVec);
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pb = reinterpret_cast<const T*>(&b);
    uint4 o;
    T* po = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < kVec / 2; ++j) {
      po[j] = Sum<T>::add(pa[2 * j], pa[2 * j + 1]);
      po[kVec / 2 + j] = Sum<T>::add(pb[2 * j], pb[2 * j + 1]);
    }
    st_stream_16(out + i * kVec, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_sum_interleaved_scalar_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t total) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += stride)
    out[i] = Sum<T>::add(in[2 * i], in[2 * i + 1]);
}

// Combine of the tensor-parallel layer over peer memory.  `in` is this rank's receive buffer
// [ranks, tokens, 2, hidden]: slot r holds the scaled expert rows that rank r's second GEMM stored
// here for this rank's slice of the tokens (partial sums over rank r's part of the intermediate
// dimension).  Each slot's two rows are first added and rounded to the element type exactly as
// moe_sum does on a rank of its own (the reference's tensor-parallel ranks round their partial
// result before the all-reduce, layers/moe/fused_moe.py:291 then mixtral_moe.py:114-116);
// the per-slot sums are then added in fp32 in slot order and rounded once, which for two ranks is
// the correctly rounded sum an all-reduce of the two partial results gives.  The result row is
// stored to row `row_offset + t` of EVERY rank's output tensor through `out_table`: the reduce
// step and the all-gather step of the all-reduce in one pass.  One rank computes a given row, so
// every rank ends up with the same bits.
constexpr int kMaxPushRanks = 8;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_sum_ranks_push_kernel(const T* __restrict__ in, T* const* __restrict__ out_table, int num_ranks,
                          int64_t row_offset, int64_t tokens, int64_t hidden) {
  constexpr int kVec = Sum<T>::kVec;
  __shared__ T* s_out[kMaxPushRanks];
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x < num_ranks) s_out[threadIdx.x] = out_table[threadIdx.x];
  __syncthreads();
  const int64_t vec_per_row = hidden / kVec;
  const int64_t total = tokens * vec_per_row;
  const int64_t slot = tokens * 2 * hidden;  // elements per rank slot
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += stride) {
    const int64_t t = i / vec_per_row, c = i - t * vec_per_row;
    const T* p = in + (t * 2) * hidden + c * kVec;
    float acc[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) acc[j] = 0.f;
#pragma unroll 4
    for (int r = 0; r < num_ranks; ++r) {
      const uint4 a = ld_stream_16(p + r * slot);
      const uint4 b = ld_stream_16(p + r * slot + hidden);
      const T* pa = reinterpret_cast<const T*>(&a);
      const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
      for (int j = 0; j < kVec; ++j) acc[j] += to_f32(Sum<T>::add0(pa[j], pb[j]));
    }
    uint4 o;
    T* po = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < kVec; ++j) po[j] = from_f32<T>(acc[j]);
    const int64_t dst = (row_offset + t) * hidden + c * kVec;
    for (int r = 0; r < num_ranks; ++r) *reinterpret_cast<uint4*>(s_out[r] + dst) = o;
  }
}

inline unsigned grid_for(int64_t work_per_thread_items, int per_thread) {
  int64_t grid = ceil_div64(work_per_thread_items, static_cast<int64_t>(kThreads) * per_thread);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return static_cast<unsigned>(grid);
}

template <typename T>
int launch(const void* in_v, void* out_v, int64_t tokens, int64_t hidden, int layout,
           cudaStream_t st) {
  constexpr int kVec = Sum<T>::kVec;
  const T* in = static_cast<const T*>(in_v);
  T* out = static_cast<T*>(out_v);
  const bool ptr_ok = aligned_to(in, 16) && aligned_to(out, 16);
  if (layout == 0) {
    if (ptr_ok && hidden % kVec == 0) {
      const int64_t total = tokens * (hidden / kVec);
      launch_pdl(moe_sum_vec_kernel<T>, dim3(grid_for(total, kUnroll)), dim3(kThreads), 0, st, in,
                 out, tokens, hidden);
    } else {
      moe_sum_scalar_kernel<T><<<grid_for(tokens * hidden, 1), kThreads, 0, st>>>(in, out, tokens,
                                                                                  hidden);
    }
  } else {
    const int64_t total = tokens * hidden;
    if (ptr_ok && total % kVec == 0) {
      moe_sum_interleaved_vec_kernel<T><<<grid_for(total / kVec, 1), kThreads, 0, st>>>(
          in, out, total / kVec);
    } else {
      moe_sum_interleaved_scalar_kernel<T><<<grid_for(total, 1), kThreads, 0, st>>>(in, out, total);
    }
  }
  return check_launch("moe_sum");
}

template <typename T>
int launch_ranks_push(const void* in_v, void* const* out_table, int num_ranks,
                             int64_t row_offset, int64_t tokens, int64_t hidden, cudaStream_t st) {
  constexpr int kVec = Sum<T>::kVec;
  if (hidden % kVec != 0 || !aligned_to(in_v, 16))
    return fail(B200MOE_ERR_ALIGN, "moe_sum_ranks_push: hidden must be a multiple of %d and the "
                "buffers 16-byte aligned", kVec);
  const int64_t total = tokens * (hidden / kVec);
  launch_pdl(moe_sum_ranks_push_kernel<T>, dim3(grid_for(total, 1)), dim3(kThreads), 0, st,
             static_cast<const T*>(in_v), reinterpret_cast<T* const*>(out_table), num_ranks,
             row_offset, tokens, hidden);
  return check_launch("moe_sum_ranks_push");
}


}  // namespace
}  // namespace b200moe

extern "C" int b200moe_moe_sum(const void* input, void* output, int dtype, int64_t num_tokens,
                               int64_t hidden, int topk, int layout, b200moe_stream_t stream) {
  using namespace b200moe;
  if (topk != 2) return fail(B200MOE_ERR_SHAPE, "moe_sum: this function is for top_k=2, got %d", topk);
  if (layout != 0 && layout != 1) return fail(B200MOE_ERR_SHAPE, "moe_sum: layout=%d", layout);
  if (num_tokens < 0 || hidden < 0)
    return fail(B200MOE_ERR_SHAPE, "moe_sum: num_tokens=%lld hidden=%lld", (long long)num_tokens, (long long)hidden);
  if (num_tokens == 0 || hidden == 0) return B200MOE_OK;
  if (!input || !output) return fail(B200MOE_ERR_NULL, "moe_sum: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200MOE_F32: return launch<float>(input, output, num_tokens, hidden, layout, st);
    case B200MOE_F16: return launch<__half>(input, output, num_tokens, hidden, layout, st);
    case B200MOE_BF16: return launch<__nv_bfloat16>(input, output, num_tokens, hidden, layout, st);
    default: return fail(B200MOE_ERR_DTYPE, "moe_sum: unsupported dtype %d", dtype);
  }
}

extern "C" int b200moe_moe_sum_ranks_push(const void* input, void* const* out_table, int num_ranks,
                                          int64_t row_offset, int dtype, int64_t num_tokens,
                                          int64_t hidden, int topk, b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "moe_sum_ranks_push";
  if (topk != 2) return fail(B200MOE_ERR_SHAPE, "%s: this function is for top_k=2, got %d", name, topk);
  if (num_ranks < 1 || num_ranks > kMaxPushRanks)
    return fail(B200MOE_ERR_SHAPE, "%s: num_ranks=%d outside [1, %d]", name, num_ranks, kMaxPushRanks);
  if (num_tokens < 0 || hidden < 0 || row_offset < 0)
    return fail(B200MOE_ERR_SHAPE, "%s: num_tokens=%lld hidden=%lld row_offset=%lld", name,
                (long long)num_tokens, (long long)hidden, (long long)row_offset);
  if (num_tokens == 0 || hidden == 0) return B200MOE_OK;
  if (!input || !out_table) return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200MOE_F32:
      return launch_ranks_push<float>(input, out_table, num_ranks, row_offset, num_tokens, hidden, st);
    case B200MOE_F16:
      return launch_ranks_push<__half>(input, out_table, num_ranks, row_offset, num_tokens, hidden, st);
    case B200MOE_BF16:
      return launch_ranks_push<__nv_bfloat16>(input, out_table, num_ranks, row_offset, num_tokens,
                                              hidden, st);
    default: return fail(B200MOE_ERR_DTYPE, "%s: unsupported dtype %d", name, dtype);
  }
}
