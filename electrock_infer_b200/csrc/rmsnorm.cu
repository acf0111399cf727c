// RMSNorm, optionally fused with the residual add, the producer of the MoE layer's input.
//
// Arithmetic follows the path the reference actually runs, RMSNorm.rms_forward / add_rms_forward
// (layers/layernorm.py:17-43; its native rms_norm / add_rms_norm, src/add_rms_norm.cu:21-200, are
// commented out at layernorm.py:50-55):
//   s = float(x) + float(residual);  residual <- cast(s);  var = mean(s^2) over the row (fp32);
//   y = cast(s * rsqrt(var + eps));  x <- y * weight  (product in the element type).
// One CTA per row, the row held in registers between the reduction and the scaling, 16-byte
// accesses: 2 reads + 2 writes of the row = 8*H bytes per token in bf16.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 8;  // 16-byte vectors per thread: rows up to 256 * 8 * 8 = 16384 elements

template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float up(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static constexpr int kVec = 8;
  __device__ static float up(__half v) { return __half2float(v); }
  __device__ static __half down(float v) { return __float2half_rn(v); }
};
template <> struct Elem<float> {
  static constexpr int kVec = 4;
  __device__ static float up(float v) { return v; }
  __device__ static float down(float v) { return v; }
};

// kNV = 16-byte vectors per thread (1, 2, 4 or 8): the row is held in kNV * kVec registers.
template <typename T, bool kResidual, int kNV>
__global__ void __launch_bounds__(kThreads)
rms_norm_kernel(T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ weight,
                int hidden, float eps) {
  constexpr int kVec = Elem<T>::kVec;
  __shared__ float s_part[kThreads / 32];
  __shared__ float s_scale;
  pdl_wait();
  pdl_launch_dependents();
  const int vecs = hidden / kVec;
  T* xrow = x + static_cast<int64_t>(blockIdx.x) * hidden;
  T* rrow = kResidual ? residual + static_cast<int64_t>(blockIdx.x) * hidden : nullptr;

  float vals[kNV][kVec];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kNV; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < vecs) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xrow + v * kVec);
      const T* xe = reinterpret_cast<const T*>(&xv);
      if (kResidual) {
        const uint4 rv = *reinterpret_cast<const uint4*>(rrow + v * kVec);
        const T* re = reinterpret_cast<const T*>(&rv);
        uint4 ov;
        T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          vals[i][j] = Elem<T>::up(xe[j]) + Elem<T>::up(re[j]);
          oe[j] = Elem<T>::down(vals[i][j]);
        }
        *reinterpret_cast<uint4*>(rrow + v * kVec) = ov;
      } else {
#pragma unroll
        for (int j = 0; j < kVec; ++j) vals[i][j] = Elem<T>::up(xe[j]);
      }
#pragma unroll
      for (int j = 0; j < kVec; ++j) sq = fmaf(vals[i][j], vals[i][j], sq);
    }
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) tot += s_part[w];
    s_scale = rsqrtf(tot / static_cast<float>(hidden) + eps);
  }
  __syncthreads();
  const float scale = s_scale;
#pragma unroll
  for (int i = 0; i < kNV; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < vecs) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight + v * kVec));
      const T* we = reinterpret_cast<const T*>(&wv);
      uint4 ov;
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const T y = Elem<T>::down(vals[i][j] * scale);
        oe[j] = Elem<T>::down(Elem<T>::up(y) * Elem<T>::up(we[j]));
      }
      *reinterpret_cast<uint4*>(xrow + v * kVec) = ov;
    }
  }
}

template <typename T>
int launch(void* x, void* residual, const void* weight, int64_t rows, int64_t hidden, float eps,
           cudaStream_t st) {
  constexpr int kVec = Elem<T>::kVec;
  if (hidden % kVec != 0 || hidden > static_cast<int64_t>(kThreads) * kMaxVec * kVec)
    return fail(B200MOE_ERR_SHAPE, "rms_norm: hidden=%lld must be a multiple of %d and at most %d",
                (long long)hidden, kVec, kThreads * kMaxVec * kVec);
  const int vecs = static_cast<int>(hidden / kVec);
  const int nv = vecs <= kThreads ? 1 : vecs <= 2 * kThreads ? 2 : vecs <= 4 * kThreads ? 4 : 8;
  const dim3 grid(static_cast<unsigned>(rows)), block(kThreads);
#define B200MOE_RMS_LAUNCH(RES, NV)                                                              \
  launch_pdl(rms_norm_kernel<T, RES, NV>, grid, block, 0, st, static_cast<T*>(x),                \
             static_cast<T*>(residual), static_cast<const T*>(weight), static_cast<int>(hidden), \
             eps)
#define B200MOE_RMS_NV(RES)                              \
  switch (nv) {                                          \
    case 1: B200MOE_RMS_LAUNCH(RES, 1); break;           \
    case 2: B200MOE_RMS_LAUNCH(RES, 2); break;           \
    case 4: B200MOE_RMS_LAUNCH(RES, 4); break;           \
    default: B200MOE_RMS_LAUNCH(RES, 8); break;          \
  }
  if (residual) {
    B200MOE_RMS_NV(true)
  } else {
    B200MOE_RMS_NV(false)
  }
#undef B200MOE_RMS_NV
#undef B200MOE_RMS_LAUNCH
  return check_launch("rms_norm");
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_add_rms_norm(void* input, void* residual, const void* weight, int dtype,
                                    int64_t num_tokens, int64_t hidden, float epsilon,
                                    b200moe_stream_t stream) {
  using namespace b200moe;
  if (num_tokens < 0 || hidden <= 0 || num_tokens > 0x7fffffffLL)
    return fail(B200MOE_ERR_SHAPE, "rms_norm: num_tokens=%lld hidden=%lld", (long long)num_tokens,
                (long long)hidden);
  if (num_tokens == 0) return B200MOE_OK;
  if (!input || !weight) return fail(B200MOE_ERR_NULL, "rms_norm: null pointer");
  if (!aligned_to(input, 16) || !aligned_to(weight, 16) || (residual && !aligned_to(residual, 16)))
    return fail(B200MOE_ERR_ALIGN, "rms_norm: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200MOE_BF16: return launch<__nv_bfloat16>(input, residual, weight, num_tokens, hidden, epsilon, st);
    case B200MOE_F16: return launch<__half>(input, residual, weight, num_tokens, hidden, epsilon, st);
    case B200MOE_F32: return launch<float>(input, residual, weight, num_tokens, hidden, epsilon, st);
    default: return fail(B200MOE_ERR_DTYPE, "rms_norm: unsupported dtype %d", dtype);
  }
}
