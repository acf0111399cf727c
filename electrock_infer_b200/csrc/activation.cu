// Stand-alone SwiGLU activation: out[r, j] = cast(silu_f32(in[r, j])) * in[r, d + j].
//
// Arithmetic follows src/activation_kernels.cu of the reference: the 16-bit kernel (:21-45)
// evaluates x / (1 + __expf(-x)) in fp32, rounds it to the element type and multiplies in the
// element type (a product of two 16-bit values rounded once); the fp32 kernel (:47-94) uses
// expf and multiplies in fp32.  The layer itself never launches this kernel (the activation is
// the epilogue of the first grouped GEMM); it exists for callers of the stand-alone op.
//
// Each thread handles 16 bytes of gate and 16 bytes of up per step; rows whose length or base
// address rule out 16-byte accesses take the scalar kernel.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float silu_fast(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_precise(float x) { return x / (1.0f + expf(-x)); }

template <typename T> struct Act;

template <> struct Act<float> {
  static constexpr int kVec = 4;
  __device__ static float one(float g, float u) { return silu_precise(g) * u; }
  __device__ static uint4 vec(uint4 g, uint4 u) {
    uint4 o;
    o.x = __float_as_uint(one(__uint_as_float(g.x), __uint_as_float(u.x)));
    o.y = __float_as_uint(one(__uint_as_float(g.y), __uint_as_float(u.y)));
    o.z = __float_as_uint(one(__uint_as_float(g.z), __uint_as_float(u.z)));
    o.w = __float_as_uint(one(__uint_as_float(g.w), __uint_as_float(u.w)));
    return o;
  }
};

template <> struct Act<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static __nv_bfloat16 one(__nv_bfloat16 g, __nv_bfloat16 u) {
    const __nv_bfloat16 s = __float2bfloat16_rn(silu_fast(__bfloat162float(g)));
    return __float2bfloat16_rn(__bfloat162float(s) * __bfloat162float(u));
  }
  __device__ static uint32_t two(uint32_t g, uint32_t u) {
    const __nv_bfloat162 gg = *reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162 uu = *reinterpret_cast<const __nv_bfloat162*>(&u);
    __nv_bfloat162 o;
    o.x = one(gg.x, uu.x);
    o.y = one(gg.y, uu.y);
    return *reinterpret_cast<uint32_t*>(&o);
  }
  __device__ static uint4 vec(uint4 g, uint4 u) {
    return make_uint4(two(g.x, u.x), two(g.y, u.y), two(g.z, u.z), two(g.w, u.w));
  }
};

template <> struct Act<__half> {
  static constexpr int kVec = 8;
  __device__ static __half one(__half g, __half u) {
    const __half s = __float2half_rn(silu_fast(__half2float(g)));
    return __float2half_rn(__half2float(s) * __half2float(u));
  }
  __device__ static uint32_t two(uint32_t g, uint32_t u) {
    const __half2 gg = *reinterpret_cast<const __half2*>(&g);
    const __half2 uu = *reinterpret_cast<const __half2*>(&u);
    __half2 o;
    o.x = one(gg.x, uu.x);
    o.y = one(gg.y, uu.y);
    return *reinterpret_cast<uint32_t*>(&o);
  }
  __device__ static uint4 vec(uint4 g, uint4 u) {
    return make_uint4(two(g.x, u.x), two(g.y, u.y), two(g.z, u.z), two(g.w, u.w));
  }
};

// Grid-stride over 16-byte output vectors; d is a multiple of kVec so a vector never straddles rows.
template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_and_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t num_rows,
                        int64_t d) {
  constexpr int kVec = Act<T>::kVec;
  const int64_t vec_per_row = d / kVec;
  const int64_t total = num_rows * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += stride) {
    const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
    const T* g = in + r * 2 * d + c * kVec;
    const uint4 gv = ld_stream_16(g);
    const uint4 uv = ld_stream_16(g + d);
    st_stream_16(out + r * d + c * kVec, Act<T>::vec(gv, uv));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_and_mul_scalar_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t num_rows,
                           int64_t d) {
  const int64_t total = num_rows * d;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += stride) {
    const int64_t r = i / d, c = i - r * d;
    out[i] = Act<T>::one(in[r * 2 * d + c], in[r * 2 * d + d + c]);
  }
}

template <typename T>
int launch(void* out, const void* in, int64_t rows, int64_t d, cudaStream_t st) {
  constexpr int kVec = Act<T>::kVec;
  const bool vec_ok = (d % kVec == 0) && aligned_to(out, 16) && aligned_to(in, 16);
  const int64_t work = vec_ok ? rows * (d / kVec) : rows * d;
  int64_t grid = ceil_div64(work, kThreads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (grid > cap) grid = cap;
  if (vec_ok)
    silu_and_mul_vec_kernel<T><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(
        static_cast<T*>(out), static_cast<const T*>(in), rows, d);
  else
    silu_and_mul_scalar_kernel<T><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(
        static_cast<T*>(out), static_cast<const T*>(in), rows, d);
  return check_launch("silu_and_mul");
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_silu_and_mul(void* out, const void* input, int dtype, int64_t num_rows,
                                    int64_t d, b200moe_stream_t stream) {
  using namespace b200moe;
  if (num_rows < 0 || d < 0)
    return fail(B200MOE_ERR_SHAPE, "silu_and_mul: num_rows=%lld d=%lld", (long long)num_rows, (long long)d);
  if (num_rows == 0 || d == 0) return B200MOE_OK;
  if (!out || !input) return fail(B200MOE_ERR_NULL, "silu_and_mul: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200MOE_F32: return launch<float>(out, input, num_rows, d, st);
    case B200MOE_F16: return launch<__half>(out, input, num_rows, d, st);
    case B200MOE_BF16: return launch<__nv_bfloat16>(out, input, num_rows, d, st);
    default: return fail(B200MOE_ERR_DTYPE, "silu_and_mul: unsupported dtype %d", dtype);
  }
}
