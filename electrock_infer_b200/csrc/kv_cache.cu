// Paged KV-cache store: the new tokens' key and value rows are copied into their slots of the
// paged caches.
//
//   key, value        [num_tokens, num_kv_heads * head_dim]   (row stride given in elements)
//   k_cache, v_cache  [num_blocks, block_size, num_kv_heads, head_dim], contiguous
//   slot_mapping      [num_tokens] int32: slot = block * block_size + offset; negative = skip
//
// The cache layout makes slot s simply row s of a [num_blocks * block_size, kv_heads * head_dim]
// matrix, which is how the reference's Triton kernel addresses it
// (layers/attention_triton_kernel.py:75-106); its HIP kernel (src/store_kv_cache.hip:12-63)
// computes the same address from (block, offset, head) and skips negative slots.  This is a pure
// copy, bound by HBM: one 64-thread group per token moves K and V rows with 16-byte accesses,
// loads issued before stores, four tokens per CTA.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 256;
constexpr int kTokensPerCta = 4;
constexpr int kGroup = kThreads / kTokensPerCta;  // 64 threads per token
constexpr int kMaxVecsPerThread = 4;              // rows up to 64 * 4 * 16 B = 4 KiB in one pass

__global__ void __launch_bounds__(kThreads)
paged_store_kvcache_kernel(const uint4* __restrict__ key, const uint4* __restrict__ value,
                           uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                           const int32_t* __restrict__ slot_mapping, int64_t num_tokens,
                           int64_t num_slots, int row_vecs, int64_t key_stride_vecs,
                           int64_t value_stride_vecs) {
  pdl_wait();
  pdl_launch_dependents();
  const int group = threadIdx.x / kGroup, t = threadIdx.x % kGroup;
  for (int64_t tok = static_cast<int64_t>(blockIdx.x) * kTokensPerCta + group; tok < num_tokens;
       tok += static_cast<int64_t>(gridDim.x) * kTokensPerCta) {
    const int64_t slot = slot_mapping[tok];
    if (slot < 0 || slot >= num_slots) continue;  // negative: not cached; too large: never written
    const uint4* ks = key + tok * key_stride_vecs;
    const uint4* vs = value + tok * value_stride_vecs;
    uint4* kd = k_cache + slot * row_vecs;
    uint4* vd = v_cache + slot * row_vecs;
    for (int c0 = t; c0 < row_vecs; c0 += kGroup * kMaxVecsPerThread) {
      uint4 k[kMaxVecsPerThread], v[kMaxVecsPerThread];
#pragma unroll
      for (int u = 0; u < kMaxVecsPerThread; ++u) {
        const int c = c0 + u * kGroup;
        if (c < row_vecs) {
          k[u] = ld_stream_16(ks + c);
          v[u] = ld_stream_16(vs + c);
        }
      }
#pragma unroll
      for (int u = 0; u < kMaxVecsPerThread; ++u) {
        const int c = c0 + u * kGroup;
        if (c < row_vecs) {
          kd[c] = k[u];
          vd[c] = v[u];
        }
      }
    }
  }
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_paged_store_kvcache(const void* key, const void* value, void* k_cache,
                                           void* v_cache, const int32_t* slot_mapping, int dtype,
                                           int64_t num_tokens, int num_kv_heads, int head_dim,
                                           int64_t key_row_stride, int64_t value_row_stride,
                                           int64_t num_blocks, int block_size,
                                           b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "paged_store_kvcache";
  int elem = 0;
  switch (dtype) {
    case B200MOE_F32: elem = 4; break;
    case B200MOE_F16:
    case B200MOE_BF16: elem = 2; break;
    default: return fail(B200MOE_ERR_DTYPE, "%s: unsupported dtype %d", name, dtype);
  }
  if (num_tokens < 0 || num_kv_heads < 1 || head_dim < 1 || num_blocks < 0 || block_size < 1)
    return fail(B200MOE_ERR_SHAPE, "%s: num_tokens=%lld kv_heads=%d head_dim=%d num_blocks=%lld "
                "block_size=%d", name, (long long)num_tokens, num_kv_heads, head_dim,
                (long long)num_blocks, block_size);
  const int64_t row_elems = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (key_row_stride < row_elems || value_row_stride < row_elems)
    return fail(B200MOE_ERR_SHAPE, "%s: row strides (%lld, %lld) smaller than a row (%lld)", name,
                (long long)key_row_stride, (long long)value_row_stride, (long long)row_elems);
  if (num_tokens == 0) return B200MOE_OK;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  const int vec = 16 / elem;
  if (row_elems % vec != 0 || key_row_stride % vec != 0 || value_row_stride % vec != 0 ||
      !aligned_to(key, 16) || !aligned_to(value, 16) || !aligned_to(k_cache, 16) ||
      !aligned_to(v_cache, 16))
    return fail(B200MOE_ERR_ALIGN, "%s: rows, row strides and base pointers must be multiples of "
                "16 bytes", name);
  int64_t grid = ceil_div64(num_tokens, kTokensPerCta);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (grid > cap) grid = cap;
  launch_pdl(paged_store_kvcache_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), static_cast<const uint4*>(key),
             static_cast<const uint4*>(value), static_cast<uint4*>(k_cache),
             static_cast<uint4*>(v_cache), slot_mapping, num_tokens,
             num_blocks * static_cast<int64_t>(block_size), static_cast<int>(row_elems / vec),
             key_row_stride / vec, value_row_stride / vec);
  return check_launch(name);
}
