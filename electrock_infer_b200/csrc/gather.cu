// Row gather into expert-sorted order: dst[s, :] = src[sorted_token_ids[s] / top_k, :].
//
// The reference's grouped GEMM gathers its A rows with per-element pointer arithmetic inside the
// K loop (layers/moe/fused_moe.py:88-91).  Here the rows are copied once, with 16-byte accesses,
// so that the tensor-core kernels read dense TMA tiles.  Padding slots are zero-filled; slots at
// or beyond *num_tokens_post_pad are not touched.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 4;  // one 64-thread group per row; each thread moves 16 B per step

__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                   const int32_t* __restrict__ sorted, const int32_t* __restrict__ npp_ptr,
                   int64_t capacity, int64_t num_src_rows, int row_vecs, int top_k) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t npp = min(static_cast<int64_t>(*npp_ptr), capacity);
  const int group = threadIdx.x / (kThreads / kRowsPerCta);
  const int t = threadIdx.x % (kThreads / kRowsPerCta);
  for (int64_t s = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + group; s < npp;
       s += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const int id = sorted[s];
    const int64_t row = id >= 0 ? id / top_k : -1;
    uint4* d = dst + s * row_vecs;
    if (row >= 0 && row < num_src_rows) {
      const uint4* p = src + row * row_vecs;
      for (int c = t; c < row_vecs; c += kThreads / kRowsPerCta) d[c] = __ldg(p + c);
    } else {
      for (int c = t; c < row_vecs; c += kThreads / kRowsPerCta) d[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Row gather whose source rows live on several GPUs: token row r is row r % rows_per_rank of the
// tensor at srcs[r / rows_per_rank] (plain loads through peer mappings).  This is the dispatch
// step of the expert-parallel layer done as a pull by the GPU that owns the expert.
__global__ void __launch_bounds__(kThreads)
gather_rows_peer_kernel(const uint4* const* __restrict__ srcs, uint4* __restrict__ dst,
                        const int32_t* __restrict__ sorted, const int32_t* __restrict__ npp_ptr,
                        int64_t capacity, int num_ranks, int64_t rows_per_rank, int row_vecs,
                        int top_k) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t npp = min(static_cast<int64_t>(*npp_ptr), capacity);
  const int group = threadIdx.x / (kThreads / kRowsPerCta);
  const int t = threadIdx.x % (kThreads / kRowsPerCta);
  for (int64_t s = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + group; s < npp;
       s += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const int id = sorted[s];
    const int64_t row = id >= 0 ? id / top_k : -1;
    const int64_t rank = row >= 0 ? row / rows_per_rank : num_ranks;
    uint4* d = dst + s * row_vecs;
    if (rank < num_ranks) {
      const uint4* p = srcs[rank] + (row - rank * rows_per_rank) * row_vecs;
      // Several loads in flight per thread: a peer load costs a few microseconds.
      for (int c = t; c < row_vecs; c += 4 * (kThreads / kRowsPerCta)) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c + u * (kThreads / kRowsPerCta);
          if (cc < row_vecs) v[u] = p[cc];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c + u * (kThreads / kRowsPerCta);
          if (cc < row_vecs) d[cc] = v[u];
        }
      }
    } else {
      for (int c = t; c < row_vecs; c += kThreads / kRowsPerCta) d[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// dst[index[i], :] = src[i, :] for i < num_rows; entries with an index outside [0, num_dst_rows)
// are skipped.
__global__ void __launch_bounds__(kThreads)
scatter_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                    const int32_t* __restrict__ index, int64_t num_rows, int64_t num_dst_rows,
                    int row_vecs) {
  const int group = threadIdx.x / (kThreads / kRowsPerCta);
  const int t = threadIdx.x % (kThreads / kRowsPerCta);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + group; i < num_rows;
       i += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const int64_t row = index[i];
    if (row < 0 || row >= num_dst_rows) continue;
    const uint4* p = src + i * row_vecs;
    uint4* d = dst + row * row_vecs;
    for (int c = t; c < row_vecs; c += kThreads / kRowsPerCta) d[c] = __ldg(p + c);
  }
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_scatter_rows(const void* src, void* dst, const int32_t* index,
                                    int64_t num_rows, int64_t num_dst_rows, int64_t row_elems,
                                    b200moe_stream_t stream) {
  using namespace b200moe;
  if (row_elems <= 0 || row_elems % 8 != 0)
    return fail(B200MOE_ERR_SHAPE, "scatter_rows: row_elems=%lld must be a positive multiple of 8",
                (long long)row_elems);
  if (num_rows < 0 || num_dst_rows < 0) return fail(B200MOE_ERR_SHAPE, "scatter_rows: negative size");
  if (num_rows == 0) return B200MOE_OK;
  if (!src || !dst || !index) return fail(B200MOE_ERR_NULL, "scatter_rows: null pointer");
  if (!aligned_to(src, 16) || !aligned_to(dst, 16))
    return fail(B200MOE_ERR_ALIGN, "scatter_rows: src and dst must be 16-byte aligned");
  int64_t grid = ceil_div64(num_rows, kRowsPerCta);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  scatter_rows_kernel<<<static_cast<unsigned>(grid), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), index, num_rows, num_dst_rows,
      static_cast<int>(row_elems / 8));
  return check_launch("scatter_rows");
}

extern "C" int b200moe_gather_rows_peer(const void* const* src_table, int num_ranks,
                                        int64_t rows_per_rank, void* dst,
                                        const int32_t* sorted_token_ids,
                                        const int32_t* num_tokens_post_pad, int64_t sorted_capacity,
                                        int64_t row_elems, int top_k, b200moe_stream_t stream) {
  using namespace b200moe;
  if (row_elems <= 0 || row_elems % 8 != 0)
    return fail(B200MOE_ERR_SHAPE, "gather_rows_peer: row_elems=%lld must be a positive multiple of 8",
                (long long)row_elems);
  if (top_k < 1 || num_ranks < 1 || rows_per_rank < 1)
    return fail(B200MOE_ERR_SHAPE, "gather_rows_peer: top_k=%d num_ranks=%d rows_per_rank=%lld", top_k,
                num_ranks, (long long)rows_per_rank);
  if (sorted_capacity < 0) return fail(B200MOE_ERR_SHAPE, "gather_rows_peer: negative size");
  if (sorted_capacity == 0) return B200MOE_OK;
  if (!src_table || !dst || !sorted_token_ids || !num_tokens_post_pad)
    return fail(B200MOE_ERR_NULL, "gather_rows_peer: null pointer");
  if (!aligned_to(dst, 16)) return fail(B200MOE_ERR_ALIGN, "gather_rows_peer: dst must be 16-byte aligned");
  int64_t grid = ceil_div64(sorted_capacity, kRowsPerCta);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  launch_pdl(gather_rows_peer_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), reinterpret_cast<const uint4* const*>(src_table),
             static_cast<uint4*>(dst), sorted_token_ids, num_tokens_post_pad, sorted_capacity,
             num_ranks, rows_per_rank, static_cast<int>(row_elems / 8), top_k);
  return check_launch("gather_rows_peer");
}

extern "C" int b200moe_gather_rows(const void* src, void* dst, const int32_t* sorted_token_ids,
                                   const int32_t* num_tokens_post_pad, int64_t sorted_capacity,
                                   int64_t num_src_rows, int64_t row_elems, int top_k,
                                   b200moe_stream_t stream) {
  using namespace b200moe;
  if (row_elems <= 0 || row_elems % 8 != 0)
    return fail(B200MOE_ERR_SHAPE, "gather_rows: row_elems=%lld must be a positive multiple of 8",
                (long long)row_elems);
  if (top_k < 1) return fail(B200MOE_ERR_SHAPE, "gather_rows: top_k=%d", top_k);
  if (sorted_capacity < 0 || num_src_rows < 0) return fail(B200MOE_ERR_SHAPE, "gather_rows: negative size");
  if (sorted_capacity == 0) return B200MOE_OK;
  if (!src || !dst || !sorted_token_ids || !num_tokens_post_pad)
    return fail(B200MOE_ERR_NULL, "gather_rows: null pointer");
  if (!aligned_to(src, 16) || !aligned_to(dst, 16))
    return fail(B200MOE_ERR_ALIGN, "gather_rows: src and dst must be 16-byte aligned");
  int64_t grid = ceil_div64(sorted_capacity, kRowsPerCta);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  launch_pdl(gather_rows_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), static_cast<const uint4*>(src),
             static_cast<uint4*>(dst), sorted_token_ids, num_tokens_post_pad, sorted_capacity,
             num_src_rows, static_cast<int>(row_elems / 8), top_k);
  return check_launch("gather_rows");
}
