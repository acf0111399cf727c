// Decode attention over the paged KV cache with grouped queries: one query token per sequence,
// context length per sequence from `context_lens`, pages from `block_table`.
//
//   q, out            [batch, q_heads, 128]
//   k_cache, v_cache  [num_blocks, block_size, kv_heads, 128]
//   block_table       [batch, max_blocks] int32, context_lens [batch] int32
//   out[b, h] = softmax(scale * q[b, h] . K[b, h / group, :ctx]) @ V[b, h / group, :ctx]
//
// The reference kernel (src/paged_attn_gqa_varlen.hip:17-213, host wrapper :216-268; block size
// 32 and head_dim 128 only) runs one CTA per (sequence, QUERY head), so every KV head is streamed
// group_size times, and does its dot products on the scalar pipes in the element type.  Here:
//
// * one CTA per (sequence, KV head, split): the group's query heads are the rows of a 16-row
//   mma.sync tile (rows beyond the group are zero), so K and V are read from HBM once per group;
// * each of the four warps streams its own 16-token chunks through a three-stage cp.async ring
//   in shared memory (16-byte copies, XOR-swizzled so that ldmatrix is conflict-free), computes
//   S = Q K^T with m16n8k16 (fp32 accumulate), keeps a running max / sum per row (online softmax
//   in the exp2 domain) and accumulates O += P V with P rounded to the element type; rows past
//   the context length are masked in S and zero-filled in V;
// * the warps' partial (max, sum, O) are merged through shared memory; with num_splits > 1 the
//   context is cut into num_splits ranges per sequence, each CTA writes an un-normalised partial
//   to the workspace and a second small kernel merges the splits (long contexts, small batches).
//
// The kernel is bound by streaming the cache: 2 * ctx * 128 * 2 bytes per (sequence, KV head).
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kHeadDim = 128;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kChunk = 16;                       // tokens per warp step
constexpr int kStages = 3;
constexpr int kRowBytes = kHeadDim * 2;          // 256
constexpr int kTileBytes = kChunk * kRowBytes;   // 4 KiB of K (or V) per chunk
constexpr int kWarpSmem = kStages * 2 * kTileBytes;  // 24 KiB
constexpr int kSmemBytes = kWarps * kWarpSmem;       // 96 KiB: two CTAs per SM
constexpr int kMaxGroup = 16;
constexpr float kLog2e = 1.4426950408889634f;

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
  __device__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Mma<__half> {
  __device__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static uint32_t pack(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static __half from_float(float v) { return __float2half_rn(v); }
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte asynchronous copy; src_bytes = 0 writes zeros without reading.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Byte offset of 16-byte column `col16` of token row `row` inside a swizzled [16][256 B] tile.
__device__ __forceinline__ uint32_t tile_offset(int row, int col16) {
  return static_cast<uint32_t>(row * kRowBytes + ((col16 ^ (row & 7)) << 4));
}

struct Params {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  void* out;
  const int32_t* block_table;
  const int32_t* context_lens;
  float* ws_o;   // [batch, q_heads, splits, 128] un-normalised partial outputs
  float* ws_ml;  // [batch, q_heads, splits, 2] running max (log2 domain) and sum
  int q_heads, kv_heads, group, block_size, max_blocks, num_splits;
  int64_t num_blocks;
  float scale_log2;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
paged_attn_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x % p.num_splits;
  const int kvh = (blockIdx.x / p.num_splits) % p.kv_heads;
  const int seq = blockIdx.x / (p.num_splits * p.kv_heads);
  pdl_wait();
  pdl_launch_dependents();

  // A context never reaches past the pages the table row can name.
  const int ctx = min(max(p.context_lens[seq], 0), p.max_blocks * p.block_size);
  // This CTA's token range: the context cut into num_splits ranges of whole chunks.
  int per_split = (ctx + p.num_splits - 1) / p.num_splits;
  per_split = (per_split + kChunk - 1) / kChunk * kChunk;
  const int t_begin = min(split * per_split, ctx);
  const int t_end = min(t_begin + per_split, ctx);
  const int num_chunks = (t_end - t_begin + kChunk - 1) / kChunk;

  // Query rows of the group as A fragments: row g (and g + 8) of a 16 x 128 tile.
  uint32_t qa[kHeadDim / 16][4];
  {
    const T* q = static_cast<const T*>(p.q) +
                 (static_cast<int64_t>(seq) * p.q_heads + static_cast<int64_t>(kvh) * p.group) * kHeadDim;
    const bool r0 = g < p.group, r1 = g + 8 < p.group;
#pragma unroll
    for (int ks = 0; ks < kHeadDim / 16; ++ks) {
      const int c = ks * 16 + 2 * t;
      qa[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(q + g * kHeadDim + c) : 0u;
      qa[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(q + (g + 8) * kHeadDim + c) : 0u;
      qa[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(q + g * kHeadDim + c + 8) : 0u;
      qa[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(q + (g + 8) * kHeadDim + c + 8) : 0u;
    }
  }

  uint8_t* wsm = smem + warp * kWarpSmem;
  const uint32_t wsm_addr = smem_addr(wsm);
  const int32_t* table = p.block_table + static_cast<int64_t>(seq) * p.max_blocks;
  const int64_t token_stride = static_cast<int64_t>(p.kv_heads) * kHeadDim;  // elements

  // Issues the copies of this warp's chunk `ci` (K tile then V tile) into ring slot `stage`.
  auto issue = [&](int ci, int stage) {
    if (ci < num_chunks) {
      const int tok0 = t_begin + ci * kChunk;
      int page = table[tok0 / p.block_size];
      if (page < 0 || page >= p.num_blocks) page = 0;  // never dereference a bad table entry
      const int64_t row0 = static_cast<int64_t>(page) * p.block_size + tok0 % p.block_size;
      const T* kbase = static_cast<const T*>(p.k_cache) + (row0 * p.kv_heads + kvh) * kHeadDim;
      const T* vbase = static_cast<const T*>(p.v_cache) + (row0 * p.kv_heads + kvh) * kHeadDim;
      const uint32_t kdst = wsm_addr + stage * 2 * kTileBytes, vdst = kdst + kTileBytes;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = j * 32 + lane;
        const int row = idx >> 4, col16 = idx & 15;
        const bool valid = tok0 + row < t_end;
        // Rows past the range stay inside the page, but may hold anything: K is masked after
        // the product, V is zero-filled here (0 * NaN would poison the output).
        const int64_t off = (valid ? row : 0) * token_stride + col16 * 8;
        cp_async_16(kdst + tile_offset(row, col16), kbase + off, valid ? 16 : 0);
        cp_async_16(vdst + tile_offset(row, col16), vbase + off, valid ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  float o[kHeadDim / 8][4];
#pragma unroll
  for (int n = 0; n < kHeadDim / 8; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8

  // Warp w owns chunks w, w + 4, w + 8, ... of the CTA's range.
  const int my_chunks = num_chunks > warp ? (num_chunks - warp + kWarps - 1) / kWarps : 0;
  auto chunk_index = [&](int i) { return i < my_chunks ? warp + i * kWarps : num_chunks; };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(chunk_index(s), s);

  for (int i = 0; i < my_chunks; ++i) {
    const int stage = i % kStages;
    issue(chunk_index(i + kStages - 1), (i + kStages - 1) % kStages);
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const uint32_t ksm = wsm_addr + stage * 2 * kTileBytes, vsm = ksm + kTileBytes;
    const int tok0 = t_begin + (warp + i * kWarps) * kChunk;

    // S = Q K^T: two n-tiles of 8 tokens.
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < kHeadDim / 16; ++ks) {
      uint32_t kb[4];
      const int mat = lane >> 3;
      const int row = (mat >> 1) * 8 + (lane & 7);
      ldmatrix_x4(kb, ksm + tile_offset(row, 2 * ks + (mat & 1)));
      Mma<T>::run(s0, qa[ks], kb[0], kb[1]);
      Mma<T>::run(s1, qa[ks], kb[2], kb[3]);
    }
    // Scale into the exp2 domain and mask tokens past the range.
    const int c0 = tok0 + 2 * t;
    const bool v00 = c0 < t_end, v01 = c0 + 1 < t_end, v10 = c0 + 8 < t_end, v11 = c0 + 9 < t_end;
    s0[0] = v00 ? s0[0] * p.scale_log2 : -INFINITY;
    s0[1] = v01 ? s0[1] * p.scale_log2 : -INFINITY;
    s0[2] = v00 ? s0[2] * p.scale_log2 : -INFINITY;
    s0[3] = v01 ? s0[3] * p.scale_log2 : -INFINITY;
    s1[0] = v10 ? s1[0] * p.scale_log2 : -INFINITY;
    s1[1] = v11 ? s1[1] * p.scale_log2 : -INFINITY;
    s1[2] = v10 ? s1[2] * p.scale_log2 : -INFINITY;
    s1[3] = v11 ? s1[3] * p.scale_log2 : -INFINITY;
    float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
    float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // A chunk always holds at least one valid token, so the new maxima are finite.
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float a0 = exp2f(m0 - n0), a1 = exp2f(m1 - n1);  // exp2(-inf) = 0 on the first chunk
    m0 = n0;
    m1 = n1;
    s0[0] = exp2f(s0[0] - n0); s0[1] = exp2f(s0[1] - n0);
    s1[0] = exp2f(s1[0] - n0); s1[1] = exp2f(s1[1] - n0);
    s0[2] = exp2f(s0[2] - n1); s0[3] = exp2f(s0[3] - n1);
    s1[2] = exp2f(s1[2] - n1); s1[3] = exp2f(s1[3] - n1);
    float sum0 = (s0[0] + s0[1]) + (s1[0] + s1[1]);
    float sum1 = (s0[2] + s0[3]) + (s1[2] + s1[3]);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * a0 + sum0;
    l1 = l1 * a1 + sum1;
    // P as the A fragment of the second product (k = the chunk's 16 tokens).
    uint32_t pa[4];
    pa[0] = Mma<T>::pack(s0[0], s0[1]);
    pa[1] = Mma<T>::pack(s0[2], s0[3]);
    pa[2] = Mma<T>::pack(s1[0], s1[1]);
    pa[3] = Mma<T>::pack(s1[2], s1[3]);
    // O = O * alpha + P V: sixteen n-tiles of 8 dims, two per ldmatrix.
#pragma unroll
    for (int n = 0; n < kHeadDim / 8; n += 2) {
      uint32_t vb[4];
      const int mat = lane >> 3;
      const int row = (mat & 1) * 8 + (lane & 7);
      ldmatrix_x4_trans(vb, vsm + tile_offset(row, n + (mat >> 1)));
      o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1;
      o[n + 1][0] *= a0; o[n + 1][1] *= a0; o[n + 1][2] *= a1; o[n + 1][3] *= a1;
      Mma<T>::run(o[n], pa, vb[0], vb[1]);
      Mma<T>::run(o[n + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();  // the slot is refilled by the next iteration's copies
  }
  cp_async_wait<0>();
  __syncthreads();

  // Merge the four warps through shared memory (the ring is free now).
  float* sm_o = reinterpret_cast<float*>(smem);                       // [warps][16][128]
  float* sm_ml = sm_o + kWarps * 16 * kHeadDim;                       // [warps][16][2]
  {
    float* wo = sm_o + warp * 16 * kHeadDim;
#pragma unroll
    for (int n = 0; n < kHeadDim / 8; ++n) {
      *reinterpret_cast<float2*>(wo + g * kHeadDim + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
      *reinterpret_cast<float2*>(wo + (g + 8) * kHeadDim + n * 8 + 2 * t) = make_float2(o[n][2], o[n][3]);
    }
    if (t == 0) {
      sm_ml[(warp * 16 + g) * 2] = m0;
      sm_ml[(warp * 16 + g) * 2 + 1] = l0;
      sm_ml[(warp * 16 + g + 8) * 2] = m1;
      sm_ml[(warp * 16 + g + 8) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  // Thread d owns output dimension d for every row of the group.
  const int d = threadIdx.x;
  for (int r = 0; r < p.group; ++r) {
    float mw[kWarps], m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      mw[w] = sm_ml[(w * 16 + r) * 2];
      m = fmaxf(m, mw[w]);
    }
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = mw[w] == -INFINITY ? 0.f : exp2f(mw[w] - m);
      l += f * sm_ml[(w * 16 + r) * 2 + 1];
      acc += f * sm_o[(w * 16 + r) * kHeadDim + d];
    }
    const int64_t head = static_cast<int64_t>(seq) * p.q_heads + static_cast<int64_t>(kvh) * p.group + r;
    if (p.num_splits == 1) {
      // An empty context gives zeros (the reference divides 0 by 0 there).
      static_cast<T*>(p.out)[head * kHeadDim + d] = Mma<T>::from_float(l > 0.f ? acc / l : 0.f);
    } else {
      p.ws_o[(head * p.num_splits + split) * kHeadDim + d] = acc;
      if (d == 0) {
        p.ws_ml[(head * p.num_splits + split) * 2] = m;
        p.ws_ml[(head * p.num_splits + split) * 2 + 1] = l;
      }
    }
  }
}

// Merges the splits of one (sequence, query head): thread d owns dimension d.
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
paged_attn_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                        T* __restrict__ out, int num_splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t head = blockIdx.x;
  const int d = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, ws_ml[(head * num_splits + s) * 2]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = ws_ml[(head * num_splits + s) * 2];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
    l += f * ws_ml[(head * num_splits + s) * 2 + 1];
    acc += f * ws_o[(head * num_splits + s) * kHeadDim + d];
  }
  out[head * kHeadDim + d] = Mma<T>::from_float(l > 0.f ? acc / l : 0.f);
}

template <typename T>
int launch(const Params& p, int batch, cudaStream_t st) {
  // Per device and per function; cheap enough to repeat on every call.
  const cudaError_t e = cudaFuncSetAttribute(
      paged_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "paged_attn_varlen: %s", cudaGetErrorString(e));
  const int64_t ctas = static_cast<int64_t>(batch) * p.kv_heads * p.num_splits;
  launch_pdl(paged_attn_kernel<T>, dim3(static_cast<unsigned>(ctas)), dim3(kThreads), kSmemBytes, st,
             p);
  if (int rc = check_launch("paged_attn_varlen")) return rc;
  if (p.num_splits > 1) {
    launch_pdl(paged_attn_merge_kernel<T>, dim3(static_cast<unsigned>(batch * p.q_heads)),
               dim3(kHeadDim), 0, st, static_cast<const float*>(p.ws_o),
               static_cast<const float*>(p.ws_ml), static_cast<T*>(p.out), p.num_splits);
    return check_launch("paged_attn_varlen (merge)");
  }
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_paged_attn_num_splits(int batch, int kv_heads, int64_t max_context) {
  using namespace b200moe;
  if (batch < 1 || kv_heads < 1 || max_context < 1) return 1;
  // Two CTAs fit an SM.  Aim for about three waves of CTAs, so that the partial last wave costs
  // little, as long as a split still covers 512 tokens or more (measured on B200: 48 sequences
  // x 8 KV heads x 4096 tokens take 133-142 us unsplit and 121 us in 3 splits; 16 x 8 x 8192
  // take 100 us in 2 splits and 89 us in 7).
  const int64_t ctas = static_cast<int64_t>(batch) * kv_heads;
  const int64_t want = ceil_div64(6ll * sm_count(), ctas);
  const int64_t by_length = max_context / 512 > 0 ? max_context / 512 : 1;
  int64_t s = want < by_length ? want : by_length;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return static_cast<int>(s);
}

extern "C" size_t b200moe_paged_attn_workspace_bytes(int batch, int q_heads, int num_splits) {
  if (batch < 1 || q_heads < 1 || num_splits <= 1) return 0;
  return static_cast<size_t>(batch) * q_heads * num_splits * (b200moe::kHeadDim + 2) * sizeof(float);
}

extern "C" int b200moe_paged_attn_varlen(const void* q, const void* k_cache, const void* v_cache,
                                         void* out, const int32_t* block_table,
                                         const int32_t* context_lens, int dtype, int batch,
                                         int q_heads, int kv_heads, int head_dim,
                                         int64_t num_blocks, int block_size, int max_blocks_per_seq,
                                         float softmax_scale, int num_splits, void* workspace,
                                         size_t workspace_bytes, b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "paged_attn_varlen";
  if (dtype != B200MOE_BF16 && dtype != B200MOE_F16)
    return fail(B200MOE_ERR_DTYPE, "%s: bf16 or fp16 only (like the reference), got dtype %d", name, dtype);
  if (head_dim != kHeadDim)
    return fail(B200MOE_ERR_SHAPE, "%s: head_dim must be 128 (as in the reference), got %d", name, head_dim);
  if (batch < 0 || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: batch=%d q_heads=%d kv_heads=%d (q_heads must be a multiple "
                "of kv_heads)", name, batch, q_heads, kv_heads);
  const int group = q_heads / kv_heads;
  if (group > kMaxGroup)
    return fail(B200MOE_ERR_UNSUPPORTED, "%s: at most %d query heads per KV head, got %d", name,
                kMaxGroup, group);
  if (block_size < kChunk || block_size % kChunk != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: block_size must be a multiple of %d, got %d", name, kChunk,
                block_size);
  if (num_blocks < 1 || max_blocks_per_seq < 1 || num_splits < 1 || num_splits > 64)
    return fail(B200MOE_ERR_SHAPE, "%s: num_blocks=%lld max_blocks_per_seq=%d num_splits=%d", name,
                (long long)num_blocks, max_blocks_per_seq, num_splits);
  if (batch == 0) return B200MOE_OK;
  if (!q || !k_cache || !v_cache || !out || !block_table || !context_lens)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(q, 16) || !aligned_to(k_cache, 16) || !aligned_to(v_cache, 16) || !aligned_to(out, 16))
    return fail(B200MOE_ERR_ALIGN, "%s: tensors must be 16-byte aligned", name);
  if (static_cast<int64_t>(batch) * kv_heads * num_splits > 0x7fffffffLL)
    return fail(B200MOE_ERR_SHAPE, "%s: too many CTAs", name);
  Params p;
  p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_table = block_table; p.context_lens = context_lens;
  p.ws_o = nullptr; p.ws_ml = nullptr;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = group; p.block_size = block_size;
  p.max_blocks = max_blocks_per_seq; p.num_splits = num_splits; p.num_blocks = num_blocks;
  p.scale_log2 = softmax_scale * kLog2e;
  if (num_splits > 1) {
    const size_t need = b200moe_paged_attn_workspace_bytes(batch, q_heads, num_splits);
    if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16))
      return fail(B200MOE_ERR_WORKSPACE, "%s: num_splits=%d needs a 16-byte aligned workspace of "
                  "%zu bytes, got %zu", name, num_splits, need, workspace_bytes);
    p.ws_o = static_cast<float*>(workspace);
    p.ws_ml = p.ws_o + static_cast<size_t>(batch) * q_heads * num_splits * kHeadDim;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == B200MOE_BF16 ? launch<__nv_bfloat16>(p, batch, st) : launch<__half>(p, batch, st);
}
