// Token alignment (moe_align_block_size): a stable counting sort of the flat (token, slot) pair
// indices by expert, each expert's run padded to a multiple of block_size.
//
// Output contract follows src/moe_align_block_size.cu:58-133 of the reference:
//   cumsum[e+1] = cumsum[e] + ceil(cnt[e] / bs) * bs;  *num_tokens_post_pad = cumsum[E];
//   expert_ids[b] = e for the blocks of e;  sorted[cumsum[e] + r] = the r-th smallest pair index
//   routed to e.
//
// The reference runs one CTA of one warp.  Here a warp ranks 128 consecutive ids per step: every
// lane loads four ids with one 16-byte load, keeps eight per-expert counters packed as bytes of a
// 64-bit word, and one packed warp prefix scan yields the stable rank of all 128 ids at once.
// Inputs up to kSinglePassMax ids run as one CTA in one launch (decode-sized batches).  Longer
// inputs use three launches over segments of kSegment ids: per-segment histogram, a one-CTA scan
// over segments, and a scatter that re-reads the ids (from L2 at these sizes).
#include <mutex>

#include <cooperative_groups.h>

#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kMaxExperts = 8;          // counters are the 8 bytes of a 64-bit word
constexpr int kIdsPerLane = 4;
constexpr int kIdsPerWarpStep = 32 * kIdsPerLane;  // 128: a per-expert count fits in a byte
constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int64_t kSinglePassMax = 8192;
constexpr int kMaxCluster = 8;                // portable thread-block-cluster size
// 8 CTAs x 8192 ids.  Above this the three-launch path is faster (measured: 512 Ki ids take 24 us
// there, while a cluster needs 26 us for 128 Ki and 40 us for 256 Ki: its warps walk their
// ranges serially).
constexpr int64_t kClusterPassMax = 65536;

constexpr int kSegThreads = 256;
constexpr int kSegWarps = kSegThreads / 32;
constexpr int kSegment = 8192;  // ids per CTA of the multi-launch path

template <typename T>
__device__ __forceinline__ void load_ids4(const T* __restrict__ ids, int64_t base, int64_t numel,
                                          int num_experts, int (&e)[4]) {
  // Expert index of ids[base .. base+3]; -1 for positions past the end or out-of-range experts.
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int x = -1;
    if (base + j < numel) {
      const long long raw = static_cast<long long>(ids[base + j]);
      x = (raw >= 0 && raw < num_experts) ? static_cast<int>(raw) : -1;
    }
    e[j] = x;
  }
}

template <>
__device__ __forceinline__ void load_ids4<int32_t>(const int32_t* __restrict__ ids, int64_t base,
                                                   int64_t numel, int num_experts, int (&e)[4]) {
  if (base + 3 < numel) {
    const int4 x = __ldg(reinterpret_cast<const int4*>(ids + base));
    e[0] = x.x; e[1] = x.y; e[2] = x.z; e[3] = x.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) e[j] = (base + j < numel) ? __ldg(ids + base + j) : -1;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (static_cast<unsigned>(e[j]) >= static_cast<unsigned>(num_experts)) e[j] = -1;
}

// Byte-packed histogram of four expert ids (-1 contributes nothing).
__device__ __forceinline__ uint64_t pack_counts(const int (&e)[4]) {
  uint64_t c = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (e[j] >= 0) c += 1ull << (8 * e[j]);
  return c;
}

// Inclusive warp prefix sum of a byte-packed histogram (each byte stays <= 128).
__device__ __forceinline__ uint64_t warp_inclusive_scan(uint64_t c, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint64_t o = __shfl_up_sync(0xffffffffu, c, d);
    if (lane >= d) c += o;
  }
  return c;
}

__device__ __forceinline__ int byte_of(uint64_t c, int e) { return static_cast<int>((c >> (8 * e)) & 0xff); }

// Counts the experts of ids[begin, end) handled by one warp; result replicated on all lanes.
template <typename T>
__device__ __forceinline__ void warp_count(const T* __restrict__ ids, int64_t begin, int64_t end,
                                           int64_t numel, int num_experts, int lane,
                                           int (&cnt)[kMaxExperts]) {
#pragma unroll
  for (int x = 0; x < kMaxExperts; ++x) cnt[x] = 0;
  for (int64_t base = begin; base < end; base += kIdsPerWarpStep) {
    int e[4];
    load_ids4<T>(ids, base + lane * kIdsPerLane, end < numel ? end : numel, num_experts, e);
    uint64_t c = pack_counts(e);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
    // A byte can reach 128 only, so no carry crosses bytes.
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) cnt[x] += byte_of(c, x);
  }
}

// Writes the stable positions of ids[begin, end) handled by one warp.  start[x] is the output
// slot of the first id of expert x in this range and is advanced as the warp walks the range.
template <typename T>
__device__ __forceinline__ void warp_scatter(const T* __restrict__ ids, int64_t begin, int64_t end,
                                             int64_t numel, int num_experts, int lane,
                                             int (&start)[kMaxExperts],
                                             int32_t* __restrict__ sorted) {
  for (int64_t base = begin; base < end; base += kIdsPerWarpStep) {
    int e[4];
    const int64_t first = base + lane * kIdsPerLane;
    load_ids4<T>(ids, first, end < numel ? end : numel, num_experts, e);
    const uint64_t mine = pack_counts(e);
    const uint64_t incl = warp_inclusive_scan(mine, lane);
    uint64_t excl = incl - mine;
    const uint64_t total = __shfl_sync(0xffffffffu, incl, 31);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (e[j] >= 0) {
        int s = 0;
#pragma unroll
        for (int x = 0; x < kMaxExperts; ++x)
          if (x == e[j]) s = start[x];
        sorted[s + byte_of(excl, e[j])] = static_cast<int32_t>(first + j);
        excl += 1ull << (8 * e[j]);
      }
    }
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) start[x] += byte_of(total, x);
  }
}

// Shared tail of both paths: given the total count per expert, thread 0 publishes the padded
// offsets; then all threads write expert_ids and (optionally) the -1 padding.
__device__ __forceinline__ void publish_offsets(const int* total, int num_experts, int block_size,
                                                int* s_cumsum,
                                                int32_t* __restrict__ num_tokens_post_pad,
                                                int32_t* __restrict__ expert_offsets,
                                                bool write_global = true) {
  int acc = 0;
  s_cumsum[0] = 0;
  for (int x = 0; x < num_experts; ++x) {
    acc += (total[x] + block_size - 1) / block_size * block_size;
    s_cumsum[x + 1] = acc;
  }
  if (!write_global) return;
  *num_tokens_post_pad = acc;
  if (expert_offsets)
    for (int x = 0; x <= num_experts; ++x) expert_offsets[x] = s_cumsum[x];
}

__device__ __forceinline__ void write_blocks_and_pads(const int* s_cumsum, const int* total,
                                                      int num_experts, int block_size,
                                                      int32_t* __restrict__ sorted,
                                                      int64_t sorted_capacity,
                                                      int32_t* __restrict__ expert_ids,
                                                      int fill_pads, int tid, int nthreads) {
  const int npp = s_cumsum[num_experts];
  const int nblocks = npp / block_size;
  for (int b = tid; b < nblocks; b += nthreads) {
    const int slot = b * block_size;
    int x = 0;
    while (x + 1 < num_experts && slot >= s_cumsum[x + 1]) ++x;
    expert_ids[b] = x;
  }
  if (fill_pads) {
    for (int x = 0; x < num_experts; ++x) {
      const int lo = s_cumsum[x] + total[x], hi = s_cumsum[x + 1];
      for (int i = lo + tid; i < hi; i += nthreads) sorted[i] = -1;
    }
    for (int64_t i = npp + tid; i < sorted_capacity; i += nthreads) sorted[i] = -1;
  }
}

// ---------------------------------------------------------------------------------------------
// One launch, one CTA: count, scan and scatter with every warp owning a contiguous range.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
align_single_cta_kernel(const T* __restrict__ ids, int64_t numel, int num_experts, int block_size,
                        int32_t* __restrict__ sorted, int64_t sorted_capacity,
                        int32_t* __restrict__ expert_ids,
                        int32_t* __restrict__ num_tokens_post_pad,
                        int32_t* __restrict__ expert_offsets, int fill_pads) {
  __shared__ int s_warp_cnt[kWarps][kMaxExperts];
  __shared__ int s_total[kMaxExperts];
  __shared__ int s_cumsum[kMaxExperts + 1];

  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Contiguous range per warp, a multiple of the 128-id warp step.
  const int64_t steps = ceil_div64(numel, kIdsPerWarpStep);
  const int64_t per_warp = ceil_div64(steps, kWarps) * kIdsPerWarpStep;
  const int64_t begin = min(static_cast<int64_t>(warp) * per_warp, numel);
  const int64_t end = min(begin + per_warp, numel);

  int cnt[kMaxExperts];
  warp_count<T>(ids, begin, end, numel, num_experts, lane, cnt);
  if (lane == 0) {
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) s_warp_cnt[warp][x] = cnt[x];
  }
  __syncthreads();

  // Exclusive scan over warps, one thread per expert (32 serial adds).
  if (threadIdx.x < kMaxExperts) {
    int acc = 0;
    for (int w = 0; w < kWarps; ++w) {
      const int c = s_warp_cnt[w][threadIdx.x];
      s_warp_cnt[w][threadIdx.x] = acc;
      acc += c;
    }
    s_total[threadIdx.x] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0)
    publish_offsets(s_total, num_experts, block_size, s_cumsum, num_tokens_post_pad,
                    expert_offsets);
  __syncthreads();

  write_blocks_and_pads(s_cumsum, s_total, num_experts, block_size, sorted, sorted_capacity,
                        expert_ids, fill_pads, threadIdx.x, kThreads);

  int start[kMaxExperts];
#pragma unroll
  for (int x = 0; x < kMaxExperts; ++x)
    start[x] = (x < num_experts ? s_cumsum[x] : 0) + s_warp_cnt[warp][x];
  warp_scatter<T>(ids, begin, end, numel, num_experts, lane, start, sorted);
}

// ---------------------------------------------------------------------------------------------
// One launch, one thread-block cluster of 2, 4 or 8 CTAs: the single-CTA scheme with the ids cut
// into one slice per CTA.  The CTAs exchange their per-expert totals through distributed shared
// memory around a hardware cluster barrier, so no global scratch and no second launch is needed
// up to kClusterPassMax ids (what a layer call of up to 32 Ki tokens produces).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
align_cluster_kernel(const T* __restrict__ ids, int64_t numel, int num_experts, int block_size,
                     int32_t* __restrict__ sorted, int64_t sorted_capacity,
                     int32_t* __restrict__ expert_ids,
                     int32_t* __restrict__ num_tokens_post_pad,
                     int32_t* __restrict__ expert_offsets, int fill_pads) {
  namespace cg = cooperative_groups;
  __shared__ int s_warp_cnt[kWarps][kMaxExperts];
  __shared__ int s_cta_total[kMaxExperts];   // read by every CTA of the cluster
  __shared__ int s_cta_prefix[kMaxExperts];  // ids of each expert in the CTAs before this one
  __shared__ int s_total[kMaxExperts];
  __shared__ int s_cumsum[kMaxExperts + 1];

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int ncta = static_cast<int>(cluster.num_blocks());
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Contiguous range per warp over the whole cluster, a multiple of the 128-id warp step.
  const int64_t steps = ceil_div64(numel, kIdsPerWarpStep);
  const int64_t per_warp = ceil_div64(steps, static_cast<int64_t>(ncta) * kWarps) * kIdsPerWarpStep;
  const int64_t begin = min((static_cast<int64_t>(rank) * kWarps + warp) * per_warp, numel);
  const int64_t end = min(begin + per_warp, numel);

  int cnt[kMaxExperts];
  warp_count<T>(ids, begin, end, numel, num_experts, lane, cnt);
  if (lane == 0) {
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) s_warp_cnt[warp][x] = cnt[x];
  }
  __syncthreads();
  if (threadIdx.x < kMaxExperts) {
    int acc = 0;
    for (int w = 0; w < kWarps; ++w) {
      const int c = s_warp_cnt[w][threadIdx.x];
      s_warp_cnt[w][threadIdx.x] = acc;
      acc += c;
    }
    s_cta_total[threadIdx.x] = acc;
  }
  cluster.sync();  // every CTA's totals are in place
  if (threadIdx.x < kMaxExperts) {
    int before = 0, all = 0;
    for (int r = 0; r < ncta; ++r) {
      const int c = cluster.map_shared_rank(s_cta_total, r)[threadIdx.x];
      before += r < rank ? c : 0;
      all += c;
    }
    s_cta_prefix[threadIdx.x] = before;
    s_total[threadIdx.x] = all;
  }
  __syncthreads();
  if (threadIdx.x == 0)
    publish_offsets(s_total, num_experts, block_size, s_cumsum, num_tokens_post_pad,
                    expert_offsets, rank == 0);
  __syncthreads();

  write_blocks_and_pads(s_cumsum, s_total, num_experts, block_size, sorted, sorted_capacity,
                        expert_ids, fill_pads, rank * kThreads + threadIdx.x, ncta * kThreads);

  int start[kMaxExperts];
#pragma unroll
  for (int x = 0; x < kMaxExperts; ++x)
    start[x] = (x < num_experts ? s_cumsum[x] : 0) + s_cta_prefix[x] + s_warp_cnt[warp][x];
  warp_scatter<T>(ids, begin, end, numel, num_experts, lane, start, sorted);
  cluster.sync();  // no CTA leaves while another may still read its totals
}

// ---------------------------------------------------------------------------------------------
// Multi-launch path.  Workspace layout: int32 seg_counts[num_segments][kMaxExperts], rewritten in
// place by the scan kernel into exclusive per-expert prefixes, followed by int32
// meta[kMaxExperts + 1 + kMaxExperts] = padded offsets and totals.
// ---------------------------------------------------------------------------------------------
// Workspace words after the per-segment counters: padded offsets, then totals per expert.
constexpr int kMetaOffsets = 0;                 // meta[0 .. kMaxExperts]
constexpr int kMetaTotals = kMaxExperts + 1;    // meta[kMaxExperts + 1 .. 2 * kMaxExperts]

constexpr int kIdsPerSegWarp = kSegment / kSegWarps;             // 1024
constexpr int kSegSteps = kIdsPerSegWarp / kIdsPerWarpStep;      // 8 steps of 128 ids per warp

// Four expert ids (or -1) packed as bytes, 0xff for "none".
__device__ __forceinline__ uint32_t pack_ids(const int (&e)[4]) {
  return (static_cast<uint32_t>(e[0]) & 0xffu) | ((static_cast<uint32_t>(e[1]) & 0xffu) << 8) |
         ((static_cast<uint32_t>(e[2]) & 0xffu) << 16) | ((static_cast<uint32_t>(e[3]) & 0xffu) << 24);
}
__device__ __forceinline__ int unpack_id(uint32_t packed, int j) {
  const int x = static_cast<int>((packed >> (8 * j)) & 0xffu);
  return x == 0xff ? -1 : x;
}

// Histogram of one segment.  All loads of a warp's 1024 ids are issued before any arithmetic.
template <typename T>
__global__ void __launch_bounds__(kSegThreads)
align_count_kernel(const T* __restrict__ ids, int64_t numel, int num_experts,
                   int32_t* __restrict__ seg_counts) {
  __shared__ int s_cnt[kSegWarps][kMaxExperts];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t seg_begin = static_cast<int64_t>(blockIdx.x) * kSegment;
  const int64_t begin = min(seg_begin + static_cast<int64_t>(warp) * kIdsPerSegWarp, numel);
  const int64_t end = min(begin + kIdsPerSegWarp, numel);
  int e[kSegSteps][4];
#pragma unroll
  for (int st = 0; st < kSegSteps; ++st)
    load_ids4<T>(ids, begin + st * kIdsPerWarpStep + lane * kIdsPerLane, end, num_experts, e[st]);
  uint64_t c = 0;  // per-lane byte counters: at most 32 per expert
#pragma unroll
  for (int st = 0; st < kSegSteps; ++st) c += pack_counts(e[st]);
  // Widen to 16-bit fields before the cross-lane sum (a warp can hold 1024 ids of one expert).
  uint64_t even = c & 0x00ff00ff00ff00ffull, odd = (c >> 8) & 0x00ff00ff00ff00ffull;
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    even += __shfl_xor_sync(0xffffffffu, even, d);
    odd += __shfl_xor_sync(0xffffffffu, odd, d);
  }
  if (lane == 0) {
#pragma unroll
    for (int x = 0; x < kMaxExperts; x += 2) {
      s_cnt[warp][x] = static_cast<int>((even >> (8 * x)) & 0xffff);
      s_cnt[warp][x + 1] = static_cast<int>((odd >> (8 * x)) & 0xffff);
    }
  }
  __syncthreads();
  if (threadIdx.x < kMaxExperts) {
    int acc = 0;
    for (int w = 0; w < kSegWarps; ++w) acc += s_cnt[w][threadIdx.x];
    seg_counts[static_cast<int64_t>(blockIdx.x) * kMaxExperts + threadIdx.x] = acc;
  }
}

// One CTA turns the per-segment counts into exclusive per-expert prefixes (in place) and publishes
// the padded offsets.  Thread t owns segment chunk_base + t: its eight counts are one 32-byte
// coalesced load; each expert is scanned block-wide (warp scan + scan of the 32 warp totals).
__global__ void __launch_bounds__(kThreads)
align_scan_kernel(int32_t* __restrict__ seg_counts, int64_t num_segments, int num_experts,
                  int block_size, int32_t* __restrict__ meta,
                  int32_t* __restrict__ num_tokens_post_pad, int32_t* __restrict__ expert_offsets) {
  __shared__ int s_warp_tot[kMaxExperts][kWarps];
  __shared__ int s_carry[kMaxExperts];
  __shared__ int s_cumsum[kMaxExperts + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < kMaxExperts) s_carry[threadIdx.x] = 0;
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  for (int64_t base = 0; base < num_segments; base += kThreads) {
    const int64_t seg = base + threadIdx.x;
    int c[kMaxExperts], incl[kMaxExperts];
    if (seg < num_segments) {
      const int4 a = *reinterpret_cast<const int4*>(seg_counts + seg * kMaxExperts);
      const int4 b = *reinterpret_cast<const int4*>(seg_counts + seg * kMaxExperts + 4);
      c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
    } else {
#pragma unroll
      for (int x = 0; x < kMaxExperts; ++x) c[x] = 0;
    }
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) {
      int v = c[x];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      incl[x] = v;
      if (lane == 31) s_warp_tot[x][warp] = v;
    }
    __syncthreads();
    if (warp < kMaxExperts) {  // warp x: exclusive scan of the 32 warp totals of expert x
      const int t = s_warp_tot[warp][lane];
      int v = t;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      s_warp_tot[warp][lane] = s_carry[warp] + v - t;
      __syncwarp();
      if (lane == 31) s_carry[warp] += v;
    }
    __syncthreads();
    if (seg < num_segments) {
      int4 a, b;
      a.x = s_warp_tot[0][warp] + incl[0] - c[0]; a.y = s_warp_tot[1][warp] + incl[1] - c[1];
      a.z = s_warp_tot[2][warp] + incl[2] - c[2]; a.w = s_warp_tot[3][warp] + incl[3] - c[3];
      b.x = s_warp_tot[4][warp] + incl[4] - c[4]; b.y = s_warp_tot[5][warp] + incl[5] - c[5];
      b.z = s_warp_tot[6][warp] + incl[6] - c[6]; b.w = s_warp_tot[7][warp] + incl[7] - c[7];
      *reinterpret_cast<int4*>(seg_counts + seg * kMaxExperts) = a;
      *reinterpret_cast<int4*>(seg_counts + seg * kMaxExperts + 4) = b;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    publish_offsets(s_carry, num_experts, block_size, s_cumsum, num_tokens_post_pad,
                    expert_offsets);
    for (int x = 0; x <= kMaxExperts; ++x)
      meta[kMetaOffsets + x] = s_cumsum[x <= num_experts ? x : num_experts];
    for (int x = 0; x < kMaxExperts; ++x) meta[kMetaTotals + x] = s_carry[x];
  }
}

// Scatter of one segment.  The ids are read once and kept in registers; ranks inside the segment
// are resolved in shared memory, so that each expert's share of the segment leaves the SM as one
// contiguous run of 4-byte-coalesced stores instead of 4-byte stores scattered over eight runs.
// The CTAs also share out the writing of expert_ids and of the -1 padding.
template <typename T>
__global__ void __launch_bounds__(kSegThreads, 3)
align_scatter_kernel(const T* __restrict__ ids, int64_t numel, int num_experts, int block_size,
                     const int32_t* __restrict__ seg_prefix, const int32_t* __restrict__ meta,
                     int32_t* __restrict__ sorted, int64_t sorted_capacity,
                     int32_t* __restrict__ expert_ids, int fill_pads) {
  __shared__ int s_cnt[kSegWarps][kMaxExperts];  // per-warp counts, then exclusive prefix over warps
  __shared__ int s_base[kMaxExperts + 1];        // start of each expert's run inside the segment
  __shared__ int s_dst[kMaxExperts];             // output slot of the first element of each run
  __shared__ int s_off[kMaxExperts + 1];         // padded offsets of the whole input
  __shared__ int32_t s_sorted[kSegment];

  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t seg_begin = static_cast<int64_t>(blockIdx.x) * kSegment;
  const int64_t begin = min(seg_begin + static_cast<int64_t>(warp) * kIdsPerSegWarp, numel);
  const int64_t end = min(begin + kIdsPerSegWarp, numel);

  uint32_t packed[kSegSteps];
  uint64_t excl[kSegSteps];
  {
    int e[kSegSteps][4];
#pragma unroll
    for (int st = 0; st < kSegSteps; ++st)
      load_ids4<T>(ids, begin + st * kIdsPerWarpStep + lane * kIdsPerLane, end, num_experts, e[st]);
#pragma unroll
    for (int st = 0; st < kSegSteps; ++st) packed[st] = pack_ids(e[st]);
  }
  int cnt[kMaxExperts];
#pragma unroll
  for (int x = 0; x < kMaxExperts; ++x) cnt[x] = 0;
#pragma unroll
  for (int st = 0; st < kSegSteps; ++st) {
    int e[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) e[j] = unpack_id(packed[st], j);
    const uint64_t mine = pack_counts(e);
    const uint64_t incl = warp_inclusive_scan(mine, lane);
    excl[st] = incl - mine;
    const uint64_t total = __shfl_sync(0xffffffffu, incl, 31);
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) cnt[x] += byte_of(total, x);
  }
  if (lane == 0) {
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) s_cnt[warp][x] = cnt[x];
  }
  if (threadIdx.x <= kMaxExperts) s_off[threadIdx.x] = meta[kMetaOffsets + threadIdx.x];
  __syncthreads();
  if (threadIdx.x < kMaxExperts) {
    int acc = 0;
    for (int w = 0; w < kSegWarps; ++w) {
      const int c = s_cnt[w][threadIdx.x];
      s_cnt[w][threadIdx.x] = acc;
      acc += c;
    }
    s_base[threadIdx.x + 1] = acc;  // count for now; turned into offsets below
    s_dst[threadIdx.x] = s_off[threadIdx.x] +
                         seg_prefix[static_cast<int64_t>(blockIdx.x) * kMaxExperts + threadIdx.x];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_base[0] = 0;
    for (int x = 0; x < kMaxExperts; ++x) s_base[x + 1] += s_base[x];
  }
  __syncthreads();

  // Rank inside the segment -> shared memory.
  int start[kMaxExperts];
#pragma unroll
  for (int x = 0; x < kMaxExperts; ++x) start[x] = s_base[x] + s_cnt[warp][x];
#pragma unroll
  for (int st = 0; st < kSegSteps; ++st) {
    const int first = static_cast<int>(begin - seg_begin) + st * kIdsPerWarpStep + lane * kIdsPerLane;
    uint64_t ex = excl[st];
    uint64_t mine = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int x = unpack_id(packed[st], j);
      if (x >= 0) {
        int sx = 0;
#pragma unroll
        for (int y = 0; y < kMaxExperts; ++y)
          if (y == x) sx = start[y];
        s_sorted[sx + byte_of(ex, x)] = first + j;
        ex += 1ull << (8 * x);
        mine += 1ull << (8 * x);
      }
    }
    const uint64_t total = __shfl_sync(0xffffffffu, excl[st] + mine, 31);
#pragma unroll
    for (int x = 0; x < kMaxExperts; ++x) start[x] += byte_of(total, x);
  }
  __syncthreads();

  // Contiguous runs -> global memory.
  const int seg_count = s_base[kMaxExperts];
  const int32_t seg_first = static_cast<int32_t>(seg_begin);
  for (int i = threadIdx.x; i < seg_count; i += kSegThreads) {
    int x = 0;
#pragma unroll
    for (int y = 1; y < kMaxExperts; ++y) x += (i >= s_base[y]) ? 1 : 0;
    sorted[s_dst[x] + (i - s_base[x])] = seg_first + s_sorted[i];
  }

  // This CTA's share of expert_ids, and of the -1 padding when asked for.
  const int npp = s_off[num_experts];
  const int nblocks = npp / block_size;
  const int per_cta = (nblocks + gridDim.x - 1) / gridDim.x;
  const int b_end = min(nblocks, static_cast<int>(blockIdx.x + 1) * per_cta);
  for (int b = blockIdx.x * per_cta + threadIdx.x; b < b_end; b += kSegThreads) {
    const int slot = b * block_size;
    int x = 0;
    while (x + 1 < num_experts && slot >= s_off[x + 1]) ++x;
    expert_ids[b] = x;
  }
  if (fill_pads) {
    for (int x = blockIdx.x; x < num_experts; x += gridDim.x)
      for (int i = s_off[x] + meta[kMetaTotals + x] + threadIdx.x; i < s_off[x + 1]; i += kSegThreads)
        sorted[i] = -1;
    if (blockIdx.x == gridDim.x - 1)
      for (int64_t i = npp + threadIdx.x; i < sorted_capacity; i += kSegThreads) sorted[i] = -1;
  }
}

template <typename T>
int run(const void* ids_v, int64_t numel, int E, int bs, int32_t* sorted, int64_t cap,
        int32_t* expert_ids, int32_t* npp, int32_t* offsets, int fill, void* ws, size_t ws_bytes,
        cudaStream_t st) {
  const T* ids = static_cast<const T*>(ids_v);
  if (numel <= kSinglePassMax) {
    launch_pdl(align_single_cta_kernel<T>, dim3(1), dim3(kThreads), 0, st, ids, numel, E, bs,
               sorted, cap, expert_ids, npp, offsets, fill);
    return check_launch("moe_align_block_size");
  }
  if (numel <= kClusterPassMax) {
    int ncta = 2;
    while (ncta < kMaxCluster && numel > ncta * kSinglePassMax) ncta *= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ncta);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ncta;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, align_cluster_kernel<T>, ids, numel, E, bs, sorted, cap, expert_ids, npp,
                       offsets, fill);
    return check_launch("moe_align_block_size");
  }
  const size_t need = b200moe_align_workspace_bytes(numel, E);
  if (!ws || ws_bytes < need)
    return fail(B200MOE_ERR_WORKSPACE,
                "moe_align_block_size: %lld ids need a workspace of %zu bytes, got %zu",
                (long long)numel, need, ws ? ws_bytes : (size_t)0);
  if (!aligned_to(ws, 16))
    return fail(B200MOE_ERR_ALIGN, "moe_align_block_size: the workspace must be 16-byte aligned");
  const int64_t nseg = ceil_div64(numel, kSegment);
  int32_t* seg = static_cast<int32_t*>(ws);
  int32_t* meta = seg + nseg * kMaxExperts;
  const dim3 segs(static_cast<unsigned>(nseg));
  launch_pdl(align_count_kernel<T>, segs, dim3(kSegThreads), 0, st, ids, numel, E, seg);
  launch_pdl(align_scan_kernel, dim3(1), dim3(kThreads), 0, st, seg, nseg, E, bs, meta, npp,
             offsets);
  note_launch();  // count and scan; the scatter launch is counted by check_launch below
  note_launch();
  launch_pdl(align_scatter_kernel<T>, segs, dim3(kSegThreads), 0, st, ids, numel, E, bs,
             static_cast<const int32_t*>(seg), static_cast<const int32_t*>(meta), sorted, cap,
             expert_ids, fill);
  return check_launch("moe_align_block_size");
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the segment counters of the multi-launch path live in a fixed array
// that is part of the loaded library image on every device, instead of a caller workspace.
// ---------------------------------------------------------------------------------------------
constexpr int64_t kStaticMaxIds = 1ll << 24;  // 16 Mi pair indices = 8 Mi tokens at top-2
constexpr int64_t kStaticScratchInts =
    (kStaticMaxIds / kSegment) * kMaxExperts + 2 * kMaxExperts + 1;  // 16401 ints, about 64 KiB

static __device__ __align__(256) int32_t g_align_scratch[kStaticScratchInts];

// Device address of g_align_scratch on the current device.  In host code the array's name is only
// a handle for the runtime, not an address a kernel may use, so the address is looked up once per
// device (with that device current) and cached.
int static_scratch(int32_t** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int32_t* cached[kMaxDevices] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "align_block_size_noalloc: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(B200MOE_ERR_UNSUPPORTED, "align_block_size_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_align_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(B200MOE_ERR_CUDA, "align_block_size_noalloc: cudaGetSymbolAddress failed: %s",
                  cudaGetErrorString(e));
    cached[dev] = static_cast<int32_t*>(ptr);
  }
  *out = cached[dev];
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

extern "C" int64_t b200moe_align_noalloc_max_numel(void) { return b200moe::kStaticMaxIds; }

extern "C" int b200moe_align_block_size_noalloc(const void* topk_ids, int ids_dtype, int64_t numel,
                                                int num_experts, int block_size,
                                                int32_t* sorted_token_ids, int64_t sorted_capacity,
                                                int32_t* expert_ids, int64_t expert_ids_capacity,
                                                int32_t* num_tokens_post_pad,
                                                int32_t* expert_offsets, int fill_pads,
                                                b200moe_stream_t stream) {
  using namespace b200moe;
  if (numel > kStaticMaxIds)
    return fail(B200MOE_ERR_SHAPE,
                "align_block_size_noalloc: numel=%lld exceeds the built-in scratch limit of %lld "
                "pair indices; use b200moe_align_block_size with a workspace",
                (long long)numel, (long long)kStaticMaxIds);
  // Inputs short enough for the one-launch kernels use no scratch at all: no address look-up then,
  // so such a call does nothing but launch (also as the first call on a device, or under capture).
  int32_t* scratch = nullptr;
  if (numel > kClusterPassMax)
    if (int rc = static_scratch(&scratch)) return rc;
  // Same validation and the same kernels as the workspace variant; only the scratch differs.
  return b200moe_align_block_size(topk_ids, ids_dtype, numel, num_experts, block_size,
                                  sorted_token_ids, sorted_capacity, expert_ids,
                                  expert_ids_capacity, num_tokens_post_pad, expert_offsets,
                                  fill_pads, scratch,
                                  scratch ? static_cast<size_t>(kStaticScratchInts) * sizeof(int32_t) : 0,
                                  stream);
}

extern "C" size_t b200moe_align_workspace_bytes(int64_t numel, int num_experts) {
  using namespace b200moe;
  (void)num_experts;
  if (numel <= kClusterPassMax) return 0;
  const int64_t nseg = ceil_div64(numel, kSegment);
  return static_cast<size_t>(nseg * kMaxExperts + 2 * kMaxExperts + 1) * sizeof(int32_t);
}

extern "C" int64_t b200moe_align_single_pass_max(void) { return b200moe::kClusterPassMax; }
extern "C" int b200moe_align_max_experts(void) { return b200moe::kMaxExperts; }

extern "C" int b200moe_align_block_size(const void* topk_ids, int ids_dtype, int64_t numel,
                                        int num_experts, int block_size, int32_t* sorted_token_ids,
                                        int64_t sorted_capacity, int32_t* expert_ids,
                                        int64_t expert_ids_capacity, int32_t* num_tokens_post_pad,
                                        int32_t* expert_offsets, int fill_pads, void* workspace,
                                        size_t workspace_bytes, b200moe_stream_t stream) {
  using namespace b200moe;
  if (num_experts < 1 || num_experts > kMaxExperts)
    return fail(B200MOE_ERR_SHAPE, "moe_align_block_size: num_experts=%d, supported 1..%d",
                num_experts, kMaxExperts);
  if (block_size < 1) return fail(B200MOE_ERR_SHAPE, "moe_align_block_size: block_size=%d", block_size);
  if (numel < 0 || numel > 0x7fffffffLL - (int64_t)num_experts * block_size)
    return fail(B200MOE_ERR_SHAPE, "moe_align_block_size: numel=%lld out of range", (long long)numel);
  const int64_t need_sorted = numel + static_cast<int64_t>(num_experts) * (block_size - 1);
  if (sorted_capacity < need_sorted)
    return fail(B200MOE_ERR_SHAPE,
                "moe_align_block_size: sorted_token_ids holds %lld, needs numel + E*(block-1) = %lld",
                (long long)sorted_capacity, (long long)need_sorted);
  if (expert_ids_capacity < ceil_div64(need_sorted, block_size))
    return fail(B200MOE_ERR_SHAPE, "moe_align_block_size: expert_ids holds %lld, needs %lld",
                (long long)expert_ids_capacity, (long long)ceil_div64(need_sorted, block_size));
  if (!sorted_token_ids || !expert_ids || !num_tokens_post_pad || (numel > 0 && !topk_ids))
    return fail(B200MOE_ERR_NULL, "moe_align_block_size: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define B200MOE_ALIGN_CASE(tag, type)                                                            \
  case tag:                                                                                      \
    return run<type>(topk_ids, numel, num_experts, block_size, sorted_token_ids, sorted_capacity, \
                     expert_ids, num_tokens_post_pad, expert_offsets, fill_pads, workspace,      \
                     workspace_bytes, st)
  switch (ids_dtype) {
    case B200MOE_I32:
      if (!aligned_to(topk_ids, 16))
        return fail(B200MOE_ERR_ALIGN, "moe_align_block_size: int32 topk_ids must be 16-byte aligned");
      return run<int32_t>(topk_ids, numel, num_experts, block_size, sorted_token_ids,
                          sorted_capacity, expert_ids, num_tokens_post_pad, expert_offsets,
                          fill_pads, workspace, workspace_bytes, st);
    B200MOE_ALIGN_CASE(B200MOE_I64, int64_t);
    B200MOE_ALIGN_CASE(B200MOE_I16, int16_t);
    B200MOE_ALIGN_CASE(B200MOE_I8, int8_t);
    B200MOE_ALIGN_CASE(B200MOE_U8, uint8_t);
    default:
      return fail(B200MOE_ERR_DTYPE, "moe_align_block_size: unsupported ids dtype %d", ids_dtype);
  }
#undef B200MOE_ALIGN_CASE
}
