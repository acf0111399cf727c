// Grouped expert GEMMs of the Mixtral MoE layer for sm_100a: tcgen05.mma with fp32 accumulators in
// tensor memory (TMEM), operands staged in shared memory by TMA, persistent warp-specialised CTAs.
//
//   mode kW13: act[s, j]  = bf16( silu(g) * u ),  g/u = rows j and inter + j of w13[e]
//   mode kW2 : out[p, n]  = bf16( topk_weights[p] * sum_k act[s, k] * w2[e, n, k] ),  p = sorted[s]
//
// Both replace the reference's Triton kernel (layers/moe/fused_moe.py:15-125) for its two call
// sites (:250-255 and :282-287); the first also absorbs _C.silu_and_mul (:272).
//
// Work decomposition.  Rows are in expert-sorted, block-padded order (the output of token
// alignment with block 128), so every 128-row M block belongs to one expert.  A tile is
// 128 rows x 256 accumulator columns; for w13 the 256 columns are 128 gate columns followed by
// the 128 matching up columns, fetched as two TMA boxes of the unmodified [E, 2*inter, hidden]
// parameter, so that SiLU(g)*u is formed inside one thread without any exchange.  Tiles are
// numbered expert-major, then by groups of M blocks whose activation rows fit a share of L2,
// then N tile, then M block (M fastest): CTAs running side by side share a weight tile through
// L2 while the group's activation rows stay L2-resident.
//
// CTA layout (192 threads, one CTA per SM, grid = number of SMs):
//   warp 0      TMA producer (one lane)         smem ring of kStages x (A 16 KiB + B 32 KiB)
//   warp 1      tcgen05.mma issuer (one lane)   owns the TMEM allocation (512 columns = 2 tiles)
//   warps 2..5  epilogue: tcgen05.ld -> math -> per-warp smem staging -> 128-byte row stores
// Two TMEM accumulators let the epilogue of tile i overlap the MMAs of tile i+1.
// Variants further down: two M blocks per tile sharing each weight stage (grouped_gemm_dual_kernel,
// chosen for long batches) and CTA pairs with tcgen05 cta_group::2 (grouped_gemm_pair_kernel).
//
// Every mbarrier wait is bounded (about a second of SM clocks).  A wait that runs out sets the
// CTA's abort flag and a device status word, every role leaves its loop, TMEM is released and the
// kernel returns; the host reads the word through b200moe_gemm_device_status().
#include <cuda.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;           // accumulator columns per tile
constexpr int kBlockK = 64;            // 64 bf16 = 128 bytes = one 128B-swizzle row
constexpr int kUmmaK = 16;
#ifndef B200MOE_STAGES
#define B200MOE_STAGES 4
#endif
constexpr int kStages = B200MOE_STAGES;  // smem ring depth of the one-CTA kernel
constexpr int kABytes = kBlockM * kBlockK * 2;   // 16384
constexpr int kBBytes = kBlockN * kBlockK * 2;   // 32768
constexpr int kStageBytes = kABytes + kBBytes;   // 49152
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr int kMaxExperts = 64;
constexpr long long kWaitCycles = 1ll << 31;

constexpr int kSmemAlignSlack = 1024;
// Per epilogue warp: 32 rows x 128 bytes of output staged in shared memory (rows padded to 144
// bytes against bank conflicts) so that global stores cover whole 128-byte lines of a row.
constexpr int kOutStageRowBytes = 128 + 16;
constexpr int kOutStageBytes = kEpilogueWarps * 32 * kOutStageRowBytes;  // 18432
constexpr int kSmemBytes = kStages * kStageBytes + kOutStageBytes + kSmemAlignSlack;

// kW13Gather is kW13 with the A rows fetched straight from the token tensor by TMA row gathers.
enum Mode { kW13 = 0, kW2 = 1, kW13Gather = 2 };

// Device status word: 0 = fine; otherwise (role << 8) | barrier kind of the wait that ran out.
__device__ int g_gemm_status = 0;

// Cycle accounting of the one-block and the two-block kernel, compiled in with -DB200MOE_MEASURE_CYCLES only (a
// measurement build: the counters cost a few clock reads per K step).  Summed over all CTAs:
//   [0] cycles epilogue warp 2 spent draining accumulators   [1] accumulators drained by it
//   [2] cycles the MMA thread waited for operand stages       [3] ... for a free accumulator
//   [4] cycles the MMA thread spent in its tile loop          [5] items (tiles) it processed
//   [6], [7] the part of [2] spent in the first / the last kDualStages K steps of two-block tiles
// Read and cleared by b200moe_gemm_measured_cycles().
__device__ unsigned long long g_gemm_cycles[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#ifdef B200MOE_MEASURE_CYCLES
#define B200MOE_CYCLES_BEGIN(var) const long long var = clock64()
#define B200MOE_CYCLES_ADD(acc, var) acc += clock64() - var
#else
#define B200MOE_CYCLES_BEGIN(var)
#define B200MOE_CYCLES_ADD(acc, var)
#endif

// ------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait.  Returns false when the barrier did not flip in time or another role aborted.
// Backing off between polls (__nanosleep of 100-500 ns in the epilogue's, the producer's or the MMA
// thread's waits) was measured and changes nothing beyond run-to-run noise (first GEMM at T = 8192:
// 2.96-3.02 ms with and without, alternating processes on one GPU).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int who) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, who);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0),
      "r"(c1)
      : "memory");
}
// Bulk tensor store of a box from shared memory (bulk-group completion), and its bookkeeping.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
      : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Shared memory of every bulk store issued by this thread has been read (it may be overwritten).
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Every bulk store issued by this thread is complete.
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Makes this thread's ordinary shared-memory writes visible to the bulk-copy engine.
__device__ __forceinline__ void fence_smem_to_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Four rows of a 2-D tensor (box = 64 columns x 1 row) gathered into four consecutive 128-byte
// rows of shared memory; the 128-byte swizzle is a function of the destination address, so 32
// such gathers lay out a 128-row tile exactly like one tiled box.
__device__ __forceinline__ void tma_gather4(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int col, int r0, int r1, int r2, int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(col),
      "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes (64 elements)
// stored with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the
// leading byte offset is unused for this layout, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  const uint32_t lo = (smem_addr & 0x3ffffu) >> 4;
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, N and M as given.
constexpr uint32_t make_instr_desc(int n, int m) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct TileCoord {
  int expert;
  int m_block;
  int n_tile;
};

// Tiles are numbered expert-major; inside an expert the M blocks are cut into groups of at most
// `m_group` blocks (sizes as even as possible), and inside a group the order is N tile, then M
// block.  CTAs running side by side therefore share one weight tile through L2, and the A rows of
// a group (a few tens of MB) stay L2-resident while the group's N tiles are swept; without the
// grouping a large expert's A rows (more than L2 holds) would be re-read from HBM for every N
// tile.  The price is that an expert's weights are streamed once per group.  m_group <= 0: one
// group per expert.
__device__ __forceinline__ TileCoord decode_tile(long long tile, int n_tiles, int num_experts,
                                                 const int* blk_off, int m_group) {
  int e = 0;
  while (e + 1 < num_experts && tile >= static_cast<long long>(blk_off[e + 1]) * n_tiles) ++e;
  const int cnt = blk_off[e + 1] - blk_off[e];
  int local = static_cast<int>(tile - static_cast<long long>(blk_off[e]) * n_tiles);
  int first = 0, size = cnt;
  if (m_group > 0 && cnt > m_group) {
    const int groups = (cnt + m_group - 1) / m_group;
    const int small = cnt / groups, big_groups = cnt % groups;  // big_groups groups of small + 1
    const int big_tiles = (small + 1) * n_tiles;
    if (local < big_groups * big_tiles) {
      const int gi = local / big_tiles;
      first = gi * (small + 1);
      size = small + 1;
      local -= gi * big_tiles;
    } else {
      local -= big_groups * big_tiles;
      const int gi = local / (small * n_tiles);
      first = big_groups * (small + 1) + gi * small;
      size = small;
      local -= gi * small * n_tiles;
    }
  }
  TileCoord c;
  c.expert = e;
  c.n_tile = local / size;
  c.m_block = blk_off[e] + first + local % size;
  return c;
}

struct GemmParams {
  const int32_t* expert_ids;
  const int32_t* npp;            // *npp = padded row count (multiple of 128)
  const int32_t* sorted;         // kW2: pair index of every slot (-1 = padding)
  const float* topk_weights;     // kW2
  __nv_bfloat16* out;            // kW13: act [capacity, inter]; kW2: out [num_pairs, hidden]
  long long capacity;            // rows of the A operand
  long long num_pairs;           // kW2
  int num_experts;
  int k_blocks;                  // K / 64
  int n_tiles;                   // kW13: inter / 128; kW2: hidden / 256
  int b_rows_per_expert;         // kW13: 2 * inter; kW2: hidden
  int inter;                     // kW13: offset of the up rows inside an expert's w13
  long long out_ld;              // leading dimension of out in elements
  int half_n;                    // kW13 (one-CTA kernel): gate columns per tile; the MMA is 2*half_n wide
  uint32_t idesc;                // one-CTA kernel: instruction descriptor for that width
  int stage_tx_bytes;            // one-CTA kernel: bytes the TMA loads of one stage deliver
  __nv_bfloat16* const* out_table;  // kW2, optional: per-rank output bases (peer mappings)
  long long pairs_per_rank;      // kW2 with out_table: pair p is row p % pairs_per_rank of rank p / ...
  int m_group;                   // M blocks per L2-resident group of an expert (0: no grouping)
  int top_k;                     // kW13Gather: A row of slot s is sorted[s] / top_k
  int num_src_rows;              // kW13Gather: rows of the token tensor
  int tma_store;                 // kW13: rows leave the SM as bulk tensor stores (half_n % 64 == 0)
  int dual_pair_cost;            // > 0: the one-block and the two-block kernel are both launched and
                                 // decide on the device which of them runs (two_block_tiles_win);
                                 // time of a two-block tile in percent of a one-block tile's
  int dual_single_cost;          // ... and of a one-block item inside the two-block kernel
  int dual_ctas;                 // CTAs the work is dealt to (the SM count)
  int dual_slots;                // odd blocks are dealt as slots (first GEMM)
};

// The choice between one and two M blocks per tile, made on the device from the real block counts
// (the host only knows an upper bound of the rows, and under expert parallelism that bound is the
// whole batch while a rank receives a fraction of it).  Both kernels of a launch pair evaluate
// it on the same counts; exactly one of them does the work, the other returns after its prologue.
//
// It compares estimated finishing times, in percent of a one-block tile's time.  One-block tiles:
// whole rounds of `ctas` tiles.  Two-block tiles, measured in interleaved runs at Mixtral shape:
// a tile of two blocks takes 1.82-1.84 one-block tiles (it issues MMAs 93-98 % of the time against
// 84 %, but the board sits at its power cap either way), an odd block's one-block item inside the
// two-block kernel 1.16 (K = 14336) to 1.4 (K = 4096, where the exposed drain weighs more).
// With slots (first GEMM) every unit costs about two and the rounds are long, so the estimate is
// the mean share plus half a unit; without (second GEMM: 16 N tiles, a handful of rounds) units are
// dealt round-robin whatever they cost (whole rounds at the mean cost of a unit), and a last round
// at most half full is dealt in halves.
// Two-block tiles must win by 3 %.  This reproduces what was measured: second GEMM, skewed
// routing: one-block tiles at T = 2048, 2560 and 3072 (-15, -3 and -7 % for two-block tiles),
// two-block tiles at T = 4096 and 8192 (+10 and +8 %); first GEMM: one-block at T = 2048 and 3072,
// two-block from T = 4096 on (0 to +8 %).
__host__ __device__ inline bool two_block_tiles_win(const int* blk_off, int num_experts, int n_tiles,
                                                    int ctas, int pair_cost, int single_cost,
                                                    bool slots) {
  long long blocks = 0, pairs = 0, singles = 0;
  for (int e = 0; e < num_experts; ++e) {
    const int cnt = blk_off[e + 1] - blk_off[e];
    blocks += cnt;
    pairs += cnt >> 1;
    singles += cnt & 1;
  }
  if (pairs == 0 || ctas <= 0) return false;
  const long long one_block = (blocks * n_tiles + ctas - 1) / ctas * 100;
  long long two_block;
  if (slots) {
    const long long work = pairs * n_tiles * pair_cost + singles * n_tiles * single_cost;
    two_block = (work + ctas - 1) / ctas + pair_cost / 2;
  } else {
    const long long items = (pairs + singles) * n_tiles;
    const long long rest = items % ctas;
    const long long mean_cost = (pairs * pair_cost + singles * single_cost) / (pairs + singles);
    two_block = items / ctas * mean_cost +
                (rest == 0 ? 0 : (2 * rest > ctas ? pair_cost : single_cost));
  }
  return two_block * 103 < one_block * 100;
}


// ------------------------------------------------------------------------------ epilogue bodies
// One epilogue warp drains its 32 rows (TMEM lanes 32*quarter ..) of one 128-row accumulator.
// `taddr` addresses the warp's lanes at the accumulator's first column; `stage_out` is the warp's
// staging area in shared memory (32 rows of kOutStageRowBytes).
//
// kW13: act = bf16(silu(gate) * up).  Up to 64 output columns at a time go through the staging
// area and are written back eight lanes per row, so every store instruction covers whole 128-byte
// lines; the rows of a tile are consecutive rows of act.
// silu(g) * u in fp32 with the two special-function instructions (exp2, reciprocal) and no
// division sequence: g / (1 + e^-g) * u to about 2^-22 relative, far inside the bf16 rounding
// that follows.
__device__ __forceinline__ float silu_mul(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * r * u;
}

// N gate and N up accumulator columns of this lane's row -> N bf16 outputs in the staging row.
template <int N>
__device__ __forceinline__ void swiglu_chunk(const uint32_t (&g)[N], const uint32_t (&u)[N],
                                             uint8_t* stage_row) {
  uint4* s4 = reinterpret_cast<uint4*>(stage_row);
#pragma unroll
  for (int q = 0; q < N / 8; ++q) {
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      o[i] = pack_bf16(silu_mul(__uint_as_float(g[8 * q + 2 * i]), __uint_as_float(u[8 * q + 2 * i])),
                       silu_mul(__uint_as_float(g[8 * q + 2 * i + 1]), __uint_as_float(u[8 * q + 2 * i + 1])));
    s4[q] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// The same for the bulk-store path: the staging area is 32 dense rows of 128 bytes in the 128-byte
// swizzle the tensor map of the output expects (16-byte piece c of row r sits at piece c ^ (r & 7)),
// which also keeps the lanes' 16-byte writes on distinct banks.  `first_piece` is 0 or 4.
__device__ __forceinline__ void swiglu_chunk_swizzled(const uint32_t (&g)[32], const uint32_t (&u)[32],
                                                      uint8_t* stage_out, int row, int first_piece) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      o[i] = pack_bf16(silu_mul(__uint_as_float(g[8 * q + 2 * i]), __uint_as_float(u[8 * q + 2 * i])),
                       silu_mul(__uint_as_float(g[8 * q + 2 * i + 1]), __uint_as_float(u[8 * q + 2 * i + 1])));
    *reinterpret_cast<uint4*>(stage_out + row * 128 + (((first_piece + q) ^ (row & 7)) << 4)) =
        make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Writes `width` (<= 64, a multiple of 8) staged columns of the warp's 32 rows to consecutive rows
// of the output, eight lanes per row.
__device__ __forceinline__ void flush_rows(const uint8_t* stage_out, __nv_bfloat16* dst, long long ld,
                                           int width, int lane) {
  __syncwarp();
  const int piece = lane & 7;
  if (piece * 8 < width) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i * 4 + (lane >> 3);
      const uint4 o = *reinterpret_cast<const uint4*>(stage_out + r * kOutStageRowBytes + piece * 16);
      *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * ld + piece * 8) = o;
    }
  }
  __syncwarp();
}

// A tensor-memory load takes several hundred cycles to return while the MMAs are running
// (measured: a drain that waited for every 16-column pair of loads took 4400 cycles per
// accumulator, twice the time its arithmetic needs).  So 32 gate and 32 up columns are loaded at
// a time into one of two register sets, and the next set's loads are in flight while the current
// one goes through the special-function unit.
__device__ __forceinline__ void drain_w13(const GemmParams& p, const CUtensorMap* tmap_out,
                                          uint32_t taddr, uint8_t* stage_out, int m_block,
                                          int n_tile, int quarter, int lane) {
#ifdef B200MOE_MEASURE_WITHOUT_EPILOGUE  // measurement builds only: results are not written
  return;
#endif
  __nv_bfloat16* tile_dst = p.out +
      (static_cast<long long>(m_block) * kBlockM + quarter * 32) * p.out_ld +
      static_cast<long long>(n_tile) * p.half_n;
  uint8_t* my_row = stage_out + lane * kOutStageRowBytes;
  const int wide = p.half_n >> 5;  // chunks of 32 columns; a 16-column remainder may follow
  uint32_t ga[32], ua[32], gb[32], ub[32];
  if (wide > 0) {
    tmem_ld_32x32(taddr, ga);
    tmem_ld_32x32(taddr + p.half_n, ua);
  }
  if (p.tma_store) {
    // 64 output columns of the warp's 32 rows leave as ONE bulk tensor store issued by one lane:
    // the warp goes on with the next columns while the copy engine drains the staging area,
    // instead of pushing sixteen 16-byte store instructions per lane through the load/store path
    // that the operand loads keep busy.  half_n is a multiple of 64 here.
    const int out_row = m_block * kBlockM + quarter * 32;
    const int out_col = n_tile * p.half_n;
#pragma unroll 1
    for (int j = 0; j < wide; j += 2) {
      tmem_ld_wait();
      tmem_ld_32x32(taddr + (j + 1) * 32, gb);
      tmem_ld_32x32(taddr + p.half_n + (j + 1) * 32, ub);
      if (lane == 0) tma_store_wait_read();  // the previous store has read the staging area
      __syncwarp();
      swiglu_chunk_swizzled(ga, ua, stage_out, lane, 0);
      tmem_ld_wait();
      if (j + 2 < wide) {
        tmem_ld_32x32(taddr + (j + 2) * 32, ga);
        tmem_ld_32x32(taddr + p.half_n + (j + 2) * 32, ua);
      }
      swiglu_chunk_swizzled(gb, ub, stage_out, lane, 4);
      fence_smem_to_async_proxy();
      __syncwarp();
      if (lane == 0) tma_store_2d(tmap_out, stage_out, out_col + j * 32, out_row);
    }
    return;
  }
#pragma unroll 1
  for (int j = 0; j < wide; j += 2) {
    tmem_ld_wait();
    if (j + 1 < wide) {
      tmem_ld_32x32(taddr + (j + 1) * 32, gb);
      tmem_ld_32x32(taddr + p.half_n + (j + 1) * 32, ub);
    }
    swiglu_chunk<32>(ga, ua, my_row);
    if (j + 1 < wide) {
      tmem_ld_wait();
      if (j + 2 < wide) {
        tmem_ld_32x32(taddr + (j + 2) * 32, ga);
        tmem_ld_32x32(taddr + p.half_n + (j + 2) * 32, ua);
      }
      swiglu_chunk<32>(gb, ub, my_row + 64);
    }
    flush_rows(stage_out, tile_dst + j * 32, p.out_ld, j + 1 < wide ? 64 : 32, lane);
  }
  if (p.half_n & 16) {
    uint32_t g[16], u[16];
    tmem_ld_32x16(taddr + wide * 32, g);
    tmem_ld_32x16(taddr + p.half_n + wide * 32, u);
    tmem_ld_wait();
    swiglu_chunk<16>(g, u, my_row);
    flush_rows(stage_out, tile_dst + wide * 32, p.out_ld, 16, lane);
  }
}

// kW2: out[pair] = bf16(topk_weights[pair] * acc).  With an output table the row goes straight to
// the GPU that owns the token (a plain store through a peer mapping): the return all-to-all is
// this epilogue.  64 columns at a time: every lane scales and packs its own row into the warp's
// staging area, then the warp writes the 32 rows back out eight lanes per row, so that each store
// instruction covers four whole 128-byte lines (what a peer mapping or L2 likes) instead of 32
// scattered 16-byte pieces.  Padding slots are skipped.
__device__ __forceinline__ void drain_w2(const GemmParams& p, uint32_t taddr, uint8_t* stage_out,
                                         int m_block, int n_tile, int quarter, int lane) {
#ifdef B200MOE_MEASURE_WITHOUT_EPILOGUE  // measurement builds only: results are not written
  return;
#endif
  const long long slot = static_cast<long long>(m_block) * kBlockM + quarter * 32 + lane;
  const int pair = p.sorted[slot];
  const bool live = pair >= 0 && pair < p.num_pairs;
  const float w = live ? p.topk_weights[pair] : 0.f;
  __nv_bfloat16* base = p.out;
  long long out_row = live ? pair : 0;
  if (p.out_table != nullptr && live) {
    const long long owner = out_row / p.pairs_per_rank;
    base = p.out_table[owner];
    out_row -= owner * p.pairs_per_rank;
  }
  __nv_bfloat16* dst = base + out_row * p.out_ld + static_cast<long long>(n_tile) * kBlockN;
  const unsigned long long dst_bits = live ? reinterpret_cast<unsigned long long>(dst) : 0ull;
  // 128 columns per wait: four tensor-memory loads are in flight together (their latency, not
  // their bandwidth, is what a drain pays for, see drain_w13).
#pragma unroll 1
  for (int half = 0; half < kBlockN / 128; ++half) {
    uint32_t v[4][32];
#pragma unroll
    for (int q = 0; q < 4; ++q) tmem_ld_32x32(taddr + half * 128 + q * 32, v[q]);
    tmem_ld_wait();
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int ch = half * 2 + c;  // 64-column chunk of the tile
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4* s4 = reinterpret_cast<uint4*>(stage_out + lane * kOutStageRowBytes + h * 64);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t* w4 = &v[c * 2 + h][8 * q];
          uint4 o;
          o.x = pack_bf16(__uint_as_float(w4[0]) * w, __uint_as_float(w4[1]) * w);
          o.y = pack_bf16(__uint_as_float(w4[2]) * w, __uint_as_float(w4[3]) * w);
          o.z = pack_bf16(__uint_as_float(w4[4]) * w, __uint_as_float(w4[5]) * w);
          o.w = pack_bf16(__uint_as_float(w4[6]) * w, __uint_as_float(w4[7]) * w);
          s4[q] = o;
        }
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = i * 4 + (lane >> 3), piece = lane & 7;
        const unsigned long long row_dst = __shfl_sync(0xffffffffu, dst_bits, r);
        if (row_dst != 0ull) {
          const uint4 o = *reinterpret_cast<const uint4*>(stage_out + r * kOutStageRowBytes + piece * 16);
          *reinterpret_cast<uint4*>(row_dst + static_cast<unsigned long long>(ch) * 128 + piece * 16) = o;
        }
      }
      __syncwarp();
    }
  }
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out,   // kW13 with p.tma_store: act
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kStages], empty_bar[kStages], tmem_full_bar[2], tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_blk_cnt[kMaxExperts];
  __shared__ int s_blk_off[kMaxExperts + 1];
  __shared__ int s_abort;

  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + kSmemAlignSlack - 1) &
      ~static_cast<uintptr_t>(kSmemAlignSlack - 1));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ------------------------------------------------------------------ prologue
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], kEpilogueWarps);
    }
    s_abort = 0;
    fence_barrier_init();
  }
  if (threadIdx.x < kMaxExperts) s_blk_cnt[threadIdx.x] = 0;
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  __syncthreads();
  pdl_wait();  // everything above touched only this CTA's shared and tensor memory
  pdl_launch_dependents();
  long long npp = *p.npp;
  if (npp > p.capacity) npp = p.capacity;
  const int num_blocks = static_cast<int>(npp / kBlockM);
  for (int b = threadIdx.x; b < num_blocks; b += kThreads) {
    const int e = p.expert_ids[b];
    if (e >= 0 && e < p.num_experts) atomicAdd(&s_blk_cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.num_experts; ++e) {
      s_blk_off[e] = acc;
      acc += s_blk_cnt[e];
    }
    s_blk_off[p.num_experts] = acc;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  long long total_tiles = static_cast<long long>(s_blk_off[p.num_experts]) * p.n_tiles;
  if (p.dual_pair_cost > 0 &&
      two_block_tiles_win(s_blk_off, p.num_experts, p.n_tiles, p.dual_ctas, p.dual_pair_cost,
                          p.dual_single_cost, p.dual_slots != 0))
    total_tiles = 0;  // the two-block kernel launched beside this one does the work
  volatile int* abort_flag = &s_abort;

  constexpr bool kIsW13 = (kMode != kW2);
  if (warp == 0 && kMode == kW13Gather) {
    // ---------------------------------------------------------------- TMA producer, gathered A
    // Lane l owns slots 4l .. 4l+3 of the M block and issues one row gather per K step; lane 0
    // also owns the barrier bookkeeping and the weight loads.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const TileCoord c = decode_tile(tile, p.n_tiles, p.num_experts, s_blk_off, p.m_group);
      const int b_row0 = c.expert * p.b_rows_per_expert + c.n_tile * p.half_n;
      int rows[4];
      {
        const int4 ids = *reinterpret_cast<const int4*>(
            p.sorted + static_cast<long long>(c.m_block) * kBlockM + lane * 4);
        const int raw[4] = {ids.x, ids.y, ids.z, ids.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = raw[j] >= 0 ? raw[j] / p.top_k : 0;  // padding slots read row 0: unused
          rows[j] = r < p.num_src_rows ? r : 0;
        }
      }
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        int good = 1;
        if (lane == 0) {
          good = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 0x101) ? 1 : 0;
          if (good) mbar_expect_tx(&full_bar[stage], p.stage_tx_bytes);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        uint8_t* sa = smem + stage * kStageBytes;
        tma_gather4(sa + lane * 512, &tmap_a, &full_bar[stage], kb * kBlockK, rows[0], rows[1],
                    rows[2], rows[3]);
        if (lane == 0) {
          uint8_t* sb = sa + kABytes;
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBlockK, b_row0);
          tma_load_2d(sb + p.half_n * (kBlockK * 2), &tmap_b, &full_bar[stage], kb * kBlockK,
                      b_row0 + p.inter);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Asking L2 for the weight boxes ahead of the ring (cp.async.bulk.prefetch.tensor, eight K
    // steps ahead, by the CTA that holds the first M block of a group, also across tile
    // boundaries) was measured and is not done: -20 % at T <= 256 (0.307 -> 0.374 ms for the first
    // GEMM, which already runs at 0.95 of the HBM rate), -0 to -8 % at T = 512 to 2048, nothing
    // at T = 4096.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord c = decode_tile(tile, p.n_tiles, p.num_experts, s_blk_off, p.m_group);
        const int a_row = c.m_block * kBlockM;
        const int b_row0 = c.expert * p.b_rows_per_expert +
                           c.n_tile * (kIsW13 ? p.half_n : kBlockN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 0x101)) { ok = false; break; }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[stage], p.stage_tx_bytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kBlockK, a_row);
          if (kIsW13) {
            // Gate rows, then the matching up rows directly behind them: one B operand of
            // 2 * half_n rows.
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBlockK, b_row0);
            tma_load_2d(sb + p.half_n * (kBlockK * 2), &tmap_b, &full_bar[stage], kb * kBlockK,
                        b_row0 + p.inter);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBlockK, b_row0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long it = 0;
      long long cyc_full = 0, cyc_tmem = 0;
      B200MOE_CYCLES_BEGIN(loop_begin);
      for (long long tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
        const int acc = static_cast<int>(it & 1);
        const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
        B200MOE_CYCLES_BEGIN(w0);
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, 0x201)) { ok = false; break; }
        B200MOE_CYCLES_ADD(cyc_tmem, w0);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          B200MOE_CYCLES_BEGIN(w1);
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, 0x202)) { ok = false; break; }
          B200MOE_CYCLES_ADD(cyc_full, w1);
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t adesc = make_smem_desc(sa + k * kUmmaK * 2);
            const uint64_t bdesc = make_smem_desc(sb + k * kUmmaK * 2);
            umma_bf16(tmem_d, adesc, bdesc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage when these MMAs are done
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);  // accumulator complete
      }
#ifdef B200MOE_MEASURE_CYCLES
      atomicAdd(&g_gemm_cycles[2], static_cast<unsigned long long>(cyc_full));
      atomicAdd(&g_gemm_cycles[3], static_cast<unsigned long long>(cyc_tmem));
      atomicAdd(&g_gemm_cycles[4], static_cast<unsigned long long>(clock64() - loop_begin));
      atomicAdd(&g_gemm_cycles[5], static_cast<unsigned long long>(it));
#endif
      (void)cyc_full;
      (void)cyc_tmem;
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;               // TMEM lanes this warp may read: 32*quarter ..
    bool ok = true;
    long long it = 0;
    long long cyc_drain = 0;
    for (long long tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      const TileCoord c = decode_tile(tile, p.n_tiles, p.num_experts, s_blk_off, p.m_group);
      const int acc = static_cast<int>(it & 1);
      const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
      // All lanes of the warp must leave together: the wait result is made warp-uniform.
      int good = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, 0x301) ? 1 : 0;
      good = __all_sync(0xffffffffu, good);
      if (!good) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * kBlockN);
      // Bulk stores read dense 128-byte rows from a 1024-byte aligned area; the other paths use
      // rows padded to 144 bytes.
      uint8_t* stage_out = smem + kStages * kStageBytes +
                           (warp - 2) * ((kIsW13 && p.tma_store) ? 32 * 128 : 32 * kOutStageRowBytes);
      B200MOE_CYCLES_BEGIN(d0);
      if (kIsW13) {
        drain_w13(p, &tmap_out, taddr, stage_out, c.m_block, c.n_tile, quarter, lane);
      } else {
        drain_w2(p, taddr, stage_out, c.m_block, c.n_tile, quarter, lane);
      }
      B200MOE_CYCLES_ADD(cyc_drain, d0);
      // Hand the accumulator back to the MMA warp.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
    }
#ifdef B200MOE_MEASURE_CYCLES
    if (warp == 2 && lane == 0) {
      atomicAdd(&g_gemm_cycles[0], static_cast<unsigned long long>(cyc_drain));
      atomicAdd(&g_gemm_cycles[1], static_cast<unsigned long long>(it));
    }
#endif
    (void)cyc_drain;
    if (kIsW13 && p.tma_store && lane == 0) tma_store_wait_all();  // before shared memory goes away
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // Give bulk copies that may still be in flight time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < (1ll << 22)) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ================================================================================================
// Two-block variant of the one-CTA kernel: one CTA computes TWO 128-row M blocks of the same expert
// against one weight stage.  Per 256 x 256 x 64 multiply-accumulates it stages 32 KiB of
// activation rows (one TMA box of 256 consecutive rows) and 32 KiB of weights, instead of 2 x 48 KiB
// for two independent 128 x 256 tiles, while the MMAs stay M = 128 and token alignment stays 128.
//
// Both 256-column halves of TMEM are accumulators of the same tile, so tile i + 1 cannot start
// while tile i is drained from both.  The overlap that is left: the epilogue drains block 0 first
// and hands its accumulator back; the MMA thread then runs block 0 of the next tile over the first
// kDualStages K steps (whose stages the producer filled during the drain) before it needs block
// 1's accumulator, and only then issues block 1's MMAs for those K steps and releases the stages.
// The last kDualStages K steps mirror that: block 0 finishes them first and is handed to the
// epilogue (its own "accumulator full" barrier) while block 1 runs them.  What stays exposed per
// tile is about twice the drain time of one accumulator minus twice kDualStages K steps.
//
// Tile sequence.  An expert with an odd number of M blocks ends in a one-block tile.  Tiles are
// dealt round-robin to the CTAs; a last round that would keep fewer than half of the CTAs busy is
// dealt as one-block tiles instead, so that round costs half as much.
// ================================================================================================
#ifndef B200MOE_DUAL_STAGES
#define B200MOE_DUAL_STAGES 3
#endif
constexpr int kDualStages = B200MOE_DUAL_STAGES;
// K step of this kernel: 64 (three stages of 64 KiB, 128-byte swizzle) or, as a build option, 32
// (six stages of 32 KiB, rows of 64 bytes with the 64-byte swizzle of TMA and of the
// shared-memory descriptors).  Measured with the cycle counters of a measurement build at
// T = 8192: with 64-wide steps the MMA thread waits for operands 13-14 % of its time (40 % with
// two stages: a stage's loads take about 2400 SM cycles to land); the 32-wide variant, meant to
// reach further ahead (five K steps of lookahead instead of two), was slower (17-18 % waiting,
// 82 k instead of 73 k cycles per first-GEMM tile): boxes of 64-byte rows are delivered less
// efficiently than boxes of 128-byte rows.  Asking L2 for the weight boxes four or eight K steps
// ahead (cp.async.bulk.prefetch.tensor) did not help either: issued by every CTA the one-block
// kernel lost 15-20 %, issued only by the one CTA that leads a weight tile it lost 0-8 %.
#ifndef B200MOE_DUAL_BLOCK_K
#define B200MOE_DUAL_BLOCK_K 64
#endif
constexpr int kDualBlockK = B200MOE_DUAL_BLOCK_K;
static_assert(kDualBlockK == 32 || kDualBlockK == 64, "K step of the two-block kernel");
constexpr int kDualRowBytes = kDualBlockK * 2;
constexpr int kDualBlockABytes = kBlockM * kDualRowBytes;     // one M block's rows of one stage
constexpr int kDualABytes = 2 * kDualBlockABytes;
constexpr int kDualBBytes = kBlockN * kDualRowBytes;
constexpr int kDualStageBytes = kDualABytes + kDualBBytes;

// Shared-memory matrix descriptor of a K-major tile in this kernel's stage layout: 8-row groups
// are 8 * row bytes apart; layout type 2 is the 128-byte swizzle, 4 the 64-byte swizzle.
__device__ __forceinline__ uint64_t make_dual_desc(uint32_t smem_addr) {
  const uint32_t lo = (smem_addr & 0x3ffffu) >> 4;
  const uint32_t hi = ((8u * kDualRowBytes) >> 4) | (1u << 14) | ((kDualRowBytes == 128 ? 2u : 4u) << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
constexpr int kDualSmemBytes = kDualStages * kDualStageBytes + kOutStageBytes + kSmemAlignSlack;
// Cost constants of two_block_tiles_win by length of the K loop (in K steps of 64): the part of
// the drain that no longer overlaps the next tile's MMAs is paid once per tile, so short K loops
// (the second GEMM of a tensor-parallel shard of eight has 28 K steps) keep the one-block kernel.
constexpr int kDualLongK = 96, kDualShortK = 48;
struct DualCost {
  int pair, single;  // percent of a one-block tile's time; pair == 0: never two-block tiles
};
inline DualCost dual_cost_for(int k_blocks) {
  if (k_blocks >= kDualLongK) return DualCost{182, 116};
  if (k_blocks >= kDualShortK) return DualCost{184, 140};
  return DualCost{0, 0};
}
// Both kernels are launched (and decide on the device) from this many M blocks per expert in the
// upper bound the host knows; below it two-block tiles never win.
constexpr int kDualHostGateBlocks = 6;

// One piece of work of the two-block kernel: m_count = 2 is two M blocks (m_block, m_block + 1) of
// one expert against one N tile; m_count = 1 is a single block.
struct WorkItem {
  int expert;
  int m_block;
  int n_tile;
  int m_count;
};

// The tile sequence of one launch: tiles are dealt round-robin to the CTAs.  An expert with an odd
// number of blocks leaves one block over, and there are two ways to deal it:
//   * slots = false: the odd block is the expert's last unit, a one-block tile per N tile.  Such a
//     tile takes about 0.64 of a two-block tile's time, so CTAs that receive some run ahead of the
//     others; CTAs that drift apart stop sharing weight tiles through L2 (the first GEMM then
//     read 45 % more from HBM than its algorithmic bytes in an ncu capture at T = 4096).
//   * slots = true: the odd block against TWO consecutive N tiles is one tile (a slot), run one
//     after the other by the same CTA, so every tile is two units of work and the CTAs stay in
//     step.  Slots sit in the expert's last group of blocks, right behind the two-block tiles
//     of the same pair of N tiles, so the weight tiles they read are the ones in flight.
//     Measured: the extra HBM reads of the first GEMM drop from 45 % to 17 %; the second GEMM,
//     whose tiles are 3.5 times longer (K = 14336), gets slower (two one-block tiles in a row
//     are a lump of 1.27 two-block times on one CTA), so it keeps slots = false.
// Inside an expert the units are cut into groups of at most unit_group (sizes as even as
// possible); inside a group the order is N tile, then unit (see decode_tile).
struct DualSeq {
  const int* blk_off;          // [E + 1] M-block offsets per expert
  const long long* tile_off;   // [E + 1] tile offsets per expert
  int n_tiles, num_experts, unit_group;
  bool slots;
  long long total;             // tiles of the launch
  long long cut;               // tiles [cut, total) are dealt in halves (one unit each)
};

__host__ __device__ inline long long dual_tiles_of_expert(int blocks, int n_tiles, bool slots) {
  if (!slots) return static_cast<long long>((blocks + 1) >> 1) * n_tiles;
  return static_cast<long long>(blocks >> 1) * n_tiles + ((blocks & 1) ? (n_tiles + 1) / 2 : 0);
}

// Where the last round would keep at most half of the CTAs busy with whole tiles, its tiles are
// dealt in halves instead: that round then costs one unit instead of two.
__host__ __device__ inline long long dual_cut(long long total, int grid) {
  const long long cut = total - total % grid;
  return 2 * (total - cut) > grid ? total : cut;
}

// Tile number -> up to two halves (each a one-block item); `joint` says that the halves are the
// two M blocks of a two-block tile (run together), otherwise they are run one after the other.
__host__ __device__ inline int dual_decode(const DualSeq& q, long long tile, WorkItem (&half)[2],
                                           bool* joint) {
  int e = 0;
  while (e + 1 < q.num_experts && tile >= q.tile_off[e + 1]) ++e;
  long long local = tile - q.tile_off[e];
  const int cnt = q.blk_off[e + 1] - q.blk_off[e];
  const int odd = cnt & 1;
  const int full = q.slots ? cnt >> 1 : (cnt + 1) >> 1;  // units dealt per N tile
  const int groups = (q.unit_group > 0 && full > q.unit_group)
                         ? (full + q.unit_group - 1) / q.unit_group : 1;
  const int small = full / groups, big = full % groups;  // `big` groups of small + 1 come first
  const long long before_last = static_cast<long long>(full - small) * q.n_tiles;
  int unit = -1, n = 0;
  if (!odd || !q.slots || local < before_last) {
    int first, size;
    const long long big_tiles = static_cast<long long>(small + 1) * q.n_tiles;
    if (local < big * big_tiles) {
      const int gi = static_cast<int>(local / big_tiles);
      first = gi * (small + 1);
      size = small + 1;
      local -= gi * big_tiles;
    } else {
      local -= big * big_tiles;
      const int gi = static_cast<int>(local / (static_cast<long long>(small) * q.n_tiles));
      first = big * (small + 1) + gi * small;
      size = small;
      local -= static_cast<long long>(gi) * small * q.n_tiles;
    }
    n = static_cast<int>(local / size);
    unit = first + static_cast<int>(local % size);
  } else {
    // The expert's last group (`small` units) with the odd block's slots woven in: per pair of N
    // tiles, the units against the first, the units against the second, then the slot.
    local -= before_last;
    const int size = small, first = full - small;
    const int pair = static_cast<int>(local / (2 * size + 1));
    const int r = static_cast<int>(local % (2 * size + 1));
    const bool last_alone = 2 * pair + 1 >= q.n_tiles;  // odd number of N tiles: a final half pair
    if (r < size) {
      n = 2 * pair;
      unit = first + r;
    } else if (!last_alone && r < 2 * size) {
      n = 2 * pair + 1;
      unit = first + r - size;
    } else {
      half[0] = WorkItem{e, q.blk_off[e] + cnt - 1, 2 * pair, 1};
      half[1] = WorkItem{e, q.blk_off[e] + cnt - 1, 2 * pair + 1, 1};
      *joint = false;
      return last_alone ? 1 : 2;
    }
  }
  half[0] = WorkItem{e, q.blk_off[e] + 2 * unit, n, 1};
  half[1] = WorkItem{e, q.blk_off[e] + 2 * unit + 1, n, 1};
  *joint = 2 * unit + 1 < cnt;
  return *joint ? 2 : 1;  // without slots the odd block is the expert's last, one-block unit
}

// The work of CTA `cta` of `grid` in its i-th turn: 0, 1 or 2 items, or -1 when it has no more.
__host__ __device__ inline int dual_items_at(const DualSeq& q, long long i, int cta, int grid,
                                             WorkItem (&items)[2]) {
  // Whole tiles are dealt round by round, and every round starts one CTA further on: the sequence
  // is periodic (an expert with 37 blocks and slots repeats every 37 tiles: 2 x 18 two-block tiles
  // and one slot), and a period that divides the grid would hand the same CTAs the dearer tiles
  // of every round.  Measured at T = 6144 with 37 blocks in the largest expert and 148 CTAs: the
  // busiest CTA's loop took 21 % longer than the mean without the rotation.
  const long long rounds = q.cut / grid;
  const int rest = static_cast<int>(q.cut - rounds * grid);
  const int last_slot = static_cast<int>((cta + rounds) % grid);
  const long long mine = rounds + (last_slot < rest ? 1 : 0);
  WorkItem half[2];
  bool joint = false;
  if (i < mine) {
    const long long tile = i * grid + (i < rounds ? (cta + i) % grid : last_slot);
    const int halves = dual_decode(q, tile, half, &joint);
    if (joint) {
      items[0] = WorkItem{half[0].expert, half[0].m_block, half[0].n_tile, 2};
      return 1;
    }
    items[0] = half[0];
    items[1] = half[1];
    return halves;
  }
  const long long v = cta + (i - mine) * grid;
  if (v >= 2 * (q.total - q.cut)) return -1;
  const int halves = dual_decode(q, q.cut + (v >> 1), half, &joint);
  if (static_cast<int>(v & 1) >= halves) return 0;
  items[0] = half[v & 1];
  return 1;
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_dual_kernel(const __grid_constant__ CUtensorMap tmap_a,    // box of 128 rows
                         const __grid_constant__ CUtensorMap tmap_a2,   // box of 256 rows
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_out,  // kW13 with p.tma_store: act
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kDualStages], empty_bar[kDualStages], tmem_full_bar[2],
      tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_blk_cnt[kMaxExperts];
  __shared__ int s_blk_off[kMaxExperts + 1];
  __shared__ long long s_tile_off[kMaxExperts + 1];
  __shared__ int s_abort;

  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + kSmemAlignSlack - 1) &
      ~static_cast<uintptr_t>(kSmemAlignSlack - 1));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, grid = gridDim.x;

  // ------------------------------------------------------------------ prologue
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_a2);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kDualStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], kEpilogueWarps);
    }
    s_abort = 0;
    fence_barrier_init();
  }
  if (threadIdx.x < kMaxExperts) s_blk_cnt[threadIdx.x] = 0;
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  __syncthreads();
  pdl_wait();  // everything above touched only this CTA's shared and tensor memory
  pdl_launch_dependents();
  long long npp = *p.npp;
  if (npp > p.capacity) npp = p.capacity;
  const int num_blocks = static_cast<int>(npp / kBlockM);
  for (int b = threadIdx.x; b < num_blocks; b += kThreads) {
    const int e = p.expert_ids[b];
    if (e >= 0 && e < p.num_experts) atomicAdd(&s_blk_cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    long long tiles = 0;
    for (int e = 0; e < p.num_experts; ++e) {
      s_blk_off[e] = acc;
      s_tile_off[e] = tiles;
      acc += s_blk_cnt[e];
      tiles += dual_tiles_of_expert(s_blk_cnt[e], p.n_tiles, kMode != kW2);
    }
    s_blk_off[p.num_experts] = acc;
    s_tile_off[p.num_experts] = tiles;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_flag = &s_abort;

  DualSeq seq;
  seq.blk_off = s_blk_off;
  seq.tile_off = s_tile_off;
  seq.n_tiles = p.n_tiles;
  seq.num_experts = p.num_experts;
  seq.unit_group = p.m_group > 0 ? (p.m_group + 1) / 2 : 0;
  seq.slots = kMode != kW2;
  seq.total = s_tile_off[p.num_experts];
  if (p.dual_pair_cost > 0 &&
      !two_block_tiles_win(s_blk_off, p.num_experts, p.n_tiles, p.dual_ctas, p.dual_pair_cost,
                           p.dual_single_cost, p.dual_slots != 0))
    seq.total = 0;  // the one-block kernel launched beside this one does the work
  seq.cut = dual_cut(seq.total, grid);

  constexpr bool kIsW13 = (kMode != kW2);
  // The host sizes K steps and stage bytes for the 64-wide K step of the other kernels.
  const int k_blocks = p.k_blocks * (kBlockK / kDualBlockK);
  const int b_tx_bytes = (p.stage_tx_bytes - kABytes) / (kBlockK / kDualBlockK);  // weight bytes of one stage
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem items[2];
      for (long long i = 0; ok; ++i) {
        const int count = dual_items_at(seq, i, cta, grid, items);
        if (count < 0) break;
        for (int s = 0; ok && s < count; ++s) {
        const WorkItem t = items[s];
        const int a_row = t.m_block * kBlockM;
        const int b_row0 = t.expert * p.b_rows_per_expert +
                           t.n_tile * (kIsW13 ? p.half_n : kBlockN);
        const uint32_t tx = b_tx_bytes + t.m_count * kDualBlockABytes;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 0x121)) { ok = false; break; }
          uint8_t* sa = smem + stage * kDualStageBytes;
          uint8_t* sb = sa + kDualABytes;
          mbar_expect_tx(&full_bar[stage], tx);
          tma_load_2d(sa, t.m_count == 2 ? &tmap_a2 : &tmap_a, &full_bar[stage], kb * kDualBlockK, a_row);
          if (kIsW13) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kDualBlockK, b_row0);
            tma_load_2d(sb + p.half_n * kDualRowBytes, &tmap_b, &full_bar[stage], kb * kDualBlockK,
                        b_row0 + p.inter);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kDualBlockK, b_row0);
          }
          if (++stage == kDualStages) { stage = 0; phase ^= 1; }
        }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long it = 0;
      WorkItem items[2];
      const uint32_t acc0 = tmem_base, acc1 = tmem_base + kBlockN;
      long long cyc_full = 0, cyc_tmem = 0, cyc_head = 0, cyc_tail = 0;
      B200MOE_CYCLES_BEGIN(loop_begin);
      for (long long i = 0; ok; ++i) {
        const int count = dual_items_at(seq, i, cta, grid, items);
        if (count < 0) break;
        for (int s = 0; ok && s < count; ++s) {
        const WorkItem t = items[s];
        const uint32_t par = static_cast<uint32_t>(it & 1);
        ++it;
        {
          B200MOE_CYCLES_BEGIN(w0);
          if (!mbar_wait(&tmem_empty_bar[0], par ^ 1, abort_flag, 0x221)) { ok = false; break; }
          B200MOE_CYCLES_ADD(cyc_tmem, w0);
        }
        tc_fence_after();
        int kb = 0;
        if (t.m_count == 2) {
          // Block 0 runs ahead over the first K steps while block 1's accumulator is drained.
          const int head = k_blocks < kDualStages ? k_blocks : kDualStages;
          for (int h = 0; ok && h < head; ++h) {
            const int st = stage + h < kDualStages ? stage + h : stage + h - kDualStages;
            const uint32_t ph = stage + h < kDualStages ? phase : phase ^ 1;
            B200MOE_CYCLES_BEGIN(w1);
            if (!mbar_wait(&full_bar[st], ph, abort_flag, 0x222)) { ok = false; break; }
            B200MOE_CYCLES_ADD(cyc_full, w1);
            B200MOE_CYCLES_ADD(cyc_head, w1);
            const uint32_t sa = smem_u32(smem + st * kDualStageBytes);
            const uint32_t sb = sa + kDualABytes;
#pragma unroll
            for (int k = 0; k < kDualBlockK / kUmmaK; ++k)
              umma_bf16(acc0, make_dual_desc(sa + k * kUmmaK * 2), make_dual_desc(sb + k * kUmmaK * 2),
                        p.idesc, (h | k) != 0 ? 1u : 0u);
          }
          if (!ok) break;
          {
            B200MOE_CYCLES_BEGIN(w2);
            if (!mbar_wait(&tmem_empty_bar[1], par ^ 1, abort_flag, 0x223)) { ok = false; break; }
            B200MOE_CYCLES_ADD(cyc_tmem, w2);
          }
          tc_fence_after();
          for (int h = 0; h < head; ++h) {
            const uint32_t sa = smem_u32(smem + stage * kDualStageBytes);
            const uint32_t sb = sa + kDualABytes;
#pragma unroll
            for (int k = 0; k < kDualBlockK / kUmmaK; ++k)
              umma_bf16(acc1, make_dual_desc(sa + kDualBlockABytes + k * kUmmaK * 2),
                        make_dual_desc(sb + k * kUmmaK * 2), p.idesc, (h | k) != 0 ? 1u : 0u);
            umma_commit(&empty_bar[stage]);
            if (++stage == kDualStages) { stage = 0; phase ^= 1; }
          }
          // The last K steps mirror the first: block 0 finishes them first and is handed to the
          // epilogue while block 1 runs them.
          const int tail = k_blocks - head >= kDualStages ? kDualStages : 0;
          for (kb = head; kb < k_blocks - tail; ++kb) {
            B200MOE_CYCLES_BEGIN(w3);
            if (!mbar_wait(&full_bar[stage], phase, abort_flag, 0x224)) { ok = false; break; }
            B200MOE_CYCLES_ADD(cyc_full, w3);
            const uint32_t sa = smem_u32(smem + stage * kDualStageBytes);
            const uint32_t sb = sa + kDualABytes;
#pragma unroll
            for (int k = 0; k < kDualBlockK / kUmmaK; ++k) {
              const uint64_t bdesc = make_dual_desc(sb + k * kUmmaK * 2);
              umma_bf16(acc0, make_dual_desc(sa + k * kUmmaK * 2), bdesc, p.idesc, 1u);
              umma_bf16(acc1, make_dual_desc(sa + kDualBlockABytes + k * kUmmaK * 2), bdesc, p.idesc, 1u);
            }
            umma_commit(&empty_bar[stage]);
            if (++stage == kDualStages) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          for (int h = 0; ok && h < tail; ++h) {
            const int st = stage + h < kDualStages ? stage + h : stage + h - kDualStages;
            const uint32_t ph = stage + h < kDualStages ? phase : phase ^ 1;
            B200MOE_CYCLES_BEGIN(w4);
            if (!mbar_wait(&full_bar[st], ph, abort_flag, 0x227)) { ok = false; break; }
            B200MOE_CYCLES_ADD(cyc_full, w4);
            B200MOE_CYCLES_ADD(cyc_tail, w4);
            const uint32_t sa = smem_u32(smem + st * kDualStageBytes);
            const uint32_t sb = sa + kDualABytes;
#pragma unroll
            for (int k = 0; k < kDualBlockK / kUmmaK; ++k)
              umma_bf16(acc0, make_dual_desc(sa + k * kUmmaK * 2), make_dual_desc(sb + k * kUmmaK * 2),
                        p.idesc, 1u);
          }
          if (!ok) break;
          umma_commit(&tmem_full_bar[0]);  // block 0 complete
          for (int h = 0; h < tail; ++h) {
            const uint32_t sa = smem_u32(smem + stage * kDualStageBytes);
            const uint32_t sb = sa + kDualABytes;
#pragma unroll
            for (int k = 0; k < kDualBlockK / kUmmaK; ++k)
              umma_bf16(acc1, make_dual_desc(sa + kDualBlockABytes + k * kUmmaK * 2),
                        make_dual_desc(sb + k * kUmmaK * 2), p.idesc, 1u);
            umma_commit(&empty_bar[stage]);
            if (++stage == kDualStages) { stage = 0; phase ^= 1; }
          }
          umma_commit(&tmem_full_bar[1]);  // block 1 complete
        } else {
          if (!mbar_wait(&tmem_empty_bar[1], par ^ 1, abort_flag, 0x225)) { ok = false; break; }
          tc_fence_after();
          for (kb = 0; kb < k_blocks; ++kb) {
            B200MOE_CYCLES_BEGIN(w5);
            if (!mbar_wait(&full_bar[stage], phase, abort_flag, 0x226)) { ok = false; break; }
            B200MOE_CYCLES_ADD(cyc_full, w5);
            const uint32_t sa = smem_u32(smem + stage * kDualStageBytes);
            const uint32_t sb = sa + kDualABytes;
#pragma unroll
            for (int k = 0; k < kDualBlockK / kUmmaK; ++k)
              umma_bf16(acc0, make_dual_desc(sa + k * kUmmaK * 2), make_dual_desc(sb + k * kUmmaK * 2),
                        p.idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit(&empty_bar[stage]);
            if (++stage == kDualStages) { stage = 0; phase ^= 1; }
          }
          if (ok) {
            umma_commit(&tmem_full_bar[0]);
            umma_commit(&tmem_full_bar[1]);  // keeps the two barriers in step; nothing to drain
          }
        }
        }
      }
#ifdef B200MOE_MEASURE_CYCLES
      atomicAdd(&g_gemm_cycles[2], static_cast<unsigned long long>(cyc_full));
      atomicAdd(&g_gemm_cycles[3], static_cast<unsigned long long>(cyc_tmem));
      atomicAdd(&g_gemm_cycles[4], static_cast<unsigned long long>(clock64() - loop_begin));
      atomicAdd(&g_gemm_cycles[5], static_cast<unsigned long long>(it));
      atomicAdd(&g_gemm_cycles[6], static_cast<unsigned long long>(cyc_head));
      atomicAdd(&g_gemm_cycles[7], static_cast<unsigned long long>(cyc_tail));
#endif
      (void)cyc_full;
      (void)cyc_tmem;
      (void)cyc_head;
      (void)cyc_tail;
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;               // TMEM lanes this warp may read: 32*quarter ..
    uint8_t* stage_out = smem + kDualStages * kDualStageBytes +
                         (warp - 2) * ((kIsW13 && p.tma_store) ? 32 * 128 : 32 * kOutStageRowBytes);
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool ok = true;
    long long it = 0, cyc_drain = 0, drains = 0;
    WorkItem items[2];
    for (long long i = 0; ok; ++i) {
      const int count = dual_items_at(seq, i, cta, grid, items);
      if (count < 0) break;
      for (int s = 0; ok && s < count; ++s) {
      const WorkItem t = items[s];
      const uint32_t par = static_cast<uint32_t>(it & 1);
      ++it;
      for (int b = 0; b < 2; ++b) {
        // All lanes of the warp must leave together: the wait result is made warp-uniform.
        int good = mbar_wait(&tmem_full_bar[b], par, abort_flag, 0x321 + b) ? 1 : 0;
        good = __all_sync(0xffffffffu, good);
        if (!good) { ok = false; break; }
        tc_fence_after();
        if (b < t.m_count) {
          B200MOE_CYCLES_BEGIN(d0);
          if (kIsW13) {
            drain_w13(p, &tmap_out, taddr + b * kBlockN, stage_out, t.m_block + b, t.n_tile, quarter, lane);
          } else {
            drain_w2(p, taddr + b * kBlockN, stage_out, t.m_block + b, t.n_tile, quarter, lane);
          }
          B200MOE_CYCLES_ADD(cyc_drain, d0);
          ++drains;
        }
        // Hand this accumulator back to the MMA warp.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[b]);
      }
      }
    }
#ifdef B200MOE_MEASURE_CYCLES
    if (warp == 2 && lane == 0) {
      atomicAdd(&g_gemm_cycles[0], static_cast<unsigned long long>(cyc_drain));
      atomicAdd(&g_gemm_cycles[1], static_cast<unsigned long long>(drains));
    }
#endif
    (void)cyc_drain;
    (void)drains;
    if (kIsW13 && p.tma_store && lane == 0) tma_store_wait_all();  // before shared memory goes away
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // Give bulk copies that may still be in flight time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < (1ll << 22)) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ================================================================================================
// Two-CTA variant (tcgen05 cta_group::2): a cluster of two CTAs on neighbouring SMs computes one
// 256 x 256 tile.  Each CTA stages its own 128 A rows and one half of the B tile (128 of the 256
// accumulator columns' weight rows), the leader CTA issues M = 256 MMAs that read both CTAs'
// shared memory, and each CTA's TMEM receives the 256 accumulator columns of its own 128 rows.
// Per SM and K step this moves 32 KiB through L2 and shared memory instead of 48 KiB.
//
// Barriers: full[s] lives in the leader only (armed by the leader's producer with the bytes of
// both CTAs; both producers' TMA loads complete on it).  empty[s] and tmem_full[a] exist in both
// CTAs and are released by the leader's tcgen05.commit, issued once per CTA.  tmem_empty[a] lives
// in the leader and collects the epilogue warps of both CTAs.  No load uses cluster multicast.
// ================================================================================================
#ifndef B200MOE_PAIR_STAGES
#define B200MOE_PAIR_STAGES 6
#endif
constexpr int kPairStages = B200MOE_PAIR_STAGES;
constexpr int kPairABytes = kBlockM * kBlockK * 2;          // 16384: this CTA's 128 A rows
constexpr int kPairBBytes = (kBlockN / 2) * kBlockK * 2;    // 16384: this CTA's half of B
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;  // 32768
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + kSmemAlignSlack;
constexpr int kPairBlockM = 2 * kBlockM;                    // rows per tile of the pair
// Instruction descriptor of the pair: M = 256 (128 rows in each CTA), N = 256.
constexpr uint32_t kPairInstrDesc = make_instr_desc(kBlockN, kPairBlockM);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
               ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0),
      "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at shared::cluster address `bar` once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_cluster_addr)
               : "memory");
}

template <int kMode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kPairStages], empty_bar[kPairStages], tmem_full_bar[2],
      tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_blk_cnt[kMaxExperts];
  __shared__ int s_blk_off[kMaxExperts + 1];
  __shared__ int s_abort;

  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + kSmemAlignSlack - 1) &
      ~static_cast<uintptr_t>(kSmemAlignSlack - 1));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();   // 0 = leader
  const uint32_t peer_rank = cta_rank ^ 1u;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs_grid = gridDim.x >> 1;

  // ------------------------------------------------------------------ prologue
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 2 * kEpilogueWarps);
    }
    s_abort = 0;
    fence_barrier_init();
  }
  if (threadIdx.x < kMaxExperts) s_blk_cnt[threadIdx.x] = 0;
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(&tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  pdl_wait();  // everything above touched only this CTA's shared and tensor memory
  pdl_launch_dependents();
  long long npp = *p.npp;
  if (npp > p.capacity) npp = p.capacity;
  const int num_blocks = static_cast<int>(npp / kPairBlockM);
  for (int b = threadIdx.x; b < num_blocks; b += kThreads) {
    const int e = p.expert_ids[b];
    if (e >= 0 && e < p.num_experts) atomicAdd(&s_blk_cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.num_experts; ++e) {
      s_blk_off[e] = acc;
      acc += s_blk_cnt[e];
    }
    s_blk_off[p.num_experts] = acc;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const long long total_tiles = static_cast<long long>(s_blk_off[p.num_experts]) * p.n_tiles;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = pair_id; ok && tile < total_tiles; tile += num_pairs_grid) {
        const TileCoord c = decode_tile(tile, p.n_tiles, p.num_experts, s_blk_off, 0);
        const int a_row = c.m_block * kPairBlockM + static_cast<int>(cta_rank) * kBlockM;
        // This CTA's half of the B tile: for w13 the leader holds the gate rows and the peer the
        // matching up rows; for w2 consecutive halves of 128 output columns.
        const int b_row = c.expert * p.b_rows_per_expert +
                          (kMode == kW13 ? c.n_tile * (kBlockN / 2) + static_cast<int>(cta_rank) * p.inter
                                         : c.n_tile * kBlockN + static_cast<int>(cta_rank) * (kBlockN / 2));
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 0x111)) { ok = false; break; }
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb = sa + kPairABytes;
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (cta_rank == 0) mbar_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          tma_load_2d_pair(sa, &tmap_a, full_leader, kb * kBlockK, a_row);
          tma_load_2d_pair(sb, &tmap_b, full_leader, kb * kBlockK, b_row);
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long it = 0;
      for (long long tile = pair_id; ok && tile < total_tiles; tile += num_pairs_grid, ++it) {
        const int acc = static_cast<int>(it & 1);
        const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, 0x211)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, 0x212)) { ok = false; break; }
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint32_t sb = sa + kPairABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t adesc = make_smem_desc(sa + k * kUmmaK * 2);
            const uint64_t bdesc = make_smem_desc(sb + k * kUmmaK * 2);
            umma_bf16_pair(tmem_d, adesc, bdesc, kPairInstrDesc, (kb | k) != 0 ? 1u : 0u);
          }
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_pair(map_to_cta(eb, 0));
          umma_commit_pair(map_to_cta(eb, 1));
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          const uint32_t fb = smem_u32(&tmem_full_bar[acc]);
          umma_commit_pair(map_to_cta(fb, 0));
          umma_commit_pair(map_to_cta(fb, 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const int row_in_cta = quarter * 32 + lane;
    bool ok = true;
    long long it = 0;
    for (long long tile = pair_id; ok && tile < total_tiles; tile += num_pairs_grid, ++it) {
      const TileCoord c = decode_tile(tile, p.n_tiles, p.num_experts, s_blk_off, 0);
      const int acc = static_cast<int>(it & 1);
      const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
      const long long slot = static_cast<long long>(c.m_block) * kPairBlockM +
                             static_cast<long long>(cta_rank) * kBlockM + row_in_cta;
      int good = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, 0x311) ? 1 : 0;
      good = __all_sync(0xffffffffu, good);
      if (!good) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * kBlockN);
      if (kMode == kW13) {
        __nv_bfloat16* dst = p.out + slot * p.out_ld + static_cast<long long>(c.n_tile) * (kBlockN / 2);
#pragma unroll 1
        for (int ch = 0; ch < (kBlockN / 2) / 32; ++ch) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + ch * 32, g);
          tmem_ld_32x32(taddr + kBlockN / 2 + ch * 32, u);
          tmem_ld_wait();
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
            const float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
            o[j] = pack_bf16(silu_mul(g0, u0), silu_mul(g1, u1));
          }
          uint4* d4 = reinterpret_cast<uint4*>(dst + ch * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            d4[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
        }
      } else {
        const int pair = p.sorted[slot];
        const bool live = pair >= 0 && pair < p.num_pairs;
        const float w = live ? p.topk_weights[pair] : 0.f;
        // With an output table the row goes straight to the GPU that owns the token (a plain
        // store through a peer mapping): the return all-to-all is this epilogue.
        __nv_bfloat16* base = p.out;
        long long out_row = live ? pair : 0;
        if (p.out_table != nullptr && live) {
          const long long owner = out_row / p.pairs_per_rank;
          base = p.out_table[owner];
          out_row -= owner * p.pairs_per_rank;
        }
        __nv_bfloat16* dst = base + out_row * p.out_ld + static_cast<long long>(c.n_tile) * kBlockN;
#pragma unroll 1
        for (int ch = 0; ch < kBlockN / 32; ++ch) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + ch * 32, v);
          tmem_ld_wait();
          if (live) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + ch * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(v[8 * q + 0]) * w, __uint_as_float(v[8 * q + 1]) * w);
              o.y = pack_bf16(__uint_as_float(v[8 * q + 2]) * w, __uint_as_float(v[8 * q + 3]) * w);
              o.z = pack_bf16(__uint_as_float(v[8 * q + 4]) * w, __uint_as_float(v[8 * q + 5]) * w);
              o.w = pack_bf16(__uint_as_float(v[8 * q + 6]) * w, __uint_as_float(v[8 * q + 7]) * w);
              d4[q] = o;
            }
          }
        }
      }
      // Hand the accumulator back: every epilogue warp of both CTAs arrives at the leader.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < (1ll << 22)) {}
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still be signalling this CTA's barriers until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  (void)peer_rank;
}

// ------------------------------------------------------------------------------------ host side
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault,
                                         &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  });
  return fn;
}

// 2-D bf16 tensor [rows, cols] (cols contiguous), box = box_rows x box_cols columns; rows of 64
// columns take the 128-byte swizzle, rows of 32 the 64-byte swizzle.
int make_tmap(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows,
              const char* what, int box_cols = kBlockK) {
  auto encode = get_encode_fn();
  if (!encode) return fail(B200MOE_ERR_CUDA, "%s: cuTensorMapEncodeTiled is unavailable", what);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            box_cols == kBlockK ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200MOE_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return B200MOE_OK;
}

template <int kMode>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout, const GemmParams& p,
           cudaStream_t st) {
  // The attribute belongs to the function in the current context; setting it on every launch is
  // cheap and keeps processes that drive several devices correct.
  const cudaError_t attr_err = cudaFuncSetAttribute(
      grouped_gemm_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (attr_err != cudaSuccess)
    return fail(B200MOE_ERR_CUDA, "grouped_gemm: cannot reserve %d bytes of shared memory: %s",
                kSmemBytes, cudaGetErrorString(attr_err));
  launch_pdl(grouped_gemm_kernel<kMode>, dim3(sm_count()), dim3(kThreads), kSmemBytes, st, ta, tb, tout,
             p);
  return check_launch("grouped_gemm");
}

template <int kMode>
int launch_dual(const CUtensorMap& ta, const CUtensorMap& ta2, const CUtensorMap& tb,
                const CUtensorMap& tout, const GemmParams& p, cudaStream_t st) {
  const cudaError_t attr_err = cudaFuncSetAttribute(
      grouped_gemm_dual_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDualSmemBytes);
  if (attr_err != cudaSuccess)
    return fail(B200MOE_ERR_CUDA, "grouped_gemm: cannot reserve %d bytes of shared memory: %s",
                kDualSmemBytes, cudaGetErrorString(attr_err));
  launch_pdl(grouped_gemm_dual_kernel<kMode>, dim3(sm_count()), dim3(kThreads), kDualSmemBytes, st,
             ta, ta2, tb, tout, p);
  return check_launch("grouped_gemm (two-block tiles)");
}

// Tiling of the one-CTA kernels: 0 = chosen by batch size, 1 = one M block per tile, 2 = two.
std::atomic<int> g_tiling{0};
// Whether the first GEMM's epilogue uses bulk tensor stores (b200moe_gemm_set_act_stores).
std::atomic<int> g_tma_act_stores{1};

// Two-block tiles pay off once most experts hold several M blocks: the weight stage is then
// shared by two blocks almost everywhere.  With one block per expert (decode-sized batches) every
// tile would be a one-block tile without the double-buffered accumulator, so the one-block kernel
// is kept there.  `capacity` = pairs + num_experts * 127 bounds the padded row count.
enum TileChoice { kOneBlock, kTwoBlock, kDecideOnDevice };

// kOneBlock when even the upper bound of the rows is too small for two-block tiles to pay (only
// the one-block kernel is launched); kDecideOnDevice otherwise: both kernels are launched and the
// real block counts decide (two_block_tiles_win).
TileChoice choose_tiles(int64_t capacity, int num_experts, const DualCost& cost) {
  const int mode = g_tiling.load(std::memory_order_relaxed);
  if (capacity < 2 * kBlockM || mode == 1) return kOneBlock;
  if (mode == 2) return kTwoBlock;
  if (cost.pair <= 0) return kOneBlock;
  const int64_t pairs = capacity - static_cast<int64_t>(num_experts) * (kBlockM - 1);
  return pairs >= static_cast<int64_t>(kBlockM) * kDualHostGateBlocks * num_experts ? kDecideOnDevice
                                                                                    : kOneBlock;
}

// Tensor maps of the two-block kernel (its own K step and swizzle): A rows in boxes of one and of
// two M blocks, and the weight rows.
struct DualMaps {
  CUtensorMap a, a2, b;
};

int make_dual_maps(DualMaps* m, const void* a, long long a_rows, long long k, const void* b,
                   long long b_rows, int b_box_rows, const char* what) {
  if (int rc = make_tmap(&m->a, a, a_rows, k, kBlockM, what, kDualBlockK)) return rc;
  if (int rc = make_tmap(&m->a2, a, a_rows, k, 2 * kBlockM, what, kDualBlockK)) return rc;
  return make_tmap(&m->b, b, b_rows, k, b_box_rows, what, kDualBlockK);
}

template <int kMode>
int launch_chosen(TileChoice choice, const DualCost& cost, const CUtensorMap& ta, const CUtensorMap& tb,
                  const CUtensorMap& tout, const DualMaps& dm, GemmParams p, cudaStream_t st) {
  if (choice == kOneBlock) return launch<kMode>(ta, tb, tout, p, st);
  if (choice == kTwoBlock) return launch_dual<kMode>(dm.a, dm.a2, dm.b, tout, p, st);
  p.dual_pair_cost = cost.pair;
  p.dual_single_cost = cost.single;
  p.dual_ctas = sm_count();
  p.dual_slots = kMode != kW2 ? 1 : 0;
  if (int rc = launch<kMode>(ta, tb, tout, p, st)) return rc;
  return launch_dual<kMode>(dm.a, dm.a2, dm.b, tout, p, st);
}

template <int kMode>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  const cudaError_t attr_err = cudaFuncSetAttribute(
      grouped_gemm_pair_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
  if (attr_err != cudaSuccess)
    return fail(B200MOE_ERR_CUDA, "grouped_gemm: cannot reserve %d bytes of shared memory: %s",
                kPairSmemBytes, cudaGetErrorString(attr_err));
  const int grid = sm_count() & ~1;  // whole clusters of two CTAs
  launch_pdl(grouped_gemm_pair_kernel<kMode>, dim3(grid), dim3(kThreads), kPairSmemBytes, st, ta,
             tb, p);
  return check_launch("grouped_gemm (2-CTA)");
}

// Gate columns per tile for the one-CTA w13 kernel.  With many tiles per SM the full 128 is best
// (the MMA is most efficient at N = 256).  With few M blocks (decode-sized batches, where the
// kernel streams weights and is HBM-bound) the tile count rarely divides by the SM count, so a
// narrower tile that fills the last wave better wins: e.g. 8 M blocks x 14336 / 128 = 896 tiles is
// 6.05 waves of 148 SMs, while 14336 / 112 gives 1024 tiles = 6.92 waves of smaller tiles.
int choose_half_n(int64_t capacity, int num_experts, int64_t inter) {
  const int64_t pairs = capacity - static_cast<int64_t>(num_experts) * (kBlockM - 1);
  const int64_t per_expert = pairs > 0 ? ceil_div64(pairs, num_experts) : 1;
  const int64_t blocks = per_expert <= 2 * kBlockM
                             ? num_experts * ceil_div64(per_expert, kBlockM)
                             : ceil_div64(pairs, kBlockM) + num_experts / 2;
  const int sms = sm_count();
  if (blocks * (inter / (kBlockN / 2)) >= 16ll * sms) return kBlockN / 2;
  int best = kBlockN / 2;
  int64_t best_cost = -1;
  for (int h = kBlockN / 2; h >= 64; h -= 16) {
    if (inter % h != 0) continue;
    const int64_t waves = ceil_div64(blocks * (inter / h), sms);
    const int64_t cost = waves * (2 * h + 16);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = h; }
  }
  return best;
}

// M blocks per group of the tile order (see decode_tile): as many 128-row blocks of the A operand
// as fit a 40 MB share of L2.  Measured on B200 (126 MB L2): with one group per expert the w13
// GEMM slows down by 12 % once an expert's A rows reach 67 MB (T = 32768), and the w2 GEMM, whose
// A rows are 3.5 times longer, re-reads them from HBM for every N tile from T = 8192 on.
int m_group_for(int64_t a_row_bytes) {
  // Budgets of 24, 64 and 96 MB measured the same within noise at T = 8192 and T = 16384.
  const int64_t budget = 40ll << 20;
  const int64_t g = budget / (static_cast<int64_t>(kBlockM) * a_row_bytes);
  return static_cast<int>(g < 4 ? 4 : (g > 4096 ? 4096 : g));
}

// Fills the fields of the one-CTA kernel that depend on the accumulator width.
void set_width(GemmParams* p, int mma_n) {
  p->idesc = make_instr_desc(mma_n, kBlockM);
  p->stage_tx_bytes = kABytes + mma_n * kBlockK * 2;
}

int check_common(const char* name, int num_experts, int64_t hidden, int64_t inter, int block_m,
                 int64_t capacity) {
  if (block_m != kBlockM && block_m != kPairBlockM)
    return fail(B200MOE_ERR_SHAPE, "%s: block_m must be %d or %d, got %d", name, kBlockM,
                kPairBlockM, block_m);
  if (num_experts < 1 || num_experts > kMaxExperts)
    return fail(B200MOE_ERR_SHAPE, "%s: num_experts=%d, supported 1..%d", name, num_experts, kMaxExperts);
  if (hidden <= 0 || inter <= 0 || capacity < 0)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld inter=%lld capacity=%lld", name, (long long)hidden,
                (long long)inter, (long long)capacity);
  if (capacity > 0x7fffffffLL - kPairBlockM) return fail(B200MOE_ERR_SHAPE, "%s: capacity too large", name);
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_grouped_gemm_w13_swiglu(const void* a_sorted, const void* w13, void* act,
                                               const int32_t* expert_ids,
                                               const int32_t* num_tokens_post_pad,
                                               int64_t sorted_capacity, int num_experts,
                                               int64_t hidden, int64_t inter, int block_m,
                                               b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "grouped_gemm_w13_swiglu";
  if (int rc = check_common(name, num_experts, hidden, inter, block_m, sorted_capacity)) return rc;
  if (hidden % kBlockK != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld must be a multiple of %d", name, (long long)hidden, kBlockK);
  if (inter % (kBlockN / 2) != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: intermediate size %lld must be a multiple of %d", name,
                (long long)inter, kBlockN / 2);
  if (sorted_capacity < block_m) return B200MOE_OK;  // no complete block can exist
  if (!a_sorted || !w13 || !act || !expert_ids || !num_tokens_post_pad)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(a_sorted, 16) || !aligned_to(w13, 16) || !aligned_to(act, 16))
    return fail(B200MOE_ERR_ALIGN, "%s: operands must be 16-byte aligned", name);
  // The two-CTA kernel has a fixed 128 + 128 column tile; the one-CTA kernels pick their width.
  const DualCost dual_cost = dual_cost_for(static_cast<int>(hidden / kBlockK));
  const TileChoice tiles = block_m == kBlockM ? choose_tiles(sorted_capacity, num_experts, dual_cost)
                                              : kOneBlock;
  const bool two_block = tiles != kOneBlock;
  const int half_n = block_m == kPairBlockM ? kBlockN / 2
                                            : choose_half_n(sorted_capacity, num_experts, inter);
  CUtensorMap ta, tb;
  DualMaps dm;
  if (int rc = make_tmap(&ta, a_sorted, sorted_capacity, hidden, kBlockM, name)) return rc;
  if (int rc = make_tmap(&tb, w13, static_cast<long long>(num_experts) * 2 * inter, hidden, half_n,
                         name))
    return rc;
  if (two_block)
    if (int rc = make_dual_maps(&dm, a_sorted, sorted_capacity, hidden, w13,
                                static_cast<long long>(num_experts) * 2 * inter, half_n, name))
      return rc;
  GemmParams p{};
  p.expert_ids = expert_ids;
  p.npp = num_tokens_post_pad;
  p.out = static_cast<__nv_bfloat16*>(act);
  p.capacity = sorted_capacity;
  p.num_experts = num_experts;
  p.k_blocks = static_cast<int>(hidden / kBlockK);
  p.n_tiles = static_cast<int>(inter / half_n);
  p.b_rows_per_expert = static_cast<int>(2 * inter);
  p.inter = static_cast<int>(inter);
  p.out_ld = inter;
  p.half_n = half_n;
  set_width(&p, 2 * half_n);
  p.m_group = m_group_for(hidden * 2);
  if (block_m == kPairBlockM) return launch_pair<kW13>(ta, tb, p, static_cast<cudaStream_t>(stream));
  // Output rows leave as bulk tensor stores of 32 rows x 64 columns where the tile width allows.
  CUtensorMap tout = ta;
  p.tma_store = (half_n % 64 == 0 && g_tma_act_stores.load(std::memory_order_relaxed)) ? 1 : 0;
  if (p.tma_store)
    if (int rc = make_tmap(&tout, act, sorted_capacity, inter, 32, name)) return rc;
  return launch_chosen<kW13>(tiles, dual_cost, ta, tb, tout, dm, p,
                             static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_grouped_gemm_w13_swiglu_gather(
    const void* tokens, int64_t num_tokens, int top_k, const int32_t* sorted_token_ids,
    const void* w13, void* act, const int32_t* expert_ids, const int32_t* num_tokens_post_pad,
    int64_t sorted_capacity, int num_experts, int64_t hidden, int64_t inter, int block_m,
    b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "grouped_gemm_w13_swiglu_gather";
  if (int rc = check_common(name, num_experts, hidden, inter, block_m, sorted_capacity)) return rc;
  if (block_m != kBlockM)
    return fail(B200MOE_ERR_SHAPE, "%s: block_m must be %d (the gathering kernel is one-CTA)", name, kBlockM);
  if (hidden % kBlockK != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld must be a multiple of %d", name, (long long)hidden, kBlockK);
  if (inter % (kBlockN / 2) != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: intermediate size %lld must be a multiple of %d", name,
                (long long)inter, kBlockN / 2);
  if (top_k < 1 || num_tokens < 0 || num_tokens > 0x7fffffffLL)
    return fail(B200MOE_ERR_SHAPE, "%s: top_k=%d num_tokens=%lld", name, top_k, (long long)num_tokens);
  if (sorted_capacity < block_m || num_tokens == 0) return B200MOE_OK;
  if (!tokens || !sorted_token_ids || !w13 || !act || !expert_ids || !num_tokens_post_pad)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(tokens, 16) || !aligned_to(w13, 16) || !aligned_to(act, 16) ||
      !aligned_to(sorted_token_ids, 16))
    return fail(B200MOE_ERR_ALIGN, "%s: operands must be 16-byte aligned", name);
  CUtensorMap ta, tb;
  const int half_n = choose_half_n(sorted_capacity, num_experts, inter);
  if (int rc = make_tmap(&ta, tokens, num_tokens, hidden, 1, name)) return rc;  // one row per box
  if (int rc = make_tmap(&tb, w13, static_cast<long long>(num_experts) * 2 * inter, hidden, half_n,
                         name))
    return rc;
  GemmParams p{};
  p.expert_ids = expert_ids;
  p.npp = num_tokens_post_pad;
  p.sorted = sorted_token_ids;
  p.out = static_cast<__nv_bfloat16*>(act);
  p.capacity = sorted_capacity;
  p.num_experts = num_experts;
  p.k_blocks = static_cast<int>(hidden / kBlockK);
  p.n_tiles = static_cast<int>(inter / half_n);
  p.b_rows_per_expert = static_cast<int>(2 * inter);
  p.inter = static_cast<int>(inter);
  p.out_ld = inter;
  p.half_n = half_n;
  set_width(&p, 2 * half_n);
  p.m_group = m_group_for(hidden * 2);
  p.top_k = top_k;
  p.num_src_rows = static_cast<int>(num_tokens);
  return launch<kW13Gather>(ta, tb, ta, p, static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_grouped_gemm_w2_scale(const void* act, const void* w2, void* out,
                                             const float* topk_weights,
                                             const int32_t* sorted_token_ids,
                                             const int32_t* expert_ids,
                                             const int32_t* num_tokens_post_pad,
                                             int64_t sorted_capacity, int64_t num_pairs,
                                             int num_experts, int64_t hidden, int64_t inter,
                                             int block_m, b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "grouped_gemm_w2_scale";
  if (int rc = check_common(name, num_experts, hidden, inter, block_m, sorted_capacity)) return rc;
  if (inter % kBlockK != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: intermediate size %lld must be a multiple of %d", name,
                (long long)inter, kBlockK);
  if (hidden % kBlockN != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld must be a multiple of %d", name, (long long)hidden, kBlockN);
  if (num_pairs < 0) return fail(B200MOE_ERR_SHAPE, "%s: num_pairs=%lld", name, (long long)num_pairs);
  if (sorted_capacity < block_m || num_pairs == 0) return B200MOE_OK;
  if (!act || !w2 || !out || !topk_weights || !sorted_token_ids || !expert_ids || !num_tokens_post_pad)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(act, 16) || !aligned_to(w2, 16) || !aligned_to(out, 16))
    return fail(B200MOE_ERR_ALIGN, "%s: operands must be 16-byte aligned", name);
  const DualCost dual_cost = dual_cost_for(static_cast<int>(inter / kBlockK));
  const TileChoice tiles = block_m == kBlockM ? choose_tiles(sorted_capacity, num_experts, dual_cost)
                                              : kOneBlock;
  const bool two_block = tiles != kOneBlock;
  CUtensorMap ta, tb;
  DualMaps dm;
  if (int rc = make_tmap(&ta, act, sorted_capacity, inter, kBlockM, name)) return rc;
  if (two_block)
    if (int rc = make_dual_maps(&dm, act, sorted_capacity, inter, w2,
                                static_cast<long long>(num_experts) * hidden, kBlockN, name))
      return rc;
  // The two-CTA kernel fetches the B tile as two boxes of 128 rows, one per CTA.
  if (int rc = make_tmap(&tb, w2, static_cast<long long>(num_experts) * hidden, inter,
                         block_m == kPairBlockM ? kBlockN / 2 : kBlockN, name))
    return rc;
  GemmParams p{};
  p.expert_ids = expert_ids;
  p.npp = num_tokens_post_pad;
  p.sorted = sorted_token_ids;
  p.topk_weights = topk_weights;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.capacity = sorted_capacity;
  p.num_pairs = num_pairs;
  p.num_experts = num_experts;
  p.k_blocks = static_cast<int>(inter / kBlockK);
  p.n_tiles = static_cast<int>(hidden / kBlockN);
  p.b_rows_per_expert = static_cast<int>(hidden);
  p.inter = 0;
  p.out_ld = hidden;
  set_width(&p, kBlockN);
  p.m_group = m_group_for(inter * 2);
  if (block_m == kPairBlockM) return launch_pair<kW2>(ta, tb, p, static_cast<cudaStream_t>(stream));
  return launch_chosen<kW2>(tiles, dual_cost, ta, tb, ta, dm, p, static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_grouped_gemm_w2_scale_peer(
    const void* act, const void* w2, void* const* out_table, int num_ranks, int64_t pairs_per_rank,
    const float* topk_weights, const int32_t* sorted_token_ids, const int32_t* expert_ids,
    const int32_t* num_tokens_post_pad, int64_t sorted_capacity, int num_experts, int64_t hidden,
    int64_t inter, int block_m, b200moe_stream_t stream) {
  using namespace b200moe;
  const char* name = "grouped_gemm_w2_scale_peer";
  if (int rc = check_common(name, num_experts, hidden, inter, block_m, sorted_capacity)) return rc;
  if (inter % kBlockK != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: intermediate size %lld must be a multiple of %d", name,
                (long long)inter, kBlockK);
  if (hidden % kBlockN != 0)
    return fail(B200MOE_ERR_SHAPE, "%s: hidden=%lld must be a multiple of %d", name, (long long)hidden, kBlockN);
  if (num_ranks < 1 || pairs_per_rank < 1 || num_ranks * pairs_per_rank > 0x7fffffffLL)
    return fail(B200MOE_ERR_SHAPE, "%s: num_ranks=%d pairs_per_rank=%lld", name, num_ranks,
                (long long)pairs_per_rank);
  if (sorted_capacity < block_m) return B200MOE_OK;
  if (!act || !w2 || !out_table || !topk_weights || !sorted_token_ids || !expert_ids ||
      !num_tokens_post_pad)
    return fail(B200MOE_ERR_NULL, "%s: null pointer", name);
  if (!aligned_to(act, 16) || !aligned_to(w2, 16))
    return fail(B200MOE_ERR_ALIGN, "%s: operands must be 16-byte aligned", name);
  const DualCost dual_cost = dual_cost_for(static_cast<int>(inter / kBlockK));
  const TileChoice tiles = block_m == kBlockM ? choose_tiles(sorted_capacity, num_experts, dual_cost)
                                              : kOneBlock;
  const bool two_block = tiles != kOneBlock;
  CUtensorMap ta, tb;
  DualMaps dm;
  if (int rc = make_tmap(&ta, act, sorted_capacity, inter, kBlockM, name)) return rc;
  if (two_block)
    if (int rc = make_dual_maps(&dm, act, sorted_capacity, inter, w2,
                                static_cast<long long>(num_experts) * hidden, kBlockN, name))
      return rc;
  if (int rc = make_tmap(&tb, w2, static_cast<long long>(num_experts) * hidden, inter,
                         block_m == kPairBlockM ? kBlockN / 2 : kBlockN, name))
    return rc;
  GemmParams p{};
  p.expert_ids = expert_ids;
  p.npp = num_tokens_post_pad;
  p.sorted = sorted_token_ids;
  p.topk_weights = topk_weights;
  p.out = nullptr;
  p.out_table = reinterpret_cast<__nv_bfloat16* const*>(out_table);
  p.pairs_per_rank = pairs_per_rank;
  p.capacity = sorted_capacity;
  p.num_pairs = static_cast<long long>(num_ranks) * pairs_per_rank;
  p.num_experts = num_experts;
  p.k_blocks = static_cast<int>(inter / kBlockK);
  p.n_tiles = static_cast<int>(hidden / kBlockN);
  p.b_rows_per_expert = static_cast<int>(hidden);
  p.inter = 0;
  p.out_ld = hidden;
  set_width(&p, kBlockN);
  p.m_group = m_group_for(inter * 2);
  if (block_m == kPairBlockM) return launch_pair<kW2>(ta, tb, p, static_cast<cudaStream_t>(stream));
  return launch_chosen<kW2>(tiles, dual_cost, ta, tb, ta, dm, p, static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_gemm_two_block_choice(const int32_t* blocks_per_expert, int num_experts,
                                             int n_tiles, int64_t k, int slots, int ctas) {
  using namespace b200moe;
  if (!blocks_per_expert || num_experts < 1 || num_experts > kMaxExperts || n_tiles < 1 || k < 1 ||
      ctas < 1)
    return fail(B200MOE_ERR_SHAPE, "gemm_two_block_choice: bad arguments");
  int blk_off[kMaxExperts + 1];
  blk_off[0] = 0;
  for (int e = 0; e < num_experts; ++e) {
    if (blocks_per_expert[e] < 0)
      return fail(B200MOE_ERR_SHAPE, "gemm_two_block_choice: negative block count");
    blk_off[e + 1] = blk_off[e] + blocks_per_expert[e];
  }
  const DualCost cost = dual_cost_for(static_cast<int>(k / kBlockK));
  if (cost.pair <= 0) return 0;
  return two_block_tiles_win(blk_off, num_experts, n_tiles, ctas, cost.pair, cost.single, slots != 0)
             ? 1 : 0;
}

extern "C" int64_t b200moe_gemm_two_block_schedule(const int32_t* blocks_per_expert, int num_experts,
                                                   int n_tiles, int m_group, int slots, int grid,
                                                   int cta, int32_t* items, int64_t max_items) {
  using namespace b200moe;
  if (!blocks_per_expert || num_experts < 1 || num_experts > kMaxExperts || n_tiles < 1 ||
      grid < 1 || cta < 0 || cta >= grid || max_items < 0 || (max_items > 0 && !items))
    return fail(B200MOE_ERR_SHAPE, "gemm_two_block_schedule: bad arguments");
  int blk_off[kMaxExperts + 1];
  long long tile_off[kMaxExperts + 1];
  blk_off[0] = 0;
  tile_off[0] = 0;
  for (int e = 0; e < num_experts; ++e) {
    if (blocks_per_expert[e] < 0)
      return fail(B200MOE_ERR_SHAPE, "gemm_two_block_schedule: negative block count");
    blk_off[e + 1] = blk_off[e] + blocks_per_expert[e];
    tile_off[e + 1] = tile_off[e] + dual_tiles_of_expert(blocks_per_expert[e], n_tiles, slots != 0);
  }
  DualSeq seq;
  seq.blk_off = blk_off;
  seq.tile_off = tile_off;
  seq.n_tiles = n_tiles;
  seq.num_experts = num_experts;
  seq.unit_group = m_group > 0 ? (m_group + 1) / 2 : 0;
  seq.slots = slots != 0;
  seq.total = tile_off[num_experts];
  seq.cut = dual_cut(seq.total, grid);
  int64_t written = 0;
  WorkItem w[2];
  for (long long i = 0;; ++i) {
    const int count = dual_items_at(seq, i, cta, grid, w);
    if (count < 0) break;
    for (int s = 0; s < count; ++s) {
      if (written < max_items) {
        items[4 * written + 0] = w[s].expert;
        items[4 * written + 1] = w[s].m_block;
        items[4 * written + 2] = w[s].n_tile;
        items[4 * written + 3] = w[s].m_count;
      }
      ++written;
    }
  }
  return written;
}

extern "C" int b200moe_gemm_set_act_stores(int bulk) {
  b200moe::g_tma_act_stores.store(bulk ? 1 : 0, std::memory_order_relaxed);
  return B200MOE_OK;
}

extern "C" int b200moe_gemm_set_tiling(int mode) {
  using namespace b200moe;
  if (mode < 0 || mode > 2)
    return fail(B200MOE_ERR_SHAPE, "gemm_set_tiling: mode must be 0 (automatic), 1 or 2, got %d", mode);
  g_tiling.store(mode, std::memory_order_relaxed);
  return B200MOE_OK;
}

extern "C" int b200moe_gemm_measured_cycles(uint64_t* out8, int reset) {
  using namespace b200moe;
  uint64_t* out6 = out8;
  if (!out6) return fail(B200MOE_ERR_NULL, "gemm_measured_cycles: null pointer");
  unsigned long long v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(v, g_gemm_cycles, sizeof(v));
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "gemm_measured_cycles: %s", cudaGetErrorString(e));
  for (int i = 0; i < 8; ++i) out6[i] = v[i];
  if (reset) {
    const unsigned long long zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_gemm_cycles, zero, sizeof(zero));
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "gemm_measured_cycles: %s", cudaGetErrorString(e));
  }
#ifdef B200MOE_MEASURE_CYCLES
  return 1;
#else
  return 0;
#endif
}

extern "C" int b200moe_gemm_device_status(int reset) {
  using namespace b200moe;
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "gemm_device_status: %s", cudaGetErrorString(e));
  if (reset && v != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "gemm_device_status: %s", cudaGetErrorString(e));
  }
  return v;
}
