/*
 * b200moe.h — C ABI of libb200moe.so: the Mixtral mixture-of-experts layer hot path for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, never synchronises, never allocates device memory and never
 * throws (the b200moe_peer_* set-up helpers and b200moe_gemm_device_status are the exceptions and
 * say so).  The return value is 0 on success or a negative B200MOE_ERR_* code; the text of the
 * most recent failure on the calling thread is available from b200moe_last_error().
 *
 * Each declaration names the reference interface it replaces (paths are relative to the
 * electrock-infer source tree).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 1

/* Element types of floating-point tensors. */
enum {
  B200MOE_F32 = 0,
  B200MOE_F16 = 1,
  B200MOE_BF16 = 2
};

/* Element types of expert-index tensors (topk_ids). */
enum {
  B200MOE_I32 = 0,
  B200MOE_I64 = 1,
  B200MOE_I16 = 2,
  B200MOE_I8 = 3,
  B200MOE_U8 = 4
};

/* Status codes. */
enum {
  B200MOE_OK = 0,
  B200MOE_ERR_SHAPE = -1,       /* a size the kernels do not support (the text says which) */
  B200MOE_ERR_DTYPE = -2,       /* unsupported element type */
  B200MOE_ERR_NULL = -3,        /* a required pointer is NULL */
  B200MOE_ERR_WORKSPACE = -4,   /* workspace missing or too small */
  B200MOE_ERR_ALIGN = -5,       /* a pointer is not aligned as required */
  B200MOE_ERR_CUDA = -6,        /* a CUDA runtime / driver call failed */
  B200MOE_ERR_UNSUPPORTED = -7  /* not built for this device */
};

/* A CUDA stream handle (cudaStream_t) passed as an opaque pointer; NULL is the default stream. */
typedef void* b200moe_stream_t;

/* ABI version of the loaded library (B200MOE_ABI_VERSION at build time). */
int b200moe_abi_version(void);

/* Kernels this library has launched in this process so far (every entry point counts its own
 * launches, including the second kernel of a grouped-GEMM launch pair): for benchmarks that report
 * how many of the library's kernels ran inside a timed region. */
int64_t b200moe_kernel_launch_count(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* b200moe_last_error(void);

/*
 * Router: row-wise softmax over num_experts fp32/bf16/fp16 logits followed by top-2 selection.
 * Replaces electrock_infer::topk_softmax (src/topk_softmax_kernels.cu:85-111, bound in
 * pytorch_bind.cpp:24-29) and, with renormalize != 0, the torch router the layer really uses
 * (layers/moe/softmax_topk.py:3-29 followed by layers/moe/fused_moe.py:161-162).
 *
 *   topk_weights  f32 [num_tokens, 2]   softmax probabilities of the two chosen experts, largest
 *                                       first; divided by their sum when renormalize != 0
 *   topk_indices  i32 [num_tokens, 2]   expert indices; on equal logits the lower index wins
 *   gating_output [num_tokens, num_experts] logits of element type logits_dtype
 *
 * Like the reference, only num_experts == 8 and topk == 2 are accepted (B200MOE_ERR_SHAPE
 * otherwise).  num_tokens may be 0 and need not be a multiple of anything.
 */
int b200moe_topk_softmax(float* topk_weights, int32_t* topk_indices, const void* gating_output,
                         int logits_dtype, int64_t num_tokens, int num_experts, int topk,
                         int renormalize, b200moe_stream_t stream);

/*
 * Gate projection fused with the router: logits[t, e] = sum_h hidden_states[t, h] * gate_weight[e, h]
 * (fp32 accumulation of bf16 inputs), then the softmax + top-2 of b200moe_topk_softmax, in one pass
 * over the activations.  Replaces the gate linear layer plus the router call of the reference's
 * MixtralMoE.forward (models/mixtral.py:59-61: ReplicatedLinear, layers/linear.py:32-54, followed
 * by fused_topk, layers/moe/fused_moe.py:130-164).
 *
 *   hidden_states bf16 [num_tokens, hidden], gate_weight bf16 [8, hidden]; hidden % 256 == 0
 *   logits_out    optional f32 [num_tokens, 8]: the logits the routing decision was made on
 *   round_logits_bf16 != 0 rounds the logits to bf16 first, like the reference's bf16 linear layer
 */
int b200moe_gate_topk_softmax(const void* hidden_states, const void* gate_weight,
                              float* topk_weights, int32_t* topk_indices, float* logits_out,
                              int64_t num_tokens, int64_t hidden, int num_experts, int topk,
                              int renormalize, int round_logits_bf16, b200moe_stream_t stream);

/*
 * Token alignment: counting sort of the flat (token, slot) pairs by expert, each expert's run
 * padded to a multiple of block_size.  Replaces electrock_infer::moe_align_block_size
 * (src/moe_align_block_size.cu:140-230, bound in pytorch_bind.cpp:43-50).
 *
 *   topk_ids             [numel] expert index of pair i (row-major [num_tokens, topk])
 *   sorted_token_ids     i32 [sorted_capacity], capacity >= numel + num_experts*(block_size-1);
 *                        slot off[e] + r receives the r-th smallest pair index routed to e
 *   expert_ids           i32 [expert_ids_capacity] expert of each block of block_size slots
 *   num_tokens_post_pad  i32 [1] total padded length (sum over experts of the padded counts)
 *   expert_offsets       optional i32 [num_experts + 1] padded start offset of every expert
 *                        (no counterpart in the reference; may be NULL)
 *
 * With fill_pads == 0 padding slots and everything beyond num_tokens_post_pad are left untouched,
 * exactly like the reference kernel, whose Python wrapper prefills -1
 * (layers/moe/moe_align_block_size.py:39-42).  With fill_pads != 0 the kernel itself writes -1
 * to every slot of sorted_token_ids that holds no pair, so no separate fill launch is needed.
 *
 * Inputs longer than b200moe_align_single_pass_max() (65536 pair indices) need a workspace of
 * b200moe_align_workspace_bytes() bytes (16-byte aligned device memory) and take three launches;
 * shorter inputs run as one launch (one CTA up to 8192 indices, one thread-block cluster of up
 * to 8 CTAs above that) and ignore it.  num_experts must lie in [1, b200moe_align_max_experts()] (8).
 * Pair indices with an expert outside [0, num_experts) are skipped.
 */
int b200moe_align_block_size(const void* topk_ids, int ids_dtype, int64_t numel, int num_experts,
                             int block_size, int32_t* sorted_token_ids, int64_t sorted_capacity,
                             int32_t* expert_ids, int64_t expert_ids_capacity,
                             int32_t* num_tokens_post_pad, int32_t* expert_offsets, int fill_pads,
                             void* workspace, size_t workspace_bytes, b200moe_stream_t stream);
size_t b200moe_align_workspace_bytes(int64_t numel, int num_experts);
int64_t b200moe_align_single_pass_max(void);
int b200moe_align_max_experts(void);

/*
 * Token alignment for hosts that must not allocate device memory.  No counterpart in the
 * reference.
 *
 * Why it exists: b200moe_align_block_size needs a caller workspace for long inputs.  Some hosts
 * cannot provide one at call time: an inference server that gave the whole device to a pre-sized
 * pool at start-up (the reference engine sizes its KV cache from the free memory it finds and
 * leaves nothing behind), a plain C or cgo/JNI host with no device allocator of its own, or a
 * latency-critical loop where cudaMalloc would stall the device.  This entry point computes the
 * same outputs, with the same arguments minus the workspace, and keeps its segment counters in a
 * fixed array inside the library image (about 64 KiB of device memory on every GPU that loads the
 * library, held until the process exits).  It calls no cudaMalloc, cudaFree or other allocating
 * routine.
 *
 * Limits and rules:
 *   - numel <= b200moe_align_noalloc_max_numel() (16 Mi pair indices); larger inputs are rejected
 *     with B200MOE_ERR_SHAPE and must use the workspace variant.
 *   - The first call on each device with more than b200moe_align_single_pass_max() indices looks up
 *     the device address of the built-in array (a runtime query, no allocation) and keeps it for
 *     the life of the process.  Make that first call during set-up, before any stream capture.
 *     Shorter inputs never touch the array.  The kept address does not survive cudaDeviceReset():
 *     a process that resets a device must not call this entry point on it afterwards.
 *   - All calls on a device share the one array.  Nothing in it has to be zero beforehand (every
 *     word a call reads is first written by that call), but two calls whose kernels overlap on the
 *     GPU - different streams without ordering between them - race on it and corrupt each other.
 *     Calls on one stream, or ordered by events, are safe.
 */
int b200moe_align_block_size_noalloc(const void* topk_ids, int ids_dtype, int64_t numel,
                                     int num_experts, int block_size, int32_t* sorted_token_ids,
                                     int64_t sorted_capacity, int32_t* expert_ids,
                                     int64_t expert_ids_capacity, int32_t* num_tokens_post_pad,
                                     int32_t* expert_offsets, int fill_pads,
                                     b200moe_stream_t stream);
int64_t b200moe_align_noalloc_max_numel(void);

/*
 * SwiGLU activation as a stand-alone op: out[r, j] = cast(silu_f32(in[r, j])) * in[r, d + j].
 * Replaces electrock_infer::silu_and_mul (src/activation_kernels.cu:97-150, bound in
 * pytorch_bind.cpp:18-22): the 16-bit types round SiLU to the element type before the product
 * and use the fast exponential; fp32 uses expf.
 *
 *   out [num_rows, d], input [num_rows, 2*d], both of element type dtype, contiguous.
 */
int b200moe_silu_and_mul(void* out, const void* input, int dtype, int64_t num_rows, int64_t d,
                         b200moe_stream_t stream);

/*
 * Combine: out[t, :] = in[t, 0, :] + in[t, 1, :] in the element type.
 * layout 0 replaces electrock_infer::moe_sum (input [num_tokens, 2, hidden],
 * src/moe_sum.cu:50-74, pytorch_bind.cpp:31-35); layout 1 replaces
 * electrock_infer::moe_sum_efficient (input [num_tokens, hidden, 2],
 * src/moe_sum_efficient.cu:52-79, pytorch_bind.cpp:37-41; bf16 is accepted here too).
 * topk must be 2, as in the reference.
 */
int b200moe_moe_sum(const void* input, void* output, int dtype, int64_t num_tokens, int64_t hidden,
                    int topk, int layout, b200moe_stream_t stream);

/*
 * RMSNorm of every row, optionally fused with the residual add that precedes it in the decoder
 * layer; this is the kernel that produces the MoE layer's input.  Replaces
 * electrock_infer::rms_norm / add_rms_norm (src/add_rms_norm.cu:145-200 and :21-142, bound in
 * pytorch_bind.cpp:53-66) with the arithmetic of the Python path the reference really runs
 * (layers/layernorm.py:17-43):
 *   residual != NULL:  s = float(input) + float(residual);  residual <- cast(s)
 *   residual == NULL:  s = float(input)
 *   input <- cast(s * rsqrt(mean(s^2) + epsilon)) * weight        (product in the element type)
 * input, residual [num_tokens, hidden] and weight [hidden] share the element type dtype; hidden must
 * be a multiple of 8 (4 for fp32) and at most 16384 (8192 for fp32).  Unlike the reference kernel
 * there is no hidden == 4096 restriction and the launch is on the caller's stream.
 */
int b200moe_add_rms_norm(void* input, void* residual, const void* weight, int dtype,
                         int64_t num_tokens, int64_t hidden, float epsilon,
                         b200moe_stream_t stream);

/*
 * Row gather into expert-sorted order: dst[s, :] = src[sorted_token_ids[s] / top_k, :] for every
 * slot s < *num_tokens_post_pad holding a pair; padding slots are zero-filled.  This is the
 * A-operand addressing of the reference's grouped GEMM (layers/moe/fused_moe.py:88-91) done once
 * ahead of the GEMM so that its tiles are dense.
 *
 *   src [num_src_rows, row_elems] bf16, dst [sorted_capacity, row_elems] bf16;
 *   row_elems must be a multiple of 8.
 */
int b200moe_gather_rows(const void* src, void* dst, const int32_t* sorted_token_ids,
                        const int32_t* num_tokens_post_pad, int64_t sorted_capacity,
                        int64_t num_src_rows, int64_t row_elems, int top_k,
                        b200moe_stream_t stream);

/*
 * Row scatter, the inverse of the gather: dst[index[i], :] = src[i, :] for i < num_rows (bf16 rows,
 * row_elems % 8 == 0); indices outside [0, num_dst_rows) are skipped.  Used by the expert-parallel
 * return path to put expert outputs back at their pair index, the addressing of the reference's
 * grouped-GEMM store (layers/moe/fused_moe.py:123-125).
 */
int b200moe_scatter_rows(const void* src, void* dst, const int32_t* index, int64_t num_rows,
                         int64_t num_dst_rows, int64_t row_elems, b200moe_stream_t stream);

/*
 * Grouped expert GEMM 1 with the SwiGLU epilogue (tcgen05 / TMEM / TMA):
 *   act[s, j] = bf16( silu(g) * u ),  g = sum_k a[s, k] * w13[e, j, k],
 *                                     u = sum_k a[s, k] * w13[e, inter + j, k],
 * for every slot s < *num_tokens_post_pad, e = expert_ids[s / block_m].  Accumulation, SiLU and
 * the product are fp32; one rounding to bf16 at the end.  Replaces the first
 * _invoke_fused_moe_kernel call plus _C.silu_and_mul (layers/moe/fused_moe.py:250-272,
 * kernel :15-125).
 *
 *   a_sorted  bf16 [sorted_capacity, hidden]   rows in expert-sorted order (b200moe_gather_rows)
 *   w13       bf16 [num_experts, 2*inter, hidden]   gate rows first, then up rows
 *   act       bf16 [sorted_capacity, inter]
 *   block_m   the block_size used for alignment: 128 (one CTA per 128 x 256 tile) or 256 (a pair
 *             of CTAs, tcgen05 cta_group::2, per 256 x 256 tile)
 *   hidden % 64 == 0, inter % 128 == 0 (inter % 64 == 0 when inter < 128 is not supported).
 */
int b200moe_grouped_gemm_w13_swiglu(const void* a_sorted, const void* w13, void* act,
                                    const int32_t* expert_ids,
                                    const int32_t* num_tokens_post_pad, int64_t sorted_capacity,
                                    int num_experts, int64_t hidden, int64_t inter, int block_m,
                                    b200moe_stream_t stream);

/*
 * The same GEMM with the row gather folded in: the A rows are fetched straight from the token
 * tensor by TMA row gathers (cp.async.bulk.tensor tile::gather4, four rows per instruction,
 * a_row(s) = sorted_token_ids[s] / top_k), which is the reference kernel's A addressing
 * (layers/moe/fused_moe.py:88-91) without a separate gather pass or an expert-sorted copy.
 * Padding slots read row 0; their results are never consumed.  block_m must be 128.
 * Measured on B200 at Mixtral shape this variant is about 2.6x slower than gather_rows followed by
 * the tiled kernel (32 four-row gathers per K step against one tiled box), so the layer uses the
 * latter; the entry point is kept for callers that cannot afford the expert-sorted copy.
 *
 *   tokens  bf16 [num_tokens, hidden];  sorted_token_ids i32 [sorted_capacity], 16-byte aligned
 */
int b200moe_grouped_gemm_w13_swiglu_gather(const void* tokens, int64_t num_tokens, int top_k,
                                           const int32_t* sorted_token_ids, const void* w13,
                                           void* act, const int32_t* expert_ids,
                                           const int32_t* num_tokens_post_pad,
                                           int64_t sorted_capacity, int num_experts,
                                           int64_t hidden, int64_t inter, int block_m,
                                           b200moe_stream_t stream);

/*
 * Grouped expert GEMM 2 with the routing-weight epilogue:
 *   out[p, n] = bf16( topk_weights[p] * sum_k act[s, k] * w2[e, n, k] ),  p = sorted_token_ids[s]
 * for every slot s holding a pair; rows of out are indexed by the flat pair index p, i.e. out is
 * the reference's [num_tokens, topk, hidden] cache.  Replaces the second
 * _invoke_fused_moe_kernel call (layers/moe/fused_moe.py:282-287, epilogue :116-125).
 *
 *   act  bf16 [sorted_capacity, inter], w2 bf16 [num_experts, hidden, inter],
 *   out  bf16 [num_pairs, hidden], topk_weights f32 [num_pairs];
 *   hidden % 256 == 0 (output tile width), inter % 64 == 0, block_m 128 or 256 as above.
 */
int b200moe_grouped_gemm_w2_scale(const void* act, const void* w2, void* out,
                                  const float* topk_weights, const int32_t* sorted_token_ids,
                                  const int32_t* expert_ids, const int32_t* num_tokens_post_pad,
                                  int64_t sorted_capacity, int64_t num_pairs, int num_experts,
                                  int64_t hidden, int64_t inter, int block_m,
                                  b200moe_stream_t stream);

/*
 * Expert-parallel variants that move rows over NVLink inside the kernels themselves (no reference
 * counterpart: the reference has no expert parallelism, layers/moe/mixtral_moe.py:9-13).
 *
 * b200moe_gather_rows_peer is b200moe_gather_rows with the token tensor split over num_ranks GPUs:
 * token row r is row r % rows_per_rank of the tensor at src_table[r / rows_per_rank].  src_table is a
 * DEVICE array of num_ranks device pointers (local memory or peer mappings); the kernel pulls the
 * rows with plain loads.  This is the dispatch step.
 *
 * b200moe_grouped_gemm_w2_scale_peer is b200moe_grouped_gemm_w2_scale whose epilogue stores output
 * row p (a global pair index) to row p % pairs_per_rank of the tensor at
 * out_table[p / pairs_per_rank] (a DEVICE array of device pointers), i.e. directly into the memory
 * of the GPU that owns the token.  This is the return step.  topk_weights holds num_ranks *
 * pairs_per_rank entries (the routing weights of all ranks).  The caller orders the ranks around
 * these kernels (every rank's source rows must be in place before any rank gathers; every rank's
 * second GEMM must have finished before a rank combines) with stream-ordered collectives.
 */
int b200moe_gather_rows_peer(const void* const* src_table, int num_ranks, int64_t rows_per_rank,
                             void* dst, const int32_t* sorted_token_ids,
                             const int32_t* num_tokens_post_pad, int64_t sorted_capacity,
                             int64_t row_elems, int top_k, b200moe_stream_t stream);
int b200moe_grouped_gemm_w2_scale_peer(const void* act, const void* w2, void* const* out_table,
                                       int num_ranks, int64_t pairs_per_rank,
                                       const float* topk_weights, const int32_t* sorted_token_ids,
                                       const int32_t* expert_ids,
                                       const int32_t* num_tokens_post_pad, int64_t sorted_capacity,
                                       int num_experts, int64_t hidden, int64_t inter, int block_m,
                                       b200moe_stream_t stream);

/*
 * Tensor-parallel combine over NVLink (no reference counterpart: the reference adds the ranks'
 * partial layer outputs with an NCCL all-reduce, layers/moe/mixtral_moe.py:114-116).
 *
 * With the intermediate dimension sharded over num_ranks GPUs, every rank's second GEMM
 * (b200moe_grouped_gemm_w2_scale_peer with out_table[j] = rank j's receive buffer + this rank's
 * slot) stores the rows of token slice j straight into rank j's receive buffer
 * input [num_ranks, num_tokens, 2, hidden] (num_tokens = tokens per slice).  This function then
 * adds each slot's two rows and rounds like b200moe_moe_sum (the per-rank partial result of the
 * reference), adds the per-slot sums in fp32 in slot order, rounds once to the element type and
 * stores the result row to row (row_offset + t) of the [*, hidden] tensor at out_table[j] for
 * EVERY j (a DEVICE array of num_ranks device pointers, local memory or peer mappings):
 * reduce-scatter and all-gather of the all-reduce without a separate collective.  The caller
 * orders the ranks around it with stream-ordered collectives (all second GEMMs done before this
 * call; all calls done before the outputs are read).  num_ranks <= 8, topk must be 2, hidden a
 * multiple of 16 bytes.
 */
int b200moe_moe_sum_ranks_push(const void* input, void* const* out_table, int num_ranks,
                               int64_t row_offset, int dtype, int64_t num_tokens, int64_t hidden,
                               int topk, b200moe_stream_t stream);

/*
 * Set-up helpers for peer-visible buffers (these DO allocate and synchronise; not for the hot
 * path).  b200moe_peer_alloc: cudaMalloc + zero fill + CUDA IPC handle (64 bytes) for the other
 * rank processes of the node.  b200moe_peer_open maps another process's buffer from its handle;
 * b200moe_peer_close unmaps it; b200moe_peer_free releases an own buffer.
 */
int b200moe_peer_alloc(size_t bytes, void** ptr, void* ipc_handle_64);
int b200moe_peer_open(const void* ipc_handle_64, void** ptr);
int b200moe_peer_close(void* ptr);
int b200moe_peer_free(void* ptr);

/*
 * Paged KV cache: the other custom-kernel family next to the MoE layer in the reference's decoder.
 *
 * b200moe_paged_store_kvcache replaces electrock_infer::paged_store_kvcache
 * (src/store_kv_cache.hip:65-110, pytorch_bind.cpp:92-99) and the Triton store_kvcache the
 * attention layer calls (layers/attention_triton_kernel.py:75-106, layers/attention.py:33):
 * token i's key and value rows ([num_kv_heads * head_dim] elements, row strides in elements) are
 * copied to slot slot_mapping[i] of k_cache / v_cache [num_blocks, block_size, num_kv_heads,
 * head_dim].  Negative slots are skipped like the reference; slots >= num_blocks * block_size
 * are skipped too (the reference would write out of bounds).  Any of the three float types.
 */
int b200moe_paged_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                                const int32_t* slot_mapping, int dtype, int64_t num_tokens,
                                int num_kv_heads, int head_dim, int64_t key_row_stride,
                                int64_t value_row_stride, int64_t num_blocks, int block_size,
                                b200moe_stream_t stream);

/*
 * b200moe_paged_attn_varlen replaces electrock_infer::paged_attn_varlen
 * (src/paged_attn_gqa_varlen.hip:216-268, pytorch_bind.cpp:68-77): decode attention of one query
 * token per sequence over the paged cache, grouped-query heads.
 *
 *   q, out [batch, q_heads, 128]; k_cache, v_cache [num_blocks, block_size, kv_heads, 128];
 *   block_table [batch, max_blocks_per_seq] int32; context_lens [batch] int32.
 *   out[b, h] = softmax(softmax_scale * q[b, h] . K[b, h / group]) @ V[b, h / group] over the first
 *   context_lens[b] tokens of sequence b.
 *
 * bf16 or fp16, head_dim 128 (as the reference); block_size any multiple of 16 (the reference:
 * 32 only); up to 16 query heads per KV head.  An empty context gives a zero row (the reference
 * divides 0 by 0).  num_splits cuts every context into that many ranges handled by separate CTAs
 * and merged by a second kernel: b200moe_paged_attn_num_splits suggests a value for a batch (1
 * when the batch alone fills the GPU); num_splits > 1 needs a workspace of
 * b200moe_paged_attn_workspace_bytes bytes.
 */
int b200moe_paged_attn_num_splits(int batch, int kv_heads, int64_t max_context);
size_t b200moe_paged_attn_workspace_bytes(int batch, int q_heads, int num_splits);
int b200moe_paged_attn_varlen(const void* q, const void* k_cache, const void* v_cache, void* out,
                              const int32_t* block_table, const int32_t* context_lens, int dtype,
                              int batch, int q_heads, int kv_heads, int head_dim,
                              int64_t num_blocks, int block_size, int max_blocks_per_seq,
                              float softmax_scale, int num_splits, void* workspace,
                              size_t workspace_bytes, b200moe_stream_t stream);

/*
 * The whole layer in one call: router (softmax, top-2, optional renormalisation) -> token alignment
 * with block 128 (writes its own padding) -> gather of the routed rows -> grouped GEMM w13 + SwiGLU
 * -> grouped GEMM w2 x routing weight -> combine, issued back to back on `stream` by the entry
 * points above.  Replaces fused_experts of layers/moe/fused_moe.py:170-293 for bf16 tensors and
 * top_k = 2; `output` may be `hidden_states` (the in-place use of FusedMoE.forward,
 * layers/moe/mixtral_moe.py:103-112).
 *
 *   hidden_states [num_tokens, hidden] bf16, gating_output [num_tokens, num_experts] of logits_dtype,
 *   w13 [num_experts, 2*inter, hidden] bf16 (gate rows first), w2 [num_experts, hidden, inter] bf16,
 *   output [num_tokens, hidden] bf16.
 * Scratch, all caller-owned, with R = b200moe_fused_experts_rows(num_tokens, top_k, num_experts):
 *   topk_weights f32 [num_tokens * top_k], topk_ids i32 [num_tokens * top_k], sorted_token_ids i32 [R],
 *   expert_ids i32 [ceil(R / 128)], num_tokens_post_pad i32 [1],
 *   align_workspace of b200moe_align_workspace_bytes(num_tokens * top_k, num_experts) bytes (may be
 *   NULL when that is 0), a_sorted bf16 [R, hidden], act bf16 [R, inter],
 *   pair_rows bf16 [num_tokens * top_k, hidden].
 * Nothing in the scratch has to be initialised.  No allocation, no host synchronisation.
 */
size_t b200moe_fused_experts_rows(int64_t num_tokens, int top_k, int num_experts);
int b200moe_fused_experts(const void* hidden_states, const void* gating_output, int logits_dtype,
                          const void* w13, const void* w2, void* output, int64_t num_tokens,
                          int num_experts, int top_k, int64_t hidden, int64_t inter, int renormalize,
                          float* topk_weights, int32_t* topk_ids, int32_t* sorted_token_ids,
                          int32_t* expert_ids, int32_t* num_tokens_post_pad, void* align_workspace,
                          size_t align_workspace_bytes, void* a_sorted, void* act, void* pair_rows,
                          b200moe_stream_t stream);

/*
 * Device-side status word of the grouped GEMMs.  Their waits on memory barriers are bounded; a
 * wait that runs out records a non-zero code here and the kernel returns.  Reading synchronises
 * with the device.  Returns the code (0 = no error) or a negative B200MOE_ERR_*; `reset` != 0
 * clears it.
 */
int b200moe_gemm_device_status(int reset);

/*
 * Cycle accounting of the two-block grouped GEMM, for measurement builds of the library
 * (csrc/grouped_gemm.cu compiled with -DB200MOE_MEASURE_CYCLES; the shipped build records
 * nothing).  Fills out8 with sums over all CTAs since the last reset: [0] SM cycles one epilogue
 * warp spent draining accumulators, [1] accumulators it drained, [2] cycles the MMA-issuing thread
 * waited for operand stages, [3] cycles it waited for a free accumulator, [4] cycles it spent in
 * its tile loop, [5] tiles it processed, [6] and [7] the part of [2] that fell into the first and
 * the last K steps of two-block tiles (where block 0 runs ahead of block 1).  Synchronises with the device.  Returns 1 for a
 * measurement build, 0 for a normal build (all zeros), or a negative B200MOE_ERR_*.
 */
int b200moe_gemm_measured_cycles(uint64_t* out8, int reset);

/*
 * Tiling of the one-CTA grouped GEMMs (block_m = 128), a process-wide setting for benchmarks and
 * tests: 0 (default) chooses by batch size, 1 forces one 128-row M block per tile (128 x 256
 * accumulator, double-buffered in tensor memory), 2 forces two M blocks of one expert per tile
 * (they share every weight stage; chosen by default, on the device from the real block counts,
 * where its estimated finishing time is 3 % below that of one-block tiles, see
 * b200moe_gemm_two_block_choice; never when K is below 3072).
 * All tilings produce the same bits.  The reference's counterpart is the tile configuration table
 * of layers/moe/fused_moe.py:327-339.  Returns 0 or B200MOE_ERR_SHAPE.
 */
int b200moe_gemm_set_tiling(int mode);

/*
 * How the first grouped GEMM writes its output, a process-wide setting for benchmarks and tests:
 * non-zero (default) = bulk tensor stores of 32 rows x 64 columns issued by one lane per epilogue
 * warp, where the tile is a multiple of 64 columns wide; 0 = 16-byte stores from every lane.  Same
 * bits either way.  No counterpart in the reference.
 */
int b200moe_gemm_set_act_stores(int bulk);

/*
 * Host-side view of the choice between one and two M blocks per tile that the grouped GEMMs make
 * on the device under b200moe_gemm_set_tiling(0): 1 when two-block tiles would run for experts
 * holding `blocks_per_expert[e]` M blocks of 128 rows, an output of `n_tiles` N tiles, a reduction
 * length `k`, `ctas` CTAs (the SM count) and the odd blocks dealt as slots (`slots` non-zero: the
 * first GEMM) or not; 0 when one-block tiles would.  The rule compares estimated finishing times
 * (see two_block_tiles_win in csrc/grouped_gemm.cu).  Runs on the host; no device is touched.
 * Returns 0, 1 or a negative B200MOE_ERR_*.  No counterpart in the reference beyond its tile
 * configuration table (layers/moe/fused_moe.py:327-339).
 */
int b200moe_gemm_two_block_choice(const int32_t* blocks_per_expert, int num_experts, int n_tiles,
                                  int64_t k, int slots, int ctas);

/*
 * Host-side view of the work list of the two-block tiling, for tests and tuning: the items that
 * CTA `cta` of `grid` processes, in order, when the experts hold `blocks_per_expert[e]` M blocks
 * of 128 rows, the output has `n_tiles` N tiles, `m_group` is the L2 grouping of M blocks and
 * `slots` says how the odd block of an expert is dealt (non-zero, the first GEMM: against two N
 * tiles in a row on one CTA; zero, the second GEMM: as a one-block tile per N tile).
 * Runs the same code as the kernel's scheduler, on the host; no device is touched.  Writes up to
 * `max_items` quadruples (expert, first M block, N tile, M blocks in the item: 1 or 2) to `items`
 * and returns the number of items of that CTA (which may exceed `max_items`), or a negative
 * B200MOE_ERR_*.  No counterpart in the reference (its launch grid is one program per tile,
 * layers/moe/fused_moe.py:296-325).
 */
int64_t b200moe_gemm_two_block_schedule(const int32_t* blocks_per_expert, int num_experts,
                                        int n_tiles, int m_group, int slots, int grid, int cta,
                                        int32_t* items, int64_t max_items);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
