/*
 * CPU oracle (test infrastructure, never part of the product path) for token alignment.
 *
 * Plain-C restatement of the reference's moe_align_block_size
 * (src/moe_align_block_size.cu:58-133 of electrock-infer) as one sequential pass:
 *   cnt[e]      = number of i with ids[i] == e                         (:87-90 summed by :95-101)
 *   cumsum[e+1] = cumsum[e] + ceil(cnt[e] / block) * block             (:105-112)
 *   *npp        = cumsum[E]                                            (:112)
 *   expert_ids[b] = e for every block b of expert e                    (:117-122)
 *   sorted[cumsum[e] + r] = i, r = number of j < i with ids[j] == e    (:125-132)
 * Slots that receive no index are left as the caller filled them, like the reference kernel.
 * Indices with an expert outside [0, E) are skipped (the reference leaves that undefined).
 *
 * Build: gcc -O2 -shared -fPIC -o _build/liboracle.so align_oracle.c
 */
#include <stdint.h>
#include <stdlib.h>

int oracle_align_block_size(const int64_t* ids, int64_t numel, int num_experts, int block_size,
                            int32_t* sorted, int64_t sorted_capacity, int32_t* expert_ids,
                            int64_t expert_ids_capacity, int32_t* num_tokens_post_pad,
                            int32_t* expert_offsets /* may be NULL, E + 1 entries */) {
  if (num_experts < 1 || block_size < 1 || numel < 0) return -1;
  int64_t* cnt = (int64_t*)calloc((size_t)num_experts, sizeof(int64_t));
  int64_t* cumsum = (int64_t*)calloc((size_t)num_experts + 1, sizeof(int64_t));
  int64_t* next = (int64_t*)calloc((size_t)num_experts, sizeof(int64_t));
  if (!cnt || !cumsum || !next) { free(cnt); free(cumsum); free(next); return -2; }
  int rc = 0;
  for (int64_t i = 0; i < numel; ++i)
    if (ids[i] >= 0 && ids[i] < num_experts) ++cnt[ids[i]];
  for (int e = 0; e < num_experts; ++e)
    cumsum[e + 1] = cumsum[e] + (cnt[e] + block_size - 1) / block_size * block_size;
  if (cumsum[num_experts] > sorted_capacity ||
      cumsum[num_experts] / block_size > expert_ids_capacity) {
    rc = -3;
  } else {
    *num_tokens_post_pad = (int32_t)cumsum[num_experts];
    if (expert_offsets)
      for (int e = 0; e <= num_experts; ++e) expert_offsets[e] = (int32_t)cumsum[e];
    for (int e = 0; e < num_experts; ++e)
      for (int64_t s = cumsum[e]; s < cumsum[e + 1]; s += block_size)
        expert_ids[s / block_size] = e;
    for (int64_t i = 0; i < numel; ++i) {
      const int64_t e = ids[i];
      if (e < 0 || e >= num_experts) continue;
      sorted[cumsum[e] + next[e]] = (int32_t)i;
      ++next[e];
    }
  }
  free(cnt); free(cumsum); free(next);
  return rc;
}
