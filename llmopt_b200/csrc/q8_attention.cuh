// Paged grouped-Q8 attention: shared declarations.
#pragma once
#include "common.cuh"

namespace llmopt {

// Q8PagedAttentionParams, lib/metal_cache_source.ml:352-369 (64 bytes).
struct PagedParams {
  uint32_t batches, query_heads, kv_heads, past_length, head_dim, mask_batches, mask_heads,
      token_elements, key_offset, value_offset, group_size, token_stride;
  float scale;
  uint32_t query_length, mask_dtype, window;
};
static_assert(sizeof(PagedParams) == 64, "parameter block is 64 bytes");

// Largest number of key-range splits one (batch, kv head) is cut into.
constexpr uint32_t kMaxAttentionSplits = 64;

// Floats of split scratch per (batch, kv head, split): 8 maxima, 8 denominators
// and 8 x head_dim accumulators.
inline size_t paged_split_record_floats(uint32_t head_dim) { return 16 + 8 * (size_t)head_dim; }

// The split path proper, on caller-provided scratch (no allocation inside).  Slot values
// >= pool_tokens are never dereferenced (0xffffffff: the caller vouches for its slot table).
int launch_paged_attention_split_on(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride,
                                    float* scratch, uint32_t splits, uint32_t pool_tokens);
uint32_t paged_pick_splits(const KernelArgs& args, const PagedParams& p);

}  // namespace llmopt
