// Paged grouped-Q8 attention for sm_100a.
//
// Replaces llmopt_attention_q8_paged_simd_{h64,generic,h256,h512,h64_gqa3,
// h64_split8,h64_gqa3_split8} (lib/metal_cache_source.ml:403-1247): query
// [b, hq, q, D] f16, current key / value [b, hkv, q, D] f16, the Q8 token pool
// addressed through a slot table, optional mask; output token-first
// [b, q, hq, D] f16.  Parameter block: 64 bytes, lib/metal_cache_source.ml:352-369.
//
// Two code paths behind the same names:
//  * `paged_rows_kernel`: one warp per (batch, head, query position) walking
//    the keys in order with the reference's single-pass online softmax. It
//    accepts everything the reference accepts (mask, window, q > 1, any
//    D <= 512) and is the fallback.
//  * the split-K flash-decode path (`paged_split_kernel` + `paged_merge_kernel`)
//    for the decode shape (q = 1, no mask, D in {64, 128}, group 32/64): the key
//    range of every (batch, kv head) is cut into splits handled by different
//    CTAs so long contexts fill the machine; each warp keeps (max, denominator,
//    accumulators) for all query heads that share the KV head, so K and V are
//    read and dequantised once per KV head; a second kernel merges the splits
//    and folds in the current token.
#include "q8_attention.cuh"
#include "q8_codec.cuh"

namespace llmopt {
namespace {

__device__ __forceinline__ bool mask_active(const uint8_t* mask, const PagedParams& p, size_t index) {
  if (mask == nullptr || p.mask_batches == 0 || p.mask_dtype == 0) return true;
  if (p.mask_dtype == 2) return __half2float(reinterpret_cast<const __half*>(mask)[index]) >= 0.0f;
  return mask[index] != 0;
}

constexpr int kMaxFragments = 16;  // D <= 512, lib/metal_cache_source.ml:491

// Faithful row kernel: lib/metal_cache_source.ml:493-583.
__global__ void paged_rows_kernel(const __half* __restrict__ query, const __half* __restrict__ current_key,
                                  const __half* __restrict__ current_value, const uint8_t* __restrict__ pool,
                                  const uint32_t* __restrict__ slots, const uint8_t* __restrict__ mask,
                                  __half* __restrict__ output, PagedParams p, uint32_t slot_batch_stride,
                                  const uint32_t* __restrict__ past_cell, uint32_t pool_tokens,
                                  uint32_t* error_word) {
  grid_chain_prologue();
  if (past_cell) p.past_length = *past_cell;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t q_len = p.query_length == 0 ? 1 : p.query_length;
  const uint32_t rows = p.batches * p.query_heads * q_len;
  if (row >= rows) return;
  const uint32_t q_pos = row % q_len;
  const uint32_t head = (row / q_len) % p.query_heads;
  const uint32_t batch = row / (q_len * p.query_heads);
  const uint32_t kv_head = head / (p.query_heads / p.kv_heads);
  const uint32_t* batch_slots = slots + (size_t)batch * slot_batch_stride;
  const size_t query_base = (((size_t)batch * p.query_heads + head) * q_len + q_pos) * p.head_dim;
  const size_t current_base = ((size_t)batch * p.kv_heads + kv_head) * q_len * p.head_dim;
  const uint32_t key_length = p.past_length + q_pos + 1;
  const uint32_t first_key = (p.window == 0 || key_length <= p.window) ? 0 : key_length - p.window;
  const uint32_t fragments = (p.head_dim + 31u) / 32u;
  const uint32_t groups_per_head = p.head_dim / p.group_size;

  float q_values[kMaxFragments], results[kMaxFragments];
#pragma unroll
  for (int f = 0; f < kMaxFragments; ++f) {
    const uint32_t d = lane + f * 32;
    q_values[f] = (f < fragments && d < p.head_dim) ? __half2float(query[query_base + d]) : 0.0f;
    results[f] = 0.0f;
  }
  float maximum = -INFINITY, denominator = 0.0f;
  for (uint32_t key = first_key; key < key_length; ++key) {
    if (mask != nullptr && p.mask_batches > 0) {
      const uint32_t mask_batch = p.mask_batches == 1 ? 0 : batch;
      const uint32_t mask_head = p.mask_heads == 1 ? 0 : head;
      const size_t stride = (size_t)p.past_length + q_len;
      const size_t index = (((size_t)mask_batch * p.mask_heads + mask_head) * q_len + q_pos) * stride + key;
      if (!mask_active(mask, p, index)) continue;
    }
    const bool past = key < p.past_length;
    const int8_t* values = nullptr;
    const __half* scales = nullptr;
    if (past) {
      // a slot outside the pool is skipped (the key contributes nothing) and reported
      const uint32_t slot = batch_slots[key];
      if (slot >= pool_tokens) {
        if (lane == 0 && error_word) atomicExch(error_word, 1u);
        continue;
      }
      const size_t slot_base = (size_t)slot * p.token_stride;
      values = reinterpret_cast<const int8_t*>(pool + slot_base);
      scales = reinterpret_cast<const __half*>(pool + slot_base + p.token_elements);
    }
    float partial = 0.0f;
#pragma unroll
    for (int f = 0; f < kMaxFragments; ++f) {
      const uint32_t d = lane + f * 32;
      if (f < fragments && d < p.head_dim) {
        float key_value;
        if (past)
          key_value = (float)values[p.key_offset + kv_head * p.head_dim + d] *
                      __half2float(scales[p.key_offset / p.group_size + kv_head * groups_per_head + d / p.group_size]);
        else
          key_value = __half2float(current_key[current_base + (size_t)(key - p.past_length) * p.head_dim + d]);
        partial += q_values[f] * key_value;
      }
    }
    const float score = warp_sum(partial) * p.scale;
    const float next_maximum = fmaxf(maximum, score);
    const float previous_scale = denominator == 0.0f ? 0.0f : expf(maximum - next_maximum);
    const float current_scale = expf(score - next_maximum);
#pragma unroll
    for (int f = 0; f < kMaxFragments; ++f) {
      const uint32_t d = lane + f * 32;
      if (f < fragments && d < p.head_dim) {
        float value;
        if (past)
          value = (float)values[p.value_offset + kv_head * p.head_dim + d] *
                  __half2float(scales[p.value_offset / p.group_size + kv_head * groups_per_head + d / p.group_size]);
        else
          value = __half2float(current_value[current_base + (size_t)(key - p.past_length) * p.head_dim + d]);
        results[f] = results[f] * previous_scale + current_scale * value;
      }
    }
    denominator = denominator * previous_scale + current_scale;
    maximum = next_maximum;
  }
  const size_t output_base = (((size_t)batch * q_len + q_pos) * p.query_heads + head) * p.head_dim;
#pragma unroll
  for (int f = 0; f < kMaxFragments; ++f) {
    const uint32_t d = lane + f * 32;
    if (f < fragments && d < p.head_dim)
      output[output_base + d] = __float2half_rn(denominator == 0.0f ? 0.0f : results[f] / denominator);
  }
}

}  // namespace

int launch_paged_attention_split(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride,
                                 uint32_t pool_tokens);
bool paged_split_supported(const PagedParams& p);
uint32_t* context_device_error(Context* ctx);

// Whether this attention dispatch can also do the rotary embedding and the cache pack of its own new
// token (`fusion`, built from the two records before it): it must take the split path, read exactly what
// those two records write, and rotate whole heads of its own geometry out of place.
bool paged_attention_takes_rotary_pack(const KernelArgs& args, const RotaryPackFusion& fusion) {
  if (args.buffer_count != 7 || (args.param_bytes != 64 && args.param_bytes != 72)) return false;
  PagedParams p;
  memcpy(&p, args.params, 64);
  const uint32_t q_len = p.query_length == 0 ? 1 : p.query_length;
  if (p.mask_batches != 0 || q_len != 1 || p.window != 0 || p.batches == 0 || p.kv_heads == 0 ||
      p.query_heads % p.kv_heads != 0 || p.head_dim == 0 || p.group_size == 0 || p.head_dim % p.group_size != 0 ||
      !paged_split_supported(p))
    return false;
  // Every split CTA repeats the rotation of its query rows: that pays while the launch it saves is a
  // visible share of the step (Llama-8B shape: batch 1 2.122 -> 2.102 ms, batch 8 3.124 -> 3.104), not at
  // large batches (batch 32: 7.43 -> 7.57 ms).
  if (p.batches > 8) return false;
  const RotaryQkParams& r = fusion.rotary;
  const AttentionCachePairParams& c = fusion.cache;
  if (r.batches != p.batches || r.q_heads != p.query_heads || r.k_heads != p.kv_heads || r.width != p.head_dim ||
      r.half_dimension * 2 != r.width)
    return false;
  if (args.buffers[0] != (void*)fusion.q_output || args.buffers[1] != (void*)fusion.k_output ||
      args.buffers[2] != (void*)fusion.v_input || args.buffers[3] != (void*)fusion.pool)
    return false;
  if (c.token_stride != p.token_stride || c.token_elements != p.token_elements || c.key_segment_offset != p.key_offset ||
      c.value_segment_offset != p.value_offset)
    return false;
  // the kernel reads the raw query rows and the trigonometric rows as 32-bit words
  if ((((uintptr_t)fusion.q_input | (uintptr_t)fusion.cosine | (uintptr_t)fusion.sine) & 3u) != 0) return false;
  // rotated rows are written while other CTAs still read the raw ones: the two must not overlap
  const size_t q_bytes = (size_t)r.batches * r.q_heads * r.width * 2, k_bytes = (size_t)r.batches * r.k_heads * r.width * 2;
  auto overlap = [](const void* a, const void* b, size_t bytes) {
    const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
    return x < y + bytes && y < x + bytes;
  };
  return !overlap(fusion.q_input, fusion.q_output, q_bytes) && !overlap(fusion.k_input, fusion.k_output, k_bytes) &&
         !overlap(fusion.k_input, fusion.q_output, q_bytes > k_bytes ? q_bytes : k_bytes) &&
         !overlap(fusion.q_input, fusion.k_output, q_bytes > k_bytes ? q_bytes : k_bytes);
}

// Buffers: [query, current_key, current_value, pool, slots, mask, output]
// (lib/metal_dispatch_attention.ml:154-157); with no mask the dispatcher binds the
// slots buffer again in the mask position and sets mask_batches = 0.
// A 72-byte block carries two extra words after the 64 standard bytes:
// slot_batch_stride (per-sequence slot tables) and a reserved word.
int launch_attention_q8_paged(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 7, "expects buffers [query, key, value, pool, slots, mask, output]");
  LLMOPT_REQUIRE(args.param_bytes == 64 || args.param_bytes == 72, "expects 64 (or 72) parameter bytes");
  PagedParams p;
  memcpy(&p, args.params, 64);
  uint32_t slot_batch_stride = 0;
  if (args.param_bytes == 72) slot_batch_stride = param_u32(args, 16);
  LLMOPT_REQUIRE(p.batches > 0 && p.query_heads > 0 && p.kv_heads > 0, "empty attention problem");
  LLMOPT_REQUIRE(p.query_heads % p.kv_heads == 0, "query_heads must be a multiple of kv_heads");
  LLMOPT_REQUIRE(p.head_dim > 0 && p.head_dim <= 512, "head_dim must be in 1..512");
  LLMOPT_REQUIRE(p.group_size > 0 && p.head_dim % p.group_size == 0, "head_dim must be a multiple of group_size");
  const uint32_t q_len = p.query_length == 0 ? 1 : p.query_length;
  const size_t rows = (size_t)p.batches * p.query_heads * q_len;
  LLMOPT_REQUIRE(args.lengths[0] >= rows * p.head_dim * 2, "query buffer is too short");
  LLMOPT_REQUIRE(args.lengths[6] >= rows * p.head_dim * 2, "output buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.batches * p.kv_heads * q_len * p.head_dim * 2 &&
                     args.lengths[2] >= (size_t)p.batches * p.kv_heads * q_len * p.head_dim * 2,
                 "current key / value buffer is too short");
  // With a replayed plan the live past length sits in a device cell; the plan refuses
  // past lengths beyond the slot tables it captured (plan_token_capacity in runtime.cu).
  if (!args.past_tokens_cell)
    LLMOPT_REQUIRE(args.lengths[4] >= ((size_t)(p.batches - 1) * slot_batch_stride + p.past_length) * 4,
                   "slots buffer is shorter than past_length");
  // Pool geometry: every byte a kernel addresses inside a token row lies in it, and only whole
  // rows of the pool buffer are addressable (slots beyond them are refused on the device).
  const uint32_t groups_per_head = p.head_dim / p.group_size;
  const size_t segment = (size_t)p.kv_heads * p.head_dim;
  LLMOPT_REQUIRE(p.token_stride > 0, "token_stride must be positive");
  LLMOPT_REQUIRE(p.key_offset + segment <= p.token_elements && p.value_offset + segment <= p.token_elements,
                 "key / value segment lies outside token_elements");
  LLMOPT_REQUIRE((size_t)p.token_elements + 2 * ((size_t)max(p.key_offset, p.value_offset) / p.group_size +
                                                 (size_t)p.kv_heads * groups_per_head) <= p.token_stride,
                 "token_elements plus the group scales exceed token_stride");
  const size_t pool_rows = args.lengths[3] / p.token_stride;
  const uint32_t pool_tokens = pool_rows > 0xffffffffull ? 0xffffffffu : (uint32_t)pool_rows;
  const uint8_t* mask = p.mask_batches == 0 ? nullptr : (const uint8_t*)args.buffers[5];
  if (mask != nullptr) {
    const size_t mask_rows = (size_t)p.mask_batches * p.mask_heads * q_len;
    LLMOPT_REQUIRE(args.past_tokens_cell != nullptr ||
                       args.lengths[5] >= mask_rows * ((size_t)p.past_length + q_len) * (p.mask_dtype == 2 ? 2 : 1),
                   "mask buffer is too short");
  }
  if (mask == nullptr && q_len == 1 && p.window == 0 && paged_split_supported(p))
    return launch_paged_attention_split(args, p, slot_batch_stride, pool_tokens);
  const uint32_t blocks = (uint32_t)((rows + 7) / 8);
  launch_kernel(args, paged_rows_kernel, dim3(blocks), dim3(256), 0,
      (const __half*)args.buffers[0], (const __half*)args.buffers[1], (const __half*)args.buffers[2],
      (const uint8_t*)args.buffers[3], (const uint32_t*)args.buffers[4], mask, (__half*)args.buffers[6], p,
      slot_batch_stride, args.past_tokens_cell, pool_tokens, args.ctx ? context_device_error(args.ctx) : nullptr);
  return check_launch(args);
}

}  // namespace llmopt
