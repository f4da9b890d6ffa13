// Grouped-Q8 codec pieces shared by the cache kernels and the attention kernel that absorbs the
// rotary + pack of the new token: the pool bound, the group quantiser and one head row of the fused
// rotary embedding + cache pack (llmopt_rotary_qk_f16_simd_h64, lib/metal_normalization_source.ml:765-802,
// followed by llmopt_cache_pack_attention_q8_pair_simd, lib/metal_cache_source.ml:124-182).
#pragma once
#include "common.cuh"

namespace llmopt {

// Token rows the pool buffer holds; slot values at or beyond it are refused on the device
// (the access is skipped and the context's error word raised).
struct PoolBound {
  uint32_t tokens;
  uint32_t* error_word;
};
__device__ __forceinline__ bool slot_in_pool(uint32_t slot, const PoolBound& bound, uint32_t lane) {
  if (slot < bound.tokens) return true;
  if (lane == 0 && bound.error_word) atomicExch(bound.error_word, 1u);
  return false;
}

struct AttentionCachePairParams {  // lib/metal_cache_source.ml:22-34
  uint32_t items, key_segment_offset, value_segment_offset, heads, head_dim, group_size,
      token_elements, token_groups, token_stride, source_items, source_offset;
};
struct RotaryQkParams {  // lib/metal_normalization_source.ml:760-763
  uint32_t batches, tokens, q_heads, k_heads, width, half_dimension, trig_batches;
};

// One warp quantises one group: scale = half(max == 0 ? 1 : max / 127) (fp32 division), q =
// clamp(rint(x / float(scale)), -127, 127) with IEEE division and round-half-even.
__device__ __forceinline__ void quantize_group(const __half* __restrict__ source, uint32_t group_size,
                                               int8_t* __restrict__ values, __half* __restrict__ scale_out,
                                               uint32_t lane) {
  float maximum = 0.0f;
  for (uint32_t index = lane; index < group_size; index += 32)
    maximum = fmaxf(maximum, fabsf(__half2float(source[index])));
  maximum = warp_max(maximum);
  const __half stored = __float2half_rn(maximum == 0.0f ? 1.0f : __fdiv_rn(maximum, 127.0f));
  const float scale = __half2float(stored);
  for (uint32_t index = lane; index < group_size; index += 32) {
    int quantized = (int)rintf(__fdiv_rn(__half2float(source[index]), scale));
    quantized = max(-127, min(127, quantized));
    values[index] = (int8_t)quantized;
  }
  if (lane == 0) *scale_out = stored;
}

// Everything the fused rotary + pack of one decode token per sequence needs.
struct RotaryPackFusion {
  const __half* q_input;
  const __half* k_input;
  const __half* v_input;
  const __half* cosine;
  const __half* sine;
  __half* q_output;
  __half* k_output;
  const uint32_t* slots;  // the new token's slot, one per sequence
  uint8_t* pool;
  RotaryQkParams rotary;
  AttentionCachePairParams cache;
  PoolBound bound;
};

// The rotary embedding in half precision, operation for operation what the reference kernel does
// (separately rounded products, then one rounded sum).
__device__ __forceinline__ __half rotary_element(const __half* input, const __half* cosine, const __half* sine,
                                                 uint32_t col, uint32_t half_dimension) {
  const uint32_t rotated_col = col < half_dimension ? col + half_dimension : col - half_dimension;
  __half rotated = input[rotated_col];
  if (col < half_dimension) rotated = __hneg(rotated);
  const __half direct = __hmul_rn(input[col], cosine[col]);
  const __half turned = __hmul_rn(rotated, sine[col]);
  return __hadd_rn(direct, turned);
}

// One head row by one warp.  kind 0: a query row (rotated into q_output); 1: a key row (rotated into
// k_output, then quantised into the new slot); 2: a value row (quantised into the new slot).  Every lane
// quantises the columns it rotated itself.
__device__ __forceinline__ void rotary_pack_row(const RotaryPackFusion& f, uint32_t kind, uint32_t batch, uint32_t head,
                                                uint32_t lane) {
  const RotaryQkParams& r = f.rotary;
  const AttentionCachePairParams& c = f.cache;
  const uint32_t heads = kind == 0 ? r.q_heads : r.k_heads;
  const size_t base = ((size_t)batch * heads + head) * r.width;  // one token: token-first and head-major rows coincide
  if (kind != 2) {
    const __half* input = (kind == 0 ? f.q_input : f.k_input) + base;
    __half* output = (kind == 0 ? f.q_output : f.k_output) + base;
    const size_t trig_base = (size_t)(r.trig_batches == 1 ? 0 : batch) * r.width;
    for (uint32_t col = lane; col < r.width; col += 32)
      output[col] = rotary_element(input, f.cosine + trig_base, f.sine + trig_base, col, r.half_dimension);
    if (kind == 0) return;
    __syncwarp();
  }
  const __half* source = kind == 2 ? f.v_input + base : f.k_output + base;
  if (!slot_in_pool(f.slots[batch], f.bound, lane)) return;
  const size_t slot_base = (size_t)f.slots[batch] * c.token_stride;
  int8_t* values = reinterpret_cast<int8_t*>(f.pool + slot_base);
  __half* scales = reinterpret_cast<__half*>(f.pool + slot_base + c.token_elements);
  const uint32_t segment = kind == 2 ? c.value_segment_offset : c.key_segment_offset;
  for (uint32_t group = 0; group < r.width / c.group_size; ++group) {
    const uint32_t local = head * r.width + group * c.group_size;
    quantize_group(source + group * c.group_size, c.group_size, values + segment + local,
                   scales + (segment + local) / c.group_size, lane);
  }
}

// Host: the fused form of a rotary record followed by the pair-pack record of the same token, or false
// when the two do not fit it.  rotary: [q_in, k_in, cosine, sine, q_out, k_out]; pack: [key, value, slots, pool].
bool make_rotary_pack_fusion(const KernelArgs& rotary, const KernelArgs& pack, RotaryPackFusion* fusion);

}  // namespace llmopt
