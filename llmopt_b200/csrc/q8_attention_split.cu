// Split-K flash-decode over the grouped-Q8 token pool (decode shape: one query
// token per sequence, no mask, head_dim 64 or 128).  Grid-level restatement of
// the reference's experimental in-threadgroup split-8 kernels
// (lib/metal_cache_source.ml:961-1247): same merge algebra
// (max, denominator, weighted accumulators), applied across CTAs.
//
// Data flow of one warp and one tile of 16 keys:
//   pool (int8, HBM) --16-byte loads, one key row per 4 or 8 lanes--> registers
//   registers --PRMT + half2 subtract: exact int8 -> fp16 integers--> shared
//   S^T[key, head]   = K[key, :] . Q^T       mma.sync m16n8k16, A = K tile (ldmatrix),
//                                            B = query heads of the KV group
//   scores scaled by the fp16 group scales in fp32, online softmax per head
//   O^T[dim, head]  += V^T[dim, key] . P^T    A = V tile (ldmatrix.trans),
//                                            B = P^T (movmatrix of the score tile,
//                                            V group scales folded into P)
// All query heads that share a KV head ride in the MMA n dimension, so K and V
// are read and converted once per KV head.  The bound is HBM: per key and KV
// head 2 D bytes of int8 plus 4 D / group bytes of scales.
//
// Each CTA (4 warps) owns one split of one (batch, kv head); warps take the
// tiles of the split round-robin and keep private (max, denominator, O^T);
// the CTA merges its warps in shared memory and writes one record to scratch;
// paged_merge_kernel merges the records of all splits and the current token.
#include "q8_attention.cuh"

namespace llmopt {
namespace {

constexpr int kTileKeys = 16;
constexpr int kWarps = 4;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Four int8 -> two half2 of exact integers: byte ^ 0x80 is the value + 128; placed
// under the exponent of 1024.0 it reads 1024 + 128 + value; subtract 1152.
__device__ __forceinline__ void int8x4_to_half2x2(uint32_t word, uint32_t& first, uint32_t& second) {
  const uint32_t biased = word ^ 0x80808080u;
  first = hsub2_u32(prmt(biased, 0x64646464u, 0x4140u), 0x64806480u);
  second = hsub2_u32(prmt(biased, 0x64646464u, 0x4342u), 0x64806480u);
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* shared_address) {
  const uint32_t address = (uint32_t)__cvta_generic_to_shared(shared_address);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* shared_address) {
  const uint32_t address = (uint32_t)__cvta_generic_to_shared(shared_address);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t value) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(value));
  return d;
}
__device__ __forceinline__ uint32_t pack_half2(float low, float high) {
  const __half2 pair = __floats2half2_rn(low, high);
  return *reinterpret_cast<const uint32_t*>(&pair);
}

template <int D, bool ALIGN16>
struct RawTile {
  // One warp-wide load instruction covers 32 * 16 bytes = 32 / (D / 16) key rows.
  static constexpr int kLanesPerKey = D / 16;
  static constexpr int kKeysPerLoad = 32 / kLanesPerKey;
  static constexpr int kLoads = kTileKeys / kKeysPerLoad;
  uint4 key[kLoads];
  uint4 value[kLoads];
};

template <bool ALIGN16>
__device__ __forceinline__ uint4 load_16_bytes(const uint8_t* address) {
  if (ALIGN16) return __ldg(reinterpret_cast<const uint4*>(address));
  const uint2 low = __ldg(reinterpret_cast<const uint2*>(address));
  const uint2 high = __ldg(reinterpret_cast<const uint2*>(address + 8));
  return make_uint4(low.x, low.y, high.x, high.y);
}

template <int D, int GROUP, bool ALIGN16>
__global__ void __launch_bounds__(kWarps * 32)
paged_split_kernel(const __half* __restrict__ query, const uint8_t* __restrict__ pool,
                   const uint32_t* __restrict__ slots, float* __restrict__ scratch, PagedParams p,
                   uint32_t slot_batch_stride, uint32_t splits, const uint32_t* __restrict__ past_cell) {
  using Raw = RawTile<D, ALIGN16>;
  constexpr int kStride = D + 8;          // halves per shared row; 16 bytes of padding
  constexpr int kSteps = D / 16;          // k-steps of QK^T, m-tiles of PV
  __shared__ __align__(16) __half tiles[kWarps][2][kTileKeys][kStride];

  const uint32_t past = past_cell ? *past_cell : p.past_length;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t r = lane >> 2, c = lane & 3u;
  const uint32_t split = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const uint32_t heads_per_kv = p.query_heads / p.kv_heads;
  constexpr int groups_per_head = D / GROUP;  // 1, 2 or 4
  constexpr int steps_per_group = GROUP / 16;

  uint32_t chunk = (past + splits - 1u) / splits;
  chunk = (chunk + kTileKeys - 1u) / kTileKeys * kTileKeys;
  const uint32_t range_begin = min(split * chunk, past);
  const uint32_t range_end = min(range_begin + chunk, past);
  const uint32_t tile_count = (range_end - range_begin + kTileKeys - 1u) / kTileKeys;

  const uint32_t* batch_slots = slots + (size_t)batch * slot_batch_stride;
  const uint32_t scale_index_key = p.key_offset / GROUP + kv_head * groups_per_head;
  const uint32_t scale_index_value = p.value_offset / GROUP + kv_head * groups_per_head;
  const uint32_t key_byte = p.key_offset + kv_head * D + (lane % Raw::kLanesPerKey) * 16;
  const uint32_t value_byte = p.value_offset + kv_head * D + (lane % Raw::kLanesPerKey) * 16;

  // Query fragments: B operand, n = head r of this KV group, k = dims 16 s + 2c (+8).
  uint32_t q_frag[kSteps][2];
  {
    const uint32_t head = kv_head * heads_per_kv + r;
    const __half* source = query + ((size_t)batch * p.query_heads + head) * D;  // q_len == 1
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      q_frag[s][0] = 0u;
      q_frag[s][1] = 0u;
      if (r < heads_per_kv) {
        q_frag[s][0] = *reinterpret_cast<const uint32_t*>(source + 16 * s + 2 * c);
        q_frag[s][1] = *reinterpret_cast<const uint32_t*>(source + 16 * s + 2 * c + 8);
      }
    }
  }

  float running_max[2] = {-INFINITY, -INFINITY};
  float running_sum[2] = {0.0f, 0.0f};  // lane-local part of the denominator
  float out[kSteps][4];
#pragma unroll
  for (int s = 0; s < kSteps; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) out[s][j] = 0.0f;

  // Slot of key (lane % 16) of a tile, or the invalid marker.
  auto load_slot = [&](uint32_t tile) -> uint32_t {
    const uint32_t position = range_begin + tile * kTileKeys + (lane & 15u);
    return (tile < tile_count && position < range_end) ? __ldg(batch_slots + position) : 0xffffffffu;
  };
  // Raw int8 rows + group scales of one tile.  Lanes 0..15 also fetch the scales
  // of key `lane`: [K scales..., V scales...] as floats.
  auto load_raw = [&](uint32_t tile_slot, Raw& raw, float (&scales)[8]) {
#pragma unroll
    for (int i = 0; i < Raw::kLoads; ++i) {
      const uint32_t key_in_tile = i * Raw::kKeysPerLoad + lane / Raw::kLanesPerKey;
      const uint32_t slot = __shfl_sync(0xffffffffu, tile_slot, key_in_tile);
      raw.key[i] = make_uint4(0u, 0u, 0u, 0u);  // absent keys read as zeros
      raw.value[i] = raw.key[i];
      if (slot != 0xffffffffu) {
        const uint8_t* row = pool + (size_t)slot * p.token_stride;
        raw.key[i] = load_16_bytes<ALIGN16>(row + key_byte);
        raw.value[i] = load_16_bytes<ALIGN16>(row + value_byte);
      }
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) scales[g] = 0.0f;
    if (lane < 16 && tile_slot != 0xffffffffu) {
      const __half* scale_row =
          reinterpret_cast<const __half*>(pool + (size_t)tile_slot * p.token_stride + p.token_elements);
#pragma unroll
      for (int g = 0; g < groups_per_head; ++g) {
        scales[g] = __half2float(__ldg(scale_row + scale_index_key + g));
        scales[4 + g] = __half2float(__ldg(scale_row + scale_index_value + g));
      }
    }
  };

  Raw raw;
  float raw_scales[8];
  uint32_t slot_now = load_slot(warp);
  uint32_t slot_next = load_slot(warp + kWarps);
  load_raw(slot_now, raw, raw_scales);

  for (uint32_t tile = warp; tile < tile_count; tile += kWarps) {
    __half(*key_tile)[kStride] = tiles[warp][0];
    __half(*value_tile)[kStride] = tiles[warp][1];
    // registers -> shared as exact fp16 integers
    __syncwarp();
#pragma unroll
    for (int i = 0; i < Raw::kLoads; ++i) {
      const uint32_t key_in_tile = i * Raw::kKeysPerLoad + lane / Raw::kLanesPerKey;
      const uint32_t dim = (lane % Raw::kLanesPerKey) * 16;
      uint4 low, high;
      int8x4_to_half2x2(raw.key[i].x, low.x, low.y);
      int8x4_to_half2x2(raw.key[i].y, low.z, low.w);
      int8x4_to_half2x2(raw.key[i].z, high.x, high.y);
      int8x4_to_half2x2(raw.key[i].w, high.z, high.w);
      *reinterpret_cast<uint4*>(&key_tile[key_in_tile][dim]) = low;
      *reinterpret_cast<uint4*>(&key_tile[key_in_tile][dim + 8]) = high;
      int8x4_to_half2x2(raw.value[i].x, low.x, low.y);
      int8x4_to_half2x2(raw.value[i].y, low.z, low.w);
      int8x4_to_half2x2(raw.value[i].z, high.x, high.y);
      int8x4_to_half2x2(raw.value[i].w, high.z, high.w);
      *reinterpret_cast<uint4*>(&value_tile[key_in_tile][dim]) = low;
      *reinterpret_cast<uint4*>(&value_tile[key_in_tile][dim + 8]) = high;
    }
    float scales[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) scales[g] = raw_scales[g];
    const bool valid_low = __shfl_sync(0xffffffffu, slot_now, r) != 0xffffffffu;
    const bool valid_high = __shfl_sync(0xffffffffu, slot_now, r + 8) != 0xffffffffu;
    // prefetch the next tile of this warp while this one is consumed
    slot_now = slot_next;
    slot_next = load_slot(tile + 2 * kWarps);
    load_raw(slot_now, raw, raw_scales);
    __syncwarp();

    // S^T[key, head]: rows r / r+8 are keys, columns 2c / 2c+1 are heads.
    float score[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int g = 0; g < groups_per_head; ++g) {
      float partial[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int s = g * steps_per_group; s < (g + 1) * steps_per_group; ++s) {
        uint32_t a[4];
        // matrices: (keys 0-7, dims +0), (keys 8-15, dims +0), (keys 0-7, dims +8), (keys 8-15, dims +8)
        ldmatrix_x4(a, &key_tile[(lane & 7u) + ((lane >> 3) & 1u) * 8u][16 * s + (lane >> 4) * 8u]);
        mma_16816(partial, a, q_frag[s][0], q_frag[s][1]);
      }
      const float scale_low = __shfl_sync(0xffffffffu, scales[g], r);
      const float scale_high = __shfl_sync(0xffffffffu, scales[g], r + 8);
      score[0] = fmaf(partial[0], scale_low, score[0]);
      score[1] = fmaf(partial[1], scale_low, score[1]);
      score[2] = fmaf(partial[2], scale_high, score[2]);
      score[3] = fmaf(partial[3], scale_high, score[3]);
    }
    score[0] = valid_low ? score[0] * p.scale : -INFINITY;
    score[1] = valid_low ? score[1] * p.scale : -INFINITY;
    score[2] = valid_high ? score[2] * p.scale : -INFINITY;
    score[3] = valid_high ? score[3] * p.scale : -INFINITY;

    // online softmax per head (columns 2c, 2c+1); the maximum is shared by the
    // eight lanes that hold the same c
    float probability[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float tile_max = fmaxf(score[h], score[h + 2]);
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
      const float next_max = fmaxf(running_max[h], tile_max);
      const float rescale = next_max == -INFINITY ? 1.0f : expf(running_max[h] - next_max);
      probability[h] = next_max == -INFINITY ? 0.0f : expf(score[h] - next_max);
      probability[h + 2] = next_max == -INFINITY ? 0.0f : expf(score[h + 2] - next_max);
      running_sum[h] = running_sum[h] * rescale + probability[h] + probability[h + 2];
      running_max[h] = next_max;
#pragma unroll
      for (int s = 0; s < kSteps; ++s) {
        out[s][h] *= rescale;
        out[s][h + 2] *= rescale;
      }
    }

    // O^T[dim, head] += V^T[dim, key] P^T[key, head], V group scales folded into P
#pragma unroll
    for (int g = 0; g < groups_per_head; ++g) {
      const float scale_low = __shfl_sync(0xffffffffu, scales[4 + g], r);
      const float scale_high = __shfl_sync(0xffffffffu, scales[4 + g], r + 8);
      const uint32_t p_low = movmatrix_trans(pack_half2(probability[0] * scale_low, probability[1] * scale_low));
      const uint32_t p_high = movmatrix_trans(pack_half2(probability[2] * scale_high, probability[3] * scale_high));
#pragma unroll
      for (int s = g * steps_per_group; s < (g + 1) * steps_per_group; ++s) {
        uint32_t a[4];
        // matrices: (keys 0-7, dims +0), (keys 0-7, dims +8), (keys 8-15, dims +0), (keys 8-15, dims +8)
        ldmatrix_x4_trans(a, &value_tile[(lane & 7u) + (lane >> 4) * 8u][16 * s + ((lane >> 3) & 1u) * 8u]);
        mma_16816(out[s], a, p_low, p_high);
      }
    }
  }

  // ---- merge the four warps, write the split record ---------------------------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 4);
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 8);
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 16);
  }
  __syncthreads();
  float* stage = reinterpret_cast<float*>(&tiles[0][0][0][0]);  // [warp][16 + 8 * D]
  constexpr int kRecord = 16 + 8 * D;
  static_assert(sizeof(tiles) >= sizeof(float) * kWarps * kRecord, "merge staging must fit the tile buffers");
  float* mine = stage + warp * kRecord;
  if (r == 0) {
    mine[2 * c] = running_max[0];
    mine[2 * c + 1] = running_max[1];
    mine[8 + 2 * c] = running_sum[0];
    mine[8 + 2 * c + 1] = running_sum[1];
  }
#pragma unroll
  for (int s = 0; s < kSteps; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t dim = 16 * s + r + ((j & 2) ? 8 : 0);
      const uint32_t head = 2 * c + (j & 1);
      mine[16 + head * D + dim] = out[s][j];
    }
  __syncthreads();
  float* record = scratch + (((size_t)batch * p.kv_heads + kv_head) * splits + split) * kRecord;
  for (uint32_t index = threadIdx.x; index < 8u * D; index += kWarps * 32) {
    const uint32_t head = index / D;
    float merged_max = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) merged_max = fmaxf(merged_max, stage[w * kRecord + head]);
    float total = 0.0f, denominator = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float warp_max_value = stage[w * kRecord + head];
      const float weight = warp_max_value == -INFINITY ? 0.0f : expf(warp_max_value - merged_max);
      total += weight * stage[w * kRecord + 16 + index];
      denominator += weight * stage[w * kRecord + 8 + head];
    }
    record[16 + index] = total;
    if (index % D == 0) {
      record[head] = merged_max;
      record[8 + head] = denominator;
    }
  }
}

// One CTA per (batch, query head): merges the split records and the current
// token (key position past_length, fp16, lib/metal_cache_source.ml:446-470),
// writes half(result / denominator) token-first.
template <int D>
__global__ void __launch_bounds__(D)
paged_merge_kernel(const __half* __restrict__ query, const __half* __restrict__ current_key,
                   const __half* __restrict__ current_value, const float* __restrict__ scratch,
                   __half* __restrict__ output, PagedParams p, uint32_t splits) {
  constexpr int kRecord = 16 + 8 * D;
  __shared__ float partial[D / 32];
  const uint32_t head = blockIdx.x, batch = blockIdx.y, d = threadIdx.x;
  const uint32_t heads_per_kv = p.query_heads / p.kv_heads;
  const uint32_t kv_head = head / heads_per_kv, local_head = head % heads_per_kv;
  const size_t query_base = ((size_t)batch * p.query_heads + head) * D;
  const size_t current_base = ((size_t)batch * p.kv_heads + kv_head) * D;
  float dot = __half2float(query[query_base + d]) * __half2float(current_key[current_base + d]);
  dot = warp_sum(dot);
  if ((d & 31u) == 0) partial[d >> 5] = dot;
  __syncthreads();
  float current_score = 0.0f;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) current_score += partial[i];
  current_score *= p.scale;

  const float* records = scratch + ((size_t)batch * p.kv_heads + kv_head) * splits * kRecord;
  float maximum = current_score;
  for (uint32_t s = 0; s < splits; ++s) maximum = fmaxf(maximum, records[s * kRecord + local_head]);
  const float current_weight = expf(current_score - maximum);
  float denominator = current_weight;
  float result = current_weight * __half2float(current_value[current_base + d]);
  for (uint32_t s = 0; s < splits; ++s) {
    const float split_max = records[s * kRecord + local_head];
    if (split_max == -INFINITY) continue;
    const float weight = expf(split_max - maximum);
    denominator += weight * records[s * kRecord + 8 + local_head];
    result += weight * records[s * kRecord + 16 + local_head * D + d];
  }
  const size_t output_base = ((size_t)batch * p.query_heads + head) * D;  // [b, q = 1, hq, D]
  output[output_base + d] = __float2half_rn(denominator == 0.0f ? 0.0f : result / denominator);
}

template <int D, int GROUP>
int launch_split(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride, float* scratch,
                 uint32_t splits) {
  const bool aligned = (p.token_stride % 16 == 0) && (((uintptr_t)args.buffers[3]) % 16 == 0);
  const dim3 grid(splits, p.kv_heads, p.batches);
  if (aligned)
    paged_split_kernel<D, GROUP, true><<<grid, kWarps * 32, 0, args.stream>>>(
        (const __half*)args.buffers[0], (const uint8_t*)args.buffers[3], (const uint32_t*)args.buffers[4], scratch,
        p, slot_batch_stride, splits, args.past_tokens_cell);
  else
    paged_split_kernel<D, GROUP, false><<<grid, kWarps * 32, 0, args.stream>>>(
        (const __half*)args.buffers[0], (const uint8_t*)args.buffers[3], (const uint32_t*)args.buffers[4], scratch,
        p, slot_batch_stride, splits, args.past_tokens_cell);
  if (int status = check_launch(args)) return status;
  paged_merge_kernel<D><<<dim3(p.query_heads, p.batches), D, 0, args.stream>>>(
      (const __half*)args.buffers[0], (const __half*)args.buffers[1], (const __half*)args.buffers[2], scratch,
      (__half*)args.buffers[6], p, splits);
  return check_launch(args);
}

}  // namespace

bool paged_split_supported(const PagedParams& p) {
  const uint32_t heads_per_kv = p.query_heads / p.kv_heads;
  return (p.head_dim == 64 || p.head_dim == 128) && (p.group_size == 32 || p.group_size == 64) &&
         heads_per_kv <= 8 && p.token_stride % 8 == 0 && p.key_offset % 16 == 0 && p.value_offset % 16 == 0 &&
         p.token_elements % 2 == 0;
}

uint32_t paged_pick_splits(const KernelArgs& args, const PagedParams& p) {
  // Enough CTAs for about three per SM; a split is never shorter than 64 keys
  // at capture time (a replayed plan keeps the count while the context grows).
  const uint32_t pairs = p.batches * p.kv_heads;
  const uint32_t target = (uint32_t)context_sm_count(args.ctx) * 3u;
  uint32_t splits = (target + pairs - 1u) / pairs;
  const uint32_t by_length = args.past_tokens_cell ? kMaxAttentionSplits : (p.past_length + 63u) / 64u;
  if (splits > by_length) splits = by_length;
  if (splits > kMaxAttentionSplits) splits = kMaxAttentionSplits;
  return splits == 0 ? 1 : splits;
}

int launch_paged_attention_split_on(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride,
                                    float* scratch, uint32_t splits) {
  LLMOPT_REQUIRE(((uintptr_t)args.buffers[3]) % 8 == 0, "pool must be 8-byte aligned");
  LLMOPT_REQUIRE(((uintptr_t)args.buffers[0]) % 4 == 0, "query must be 4-byte aligned");
  if (p.head_dim == 64)
    return p.group_size == 64 ? launch_split<64, 64>(args, p, slot_batch_stride, scratch, splits)
                              : launch_split<64, 32>(args, p, slot_batch_stride, scratch, splits);
  return p.group_size == 64 ? launch_split<128, 64>(args, p, slot_batch_stride, scratch, splits)
                            : launch_split<128, 32>(args, p, slot_batch_stride, scratch, splits);
}

int launch_paged_attention_split(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride) {
  const uint32_t splits = paged_pick_splits(args, p);
  const size_t bytes =
      (size_t)p.batches * p.kv_heads * splits * paged_split_record_floats(p.head_dim) * sizeof(float);
  float* scratch = (float*)context_scratch(args.ctx, bytes, args.error);
  if (scratch == nullptr) return 1;
  return launch_paged_attention_split_on(args, p, slot_batch_stride, scratch, splits);
}

}  // namespace llmopt
