// Split-K flash-decode over the grouped-Q8 token pool (decode shape: one query
// token per sequence, no mask, head_dim 64 or 128).  Grid-level restatement of
// the reference's experimental in-threadgroup split-8 kernels
// (lib/metal_cache_source.ml:961-1247): same merge algebra
// (max, denominator, weighted accumulators), applied across CTAs.
//
// Data flow of one warp and one tile of 16 keys:
//   pool (int8, HBM) --cp.async, 16 bytes per lane--> the warp's ring of raw tiles in
//                                            shared memory (several tiles in flight)
//   raw int8 words --PRMT + half2 subtract: exact int8 -> fp16 integers--> MMA fragments
//                                            (no fp16 copy of the tile is ever stored)
//   S^T[key, head]   = K[key, :] . Q^T       mma.sync m16n8k16, A = K tile,
//                                            B = query heads of the KV group
//   scores scaled by the fp16 group scales in fp32, online softmax per head
//   O^T[dim, head]  += V^T[dim, key] . P^T    A = V tile (bytes of two keys interleaved
//                                            by PRMT), B = P^T (movmatrix of the score
//                                            tile, V group scales folded into P)
// The contraction index of an MMA may be permuted freely as long as both operands agree,
// and so may the row index of the PV product as long as the writeback agrees.  Both
// are chosen so that each lane reads whole 32-bit words of int8 and the reads of a
// warp fall into 32 different banks (rows are padded by 16 bytes):
//   QK^T, k-step s: lane (r, c) holds dims 16 s + 4 c .. + 3 of keys r and r + 8;
//   PV, word w = r + 8 j: dims 4 w .. 4 w + 3 of keys 2c, 2c+1, 2c+8, 2c+9 feed rows
//   r and r + 8 of the two m-tiles 2 j and 2 j + 1.
// All query heads that share a KV head ride in the MMA n dimension, so K and V
// are read and converted once per KV head.  The bound is HBM: per key and KV
// head 2 D bytes of int8 plus 4 D / group bytes of scales.
//
// Each CTA (4 warps) owns one split of one (batch, kv head); warps take the
// tiles of the split round-robin and keep private (max, denominator, O^T);
// the CTA merges its warps in shared memory and writes one record to scratch;
// paged_merge_kernel merges the records of all splits and the current token.
#include <cstdlib>
#include "q8_attention.cuh"
#include "q8_codec.cuh"

namespace llmopt {
uint32_t* context_device_error(Context* ctx);
namespace {

constexpr int kTileKeys = 16;
constexpr int kWarps = 4;
constexpr int kResidentCtas = 4;  // per SM, by shared memory and registers (128 per thread)
constexpr uint32_t kNoSlot = 0xffffffffu;
constexpr float kLowest = -1.0e30f;  // "no key yet" maximum; keeps the softmax free of inf - inf

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
// Four bytes already XORed with 0x80 (value + 128) -> two half2 of exact integers:
// a byte placed under the exponent of 1024.0 reads 1024 + 128 + value; subtract 1152.
__device__ __forceinline__ void biased_bytes_to_half2x2(uint32_t biased, uint32_t& first, uint32_t& second) {
  first = hsub2_u32(prmt(biased, 0x64646464u, 0x4140u), 0x64806480u);
  second = hsub2_u32(prmt(biased, 0x64646464u, 0x4342u), 0x64806480u);
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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
__device__ __forceinline__ uint32_t lds32(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(address));
  return v;
}
__device__ __forceinline__ float exp2_fast(float x) {  // 2^x; -inf and very negative x give 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Asynchronous copy of CP bytes; source_bytes == 0 writes zeros and reads nothing.
template <int CP>
__device__ __forceinline__ void copy_async(uint32_t shared_address, const void* source, uint32_t source_bytes) {
  if (CP == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(shared_address), "l"(source),
                 "r"(source_bytes)
                 : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(shared_address), "l"(source),
                 "r"(source_bytes)
                 : "memory");
}
// Small asynchronous copy (4 or 8 bytes) for the group scales.
template <int BYTES>
__device__ __forceinline__ void copy_async_small(uint32_t shared_address, const void* source, uint32_t source_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(shared_address), "l"(source), "n"(BYTES),
               "r"(source_bytes)
               : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// Shared-memory shape of one warp's ring.  CP is the copy size: 16 bytes, or 8 for
// pools whose rows are only 8-byte aligned.
template <int D, int CP>
struct SplitShape {
  static constexpr int kRowBytes = D + 16;  // the padding spreads the fragment reads over all banks
  static constexpr int kTileBytes = kTileKeys * kRowBytes;
  static constexpr int kScaleBytes = 2 * kTileKeys * 8;  // [K | V][key][up to 4 halves]
  static constexpr int kStageBytes = 2 * kTileBytes + kScaleBytes;
  // Sixteen warps per SM hide the latencies of the conversion and MMA chain better than
  // a deeper ring under fewer warps does (measured: 2 stages x 4 CTAs beats 3 x 3 and 5 x 2).
  static constexpr int kStages = D == 128 ? 2 : 4;
  static constexpr int kLanesPerKey = D / CP;
  static constexpr int kKeysPerPass = 32 / kLanesPerKey;
  static constexpr int kPasses = kTileKeys / kKeysPerPass;
  static constexpr int kRingBytes = kWarps * kStages * kStageBytes;
};

// FUSED: the launch also does the rotary embedding and the cache pack of the new token (`fusion`), which
// otherwise are a kernel of their own right before this one.  Every CTA rotates the query rows of its KV
// group in registers on the way into the MMA fragments (same rounding sequence as rotary_element); the
// writes of the rotated query / key rows (the merge kernel reads them) and the Q8 pack of the new key and
// value rows are warp tasks handed out over the CTAs of a (batch, KV head), done while the first tiles are
// in flight.
template <int D, int GROUP, int CP, bool FUSED = false>
__global__ void __launch_bounds__(kWarps * 32, kResidentCtas)
paged_split_kernel(const __half* __restrict__ query, const uint8_t* __restrict__ pool,
                   const uint32_t* __restrict__ slots, float* __restrict__ scratch, PagedParams p,
                   uint32_t slot_batch_stride, uint32_t splits, const uint32_t* __restrict__ past_cell,
                   uint32_t pool_tokens, uint32_t* error_word, RotaryPackFusion fusion) {
  grid_chain_prologue();
  using Shape = SplitShape<D, CP>;
  constexpr int kSteps = D / 16;  // k-steps of QK^T, m-tiles of PV
  constexpr int kStages = Shape::kStages;
  constexpr int groups_per_head = D / GROUP;  // 1, 2 or 4
  constexpr int steps_per_group = GROUP / 16;
  extern __shared__ __align__(16) uint8_t ring[];

  const uint32_t past = past_cell ? *past_cell : p.past_length;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t r = lane >> 2, c = lane & 3u;
  const uint32_t split = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const uint32_t heads_per_kv = p.query_heads / p.kv_heads;

  uint32_t chunk = (past + splits - 1u) / splits;
  chunk = (chunk + kTileKeys - 1u) / kTileKeys * kTileKeys;
  const uint32_t range_begin = min(split * chunk, past);
  const uint32_t range_end = min(range_begin + chunk, past);
  const uint32_t tile_count = (range_end - range_begin + kTileKeys - 1u) / kTileKeys;
  // this warp's tiles: warp, warp + kWarps, ...
  const uint32_t my_tiles = tile_count > warp ? (tile_count - warp + kWarps - 1u) / kWarps : 0u;

  const uint32_t* batch_slots = slots + (size_t)batch * slot_batch_stride;
  const uint32_t copy_lane = lane % Shape::kLanesPerKey;
  const uint32_t key_byte = p.key_offset + kv_head * D + copy_lane * CP;
  const uint32_t value_byte = p.value_offset + kv_head * D + copy_lane * CP;
  // lanes 0..15 fetch the K scales of key `lane`, lanes 16..31 the V scales of key `lane - 16`
  // The scales of one head are 2, 4 or 8 bytes; they travel as one 4- or 8-byte copy (a single
  // half rides in the aligned word that holds it and is picked out by scale_pick).
  constexpr int kScaleCopy = groups_per_head == 4 ? 8 : 4;
  const uint32_t scale_byte =
      p.token_elements + 2u * ((lane < 16 ? p.key_offset : p.value_offset) / GROUP + kv_head * groups_per_head);
  const uint32_t scale_pick_key = ((p.token_elements + 2u * (p.key_offset / GROUP + kv_head)) >> 1) & 1u;
  const uint32_t scale_pick_value = ((p.token_elements + 2u * (p.value_offset / GROUP + kv_head)) >> 1) & 1u;
  const uint8_t* const pool_scale = pool + (groups_per_head == 1 ? (scale_byte & ~3u) : scale_byte);
  const uint32_t ring_base = (uint32_t)__cvta_generic_to_shared(ring) + warp * kStages * Shape::kStageBytes;

  // Query fragments: B operand, n = head r of this KV group, k = dims 16 s + 4 c .. + 3.
  uint32_t q_frag[kSteps][2];
  if (!FUSED) {
    const uint32_t head = kv_head * heads_per_kv + r;
    const __half* source = query + ((size_t)batch * p.query_heads + head) * D;  // q_len == 1
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      q_frag[s][0] = 0u;
      q_frag[s][1] = 0u;
      if (r < heads_per_kv) {
        q_frag[s][0] = *reinterpret_cast<const uint32_t*>(source + 16 * s + 4 * c);
        q_frag[s][1] = *reinterpret_cast<const uint32_t*>(source + 16 * s + 4 * c + 2);
      }
    }
  }

  // Scores are kept in units of log2(e), so that every exponential is one ex2.
  const float score_scale = p.scale * 1.4426950408889634f;
  float running_max[2] = {kLowest, kLowest};
  float running_sum[2] = {0.0f, 0.0f};  // lane-local part of the denominator
  // out[2 j + e][i]: dim 4 (r + 8 j) + 2 e + (i >> 1), head 2 c + (i & 1)
  float out[kSteps][4];
#pragma unroll
  for (int s = 0; s < kSteps; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) out[s][j] = 0.0f;

  // Slot of key (lane % 16) of this warp's tile `index`, or kNoSlot.  A slot outside the pool
  // is reported through the error word and read as slot 0, so no copy leaves the pool.
  auto load_slot = [&](uint32_t index) -> uint32_t {
    const uint32_t position = range_begin + (warp + index * kWarps) * kTileKeys + (lane & 15u);
    if (!(index < my_tiles && position < range_end)) return kNoSlot;
    uint32_t slot = __ldg(batch_slots + position);
    if (slot >= pool_tokens) {
      if (error_word) atomicExch(error_word, 1u);
      slot = 0u;
    }
    return slot;
  };
  // A tile's row addresses depend on its slots, so the slots run four tiles ahead of
  // the copies.
  uint32_t slot_0 = load_slot(0), slot_1 = load_slot(1), slot_2 = load_slot(2), slot_3 = load_slot(3);
  const uint8_t* const pool_key = pool + key_byte;
  const uint8_t* const pool_value = pool + value_byte;
  const uint32_t copy_target = (lane / Shape::kLanesPerKey) * Shape::kRowBytes + copy_lane * CP;

  // Starts the copies of tile `index` into ring stage `stage` and rotates the slot registers.
  auto issue = [&](uint32_t index, uint32_t stage) {
    if (index < my_tiles) {
      const uint32_t stage_base = ring_base + stage * Shape::kStageBytes;
      const uint32_t target = stage_base + copy_target;
      const bool whole = range_begin + (warp + index * kWarps + 1u) * kTileKeys <= range_end;
      if (whole) {
#pragma unroll
        for (int i = 0; i < Shape::kPasses; ++i) {
          const uint32_t slot = __shfl_sync(0xffffffffu, slot_0, i * Shape::kKeysPerPass + lane / Shape::kLanesPerKey);
          const size_t row = (size_t)slot * p.token_stride;
          copy_async<CP>(target + i * Shape::kKeysPerPass * Shape::kRowBytes, pool_key + row, CP);
          copy_async<CP>(target + i * Shape::kKeysPerPass * Shape::kRowBytes + Shape::kTileBytes, pool_value + row, CP);
        }
      } else {
#pragma unroll
        for (int i = 0; i < Shape::kPasses; ++i) {
          const uint32_t slot = __shfl_sync(0xffffffffu, slot_0, i * Shape::kKeysPerPass + lane / Shape::kLanesPerKey);
          const bool present = slot != kNoSlot;  // absent keys read as zeros
          const size_t row = (size_t)(present ? slot : 0u) * p.token_stride;
          copy_async<CP>(target + i * Shape::kKeysPerPass * Shape::kRowBytes, pool_key + row, present ? CP : 0);
          copy_async<CP>(target + i * Shape::kKeysPerPass * Shape::kRowBytes + Shape::kTileBytes, pool_value + row,
                         present ? CP : 0);
        }
      }
      {
        const bool present = slot_0 != kNoSlot;
        copy_async_small<kScaleCopy>(stage_base + 2 * Shape::kTileBytes + lane * 8u,
                                     pool_scale + (size_t)(present ? slot_0 : 0u) * p.token_stride,
                                     present ? kScaleCopy : 0);
      }
    }
    copy_async_commit();
    slot_0 = slot_1;
    slot_1 = slot_2;
    slot_2 = slot_3;
    slot_3 = load_slot(index + 4u);
  };

  auto consume = [&](uint32_t index, uint32_t stage) {
    const uint32_t key_tile = ring_base + stage * Shape::kStageBytes;
    const uint32_t value_tile = key_tile + Shape::kTileBytes;
    const uint32_t scale_tile = value_tile + Shape::kTileBytes;
    const uint32_t first_position = range_begin + (warp + index * kWarps) * kTileKeys;
    const bool valid_low = first_position + r < range_end;
    const bool valid_high = first_position + r + 8u < range_end;
    // group scales of keys r and r + 8: halves [g] of K, then of V
    float key_scale_low[4], key_scale_high[4], value_scale_low[4], value_scale_high[4];
    auto read_scales = [&](uint32_t address, uint32_t pick, float (&scales)[4]) {
      if (groups_per_head == 4) {
        uint2 raw;
        asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "r"(address));
        const float2 first = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 second = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        scales[0] = first.x;
        scales[1] = first.y;
        scales[2] = second.x;
        scales[3] = second.y;
      } else {
        const uint32_t raw = lds32(address);
        const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&raw));
        scales[0] = groups_per_head == 1 && pick ? pair.y : pair.x;
        scales[1] = pair.y;
        scales[2] = scales[3] = 0.0f;
      }
    };
    read_scales(scale_tile + r * 8u, scale_pick_key, key_scale_low);
    read_scales(scale_tile + (r + 8u) * 8u, scale_pick_key, key_scale_high);
    read_scales(scale_tile + 128u + r * 8u, scale_pick_value, value_scale_low);
    read_scales(scale_tile + 128u + (r + 8u) * 8u, scale_pick_value, value_scale_high);

    // S^T[key, head]: rows r / r+8 are keys, columns 2c / 2c+1 are heads.
    float score[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int g = 0; g < groups_per_head; ++g) {
      float partial[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int s = g * steps_per_group; s < (g + 1) * steps_per_group; ++s) {
        const uint32_t word_low = lds32(key_tile + r * Shape::kRowBytes + 16 * s + 4 * c) ^ 0x80808080u;
        const uint32_t word_high = lds32(key_tile + (r + 8u) * Shape::kRowBytes + 16 * s + 4 * c) ^ 0x80808080u;
        uint32_t a[4];
        biased_bytes_to_half2x2(word_low, a[0], a[2]);
        biased_bytes_to_half2x2(word_high, a[1], a[3]);
        mma_16816(partial, a, q_frag[s][0], q_frag[s][1]);
      }
      score[0] = fmaf(partial[0], key_scale_low[g], score[0]);
      score[1] = fmaf(partial[1], key_scale_low[g], score[1]);
      score[2] = fmaf(partial[2], key_scale_high[g], score[2]);
      score[3] = fmaf(partial[3], key_scale_high[g], score[3]);
    }
    score[0] = valid_low ? score[0] * score_scale : -INFINITY;
    score[1] = valid_low ? score[1] * score_scale : -INFINITY;
    score[2] = valid_high ? score[2] * score_scale : -INFINITY;
    score[3] = valid_high ? score[3] * score_scale : -INFINITY;

    // online softmax per head (columns 2c, 2c+1); the maximum is shared by the
    // eight lanes that hold the same c
    float probability[4], rescale[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float tile_max = fmaxf(score[h], score[h + 2]);
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
      const float next_max = fmaxf(running_max[h], tile_max);  // finite: at least kLowest
      rescale[h] = exp2_fast(running_max[h] - next_max);
      probability[h] = exp2_fast(score[h] - next_max);
      probability[h + 2] = exp2_fast(score[h + 2] - next_max);
      running_sum[h] = running_sum[h] * rescale[h] + probability[h] + probability[h + 2];
      running_max[h] = next_max;
    }
    // the maxima settle after a few tiles; skip the rescaling sweep when no lane needs it
    if (__any_sync(0xffffffffu, rescale[0] != 1.0f || rescale[1] != 1.0f)) {
#pragma unroll
      for (int s = 0; s < kSteps; ++s) {
        out[s][0] *= rescale[0];
        out[s][1] *= rescale[1];
        out[s][2] *= rescale[0];
        out[s][3] *= rescale[1];
      }
    }

    // O^T[dim, head] += V^T[dim, key] P^T[key, head], V group scales folded into P
#pragma unroll
    for (int g = 0; g < groups_per_head; ++g) {
      const uint32_t p_low = movmatrix_trans(
          pack_half2(probability[0] * value_scale_low[g], probability[1] * value_scale_low[g]));
      const uint32_t p_high = movmatrix_trans(
          pack_half2(probability[2] * value_scale_high[g], probability[3] * value_scale_high[g]));
#pragma unroll
      for (int j = g * (GROUP / 32); j < (g + 1) * (GROUP / 32); ++j) {
        const uint32_t word = value_tile + (2u * c) * Shape::kRowBytes + 4u * (r + 8u * j);
        const uint32_t key_0 = lds32(word), key_1 = lds32(word + Shape::kRowBytes);
        const uint32_t key_8 = lds32(word + 8 * Shape::kRowBytes), key_9 = lds32(word + 9 * Shape::kRowBytes);
        // bytes (dim, key): [d0 k0, d0 k1, d1 k0, d1 k1] and [d2 k0, d2 k1, d3 k0, d3 k1]
        const uint32_t near_01 = prmt(key_0, key_1, 0x5140u) ^ 0x80808080u;
        const uint32_t near_23 = prmt(key_0, key_1, 0x7362u) ^ 0x80808080u;
        const uint32_t far_01 = prmt(key_8, key_9, 0x5140u) ^ 0x80808080u;
        const uint32_t far_23 = prmt(key_8, key_9, 0x7362u) ^ 0x80808080u;
        uint32_t a[4], b[4];
        biased_bytes_to_half2x2(near_01, a[0], a[1]);
        biased_bytes_to_half2x2(far_01, a[2], a[3]);
        biased_bytes_to_half2x2(near_23, b[0], b[1]);
        biased_bytes_to_half2x2(far_23, b[2], b[3]);
        mma_16816(out[2 * j], a, p_low, p_high);
        mma_16816(out[2 * j + 1], b, p_low, p_high);
      }
    }
  };

  // prologue: kStages - 1 tiles in flight
#pragma unroll 1
  for (uint32_t index = 0; index < (uint32_t)(kStages - 1); ++index) issue(index, index);
  uint32_t consume_stage = 0, issue_stage = kStages - 1;
  if (FUSED) {
    // this lane's query dims 16 s + 4 c + j pair with 16 (s + kSteps / 2) + 4 c + j: both halves of a
    // rotation sit in the same lane
    const uint32_t head = kv_head * heads_per_kv + r;
    const size_t row = ((size_t)batch * p.query_heads + head) * D;
    const size_t trig = (size_t)(fusion.rotary.trig_batches == 1 ? 0 : batch) * D;
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      q_frag[s][0] = 0u;
      q_frag[s][1] = 0u;
    }
    if (r < heads_per_kv) {
      const __half* raw = fusion.q_input + row;
      const __half* cosine = fusion.cosine + trig;
      const __half* sine = fusion.sine + trig;
      // the four halves at dims `first` .. + 3 as two 32-bit loads
      auto four = [](const __half* base, uint32_t first, __half (&out)[4]) {
        const uint32_t low = *reinterpret_cast<const uint32_t*>(base + first);
        const uint32_t high = *reinterpret_cast<const uint32_t*>(base + first + 2);
        out[0] = __ushort_as_half((unsigned short)(low & 0xffffu));
        out[1] = __ushort_as_half((unsigned short)(low >> 16));
        out[2] = __ushort_as_half((unsigned short)(high & 0xffffu));
        out[3] = __ushort_as_half((unsigned short)(high >> 16));
      };
      auto pack = [](const __half (&v)[4], uint32_t (&words)[2]) {
        words[0] = (uint32_t)__half_as_ushort(v[0]) | ((uint32_t)__half_as_ushort(v[1]) << 16);
        words[1] = (uint32_t)__half_as_ushort(v[2]) | ((uint32_t)__half_as_ushort(v[3]) << 16);
      };
#pragma unroll
      for (int s = 0; s < kSteps / 2; ++s) {
        const uint32_t low_dim = 16 * s + 4 * c, high_dim = low_dim + D / 2;
        __half x_low[4], x_high[4], cos_low[4], cos_high[4], sin_low[4], sin_high[4], out_low[4], out_high[4];
        four(raw, low_dim, x_low);
        four(raw, high_dim, x_high);
        four(cosine, low_dim, cos_low);
        four(cosine, high_dim, cos_high);
        four(sine, low_dim, sin_low);
        four(sine, high_dim, sin_high);
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // rotary_element for col < D / 2 and for col >= D / 2
          out_low[j] = __hadd_rn(__hmul_rn(x_low[j], cos_low[j]), __hmul_rn(__hneg(x_high[j]), sin_low[j]));
          out_high[j] = __hadd_rn(__hmul_rn(x_high[j], cos_high[j]), __hmul_rn(x_low[j], sin_high[j]));
        }
        pack(out_low, q_frag[s]);
        pack(out_high, q_frag[s + kSteps / 2]);
      }
    }
    // warp tasks of this (batch, KV head): its query rows, its key row, its value row
    const uint32_t tasks = heads_per_kv + 2u;
    for (uint32_t task = split + warp * splits; task < tasks; task += splits * kWarps) {
      if (task < heads_per_kv)
        rotary_pack_row(fusion, 0u, batch, kv_head * heads_per_kv + task, lane);
      else
        rotary_pack_row(fusion, task == heads_per_kv ? 1u : 2u, batch, kv_head, lane);
    }
  }
#pragma unroll 1
  for (uint32_t index = 0; index < my_tiles; ++index) {
    issue(index + kStages - 1, issue_stage);
    copy_async_wait<kStages - 1>();  // all but the newest kStages - 1 groups have landed: tile `index` is here
    __syncwarp();
    consume(index, consume_stage);
    __syncwarp();  // the next issue overwrites this stage
    issue_stage = consume_stage;
    consume_stage = consume_stage + 1 == kStages ? 0 : consume_stage + 1;
  }
  copy_async_wait<0>();

  // ---- merge the four warps, write the split record ---------------------------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 4);
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 8);
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 16);
  }
  __syncthreads();
  float* stage = reinterpret_cast<float*>(ring);  // [warp][16 + 8 * D]
  constexpr int kRecord = 16 + 8 * D;
  static_assert(Shape::kRingBytes >= (int)sizeof(float) * kWarps * kRecord, "merge staging must fit the ring");
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
      const uint32_t dim = 4u * (r + 8u * (s >> 1)) + 2u * (s & 1) + (j >> 1);
      const uint32_t head = 2 * c + (j & 1);
      mine[16 + head * D + dim] = out[s][j];
    }
  __syncthreads();
  float* record = scratch + (((size_t)batch * p.kv_heads + kv_head) * splits + split) * kRecord;
  // only the columns of heads that exist are merged and written (the merge kernel reads no others)
  for (uint32_t index = threadIdx.x; index < min(heads_per_kv, 8u) * D; index += kWarps * 32) {
    const uint32_t head = index / D;
    float merged_max = kLowest;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) merged_max = fmaxf(merged_max, stage[w * kRecord + head]);
    float total = 0.0f, denominator = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float weight = exp2_fast(stage[w * kRecord + head] - merged_max);
      total += weight * stage[w * kRecord + 16 + index];
      denominator += weight * stage[w * kRecord + 8 + head];
    }
    record[16 + index] = total;
    if (index % D == 0) {
      // records carry the maximum in natural units; a split without keys says -inf
      record[head] = merged_max <= 0.5f * kLowest ? -INFINITY : merged_max * 0.6931471805599453f;
      record[8 + head] = denominator;
    }
  }
}

// One CTA per (batch, query head): merges the split records and the current
// token (key position past_length, fp16, lib/metal_cache_source.ml:446-470),
// writes half(result / denominator) token-first.  Thread s first weighs split s
// (maxima and denominators are read side by side, not one after the other); then the
// kMergeParts thread groups each sum dimension d over a quarter of the splits with all of
// their loads in flight at once (the kernel is a chain of L2 latencies, not of bytes), and
// the quarters are added in order.
constexpr int kMergeParts = 4;
template <int D>
__global__ void __launch_bounds__(D * kMergeParts)
paged_merge_kernel(const __half* __restrict__ query, const __half* __restrict__ current_key,
                   const __half* __restrict__ current_value, const float* __restrict__ scratch,
                   __half* __restrict__ output, PagedParams p, uint32_t splits) {
  grid_chain_prologue();
  constexpr int kRecord = 16 + 8 * D;
  static_assert(D >= (int)kMaxAttentionSplits, "one thread per split in the weighing phase");
  __shared__ float partial[3][D / 32];
  __shared__ float weights[kMaxAttentionSplits];
  __shared__ float part_sums[kMergeParts - 1][D];
  const uint32_t head = blockIdx.x, batch = blockIdx.y, d = threadIdx.x % D, part = threadIdx.x / D;
  const uint32_t heads_per_kv = p.query_heads / p.kv_heads;
  const uint32_t kv_head = head / heads_per_kv, local_head = head % heads_per_kv;
  const size_t query_base = ((size_t)batch * p.query_heads + head) * D;
  const size_t current_base = ((size_t)batch * p.kv_heads + kv_head) * D;
  const float* records = scratch + ((size_t)batch * p.kv_heads + kv_head) * splits * kRecord;

  // this part's share of the split columns: issued first, consumed last
  constexpr int kShare = (int)kMaxAttentionSplits / kMergeParts;
  const uint32_t first_split = part * kShare;
  const float* column = records + 16 + local_head * D + d;
  float values[kShare];
#pragma unroll
  for (int i = 0; i < kShare; ++i)
    values[i] = first_split + i < splits ? column[(size_t)(first_split + i) * kRecord] : 0.0f;

  // the weighing phase runs on the first D threads; every global load of it is issued before
  // the first reduction
  const bool weigher = part == 0;
  const float split_max = weigher && d < splits ? records[d * kRecord + local_head] : -INFINITY;
  const float split_sum = weigher && d < splits ? records[d * kRecord + 8 + local_head] : 0.0f;
  const float current_v = __half2float(current_value[current_base + d]);
  float dot = __half2float(query[query_base + d]) * __half2float(current_key[current_base + d]);
  dot = warp_sum(dot);
  const float warp_maximum = warp_max(split_max);
  if (weigher && (d & 31u) == 0) {
    partial[0][d >> 5] = dot;
    partial[1][d >> 5] = warp_maximum;
  }
  __syncthreads();
  float current_score = 0.0f, maximum = -INFINITY;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) {
    current_score += partial[0][i];
    maximum = fmaxf(maximum, partial[1][i]);
  }
  current_score *= p.scale;
  maximum = fmaxf(maximum, current_score);
  const float current_weight = expf(current_score - maximum);
  const float weight = split_max == -INFINITY ? 0.0f : expf(split_max - maximum);
  if (weigher && d < splits) weights[d] = weight;
  const float weighted = warp_sum(weight * split_sum);
  if (weigher && (d & 31u) == 0) partial[2][d >> 5] = weighted;
  __syncthreads();
  float denominator = current_weight;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) denominator += partial[2][i];

  float result = weigher ? current_weight * current_v : 0.0f;
#pragma unroll
  for (int i = 0; i < kShare; ++i)
    if (first_split + i < splits) result = fmaf(weights[first_split + i], values[i], result);
  if (!weigher) part_sums[part - 1][d] = result;
  __syncthreads();
  if (!weigher) return;
#pragma unroll
  for (int other = 0; other < kMergeParts - 1; ++other) result += part_sums[other][d];
  const size_t output_base = ((size_t)batch * p.query_heads + head) * D;  // [b, q = 1, hq, D]
  output[output_base + d] = __float2half_rn(denominator == 0.0f ? 0.0f : result / denominator);
}

template <int D, int GROUP, int CP>
int launch_split_copy(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride, float* scratch,
                      uint32_t splits, uint32_t pool_tokens) {
  auto kernel = args.rotary_fusion ? paged_split_kernel<D, GROUP, CP, true> : paged_split_kernel<D, GROUP, CP, false>;
  constexpr int ring_bytes = SplitShape<D, CP>::kRingBytes;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes) != cudaSuccess) {
    cudaGetLastError();
    return fail(args, "paged attention: the device cannot give one CTA its tile ring");
  }
  const RotaryPackFusion fusion = args.rotary_fusion ? *args.rotary_fusion : RotaryPackFusion{};
  launch_kernel(args, kernel, dim3(splits, p.kv_heads, p.batches), dim3(kWarps * 32), ring_bytes,
      (const __half*)args.buffers[0], (const uint8_t*)args.buffers[3], (const uint32_t*)args.buffers[4], scratch, p,
      slot_batch_stride, splits, args.past_tokens_cell, pool_tokens,
      args.ctx ? context_device_error(args.ctx) : nullptr, fusion);
  return check_launch(args);
}

template <int D, int GROUP>
int launch_split(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride, float* scratch,
                 uint32_t splits, uint32_t pool_tokens) {
  const bool aligned = (p.token_stride % 16 == 0) && (((uintptr_t)args.buffers[3]) % 16 == 0);
  const int status = aligned ? launch_split_copy<D, GROUP, 16>(args, p, slot_batch_stride, scratch, splits, pool_tokens)
                             : launch_split_copy<D, GROUP, 8>(args, p, slot_batch_stride, scratch, splits, pool_tokens);
  if (status) return status;
  launch_kernel(args, paged_merge_kernel<D>, dim3(p.query_heads, p.batches), dim3(D * kMergeParts), 0,
      (const __half*)args.buffers[0], (const __half*)args.buffers[1], (const __half*)args.buffers[2], scratch,
      (__half*)args.buffers[6], p, splits);
  return check_launch(args);
}

}  // namespace

bool paged_split_supported(const PagedParams& p) {
  const uint32_t heads_per_kv = p.query_heads / p.kv_heads;
  if (!((p.head_dim == 64 || p.head_dim == 128) && (p.group_size == 32 || p.group_size == 64) &&
        heads_per_kv <= 8 && p.token_stride % 8 == 0 && p.key_offset % 16 == 0 && p.value_offset % 16 == 0))
    return false;
  // the group scales of one head are fetched with a single load of that size
  const uint32_t scale_bytes = 2u * p.head_dim / p.group_size;
  return (p.token_elements + 2u * (p.key_offset / p.group_size)) % scale_bytes == 0 &&
         (p.token_elements + 2u * (p.value_offset / p.group_size)) % scale_bytes == 0;
}

uint32_t paged_pick_splits(const KernelArgs& args, const PagedParams& p) {
  // kResidentCtas CTAs are resident per SM.  Few (batch, KV head) pairs: as many splits as
  // allowed, the machine cannot be filled anyway and a short split is a short dependent chain.
  // Otherwise: from the smallest count that fills 85% of the CTA slots up to four times that,
  // the one whose waves fill the machine best, charging a little for every extra record the merge
  // has to read.  A split is never shorter than 64 keys at capture time (a replayed plan keeps the
  // count while the context grows).
  const uint32_t pairs = p.batches * p.kv_heads;
  const uint32_t resident = (uint32_t)context_sm_count(args.ctx) * (uint32_t)kResidentCtas;
  uint32_t limit = args.past_tokens_cell ? kMaxAttentionSplits : (p.past_length + 63u) / 64u;
  if (limit > kMaxAttentionSplits) limit = kMaxAttentionSplits;
  if (limit == 0) return 1;
  // LLMOPT_CUDA_ATTENTION_SPLITS pins the count (within the limit), for tuning
  static const uint32_t pinned = []() -> uint32_t {
    const char* text = getenv("LLMOPT_CUDA_ATTENTION_SPLITS");
    const long value = text ? strtol(text, nullptr, 10) : 0;
    return value > 0 ? (uint32_t)value : 0u;
  }();
  if (pinned != 0u) return pinned < limit ? pinned : limit;
  const uint32_t fill_target = (resident * 85u + 99u) / 100u;
  const uint32_t first = (fill_target + pairs - 1u) / pairs;
  if (first >= limit) return limit;
  uint32_t last = first * 4u > first + 8u ? first * 4u : first + 8u;
  if (last > limit) last = limit;
  uint32_t best = first;
  float best_score = -1.0f;
  for (uint32_t splits = first; splits <= last; ++splits) {
    const uint32_t ctas = pairs * splits;
    const uint32_t waves = (ctas + resident - 1u) / resident;
    const float score = (float)ctas / (float)(waves * resident) - 0.002f * (float)splits;
    if (score > best_score) {
      best_score = score;
      best = splits;
    }
  }
  return best;
}

int launch_paged_attention_split_on(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride,
                                    float* scratch, uint32_t splits, uint32_t pool_tokens) {
  LLMOPT_REQUIRE(((uintptr_t)args.buffers[3]) % 8 == 0, "pool must be 8-byte aligned");
  LLMOPT_REQUIRE(((uintptr_t)args.buffers[0]) % 4 == 0, "query must be 4-byte aligned");
  if (p.head_dim == 64)
    return p.group_size == 64 ? launch_split<64, 64>(args, p, slot_batch_stride, scratch, splits, pool_tokens)
                              : launch_split<64, 32>(args, p, slot_batch_stride, scratch, splits, pool_tokens);
  return p.group_size == 64 ? launch_split<128, 64>(args, p, slot_batch_stride, scratch, splits, pool_tokens)
                            : launch_split<128, 32>(args, p, slot_batch_stride, scratch, splits, pool_tokens);
}

int launch_paged_attention_split(const KernelArgs& args, const PagedParams& p, uint32_t slot_batch_stride,
                                 uint32_t pool_tokens) {
  const uint32_t splits = paged_pick_splits(args, p);
  const size_t bytes =
      (size_t)p.batches * p.kv_heads * splits * paged_split_record_floats(p.head_dim) * sizeof(float);
  float* scratch = (float*)context_scratch(args.ctx, bytes, args.error);
  if (scratch == nullptr) return 1;
  return launch_paged_attention_split_on(args, p, slot_batch_stride, scratch, splits, pool_tokens);
}

}  // namespace llmopt
