// Grouped-Q8 cache codec for sm_100a: attention K/V pack / unpack and recurrent
// checkpoint pack / unpack.  Bit-exact restatement of
//   llmopt_cache_pack_attention_q8{,_simd,_pair_simd}   lib/metal_cache_source.ml:46-182
//   llmopt_cache_unpack_attention_q8{,_vec4}            lib/metal_cache_source.ml:184-243
//   llmopt_cache_{pack,unpack}_checkpoint_q8{,_simd,_vec4}  lib/metal_cache_source.ml:245-347
// Integer results and stored scales must equal the reference byte for byte:
// scale = half(max == 0 ? 1 : max / 127) (fp32 division), q = clamp(rint(x /
// float(scale)), -127, 127) with IEEE division and round-half-even.
//
// One warp owns one quantisation group (the reference's *_simd mapping); lanes
// stride the group so any group size works.  HBM-bound and tiny: 2 bytes read,
// 1 + 2/G written per element.
#include "q8_codec.cuh"

namespace llmopt {
uint32_t* context_device_error(Context* ctx);
namespace {

struct AttentionCacheParams {  // lib/metal_cache_source.ml:9-20
  uint32_t items, segment_offset, heads, head_dim, group_size, token_elements, token_groups,
      token_stride, source_items, source_offset;
};
struct CheckpointCacheParams {  // lib/metal_cache_source.ml:36-44
  uint32_t checkpoint, layer, layer_elements, group_size, checkpoint_elements, checkpoint_groups,
      checkpoint_stride;
};

__global__ void pack_attention_kernel(const __half* __restrict__ source, const uint32_t* __restrict__ slots,
                                      uint8_t* __restrict__ pool, AttentionCacheParams p, PoolBound bound) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t logical_group = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t groups_per_head = p.head_dim / p.group_size;
  const uint32_t segment_groups = p.heads * groups_per_head;
  if (logical_group >= p.items * segment_groups) return;
  const uint32_t item = logical_group / segment_groups;
  const uint32_t local_group = logical_group - item * segment_groups;
  const uint32_t head = local_group / groups_per_head;
  const uint32_t group_in_head = local_group - head * groups_per_head;
  const size_t source_base = ((size_t)head * p.source_items + p.source_offset + item) * p.head_dim +
                             (size_t)group_in_head * p.group_size;
  if (!slot_in_pool(slots[item], bound, lane)) return;
  const size_t slot_base = (size_t)slots[item] * p.token_stride;
  int8_t* values = reinterpret_cast<int8_t*>(pool + slot_base);
  __half* scales = reinterpret_cast<__half*>(pool + slot_base + p.token_elements);
  const uint32_t value_base = p.segment_offset + head * p.head_dim + group_in_head * p.group_size;
  quantize_group(source + source_base, p.group_size, values + value_base,
                 scales + p.segment_offset / p.group_size + local_group, lane);
}

__global__ void pack_attention_pair_kernel(const __half* __restrict__ key_source,
                                           const __half* __restrict__ value_source,
                                           const uint32_t* __restrict__ slots, uint8_t* __restrict__ pool,
                                           AttentionCachePairParams p, PoolBound bound) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t logical_group = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t groups_per_head = p.head_dim / p.group_size;
  const uint32_t segment_groups = p.heads * groups_per_head;
  if (logical_group >= p.items * segment_groups) return;
  const uint32_t item = logical_group / segment_groups;
  const uint32_t local_group = logical_group - item * segment_groups;
  const uint32_t head = local_group / groups_per_head;
  const uint32_t group_in_head = local_group - head * groups_per_head;
  const size_t source_base = ((size_t)head * p.source_items + p.source_offset + item) * p.head_dim +
                             (size_t)group_in_head * p.group_size;
  if (!slot_in_pool(slots[item], bound, lane)) return;
  const size_t slot_base = (size_t)slots[item] * p.token_stride;
  int8_t* values = reinterpret_cast<int8_t*>(pool + slot_base);
  __half* scales = reinterpret_cast<__half*>(pool + slot_base + p.token_elements);
  const uint32_t local_offset = head * p.head_dim + group_in_head * p.group_size;
  quantize_group(key_source + source_base, p.group_size, values + p.key_segment_offset + local_offset,
                 scales + p.key_segment_offset / p.group_size + local_group, lane);
  quantize_group(value_source + source_base, p.group_size, values + p.value_segment_offset + local_offset,
                 scales + p.value_segment_offset / p.group_size + local_group, lane);
}

// One decode token per sequence: the rotary embedding of Q and K (llmopt_rotary_qk_f16_simd_h64,
// lib/metal_normalization_source.ml:765-802) and the Q8 pack of the rotated K row and the V row
// into the new cache slot (llmopt_cache_pack_attention_q8_pair_simd) as one launch; a prebaked
// plan takes it when the two records are adjacent and the pack reads what the rotary wrote.
// One warp per head row (rotary_pack_row); every lane quantises the columns it rotated itself, with the
// same half-precision operation sequence and the same codec as the two kernels, so all bytes are equal.
__global__ void rotary_pack_kernel(RotaryPackFusion f) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t q_rows = f.rotary.batches * f.rotary.q_heads, k_rows = f.rotary.batches * f.rotary.k_heads;
  if (row >= q_rows + 2u * k_rows) return;
  const uint32_t kind = row < q_rows ? 0u : (row < q_rows + k_rows ? 1u : 2u);
  const uint32_t local_row = kind == 0 ? row : (kind == 1 ? row - q_rows : row - q_rows - k_rows);
  const uint32_t heads = kind == 0 ? f.rotary.q_heads : f.rotary.k_heads;
  rotary_pack_row(f, kind, local_row / heads, local_row % heads, lane);
}

__global__ void unpack_attention_kernel(const uint8_t* __restrict__ pool, const uint32_t* __restrict__ slots,
                                        __half* __restrict__ destination, AttentionCacheParams p,
                                        PoolBound bound) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t segment_elements = p.heads * p.head_dim;
  if (gid >= p.items * segment_elements) return;
  const uint32_t item = gid / segment_elements;
  const uint32_t local = gid - item * segment_elements;
  const uint32_t head = local / p.head_dim;
  const uint32_t within_head = local - head * p.head_dim;
  const uint32_t groups_per_head = p.head_dim / p.group_size;
  const uint32_t local_group = head * groups_per_head + within_head / p.group_size;
  const size_t destination_index = ((size_t)head * p.items + item) * p.head_dim + within_head;
  if (!slot_in_pool(slots[item], bound, 0u)) {
    destination[destination_index] = __float2half_rn(0.0f);
    return;
  }
  const size_t slot_base = (size_t)slots[item] * p.token_stride;
  const int8_t* values = reinterpret_cast<const int8_t*>(pool + slot_base);
  const __half* scales = reinterpret_cast<const __half*>(pool + slot_base + p.token_elements);
  destination[destination_index] = __float2half_rn(
      (float)values[p.segment_offset + local] *
      __half2float(scales[p.segment_offset / p.group_size + local_group]));
}

__global__ void pack_checkpoint_kernel(const __half* __restrict__ source, uint8_t* __restrict__ pool,
                                       CheckpointCacheParams p, const uint32_t* __restrict__ checkpoint_cell,
                                       PoolBound bound) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t logical_group = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t layer_groups = p.layer_elements / p.group_size;
  if (logical_group >= layer_groups) return;
  const uint32_t checkpoint = checkpoint_cell ? *checkpoint_cell : p.checkpoint;
  if (!slot_in_pool(checkpoint, bound, lane)) return;
  const size_t base = (size_t)checkpoint * p.checkpoint_stride;
  int8_t* values = reinterpret_cast<int8_t*>(pool + base);
  __half* scales = reinterpret_cast<__half*>(pool + base + p.checkpoint_elements);
  quantize_group(source + (size_t)logical_group * p.group_size, p.group_size,
                 values + (size_t)p.layer * p.layer_elements + (size_t)logical_group * p.group_size,
                 scales + (size_t)p.layer * layer_groups + logical_group, lane);
}

__global__ void unpack_checkpoint_kernel(const uint8_t* __restrict__ pool, __half* __restrict__ destination,
                                         CheckpointCacheParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.layer_elements) return;
  const size_t base = (size_t)p.checkpoint * p.checkpoint_stride;
  const int8_t* values = reinterpret_cast<const int8_t*>(pool + base);
  const __half* scales = reinterpret_cast<const __half*>(pool + base + p.checkpoint_elements);
  const uint32_t layer_groups = p.layer_elements / p.group_size;
  destination[gid] = __float2half_rn((float)values[(size_t)p.layer * p.layer_elements + gid] *
                                     __half2float(scales[(size_t)p.layer * layer_groups + gid / p.group_size]));
}

// ---- Tile32 affine cache with a 32-point Walsh-Hadamard rotation ------------------------------------
// llmopt_cache_{pack,unpack}_attention_tile32_affine{8,4}_fwht_simd, lib/metal_cache_source.ml:1249-1393.
// One warp per tile of 32 consecutive head dimensions: the tile is rotated by the normalised
// Hadamard transform (butterflies over lane distance 1, 2, 4, 8, 16, then * 1 / sqrt(32)),
// quantised with a per-tile fp16 scale = range / (2^bits - 1) and fp16 minimum, and stored as
// {scale, minimum, codes} — 36 bytes with 8-bit codes, 20 bytes with 4-bit codes (low nibble =
// lanes 0..15, high nibble = lanes 16..31).  Unpack dequantises and applies the same transform
// (it is its own inverse).  Every operation is an fp32 operation in the reference's order, so pack
// and unpack results equal the reference's byte for byte.
__device__ __forceinline__ float fwht32(float x, uint32_t lane) {
#pragma unroll
  for (uint32_t s = 1; s < 32; s <<= 1) {
    const float partner = __shfl_xor_sync(0xffffffffu, x, s);
    x = (lane & s) == 0u ? __fadd_rn(x, partner) : __fsub_rn(partner, x);
  }
  return __fmul_rn(x, 0.17677669529663689f);
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

template <int BITS>
__global__ void pack_attention_fwht_kernel(const __half* __restrict__ source, const uint32_t* __restrict__ slots,
                                           uint8_t* __restrict__ pool, AttentionCacheParams p, PoolBound bound) {
  grid_chain_prologue();
  constexpr uint32_t kTileBytes = BITS == 8 ? 36u : 20u;
  constexpr float kLevels = BITS == 8 ? 255.0f : 15.0f;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t logical_tile = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t tiles_per_head = p.head_dim >> 5, segment_tiles = p.heads * tiles_per_head;
  if (logical_tile >= p.items * segment_tiles) return;
  const uint32_t item = logical_tile / segment_tiles, local_tile = logical_tile - item * segment_tiles;
  const uint32_t head = local_tile / tiles_per_head, tile_in_head = local_tile - head * tiles_per_head;
  const size_t source_base = ((size_t)head * p.source_items + p.source_offset + item) * p.head_dim + (tile_in_head << 5);
  const float rotated = fwht32(__half2float(source[source_base + lane]), lane);
  const float low = warp_min(rotated), high = warp_max(rotated);
  const float range = fmaxf(0.0f, __fsub_rn(high, low));
  const __half stored_scale = __float2half_rn(__fdiv_rn(range, kLevels)), stored_minimum = __float2half_rn(low);
  const float scale = __half2float(stored_scale), minimum = __half2float(stored_minimum);
  if (!slot_in_pool(slots[item], bound, lane)) return;
  uint8_t* tile = pool + (size_t)slots[item] * p.token_stride + (size_t)((p.segment_offset >> 5) + local_tile) * kTileBytes;
  if (lane == 0) {
    *reinterpret_cast<__half*>(tile) = stored_scale;
    *reinterpret_cast<__half*>(tile + 2) = stored_minimum;
  }
  uint32_t code = 0;
  if (scale > 1e-8f) code = (uint32_t)max(0, min((int)kLevels, (int)rintf(__fdiv_rn(__fsub_rn(rotated, minimum), scale))));
  if (BITS == 8) {
    tile[4 + lane] = (uint8_t)code;
  } else {
    const uint32_t upper = __shfl_xor_sync(0xffffffffu, code, 16);
    if (lane < 16) tile[4 + lane] = (uint8_t)((code & 15u) | ((upper & 15u) << 4));
  }
}

template <int BITS>
__global__ void unpack_attention_fwht_kernel(const uint8_t* __restrict__ pool, const uint32_t* __restrict__ slots,
                                             __half* __restrict__ destination, AttentionCacheParams p, PoolBound bound) {
  grid_chain_prologue();
  constexpr uint32_t kTileBytes = BITS == 8 ? 36u : 20u;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t logical_tile = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t tiles_per_head = p.head_dim >> 5, segment_tiles = p.heads * tiles_per_head;
  if (logical_tile >= p.items * segment_tiles) return;
  const uint32_t item = logical_tile / segment_tiles, local_tile = logical_tile - item * segment_tiles;
  const uint32_t head = local_tile / tiles_per_head, tile_in_head = local_tile - head * tiles_per_head;
  const size_t destination_index = ((size_t)head * p.items + item) * p.head_dim + (tile_in_head << 5) + lane;
  if (!slot_in_pool(slots[item], bound, lane)) {
    destination[destination_index] = __float2half_rn(0.0f);
    return;
  }
  const uint8_t* tile = pool + (size_t)slots[item] * p.token_stride + (size_t)((p.segment_offset >> 5) + local_tile) * kTileBytes;
  const float scale = __half2float(*reinterpret_cast<const __half*>(tile));
  const float minimum = __half2float(*reinterpret_cast<const __half*>(tile + 2));
  uint32_t code;
  if (BITS == 8) {
    code = tile[4 + lane];
  } else {
    const uint8_t packed = tile[4 + (lane & 15u)];
    code = lane < 16 ? (packed & 15u) : (packed >> 4);
  }
  const float rotated = __fadd_rn(__fmul_rn(scale, (float)code), minimum);
  destination[destination_index] = __float2half_rn(fwht32(rotated, lane));
}

template <typename P>
bool read_params(const KernelArgs& args, P* out) {
  if (args.param_bytes != sizeof(P)) return false;
  memcpy(out, args.params, sizeof(P));
  return true;
}

bool valid_geometry(uint32_t head_dim, uint32_t group_size) {
  return group_size > 0 && head_dim > 0 && head_dim % group_size == 0;
}

// A token row holds the int8 payload of every segment and, after token_elements bytes, one fp16
// scale per group: both the segment and its scales must lie inside the row.
bool segment_in_token(uint32_t segment_offset, uint32_t heads, uint32_t head_dim, uint32_t group_size,
                      uint32_t token_elements, uint32_t token_stride) {
  const size_t segment_end = (size_t)segment_offset + (size_t)heads * head_dim;
  return token_stride > 0 && segment_end <= token_elements &&
         (size_t)token_elements + 2 * ((segment_end + group_size - 1) / group_size) <= token_stride;
}

PoolBound pool_bound(const KernelArgs& args, int pool_index, uint32_t row_stride) {
  const size_t rows = row_stride ? args.lengths[pool_index] / row_stride : 0;
  return {rows > 0xffffffffull ? 0xffffffffu : (uint32_t)rows, args.ctx ? context_device_error(args.ctx) : nullptr};
}

}  // namespace

// Buffers: [source f16, slots u32, pool u8]; params 40 bytes (lib/metal_cache.ml:315-318).
int launch_cache_pack_attention_q8(const KernelArgs& args) {
  AttentionCacheParams p;
  LLMOPT_REQUIRE(args.buffer_count == 3, "expects buffers [source, slots, pool]");
  LLMOPT_REQUIRE(read_params(args, &p), "expects 40 parameter bytes");
  LLMOPT_REQUIRE(valid_geometry(p.head_dim, p.group_size), "head_dim must be a multiple of group_size");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.items * 4, "slots buffer is shorter than items");
  LLMOPT_REQUIRE(args.lengths[0] >= ((size_t)(p.heads - 1) * p.source_items + p.source_offset + p.items) * p.head_dim * 2,
                 "source buffer is shorter than the packed range");
  LLMOPT_REQUIRE(segment_in_token(p.segment_offset, p.heads, p.head_dim, p.group_size, p.token_elements, p.token_stride),
                 "segment or its scales lie outside the token row");
  const uint32_t groups = p.items * p.heads * (p.head_dim / p.group_size);
  if (groups == 0) return 0;
  launch_kernel(args, pack_attention_kernel, dim3((groups + 7) / 8), dim3(256), 0,
      (const __half*)args.buffers[0], (const uint32_t*)args.buffers[1], (uint8_t*)args.buffers[2], p,
      pool_bound(args, 2, p.token_stride));
  return check_launch(args);
}

// Tile32 affine + FWHT cache: buffers and the 40-byte block of the Q8 pack / unpack; segment_offset
// counts ELEMENTS (32 per tile), a token row holds token_elements / 32 tiles of 36 or 20 bytes.
template <int BITS, bool PACK>
static int launch_cache_fwht(const KernelArgs& args) {
  AttentionCacheParams p;
  LLMOPT_REQUIRE(args.buffer_count == 3, PACK ? "expects buffers [source, slots, pool]" : "expects buffers [pool, slots, destination]");
  LLMOPT_REQUIRE(read_params(args, &p), "expects 40 parameter bytes");
  LLMOPT_REQUIRE(p.head_dim > 0 && p.head_dim % 32 == 0 && p.segment_offset % 32 == 0, "head_dim and segment_offset must be multiples of 32");
  constexpr size_t kTileBytes = BITS == 8 ? 36 : 20;
  const int pool_index = PACK ? 2 : 0, data_index = PACK ? 0 : 2;
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.items * 4, "slots buffer is shorter than items");
  const size_t segment_end = (size_t)p.segment_offset + (size_t)p.heads * p.head_dim;
  LLMOPT_REQUIRE(p.token_stride > 0 && segment_end / 32 * kTileBytes <= p.token_stride, "segment lies outside the token row");
  const size_t elements = PACK ? ((size_t)(p.heads ? p.heads - 1 : 0) * p.source_items + p.source_offset + p.items) * p.head_dim
                               : (size_t)p.items * p.heads * p.head_dim;
  LLMOPT_REQUIRE(args.lengths[data_index] >= elements * 2, PACK ? "source buffer is shorter than the packed range" : "destination buffer is too short");
  const uint32_t tiles = p.items * p.heads * (p.head_dim / 32);
  if (tiles == 0) return 0;
  const PoolBound bound = pool_bound(args, pool_index, p.token_stride);
  if (PACK)
    launch_kernel(args, pack_attention_fwht_kernel<BITS>, dim3((tiles + 7) / 8), dim3(256), 0, (const __half*)args.buffers[0],
                  (const uint32_t*)args.buffers[1], (uint8_t*)args.buffers[2], p, bound);
  else
    launch_kernel(args, unpack_attention_fwht_kernel<BITS>, dim3((tiles + 7) / 8), dim3(256), 0, (const uint8_t*)args.buffers[0],
                  (const uint32_t*)args.buffers[1], (__half*)args.buffers[2], p, bound);
  return check_launch(args);
}
int launch_cache_pack_tile32_affine8_fwht(const KernelArgs& args) { return launch_cache_fwht<8, true>(args); }
int launch_cache_unpack_tile32_affine8_fwht(const KernelArgs& args) { return launch_cache_fwht<8, false>(args); }
int launch_cache_pack_tile32_affine4_fwht(const KernelArgs& args) { return launch_cache_fwht<4, true>(args); }
int launch_cache_unpack_tile32_affine4_fwht(const KernelArgs& args) { return launch_cache_fwht<4, false>(args); }

// Buffers: [key source, value source, slots, pool]; params 44 bytes (lib/metal_cache.ml:344-347).
int launch_cache_pack_attention_q8_pair(const KernelArgs& args) {
  AttentionCachePairParams p;
  LLMOPT_REQUIRE(args.buffer_count == 4, "expects buffers [key, value, slots, pool]");
  LLMOPT_REQUIRE(read_params(args, &p), "expects 44 parameter bytes");
  LLMOPT_REQUIRE(valid_geometry(p.head_dim, p.group_size), "head_dim must be a multiple of group_size");
  LLMOPT_REQUIRE(args.lengths[2] >= (size_t)p.items * 4, "slots buffer is shorter than items");
  const size_t source_bytes = ((size_t)(p.heads - 1) * p.source_items + p.source_offset + p.items) * p.head_dim * 2;
  LLMOPT_REQUIRE(p.heads > 0 && args.lengths[0] >= source_bytes && args.lengths[1] >= source_bytes,
                 "source buffer is shorter than the packed range");
  LLMOPT_REQUIRE(segment_in_token(p.key_segment_offset, p.heads, p.head_dim, p.group_size, p.token_elements, p.token_stride) &&
                     segment_in_token(p.value_segment_offset, p.heads, p.head_dim, p.group_size, p.token_elements, p.token_stride),
                 "segment or its scales lie outside the token row");
  const uint32_t groups = p.items * p.heads * (p.head_dim / p.group_size);
  if (groups == 0) return 0;
  launch_kernel(args, pack_attention_pair_kernel, dim3((groups + 7) / 8), dim3(256), 0,
      (const __half*)args.buffers[0], (const __half*)args.buffers[1], (const uint32_t*)args.buffers[2],
      (uint8_t*)args.buffers[3], p, pool_bound(args, 3, p.token_stride));
  return check_launch(args);
}

// The fused form of a rotary record followed by the pair-pack record of the same token, or false when
// the two do not fit it.  rotary: [q_in, k_in, cosine, sine, q_out, k_out]; pack: [key, value, slots, pool].
bool make_rotary_pack_fusion(const KernelArgs& rotary, const KernelArgs& pack, RotaryPackFusion* fusion) {
  RotaryQkParams r;
  AttentionCachePairParams c;
  if (rotary.buffer_count != 6 || rotary.param_bytes != sizeof(r) || pack.buffer_count != 4 || !read_params(pack, &c))
    return false;
  memcpy(&r, rotary.params, sizeof(r));
  if (r.tokens != 1 || r.width == 0 || r.half_dimension * 2 > r.width || r.batches == 0 || r.k_heads == 0) return false;
  if (pack.buffers[0] != rotary.buffers[5] || c.items != r.batches || c.source_items != c.items || c.source_offset != 0)
    return false;
  if (c.group_size == 0 || r.width % c.group_size != 0 || !valid_geometry(c.head_dim, c.group_size)) return false;
  if ((size_t)c.heads * c.head_dim != (size_t)r.k_heads * r.width || (c.heads != 1 && c.items != 1)) return false;
  if ((c.key_segment_offset | c.value_segment_offset) % c.group_size != 0) return false;
  if (!segment_in_token(c.key_segment_offset, c.heads, c.head_dim, c.group_size, c.token_elements, c.token_stride) ||
      !segment_in_token(c.value_segment_offset, c.heads, c.head_dim, c.group_size, c.token_elements, c.token_stride))
    return false;  // the stand-alone pack launcher reports it
  const size_t q_bytes = (size_t)r.batches * r.q_heads * r.width * 2, k_bytes = (size_t)r.batches * r.k_heads * r.width * 2;
  const size_t trig_bytes = (size_t)(r.trig_batches == 1 ? 1 : r.batches) * r.width * 2;
  if (rotary.lengths[0] < q_bytes || rotary.lengths[4] < q_bytes || rotary.lengths[1] < k_bytes ||
      rotary.lengths[5] < k_bytes || rotary.lengths[2] < trig_bytes || rotary.lengths[3] < trig_bytes ||
      pack.lengths[1] < k_bytes || pack.lengths[2] < (size_t)c.items * 4)
    return false;
  fusion->q_input = (const __half*)rotary.buffers[0];
  fusion->k_input = (const __half*)rotary.buffers[1];
  fusion->v_input = (const __half*)pack.buffers[1];
  fusion->cosine = (const __half*)rotary.buffers[2];
  fusion->sine = (const __half*)rotary.buffers[3];
  fusion->q_output = (__half*)rotary.buffers[4];
  fusion->k_output = (__half*)rotary.buffers[5];
  fusion->slots = (const uint32_t*)pack.buffers[2];
  fusion->pool = (uint8_t*)pack.buffers[3];
  fusion->rotary = r;
  fusion->cache = c;
  const PoolBound bound = pool_bound(pack, 3, c.token_stride);
  fusion->bound = bound;
  return true;
}

// Returns -1 when the two records do not fit the fused form (the caller then runs them one after the
// other), 0 on success, 1 on a launch failure.
int launch_rotary_pack_fused(const KernelArgs& rotary, const KernelArgs& pack) {
  RotaryPackFusion fusion;
  if (!make_rotary_pack_fusion(rotary, pack, &fusion)) return -1;
  const uint32_t rows = fusion.rotary.batches * (fusion.rotary.q_heads + 2u * fusion.rotary.k_heads);
  launch_kernel(rotary, rotary_pack_kernel, dim3((rows + 7) / 8), dim3(256), 0, fusion);
  return check_launch(rotary);
}

// Buffers: [pool, slots, destination]; params 40 bytes.
int launch_cache_unpack_attention_q8(const KernelArgs& args) {
  AttentionCacheParams p;
  LLMOPT_REQUIRE(args.buffer_count == 3, "expects buffers [pool, slots, destination]");
  LLMOPT_REQUIRE(read_params(args, &p), "expects 40 parameter bytes");
  LLMOPT_REQUIRE(valid_geometry(p.head_dim, p.group_size), "head_dim must be a multiple of group_size");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.items * 4, "slots buffer is shorter than items");
  const size_t elements = (size_t)p.items * p.heads * p.head_dim;
  LLMOPT_REQUIRE(args.lengths[2] >= elements * 2, "destination buffer is too short");
  LLMOPT_REQUIRE(segment_in_token(p.segment_offset, p.heads, p.head_dim, p.group_size, p.token_elements, p.token_stride),
                 "segment or its scales lie outside the token row");
  if (elements == 0) return 0;
  launch_kernel(args, unpack_attention_kernel, dim3((uint32_t)((elements + 255) / 256)), dim3(256), 0,
      (const uint8_t*)args.buffers[0], (const uint32_t*)args.buffers[1], (__half*)args.buffers[2], p,
      pool_bound(args, 0, p.token_stride));
  return check_launch(args);
}

// Buffers: [source, pool]; params 28 bytes (lib/metal_cache.ml:544-547).
int launch_cache_pack_checkpoint_q8(const KernelArgs& args) {
  CheckpointCacheParams p;
  LLMOPT_REQUIRE(args.buffer_count == 2, "expects buffers [source, pool]");
  LLMOPT_REQUIRE(read_params(args, &p), "expects 28 parameter bytes");
  LLMOPT_REQUIRE(p.group_size > 0 && p.layer_elements % p.group_size == 0, "layer_elements must be a multiple of group_size");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)p.layer_elements * 2, "source buffer is too short");
  const uint32_t groups = p.layer_elements / p.group_size;
  LLMOPT_REQUIRE(((size_t)p.layer + 1) * p.layer_elements <= p.checkpoint_elements &&
                     (size_t)p.checkpoint_elements + 2 * ((size_t)p.layer + 1) * groups <= p.checkpoint_stride,
                 "layer or its scales lie outside the checkpoint row");
  const PoolBound bound = pool_bound(args, 1, p.checkpoint_stride);
  LLMOPT_REQUIRE(args.checkpoint_cell != nullptr || p.checkpoint < bound.tokens, "checkpoint lies outside the pool");
  if (groups == 0) return 0;
  launch_kernel(args, pack_checkpoint_kernel, dim3((groups + 7) / 8), dim3(256), 0,
      (const __half*)args.buffers[0], (uint8_t*)args.buffers[1], p, args.checkpoint_cell, bound);
  return check_launch(args);
}

// Buffers: [pool, destination]; params 28 bytes.
int launch_cache_unpack_checkpoint_q8(const KernelArgs& args) {
  CheckpointCacheParams p;
  LLMOPT_REQUIRE(args.buffer_count == 2, "expects buffers [pool, destination]");
  LLMOPT_REQUIRE(read_params(args, &p), "expects 28 parameter bytes");
  LLMOPT_REQUIRE(p.group_size > 0 && p.layer_elements % p.group_size == 0, "layer_elements must be a multiple of group_size");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.layer_elements * 2, "destination buffer is too short");
  LLMOPT_REQUIRE(((size_t)p.layer + 1) * p.layer_elements <= p.checkpoint_elements &&
                     (size_t)p.checkpoint_elements + 2 * ((size_t)p.layer + 1) * (p.layer_elements / p.group_size) <=
                         p.checkpoint_stride,
                 "layer or its scales lie outside the checkpoint row");
  LLMOPT_REQUIRE(p.checkpoint < pool_bound(args, 0, p.checkpoint_stride).tokens, "checkpoint lies outside the pool");
  if (p.layer_elements == 0) return 0;
  launch_kernel(args, unpack_checkpoint_kernel, dim3((p.layer_elements + 255) / 256), dim3(256), 0,
      (const uint8_t*)args.buffers[0], (__half*)args.buffers[1], p);
  return check_launch(args);
}

}  // namespace llmopt
