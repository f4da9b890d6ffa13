// Dense fp16 attention for prefill: softmax(Q K^T scale + causal / mask) V.
// Reference: llmopt_attention_f16_simd_h<D> and llmopt_attention_f16
// (lib/metal_attention_source.ml), dispatch_attention (lib/metal_dispatch_attention.ml:6-102),
// CPU Cpu.attention (lib/cpu.ml:606-717).  Buffers [query, key, value, mask, output]; the 56-byte
// parameter block of lib/metal_parameters.ml:95-117.
//   query [b, h, q, D]; key [b, kvh, k, D]; value [b, kvh, k, D] or token-first [b, k, kvh, D];
//   output [b, h, q, D] or token-first [b, q, h, D]; causal: key ki is visible to query qi when
//   ki <= qi + past_length; mask dtype 2: f16, a value >= 0 keeps the key, other dtypes: a
//   nonzero byte keeps it (llmopt_attention_allowed, lib/metal_attention_source.ml:257-274).
//
// Two kernels behind the names:
//  * D in {64, 128}: a flash-attention forward pass on mma.sync.m16n8k16: one CTA per 64 queries
//    of one (batch, head), four warps of 16 query rows; K and V tiles staged in padded shared
//    memory; S = Q K^T with K rows as the col-major B operand (ldmatrix), online softmax in
//    fp32 per row (units of log2 e), P rounded to half before P V like the reference's SIMD
//    kernel (lib/metal_attention_source.ml:183-189), V as B operand through ldmatrix.trans.
//  * any other head size: one warp per (batch, head, query) walking the keys with a
//    single-pass online softmax in fp32.
// The work is O(q k D) on small prefill lengths; it is not on the HBM-bound decode path.
#include "common.cuh"

namespace llmopt {
namespace {

struct DenseParams {  // lib/metal_parameters.ml:95-117
  uint32_t batches, heads, q_len, k_len, dim, mask_batches, mask_heads, causal;
  float scale;
  uint32_t kv_heads, token_first_output, past_length, token_first_value, mask_dtype;
};
static_assert(sizeof(DenseParams) == 56, "parameter block is 56 bytes");

__device__ __forceinline__ bool key_allowed(const DenseParams& p, const uint8_t* mask, uint32_t batch, uint32_t head,
                                            uint32_t qi, uint32_t ki) {
  if (p.causal && ki > qi + p.past_length) return false;
  if (mask != nullptr && p.mask_batches > 0) {
    const uint32_t mb = p.mask_batches == 1 ? 0u : batch, mh = p.mask_heads == 1 ? 0u : head;
    const size_t index = (((size_t)mb * p.mask_heads + mh) * p.q_len + qi) * p.k_len + ki;
    if (p.mask_dtype == 2) return __half2float(reinterpret_cast<const __half*>(mask)[index]) >= 0.0f;
    return mask[index] != 0;
  }
  return true;
}
__device__ __forceinline__ size_t value_index(const DenseParams& p, uint32_t batch, uint32_t kv_head, uint32_t ki) {
  return p.token_first_value ? (((size_t)batch * p.k_len + ki) * p.kv_heads + kv_head) * p.dim
                             : (((size_t)batch * p.kv_heads + kv_head) * p.k_len + ki) * p.dim;
}
__device__ __forceinline__ size_t output_index(const DenseParams& p, uint32_t batch, uint32_t head, uint32_t qi) {
  return p.token_first_output ? (((size_t)batch * p.q_len + qi) * p.heads + head) * p.dim
                              : (((size_t)batch * p.heads + head) * p.q_len + qi) * p.dim;
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
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float low, float high) {
  const __half2 pair = __floats2half2_rn(low, high);
  return *reinterpret_cast<const uint32_t*>(&pair);
}
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int kQueryTile = 64;
constexpr float kLowest = -1.0e30f;

// 16-byte asynchronous copy global -> shared; `bytes` = 0 writes zeros (rows past the end)
__device__ __forceinline__ void copy_async_16(void* shared_target, const void* source, uint32_t bytes) {
  const uint32_t address = (uint32_t)__cvta_generic_to_shared(shared_target);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(address), "l"(source), "r"(bytes) : "memory");
}

// 64 query rows per CTA (16 per warp), KT keys per tile.  K and V tiles are double-buffered in dynamic
// shared memory and fetched with cp.async one tile ahead of the arithmetic; a tile every key of which
// every query row of the warp may see (no mask, inside the causal triangle, inside k_len) skips the
// per-element visibility test.
template <int D, int KT>
__global__ void __launch_bounds__(128) dense_attention_mma_kernel(const __half* __restrict__ query,
                                                                  const __half* __restrict__ key,
                                                                  const __half* __restrict__ value,
                                                                  const uint8_t* __restrict__ mask,
                                                                  __half* __restrict__ output, DenseParams p) {
  grid_chain_prologue();
  constexpr int kStride = D + 8;  // halves per shared row: 16 bytes of padding against bank conflicts
  extern __shared__ __align__(16) unsigned char dense_shared[];
  typedef __half Row[kStride];
  Row* q_tile = reinterpret_cast<Row*>(dense_shared);                 // [kQueryTile]
  Row* k_tiles = q_tile + kQueryTile;                                  // [2][KT]
  Row* v_tiles = k_tiles + 2 * KT;                                     // [2][KT]
  // the last query tiles see the most keys under a causal mask: they are scheduled first
  const uint32_t q0 = (gridDim.x - 1u - blockIdx.x) * kQueryTile, head = blockIdx.y, batch = blockIdx.z;
  const uint32_t kv_head = head / (p.heads / p.kv_heads);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, r = lane >> 2, c = lane & 3u;
  constexpr int kChunks = D / 8;  // 16-byte chunks per row

  // keys beyond the last visible one of this query tile are never touched
  uint32_t key_end = p.k_len;
  if (p.causal) {
    const uint32_t last_query = min(q0 + kQueryTile, p.q_len) - 1u;
    key_end = min(p.k_len, last_query + p.past_length + 1u);
  }
  const uint32_t tiles = (key_end + KT - 1) / KT;
  auto fetch_tile = [&](uint32_t tile) {
    if (tile < tiles) {
      const uint32_t k0 = tile * KT;
      Row* k_tile = k_tiles + (tile & 1u) * KT;
      Row* v_tile = v_tiles + (tile & 1u) * KT;
      for (uint32_t index = threadIdx.x; index < KT * kChunks; index += 128) {
        const uint32_t row = index / kChunks, chunk = index % kChunks;
        const bool present = k0 + row < p.k_len;
        const uint32_t ki = present ? k0 + row : 0u;
        copy_async_16(&k_tile[row][chunk * 8],
                      key + (((size_t)batch * p.kv_heads + kv_head) * p.k_len + ki) * D + chunk * 8, present ? 16u : 0u);
        copy_async_16(&v_tile[row][chunk * 8], value + value_index(p, batch, kv_head, ki) + chunk * 8, present ? 16u : 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch_tile(0);

  for (uint32_t index = threadIdx.x; index < kQueryTile * kChunks; index += 128) {
    const uint32_t row = index / kChunks, chunk = index % kChunks;
    uint4 data = make_uint4(0u, 0u, 0u, 0u);
    if (q0 + row < p.q_len)
      data = *reinterpret_cast<const uint4*>(query + (((size_t)batch * p.heads + head) * p.q_len + q0 + row) * D + chunk * 8);
    *reinterpret_cast<uint4*>(&q_tile[row][chunk * 8]) = data;
  }
  __syncthreads();
  // this warp's 16 query rows as A fragments for every 16-wide step of D
  uint32_t q_frag[D / 16][4];
#pragma unroll
  for (int s = 0; s < D / 16; ++s)
    ldmatrix_x4(q_frag[s], &q_tile[warp * 16 + (lane & 7u) + ((lane >> 3) & 1u) * 8u][16 * s + (lane >> 4) * 8u]);

  const uint32_t row_low = q0 + warp * 16 + r, row_high = row_low + 8;  // the two query rows of this lane
  const float score_scale = p.scale * 1.4426950408889634f;
  float running_max[2] = {kLowest, kLowest}, running_sum[2] = {0.0f, 0.0f};
  float out[D / 8][4];
#pragma unroll
  for (int t = 0; t < D / 8; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) out[t][j] = 0.0f;

  for (uint32_t tile = 0; tile < tiles; ++tile) {
    const uint32_t k0 = tile * KT;
    fetch_tile(tile + 1);  // into the other buffer, which the previous iteration's last barrier released
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // this tile has landed (the next one may be in flight)
    __syncthreads();
    Row* k_tile = k_tiles + (tile & 1u) * KT;
    Row* v_tile = v_tiles + (tile & 1u) * KT;

    // S[16 x KT] = Q K^T: n-tile j covers keys 8j .. 8j+7
    float score[KT / 8][4];
#pragma unroll
    for (int j = 0; j < KT / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) score[j][i] = 0.0f;
#pragma unroll
    for (int s = 0; s < D / 16; ++s)
#pragma unroll
      for (int j = 0; j < KT / 16; ++j) {
        uint32_t b[4];  // (keys 16j..+7, dims 16s..+7), (same keys, dims +8), (keys +8, dims +0), (keys +8, dims +8)
        ldmatrix_x4(b, &k_tile[16 * j + (lane & 7u) + (lane >> 4) * 8u][16 * s + ((lane >> 3) & 1u) * 8u]);
        mma_16816(score[2 * j], q_frag[s], b[0], b[1]);
        mma_16816(score[2 * j + 1], q_frag[s], b[2], b[3]);
      }

    // visibility and the tile maximum of the two rows
    float tile_max[2] = {kLowest, kLowest};
    const bool all_visible = mask == nullptr && k0 + KT <= p.k_len && q0 + warp * 16 + 15u < p.q_len &&
                             (!p.causal || k0 + KT - 1u <= q0 + warp * 16 + p.past_length);
    if (all_visible) {
#pragma unroll
      for (int j = 0; j < KT / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          score[j][i] *= score_scale;
          tile_max[i >> 1] = fmaxf(tile_max[i >> 1], score[j][i]);
        }
    } else {
#pragma unroll
      for (int j = 0; j < KT / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t qi = (i & 2) ? row_high : row_low, ki = k0 + 8 * j + 2 * c + (i & 1);
          const bool visible = qi < p.q_len && ki < p.k_len && key_allowed(p, mask, batch, head, qi, ki);
          score[j][i] = visible ? score[j][i] * score_scale : -INFINITY;
          tile_max[i >> 1] = fmaxf(tile_max[i >> 1], score[j][i]);
        }
    }
    float rescale[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float next_max = fmaxf(running_max[h], tile_max[h]);  // finite: at least kLowest
      rescale[h] = exp2_fast(running_max[h] - next_max);
      running_max[h] = next_max;
      running_sum[h] *= rescale[h];
    }
#pragma unroll
    for (int t = 0; t < D / 8; ++t) {
      out[t][0] *= rescale[0];
      out[t][1] *= rescale[0];
      out[t][2] *= rescale[1];
      out[t][3] *= rescale[1];
    }
    // P = exp2(S - max), rounded to half; the denominator adds the rounded values that P V uses
    uint32_t p_frag[KT / 16][4];
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
      float e[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) e[i] = exp2_fast(score[j][i] - running_max[i >> 1]);
      const __half2 low = __floats2half2_rn(e[0], e[1]), high = __floats2half2_rn(e[2], e[3]);
      const float2 low_f = __half22float2(low), high_f = __half22float2(high);
      running_sum[0] += low_f.x + low_f.y;
      running_sum[1] += high_f.x + high_f.y;
      // C layout of n-tiles (2t, 2t+1) = A layout of the 16-key step t
      p_frag[j >> 1][(j & 1) * 2] = *reinterpret_cast<const uint32_t*>(&low);
      p_frag[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&high);
    }
    // O[16 x D] += P V
#pragma unroll
    for (int s = 0; s < KT / 16; ++s)
#pragma unroll
      for (int t = 0; t < D / 16; ++t) {
        uint32_t b[4];  // (keys 16s..+7, dims 16t..+7), (keys +8, dims +0), (keys +0, dims +8), (keys +8, dims +8)
        ldmatrix_x4_trans(b, &v_tile[16 * s + (lane & 7u) + ((lane >> 3) & 1u) * 8u][16 * t + (lane >> 4) * 8u]);
        mma_16816(out[2 * t], p_frag[s], b[0], b[1]);
        mma_16816(out[2 * t + 1], p_frag[s], b[2], b[3]);
      }
    __syncthreads();  // every warp is done with this buffer before the next iteration's fetch refills it
  }
  asm volatile("cp.async.wait_all;" ::: "memory");

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 1);
    running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t qi = h ? row_high : row_low;
    if (qi >= p.q_len) continue;
    const float inverse = running_sum[h] == 0.0f ? 0.0f : 1.0f / running_sum[h];
    __half* target = output + output_index(p, batch, head, qi);
#pragma unroll
    for (int t = 0; t < D / 8; ++t)
      *reinterpret_cast<uint32_t*>(target + 8 * t + 2 * c) =
          pack_half2(out[t][2 * h] * inverse, out[t][2 * h + 1] * inverse);
  }
}

constexpr int kMaxFragments = 16;  // D <= 512

// One warp per (batch, head, query): single-pass online softmax, lib/metal_attention_source.ml:294-381.
__global__ void __launch_bounds__(256) dense_attention_rows_kernel(const __half* __restrict__ query,
                                                                   const __half* __restrict__ key,
                                                                   const __half* __restrict__ value,
                                                                   const uint8_t* __restrict__ mask,
                                                                   __half* __restrict__ output, DenseParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= p.batches * p.heads * p.q_len) return;
  const uint32_t qi = row % p.q_len, head = (row / p.q_len) % p.heads, batch = row / (p.q_len * p.heads);
  const uint32_t kv_head = head / (p.heads / p.kv_heads);
  const __half* q_row = query + (((size_t)batch * p.heads + head) * p.q_len + qi) * p.dim;
  const uint32_t fragments = (p.dim + 31) / 32;
  float q_values[kMaxFragments], results[kMaxFragments];
#pragma unroll
  for (int f = 0; f < kMaxFragments; ++f) {
    const uint32_t d = lane + f * 32;
    q_values[f] = (f < (int)fragments && d < p.dim) ? __half2float(q_row[d]) : 0.0f;
    results[f] = 0.0f;
  }
  float maximum = -INFINITY, denominator = 0.0f;
  for (uint32_t ki = 0; ki < p.k_len; ++ki) {
    if (!key_allowed(p, mask, batch, head, qi, ki)) continue;
    const __half* k_row = key + (((size_t)batch * p.kv_heads + kv_head) * p.k_len + ki) * p.dim;
    float dot = 0.0f;
#pragma unroll
    for (int f = 0; f < kMaxFragments; ++f) {
      const uint32_t d = lane + f * 32;
      if (f < (int)fragments && d < p.dim) dot = fmaf(q_values[f], __half2float(k_row[d]), dot);
    }
    const float score = warp_sum(dot) * p.scale;
    const float next_max = fmaxf(maximum, score);
    const float rescale = maximum == -INFINITY ? 0.0f : expf(maximum - next_max);
    const float weight = expf(score - next_max);
    const __half* v_row = value + value_index(p, batch, kv_head, ki);
#pragma unroll
    for (int f = 0; f < kMaxFragments; ++f) {
      const uint32_t d = lane + f * 32;
      if (f < (int)fragments && d < p.dim) results[f] = results[f] * rescale + weight * __half2float(v_row[d]);
    }
    denominator = denominator * rescale + weight;
    maximum = next_max;
  }
  __half* target = output + output_index(p, batch, head, qi);
#pragma unroll
  for (int f = 0; f < kMaxFragments; ++f) {
    const uint32_t d = lane + f * 32;
    if (f < (int)fragments && d < p.dim)
      target[d] = __float2half_rn(denominator == 0.0f ? 0.0f : results[f] / denominator);
  }
}

}  // namespace

// Buffers [query, key, value, mask (the query again when there is none), output]; 56 parameter bytes.
int launch_attention_dense(const KernelArgs& args) {
  DenseParams p;
  LLMOPT_REQUIRE(args.buffer_count == 5 && args.param_bytes == sizeof(p), "expects 5 buffers and 56 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  if (p.kv_heads == 0) p.kv_heads = p.heads;
  LLMOPT_REQUIRE(p.batches > 0 && p.heads > 0 && p.q_len > 0 && p.k_len > 0, "needs positive sizes");
  LLMOPT_REQUIRE(p.dim > 0 && p.dim <= 512, "head_dim must be in 1..512");
  LLMOPT_REQUIRE(p.heads % p.kv_heads == 0, "heads must be a multiple of kv_heads");
  const size_t q_elements = (size_t)p.batches * p.heads * p.q_len * p.dim;
  const size_t k_elements = (size_t)p.batches * p.kv_heads * p.k_len * p.dim;
  LLMOPT_REQUIRE(args.lengths[0] >= q_elements * 2 && args.lengths[4] >= q_elements * 2, "query or output buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= k_elements * 2 && args.lengths[2] >= k_elements * 2, "key or value buffer is too short");
  const uint8_t* mask = p.mask_batches == 0 ? nullptr : (const uint8_t*)args.buffers[3];
  if (mask != nullptr) {
    LLMOPT_REQUIRE(p.mask_heads > 0, "mask_heads must be positive with a mask");
    const size_t mask_elements = (size_t)p.mask_batches * p.mask_heads * p.q_len * p.k_len;
    LLMOPT_REQUIRE(args.lengths[3] >= mask_elements * (p.mask_dtype == 2 ? 2 : 1), "mask buffer is too short");
  }
  const bool aligned = (((uintptr_t)args.buffers[0] | (uintptr_t)args.buffers[1] | (uintptr_t)args.buffers[2]) & 15u) == 0 &&
                       ((uintptr_t)args.buffers[4] & 3u) == 0;
  const dim3 grid((p.q_len + kQueryTile - 1) / kQueryTile, p.heads, p.batches);
  auto shared_bytes = [](uint32_t dim, uint32_t keys) { return (size_t)(kQueryTile + 4 * keys) * (dim + 8) * sizeof(__half); };
  if (aligned && p.dim == 64) {
    auto kernel = dense_attention_mma_kernel<64, 64>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared_bytes(64, 64));
    launch_kernel(args, kernel, grid, dim3(128), shared_bytes(64, 64), (const __half*)args.buffers[0],
                  (const __half*)args.buffers[1], (const __half*)args.buffers[2], mask, (__half*)args.buffers[4], p);
  } else if (aligned && p.dim == 128) {
    auto kernel = dense_attention_mma_kernel<128, 64>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared_bytes(128, 64));
    launch_kernel(args, kernel, grid, dim3(128), shared_bytes(128, 64), (const __half*)args.buffers[0],
                  (const __half*)args.buffers[1], (const __half*)args.buffers[2], mask, (__half*)args.buffers[4], p);
  } else {
    const size_t rows = (size_t)p.batches * p.heads * p.q_len;
    launch_kernel(args, dense_attention_rows_kernel, dim3((uint32_t)((rows + 7) / 8)), dim3(256), 0,
                  (const __half*)args.buffers[0], (const __half*)args.buffers[1], (const __half*)args.buffers[2], mask,
                  (__half*)args.buffers[4], p);
  }
  return check_launch(args);
}

}  // namespace llmopt
