// Q4_0-block quantised linears (GGUF layout): block = 18 bytes {f16 d; u8 qs[16]} for 32 weights,
// element i < 16 is (qs[i] & 15) - 8, element i >= 16 is (qs[i - 16] >> 4) - 8, w = d * q; a weight
// row of K elements is K / 32 consecutive blocks (row stride (K / 32) * 18 bytes).
// Reference: lib/metal_q4_0_source.ml (dequant and gated kernels), lib/metal_quant_qkv_source.ml
// (fused QKV), the generated llmopt_q4_0_linear_f16* tactics (lib/metal_block_codegen.ml) and
// dispatch_quant_linear (lib/metal_dispatch_common.ml:299-420).  The reference ships one kernel per
// tiling tactic (_x4, _x8, _x16, _m2, _m4, _m16, _m32, ...); the tactic only changes how rows and
// columns are tiled, not the arithmetic, so all of those names resolve to the kernels below.
//
// The same kernel serves the Tile32 affine formats (lib/block_schema.ml:706-741; kernels
// llmopt_tile32_affine{4,8}_linear_f16_{x8,m16,m32,simd}, lib/metal_block_codegen.ml:54-722): a block
// of 32 weights is {f16 scale; f16 minimum; codes}, 20 bytes with 4-bit codes (low nibble of byte
// j = element j, high nibble = element j + 16, as in Q4_0) or 36 bytes with 8-bit codes, and
// w = scale * code + minimum; the block's contribution is scale * sum(x code) + minimum * sum(x),
// the association the reference kernels use (:108-143).
//
// Two forms.  The general one: one warp per output column, the lanes take the row's blocks round-robin
// (a warp reads 32 x 18 contiguous bytes per step), each lane multiplies its block with the 32 matching
// activations of up to four batch rows, fp32 accumulation, one warp reduction per (row, column); more rows
// are served in tiles of four over the same weight row (which stays in L1).
// The tensor-core one (Q4_0 rows that are a whole number of 16-byte vectors, i.e. K a multiple of 256): a CTA
// works on 16 weight rows at a time, copied to shared memory with 16-byte cp.async (the first copies before it
// waits for its predecessor: weights do not depend on it), and its eight warps share out the blocks.  Up to 8
// batch rows it is a stream (a few CTAs per SM walk over the tiles, every warp with a private two-deep ring of
// its own K slices), beyond that a CTA per tile with K chunks of 4096 (up to 32 rows per pass).
// A block is two mma.sync.m16n8k16: the low nibbles (elements 0..15)
// as halves 1024 + u, the high nibbles (16..31), read in place, as 64 + u, one LOP3 per pair of weights; the
// offsets 1032 and 72 (u - 8 is the weight) leave as a per-block term -(1032 sum(x low) + 72 sum(x high)) that
// seeds the accumulator, and the block's fp32 sum is scaled by d.  The activations are staged once per CTA in
// the order of the B fragments.  HBM-bound at M = 1: 0.5625 bytes per weight.
#include <cstdlib>
#include <initializer_list>

#include "w4a16_gemv_device.cuh"

namespace llmopt {
namespace {

constexpr int kRowTile = 4;

// The block's 16 quant bytes start 2 bytes after an 18-byte stride: only 2-byte alignment holds.
__device__ __forceinline__ void load_block(const uint8_t* block, float& d, uint32_t (&qs)[4]) {
  const unsigned short* halves = reinterpret_cast<const unsigned short*>(block);
  const unsigned short scale = __ldg(halves);
  d = __half2float(*reinterpret_cast<const __half*>(&scale));
#pragma unroll
  for (int i = 0; i < 4; ++i)
    qs[i] = (uint32_t)__ldg(halves + 1 + 2 * i) | ((uint32_t)__ldg(halves + 2 + 2 * i) << 16);
}

// sum over the block of x[i] * q[i] for one activation row (32 halves at `x`, 16-byte aligned)
__device__ __forceinline__ float block_dot(const __half* x, const uint32_t (&qs)[4]) {
  float acc = 0.0f;
  const uint4* vectors = reinterpret_cast<const uint4*>(x);
  const uint4 low[2] = {vectors[0], vectors[1]};    // x[0..15]  pair with the low nibbles
  const uint4 high[2] = {vectors[2], vectors[3]};   // x[16..31] pair with the high nibbles
  const uint32_t* low_words = reinterpret_cast<const uint32_t*>(low);
  const uint32_t* high_words = reinterpret_cast<const uint32_t*>(high);
#pragma unroll
  for (int w = 0; w < 4; ++w)
#pragma unroll
    for (int pair = 0; pair < 2; ++pair) {
      // bytes 4w + 2 pair and 4w + 2 pair + 1 of the block
      const uint32_t two = (qs[w] >> (16 * pair)) & 0xffffu;
      const float2 x_low = __half22float2(*reinterpret_cast<const __half2*>(&low_words[2 * w + pair]));
      const float2 x_high = __half22float2(*reinterpret_cast<const __half2*>(&high_words[2 * w + pair]));
      acc = fmaf(x_low.x, (float)((int)(two & 15u) - 8), acc);
      acc = fmaf(x_high.x, (float)((int)((two >> 4) & 15u) - 8), acc);
      acc = fmaf(x_low.y, (float)((int)((two >> 8) & 15u) - 8), acc);
      acc = fmaf(x_high.y, (float)((int)(two >> 12) - 8), acc);
    }
  return acc;
}

enum BlockFormat { kQ4_0 = 0, kAffine4 = 1, kAffine8 = 2 };
template <int FORMAT> constexpr uint32_t kBlockBytes = FORMAT == kQ4_0 ? 18u : (FORMAT == kAffine4 ? 20u : 36u);

// Tile32 affine blocks are 4-byte aligned (20 / 36-byte stride on a 4-byte aligned row).
// scale * sum(x[i] * code[i]) + minimum * sum(x[i]) for one activation row.
template <int FORMAT>
__device__ __forceinline__ float affine_block_dot(const __half* x, const uint8_t* block) {
  const uint32_t* words = reinterpret_cast<const uint32_t*>(block);
  const uint32_t header = __ldg(words);
  const float scale = __half2float(__ushort_as_half((unsigned short)(header & 0xffffu)));
  const float minimum = __half2float(__ushort_as_half((unsigned short)(header >> 16)));
  const uint4* vectors = reinterpret_cast<const uint4*>(x);
  uint32_t x_words[16];
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint4 raw = vectors[v];
    x_words[4 * v] = raw.x, x_words[4 * v + 1] = raw.y, x_words[4 * v + 2] = raw.z, x_words[4 * v + 3] = raw.w;
  }
  float coded = 0.0f, plain = 0.0f;
  if (FORMAT == kAffine4) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t codes = __ldg(words + 1 + w);  // bytes 4w .. 4w+3: elements 4w+j (low) and 16+4w+j (high)
#pragma unroll
      for (int pair = 0; pair < 2; ++pair) {
        const float2 low = __half22float2(*reinterpret_cast<const __half2*>(&x_words[2 * w + pair]));
        const float2 high = __half22float2(*reinterpret_cast<const __half2*>(&x_words[8 + 2 * w + pair]));
        const uint32_t two = (codes >> (16 * pair)) & 0xffffu;
        coded = fmaf(low.x, (float)(two & 15u), coded);
        coded = fmaf(high.x, (float)((two >> 4) & 15u), coded);
        coded = fmaf(low.y, (float)((two >> 8) & 15u), coded);
        coded = fmaf(high.y, (float)(two >> 12), coded);
        plain += (low.x + high.x) + (low.y + high.y);
      }
    }
  } else {
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t codes = __ldg(words + 1 + w);  // elements 4w .. 4w+3
      const float2 first = __half22float2(*reinterpret_cast<const __half2*>(&x_words[2 * w]));
      const float2 second = __half22float2(*reinterpret_cast<const __half2*>(&x_words[2 * w + 1]));
      coded = fmaf(first.x, (float)(codes & 255u), coded);
      coded = fmaf(first.y, (float)((codes >> 8) & 255u), coded);
      coded = fmaf(second.x, (float)((codes >> 16) & 255u), coded);
      coded = fmaf(second.y, (float)(codes >> 24), coded);
      plain += (first.x + first.y) + (second.x + second.y);
    }
  }
  return fmaf(scale, coded, minimum * plain);
}

// acc[r] = x[row0 + r, :] . w[col, :] for r < rows (<= kRowTile), all lanes hold the sums
template <int FORMAT = kQ4_0>
__device__ __forceinline__ void column_dots(const __half* x, const uint8_t* weight_row, uint32_t k, uint32_t row0,
                                            uint32_t rows, uint32_t lane, float (&acc)[kRowTile]) {
#pragma unroll
  for (int r = 0; r < kRowTile; ++r) acc[r] = 0.0f;
  const uint32_t blocks = k >> 5;
  for (uint32_t b = lane; b < blocks; b += 32) {
    if (FORMAT == kQ4_0) {
      float d;
      uint32_t qs[4];
      load_block(weight_row + (size_t)b * 18u, d, qs);
#pragma unroll
      for (int r = 0; r < kRowTile; ++r)
        if ((uint32_t)r < rows) acc[r] = fmaf(d, block_dot(x + (size_t)(row0 + r) * k + b * 32u, qs), acc[r]);
    } else {
#pragma unroll
      for (int r = 0; r < kRowTile; ++r)
        if ((uint32_t)r < rows)
          acc[r] += affine_block_dot<FORMAT>(x + (size_t)(row0 + r) * k + b * 32u, weight_row + (size_t)b * kBlockBytes<FORMAT>);
    }
  }
#pragma unroll
  for (int r = 0; r < kRowTile; ++r) acc[r] = warp_sum(acc[r]);
}

struct QuantLinearParams {  // lib/metal_quant_source.ml:17-22
  uint32_t m, n, k, mode;
};

// llmopt_q4_0_linear_f16* / llmopt_tile32_affine{4,8}_linear_f16_*: mode 0 none, 1 bias[n], 2 residual[m, n]
template <int FORMAT>
__global__ void __launch_bounds__(256) quant_linear_kernel(const __half* __restrict__ x,
                                                           const uint8_t* __restrict__ weight,
                                                           const __half* __restrict__ additive,
                                                           __half* __restrict__ y, QuantLinearParams p,
                                                           float* __restrict__ y_f32) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u, col = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (col >= p.n) return;
  const uint8_t* weight_row = weight + (size_t)col * (p.k >> 5) * kBlockBytes<FORMAT>;
  for (uint32_t row0 = 0; row0 < p.m; row0 += kRowTile) {
    const uint32_t rows = min((uint32_t)kRowTile, p.m - row0);
    float acc[kRowTile];
    column_dots<FORMAT>(x, weight_row, p.k, row0, rows, lane, acc);
    if (lane < rows) {
      float value = acc[0];
#pragma unroll
      for (int r = 1; r < kRowTile; ++r)
        if (lane == (uint32_t)r) value = acc[r];
      const uint32_t row = row0 + lane;
      if (y_f32 != nullptr) {  // the unrounded sums, for an epilogue that runs after this kernel
        y_f32[(size_t)row * p.n + col] = value;
        continue;
      }
      if (p.mode == 1) value += __half2float(additive[col]);
      if (p.mode == 2) value += __half2float(additive[(size_t)row * p.n + col]);
      y[(size_t)row * p.n + col] = __float2half_rn(value);
    }
  }
}

// llmopt_gated_product, lib/metal_quant_source.ml:24-42
__device__ __forceinline__ __half gated_product(float gate_acc, float up_acc, uint32_t activation) {
  const float gate = __half2float(__float2half_rn(gate_acc));
  const __half up = __float2half_rn(up_acc);
  float activated;
  if (activation == 0u) {
    activated = gate / (1.0f + expf(-gate));
  } else if (activation == 1u) {
    const float inner = fminf(fmaxf(0.7978845608f * (gate + 0.044715f * gate * gate * gate), -10.0f), 10.0f);
    activated = 0.5f * gate * (1.0f + tanhf(inner));
  } else {
    activated = 1.0f / (1.0f + expf(-gate));
  }
  return __hmul(__float2half_rn(activated), up);
}

// llmopt_q4_0_gated_linear_f16*: product[m, n] = gated(x Wg^T, x Wu^T); `mode` selects the activation
__global__ void __launch_bounds__(256) q4_0_gated_kernel(const __half* __restrict__ x,
                                                         const uint8_t* __restrict__ gate_weight,
                                                         const uint8_t* __restrict__ up_weight,
                                                         __half* __restrict__ product, QuantLinearParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u, col = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (col >= p.n) return;
  const size_t row_bytes = (size_t)(p.k >> 5) * 18u;
  for (uint32_t row0 = 0; row0 < p.m; row0 += kRowTile) {
    const uint32_t rows = min((uint32_t)kRowTile, p.m - row0);
    float gate[kRowTile], up[kRowTile];
    column_dots(x, gate_weight + col * row_bytes, p.k, row0, rows, lane, gate);
    column_dots(x, up_weight + col * row_bytes, p.k, row0, rows, lane, up);
    if (lane < rows) {
      float g = gate[0], u = up[0];
#pragma unroll
      for (int r = 1; r < kRowTile; ++r)
        if (lane == (uint32_t)r) {
          g = gate[r];
          u = up[r];
        }
      product[(size_t)(row0 + lane) * p.n + col] = gated_product(g, u, p.mode);
    }
  }
}

struct QuantQkvParams {  // lib/metal_quant_qkv_source.ml:7-13
  uint32_t m, k, n_q, n_k, n_v;
};

// llmopt_q4_0_qkv_linear_f16*: three products in one launch, three separate outputs
__global__ void __launch_bounds__(256) q4_0_qkv_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ q_weight,
                                                       const uint8_t* __restrict__ k_weight,
                                                       const uint8_t* __restrict__ v_weight, __half* __restrict__ q_out,
                                                       __half* __restrict__ k_out, __half* __restrict__ v_out,
                                                       QuantQkvParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  uint32_t col = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (col >= p.n_q + p.n_k + p.n_v) return;
  const uint8_t* weight = q_weight;
  __half* out = q_out;
  uint32_t n = p.n_q;
  if (col >= p.n_q + p.n_k) {
    col -= p.n_q + p.n_k;
    weight = v_weight;
    out = v_out;
    n = p.n_v;
  } else if (col >= p.n_q) {
    col -= p.n_q;
    weight = k_weight;
    out = k_out;
    n = p.n_k;
  }
  const uint8_t* weight_row = weight + (size_t)col * (p.k >> 5) * 18u;
  for (uint32_t row0 = 0; row0 < p.m; row0 += kRowTile) {
    const uint32_t rows = min((uint32_t)kRowTile, p.m - row0);
    float acc[kRowTile];
    column_dots(x, weight_row, p.k, row0, rows, lane, acc);
    if (lane < rows) {
      float value = acc[0];
#pragma unroll
      for (int r = 1; r < kRowTile; ++r)
        if (lane == (uint32_t)r) value = acc[r];
      out[(size_t)(row0 + lane) * n + col] = __float2half_rn(value);
    }
  }
}

// llmopt_dequant_q4_0, lib/metal_q4_0_source.ml:9-23: one thread per element
__global__ void __launch_bounds__(256) q4_0_dequant_kernel(const uint8_t* __restrict__ blocks, __half* __restrict__ out,
                                                           uint32_t total_blocks) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x, block = gid >> 5, i = gid & 31u;
  if (block >= total_blocks) return;
  const uint8_t* source = blocks + (size_t)block * 18u;
  const unsigned short scale = *reinterpret_cast<const unsigned short*>(source);
  const float d = __half2float(*reinterpret_cast<const __half*>(&scale));
  const uint8_t byte = i < 16u ? source[2 + i] : source[2 + i - 16u];
  const int q = (int)(i < 16u ? (byte & 15u) : (byte >> 4)) - 8;
  out[(size_t)block * 32u + i] = __float2half_rn(d * (float)q);
}

// ---- tensor-core form ----------------------------------------------------------------------------
constexpr int kMmaRows = 16;                // weight rows (output columns) of a CTA
constexpr int kMmaWarps = 8;
constexpr uint32_t kChunkBlocks = 128;      // blocks of a K chunk: 4096 elements, 2304 bytes of a row
constexpr uint32_t kChunkPitch = kChunkBlocks * 18u + 16u;  // 145 vectors: rows 0..7 start 4 banks apart
constexpr int kCopyParts = 4;               // commit groups of a chunk: the first blocks are used while the rest lands
constexpr int kMaxRowTiles = 4;             // batch rows of a launch: 8 per tile

struct MmaProblem {
  uint32_t m, k, mode;          // mode: epilogue (linear), activation (gated)
  uint32_t matrices;            // 1, or 3 for the fused QKV (NMAT == 1); gate and up are one "matrix" of NMAT == 2
  const uint8_t* weight[3];     // gated: {gate, up}
  __half* out[3];
  uint32_t n[3], first_tile[3];  // columns and first CTA of every matrix
  const __half* additive;
  float* out_f32;               // != null (one matrix, linear form): the unrounded sums [m, n] instead of the halves
  uint32_t chunk_buffers;       // 1 or 2
  uint32_t staged_rows;         // batch rows the activation staging is sized for (1..8)
  uint32_t tiles_total;         // 16-row tiles of all matrices
};

// [address + OFFSET] with the offset in the instruction (an address operand of inline PTX costs a register and an add)
template <uint32_t OFFSET>
__device__ __forceinline__ uint32_t shared_load_32_at(uint32_t address) {
  uint32_t value;
  asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(value) : "r"(address), "n"(OFFSET) : "memory");
  return value;
}
// D = A B + C with C in registers of its own: the first MMA of a block takes the offset term without seeding moves
__device__ __forceinline__ void mma_16816_seeded(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1, float c0, float c1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ uint4 shared_load_128(uint32_t address) {
  uint4 value;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w) : "r"(address) : "memory");
  return value;
}
// two float2 that lie 32 bytes apart: the offset terms of a lane's two columns, for a block and for the next one
__device__ __forceinline__ float4 shared_load_float2_pair(uint32_t address) {
  float4 value;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(value.x), "=f"(value.y) : "r"(address) : "memory");
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2+32];" : "=f"(value.z), "=f"(value.w) : "r"(address) : "memory");
  return value;
}
__device__ __forceinline__ void copy_wait(int pending) {  // cp.async.wait_group takes an immediate
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}

// One pair of blocks (36 bytes of every row, word aligned) of a staged chunk against one batch-row tile: four MMAs per
// weight tile.  `fragment_at`: this lane's B fragment of the pair's first block (the second `fragment_stride` further);
// `offsets_at`: the offset terms of columns 2c, 2c + 1 of the first block (the second block's 32 bytes further).
template <int NMAT, uint32_t PITCH>
__device__ __forceinline__ void block_pair_step(uint32_t buffer_at, uint32_t pair, uint32_t fragment_at, uint32_t fragment_stride,
                                                uint32_t offsets_at, bool has_row, uint32_t r, uint32_t c, float (&acc)[NMAT][4]) {
  using namespace gemv;
  uint4 b_even = make_uint4(0u, 0u, 0u, 0u), b_odd = b_even;
  if (has_row) {
    b_even = shared_load_128(fragment_at);
    b_odd = shared_load_128(fragment_at + fragment_stride);
  }
  const float4 offsets = shared_load_float2_pair(offsets_at);  // {even block: columns 2c, 2c + 1; odd block: the same}
#pragma unroll
  for (int a = 0; a < NMAT; ++a) {
    // the pair of one row: {d, 16 quant bytes} {d, 16 quant bytes} = nine words; rows r and r + 8
    const uint32_t row_at = buffer_at + (a * kMmaRows + r) * PITCH + 36u * pair, quad_at = row_at + 4u * c;
    const uint32_t head_a = shared_load_32_at<0>(row_at), tail_a = shared_load_32_at<16>(row_at);
    const uint32_t head_b = shared_load_32_at<8 * PITCH>(row_at), tail_b = shared_load_32_at<8 * PITCH + 16>(row_at);
    // even block: its quant word c starts two bytes into word c; odd block: quant word c is word 5 + c
    const uint32_t even_a = __funnelshift_r(shared_load_32_at<0>(quad_at), shared_load_32_at<4>(quad_at), 16);
    const uint32_t even_b = __funnelshift_r(shared_load_32_at<8 * PITCH>(quad_at), shared_load_32_at<8 * PITCH + 4>(quad_at), 16);
    const uint32_t odd_a = shared_load_32_at<20>(quad_at), odd_b = shared_load_32_at<8 * PITCH + 20>(quad_at);
    // d of the even block is the low half of the pair's first word, d of the odd block the high half of its fifth
    const float d_even_a = __low2float(*reinterpret_cast<const __half2*>(&head_a)), d_odd_a = __high2float(*reinterpret_cast<const __half2*>(&tail_a));
    const float d_even_b = __low2float(*reinterpret_cast<const __half2*>(&head_b)), d_odd_b = __high2float(*reinterpret_cast<const __half2*>(&tail_b));
    float sum[4], next[4];
    // low nibbles of bytes (0, 2) and (1, 3): elements (4c, 4c + 2), (4c + 1, 4c + 3) as 1024 + u
    mma_16816_seeded(sum, lop3_and_xor(even_a, 0x000F000Fu, 0x64006400u), lop3_and_xor(even_b, 0x000F000Fu, 0x64006400u),
                     lop3_and_xor(even_a >> 8, 0x000F000Fu, 0x64006400u), lop3_and_xor(even_b >> 8, 0x000F000Fu, 0x64006400u),
                     b_even.x, b_even.y, offsets.x, offsets.y);
    // high nibbles in place: elements 16 + the same, as 64 + u
    mma_16816(sum, lop3_and_xor(even_a, 0x00F000F0u, 0x54005400u), lop3_and_xor(even_b, 0x00F000F0u, 0x54005400u),
              lop3_and_xor(even_a >> 8, 0x00F000F0u, 0x54005400u), lop3_and_xor(even_b >> 8, 0x00F000F0u, 0x54005400u),
              b_even.z, b_even.w);
    mma_16816_seeded(next, lop3_and_xor(odd_a, 0x000F000Fu, 0x64006400u), lop3_and_xor(odd_b, 0x000F000Fu, 0x64006400u),
                     lop3_and_xor(odd_a >> 8, 0x000F000Fu, 0x64006400u), lop3_and_xor(odd_b >> 8, 0x000F000Fu, 0x64006400u),
                     b_odd.x, b_odd.y, offsets.z, offsets.w);
    mma_16816(next, lop3_and_xor(odd_a, 0x00F000F0u, 0x54005400u), lop3_and_xor(odd_b, 0x00F000F0u, 0x54005400u),
              lop3_and_xor(odd_a >> 8, 0x00F000F0u, 0x54005400u), lop3_and_xor(odd_b >> 8, 0x00F000F0u, 0x54005400u),
              b_odd.z, b_odd.w);
    acc[a][0] = fmaf(d_odd_a, next[0], fmaf(d_even_a, sum[0], acc[a][0]));
    acc[a][1] = fmaf(d_odd_a, next[1], fmaf(d_even_a, sum[1], acc[a][1]));
    acc[a][2] = fmaf(d_odd_b, next[2], fmaf(d_even_b, sum[2], acc[a][2]));
    acc[a][3] = fmaf(d_odd_b, next[3], fmaf(d_even_b, sum[3], acc[a][3]));
  }
}

// One quad of a batch row's block in B-fragment order (k slots (2 quad, 2 quad + 1) hold elements (4 quad, 4 quad + 2),
// slots (+8, +9) elements (4 quad + 1, 4 quad + 3); the same for the upper sixteen), and its sums of x.
__device__ __forceinline__ uint4 fragment_of(const __half* source, float& low_sum, float& high_sum) {
  using namespace gemv;
  const uint2 low = *reinterpret_cast<const uint2*>(source), high = *reinterpret_cast<const uint2*>(source + 16);
  const float2 l0 = __half22float2(*reinterpret_cast<const __half2*>(&low.x));
  const float2 l1 = __half22float2(*reinterpret_cast<const __half2*>(&low.y));
  const float2 h0 = __half22float2(*reinterpret_cast<const __half2*>(&high.x));
  const float2 h1 = __half22float2(*reinterpret_cast<const __half2*>(&high.y));
  low_sum = (l0.x + l0.y) + (l1.x + l1.y);
  high_sum = (h0.x + h0.y) + (h1.x + h1.y);
  return make_uint4(prmt(low.x, low.y, 0x5410u), prmt(low.x, low.y, 0x7632u), prmt(high.x, high.y, 0x5410u), prmt(high.x, high.y, 0x7632u));
}

// Shared memory: [chunk buffers][NMAT][16 rows][kChunkPitch] | fragments [128 blocks][staged_rows][4] uint4 |
// bias [128 blocks][8] float | (the reduction reuses the fragments).
template <int NMAT>
__host__ __device__ inline size_t mma_shared_bytes(uint32_t chunk_buffers, uint32_t staged_rows) {
  const size_t fragments = (size_t)kChunkBlocks * staged_rows * 64u;
  const size_t reduction = (size_t)NMAT * kMmaWarps * kMmaRows * 8u * 4u;
  return (size_t)chunk_buffers * NMAT * kMmaRows * kChunkPitch + (fragments > reduction ? fragments : reduction) +
         (size_t)kChunkBlocks * 8u * 4u;
}

// TILES: batch-row tiles of eight the accumulators are built for (1: up to 8 rows, 4: up to 32)
template <int NMAT, int TILES>
__global__ void __launch_bounds__(kMmaWarps * 32, NMAT == 1 ? 4 : 2) q4_0_mma_kernel(const __half* __restrict__ x, MmaProblem p) {
  using namespace gemv;
  extern __shared__ __align__(16) uint8_t shared[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, r = lane >> 2, c = lane & 3u;
  // which matrix and which 16 of its rows
  uint32_t which = 0;
  if (NMAT == 1 && p.matrices == 3) which = blockIdx.x >= p.first_tile[2] ? 2u : (blockIdx.x >= p.first_tile[1] ? 1u : 0u);
  // (selected with constant indices: a dynamic index would put the parameter block on the stack)
  const uint32_t n = which == 0u ? p.n[0] : which == 1u ? p.n[1] : p.n[2];
  const uint32_t n0 = (blockIdx.x - (which == 0u ? p.first_tile[0] : which == 1u ? p.first_tile[1] : p.first_tile[2])) * kMmaRows;
  const uint8_t* const own_weight = which == 0u ? p.weight[0] : which == 1u ? p.weight[1] : p.weight[2];
  __half* const own_out = which == 0u ? p.out[0] : which == 1u ? p.out[1] : p.out[2];
  const uint32_t blocks = p.k >> 5, chunks = (blocks + kChunkBlocks - 1) / kChunkBlocks;
  const size_t row_bytes = (size_t)blocks * 18u;
  uint8_t* const weights = shared;
  uint4* const fragments = reinterpret_cast<uint4*>(shared + (size_t)p.chunk_buffers * NMAT * kMmaRows * kChunkPitch);
  const size_t fragment_bytes = (size_t)kChunkBlocks * p.staged_rows * 64u, reduction_bytes = (size_t)NMAT * kMmaWarps * kMmaRows * 32u;
  float* const bias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(fragments) +
                                                (fragment_bytes > reduction_bytes ? fragment_bytes : reduction_bytes));
  float* const reduction = reinterpret_cast<float*>(fragments);

  // one chunk of the CTA's rows -> buffer, as kCopyParts commit groups (rows past n re-read the last row):
  // sixteen consecutive threads copy consecutive vectors of one row
  const uint32_t copy_row = threadIdx.x >> 4, copy_lane = threadIdx.x & 15u;
  const uint8_t* copy_from[NMAT];
#pragma unroll
  for (int a = 0; a < NMAT; ++a)
    copy_from[a] = (NMAT == 2 ? p.weight[a] : own_weight) + (size_t)min(n0 + copy_row, n - 1u) * row_bytes + copy_lane * 16u;
  auto copy_chunk = [&](uint32_t chunk) {
    const uint32_t chunk_blocks = min(kChunkBlocks, blocks - chunk * kChunkBlocks);
    const uint32_t vectors = (chunk_blocks * 18u) >> 4, share = (vectors + kCopyParts - 1) / kCopyParts;
    const uint32_t buffer = (uint32_t)__cvta_generic_to_shared(weights) + (chunk % p.chunk_buffers) * (NMAT * kMmaRows * kChunkPitch) +
                            copy_row * kChunkPitch + copy_lane * 16u;
#pragma unroll
    for (int part = 0; part < kCopyParts; ++part) {
      const uint32_t end = min(vectors, (part + 1) * share);
      for (uint32_t vector = part * share + copy_lane; vector < end; vector += 16) {
#pragma unroll
        for (int a = 0; a < NMAT; ++a)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(buffer + a * (kMmaRows * kChunkPitch) + (vector - copy_lane) * 16u),
                       "l"(copy_from[a] + (size_t)chunk * (kChunkBlocks * 18u) + (size_t)(vector - copy_lane) * 16u)
                       : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  };
  copy_chunk(0);  // ahead of the predecessor's results
  grid_chain_prologue();

  const uint32_t row_tiles = (p.m + 7u) / 8u;
  float acc[TILES][NMAT][4];
#pragma unroll
  for (int t = 0; t < TILES; ++t)
#pragma unroll
    for (int a = 0; a < NMAT; ++a)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][a][i] = 0.0f;

  for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
    const bool ahead = chunk + 1u < chunks && p.chunk_buffers == 2u;
    if (ahead) copy_chunk(chunk + 1u);  // its buffer was released by the barrier that ended chunk - 1
    const uint32_t chunk_blocks = min(kChunkBlocks, blocks - chunk * kChunkBlocks);
    const uint32_t vectors = (chunk_blocks * 18u) >> 4, share = (vectors + kCopyParts - 1) / kCopyParts;
    // shared-window addresses: the loads of the block loop are ld.shared with 32-bit address arithmetic
    const uint32_t buffer_at = (uint32_t)__cvta_generic_to_shared(weights) + (chunk % p.chunk_buffers) * (NMAT * kMmaRows * kChunkPitch);
    const uint32_t fragments_at = (uint32_t)__cvta_generic_to_shared(fragments), bias_at = (uint32_t)__cvta_generic_to_shared(bias);
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
      if ((uint32_t)t >= row_tiles) break;
      const uint32_t rows = min(8u, p.m - 8u * t);
      // the tile's activations of this chunk in B-fragment order, and the per-block offset term
      // (only the rows that exist: with one row every thread stages two quads of it, all loads at once)
#pragma unroll 2
      for (uint32_t item = threadIdx.x; item < chunk_blocks * rows * 4u; item += kMmaWarps * 32) {
        const uint32_t block = rows == 1u ? item >> 2 : (item >> 2) / rows, row = (item >> 2) - block * rows, quad = item & 3u;
        float low_sum, high_sum;
        fragments[(block * p.staged_rows + row) * 4u + quad] =
            fragment_of(x + (size_t)(8u * t + row) * p.k + (size_t)(chunk * kChunkBlocks + block) * 32u + 4u * quad, low_sum, high_sum);
        low_sum += __shfl_xor_sync(0xffffffffu, low_sum, 1);
        low_sum += __shfl_xor_sync(0xffffffffu, low_sum, 2);
        high_sum += __shfl_xor_sync(0xffffffffu, high_sum, 1);
        high_sum += __shfl_xor_sync(0xffffffffu, high_sum, 2);
        if (quad == 0u) bias[block * 8u + row] = -(1032.0f * low_sum + 72.0f * high_sum);
      }
      uint32_t begin = 0;
#pragma unroll
      for (int part = 0; part < kCopyParts; ++part) {
        // the chunk's copies up to this part have landed (on the first tile; later tiles find them there)
        copy_wait((ahead ? kCopyParts : 0) + kCopyParts - 1 - part);
        __syncthreads();  // everybody's copies, and (part 0) the fragments
        // whole PAIRS of blocks (36 bytes, word aligned) inside the bytes landed so far; a warp takes every eighth pair
        const uint32_t end = (part == kCopyParts - 1 ? chunk_blocks : min(chunk_blocks, (min(vectors, (part + 1) * share) * 16u) / 18u)) & ~1u;
        for (uint32_t pair = begin / 2u + ((warp + kMmaWarps - (begin / 2u) % kMmaWarps) % kMmaWarps); 2u * pair < end; pair += kMmaWarps) {
          block_pair_step<NMAT, kChunkPitch>(buffer_at, pair, fragments_at + ((2u * pair * p.staged_rows + r) * 4u + c) * 16u,
                                p.staged_rows * 64u, bias_at + (2u * pair * 8u + 2u * c) * 4u, r < rows, r, c, acc[t]);
        }
        begin = end;
      }
      __syncthreads();  // the fragments (and, after the last tile, the chunk buffer) may be overwritten
    }
  }

  // the eight warps' sums meet in shared memory; thread (row, column) adds them in warp order and writes
#pragma unroll
  for (int t = 0; t < TILES; ++t) {
    if ((uint32_t)t >= row_tiles) break;
#pragma unroll
    for (int a = 0; a < NMAT; ++a) {
      float* mine = reduction + ((a * kMmaWarps + warp) * kMmaRows) * 8u;
      *reinterpret_cast<float2*>(mine + r * 8u + 2u * c) = make_float2(acc[t][a][0], acc[t][a][1]);
      *reinterpret_cast<float2*>(mine + (r + 8u) * 8u + 2u * c) = make_float2(acc[t][a][2], acc[t][a][3]);
    }
    __syncthreads();
    if (threadIdx.x < kMmaRows * 8) {
      const uint32_t row = threadIdx.x >> 3, batch_row = 8u * t + (threadIdx.x & 7u), column = n0 + row;
      float value[NMAT];
#pragma unroll
      for (int a = 0; a < NMAT; ++a) {
        value[a] = 0.0f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) value[a] += reduction[((a * kMmaWarps + w) * kMmaRows + row) * 8u + (threadIdx.x & 7u)];
      }
      if (batch_row < p.m && column < n) {
        if (NMAT == 2) {
          p.out[0][(size_t)batch_row * n + column] = gated_product(value[0], value[NMAT - 1], p.mode);
        } else {
          if (p.out_f32 != nullptr) {
            p.out_f32[(size_t)batch_row * n + column] = value[0];
          } else {
            if (p.mode == 1) value[0] += __half2float(p.additive[column]);
            if (p.mode == 2) value[0] += __half2float(p.additive[(size_t)batch_row * n + column]);
            own_out[(size_t)batch_row * n + column] = __float2half_rn(value[0]);
          }
        }
      }
    }
    __syncthreads();
  }
}

// The same arithmetic as a STREAM: up to 8 batch rows whose fragments of ALL of K fit shared memory.  A CTA stages the
// activations once, then walks over weight tiles blockIdx.x, + gridDim.x, ...  Every warp has a weight stream of its
// own: of each 128 blocks of K it owns 16 consecutive ones (288 contiguous bytes of each of the tile's rows), copies
// them with its own cp.async groups into a two-deep private ring and waits for nothing but its own copies, so the
// weight stream of an SM does not stop for a tile's reduction or a CTA's prologue; the CTA meets only to add the eight
// warps' sums of a tile.
constexpr uint32_t kSliceBlocks = 16, kSlicePitch = kSliceBlocks * 18u + 16u;  // 19 vectors: rows 0..7 start 4 banks apart
constexpr uint32_t kSliceSpan = kMmaWarps * kSliceBlocks;                      // blocks of K the eight slices cover
template <int NMAT>
__host__ __device__ inline size_t stream_shared_bytes(uint32_t blocks, uint32_t staged_rows) {
  return (size_t)kMmaWarps * 2u * NMAT * kMmaRows * kSlicePitch + (size_t)blocks * staged_rows * 64u + (size_t)blocks * 32u +
         (size_t)NMAT * kMmaWarps * kMmaRows * 32u;
}

template <int NMAT>
__global__ void __launch_bounds__(kMmaWarps * 32, 2) q4_0_mma_stream_kernel(const __half* __restrict__ x, MmaProblem p) {
  using namespace gemv;
  extern __shared__ __align__(16) uint8_t shared[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, r = lane >> 2, c = lane & 3u;
  const uint32_t blocks = p.k >> 5;
  constexpr uint32_t kStageBytes = NMAT * kMmaRows * kSlicePitch;
  const size_t row_bytes = (size_t)blocks * 18u;
  uint4* const fragments = reinterpret_cast<uint4*>(shared + kMmaWarps * 2u * kStageBytes);
  float* const bias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(fragments) + (size_t)blocks * p.staged_rows * 64u);
  float* const reduction = bias + (size_t)blocks * 8u;
  const uint32_t ring_at = (uint32_t)__cvta_generic_to_shared(shared) + warp * 2u * kStageBytes;
  const uint32_t fragments_at = (uint32_t)__cvta_generic_to_shared(fragments), bias_at = (uint32_t)__cvta_generic_to_shared(bias);

  const uint32_t my_tiles = blockIdx.x < p.tiles_total ? (p.tiles_total - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
  // this warp's slices of one row: blocks [span * kSliceSpan + warp * kSliceBlocks, + kSliceBlocks) while inside K
  const uint32_t first_slice = warp * kSliceBlocks;
  const uint32_t slices = blocks > first_slice ? (blocks - first_slice + kSliceSpan - 1u) / kSliceSpan : 0u;
  const uint32_t total = my_tiles * slices;
  // the matrix, its width and the first row of a tile
  auto locate = [&](uint32_t tile, uint32_t& which, uint32_t& n, uint32_t& n0) {
    which = 0;
    if (NMAT == 1 && p.matrices == 3) which = tile >= p.first_tile[2] ? 2u : (tile >= p.first_tile[1] ? 1u : 0u);
    n = which == 0u ? p.n[0] : which == 1u ? p.n[1] : p.n[2];
    n0 = (tile - (which == 0u ? p.first_tile[0] : which == 1u ? p.first_tile[1] : p.first_tile[2])) * kMmaRows;
  };
  // slice `sequence` of this warp (tile sequence / slices, span sequence % slices) -> ring stage sequence % 2: one commit group
  auto copy_slice = [&](uint32_t sequence) {
    if (sequence < total) {
      const uint32_t tile = blockIdx.x + (sequence / slices) * gridDim.x, start = (sequence % slices) * kSliceSpan + first_slice;
      uint32_t which, n, n0;
      locate(tile, which, n, n0);
      const uint32_t vectors = (min(kSliceBlocks, blocks - start) * 18u) >> 4;  // of one row: 18, or 9 for a last half slice
      const uint32_t target = ring_at + (sequence & 1u) * kStageBytes;
      const uint8_t* matrix = which == 0u ? p.weight[0] : which == 1u ? p.weight[1] : p.weight[2];
      uint32_t row = lane / vectors, vector = lane % vectors;
      const uint32_t row_step = 32u / vectors, vector_step = 32u % vectors;
      while (row < kMmaRows) {
        const size_t source = (size_t)min(n0 + row, n - 1u) * row_bytes + (size_t)start * 18u + vector * 16u;  // rows past n re-read the last
#pragma unroll
        for (int a = 0; a < NMAT; ++a)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target + (a * kMmaRows + row) * kSlicePitch + vector * 16u),
                       "l"((NMAT == 2 ? p.weight[a] : matrix) + source)
                       : "memory");
        row += row_step;
        vector += vector_step;
        if (vector >= vectors) {
          vector -= vectors;
          ++row;
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  copy_slice(0);  // ahead of the predecessor's results
  copy_slice(1);
  grid_chain_prologue();
  if (my_tiles == 0u) return;

  // the activations of all of K, once
  const uint32_t rows = p.m;
#pragma unroll 2
  for (uint32_t item = threadIdx.x; item < blocks * rows * 4u; item += kMmaWarps * 32) {
    const uint32_t block = rows == 1u ? item >> 2 : (item >> 2) / rows, row = (item >> 2) - block * rows, quad = item & 3u;
    float low_sum, high_sum;
    fragments[(block * p.staged_rows + row) * 4u + quad] = fragment_of(x + (size_t)row * p.k + (size_t)block * 32u + 4u * quad, low_sum, high_sum);
    low_sum += __shfl_xor_sync(0xffffffffu, low_sum, 1);
    low_sum += __shfl_xor_sync(0xffffffffu, low_sum, 2);
    high_sum += __shfl_xor_sync(0xffffffffu, high_sum, 1);
    high_sum += __shfl_xor_sync(0xffffffffu, high_sum, 2);
    if (quad == 0u) bias[block * 8u + row] = -(1032.0f * low_sum + 72.0f * high_sum);
  }
  __syncthreads();

  uint32_t sequence = 0;
  for (uint32_t mine = 0; mine < my_tiles; ++mine) {
    float acc[NMAT][4];
#pragma unroll
    for (int a = 0; a < NMAT; ++a)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[a][i] = 0.0f;
    for (uint32_t span = 0; span < slices; ++span, ++sequence) {
      // this slice has landed: all of this lane's groups but the one after it
      if (sequence + 1u < total) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncwarp();
      const uint32_t start = span * kSliceSpan + first_slice, count = min(kSliceBlocks, blocks - start);
      const uint32_t stage_at = ring_at + (sequence & 1u) * kStageBytes;
      for (uint32_t pair = 0; 2u * pair < count; ++pair) {
        const uint32_t block = start + 2u * pair;  // of the row: what the fragments are indexed by
        block_pair_step<NMAT, kSlicePitch>(stage_at, pair, fragments_at + ((block * p.staged_rows + r) * 4u + c) * 16u, p.staged_rows * 64u,
                              bias_at + (block * 8u + 2u * c) * 4u, r < rows, r, c, acc);
      }
      __syncwarp();  // every lane is done with the stage
      copy_slice(sequence + 2u);
    }
    // the tile is summed: the eight warps' parts meet in shared memory, thread (row, column) adds them in warp order
    uint32_t which, n, n0;
    locate(blockIdx.x + mine * gridDim.x, which, n, n0);
#pragma unroll
    for (int a = 0; a < NMAT; ++a) {
      float* part = reduction + ((a * kMmaWarps + warp) * kMmaRows) * 8u;
      *reinterpret_cast<float2*>(part + r * 8u + 2u * c) = make_float2(acc[a][0], acc[a][1]);
      *reinterpret_cast<float2*>(part + (r + 8u) * 8u + 2u * c) = make_float2(acc[a][2], acc[a][3]);
    }
    __syncthreads();
    if (threadIdx.x < kMmaRows * 8) {
      const uint32_t row = threadIdx.x >> 3, batch_row = threadIdx.x & 7u, column = n0 + row;
      float value[NMAT];
#pragma unroll
      for (int a = 0; a < NMAT; ++a) {
        value[a] = 0.0f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) value[a] += reduction[((a * kMmaWarps + w) * kMmaRows + row) * 8u + batch_row];
      }
      if (batch_row < p.m && column < n) {
        if (NMAT == 2) {
          p.out[0][(size_t)batch_row * n + column] = gated_product(value[0], value[NMAT - 1], p.mode);
        } else {
          __half* out = which == 0u ? p.out[0] : which == 1u ? p.out[1] : p.out[2];
          if (p.out_f32 != nullptr) {
            p.out_f32[(size_t)batch_row * n + column] = value[0];
          } else {
            if (p.mode == 1) value[0] += __half2float(p.additive[column]);
            if (p.mode == 2) value[0] += __half2float(p.additive[(size_t)batch_row * n + column]);
            out[(size_t)batch_row * n + column] = __float2half_rn(value[0]);
          }
        }
      }
    }
    __syncthreads();  // the reduction area may be overwritten
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// The tensor-core form takes rows of whole 16-byte vectors (K a multiple of 256) on 16-byte boundaries.
// LLMOPT_CUDA_Q4_0_MMA=0 keeps every launch on the general kernels.
bool mma_form_ok(uint32_t k, std::initializer_list<const void*> weights) {
  static const bool allowed = getenv("LLMOPT_CUDA_Q4_0_MMA") == nullptr || getenv("LLMOPT_CUDA_Q4_0_MMA")[0] != '0';
  if (!allowed || k % 256u != 0u) return false;
  for (const void* weight : weights)
    if (((uintptr_t)weight & 15u) != 0) return false;
  return true;
}

// Launches the tensor-core form over all rows (passes of up to 32); false when the device refuses the shared memory.
template <int NMAT>
bool launch_mma_form(const KernelArgs& args, const __half* x, MmaProblem p, uint32_t tiles) {
  const uint32_t m = p.m;
  p.tiles_total = tiles;
  // up to 8 rows whose fragments of all of K fit beside the copy buffers: the stream form, a few CTAs per SM
  static const bool stream_allowed = getenv("LLMOPT_CUDA_Q4_0_STREAM") == nullptr || getenv("LLMOPT_CUDA_Q4_0_STREAM")[0] != '0';
  if (stream_allowed && m <= 8u && args.ctx != nullptr) {
    p.staged_rows = m;
    const size_t shared = stream_shared_bytes<NMAT>(p.k >> 5, p.staged_rows);
    // two CTAs per SM where they fit, else one (still ahead of the one-shot form at 4 and 8 rows, level with it at K = 14336)
    const uint32_t resident = shared * 2u <= (size_t)(220u << 10) ? 2u : 1u;
    if (shared <= (size_t)(200u << 10)) {
      auto kernel = q4_0_mma_stream_kernel<NMAT>;
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200u << 10)) == cudaSuccess) {
        const uint32_t ctas = min(tiles, resident * (uint32_t)context_sm_count(args.ctx));
        launch_kernel(args, kernel, dim3(ctas), dim3(kMmaWarps * 32), shared, x, p);
        return true;
      }
      cudaGetLastError();
    }
  }
  p.chunk_buffers = (p.k >> 5) > kChunkBlocks ? 2u : 1u;
  p.staged_rows = m < 8u ? m : 8u;
  const size_t shared = mma_shared_bytes<NMAT>(p.chunk_buffers, p.staged_rows);
  auto kernel = m <= 8u ? q4_0_mma_kernel<NMAT, 1> : q4_0_mma_kernel<NMAT, kMaxRowTiles>;
  if (shared > (48u << 10) &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_shared_bytes<NMAT>(2, 8)) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  for (uint32_t row0 = 0; row0 < m; row0 += 8u * kMaxRowTiles) {
    MmaProblem pass = p;
    pass.m = min(m - row0, 8u * (uint32_t)kMaxRowTiles);
    for (uint32_t i = 0; i < 3; ++i)
      if (pass.out[i] != nullptr) pass.out[i] += (size_t)row0 * p.n[i];
    if (NMAT == 1 && p.mode == 2 && pass.additive != nullptr) pass.additive += (size_t)row0 * p.n[0];
    if (pass.out_f32 != nullptr) pass.out_f32 += (size_t)row0 * p.n[0];
    launch_kernel(args, kernel, dim3(tiles), dim3(kMmaWarps * 32), shared, x + (size_t)row0 * p.k, pass);
  }
  return true;
}

bool shape_ok(uint32_t k, const void* x) { return k > 0 && k % 32 == 0 && ((uintptr_t)x & 15u) == 0 && k % 8 == 0; }

}  // namespace

// Buffers [input, weight, additive, output]; params {m, n, k, epilogue_mode}.
template <int FORMAT>
static int launch_quant_linear(const KernelArgs& args) {
  QuantLinearParams p;
  LLMOPT_REQUIRE(args.buffer_count == 4 && args.param_bytes == sizeof(p), "expects 4 buffers and 16 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.m > 0 && p.n > 0 && shape_ok(p.k, args.buffers[0]), "needs m, n > 0, k a multiple of 32, aligned input");
  LLMOPT_REQUIRE(p.mode <= 2, "epilogue mode must be 0, 1 or 2");
  LLMOPT_REQUIRE(FORMAT == kQ4_0 || ((uintptr_t)args.buffers[1] & 3u) == 0, "affine weight blocks must be 4-byte aligned");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)p.m * p.k * 2 && args.lengths[1] >= (size_t)p.n * (p.k / 32) * kBlockBytes<FORMAT> &&
                     args.lengths[3] >= (size_t)p.m * p.n * 2, "buffer is too short");
  if (p.mode == 1) LLMOPT_REQUIRE(args.lengths[2] >= (size_t)p.n * 2, "bias buffer is too short");
  if (p.mode == 2) LLMOPT_REQUIRE(args.lengths[2] >= (size_t)p.m * p.n * 2, "residual buffer is too short");
  if (FORMAT == kQ4_0 && mma_form_ok(p.k, {args.buffers[1]})) {
    MmaProblem problem = {};
    problem.m = p.m, problem.k = p.k, problem.mode = p.mode, problem.matrices = 1;
    problem.weight[0] = (const uint8_t*)args.buffers[1];
    problem.out[0] = (__half*)args.buffers[3];
    problem.n[0] = p.n;
    problem.additive = (const __half*)args.buffers[2];
    if (launch_mma_form<1>(args, (const __half*)args.buffers[0], problem, (p.n + kMmaRows - 1) / kMmaRows)) return check_launch(args);
  }
  launch_kernel(args, quant_linear_kernel<FORMAT>, dim3((p.n + 7) / 8), dim3(256), 0, (const __half*)args.buffers[0],
                (const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], (__half*)args.buffers[3], p, (float*)nullptr);
  return check_launch(args);
}

// The unrounded Q4_0 product x W^T as fp32 [m, n], for an epilogue that runs as a kernel of its own
// (the expression epilogues): the tensor-core form where the rows allow it, else the general kernel.
int launch_q4_0_product_f32(const KernelArgs& args, const __half* x, const uint8_t* weight, float* out, uint32_t m, uint32_t n,
                            uint32_t k) {
  if (mma_form_ok(k, {weight})) {
    MmaProblem problem = {};
    problem.m = m, problem.k = k, problem.mode = 0, problem.matrices = 1;
    problem.weight[0] = weight;
    problem.n[0] = n;
    problem.out_f32 = out;
    if (launch_mma_form<1>(args, x, problem, (n + kMmaRows - 1) / kMmaRows)) return check_launch(args);
  }
  const QuantLinearParams p = {m, n, k, 0u};
  launch_kernel(args, quant_linear_kernel<kQ4_0>, dim3((n + 7) / 8), dim3(256), 0, x, weight, (const __half*)nullptr,
                (__half*)nullptr, p, out);
  return check_launch(args);
}
int launch_q4_0_linear(const KernelArgs& args) { return launch_quant_linear<kQ4_0>(args); }
int launch_tile32_affine4_linear(const KernelArgs& args) { return launch_quant_linear<kAffine4>(args); }
int launch_tile32_affine8_linear(const KernelArgs& args) { return launch_quant_linear<kAffine8>(args); }

// Buffers [input, gate_weight, up_weight, product]; params {m, n, k, activation}.
int launch_q4_0_gated_linear(const KernelArgs& args) {
  QuantLinearParams p;
  LLMOPT_REQUIRE(args.buffer_count == 4 && args.param_bytes == sizeof(p), "expects 4 buffers and 16 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.m > 0 && p.n > 0 && shape_ok(p.k, args.buffers[0]), "needs m, n > 0, k a multiple of 32, aligned input");
  const size_t weight_bytes = (size_t)p.n * (p.k / 32) * 18;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)p.m * p.k * 2 && args.lengths[1] >= weight_bytes &&
                     args.lengths[2] >= weight_bytes && args.lengths[3] >= (size_t)p.m * p.n * 2, "buffer is too short");
  if (mma_form_ok(p.k, {args.buffers[1], args.buffers[2]})) {
    MmaProblem problem = {};
    problem.m = p.m, problem.k = p.k, problem.mode = p.mode, problem.matrices = 1;
    problem.weight[0] = (const uint8_t*)args.buffers[1];
    problem.weight[1] = (const uint8_t*)args.buffers[2];
    problem.out[0] = (__half*)args.buffers[3];
    problem.n[0] = p.n;
    if (launch_mma_form<2>(args, (const __half*)args.buffers[0], problem, (p.n + kMmaRows - 1) / kMmaRows)) return check_launch(args);
  }
  launch_kernel(args, q4_0_gated_kernel, dim3((p.n + 7) / 8), dim3(256), 0, (const __half*)args.buffers[0],
                (const uint8_t*)args.buffers[1], (const uint8_t*)args.buffers[2], (__half*)args.buffers[3], p);
  return check_launch(args);
}

// Buffers [input, q_weight, k_weight, v_weight, q_out, k_out, v_out]; params {m, k, n_q, n_k, n_v}.
int launch_q4_0_qkv_linear(const KernelArgs& args) {
  QuantQkvParams p;
  LLMOPT_REQUIRE(args.buffer_count == 7 && args.param_bytes == sizeof(p), "expects 7 buffers and 20 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.m > 0 && p.n_q + p.n_k + p.n_v > 0 && shape_ok(p.k, args.buffers[0]),
                 "needs m > 0, some columns, k a multiple of 32, aligned input");
  const size_t row_bytes = (size_t)(p.k / 32) * 18;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)p.m * p.k * 2 && args.lengths[1] >= p.n_q * row_bytes &&
                     args.lengths[2] >= p.n_k * row_bytes && args.lengths[3] >= p.n_v * row_bytes, "input or weight buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= (size_t)p.m * p.n_q * 2 && args.lengths[5] >= (size_t)p.m * p.n_k * 2 &&
                     args.lengths[6] >= (size_t)p.m * p.n_v * 2, "output buffer is too short");
  const uint32_t columns = p.n_q + p.n_k + p.n_v;
  if (mma_form_ok(p.k, {args.buffers[1], args.buffers[2], args.buffers[3]})) {
    MmaProblem problem = {};
    problem.m = p.m, problem.k = p.k, problem.mode = 0, problem.matrices = 3;
    const uint32_t widths[3] = {p.n_q, p.n_k, p.n_v};
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < 3; ++i) {
      problem.weight[i] = (const uint8_t*)args.buffers[1 + i];
      problem.out[i] = (__half*)args.buffers[4 + i];
      problem.n[i] = widths[i];
      problem.first_tile[i] = tiles;
      tiles += (widths[i] + kMmaRows - 1) / kMmaRows;
    }
    if (launch_mma_form<1>(args, (const __half*)args.buffers[0], problem, tiles)) return check_launch(args);
  }
  launch_kernel(args, q4_0_qkv_kernel, dim3((columns + 7) / 8), dim3(256), 0, (const __half*)args.buffers[0],
                (const uint8_t*)args.buffers[1], (const uint8_t*)args.buffers[2], (const uint8_t*)args.buffers[3],
                (__half*)args.buffers[4], (__half*)args.buffers[5], (__half*)args.buffers[6], p);
  return check_launch(args);
}

// Buffers [blocks, output]; params {total_blocks}.
int launch_q4_0_dequant(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2 && args.param_bytes == 4, "expects 2 buffers and 4 parameter bytes");
  const uint32_t total_blocks = param_u32(args, 0);
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)total_blocks * 18 && args.lengths[1] >= (size_t)total_blocks * 64,
                 "buffer is too short");
  if (total_blocks == 0) return 0;
  launch_kernel(args, q4_0_dequant_kernel, dim3((total_blocks * 32 + 255) / 256), dim3(256), 0,
                (const uint8_t*)args.buffers[0], (__half*)args.buffers[1], total_blocks);
  return check_launch(args);
}

}  // namespace llmopt
