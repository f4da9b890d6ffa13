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
// One warp per output column: the lanes take the row's blocks round-robin (a warp reads 32 x 18
// contiguous bytes per step), each lane multiplies its block with the 32 matching activations of up
// to four batch rows, fp32 accumulation, one warp reduction per (row, column).  More rows are
// served in tiles of four over the same weight row (which stays in L1).  HBM-bound at M = 1:
// 0.5625 bytes per weight.
#include "common.cuh"

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
                                                           __half* __restrict__ y, QuantLinearParams p) {
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
  launch_kernel(args, quant_linear_kernel<FORMAT>, dim3((p.n + 7) / 8), dim3(256), 0, (const __half*)args.buffers[0],
                (const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], (__half*)args.buffers[3], p);
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
