// Device helpers shared by the W4A16 decode kernels.
#pragma once
#include "w4a16_gemv.cuh"

namespace llmopt {
namespace gemv {

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Nibbles (0,4) / (1,5) of the low 16+16 bits pattern of `word` as exact half2
// integers in [-8, 7] (SIGNED: two's complement) or [-8, 7] = u - 8 (unsigned).
template <bool SIGNED>
__device__ __forceinline__ void nibbles_to_half2(uint32_t word, uint32_t& low_pair, uint32_t& high_pair) {
  // (word & mask) ^ constant: the constant carries the fp16 exponent of 1024 and,
  // for two's complement input, flips bit 3 of each nibble (q + 8 = n ^ 8).
  constexpr uint32_t low_constant = SIGNED ? 0x64086408u : 0x64006400u;
  constexpr uint32_t high_constant = SIGNED ? 0x64806480u : 0x64006400u;
  const uint32_t low = lop3_and_xor(word, 0x000F000Fu, low_constant);     // 1024 + (q + 8)
  const uint32_t high = lop3_and_xor(word, 0x00F000F0u, high_constant);   // 1024 + 16 (q + 8)
  low_pair = hsub2_u32(low, 0x64086408u);                                 // - 1032
  high_pair = hfma2_u32(high, 0x2C002C00u, 0xD480D480u);                  // / 16 - 72
}

__device__ __forceinline__ float epilogue_gelu(float acc) {
  float inner = 0.7978845608f * (acc + 0.044715f * acc * acc * acc);
  inner = fminf(fmaxf(inner, -10.0f), 10.0f);
  return 0.5f * acc * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float epilogue_tagged(uint32_t tag, float acc, float first, float second) {
  const float silu = acc * (1.0f / (1.0f + expf(-acc)));
  switch (tag) {
    case 0: return acc;
    case 1: return acc + first;
    case 2: return silu;
    case 3: return epilogue_gelu(acc);
    case 4: return silu * first;
    case 5: return epilogue_gelu(acc) * first;
    case 6: return acc + first;
    case 7: return (acc + first) + second;
    case 8: return silu * first + second;
    default: return epilogue_gelu(acc) * first + second;
  }
}


// Writes the 16 x (8 NT) accumulator tile of one warp: element j of batch tile t is
// (column = local_tile*16 + r + 8*(j>>1), row = t*8 + 2c + (j&1)).
template <int NT, int NMAT, int EPI>
__device__ __forceinline__ void write_tile(const GemvProblem& p, float (&acc)[NMAT][NT][4], uint32_t matrix,
                                           uint32_t local_tile, uint32_t n, uint32_t lane) {
  const uint32_t r = lane >> 2, c = lane & 3u;
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t column = local_tile * 16u + r + ((j & 2) ? 8u : 0u);
      if (EPI == kEpiSplitF32) {
        // slots r<4 of an 8-row tile carry the high halves, r>=4 the low halves
        const float value = acc[0][t][j] + __shfl_xor_sync(0xffffffffu, acc[0][t][j], 2);
        const uint32_t row = t * 4 + 2 * c + (j & 1);
        if (c < 2 && row < p.m && column < n) p.out_f32[(size_t)row * n + column] = value;
        continue;
      }
      const uint32_t row = t * 8 + 2 * c + (j & 1);
      if (row >= p.m || column >= n) continue;
      const float value = acc[0][t][j];
      if (EPI == kEpiLinear) {
        float result = value;
        if (p.has_aux) result += __half2float(p.aux0[(size_t)row * p.aux_row_stride + column]);
        if (p.out_f32)  // unrounded partial sum of a K-split product (tensor-parallel row split)
          p.out_f32[(size_t)row * n + column] = result;
        else
          p.out[0][(size_t)row * n + column] = __float2half_rn(result);
      } else if (EPI == kEpiQkv) {
        p.out[matrix][(size_t)row * n + column] = __float2half_rn(value);
      } else if (EPI == kEpiDualSwiglu) {
        const float gate = value, up = acc[NMAT - 1][t][j];
        const float silu = gate / (1.0f + expf(-gate));
        p.out[0][(size_t)row * n + column] = __float2half_rn(silu * up);
      } else if (EPI == kEpiTagged) {
        const float first = p.aux0 ? __half2float(p.aux0[column]) : 0.0f;
        const float second = p.aux1 ? __half2float(p.aux1[column]) : 0.0f;
        p.out[0][(size_t)row * n + column] = __float2half_rn(epilogue_tagged(p.tag, value, first, second));
      }
    }
}

// The same writeback for ONE accumulator position (batch tile t, register j, lane):
// `value[a]` are the finished sums of the NMAT matrices at that position and
// `partner` the sum at lane ^ 2 (only read by the split-fp32 form).
template <int NT, int NMAT, int EPI>
__device__ __forceinline__ void write_position(const GemvProblem& p, const float (&value)[NMAT], float partner,
                                               uint32_t matrix, uint32_t local_tile, uint32_t n, uint32_t t,
                                               uint32_t j, uint32_t lane) {
  const uint32_t r = lane >> 2, c = lane & 3u;
  const uint32_t column = local_tile * 16u + r + ((j & 2) ? 8u : 0u);
  if (EPI == kEpiSplitF32) {
    const uint32_t row = t * 4 + 2 * c + (j & 1);
    if (c < 2 && row < p.m && column < n) p.out_f32[(size_t)row * n + column] = value[0] + partner;
    return;
  }
  const uint32_t row = t * 8 + 2 * c + (j & 1);
  if (row >= p.m || column >= n) return;
  if (EPI == kEpiLinear) {
    float result = value[0];
    if (p.has_aux) result += __half2float(p.aux0[(size_t)row * p.aux_row_stride + column]);
    if (p.out_f32)
      p.out_f32[(size_t)row * n + column] = result;
    else
      p.out[0][(size_t)row * n + column] = __float2half_rn(result);
  } else if (EPI == kEpiQkv) {
    p.out[matrix][(size_t)row * n + column] = __float2half_rn(value[0]);
  } else if (EPI == kEpiDualSwiglu) {
    const float gate = value[0], up = value[NMAT - 1];
    const float silu = gate / (1.0f + expf(-gate));
    p.out[0][(size_t)row * n + column] = __float2half_rn(silu * up);
  } else if (EPI == kEpiTagged) {
    const float first = p.aux0 ? __half2float(p.aux0[column]) : 0.0f;
    const float second = p.aux1 ? __half2float(p.aux1[column]) : 0.0f;
    p.out[0][(size_t)row * n + column] = __float2half_rn(epilogue_tagged(p.tag, value[0], first, second));
  }
}

}  // namespace gemv
}  // namespace llmopt
