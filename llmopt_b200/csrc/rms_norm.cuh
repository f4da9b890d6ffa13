// Row-wise RMS normalisation, one CTA of 256 threads per row.
#pragma once
#include "common.cuh"

namespace llmopt {

// Eight consecutive elements as floats (one 16-byte load of halves, two of floats).
__device__ __forceinline__ void load_eight(const __half* source, float (&values)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(source);
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&words[i]));
    values[2 * i] = pair.x;
    values[2 * i + 1] = pair.y;
  }
}
__device__ __forceinline__ void load_eight(const float* source, float (&values)[8]) {
  const float4 low = *reinterpret_cast<const float4*>(source);
  const float4 high = *reinterpret_cast<const float4*>(source + 4);
  values[0] = low.x, values[1] = low.y, values[2] = low.z, values[3] = low.w;
  values[4] = high.x, values[5] = high.y, values[6] = high.z, values[7] = high.w;
}

// output[row, i] = half(input[row, i] * inverse_rms(row) * weight[i]).
// WEIGHT_FIRST chooses the association the respective reference kernel uses:
//   false: (x * inverse) * w   lib/metal_normalization_source.ml (rms_norm simd kernels)
//   true:  (x * w) * inverse   lib/metal_w4a16_source.ml:480-492 (SwiGLU-FFN prologue)
// VECTOR needs width % 8 == 0 and 16-byte aligned rows (32-byte for fp32 input); rows up to
// 4096 wide then stay in registers between the two passes.
template <typename T, bool VECTOR, bool WEIGHT_FIRST>
__global__ void __launch_bounds__(256) rms_norm_row_kernel(const T* __restrict__ input,
                                                           const __half* __restrict__ weight,
                                                           __half* __restrict__ output, uint32_t width,
                                                           float epsilon) {
  grid_chain_prologue();
  __shared__ float partial[8];
  const uint32_t tid = threadIdx.x;
  const T* source = input + (size_t)blockIdx.x * width;
  __half* target = output + (size_t)blockIdx.x * width;
  constexpr int kCached = 2;
  float cache[kCached][8];
  float sum = 0.0f;
  if (VECTOR) {
#pragma unroll
    for (int j = 0; j < kCached; ++j) {
      const uint32_t i = (tid + j * 256u) * 8u;
#pragma unroll
      for (int e = 0; e < 8; ++e) cache[j][e] = 0.0f;
      if (i < width) load_eight(source + i, cache[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum = fmaf(cache[j][e], cache[j][e], sum);
    }
    for (uint32_t i = (tid + kCached * 256u) * 8u; i < width; i += 2048u) {
      float values[8];
      load_eight(source + i, values);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum = fmaf(values[e], values[e], sum);
    }
  } else {
    for (uint32_t i = tid; i < width; i += 256u) {
      const float value = (float)source[i];
      sum = fmaf(value, value, sum);
    }
  }
  sum = warp_sum(sum);
  if ((tid & 31u) == 0) partial[tid >> 5] = sum;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += partial[i];
  const float inverse = rsqrtf(total / (float)width + epsilon);
  auto scaled = [&](float value, float w) {
    return __float2half_rn(WEIGHT_FIRST ? (value * w) * inverse : (value * inverse) * w);
  };
  if (VECTOR) {
    auto store = [&](uint32_t i, const float (&values)[8]) {
      float w[8];
      load_eight(weight + i, w);
      __half2 packed[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) packed[e] = __halves2half2(scaled(values[2 * e], w[2 * e]), scaled(values[2 * e + 1], w[2 * e + 1]));
      *reinterpret_cast<uint4*>(target + i) = *reinterpret_cast<const uint4*>(packed);
    };
#pragma unroll
    for (int j = 0; j < kCached; ++j) {
      const uint32_t i = (tid + j * 256u) * 8u;
      if (i < width) store(i, cache[j]);
    }
    for (uint32_t i = (tid + kCached * 256u) * 8u; i < width; i += 2048u) {
      float values[8];
      load_eight(source + i, values);
      store(i, values);
    }
  } else {
    for (uint32_t i = tid; i < width; i += 256u) target[i] = scaled((float)source[i], __half2float(weight[i]));
  }
}

// Host side: picks the vector form when the geometry allows.
template <typename T, bool WEIGHT_FIRST>
inline void launch_rms_norm_rows(const KernelArgs& args, const T* input, const __half* weight, __half* output,
                                 uint32_t rows, uint32_t width, float epsilon) {
  const bool vector = width % 8 == 0 && ((uintptr_t)input) % (8 * sizeof(T)) == 0 && ((uintptr_t)weight) % 16 == 0 &&
                      ((uintptr_t)output) % 16 == 0;
  if (vector)
    launch_kernel(args, rms_norm_row_kernel<T, true, WEIGHT_FIRST>, dim3(rows), dim3(256), 0, input, weight, output,
                  width, epsilon);
  else
    launch_kernel(args, rms_norm_row_kernel<T, false, WEIGHT_FIRST>, dim3(rows), dim3(256), 0, input, weight, output,
                  width, epsilon);
}

}  // namespace llmopt
