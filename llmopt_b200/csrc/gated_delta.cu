// Gated-delta linear-attention scan and the triangular recurrence that prepares its chunked form.
// Restatements of
//   llmopt_gated_delta_f32_d<W> / llmopt_gated_delta_tm_f16_d<W>   lib/metal_recurrent_source.ml:315-410
//   llmopt_triangular_recurrence_f32                                lib/metal_recurrent_source.ml:271-307
// with the CPU statements lib/cpu.ml:909-976 and :424-460 as the arithmetic contract.
//
// Gated delta, per (batch, head): a W x W state S (zero at the first token) and per token
//   S <- S * exp(gate);  delta_r = (v_r - S_r . k) * beta;  S_r <- S_r + k * delta_r;  out_r = (S_r . q) / sqrt(W)
// Rows of S are independent: one warp owns one row, lane l holds columns l, l + 32, ... in
// registers for the whole scan, and the two dot products per token are warp reductions.  The
// work is a chain of T dependent steps per row; a launch has batch * heads * W rows (warps).
//
// Triangular recurrence, per W x W matrix (W <= 64): for row = start .. stop - 1, the entries
// left of the diagonal become row[c] + sum_{i < row} row[i] * M[i][c], with every product and
// every partial sum rounded to fp32 on its own (the reference marks the product volatile to stop
// fused multiply-adds), in the order i = 0, 1, ... — so results are bit-identical to the CPU
// statement.
#include "common.cuh"

namespace llmopt {
namespace {

struct GatedDeltaParams {  // lib/metal_recurrent_source.ml:333-335
  uint32_t batch, heads, tokens, width;
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

// T: float with head-major vectors [b, h, t, w] (gate, beta [b, h, t]); __half with token-major
// vectors [b, t, h, w] (gate f32, beta f16 [b, t, h]).  Output always token-major f16 [b, t, h, w].
template <typename T, bool TOKEN_MAJOR, int SEGMENTS>
__global__ void __launch_bounds__(128) gated_delta_kernel(const T* __restrict__ query, const T* __restrict__ key,
                                                          const T* __restrict__ value, const float* __restrict__ gate,
                                                          const T* __restrict__ beta, __half* __restrict__ output,
                                                          GatedDeltaParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t state_row = blockIdx.x * 4u + (threadIdx.x >> 5);
  if (state_row >= p.batch * p.heads * p.width) return;
  const uint32_t row = state_row % p.width, head_batch = state_row / p.width;
  const uint32_t head = head_batch % p.heads, batch = head_batch / p.heads;
  float state[SEGMENTS];
#pragma unroll
  for (int s = 0; s < SEGMENTS; ++s) state[s] = 0.0f;
  const float scale = rsqrtf((float)p.width);
  for (uint32_t token = 0; token < p.tokens; ++token) {
    const size_t scalar_index = TOKEN_MAJOR ? ((size_t)batch * p.tokens + token) * p.heads + head
                                            : ((size_t)batch * p.heads + head) * p.tokens + token;
    const size_t vector_base = scalar_index * p.width;
    const float decay = expf(gate[scalar_index]);
    float keys[SEGMENTS];
    float state_dot_key = 0.0f;
#pragma unroll
    for (int s = 0; s < SEGMENTS; ++s) {
      keys[s] = to_float(key[vector_base + s * 32 + lane]);
      state[s] *= decay;
      state_dot_key = fmaf(state[s], keys[s], state_dot_key);
    }
    state_dot_key = warp_sum(state_dot_key);
    const float delta = (to_float(value[vector_base + row]) - state_dot_key) * to_float(beta[scalar_index]);
    float state_dot_query = 0.0f;
#pragma unroll
    for (int s = 0; s < SEGMENTS; ++s) {
      state[s] = fmaf(keys[s], delta, state[s]);
      state_dot_query = fmaf(state[s], to_float(query[vector_base + s * 32 + lane]), state_dot_query);
    }
    state_dot_query = warp_sum(state_dot_query);
    if (lane == 0)
      output[(((size_t)batch * p.tokens + token) * p.heads + head) * p.width + row] = __float2half_rn(state_dot_query * scale);
  }
}

struct TriangularParams {  // :272-274
  uint32_t outer, width, start, stop;
};

__global__ void __launch_bounds__(64) triangular_recurrence_kernel(const float* __restrict__ input,
                                                                   float* __restrict__ output, TriangularParams p) {
  grid_chain_prologue();
  __shared__ float state[64 * 64];
  __shared__ float row_values[64];
  const uint32_t tid = threadIdx.x, elements = p.width * p.width;
  const size_t base = (size_t)blockIdx.x * elements;
  for (uint32_t offset = tid; offset < elements; offset += 64) state[offset] = input[base + offset];
  __syncthreads();
  for (uint32_t row = p.start; row < p.stop; ++row) {
    if (tid < row) row_values[tid] = state[row * p.width + tid];
    __syncthreads();
    if (tid < row) {
      float accumulator = 0.0f;
      for (uint32_t inner = 0; inner < row; ++inner)
        accumulator = __fadd_rn(accumulator, __fmul_rn(row_values[inner], state[inner * p.width + tid]));
      state[row * p.width + tid] = __fadd_rn(row_values[tid], accumulator);
    }
    __syncthreads();
  }
  for (uint32_t offset = tid; offset < elements; offset += 64) output[base + offset] = state[offset];
}

template <typename T, bool TOKEN_MAJOR>
int launch_gated_delta(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 6, "expects buffers [query, key, value, gate, beta, output]");
  LLMOPT_REQUIRE(args.param_bytes == sizeof(GatedDeltaParams), "expects 16 parameter bytes {batch, heads, tokens, width}");
  GatedDeltaParams p;
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.width > 0 && p.width % 32 == 0 && p.width <= 256, "width must be a multiple of 32, at most 256");
  const size_t scalars = (size_t)p.batch * p.heads * p.tokens, vectors = scalars * p.width;
  const size_t rows = (size_t)p.batch * p.heads * p.width;
  if (rows == 0 || p.tokens == 0) return 0;
  for (int i = 0; i < 3; ++i) LLMOPT_REQUIRE(args.lengths[i] >= vectors * sizeof(T), "query / key / value buffer is too short");
  LLMOPT_REQUIRE(args.lengths[3] >= scalars * 4 && args.lengths[4] >= scalars * sizeof(T), "gate / beta buffer is too short");
  LLMOPT_REQUIRE(args.lengths[5] >= vectors * 2, "output buffer is too short");
  const dim3 grid((uint32_t)((rows + 3) / 4)), block(128);
  auto run = [&](auto kernel) {
    launch_kernel(args, kernel, grid, block, 0, (const T*)args.buffers[0], (const T*)args.buffers[1],
                  (const T*)args.buffers[2], (const float*)args.buffers[3], (const T*)args.buffers[4],
                  (__half*)args.buffers[5], p);
  };
  switch (p.width / 32) {
    case 1: run(gated_delta_kernel<T, TOKEN_MAJOR, 1>); break;
    case 2: run(gated_delta_kernel<T, TOKEN_MAJOR, 2>); break;
    case 3: run(gated_delta_kernel<T, TOKEN_MAJOR, 3>); break;
    case 4: run(gated_delta_kernel<T, TOKEN_MAJOR, 4>); break;
    case 5: run(gated_delta_kernel<T, TOKEN_MAJOR, 5>); break;
    case 6: run(gated_delta_kernel<T, TOKEN_MAJOR, 6>); break;
    case 7: run(gated_delta_kernel<T, TOKEN_MAJOR, 7>); break;
    default: run(gated_delta_kernel<T, TOKEN_MAJOR, 8>); break;
  }
  return check_launch(args);
}

}  // namespace

// The width is part of the reference's kernel name (llmopt_gated_delta_f32_d128); every name maps
// to the launcher of its layout, which checks that the parameter block agrees.
int launch_gated_delta_f32(const KernelArgs& args) { return launch_gated_delta<float, false>(args); }
int launch_gated_delta_tm_f16(const KernelArgs& args) { return launch_gated_delta<__half, true>(args); }

// Buffers [input, output] f32 [outer, W, W]; params {outer, width, start, stop}.
int launch_triangular_recurrence(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2 && args.param_bytes == sizeof(TriangularParams),
                 "expects buffers [input, output] and 16 parameter bytes");
  TriangularParams p;
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.width > 0 && p.width <= 64, "unsupported triangular recurrence shape: width must be 1..64");
  LLMOPT_REQUIRE(p.start <= p.stop && p.stop <= p.width, "row range lies outside the matrix");
  const size_t bytes = (size_t)p.outer * p.width * p.width * 4;
  LLMOPT_REQUIRE(args.lengths[0] >= bytes && args.lengths[1] >= bytes, "buffer is too short");
  if (p.outer == 0) return 0;
  launch_kernel(args, triangular_recurrence_kernel, dim3(p.outer), dim3(64), 0, (const float*)args.buffers[0],
                (float*)args.buffers[1], p);
  return check_launch(args);
}

}  // namespace llmopt
