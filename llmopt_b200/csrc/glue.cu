// The few non-quantised kernels a whole decode step needs around the W4A16 /
// Q8 hot path: RMSNorm, rotary embedding of Q and K, embedding row gather,
// token chaining.  Restatements of
//   llmopt_rms_norm_{f16,f32_f16}{,_simd}   lib/metal_normalization_source.ml:14-91
//   llmopt_rotary_qk_f16_simd_h64           lib/metal_normalization_source.ml:765-802
//   llmopt_embedding_f16                    lib/metal_tensor_source.ml:306-320
//   llmopt_chain_token_id                   lib/metal_tensor_source.ml:465-470
// Launch-latency bound (a few KB each); one warp per row, 16-byte accesses
// where the layout allows.
#include "common.cuh"
#include "rms_norm.cuh"

namespace llmopt {
namespace {

struct RotaryQkParams {  // lib/metal_normalization_source.ml:760-763
  uint32_t batches, tokens, q_heads, k_heads, width, half_dimension, trig_batches;
};

// Inputs token-first [b, t, heads, w]; outputs head-major [b, heads, t, w]; the
// products and the sum are rounded to half one by one, as the reference computes
// in half precision.
__global__ void rotary_qk_kernel(const __half* __restrict__ q_input, const __half* __restrict__ k_input,
                                 const __half* __restrict__ cosine, const __half* __restrict__ sine,
                                 __half* __restrict__ q_output, __half* __restrict__ k_output, RotaryQkParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t total_rows = p.batches * (p.q_heads + p.k_heads) * p.tokens;
  if (row >= total_rows) return;
  const uint32_t q_rows = p.batches * p.q_heads * p.tokens;
  const bool is_q = row < q_rows;
  const uint32_t local_row = is_q ? row : row - q_rows;
  const uint32_t heads = is_q ? p.q_heads : p.k_heads;
  const uint32_t batch = local_row / (heads * p.tokens);
  const uint32_t head_token = local_row % (heads * p.tokens);
  const uint32_t head = head_token / p.tokens;
  const uint32_t token = head_token % p.tokens;
  const size_t input_base = (((size_t)batch * p.tokens + token) * heads + head) * p.width;
  const __half* input = is_q ? q_input : k_input;
  __half* output = is_q ? q_output : k_output;
  const uint32_t trig_batch = p.trig_batches == 1 ? 0 : batch;
  const size_t trig_base = ((size_t)trig_batch * p.tokens + token) * p.width;
  const size_t output_base = (size_t)local_row * p.width;
  for (uint32_t col = lane; col < p.width; col += 32) {
    const uint32_t rotated_col = col < p.half_dimension ? col + p.half_dimension : col - p.half_dimension;
    __half rotated = input[input_base + rotated_col];
    if (col < p.half_dimension) rotated = __hneg(rotated);
    // *_rn: each operation rounds on its own, never contracted into an fma
    const __half direct = __hmul_rn(input[input_base + col], cosine[trig_base + col]);
    const __half turned = __hmul_rn(rotated, sine[trig_base + col]);
    output[output_base + col] = __hadd_rn(direct, turned);
  }
}

struct EmbeddingParams {  // lib/metal_tensor_source.ml:237
  uint32_t tokens, vocabulary, width;
};

__global__ void embedding_kernel(const long long* __restrict__ indices, const __half* __restrict__ weight,
                                 __half* __restrict__ output, EmbeddingParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.tokens * p.width) return;
  const uint32_t token = gid / p.width, dimension = gid % p.width;
  const long long index = indices[token];
  output[gid] = (index >= 0 && index < (long long)p.vocabulary)
                    ? weight[(size_t)index * p.width + dimension]
                    : __float2half_rn(0.0f);
}

__global__ void chain_token_kernel(const uint32_t* __restrict__ argmax_in, long long* __restrict__ token_out) {
  grid_chain_prologue();
  if (blockIdx.x == 0 && threadIdx.x == 0) token_out[0] = (long long)argmax_in[0];
}

__global__ void chain_tokens_kernel(const uint32_t* __restrict__ argmax_in, long long* __restrict__ token_out,
                                    uint32_t count) {
  grid_chain_prologue();
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) token_out[i] = (long long)argmax_in[i];
}

__global__ void argmax_f16_kernel(const __half* __restrict__ values, uint32_t count, int* __restrict__ result) {
  grid_chain_prologue();
  // strict '>' keeps the first maximum (native/ocaml_metal_stubs.m:787-794)
  __shared__ float best_values[256];
  __shared__ uint32_t best_indices[256];
  const uint32_t tid = threadIdx.x;
  float best = -INFINITY;
  uint32_t best_index = 0xffffffffu;
  for (uint32_t i = tid; i < count; i += 256) {
    const float value = __half2float(values[i]);
    if (best_index == 0xffffffffu || value > best) {
      best = value;
      best_index = i;
    }
  }
  best_values[tid] = best;
  best_indices[tid] = best_index;
  __syncthreads();
  for (uint32_t width = 128; width > 0; width >>= 1) {
    if (tid < width) {
      const float other = best_values[tid + width];
      const uint32_t other_index = best_indices[tid + width];
      if (other_index != 0xffffffffu &&
          (best_indices[tid] == 0xffffffffu || other > best_values[tid] ||
           (other == best_values[tid] && other_index < best_indices[tid]))) {
        best_values[tid] = other;
        best_indices[tid] = other_index;
      }
    }
    __syncthreads();
  }
  if (tid == 0) *result = best_indices[0] == 0xffffffffu ? 0 : (int)best_indices[0];
}

}  // namespace

void launch_argmax_f16(const __half* values, uint32_t count, int* result, cudaStream_t stream) {
  argmax_f16_kernel<<<1, 256, 0, stream>>>(values, count, result);
}

// Buffers [input, weight, output]; params {rows, width, epsilon} (lib/metal_parameters.ml:24-29).
template <bool INPUT_F32>
int launch_rms_norm(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 3 && args.param_bytes == 12, "expects 3 buffers and 12 parameter bytes");
  const uint32_t rows = param_u32(args, 0), width = param_u32(args, 1);
  LLMOPT_REQUIRE(rows > 0 && width > 0, "needs rows, width > 0");
  const size_t elements = (size_t)rows * width;
  LLMOPT_REQUIRE(args.lengths[0] >= elements * (INPUT_F32 ? 4 : 2) && args.lengths[1] >= (size_t)width * 2 &&
                     args.lengths[2] >= elements * 2, "buffer is too short");
  if (INPUT_F32)
    launch_rms_norm_rows<float, false>(args, (const float*)args.buffers[0], (const __half*)args.buffers[1],
                                       (__half*)args.buffers[2], rows, width, param_f32(args, 2));
  else
    launch_rms_norm_rows<__half, false>(args, (const __half*)args.buffers[0], (const __half*)args.buffers[1],
                                        (__half*)args.buffers[2], rows, width, param_f32(args, 2));
  return check_launch(args);
}
template int launch_rms_norm<false>(const KernelArgs&);
template int launch_rms_norm<true>(const KernelArgs&);

// Buffers [q_in, k_in, cosine, sine, q_out, k_out]; params 28 bytes.
int launch_rotary_qk(const KernelArgs& args) {
  RotaryQkParams p;
  LLMOPT_REQUIRE(args.buffer_count == 6 && args.param_bytes == sizeof(p), "expects 6 buffers and 28 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.width > 0 && p.half_dimension * 2 <= p.width, "invalid rotary geometry");
  const size_t q_elements = (size_t)p.batches * p.tokens * p.q_heads * p.width;
  const size_t k_elements = (size_t)p.batches * p.tokens * p.k_heads * p.width;
  const size_t trig = (size_t)(p.trig_batches == 1 ? 1 : p.batches) * p.tokens * p.width;
  LLMOPT_REQUIRE(args.lengths[0] >= q_elements * 2 && args.lengths[4] >= q_elements * 2, "q buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= k_elements * 2 && args.lengths[5] >= k_elements * 2, "k buffer is too short");
  LLMOPT_REQUIRE(args.lengths[2] >= trig * 2 && args.lengths[3] >= trig * 2, "cosine/sine buffer is too short");
  const uint32_t rows = p.batches * (p.q_heads + p.k_heads) * p.tokens;
  if (rows == 0) return 0;
  launch_kernel(args, rotary_qk_kernel, dim3((rows + 7) / 8), dim3(256), 0,
      (const __half*)args.buffers[0], (const __half*)args.buffers[1], (const __half*)args.buffers[2],
      (const __half*)args.buffers[3], (__half*)args.buffers[4], (__half*)args.buffers[5], p);
  return check_launch(args);
}

// Buffers [indices i64, table f16, output]; params {tokens, vocabulary, width}.
int launch_embedding_f16(const KernelArgs& args) {
  EmbeddingParams p;
  LLMOPT_REQUIRE(args.buffer_count == 3 && args.param_bytes == sizeof(p), "expects 3 buffers and 12 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  const size_t elements = (size_t)p.tokens * p.width;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)p.tokens * 8 && args.lengths[1] >= (size_t)p.vocabulary * p.width * 2 &&
                     args.lengths[2] >= elements * 2, "buffer is too short");
  if (elements == 0) return 0;
  launch_kernel(args, embedding_kernel, dim3((uint32_t)((elements + 255) / 256)), dim3(256), 0,
      (const long long*)args.buffers[0], (const __half*)args.buffers[1], (__half*)args.buffers[2], p);
  return check_launch(args);
}

// Buffers [argmax u32, token i64]; no parameters.
int launch_chain_token_id(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2, "expects 2 buffers");
  LLMOPT_REQUIRE(args.lengths[0] >= 4 && args.lengths[1] >= 8, "buffer is too short");
  launch_kernel(args, chain_token_kernel, dim3(1), dim3(32), 0, (const uint32_t*)args.buffers[0], (long long*)args.buffers[1]);
  return check_launch(args);
}

// Batched form of the token chain (one id per sequence): buffers [argmax u32[n],
// token i64[n]], params {count}. No counterpart in the reference, whose decode
// steps carry one sequence.
int launch_chain_token_ids(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2 && args.param_bytes == 4, "expects 2 buffers and 4 parameter bytes");
  const uint32_t count = param_u32(args, 0);
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)count * 4 && args.lengths[1] >= (size_t)count * 8, "buffer is too short");
  if (count == 0) return 0;
  launch_kernel(args, chain_tokens_kernel, dim3((count + 127) / 128), dim3(128), 0, (const uint32_t*)args.buffers[0],
                                                                     (long long*)args.buffers[1], count);
  return check_launch(args);
}

}  // namespace llmopt
