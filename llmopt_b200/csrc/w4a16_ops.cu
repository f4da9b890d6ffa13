// Name-level launchers of the W4A16 group-64 family: they decode the
// reference's buffer order and parameter bytes, validate sizes the way the
// reference dispatchers do, and hand the product to the decode GEMV (M < 64
// rows per pass) — see w4a16_gemv.cu.
//
// Reference call sites:
//   dispatch_w4a16_linear              lib/metal_dispatch_linear.ml:938-982
//   dispatch_w4a16_qkv_linear_command  lib/metal_dispatch_linear.ml:398-455
//   dispatch_w4a16_swiglu_ffn_command  lib/metal_dispatch_linear.ml:252-396
//   dispatch_w4a16_lm_head_argmax_command  lib/metal_dispatch_linear.ml:570-721
#include <float.h>

#include "rms_norm.cuh"
#include "w4a16_gemv.cuh"

namespace llmopt {
namespace {

// ---- RMSNorm prologues --------------------------------------------------------

// llmopt_w4a16_swiglu_rms_{f16,f32}_g64, lib/metal_w4a16_source.ml:496-526:
// normalized = half(x * w * rsqrt(mean(x^2) + eps)); one CTA per row.
// LM-head prologue, lib/metal_w4a16_source.ml:1022-1043: the reference keeps the
// normalised row in fp32.  The tensor-core product takes fp16 operands, so the
// fp32 value is carried as an exact-to-2^-22 pair hi = half(v), lo = half(v - hi)
// in "slot" rows: slot tile t holds rows 4t..4t+3 as [hi0..hi3, lo0..lo3].
template <typename T>
__global__ void __launch_bounds__(256) rms_split_rows_kernel(const T* __restrict__ input,
                                                             const __half* __restrict__ weight,
                                                             __half* __restrict__ slots, uint32_t k,
                                                             float epsilon) {
  grid_chain_prologue();
  __shared__ float partial[8];
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  const T* source = input + (size_t)row * k;
  float sum = 0.0f;
  for (uint32_t i = tid; i < k; i += 256) {
    const float value = (float)source[i];
    sum += value * value;
  }
  sum = warp_sum(sum);
  if ((tid & 31u) == 0) partial[tid >> 5] = sum;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += partial[i];
  const float inverse = rsqrtf(total / (float)k + epsilon);
  const uint32_t tile = row / 4, within = row % 4;
  __half* high = slots + ((size_t)tile * 8 + within) * k;
  __half* low = slots + ((size_t)tile * 8 + 4 + within) * k;
  for (uint32_t i = tid; i < k; i += 256) {
    const float value = (float)source[i] * __half2float(weight[i]) * inverse;
    const __half top = __float2half_rn(value);
    high[i] = top;
    low[i] = __float2half_rn(value - __half2float(top));
  }
}

// ---- arg-max over fp32 logits -------------------------------------------------

struct Candidate {  // lib/metal_w4a16_source.ml:1286-1315 {float value; uint index}
  float value;
  uint32_t index;
};
__device__ __forceinline__ bool better(float value, uint32_t index, float best, uint32_t best_index) {
  return value > best || (value == best && index < best_index);
}

// grid (parts, m): part g scans columns g*256 + tid + 256*parts*i; writes
// candidates[row * parts + g] and optionally half logits.
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits,
                                                             Candidate* __restrict__ candidates,
                                                             __half* __restrict__ half_logits, uint32_t n) {
  grid_chain_prologue();
  __shared__ float values[256];
  __shared__ uint32_t indices[256];
  const uint32_t row = blockIdx.y, part = blockIdx.x, parts = gridDim.x, tid = threadIdx.x;
  float best = -FLT_MAX;
  uint32_t best_index = 0;
  for (uint32_t col = part * 256 + tid; col < n; col += parts * 256) {
    const float value = logits[(size_t)row * n + col];
    if (better(value, col, best, best_index)) {
      best = value;
      best_index = col;
    }
    if (half_logits) half_logits[(size_t)row * n + col] = __float2half_rn(value);
  }
  values[tid] = best;
  indices[tid] = best_index;
  __syncthreads();
  for (uint32_t width = 128; width > 0; width >>= 1) {
    if (tid < width && better(values[tid + width], indices[tid + width], values[tid], indices[tid])) {
      values[tid] = values[tid + width];
      indices[tid] = indices[tid + width];
    }
    __syncthreads();
  }
  if (tid == 0) {
    candidates[(size_t)row * parts + part].value = values[0];
    candidates[(size_t)row * parts + part].index = indices[0];
  }
}

// llmopt_w4a16_lm_head_reduce, lib/metal_w4a16_source.ml:1286-1315: best of 256
// candidates per row, ties to the lowest index.
__global__ void __launch_bounds__(256) argmax_reduce_kernel(const Candidate* __restrict__ candidates,
                                                            uint32_t* __restrict__ token_ids, uint32_t parts) {
  grid_chain_prologue();
  __shared__ float values[256];
  __shared__ uint32_t indices[256];
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  float best = -FLT_MAX;
  uint32_t best_index = 0xffffffffu;
  for (uint32_t i = tid; i < parts; i += 256) {
    const Candidate candidate = candidates[(size_t)row * parts + i];
    if (better(candidate.value, candidate.index, best, best_index)) {
      best = candidate.value;
      best_index = candidate.index;
    }
  }
  values[tid] = best;
  indices[tid] = best_index;
  __syncthreads();
  for (uint32_t width = 128; width > 0; width >>= 1) {
    if (tid < width && better(values[tid + width], indices[tid + width], values[tid], indices[tid])) {
      values[tid] = values[tid + width];
      indices[tid] = indices[tid + width];
    }
    __syncthreads();
  }
  if (tid == 0) token_ids[row] = indices[0] == 0xffffffffu ? 0u : indices[0];
}

constexpr uint32_t kCandidateParts = 256;  // candidates per row in the two-stage form

int lm_head_stage(const KernelArgs& args, bool input_f32, const void* input, const __half* norm_weight,
                  const uint8_t* weight, const __half* scale, Candidate* candidates, __half* logits, uint32_t m,
                  uint32_t n, uint32_t k, float epsilon) {
  LLMOPT_REQUIRE(m <= 32, "LM head handles at most 32 rows per dispatch");
  const uint32_t tiles = (m + 3) / 4;
  const size_t slot_bytes = (size_t)tiles * 8 * k * sizeof(__half);
  const size_t logit_bytes = (size_t)m * n * sizeof(float);
  const size_t slot_aligned = (slot_bytes + 255) / 256 * 256;
  uint8_t* scratch = (uint8_t*)context_scratch(args.ctx, slot_aligned + logit_bytes, args.error);
  if (!scratch) return 1;
  __half* slots = (__half*)scratch;
  float* logits_f32 = (float*)(scratch + slot_aligned);
  if (tiles * 8 > m * 2 || (m % 4) != 0)  // unused slot rows must read as zeros
    cudaMemsetAsync(slots, 0, slot_bytes, args.stream);
  if (input_f32)
    launch_kernel(args, rms_split_rows_kernel<float>, dim3(m), dim3(256), 0, (const float*)input, norm_weight, slots, k, epsilon);
  else
    launch_kernel(args, rms_split_rows_kernel<__half>, dim3(m), dim3(256), 0, (const __half*)input, norm_weight, slots, k, epsilon);
  if (int status = check_launch(args)) return status;
  GemvProblem problem = {};
  problem.x = slots;
  problem.x_rows = tiles * 8;
  problem.m = m;
  problem.k = k;
  problem.mat[0] = {weight, scale, nullptr, n};
  problem.matrices = 1;
  problem.out_f32 = logits_f32;
  // At most 16 rows (32 hi/lo slot rows) per launch: that is what the pipelined kernel takes, and two
  // passes over the weights through it beat one pass through the direct-load kernel (batch 32: 583 -> ~500 us).
  if (m > 16u) {
    // 17..32 rows: one pass over the weights on the tensor-core kernel (weights converted into tensor memory)
    problem.x_rows = tiles * 8;
    problem.m = m;
    const int status = launch_w4a16_gemm_tc_batch(args, problem, kEpiSplitF32, false);
    if (status > 0) return status;
    if (status == 0) {
      launch_kernel(args, argmax_partial_kernel, dim3(kCandidateParts, m), dim3(256), 0, logits_f32, candidates, logits, n);
      return check_launch(args);
    }
  }
  for (uint32_t first = 0; first < m; first += 16u) {
    const uint32_t rows = m - first < 16u ? m - first : 16u;
    problem.x = slots + (size_t)(first / 4u) * 8u * k;
    problem.x_rows = ((rows + 3u) / 4u) * 8u;
    problem.m = rows;
    problem.out_f32 = logits_f32 + (size_t)first * n;
    if (int status = launch_w4a16_gemv(args, problem, kEpiSplitF32, false)) return status;
  }
  launch_kernel(args, argmax_partial_kernel, dim3(kCandidateParts, m), dim3(256), 0, logits_f32, candidates, logits, n);
  return check_launch(args);
}

// The plan builder may have folded the norm that produced this dispatch's input into it.
void apply_fused_norm(const KernelArgs& args, GemvProblem* problem) {
  if (args.fused_norm == nullptr) return;
  problem->x = args.fused_norm->input;
  problem->norm_weight = args.fused_norm->weight;
  problem->norm_out = args.fused_norm->normalized;
  problem->norm_epsilon = args.fused_norm->epsilon;
  problem->norm_weight_first = args.fused_norm->weight_first;
}

bool weight_sizes_ok(const KernelArgs& args, int weight_index, int scale_index, uint32_t n, uint32_t k) {
  return args.lengths[weight_index] >= (size_t)n * (k / 2) && args.lengths[scale_index] >= (size_t)n * (k / 64) * 2;
}

}  // namespace

// Buffers [input, packed_weight, scale, bias_or_scale, output]; params u32
// {m, n, k, has_bias, bias_row_stride} (lib/metal_w4a16_source.ml:7). When there
// is no bias the dispatcher binds the scale buffer in the bias position.
// The same launcher serves the _g64, _g64_m4 and _g64_m8 names.
int launch_w4a16_linear(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 5, "expects buffers [input, weight, scale, bias, output]");
  LLMOPT_REQUIRE(args.param_bytes == 20, "expects 20 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  const uint32_t has_bias = param_u32(args, 3), stride = param_u32(args, 4);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs m, n > 0 and k a positive multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 1, 2, n, k), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= (size_t)m * n * 2, "output buffer is too short");
  if (has_bias) LLMOPT_REQUIRE(args.lengths[3] >= ((size_t)(m - 1) * stride + n) * 2, "bias buffer is too short");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = k;
  problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], nullptr, n};
  problem.matrices = 1;
  problem.out[0] = (__half*)args.buffers[4];
  problem.aux0 = (const __half*)args.buffers[3];
  problem.aux_row_stride = stride;
  problem.has_aux = has_bias;
  apply_fused_norm(args, &problem);
  return launch_w4a16_gemv(args, problem, kEpiLinear, false);
}

// Extension for tensor-parallel row splits (no reference counterpart): the same product with the
// fp32 accumulator written unrounded, buffers [input, weight, scale, output f32], params {m, n, k}.
// The ranks' partial sums are added and rounded once by llmopt_tp_exchange_sum_f16.
int launch_w4a16_linear_partial_f32(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 4 && args.param_bytes == 12, "expects 4 buffers and 12 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs m > 0, n > 0 and k a multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 1, 2, n, k), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[3] >= (size_t)m * n * 4, "output buffer is too short");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = k;
  problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], nullptr, n};
  problem.matrices = 1;
  problem.out_f32 = (float*)args.buffers[3];
  if (m > 32) {
    // prompt rows: the tensor-core kernel with the weights in tensor memory writes the fp32 accumulator
    const int status = launch_w4a16_gemm_tc_batch(args, problem, kEpiLinear, false);
    LLMOPT_REQUIRE(status >= 0, "more than 32 rows need K a multiple of 64 and 16-byte aligned operands");
    return status;
  }
  return launch_w4a16_gemv(args, problem, kEpiLinear, false);
}

// Affine variant (unsigned nibbles with an fp16 zero point per group,
// w = (u - z) s): buffers [input, weight, scale, zero, bias, output], same
// parameter block. No counterpart kernel name in the reference; the algebra is
// the reference's Tile32_Affine4 (lib/block_schema.ml:706-741) at group 64.
int launch_w4a16_linear_affine(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 6, "expects buffers [input, weight, scale, zero, bias, output]");
  LLMOPT_REQUIRE(args.param_bytes == 20, "expects 20 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  const uint32_t has_bias = param_u32(args, 3), stride = param_u32(args, 4);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs m, n > 0 and k a positive multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 1, 2, n, k), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[3] >= (size_t)n * (k / 64) * 2, "zero-point buffer is too short");
  LLMOPT_REQUIRE(args.lengths[5] >= (size_t)m * n * 2, "output buffer is too short");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = k;
  problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], (const __half*)args.buffers[3], n};
  problem.matrices = 1;
  problem.out[0] = (__half*)args.buffers[5];
  problem.aux0 = (const __half*)args.buffers[4];
  problem.aux_row_stride = stride;
  problem.has_aux = has_bias;
  return launch_w4a16_gemv(args, problem, kEpiLinear, true);
}

// Buffers [input, qw, qs, kw, ks, vw, vs, q_out, k_out, v_out]; params u32
// {m, k, n_q, n_k, n_v} (lib/metal_dispatch_linear.ml:423-450).
int launch_w4a16_qkv_linear(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 10, "expects 10 buffers [input, 3 x (weight, scale), 3 outputs]");
  LLMOPT_REQUIRE(args.param_bytes == 20, "expects 20 parameter bytes");
  const uint32_t m = param_u32(args, 0), k = param_u32(args, 1);
  const uint32_t n[3] = {param_u32(args, 2), param_u32(args, 3), param_u32(args, 4)};
  LLMOPT_REQUIRE(m > 0 && k > 0 && k % 64 == 0 && n[0] > 0 && n[1] > 0 && n[2] > 0,
                 "needs positive sizes and k a multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = k;
  problem.matrices = 3;
  for (int i = 0; i < 3; ++i) {
    LLMOPT_REQUIRE(weight_sizes_ok(args, 1 + 2 * i, 2 + 2 * i, n[i], k), "weight or scale buffer is too short");
    LLMOPT_REQUIRE(args.lengths[7 + i] >= (size_t)m * n[i] * 2, "output buffer is too short");
    problem.mat[i] = {(const uint8_t*)args.buffers[1 + 2 * i], (const __half*)args.buffers[2 + 2 * i], nullptr, n[i]};
    problem.out[i] = (__half*)args.buffers[7 + i];
  }
  apply_fused_norm(args, &problem);
  return launch_w4a16_gemv(args, problem, kEpiQkv, false);
}

// Buffers [input, norm_weight, normalized]; params {m, n, k, epsilon}
// (lib/metal_parameters.ml:38-50): k is the hidden width.
int launch_w4a16_swiglu_rms_f16(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 3 && args.param_bytes == 16, "expects 3 buffers and 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && k > 0, "needs m, k > 0");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2 && args.lengths[1] >= (size_t)k * 2 &&
                     args.lengths[2] >= (size_t)m * k * 2, "buffer is too short");
  launch_rms_norm_rows<__half, true>(args, (const __half*)args.buffers[0], (const __half*)args.buffers[1],
                                     (__half*)args.buffers[2], m, k, param_f32(args, 3));
  return check_launch(args);
}
int launch_w4a16_swiglu_rms_f32(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 3 && args.param_bytes == 16, "expects 3 buffers and 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && k > 0, "needs m, k > 0");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 4 && args.lengths[1] >= (size_t)k * 2 &&
                     args.lengths[2] >= (size_t)m * k * 2, "buffer is too short");
  launch_rms_norm_rows<float, true>(args, (const float*)args.buffers[0], (const __half*)args.buffers[1],
                                    (__half*)args.buffers[2], m, k, param_f32(args, 3));
  return check_launch(args);
}

// Buffers [normalized, gate_w, gate_s, up_w, up_s, product]; params {m, n, k, eps}:
// product[m, n] = half(silu(x Wg^T) * (x Wu^T)).
int launch_w4a16_dual_swiglu(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 6 && args.param_bytes == 16, "expects 6 buffers and 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs positive sizes and k a multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 1, 2, n, k) && weight_sizes_ok(args, 3, 4, n, k),
                 "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[5] >= (size_t)m * n * 2, "product buffer is too short");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = k;
  problem.matrices = 2;
  problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], nullptr, n};
  problem.mat[1] = {(const uint8_t*)args.buffers[3], (const __half*)args.buffers[4], nullptr, n};
  problem.out[0] = (__half*)args.buffers[5];
  apply_fused_norm(args, &problem);
  return launch_w4a16_gemv(args, problem, kEpiDualSwiglu, false);
}

// Buffers [product, down_w, down_s, residual, output]; params {m, n, k, eps}:
// output[m, k] = half(product Wd^T + residual); the inner width is n.
int launch_w4a16_down_add(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 5 && args.param_bytes == 16, "expects 5 buffers and 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && n % 64 == 0, "needs positive sizes and n a multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * n * 2, "product buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 1, 2, k, n), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[3] >= (size_t)m * k * 2 && args.lengths[4] >= (size_t)m * k * 2,
                 "residual or output buffer is too short");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = n;
  problem.matrices = 1;
  problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], nullptr, k};
  problem.out[0] = (__half*)args.buffers[4];
  problem.aux0 = (const __half*)args.buffers[3];
  problem.aux_row_stride = k;
  problem.has_aux = 1;
  return launch_w4a16_gemv(args, problem, kEpiLinear, false);
}

// Tagged epilogue forms of the m = 1 kernel, lib/metal_parametric_codegen.ml:4-39:
// buffers [input, weight, scale, bias_or_scale, output, <epilogue operands>], the
// operands in Epilogue.inputs order (lib/epilogue.ml:186-215), params as the
// plain linear. One launcher per tag is registered under
// llmopt_w4a16_linear_f16_g64_epi_<tag>.
template <int TAG>
int launch_w4a16_linear_tagged(const KernelArgs& args) {
  constexpr int operands = (TAG == 0 || TAG == 2 || TAG == 3) ? 0 : (TAG >= 7 ? 2 : 1);
  LLMOPT_REQUIRE(args.buffer_count == 5 + operands, "unexpected buffer count for this epilogue");
  LLMOPT_REQUIRE(args.param_bytes == 20, "expects 20 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs m, n > 0 and k a positive multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 1, 2, n, k), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= (size_t)m * n * 2, "output buffer is too short");
  for (int i = 0; i < operands; ++i)
    LLMOPT_REQUIRE(args.lengths[5 + i] >= (size_t)n * 2, "epilogue operand is shorter than n");
  GemvProblem problem = {};
  problem.x = (const __half*)args.buffers[0];
  problem.x_rows = m;
  problem.m = m;
  problem.k = k;
  problem.matrices = 1;
  problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], nullptr, n};
  problem.out[0] = (__half*)args.buffers[4];
  problem.aux0 = operands > 0 ? (const __half*)args.buffers[5] : nullptr;
  problem.aux1 = operands > 1 ? (const __half*)args.buffers[6] : nullptr;
  problem.tag = TAG;
  return launch_w4a16_gemv(args, problem, kEpiTagged, false);
}
template int launch_w4a16_linear_tagged<0>(const KernelArgs&);
template int launch_w4a16_linear_tagged<1>(const KernelArgs&);
template int launch_w4a16_linear_tagged<2>(const KernelArgs&);
template int launch_w4a16_linear_tagged<3>(const KernelArgs&);
template int launch_w4a16_linear_tagged<4>(const KernelArgs&);
template int launch_w4a16_linear_tagged<5>(const KernelArgs&);
template int launch_w4a16_linear_tagged<6>(const KernelArgs&);
template int launch_w4a16_linear_tagged<7>(const KernelArgs&);
template int launch_w4a16_linear_tagged<8>(const KernelArgs&);
template int launch_w4a16_linear_tagged<9>(const KernelArgs&);

// Single-pass LM head: buffers [input, norm_weight, weight, scale, token_ids
// (, logits)]; params {m, n, k, epsilon} (lib/metal_w4a16_source.ml:1006-1141).
template <bool F32, bool EXTRA>
int launch_w4a16_lm_head_argmax(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == (EXTRA ? 6 : 5), "unexpected buffer count");
  LLMOPT_REQUIRE(args.param_bytes == 16, "expects 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs positive sizes and k a multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * (F32 ? 4 : 2) && args.lengths[1] >= (size_t)k * 2,
                 "input or norm weight buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 2, 3, n, k), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= (size_t)m * 4, "token id buffer is too short");
  if (EXTRA) LLMOPT_REQUIRE(args.lengths[5] >= (size_t)m * n * 2, "logits buffer is too short");
  // candidates live in context scratch, after the slot rows and fp32 logits
  const uint32_t tiles = (m + 3) / 4;
  const size_t slot_aligned = ((size_t)tiles * 8 * k * 2 + 255) / 256 * 256;
  const size_t logit_aligned = ((size_t)m * n * 4 + 255) / 256 * 256;
  const size_t total = slot_aligned + logit_aligned + (size_t)m * kCandidateParts * sizeof(Candidate);
  uint8_t* scratch = (uint8_t*)context_scratch(args.ctx, total, args.error);
  if (!scratch) return 1;
  Candidate* candidates = (Candidate*)(scratch + slot_aligned + logit_aligned);
  if (int status = lm_head_stage(args, F32, args.buffers[0], (const __half*)args.buffers[1],
                                 (const uint8_t*)args.buffers[2], (const __half*)args.buffers[3], candidates,
                                 EXTRA ? (__half*)args.buffers[5] : nullptr, m, n, k, param_f32(args, 3)))
    return status;
  launch_kernel(args, argmax_reduce_kernel, dim3(m), dim3(256), 0, candidates, (uint32_t*)args.buffers[4], kCandidateParts);
  return check_launch(args);
}
template int launch_w4a16_lm_head_argmax<false, false>(const KernelArgs&);
template int launch_w4a16_lm_head_argmax<false, true>(const KernelArgs&);
template int launch_w4a16_lm_head_argmax<true, false>(const KernelArgs&);
template int launch_w4a16_lm_head_argmax<true, true>(const KernelArgs&);

// Two-stage form: stage 1 buffers [input, norm_weight, weight, scale, candidates
// (, logits)], candidates = {float, u32} x 256 per row
// (lib/metal_dispatch_linear.ml:640-678); stage 2 is llmopt_w4a16_lm_head_reduce.
template <bool F32, bool EXTRA>
int launch_w4a16_lm_head_stage1(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == (EXTRA ? 6 : 5), "unexpected buffer count");
  LLMOPT_REQUIRE(args.param_bytes == 16, "expects 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs positive sizes and k a multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * (F32 ? 4 : 2) && args.lengths[1] >= (size_t)k * 2,
                 "input or norm weight buffer is too short");
  LLMOPT_REQUIRE(weight_sizes_ok(args, 2, 3, n, k), "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= (size_t)m * kCandidateParts * sizeof(Candidate), "candidate buffer is too short");
  if (EXTRA) LLMOPT_REQUIRE(args.lengths[5] >= (size_t)m * n * 2, "logits buffer is too short");
  return lm_head_stage(args, F32, args.buffers[0], (const __half*)args.buffers[1], (const uint8_t*)args.buffers[2],
                       (const __half*)args.buffers[3], (Candidate*)args.buffers[4],
                       EXTRA ? (__half*)args.buffers[5] : nullptr, m, n, k, param_f32(args, 3));
}
template int launch_w4a16_lm_head_stage1<false, false>(const KernelArgs&);
template int launch_w4a16_lm_head_stage1<false, true>(const KernelArgs&);
template int launch_w4a16_lm_head_stage1<true, false>(const KernelArgs&);
template int launch_w4a16_lm_head_stage1<true, true>(const KernelArgs&);

// Buffers [candidates, token_ids]; params {m}.
int launch_w4a16_lm_head_reduce(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2 && args.param_bytes == 4, "expects 2 buffers and 4 parameter bytes");
  const uint32_t m = param_u32(args, 0);
  LLMOPT_REQUIRE(m > 0, "needs m > 0");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * kCandidateParts * sizeof(Candidate) && args.lengths[1] >= (size_t)m * 4,
                 "buffer is too short");
  launch_kernel(args, argmax_reduce_kernel, dim3(m), dim3(256), 0, (const Candidate*)args.buffers[0], (uint32_t*)args.buffers[1],
                                                   kCandidateParts);
  return check_launch(args);
}

}  // namespace llmopt
