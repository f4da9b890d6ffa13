// The rest of the non-quantised glue a compiled decode list can name around the W4A16 / Q8 hot
// path: the RMS / L2 norm variants, the fused RMS-norm + rotary kernels, casts and the broadcasting
// pointwise kernels.  Restatements of
//   llmopt_rms_norm_{f32_f16,f16}_wf32_simd, ..._f16_wf32_wide            lib/metal_normalization_source.ml:92-190
//   llmopt_rms_norm_add{,_scale}_f16_wf32_{simd,wide}, ..._scale_...      :136-346
//   llmopt_rms_norm_unweighted{,_add}_f16_{simd,wide}                    :348-447
//   llmopt_l2_norm_f16_simd, llmopt_l2_norm_slice_f16_simd               :518-585
//   llmopt_rms_rope_f16_{simd_h64,wf32_simd}                             :594-658
//   llmopt_rms_rope_qk_f16_{simd_h64,wf32_simd}                          :670-757
//   llmopt_cast_{f16_f32,f32_f16,i64_f32}                                lib/metal_tensor_source.ml:905-926
//   llmopt_{add,mul,div}_f16, llmopt_{add,sub,mul}_f32, llmopt_{silu,gelu,sigmoid}_mul_f16,
//   llmopt_mul_f16_f32{,_f16}, llmopt_mul_f32_f16_f16, unary silu / sigmoid / tanh / neg / exp / rsqrt
//                                                                        lib/metal_tensor_source.ml:940-1108
// Rounding points are the reference kernels': sums and the normalisation in fp32, one rounding to
// half for the normalised value, then half-precision add (residual) and an fp32 multiply rounded
// to half (layer scalar), each on its own.  All of them move a few KB: launch-latency bound.
#include "common.cuh"

namespace llmopt {
namespace {

__device__ __forceinline__ float as_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float as_float(float v) { return v; }

__device__ __forceinline__ float block_sum_256(float value, float* partial) {
  value = warp_sum(value);
  if ((threadIdx.x & 31u) == 0) partial[threadIdx.x >> 5] = value;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += partial[i];
  return total;
}

struct NormGeometry {
  uint32_t rows, width;       // output rows and their width
  uint32_t groups;            // slices per input row (1 unless the slice form)
  uint32_t input_width;       // stride of an input row
  uint32_t offset;            // first column of the first slice
  float epsilon;
};

// One CTA of 256 threads per output row.
//   WEIGHT: 0 none, 1 half, 2 float.  ADD: half(normalized + residual).  SCALE: half(float(.) * *scalar).
//   L2: inverse = rsqrt(sum + eps) instead of rsqrt(sum / width + eps).
template <typename IN, int WEIGHT, bool ADD, bool SCALE, bool L2>
__global__ void __launch_bounds__(256) norm_family_kernel(const IN* __restrict__ input, const void* __restrict__ weight,
                                                          const __half* __restrict__ residual,
                                                          const float* __restrict__ layer_scalar,
                                                          __half* __restrict__ output, NormGeometry g) {
  grid_chain_prologue();
  __shared__ float partial[8];
  const uint32_t row = blockIdx.x;
  const size_t input_base = (size_t)(row / g.groups) * g.input_width + g.offset + (size_t)(row % g.groups) * g.width;
  const size_t output_base = (size_t)row * g.width;
  float sum = 0.0f;
  for (uint32_t col = threadIdx.x; col < g.width; col += 256u) {
    const float value = as_float(input[input_base + col]);
    sum = fmaf(value, value, sum);
  }
  sum = block_sum_256(sum, partial);
  const float inverse = L2 ? rsqrtf(sum + g.epsilon) : rsqrtf(sum / (float)g.width + g.epsilon);
  const float scale = SCALE ? *layer_scalar : 1.0f;
  for (uint32_t col = threadIdx.x; col < g.width; col += 256u) {
    float value = as_float(input[input_base + col]) * inverse;
    if (WEIGHT == 1) value *= __half2float(static_cast<const __half*>(weight)[col]);
    if (WEIGHT == 2) value *= static_cast<const float*>(weight)[col];
    __half result = __float2half_rn(value);
    if (ADD) result = __hadd_rn(result, residual[output_base + col]);
    if (SCALE) result = __float2half_rn(__half2float(result) * scale);
    output[output_base + col] = result;
  }
}

struct RmsRopeParams {  // lib/metal_normalization_source.ml:596-599
  uint32_t batches, tokens, heads, width, half_dimension, trig_batches;
  float epsilon;
};
struct RmsRopeQkParams {  // :673-677
  uint32_t batches, tokens, q_heads, k_heads, width, half_dimension, trig_batches;
  float epsilon;
};

// One warp per (batch, head, token) row: RMS norm of the head row, then the rotary embedding in
// half precision (each product and the sum rounded on their own).  Input token-first
// [b, t, heads, w], output head-major [b, heads, t, w].
template <typename W>
__device__ __forceinline__ void rms_rope_row(const __half* __restrict__ input, const W* __restrict__ weight,
                                             const __half* __restrict__ cosine, const __half* __restrict__ sine,
                                             __half* __restrict__ output, size_t input_base, size_t trig_base,
                                             size_t output_base, uint32_t width, uint32_t half_dimension, float epsilon,
                                             uint32_t lane) {
  float sum = 0.0f;
  for (uint32_t col = lane; col < width; col += 32) {
    const float value = __half2float(input[input_base + col]);
    sum = fmaf(value, value, sum);
  }
  sum = warp_sum(sum);
  const float inverse = rsqrtf(sum / (float)width + epsilon);
  for (uint32_t col = lane; col < width; col += 32) {
    const __half normalized = __float2half_rn(__half2float(input[input_base + col]) * inverse * as_float(weight[col]));
    const uint32_t rotated_col = col < half_dimension ? col + half_dimension : col - half_dimension;
    __half rotated = __float2half_rn(__half2float(input[input_base + rotated_col]) * inverse * as_float(weight[rotated_col]));
    if (col < half_dimension) rotated = __hneg(rotated);
    const __half direct = __hmul_rn(normalized, cosine[trig_base + col]);
    const __half turned = __hmul_rn(rotated, sine[trig_base + col]);
    output[output_base + col] = __hadd_rn(direct, turned);
  }
}

template <typename W>
__global__ void rms_rope_kernel(const __half* __restrict__ input, const W* __restrict__ weight,
                                const __half* __restrict__ cosine, const __half* __restrict__ sine,
                                __half* __restrict__ output, RmsRopeParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u, row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= p.batches * p.heads * p.tokens) return;
  const uint32_t batch = row / (p.heads * p.tokens), head_token = row % (p.heads * p.tokens);
  const uint32_t head = head_token / p.tokens, token = head_token % p.tokens;
  const size_t input_base = (((size_t)batch * p.tokens + token) * p.heads + head) * p.width;
  const size_t trig_base = ((size_t)(p.trig_batches == 1 ? 0 : batch) * p.tokens + token) * p.width;
  rms_rope_row(input, weight, cosine, sine, output, input_base, trig_base, (size_t)row * p.width, p.width,
               p.half_dimension, p.epsilon, lane);
}

template <typename W>
__global__ void rms_rope_qk_kernel(const __half* __restrict__ q_input, const W* __restrict__ q_weight,
                                   const __half* __restrict__ k_input, const W* __restrict__ k_weight,
                                   const __half* __restrict__ cosine, const __half* __restrict__ sine,
                                   __half* __restrict__ q_output, __half* __restrict__ k_output, RmsRopeQkParams p) {
  grid_chain_prologue();
  const uint32_t lane = threadIdx.x & 31u, row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= p.batches * (p.q_heads + p.k_heads) * p.tokens) return;
  const uint32_t q_rows = p.batches * p.q_heads * p.tokens;
  const bool is_q = row < q_rows;
  const uint32_t local_row = is_q ? row : row - q_rows, heads = is_q ? p.q_heads : p.k_heads;
  const uint32_t batch = local_row / (heads * p.tokens), head_token = local_row % (heads * p.tokens);
  const uint32_t head = head_token / p.tokens, token = head_token % p.tokens;
  const size_t input_base = (((size_t)batch * p.tokens + token) * heads + head) * p.width;
  const size_t trig_base = ((size_t)(p.trig_batches == 1 ? 0 : batch) * p.tokens + token) * p.width;
  rms_rope_row(is_q ? q_input : k_input, is_q ? q_weight : k_weight, cosine, sine, is_q ? q_output : k_output,
               input_base, trig_base, (size_t)local_row * p.width, p.width, p.half_dimension, p.epsilon, lane);
}

// ---- casts and pointwise ------------------------------------------------------------------

template <typename IN, typename OUT>
__global__ void cast_kernel(const IN* __restrict__ input, OUT* __restrict__ output, uint32_t count) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= count) return;
  if constexpr (sizeof(OUT) == 2) output[gid] = __float2half_rn((float)input[gid]);
  else if constexpr (sizeof(IN) == 2) output[gid] = __half2float(input[gid]);
  else output[gid] = (OUT)input[gid];
}

struct PointwiseParams {  // lib/metal_tensor_source.ml:1007-1011, 136 bytes
  uint32_t count, rank, left_scalar, right_scalar;
  uint32_t output_shape[8], left_shape[8], right_shape[8];
  long long left_i64, right_i64;
  float left_f32, right_f32;
};
static_assert(sizeof(PointwiseParams) == 136, "pointwise parameter block is 136 bytes");

// llmopt_pointwise_offset (:1014-1029): the flat offset of output element `gid` in an operand
// whose size-one axes broadcast.
__device__ __forceinline__ uint32_t pointwise_offset(uint32_t gid, const PointwiseParams& p, bool is_left) {
  uint32_t remaining = gid, offset = 0, stride = 1;
  for (int axis = (int)p.rank - 1; axis >= 0; --axis) {
    const uint32_t output_dimension = p.output_shape[axis];
    const uint32_t coordinate = remaining % output_dimension;
    remaining /= output_dimension;
    const uint32_t input_dimension = is_left ? p.left_shape[axis] : p.right_shape[axis];
    offset += (input_dimension == 1 ? 0 : coordinate) * stride;
    stride *= input_dimension;
  }
  return offset;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.0f + tanhf(fminf(fmaxf(0.7978845608f * (x + 0.044715f * x * x * x), -10.0f), 10.0f)));
}

enum Binary { kAdd, kSub, kMul, kDiv, kSiluMul, kGeluMul, kSigmoidMul };
enum Unary { kNeg, kSilu, kSigmoid, kTanh, kExp, kRsqrt, kCos, kSin, kSoftplus };

// both operands half, result half: arithmetic in half precision, each operation rounded once
template <int OP>
__device__ __forceinline__ __half binary_half(__half l, __half r) {
  switch (OP) {
    case kAdd: return __hadd_rn(l, r);
    case kSub: return __hsub_rn(l, r);
    case kMul: return __hmul_rn(l, r);
    case kDiv: return __float2half_rn(__half2float(l) / __half2float(r));
    case kSiluMul: return __hmul_rn(__float2half_rn(__half2float(l) / (1.0f + expf(-__half2float(l)))), r);
    case kGeluMul: return __hmul_rn(__float2half_rn(gelu_tanh(__half2float(l))), r);
    default: return __hmul_rn(__float2half_rn(1.0f / (1.0f + expf(-__half2float(l)))), r);
  }
}
template <int OP>
__device__ __forceinline__ float binary_float(float l, float r) {
  switch (OP) {
    case kAdd: return __fadd_rn(l, r);
    case kSub: return __fsub_rn(l, r);
    default: return __fmul_rn(l, r);
  }
}

template <int OP>
__global__ void pointwise_f16_kernel(const __half* __restrict__ left, const __half* __restrict__ right,
                                     __half* __restrict__ output, PointwiseParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.count) return;
  const __half l = p.left_scalar ? __float2half_rn(p.left_f32) : left[pointwise_offset(gid, p, true)];
  const __half r = p.right_scalar ? __float2half_rn(p.right_f32) : right[pointwise_offset(gid, p, false)];
  output[gid] = binary_half<OP>(l, r);
}
template <int OP>
__global__ void pointwise_f32_kernel(const float* __restrict__ left, const float* __restrict__ right,
                                     float* __restrict__ output, PointwiseParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.count) return;
  const float l = p.left_scalar ? p.left_f32 : left[pointwise_offset(gid, p, true)];
  const float r = p.right_scalar ? p.right_f32 : right[pointwise_offset(gid, p, false)];
  output[gid] = binary_float<OP>(l, r);
}
// mixed multiplies: float(left) * float(right) in fp32, stored as OUT
template <typename L, typename R, typename OUT>
__global__ void pointwise_mixed_mul_kernel(const L* __restrict__ left, const R* __restrict__ right,
                                           OUT* __restrict__ output, PointwiseParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.count) return;
  const float product = __fmul_rn(as_float(left[pointwise_offset(gid, p, true)]), as_float(right[pointwise_offset(gid, p, false)]));
  if constexpr (sizeof(OUT) == 2) output[gid] = __float2half_rn(product);
  else output[gid] = product;
}

template <int OP>
__device__ __forceinline__ float unary_float(float v) {
  switch (OP) {
    case kNeg: return -v;
    case kSilu: return v / (1.0f + expf(-v));
    case kSigmoid: return 1.0f / (1.0f + expf(-v));
    case kTanh: return tanhf(v);
    case kExp: return expf(v);
    case kRsqrt: return rsqrtf(v);
    case kCos: return cosf(v);
    case kSin: return sinf(v);
    default: return v > 20.0f ? v : logf(1.0f + expf(v));
  }
}
template <typename T, int OP>
__global__ void unary_kernel(const T* __restrict__ input, T* __restrict__ output, uint32_t count) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= count) return;
  if constexpr (sizeof(T) == 2) output[gid] = OP == kNeg ? __hneg(input[gid]) : __float2half_rn(unary_float<OP>(__half2float(input[gid])));
  else output[gid] = unary_float<OP>(input[gid]);
}

}  // namespace

// ---- launchers --------------------------------------------------------------------------------

// Buffers in the reference's binding order: input, [weight], [residual], [layer scalar], output;
// params {rows, width, epsilon} (12 bytes), or the 24-byte slice block
// {input_rows, groups, width, input_width, offset, epsilon}.
template <typename IN, int WEIGHT, bool ADD, bool SCALE, bool L2, bool SLICE>
int launch_norm_family(const KernelArgs& args) {
  constexpr int kBuffers = 2 + (WEIGHT ? 1 : 0) + (ADD ? 1 : 0) + (SCALE ? 1 : 0);
  LLMOPT_REQUIRE(args.buffer_count == kBuffers, "unexpected buffer count for this norm kernel");
  NormGeometry g;
  if (SLICE) {
    LLMOPT_REQUIRE(args.param_bytes == 24, "expects 24 parameter bytes {input_rows, groups, width, input_width, offset, epsilon}");
    g.groups = param_u32(args, 1);
    g.rows = param_u32(args, 0) * g.groups;
    g.width = param_u32(args, 2);
    g.input_width = param_u32(args, 3);
    g.offset = param_u32(args, 4);
    g.epsilon = param_f32(args, 5);
    LLMOPT_REQUIRE(g.groups > 0 && (size_t)g.offset + (size_t)g.groups * g.width <= g.input_width,
                   "slices lie outside the input row");
  } else {
    LLMOPT_REQUIRE(args.param_bytes == 12, "expects 12 parameter bytes {rows, width, epsilon}");
    g.rows = param_u32(args, 0);
    g.width = param_u32(args, 1);
    g.groups = 1;
    g.input_width = g.width;
    g.offset = 0;
    g.epsilon = param_f32(args, 2);
  }
  if (g.rows == 0 || g.width == 0) return 0;
  int index = 0;
  const size_t input_rows = g.rows / g.groups;
  LLMOPT_REQUIRE(args.lengths[index] >= input_rows * g.input_width * sizeof(IN), "input buffer is too short");
  const IN* input = (const IN*)args.buffers[index++];
  const void* weight = nullptr;
  if (WEIGHT) {
    LLMOPT_REQUIRE(args.lengths[index] >= (size_t)g.width * (WEIGHT == 1 ? 2 : 4), "weight buffer is too short");
    weight = args.buffers[index++];
  }
  const __half* residual = nullptr;
  if (ADD) {
    LLMOPT_REQUIRE(args.lengths[index] >= (size_t)g.rows * g.width * 2, "residual buffer is too short");
    residual = (const __half*)args.buffers[index++];
  }
  const float* scalar = nullptr;
  if (SCALE) {
    LLMOPT_REQUIRE(args.lengths[index] >= 4, "layer scalar buffer is too short");
    scalar = (const float*)args.buffers[index++];
  }
  LLMOPT_REQUIRE(args.lengths[index] >= (size_t)g.rows * g.width * 2, "output buffer is too short");
  launch_kernel(args, norm_family_kernel<IN, WEIGHT, ADD, SCALE, L2>, dim3(g.rows), dim3(256), 0, input, weight,
                residual, scalar, (__half*)args.buffers[index], g);
  return check_launch(args);
}

#define LLMOPT_NORM_LAUNCHER(name, ...) \
  int name(const KernelArgs& args) { return launch_norm_family<__VA_ARGS__>(args); }
LLMOPT_NORM_LAUNCHER(launch_rms_norm_f32_wf32, float, 2, false, false, false, false)
LLMOPT_NORM_LAUNCHER(launch_rms_norm_f16_wf32, __half, 2, false, false, false, false)
LLMOPT_NORM_LAUNCHER(launch_rms_norm_add_f16_wf32, __half, 2, true, false, false, false)
LLMOPT_NORM_LAUNCHER(launch_rms_norm_scale_f16_wf32, __half, 2, false, true, false, false)
LLMOPT_NORM_LAUNCHER(launch_rms_norm_add_scale_f16_wf32, __half, 2, true, true, false, false)
LLMOPT_NORM_LAUNCHER(launch_rms_norm_unweighted_f16, __half, 0, false, false, false, false)
LLMOPT_NORM_LAUNCHER(launch_rms_norm_unweighted_add_f16, __half, 0, true, false, false, false)
LLMOPT_NORM_LAUNCHER(launch_l2_norm_f16, __half, 0, false, false, true, false)
LLMOPT_NORM_LAUNCHER(launch_l2_norm_slice_f16, __half, 0, false, false, true, true)
#undef LLMOPT_NORM_LAUNCHER

// Buffers [input, weight, cosine, sine, output]; params 28 bytes.
template <typename W>
int launch_rms_rope(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 5, "expects buffers [input, weight, cosine, sine, output]");
  LLMOPT_REQUIRE(args.param_bytes == sizeof(RmsRopeParams), "expects 28 parameter bytes");
  RmsRopeParams p;
  memcpy(&p, args.params, sizeof(p));
  const size_t rows = (size_t)p.batches * p.heads * p.tokens;
  if (rows == 0 || p.width == 0) return 0;
  LLMOPT_REQUIRE(p.half_dimension * 2 <= p.width, "half_dimension exceeds half of the width");
  const size_t trig = (size_t)(p.trig_batches == 1 ? 1 : p.batches) * p.tokens * p.width * 2;
  LLMOPT_REQUIRE(args.lengths[0] >= rows * p.width * 2 && args.lengths[4] >= rows * p.width * 2, "input / output buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.width * sizeof(W), "weight buffer is too short");
  LLMOPT_REQUIRE(args.lengths[2] >= trig && args.lengths[3] >= trig, "cosine / sine buffer is too short");
  launch_kernel(args, rms_rope_kernel<W>, dim3((uint32_t)((rows + 7) / 8)), dim3(256), 0, (const __half*)args.buffers[0],
                (const W*)args.buffers[1], (const __half*)args.buffers[2], (const __half*)args.buffers[3],
                (__half*)args.buffers[4], p);
  return check_launch(args);
}
template int launch_rms_rope<__half>(const KernelArgs&);
template int launch_rms_rope<float>(const KernelArgs&);

// Buffers [q_input, q_weight, k_input, k_weight, cosine, sine, q_output, k_output]; params 32 bytes.
template <typename W>
int launch_rms_rope_qk(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 8, "expects buffers [q, q_weight, k, k_weight, cosine, sine, q_out, k_out]");
  LLMOPT_REQUIRE(args.param_bytes == sizeof(RmsRopeQkParams), "expects 32 parameter bytes");
  RmsRopeQkParams p;
  memcpy(&p, args.params, sizeof(p));
  const size_t q_rows = (size_t)p.batches * p.q_heads * p.tokens, k_rows = (size_t)p.batches * p.k_heads * p.tokens;
  if (q_rows + k_rows == 0 || p.width == 0) return 0;
  LLMOPT_REQUIRE(p.half_dimension * 2 <= p.width, "half_dimension exceeds half of the width");
  const size_t trig = (size_t)(p.trig_batches == 1 ? 1 : p.batches) * p.tokens * p.width * 2;
  LLMOPT_REQUIRE(args.lengths[0] >= q_rows * p.width * 2 && args.lengths[6] >= q_rows * p.width * 2, "q buffer is too short");
  LLMOPT_REQUIRE(args.lengths[2] >= k_rows * p.width * 2 && args.lengths[7] >= k_rows * p.width * 2, "k buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.width * sizeof(W) && args.lengths[3] >= (size_t)p.width * sizeof(W),
                 "weight buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= trig && args.lengths[5] >= trig, "cosine / sine buffer is too short");
  launch_kernel(args, rms_rope_qk_kernel<W>, dim3((uint32_t)((q_rows + k_rows + 7) / 8)), dim3(256), 0,
                (const __half*)args.buffers[0], (const W*)args.buffers[1], (const __half*)args.buffers[2],
                (const W*)args.buffers[3], (const __half*)args.buffers[4], (const __half*)args.buffers[5],
                (__half*)args.buffers[6], (__half*)args.buffers[7], p);
  return check_launch(args);
}
template int launch_rms_rope_qk<__half>(const KernelArgs&);
template int launch_rms_rope_qk<float>(const KernelArgs&);

// Buffers [input, output]; params {count}.
template <typename IN, typename OUT>
int launch_cast(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2 && args.param_bytes == 4, "expects buffers [input, output] and 4 parameter bytes");
  const uint32_t count = param_u32(args, 0);
  if (count == 0) return 0;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)count * sizeof(IN) && args.lengths[1] >= (size_t)count * sizeof(OUT), "buffer is too short");
  launch_kernel(args, cast_kernel<IN, OUT>, dim3((count + 255) / 256), dim3(256), 0, (const IN*)args.buffers[0],
                (OUT*)args.buffers[1], count);
  return check_launch(args);
}
template int launch_cast<__half, float>(const KernelArgs&);
template int launch_cast<float, __half>(const KernelArgs&);
template int launch_cast<long long, float>(const KernelArgs&);

namespace {
// Validates a pointwise block against the bound buffers: the operands hold as many elements as
// their (broadcast) shapes say, the output `count`.
template <typename L, typename R, typename OUT>
int check_pointwise(const KernelArgs& args, PointwiseParams* out) {
  LLMOPT_REQUIRE(args.buffer_count == 3, "expects buffers [left, right, output]");
  LLMOPT_REQUIRE(args.param_bytes == sizeof(PointwiseParams), "expects 136 parameter bytes");
  memcpy(out, args.params, sizeof(PointwiseParams));
  const PointwiseParams& p = *out;
  LLMOPT_REQUIRE(p.rank <= 8, "pointwise rank exceeds 8");
  size_t left = 1, right = 1, total = 1;
  for (uint32_t axis = 0; axis < p.rank; ++axis) {
    LLMOPT_REQUIRE(p.output_shape[axis] > 0, "pointwise output shape has an empty axis");
    LLMOPT_REQUIRE((p.left_shape[axis] == 1 || p.left_shape[axis] == p.output_shape[axis]) &&
                       (p.right_shape[axis] == 1 || p.right_shape[axis] == p.output_shape[axis]),
                   "pointwise operand shape does not broadcast to the output shape");
    left *= p.left_shape[axis], right *= p.right_shape[axis], total *= p.output_shape[axis];
  }
  LLMOPT_REQUIRE(p.count <= total, "pointwise count exceeds the output shape");
  LLMOPT_REQUIRE(p.left_scalar || args.lengths[0] >= left * sizeof(L), "left buffer is too short");
  LLMOPT_REQUIRE(p.right_scalar || args.lengths[1] >= right * sizeof(R), "right buffer is too short");
  LLMOPT_REQUIRE(args.lengths[2] >= (size_t)p.count * sizeof(OUT), "output buffer is too short");
  return 0;
}
}  // namespace

template <int OP>
int launch_pointwise_f16(const KernelArgs& args) {
  PointwiseParams p;
  if (int status = check_pointwise<__half, __half, __half>(args, &p)) return status;
  if (p.count == 0) return 0;
  launch_kernel(args, pointwise_f16_kernel<OP>, dim3((p.count + 255) / 256), dim3(256), 0, (const __half*)args.buffers[0],
                (const __half*)args.buffers[1], (__half*)args.buffers[2], p);
  return check_launch(args);
}
template <int OP>
int launch_pointwise_f32(const KernelArgs& args) {
  PointwiseParams p;
  if (int status = check_pointwise<float, float, float>(args, &p)) return status;
  if (p.count == 0) return 0;
  launch_kernel(args, pointwise_f32_kernel<OP>, dim3((p.count + 255) / 256), dim3(256), 0, (const float*)args.buffers[0],
                (const float*)args.buffers[1], (float*)args.buffers[2], p);
  return check_launch(args);
}
template <typename L, typename R, typename OUT>
int launch_pointwise_mixed_mul(const KernelArgs& args) {
  PointwiseParams p;
  if (int status = check_pointwise<L, R, OUT>(args, &p)) return status;
  LLMOPT_REQUIRE(!p.left_scalar && !p.right_scalar, "the mixed multiplies take tensor operands only");
  if (p.count == 0) return 0;
  launch_kernel(args, pointwise_mixed_mul_kernel<L, R, OUT>, dim3((p.count + 255) / 256), dim3(256), 0,
                (const L*)args.buffers[0], (const R*)args.buffers[1], (OUT*)args.buffers[2], p);
  return check_launch(args);
}
template <typename T, int OP>
int launch_unary(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 2 && args.param_bytes == 4, "expects buffers [input, output] and 4 parameter bytes");
  const uint32_t count = param_u32(args, 0);
  if (count == 0) return 0;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)count * sizeof(T) && args.lengths[1] >= (size_t)count * sizeof(T), "buffer is too short");
  launch_kernel(args, unary_kernel<T, OP>, dim3((count + 255) / 256), dim3(256), 0, (const T*)args.buffers[0],
                (T*)args.buffers[1], count);
  return check_launch(args);
}

// name -> launcher table of this file, appended to the registry by the runtime
struct NamedLauncher {
  const char* name;
  Launcher launcher;
};
const NamedLauncher* norm_family_launchers(size_t* count) {
  static const NamedLauncher table[] = {
      {"llmopt_rms_norm_f32_f16_wf32_simd", launch_rms_norm_f32_wf32},
      {"llmopt_rms_norm_f16_wf32_simd", launch_rms_norm_f16_wf32},
      {"llmopt_rms_norm_f16_wf32_wide", launch_rms_norm_f16_wf32},
      {"llmopt_rms_norm_add_f16_wf32_simd", launch_rms_norm_add_f16_wf32},
      {"llmopt_rms_norm_add_f16_wf32_wide", launch_rms_norm_add_f16_wf32},
      {"llmopt_rms_norm_scale_f16_wf32_simd", launch_rms_norm_scale_f16_wf32},
      {"llmopt_rms_norm_scale_f16_wf32_wide", launch_rms_norm_scale_f16_wf32},
      {"llmopt_rms_norm_add_scale_f16_wf32_simd", launch_rms_norm_add_scale_f16_wf32},
      {"llmopt_rms_norm_add_scale_f16_wf32_wide", launch_rms_norm_add_scale_f16_wf32},
      {"llmopt_rms_norm_unweighted_f16_simd", launch_rms_norm_unweighted_f16},
      {"llmopt_rms_norm_unweighted_f16_wide", launch_rms_norm_unweighted_f16},
      {"llmopt_rms_norm_unweighted_add_f16_simd", launch_rms_norm_unweighted_add_f16},
      {"llmopt_rms_norm_unweighted_add_f16_wide", launch_rms_norm_unweighted_add_f16},
      {"llmopt_l2_norm_f16_simd", launch_l2_norm_f16},
      {"llmopt_l2_norm_slice_f16_simd", launch_l2_norm_slice_f16},
      {"llmopt_rms_rope_f16_simd_h64", launch_rms_rope<__half>},
      {"llmopt_rms_rope_f16_wf32_simd", launch_rms_rope<float>},
      {"llmopt_rms_rope_qk_f16_simd_h64", launch_rms_rope_qk<__half>},
      {"llmopt_rms_rope_qk_f16_wf32_simd", launch_rms_rope_qk<float>},
      {"llmopt_cast_f16_f32", launch_cast<__half, float>},
      {"llmopt_cast_f32_f16", launch_cast<float, __half>},
      {"llmopt_cast_i64_f32", launch_cast<long long, float>},
      {"llmopt_add_f16", launch_pointwise_f16<kAdd>},
      {"llmopt_mul_f16", launch_pointwise_f16<kMul>},
      {"llmopt_div_f16", launch_pointwise_f16<kDiv>},
      {"llmopt_silu_mul_f16", launch_pointwise_f16<kSiluMul>},
      {"llmopt_gelu_mul_f16", launch_pointwise_f16<kGeluMul>},
      {"llmopt_sigmoid_mul_f16", launch_pointwise_f16<kSigmoidMul>},
      {"llmopt_add_f32", launch_pointwise_f32<kAdd>},
      {"llmopt_sub_f32", launch_pointwise_f32<kSub>},
      {"llmopt_mul_f32", launch_pointwise_f32<kMul>},
      {"llmopt_mul_f16_f32", launch_pointwise_mixed_mul<__half, float, float>},
      {"llmopt_mul_f16_f32_f16", launch_pointwise_mixed_mul<__half, float, __half>},
      {"llmopt_mul_f32_f16_f16", launch_pointwise_mixed_mul<float, __half, __half>},
      {"llmopt_neg_f16", launch_unary<__half, kNeg>},
      {"llmopt_neg_f32", launch_unary<float, kNeg>},
      {"llmopt_silu_f16", launch_unary<__half, kSilu>},
      {"llmopt_silu_f32", launch_unary<float, kSilu>},
      {"llmopt_sigmoid_f16", launch_unary<__half, kSigmoid>},
      {"llmopt_tanh_f16", launch_unary<__half, kTanh>},
      {"llmopt_exp_f32", launch_unary<float, kExp>},
      {"llmopt_rsqrt_f16", launch_unary<__half, kRsqrt>},
      {"llmopt_rsqrt_f32", launch_unary<float, kRsqrt>},
      {"llmopt_cos_f32", launch_unary<float, kCos>},
      {"llmopt_sin_f32", launch_unary<float, kSin>},
      {"llmopt_softplus_f32", launch_unary<float, kSoftplus>},
  };
  *count = sizeof(table) / sizeof(table[0]);
  return table;
}

}  // namespace llmopt
