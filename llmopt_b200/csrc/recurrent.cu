// Recurrent-state (gated short convolution) kernels for sm_100a.
// Restatement of lib/metal_recurrent_source.ml:9-269:
//   llmopt_short_conv_f16{,_f32}           depthwise conv1d, channel-major
//   llmopt_short_conv_silu_tm_{f16,f32}    token-major conv + SiLU
//   llmopt_short_conv_step{,_fused}_f16    one decode token, state updated in place
//   llmopt_short_conv_prefill{,_init}_f16  the same recurrence over T tokens
// All arithmetic in fp32, one rounding to half per stored value, as the
// reference kernels do. These move a few KB per call; launch latency is the
// bound, so they stay one thread per output element.
#include "common.cuh"

namespace llmopt {
namespace {

struct ShortConvParams {  // lib/metal_recurrent_source.ml:10-13
  uint32_t batches, channels, input_width, output_width, kernel_width, stride, padding, dilation;
};
struct ShortConvSiluTmParams {  // lib/metal_recurrent_source.ml:67-70
  uint32_t batches, tokens, channels, kernel_width, stride, padding, dilation, output_start;
};

template <typename W>
__global__ void short_conv_kernel(const __half* __restrict__ input, const W* __restrict__ weight,
                                  __half* __restrict__ output, ShortConvParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.batches * p.channels * p.output_width) return;
  const uint32_t position = gid % p.output_width;
  const uint32_t channel = (gid / p.output_width) % p.channels;
  const uint32_t batch = gid / (p.output_width * p.channels);
  float accumulator = 0.0f;
  for (uint32_t tap = 0; tap < p.kernel_width; ++tap) {
    const int source = (int)(position * p.stride) - (int)p.padding + (int)(tap * p.dilation);
    if (source >= 0 && source < (int)p.input_width)
      accumulator += __half2float(input[((size_t)batch * p.channels + channel) * p.input_width + (uint32_t)source]) *
                     (float)weight[channel * p.kernel_width + tap];
  }
  output[gid] = __float2half_rn(accumulator);
}

template <typename W>
__global__ void short_conv_silu_tm_kernel(const __half* __restrict__ input, const W* __restrict__ weight,
                                          __half* __restrict__ output, ShortConvSiluTmParams p) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= p.batches * p.tokens * p.channels) return;
  const uint32_t channel = gid % p.channels;
  const uint32_t token = (gid / p.channels) % p.tokens;
  const uint32_t batch = gid / (p.tokens * p.channels);
  float accumulator = 0.0f;
  for (uint32_t tap = 0; tap < p.kernel_width; ++tap) {
    const int source = (int)((token + p.output_start) * p.stride) - (int)p.padding + (int)(tap * p.dilation);
    if (source >= 0 && source < (int)p.tokens)
      accumulator += __half2float(input[((size_t)batch * p.tokens + (uint32_t)source) * p.channels + channel]) *
                     (float)weight[channel * p.kernel_width + tap];
  }
  // the convolved value is rounded to half before SiLU (lib/metal_recurrent_source.ml:94-96)
  const float value = __half2float(__float2half_rn(accumulator));
  output[gid] = __float2half_rn(value / (1.0f + expf(-value)));
}

__global__ void short_conv_step_kernel(const __half* __restrict__ in_proj, __half* __restrict__ conv_state,
                                       const __half* __restrict__ conv_weight, __half* __restrict__ output,
                                       uint32_t channels) {
  grid_chain_prologue();
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const float x0 = __half2float(in_proj[c]);
  const float x1 = __half2float(in_proj[channels + c]);
  const float x2 = __half2float(in_proj[2 * channels + c]);
  const float g = x0 * x2;
  const float s0 = __half2float(conv_state[c * 3 + 1]);
  const float s1 = __half2float(conv_state[c * 3 + 2]);
  const float s2 = g;
  conv_state[c * 3 + 0] = __float2half_rn(s0);
  conv_state[c * 3 + 1] = __float2half_rn(s1);
  conv_state[c * 3 + 2] = __float2half_rn(s2);
  const float w0 = __half2float(conv_weight[c * 3 + 0]);
  const float w1 = __half2float(conv_weight[c * 3 + 1]);
  const float w2 = __half2float(conv_weight[c * 3 + 2]);
  const float conv_out = s0 * w0 + s1 * w1 + s2 * w2;
  output[c] = __float2half_rn(x1 * conv_out);
}

__global__ void short_conv_prefill_kernel(const __half* __restrict__ in_proj, const __half* __restrict__ conv_weight,
                                          __half* __restrict__ output, __half* __restrict__ state_out,
                                          const __half* __restrict__ state_in, uint32_t tokens, uint32_t channels,
                                          uint32_t has_initial_state) {
  grid_chain_prologue();
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const float w0 = __half2float(conv_weight[c * 3 + 0]);
  const float w1 = __half2float(conv_weight[c * 3 + 1]);
  const float w2 = __half2float(conv_weight[c * 3 + 2]);
  float prev3 = 0.0f, prev2 = 0.0f, prev1 = 0.0f;
  if (has_initial_state != 0 && state_in != nullptr) {
    prev3 = __half2float(state_in[c * 3 + 0]);
    prev2 = __half2float(state_in[c * 3 + 1]);
    prev1 = __half2float(state_in[c * 3 + 2]);
  }
  for (uint32_t t = 0; t < tokens; ++t) {
    const size_t offset = (size_t)t * 3 * channels + c;
    const float x0 = __half2float(in_proj[offset]);
    const float x1 = __half2float(in_proj[offset + channels]);
    const float x2 = __half2float(in_proj[offset + 2 * channels]);
    const float current = x0 * x2;
    const float conv_out = prev2 * w0 + prev1 * w1 + current * w2;
    output[(size_t)t * channels + c] = __float2half_rn(x1 * conv_out);
    prev3 = prev2;
    prev2 = prev1;
    prev1 = current;
  }
  state_out[c * 3 + 0] = __float2half_rn(prev3);
  state_out[c * 3 + 1] = __float2half_rn(prev2);
  state_out[c * 3 + 2] = __float2half_rn(prev1);
}

}  // namespace

// Buffers [input, weight, output]; params 32 bytes (lib/metal_dispatch_recurrent.ml:175-180).
template <bool WEIGHT_F32>
int launch_short_conv(const KernelArgs& args) {
  ShortConvParams p;
  LLMOPT_REQUIRE(args.buffer_count == 3 && args.param_bytes == sizeof(p), "expects 3 buffers and 32 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  const size_t count = (size_t)p.batches * p.channels * p.output_width;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)p.batches * p.channels * p.input_width * 2, "input buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.channels * p.kernel_width * (WEIGHT_F32 ? 4 : 2), "weight buffer is too short");
  LLMOPT_REQUIRE(args.lengths[2] >= count * 2, "output buffer is too short");
  if (count == 0) return 0;
  const uint32_t blocks = (uint32_t)((count + 255) / 256);
  if (WEIGHT_F32)
    launch_kernel(args, short_conv_kernel<float>, dim3(blocks), dim3(256), 0, (const __half*)args.buffers[0], (const float*)args.buffers[1],
                                                              (__half*)args.buffers[2], p);
  else
    launch_kernel(args, short_conv_kernel<__half>, dim3(blocks), dim3(256), 0, (const __half*)args.buffers[0], (const __half*)args.buffers[1],
                                                               (__half*)args.buffers[2], p);
  return check_launch(args);
}
template int launch_short_conv<false>(const KernelArgs&);
template int launch_short_conv<true>(const KernelArgs&);

// Buffers [input, weight, output]; params 32 bytes (lib/metal_dispatch_recurrent.ml:210-217).
template <bool WEIGHT_F32>
int launch_short_conv_silu_tm(const KernelArgs& args) {
  ShortConvSiluTmParams p;
  LLMOPT_REQUIRE(args.buffer_count == 3 && args.param_bytes == sizeof(p), "expects 3 buffers and 32 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  const size_t count = (size_t)p.batches * p.tokens * p.channels;
  LLMOPT_REQUIRE(args.lengths[0] >= count * 2 && args.lengths[2] >= count * 2, "input or output buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)p.channels * p.kernel_width * (WEIGHT_F32 ? 4 : 2), "weight buffer is too short");
  if (count == 0) return 0;
  const uint32_t blocks = (uint32_t)((count + 255) / 256);
  if (WEIGHT_F32)
    launch_kernel(args, short_conv_silu_tm_kernel<float>, dim3(blocks), dim3(256), 0,
        (const __half*)args.buffers[0], (const float*)args.buffers[1], (__half*)args.buffers[2], p);
  else
    launch_kernel(args, short_conv_silu_tm_kernel<__half>, dim3(blocks), dim3(256), 0,
        (const __half*)args.buffers[0], (const __half*)args.buffers[1], (__half*)args.buffers[2], p);
  return check_launch(args);
}
template int launch_short_conv_silu_tm<false>(const KernelArgs&);
template int launch_short_conv_silu_tm<true>(const KernelArgs&);

// Buffers [in_proj [3C], conv_state [C,3] (in/out), conv_weight [C,3], output [C]];
// params {channels} (lib/metal_dispatch_recurrent.ml:91-113).
int launch_short_conv_step(const KernelArgs& args) {
  LLMOPT_REQUIRE(args.buffer_count == 4 && args.param_bytes == 4, "expects 4 buffers and 4 parameter bytes");
  const uint32_t channels = param_u32(args, 0);
  LLMOPT_REQUIRE(channels > 0, "needs channels > 0");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)channels * 6 && args.lengths[1] >= (size_t)channels * 6 &&
                     args.lengths[2] >= (size_t)channels * 6 && args.lengths[3] >= (size_t)channels * 2,
                 "buffer is too short");
  launch_kernel(args, short_conv_step_kernel, dim3((channels + 255) / 256), dim3(256), 0,
      (const __half*)args.buffers[0], (__half*)args.buffers[1], (const __half*)args.buffers[2], (__half*)args.buffers[3],
      channels);
  return check_launch(args);
}

// llmopt_short_conv_prefill_f16: buffers [in_proj, conv_weight, output, state_out
// (, state_in after the parameter slot)]; the _init form binds state_in as the
// fifth buffer (lib/metal_recurrent_source.ml:254-269). params {tokens, channels,
// has_initial_state}.
int launch_short_conv_prefill(const KernelArgs& args) {
  LLMOPT_REQUIRE((args.buffer_count == 4 || args.buffer_count == 5) && args.param_bytes == 12,
                 "expects 4 or 5 buffers and 12 parameter bytes");
  const uint32_t tokens = param_u32(args, 0), channels = param_u32(args, 1), has_initial = param_u32(args, 2);
  LLMOPT_REQUIRE(channels > 0, "needs channels > 0");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)tokens * channels * 6 && args.lengths[1] >= (size_t)channels * 6 &&
                     args.lengths[2] >= (size_t)tokens * channels * 2 && args.lengths[3] >= (size_t)channels * 6,
                 "buffer is too short");
  const __half* state_in = nullptr;
  if (args.buffer_count == 5) {
    LLMOPT_REQUIRE(args.lengths[4] >= (size_t)channels * 6, "initial state buffer is too short");
    state_in = (const __half*)args.buffers[4];
  }
  launch_kernel(args, short_conv_prefill_kernel, dim3((channels + 255) / 256), dim3(256), 0,
      (const __half*)args.buffers[0], (const __half*)args.buffers[1], (__half*)args.buffers[2], (__half*)args.buffers[3],
      state_in, tokens, channels, has_initial);
  return check_launch(args);
}

}  // namespace llmopt
