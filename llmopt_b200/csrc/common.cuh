// Shared device/host helpers for the llmopt B200 kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace llmopt {

constexpr int kMaxBuffers = 16;     // native/ocaml_metal_stubs.m:80-96 (record limits)
constexpr int kMaxParamBytes = 256;

struct Context;

// A row-wise RMS normalisation folded, by the plan builder, into the kernel that reads its
// output: that kernel normalises the raw rows itself and one of its CTAs still writes the
// normalised tensor, so the plan's buffers end up exactly as with the two separate kernels.
struct FusedNorm {
  const __half* input;    // un-normalised rows [m, k]
  const __half* weight;   // [k]
  __half* normalized;     // [m, k], what the separate kernel would have written
  float epsilon;
  uint32_t weight_first;  // (x w) inv instead of (x inv) w
};

// One dispatch as the reference's stubs receive it: kernel name already
// resolved to a launcher, buffers in binding order, raw little-endian
// parameter bytes, Metal-style grid (threads) and threadgroup.
struct KernelArgs {
  Context* ctx;
  cudaStream_t stream;
  void* buffers[kMaxBuffers];
  size_t lengths[kMaxBuffers];
  int buffer_count;
  const uint8_t* params;
  size_t param_bytes;
  uint32_t grid[3];
  uint32_t group[3];
  // Device cells holding {past_tokens, checkpoint} for replayed plans; null for
  // immediate dispatch (the values in the parameter block are used then).
  const uint32_t* past_tokens_cell;
  const uint32_t* checkpoint_cell;
  const char* name;
  std::string* error;
  const FusedNorm* fused_norm;  // null unless the plan builder folded a norm into this dispatch
  // null unless the plan builder handed the rotary + cache pack of the new token to this (attention) dispatch
  const struct RotaryPackFusion* rotary_fusion;
};

typedef int (*Launcher)(const KernelArgs&);

// Scratch owned by the context; grows on demand outside graph capture.
void* context_scratch(Context* ctx, size_t bytes, std::string* error);
int context_sm_count(Context* ctx);

inline int fail(const KernelArgs& args, const std::string& message) {
  if (args.error) *args.error = std::string(args.name ? args.name : "kernel") + ": " + message;
  return 1;
}

inline uint32_t param_u32(const KernelArgs& args, size_t index) {
  uint32_t value;
  memcpy(&value, args.params + index * 4, 4);
  return value;
}
inline float param_f32(const KernelArgs& args, size_t index) {
  float value;
  memcpy(&value, args.params + index * 4, 4);
  return value;
}

#define LLMOPT_REQUIRE(cond, msg) \
  do {                            \
    if (!(cond)) return fail(args, msg); \
  } while (0)

// Whether launches of this context may overlap the tail of their predecessor
// (programmatic dependent launch); off with LLMOPT_CUDA_OVERLAP=0.
bool context_overlap(Context* ctx);

// Launch on the dispatch's stream.  With overlap allowed the grid may become
// resident while its predecessor in the stream is still draining; every kernel
// therefore calls grid_dependency_wait() before it touches anything another
// kernel of the stream may write or still read (weights are never written by a
// kernel, so a weight prefetch may run ahead of the wait).
template <typename... Params, typename... Args>
inline void launch_kernel(const KernelArgs& launch, void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared,
                          Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = launch.stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = context_overlap(launch.ctx) ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<Args&&>(args)...);
}

inline int check_launch(const KernelArgs& args) {
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return fail(args, std::string("launch failed: ") + cudaGetErrorString(status));
  return 0;
}

// ---- device helpers ---------------------------------------------------------
// Blocks until every kernel this grid depends on has finished and its writes are
// visible; returns at once for a launch without a programmatic dependency.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel of the stream start its launch; it still waits (above) for
// this grid to finish before it reads what this grid writes.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// The two together: the prologue of a kernel with nothing to do ahead of its inputs.
__device__ __forceinline__ void grid_chain_prologue() {
  grid_launch_dependents();
  grid_dependency_wait();
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

}  // namespace llmopt
