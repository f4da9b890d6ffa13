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

inline int check_launch(const KernelArgs& args) {
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return fail(args, std::string("launch failed: ") + cudaGetErrorString(status));
  return 0;
}

// ---- device helpers ---------------------------------------------------------
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
