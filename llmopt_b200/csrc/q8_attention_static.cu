// Paged grouped-Q8 decode attention for callers that must not allocate.
//
// Some hosts of this library cannot let it call cudaMalloc: an inference server
// that has already handed every free byte of HBM to its own KV-cache pool, a
// process running under a fixed device-memory budget, or code on a latency path
// where an allocation (which may synchronise the whole device) is forbidden.
// For them this file offers the split-K flash-decode of q8_attention_split.cu
// with its per-split scratch records held in a file-scope device array instead of
// the context's growable scratch.  The array is part of the loaded module: every
// GPU that loads the library holds kStaticScratchBytes of it until the process
// exits, whether or not this entry point is ever called.
//
// The entry point performs no allocation of any kind (no cudaMalloc / cudaFree,
// no context, no library workspace).  Its first call on a device looks up the
// device address of the array (cudaGetSymbolAddress) and the SM count; make that
// first call before starting any stream capture.  All calls share the one array
// and it keeps whatever the previous call left in it: the kernels rewrite every
// record they later read, so nothing has to be cleared, but two calls whose
// kernels overlap on the GPU (different streams, or several host threads) race
// on it — serialise them.
#include <mutex>

#include "../../include/llmopt_cuda.h"
#include "q8_attention.cuh"

namespace llmopt {

extern thread_local std::string g_last_error;
bool paged_split_supported(const PagedParams& p);

namespace {

// 8 MiB: 2016 split records at head_dim 128 (4160 bytes each), 3971 at head_dim 64 (2112 bytes each).
constexpr size_t kStaticScratchBytes = (size_t)8 << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

constexpr int kMaxDevices = 64;
struct DeviceSetup {
  bool ready = false;
  float* scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
};
DeviceSetup g_devices[kMaxDevices];
std::mutex g_setup_mutex;

int fail_with(int code, const std::string& message) {
  g_last_error = message;
  return code;
}

// Once per device, with that device current: in host code the array's name is only
// a handle, the address a kernel can use comes from cudaGetSymbolAddress.
int setup_current_device(DeviceSetup** out) {
  int device = 0;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess)
    return fail_with(LLMOPT_CUDA_FAILURE, std::string("cudaGetDevice failed: ") + cudaGetErrorString(status));
  if (device < 0 || device >= kMaxDevices)
    return fail_with(LLMOPT_CUDA_FAILURE, "device index is outside the static-scratch table");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  DeviceSetup& setup = g_devices[device];
  if (!setup.ready) {
    void* address = nullptr;
    status = cudaGetSymbolAddress(&address, g_static_scratch);
    if (status != cudaSuccess)
      return fail_with(LLMOPT_CUDA_FAILURE,
                       std::string("cudaGetSymbolAddress(static scratch) failed: ") + cudaGetErrorString(status));
    int sm_count = 0;
    status = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    if (status != cudaSuccess || sm_count <= 0)
      return fail_with(LLMOPT_CUDA_FAILURE, "could not read the SM count of the current device");
    setup.scratch = static_cast<float*>(address);
    setup.sm_count = sm_count;
    setup.ready = true;
  }
  *out = &setup;
  return LLMOPT_CUDA_OK;
}

}  // namespace
}  // namespace llmopt

using namespace llmopt;

extern "C" int llmopt_cuda_attention_q8_paged_static(const void* query, const void* current_key,
                                                     const void* current_value, const void* pool,
                                                     const void* slots, void* output, const void* parameters,
                                                     size_t parameter_bytes, uint32_t slot_batch_stride,
                                                     void* stream) {
  if (!query || !current_key || !current_value || !pool || !slots || !output || !parameters)
    return fail_with(LLMOPT_CUDA_INVALID_ARGUMENT, "static paged attention received a null pointer");
  if (parameter_bytes != sizeof(PagedParams))
    return fail_with(LLMOPT_CUDA_INVALID_ARGUMENT, "static paged attention expects the 64-byte parameter block");
  PagedParams p;
  memcpy(&p, parameters, sizeof(p));
  if (p.batches == 0 || p.query_heads == 0 || p.kv_heads == 0 || p.query_heads % p.kv_heads != 0)
    return fail_with(LLMOPT_CUDA_INVALID_ARGUMENT, "static paged attention: inconsistent head counts");
  const uint32_t q_len = p.query_length == 0 ? 1 : p.query_length;
  if (q_len != 1 || p.mask_batches != 0 || p.window != 0 || p.group_size == 0 || !paged_split_supported(p))
    return fail_with(LLMOPT_CUDA_INVALID_ARGUMENT,
                     "static paged attention handles the decode shape only: one query token, no mask, no window, "
                     "head_dim 64 or 128, group 32 or 64, at most 8 query heads per KV head");
  DeviceSetup* setup = nullptr;
  if (int status = setup_current_device(&setup)) return status;

  const size_t record_bytes = paged_split_record_floats(p.head_dim) * sizeof(float);
  const size_t capacity = kStaticScratchBytes / record_bytes;  // records the array can hold
  const size_t pairs = (size_t)p.batches * p.kv_heads;
  if (pairs > capacity)
    return fail_with(LLMOPT_CUDA_INVALID_ARGUMENT,
                     "static paged attention: batches x kv_heads = " + std::to_string(pairs) +
                         " exceeds the " + std::to_string(capacity) + " split records the " +
                         std::to_string(kStaticScratchBytes >> 20) + " MiB static scratch holds at head_dim " +
                         std::to_string(p.head_dim));
  // as many splits as fill the machine about three times over, bounded by the array
  uint32_t splits = (uint32_t)(((size_t)setup->sm_count * 3 + pairs - 1) / pairs);
  const uint32_t by_length = (p.past_length + 63u) / 64u;
  if (splits > by_length) splits = by_length;
  if (splits > kMaxAttentionSplits) splits = kMaxAttentionSplits;
  if ((size_t)splits > capacity / pairs) splits = (uint32_t)(capacity / pairs);
  if (splits == 0) splits = 1;

  KernelArgs args = {};
  args.ctx = nullptr;
  args.stream = static_cast<cudaStream_t>(stream);
  args.buffer_count = 7;
  args.buffers[0] = const_cast<void*>(query);
  args.buffers[1] = const_cast<void*>(current_key);
  args.buffers[2] = const_cast<void*>(current_value);
  args.buffers[3] = const_cast<void*>(pool);
  args.buffers[4] = const_cast<void*>(slots);
  args.buffers[5] = const_cast<void*>(slots);
  args.buffers[6] = output;
  args.name = "llmopt_cuda_attention_q8_paged_static";
  std::string message;
  args.error = &message;
  if (launch_paged_attention_split_on(args, p, slot_batch_stride, setup->scratch, splits, 0xffffffffu) != 0)
    return fail_with(LLMOPT_CUDA_FAILURE, message);
  return LLMOPT_CUDA_OK;
}
