// Host-side token sampler and the hardware probe of the native boundary.
//
//  * llmopt_cuda_sample_f16: temperature / top-k / min-p / top-p sampling over one row of fp16
//    logits held in HOST memory (the reference samples on the host from the logits it read back),
//    the counterpart of caml_llmopt_sample_f16_native (native/ocaml_metal_stubs.m:2629-2765).  The
//    pick must not depend on which native layer is loaded, so the arithmetic (fp32 weights,
//    expf, the order of the min-p and top-p cuts), the bounded candidate set (a streaming
//    top-k kept in a min-heap of at most 256 entries, ties resolved by the heap's own order) and
//    the generator (xoroshiro128+ seeded from one integer, one draw) follow it exactly.
//  * llmopt_cuda_measure_hardware: median launch-to-completion time of an empty kernel and median
//    copy bandwidth of a device-to-device copy kernel, the counterpart of
//    caml_llmopt_metal_measure_hardware (native/ocaml_metal_stubs.m:477-611).  Read-only with
//    respect to the device: it queries properties and runs two kernels; no clock, power or mode
//    setting is touched.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/llmopt_cuda.h"
#include "common.cuh"

namespace llmopt {

extern thread_local std::string g_last_error;

namespace {

int sampler_fail(int code, const std::string& message) {
  g_last_error = message;
  return code;
}

struct Candidate {
  uint32_t token;
  float logit;
};

// A binary min-heap on `logit` over a fixed array: the root is the smallest kept candidate.
// `settle_down` restores the heap below `index`, preferring the left child on equal logits
// (strict comparisons), `settle_up` lifts a new leaf while it is strictly smaller than its parent.
struct CandidateHeap {
  Candidate item[256];
  int size = 0;

  void settle_down(int index, int limit) {
    for (;;) {
      int least = index;
      const int left = 2 * index + 1, right = left + 1;
      if (left < limit && item[left].logit < item[least].logit) least = left;
      if (right < limit && item[right].logit < item[least].logit) least = right;
      if (least == index) return;
      std::swap(item[index], item[least]);
      index = least;
    }
  }
  void settle_up(int index) {
    while (index > 0) {
      const int parent = (index - 1) / 2;
      if (!(item[index].logit < item[parent].logit)) return;
      std::swap(item[index], item[parent]);
      index = parent;
    }
  }
};

// xoroshiro128+ (Blackman / Vigna), one 64-bit output per call.
uint64_t next_random(uint64_t (&state)[2]) {
  const uint64_t s0 = state[0];
  uint64_t s1 = state[1];
  const uint64_t out = s0 + s1;
  s1 ^= s0;
  state[0] = ((s0 << 24) | (s0 >> 40)) ^ s1 ^ (s1 << 16);
  state[1] = (s1 << 37) | (s1 >> 27);
  return out;
}

__global__ void probe_empty_kernel() {}

__global__ void probe_copy_kernel(const uint4* __restrict__ source, uint4* __restrict__ destination, size_t vectors) {
  for (size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x; index < vectors;
       index += (size_t)gridDim.x * blockDim.x)
    destination[index] = source[index];
}

double median_of(std::vector<double>& samples) {
  std::sort(samples.begin(), samples.end());
  const size_t n = samples.size();
  return n % 2 ? samples[n / 2] : 0.5 * (samples[n / 2 - 1] + samples[n / 2]);
}

}  // namespace
}  // namespace llmopt

using namespace llmopt;

extern "C" int llmopt_cuda_sample_f16(const void* halves, size_t count, double temperature, int top_k, double top_p,
                                      double min_p, uint64_t seed, int64_t* token) {
  if (token == nullptr) return sampler_fail(LLMOPT_CUDA_INVALID_ARGUMENT, "sample_f16: null result pointer");
  *token = 0;
  if (count == 0) return LLMOPT_CUDA_OK;
  if (halves == nullptr) return sampler_fail(LLMOPT_CUDA_INVALID_ARGUMENT, "sample_f16: null logits");
  const __half* logits = static_cast<const __half*>(halves);
  const float temp = (float)temperature, nucleus = (float)top_p, floor_p = (float)min_p;

  // greedy: first maximum of the row, compared as halves
  if (temp <= 0.0001f || top_k == 1) {
    float best = __half2float(logits[0]);
    size_t best_index = 0;
    for (size_t i = 1; i < count; ++i) {
      const float value = __half2float(logits[i]);
      if (value > best) {
        best = value;
        best_index = i;
      }
    }
    *token = (int64_t)best_index;
    return LLMOPT_CUDA_OK;
  }

  // candidate set: the top_k largest (64 when top_k <= 0, at most 256), one streaming pass
  int keep = 64;
  if (top_k > 0 && top_k <= 256) keep = top_k;
  else if (top_k > 256) keep = 256;
  CandidateHeap heap;
  for (size_t i = 0; i < count; ++i) {
    const float value = __half2float(logits[i]);
    if (heap.size < keep) {
      heap.item[heap.size] = {(uint32_t)i, value};
      heap.settle_up(heap.size);
      heap.size += 1;
    } else if (value > heap.item[0].logit) {
      heap.item[0] = {(uint32_t)i, value};
      heap.settle_down(0, keep);
    }
  }
  // pop ascending, fill from the back: descending order
  Candidate ordered[256];
  const int candidates = heap.size;
  for (int i = candidates - 1; i >= 0; --i) {
    ordered[i] = heap.item[0];
    heap.item[0] = heap.item[heap.size - 1];
    heap.size -= 1;
    heap.settle_down(0, heap.size);
  }

  const float top = ordered[0].logit, inverse_temp = 1.0f / temp;
  float weight[256];
  float total = 0.0f;
  for (int i = 0; i < candidates; ++i) {
    weight[i] = expf((ordered[i].logit - top) * inverse_temp);
    total += weight[i];
  }
  int valid = candidates;
  if (floor_p > 0.0f && total > 0.0f) {  // min-p: drop the tail below min_p times the best probability
    const float threshold = weight[0] / total * floor_p;
    float kept_total = 0.0f;
    int kept = 0;
    for (int i = 0; i < candidates; ++i) {
      if (!(weight[i] / total >= threshold)) break;
      kept_total += weight[i];
      kept += 1;
    }
    if (kept > 0) {
      valid = kept;
      total = kept_total;
    }
  }
  if (nucleus > 0.0f && nucleus < 1.0f && total > 0.0f) {  // top-p: the shortest prefix reaching top_p
    float cumulative = 0.0f, prefix_total = 0.0f;
    int cutoff = valid;
    for (int i = 0; i < valid; ++i) {
      cumulative += weight[i] / total;
      prefix_total += weight[i];
      if (cumulative >= nucleus) {
        cutoff = i + 1;
        break;
      }
    }
    valid = cutoff;
    total = prefix_total;
  }

  if (seed == 0)  // unseeded: any value that changes from call to call
    seed = (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count();
  uint64_t state[2] = {seed ^ 0x9E3779B97F4A7C15ull, (seed << 31) | (seed >> 33)};
  if (state[0] == 0 && state[1] == 0) {
    state[0] = 1;
    state[1] = 2;
  }
  const float uniform = (float)(next_random(state) >> 11) * (1.0f / 9007199254740992.0f);
  const float target = uniform * total;
  float running = 0.0f;
  uint32_t chosen = ordered[0].token;
  for (int i = 0; i < valid; ++i) {
    running += weight[i];
    if (running >= target) {
      chosen = ordered[i].token;
      break;
    }
  }
  *token = (int64_t)chosen;
  return LLMOPT_CUDA_OK;
}

extern "C" int llmopt_cuda_measure_hardware(int device, int warmup, int repeats, int64_t bytes, char* name,
                                            size_t name_capacity, int* max_threads_per_block,
                                            double* dispatch_seconds, double* bandwidth_gbps) {
  if (warmup < 0 || repeats <= 0 || bytes < 4096 || bytes % 16 != 0)
    return sampler_fail(LLMOPT_CUDA_INVALID_ARGUMENT,
                        "CUDA hardware probe requires warmup >= 0, repeats > 0, and 16-byte-aligned bytes >= 4096");
  if (device >= 0 && cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return sampler_fail(LLMOPT_CUDA_FAILURE, "CUDA hardware probe could not select the device");
  }
  int current = 0;
  cudaDeviceProp properties;
  if (cudaGetDevice(&current) != cudaSuccess || cudaGetDeviceProperties(&properties, current) != cudaSuccess) {
    cudaGetLastError();
    return sampler_fail(LLMOPT_CUDA_FAILURE, "CUDA hardware probe could not create a device queue");
  }
  cudaStream_t stream = nullptr;
  void *input = nullptr, *output = nullptr;
  cudaEvent_t begin = nullptr, end = nullptr;
  cudaError_t status = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  if (status == cudaSuccess) status = cudaMalloc(&input, (size_t)bytes);
  if (status == cudaSuccess) status = cudaMalloc(&output, (size_t)bytes);
  if (status == cudaSuccess) status = cudaMemsetAsync(input, 0x5a, (size_t)bytes, stream);
  if (status == cudaSuccess) status = cudaEventCreate(&begin);
  if (status == cudaSuccess) status = cudaEventCreate(&end);
  std::vector<double> dispatch_samples, copy_samples;
  const size_t vectors = (size_t)bytes / 16;
  const int threads = std::min(properties.maxThreadsPerBlock, 256);
  const unsigned blocks = (unsigned)std::min<size_t>((vectors + threads - 1) / threads,
                                                     (size_t)properties.multiProcessorCount * 32);
  for (int iteration = 0; status == cudaSuccess && iteration < warmup + repeats; ++iteration) {
    // launch-to-completion round trip of an empty kernel, host clock
    if ((status = cudaStreamSynchronize(stream)) != cudaSuccess) break;
    const auto started = std::chrono::steady_clock::now();
    probe_empty_kernel<<<1, 1, 0, stream>>>();
    status = cudaStreamSynchronize(stream);
    const auto finished = std::chrono::steady_clock::now();
    if (status != cudaSuccess) break;
    // device-to-device copy, device clock
    cudaEventRecord(begin, stream);
    probe_copy_kernel<<<blocks, threads, 0, stream>>>((const uint4*)input, (uint4*)output, vectors);
    cudaEventRecord(end, stream);
    if ((status = cudaStreamSynchronize(stream)) != cudaSuccess) break;
    float copy_ms = 0.0f;
    cudaEventElapsedTime(&copy_ms, begin, end);
    if (iteration >= warmup) {
      dispatch_samples.push_back(std::chrono::duration<double>(finished - started).count());
      copy_samples.push_back((double)copy_ms * 1e-3);
    }
  }
  if (status == cudaSuccess) status = cudaGetLastError();
  if (begin) cudaEventDestroy(begin);
  if (end) cudaEventDestroy(end);
  if (input) cudaFree(input);
  if (output) cudaFree(output);
  if (stream) cudaStreamDestroy(stream);
  if (status != cudaSuccess) {
    cudaGetLastError();
    return sampler_fail(LLMOPT_CUDA_FAILURE, std::string("CUDA hardware probe failed: ") + cudaGetErrorString(status));
  }
  if (name && name_capacity) {
    strncpy(name, properties.name, name_capacity - 1);
    name[name_capacity - 1] = '\0';
  }
  if (max_threads_per_block) *max_threads_per_block = properties.maxThreadsPerBlock;
  if (dispatch_seconds) *dispatch_seconds = median_of(dispatch_samples);
  const double copy_seconds = median_of(copy_samples);
  if (bandwidth_gbps) *bandwidth_gbps = copy_seconds > 0.0 ? 2.0 * (double)bytes / copy_seconds / 1e9 : 0.0;
  return LLMOPT_CUDA_OK;
}
