// Tensor-parallel exchange steps over peer memory (one process per GPU, NVLink / NVSwitch).
// The reference has no multi-device path; these kernels implement the one exchange that
// a row-split (K-split) linear and a vocabulary-split LM head need.
//
// Every rank owns one "region" of device memory that its peers map through CUDA IPC:
//   bytes [0, 4)     epoch: number of exchanges this rank has completed (local use only)
//   bytes [4, 8)     CTA arrival counter of the running exchange (local use only)
//   bytes [64, 128)  flags[16]: flags[s] = last epoch announced by rank s (written by rank s)
//   bytes [256, ...) data slots; the host assigns a slot to every exchange of its plan so that
//                    two uses of a slot are at least two exchanges apart
// An exchange on rank r: (1) the kernel before it on the stream has written r's contribution
// into its own slot; (2) one thread per peer makes those writes visible system-wide and
// stores the new epoch into flags[r] of that peer's region; (3) every CTA waits, with a bound,
// until its own region's flags all reach the epoch; (4) it reads all contributions with plain
// loads over NVLink and combines them in rank order, so every rank computes the same bits.
// A slot may be rewritten two exchanges later: by then every peer has announced an epoch that
// it only reaches after it finished reading this one.
// A wait that runs out raises the context's error word; the kernel returns without output.
#include <float.h>

#include <algorithm>

#include "common.cuh"

namespace llmopt {

uint32_t* context_device_error(Context* ctx);

namespace {

constexpr uint32_t kMaxRanks = 8;
constexpr uint32_t kFlagsOffset = 64;
constexpr unsigned long long kWaitNanoseconds = 2000ull * 1000ull * 1000ull;  // a peer may be two seconds late

struct Regions {
  uint8_t* base[kMaxRanks];
};

__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* address) {
  uint32_t value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}
__device__ __forceinline__ unsigned long long global_nanoseconds() {
  unsigned long long now;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
  return now;
}
__device__ __forceinline__ void store_release_system(uint32_t* address, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

// Steps (2) and (3); returns the epoch of this exchange, or 0 after a wait ran out.
__device__ uint32_t announce_and_wait(const Regions& regions, uint32_t ranks, uint32_t rank, uint32_t* error_word) {
  __shared__ uint32_t shared_epoch;
  __shared__ uint32_t failed;
  uint8_t* mine = regions.base[rank];
  if (threadIdx.x == 0) {
    shared_epoch = *reinterpret_cast<volatile uint32_t*>(mine) + 1u;
    failed = 0u;
  }
  __syncthreads();
  const uint32_t epoch = shared_epoch;
  if (blockIdx.x == 0 && threadIdx.x < ranks) {
    __threadfence_system();  // the contribution written by the previous kernel, visible to the peers
    store_release_system(reinterpret_cast<uint32_t*>(regions.base[threadIdx.x] + kFlagsOffset) + rank, epoch);
  }
  if (threadIdx.x < ranks) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + kFlagsOffset) + threadIdx.x;
    const unsigned long long deadline = global_nanoseconds() + kWaitNanoseconds;
    // epochs only grow; the signed difference tolerates the 32-bit wrap
    while ((int32_t)(load_acquire_system(flag) - epoch) < 0) {
      if (global_nanoseconds() > deadline) {
        failed = 1u;
        if (error_word) atomicExch(error_word, 1u);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return failed ? 0u : epoch;
}

// Last CTA to finish publishes the new epoch for the next exchange of this rank.
__device__ void complete_exchange(uint8_t* mine, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* arrivals = reinterpret_cast<uint32_t*>(mine + 4);
    if (atomicAdd(arrivals, 1u) == gridDim.x - 1u) {
      *arrivals = 0u;
      *reinterpret_cast<volatile uint32_t*>(mine) = epoch;
      __threadfence();
    }
  }
}

struct SumParams {
  uint32_t ranks, rank, rows, width, slot_offset, has_residual;
};

// output[row, col] = half(residual[row, col] + sum over ranks (in rank order) of partial_r[row, col])
__global__ void __launch_bounds__(256) exchange_sum_kernel(Regions regions, const __half* __restrict__ residual,
                                                           __half* __restrict__ output, SumParams p,
                                                           uint32_t* error_word) {
  grid_chain_prologue();
  const uint32_t epoch = announce_and_wait(regions, p.ranks, p.rank, error_word);
  if (epoch != 0u) {
    const uint32_t elements = p.rows * p.width;
    for (uint32_t index = (blockIdx.x * 256u + threadIdx.x) * 4u; index < elements; index += gridDim.x * 1024u) {
      // all peers' loads are issued before the first one is used: one NVLink round trip, not one per rank
      float4 parts[kMaxRanks];
#pragma unroll
      for (uint32_t r = 0; r < kMaxRanks; ++r)
        if (r < p.ranks)
          parts[r] = *reinterpret_cast<const float4*>(regions.base[r] + p.slot_offset + (size_t)index * 4u);
      float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (uint32_t r = 0; r < kMaxRanks; ++r)
        if (r < p.ranks) {  // rank order: every rank adds the same numbers in the same order
          sum.x += parts[r].x;
          sum.y += parts[r].y;
          sum.z += parts[r].z;
          sum.w += parts[r].w;
        }
      if (p.has_residual) {
        const __half2* add = reinterpret_cast<const __half2*>(residual + index);
        const float2 low = __half22float2(add[0]), high = __half22float2(add[1]);
        sum.x += low.x;
        sum.y += low.y;
        sum.z += high.x;
        sum.w += high.y;
      }
      __half2* target = reinterpret_cast<__half2*>(output + index);
      target[0] = __floats2half2_rn(sum.x, sum.y);
      target[1] = __floats2half2_rn(sum.z, sum.w);
    }
  }
  complete_exchange(regions.base[p.rank], epoch != 0u ? epoch : *reinterpret_cast<volatile uint32_t*>(regions.base[p.rank]) + 1u);
}

struct RowsParams {
  uint32_t ranks, rank, rows, width, slot_offset, has_residual, slice_offset;
};
__device__ __forceinline__ void rows_of_rank(const RowsParams& p, uint32_t rank, uint32_t& first, uint32_t& last) {
  const uint32_t share = (p.rows + p.ranks - 1u) / p.ranks;
  first = min(rank * share, p.rows);
  last = min(first + share, p.rows);
}

// Prompt rows (many rows per exchange): the sum is a reduce-scatter followed by an all-gather, so that a rank
// reads every partial once for ITS rows only instead of all rows of all ranks.
// Step 1: this rank's share of the rows = half(residual + sum over ranks, in rank order, of the fp32 partials);
// written to `output` and, for the peers, into this rank's own region at `slice_offset` (fp16, same row layout).
__global__ void __launch_bounds__(256) exchange_reduce_rows_kernel(Regions regions, const __half* __restrict__ residual,
                                                                   __half* __restrict__ output, RowsParams p,
                                                                   uint32_t* error_word) {
  grid_chain_prologue();
  const uint32_t epoch = announce_and_wait(regions, p.ranks, p.rank, error_word);
  if (epoch != 0u) {
    uint32_t first, last;
    rows_of_rank(p, p.rank, first, last);
    __half* slice = reinterpret_cast<__half*>(regions.base[p.rank] + p.slice_offset);
    const uint32_t begin = first * p.width, end = last * p.width;
    for (uint32_t index = begin + (blockIdx.x * 256u + threadIdx.x) * 4u; index < end; index += gridDim.x * 1024u) {
      float4 parts[kMaxRanks];
#pragma unroll
      for (uint32_t r = 0; r < kMaxRanks; ++r)
        if (r < p.ranks)
          parts[r] = *reinterpret_cast<const float4*>(regions.base[r] + p.slot_offset + (size_t)index * 4u);
      float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (uint32_t r = 0; r < kMaxRanks; ++r)
        if (r < p.ranks) {
          sum.x += parts[r].x;
          sum.y += parts[r].y;
          sum.z += parts[r].z;
          sum.w += parts[r].w;
        }
      if (p.has_residual) {
        const __half2* add = reinterpret_cast<const __half2*>(residual + index);
        const float2 low = __half22float2(add[0]), high = __half22float2(add[1]);
        sum.x += low.x;
        sum.y += low.y;
        sum.z += high.x;
        sum.w += high.y;
      }
      const __half2 low = __floats2half2_rn(sum.x, sum.y), high = __floats2half2_rn(sum.z, sum.w);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&low);
      packed.y = *reinterpret_cast<const uint32_t*>(&high);
      *reinterpret_cast<uint2*>(output + index) = packed;
      *reinterpret_cast<uint2*>(slice + index) = packed;
    }
  }
  complete_exchange(regions.base[p.rank], epoch != 0u ? epoch : *reinterpret_cast<volatile uint32_t*>(regions.base[p.rank]) + 1u);
}

// Step 2 (its own exchange: the announcement says "my share is written"): the other ranks' shares of the rows,
// copied from their regions into `output`.
__global__ void __launch_bounds__(256) exchange_gather_rows_kernel(Regions regions, __half* __restrict__ output,
                                                                   RowsParams p, uint32_t* error_word) {
  grid_chain_prologue();
  const uint32_t epoch = announce_and_wait(regions, p.ranks, p.rank, error_word);
  if (epoch != 0u) {
    for (uint32_t r = 0; r < p.ranks; ++r) {
      if (r == p.rank) continue;
      uint32_t first, last;
      rows_of_rank(p, r, first, last);
      const __half* slice = reinterpret_cast<const __half*>(regions.base[r] + p.slice_offset);
      const uint32_t begin = first * p.width, end = last * p.width;
      for (uint32_t index = begin + (blockIdx.x * 256u + threadIdx.x) * 8u; index < end; index += gridDim.x * 2048u) {
        if (index + 8u <= end) {
          *reinterpret_cast<uint4*>(output + index) = *reinterpret_cast<const uint4*>(slice + index);
        } else {
          for (uint32_t i = index; i < end; ++i) output[i] = slice[i];
        }
      }
    }
  }
  complete_exchange(regions.base[p.rank], epoch != 0u ? epoch : *reinterpret_cast<volatile uint32_t*>(regions.base[p.rank]) + 1u);
}

struct SumNormParams {
  uint32_t ranks, rank, rows, width, slot_offset, has_residual;
  float epsilon;
  uint32_t weight_first;
};

// The exchange sum followed by the RMS normalisation of the result, one CTA per row:
//   hidden[row]     = half(residual[row] + sum over ranks of partial_r[row])      (as exchange_sum_kernel)
//   normalized[row] = half(hidden * inverse_rms(hidden) * weight)                 (as rms_norm_row_kernel;
//                     weight_first picks (x w) inv over (x inv) w)
// The mean of squares is taken over the ROUNDED hidden values, which is what the separate kernels
// compute.  Rows up to 8192 wide stay in registers between the passes.
// One CTA of 1024 threads per row: a 4096-wide row is one float4 per thread, so all of a row's peer loads
// are one round trip over NVLink (with 256 threads the four vectors of a thread were four trips in a row,
// because the stores to `hidden` between them may alias the regions).
constexpr int kSumNormThreads = 1024;
__global__ void __launch_bounds__(kSumNormThreads) exchange_sum_norm_kernel(Regions regions, const __half* __restrict__ residual,
                                                                __half* __restrict__ hidden,
                                                                const __half* __restrict__ norm_weight,
                                                                __half* __restrict__ normalized, SumNormParams p,
                                                                uint32_t* error_word) {
  grid_chain_prologue();
  __shared__ float partial[kSumNormThreads / 32];
  const uint32_t epoch = announce_and_wait(regions, p.ranks, p.rank, error_word);
  if (epoch != 0u) {
    constexpr int kVectors = 2;  // float4 per thread: 1024 * 2 * 4 = 8192 columns
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float4 values[kVectors];
    float squares = 0.0f;
#pragma unroll
    for (int v = 0; v < kVectors; ++v) {
      const uint32_t column = (tid + v * (uint32_t)kSumNormThreads) * 4u;
      values[v] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (column >= p.width) continue;
      const size_t index = (size_t)row * p.width + column;
      float4 parts[kMaxRanks];
#pragma unroll
      for (uint32_t r = 0; r < kMaxRanks; ++r)
        if (r < p.ranks) parts[r] = *reinterpret_cast<const float4*>(regions.base[r] + p.slot_offset + index * 4u);
      float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (uint32_t r = 0; r < kMaxRanks; ++r)
        if (r < p.ranks) {
          sum.x += parts[r].x;
          sum.y += parts[r].y;
          sum.z += parts[r].z;
          sum.w += parts[r].w;
        }
      if (p.has_residual) {
        const __half2* add = reinterpret_cast<const __half2*>(residual + index);
        const float2 low = __half22float2(add[0]), high = __half22float2(add[1]);
        sum.x += low.x;
        sum.y += low.y;
        sum.z += high.x;
        sum.w += high.y;
      }
      const __half2 low = __floats2half2_rn(sum.x, sum.y), high = __floats2half2_rn(sum.z, sum.w);
      __half2* target = reinterpret_cast<__half2*>(hidden + index);
      target[0] = low;
      target[1] = high;
      const float2 low_f = __half22float2(low), high_f = __half22float2(high);
      values[v] = make_float4(low_f.x, low_f.y, high_f.x, high_f.y);
      squares = fmaf(low_f.x, low_f.x, squares);
      squares = fmaf(low_f.y, low_f.y, squares);
      squares = fmaf(high_f.x, high_f.x, squares);
      squares = fmaf(high_f.y, high_f.y, squares);
    }
    squares = warp_sum(squares);
    if ((tid & 31u) == 0) partial[tid >> 5] = squares;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < kSumNormThreads / 32; ++i) total += partial[i];
    const float inverse = rsqrtf(total / (float)p.width + p.epsilon);
#pragma unroll
    for (int v = 0; v < kVectors; ++v) {
      const uint32_t column = (tid + v * (uint32_t)kSumNormThreads) * 4u;
      if (column >= p.width) continue;
      const __half2* weights = reinterpret_cast<const __half2*>(norm_weight + column);
      const float2 w_low = __half22float2(weights[0]), w_high = __half22float2(weights[1]);
      float4 y;
      if (p.weight_first) {
        y = make_float4((values[v].x * w_low.x) * inverse, (values[v].y * w_low.y) * inverse,
                        (values[v].z * w_high.x) * inverse, (values[v].w * w_high.y) * inverse);
      } else {
        y = make_float4((values[v].x * inverse) * w_low.x, (values[v].y * inverse) * w_low.y,
                        (values[v].z * inverse) * w_high.x, (values[v].w * inverse) * w_high.y);
      }
      __half2* target = reinterpret_cast<__half2*>(normalized + (size_t)row * p.width + column);
      target[0] = __floats2half2_rn(y.x, y.y);
      target[1] = __floats2half2_rn(y.z, y.w);
    }
  }
  complete_exchange(regions.base[p.rank], epoch != 0u ? epoch : *reinterpret_cast<volatile uint32_t*>(regions.base[p.rank]) + 1u);
}

struct ArgmaxParams {
  uint32_t ranks, rank, rows, parts, slot_offset, shard_columns;
};
struct Candidate {
  float value;
  uint32_t index;
};
__device__ __forceinline__ bool better(float value, uint32_t index, float best, uint32_t best_index) {
  return value > best || (value == best && index < best_index);
}

// token_ids[row] = global index of the best candidate over all ranks; rank r's candidate indices
// are local to its vocabulary shard [r * shard_columns, (r + 1) * shard_columns); ties go to the
// lowest global index (lib/metal_w4a16_source.ml:1286-1315).  One CTA per row.
__global__ void __launch_bounds__(256) exchange_argmax_kernel(Regions regions, uint32_t* __restrict__ token_ids,
                                                              ArgmaxParams p, uint32_t* error_word) {
  grid_chain_prologue();
  __shared__ float values[256];
  __shared__ uint32_t indices[256];
  const uint32_t epoch = announce_and_wait(regions, p.ranks, p.rank, error_word);
  if (epoch != 0u) {
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float best = -FLT_MAX;
    uint32_t best_index = 0xffffffffu;
    for (uint32_t i = tid; i < p.ranks * p.parts; i += 256u) {
      const uint32_t r = i / p.parts, part = i - r * p.parts;
      const Candidate candidate =
          reinterpret_cast<const Candidate*>(regions.base[r] + p.slot_offset)[(size_t)row * p.parts + part];
      const uint32_t global_index = candidate.index + r * p.shard_columns;
      if (better(candidate.value, global_index, best, best_index)) {
        best = candidate.value;
        best_index = global_index;
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
  complete_exchange(regions.base[p.rank], epoch != 0u ? epoch : *reinterpret_cast<volatile uint32_t*>(regions.base[p.rank]) + 1u);
}

bool collect_regions(const KernelArgs& args, uint32_t ranks, size_t needed, Regions* regions) {
  for (uint32_t r = 0; r < kMaxRanks; ++r) regions->base[r] = nullptr;
  for (uint32_t r = 0; r < ranks; ++r) {
    if (args.lengths[r] < needed || ((uintptr_t)args.buffers[r] & 15u) != 0) return false;
    regions->base[r] = (uint8_t*)args.buffers[r];
  }
  return true;
}

}  // namespace

// Buffers [region_0 .. region_{ranks-1}, residual, output]; params u32 {ranks, rank, rows, width,
// slot_offset, has_residual}.  region_rank is this rank's own region.
int launch_tp_exchange_sum(const KernelArgs& args) {
  SumParams p;
  LLMOPT_REQUIRE(args.param_bytes == sizeof(p), "expects 24 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.ranks >= 1 && p.ranks <= kMaxRanks && p.rank < p.ranks, "needs 1 <= ranks <= 8 and rank < ranks");
  LLMOPT_REQUIRE((uint32_t)args.buffer_count == p.ranks + 2, "expects one region per rank, a residual and an output");
  LLMOPT_REQUIRE(p.rows > 0 && p.width > 0 && p.width % 4 == 0 && p.slot_offset >= 256 && p.slot_offset % 16 == 0,
                 "needs rows > 0, width a multiple of 4 and a 16-byte aligned slot behind the header");
  const size_t elements = (size_t)p.rows * p.width;
  Regions regions;
  LLMOPT_REQUIRE(collect_regions(args, p.ranks, (size_t)p.slot_offset + elements * 4, &regions),
                 "a region is too short or misaligned");
  LLMOPT_REQUIRE(args.lengths[p.ranks + 1] >= elements * 2 && (!p.has_residual || args.lengths[p.ranks] >= elements * 2),
                 "residual or output buffer is too short");
  // decode rows: a few CTAs; prompt rows (megabytes per rank): enough CTAs to keep NVLink busy
  uint32_t ctas = (uint32_t)((elements + 1023) / 1024);
  const uint32_t most = elements > (1u << 18) ? 4u * (uint32_t)context_sm_count(args.ctx) : 32u;
  if (ctas > most) ctas = most;
  launch_kernel(args, exchange_sum_kernel, dim3(ctas), dim3(256), 0, regions, (const __half*)args.buffers[p.ranks],
                (__half*)args.buffers[p.ranks + 1], p, context_device_error(args.ctx));
  return check_launch(args);
}

// Prompt rows, step 1.  Buffers [region_0 .. region_{ranks-1}, residual, output]; params u32 {ranks, rank, rows,
// width, slot_offset (fp32 partials), has_residual, slice_offset (fp16 shares, a different slot)}.
int launch_tp_exchange_reduce_rows(const KernelArgs& args) {
  RowsParams p;
  LLMOPT_REQUIRE(args.param_bytes == sizeof(p), "expects 28 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.ranks >= 1 && p.ranks <= kMaxRanks && p.rank < p.ranks, "needs 1 <= ranks <= 8 and rank < ranks");
  LLMOPT_REQUIRE((uint32_t)args.buffer_count == p.ranks + 2, "expects one region per rank, a residual and an output");
  LLMOPT_REQUIRE(p.rows > 0 && p.width > 0 && p.width % 8 == 0 && p.slot_offset >= 256 && p.slot_offset % 16 == 0 &&
                     p.slice_offset >= 256 && p.slice_offset % 16 == 0,
                 "needs rows > 0, width a multiple of 8 and 16-byte aligned slots behind the header");
  const size_t elements = (size_t)p.rows * p.width;
  const bool apart = (size_t)p.slice_offset >= (size_t)p.slot_offset + elements * 4 ||
                     (size_t)p.slot_offset >= (size_t)p.slice_offset + elements * 2;
  LLMOPT_REQUIRE(apart, "the fp32 partials and the fp16 shares must be different slots");
  Regions regions;
  const size_t needed = std::max((size_t)p.slot_offset + elements * 4, (size_t)p.slice_offset + elements * 2);
  LLMOPT_REQUIRE(collect_regions(args, p.ranks, needed, &regions), "a region is too short or misaligned");
  LLMOPT_REQUIRE(args.lengths[p.ranks + 1] >= elements * 2 && (!p.has_residual || args.lengths[p.ranks] >= elements * 2),
                 "residual or output buffer is too short");
  const size_t share = ((size_t)(p.rows + p.ranks - 1) / p.ranks) * p.width;
  uint32_t ctas = (uint32_t)((share + 1023) / 1024);
  const uint32_t most = 4u * (uint32_t)context_sm_count(args.ctx);
  if (ctas > most) ctas = most;
  if (ctas == 0) ctas = 1;
  launch_kernel(args, exchange_reduce_rows_kernel, dim3(ctas), dim3(256), 0, regions, (const __half*)args.buffers[p.ranks],
                (__half*)args.buffers[p.ranks + 1], p, context_device_error(args.ctx));
  return check_launch(args);
}

// Prompt rows, step 2.  Buffers [region_0 .. region_{ranks-1}, output]; the same 28 parameter bytes.
int launch_tp_exchange_gather_rows(const KernelArgs& args) {
  RowsParams p;
  LLMOPT_REQUIRE(args.param_bytes == sizeof(p), "expects 28 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.ranks >= 1 && p.ranks <= kMaxRanks && p.rank < p.ranks, "needs 1 <= ranks <= 8 and rank < ranks");
  LLMOPT_REQUIRE((uint32_t)args.buffer_count == p.ranks + 1, "expects one region per rank and an output");
  LLMOPT_REQUIRE(p.rows > 0 && p.width > 0 && p.width % 8 == 0 && p.slice_offset >= 256 && p.slice_offset % 16 == 0,
                 "needs rows > 0, width a multiple of 8 and a 16-byte aligned slot behind the header");
  const size_t elements = (size_t)p.rows * p.width;
  Regions regions;
  LLMOPT_REQUIRE(collect_regions(args, p.ranks, (size_t)p.slice_offset + elements * 2, &regions),
                 "a region is too short or misaligned");
  LLMOPT_REQUIRE(args.lengths[p.ranks] >= elements * 2 && ((uintptr_t)args.buffers[p.ranks] & 15u) == 0,
                 "output buffer is too short or misaligned");
  const size_t share = ((size_t)(p.rows + p.ranks - 1) / p.ranks) * p.width;
  uint32_t ctas = (uint32_t)((share + 2047) / 2048);
  const uint32_t most = 4u * (uint32_t)context_sm_count(args.ctx);
  if (ctas > most) ctas = most;
  if (ctas == 0) ctas = 1;
  launch_kernel(args, exchange_gather_rows_kernel, dim3(ctas), dim3(256), 0, regions, (__half*)args.buffers[p.ranks], p,
                context_device_error(args.ctx));
  return check_launch(args);
}

// Buffers [region_0 .. region_{ranks-1}, residual, hidden output, norm weight, normalized output];
// params {ranks, rank, rows, width, slot_offset, has_residual, epsilon f32, weight_first}.
int launch_tp_exchange_sum_norm(const KernelArgs& args) {
  SumNormParams p;
  LLMOPT_REQUIRE(args.param_bytes == sizeof(p), "expects 32 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.ranks >= 1 && p.ranks <= kMaxRanks && p.rank < p.ranks, "needs 1 <= ranks <= 8 and rank < ranks");
  LLMOPT_REQUIRE((uint32_t)args.buffer_count == p.ranks + 4, "expects one region per rank and four more buffers");
  LLMOPT_REQUIRE(p.rows > 0 && p.width > 0 && p.width % 4 == 0 && p.width <= 8192 && p.slot_offset >= 256 &&
                     p.slot_offset % 16 == 0 && p.epsilon > 0.0f,
                 "needs rows > 0, width a multiple of 4 up to 8192, a 16-byte aligned slot and a positive epsilon");
  const size_t elements = (size_t)p.rows * p.width;
  Regions regions;
  LLMOPT_REQUIRE(collect_regions(args, p.ranks, (size_t)p.slot_offset + elements * 4, &regions),
                 "a region is too short or misaligned");
  LLMOPT_REQUIRE((!p.has_residual || args.lengths[p.ranks] >= elements * 2) && args.lengths[p.ranks + 1] >= elements * 2 &&
                     args.lengths[p.ranks + 2] >= (size_t)p.width * 2 && args.lengths[p.ranks + 3] >= elements * 2,
                 "residual, output or weight buffer is too short");
  launch_kernel(args, exchange_sum_norm_kernel, dim3(p.rows), dim3(kSumNormThreads), 0, regions,
                (const __half*)args.buffers[p.ranks], (__half*)args.buffers[p.ranks + 1],
                (const __half*)args.buffers[p.ranks + 2], (__half*)args.buffers[p.ranks + 3], p,
                context_device_error(args.ctx));
  return check_launch(args);
}

// Buffers [region_0 .. region_{ranks-1}, token_ids]; params u32 {ranks, rank, rows, parts,
// slot_offset, shard_columns}.  Every region's slot holds rows x parts {float value, u32 index}.
int launch_tp_exchange_argmax(const KernelArgs& args) {
  ArgmaxParams p;
  LLMOPT_REQUIRE(args.param_bytes == sizeof(p), "expects 24 parameter bytes");
  memcpy(&p, args.params, sizeof(p));
  LLMOPT_REQUIRE(p.ranks >= 1 && p.ranks <= kMaxRanks && p.rank < p.ranks, "needs 1 <= ranks <= 8 and rank < ranks");
  LLMOPT_REQUIRE((uint32_t)args.buffer_count == p.ranks + 1, "expects one region per rank and the token ids");
  LLMOPT_REQUIRE(p.rows > 0 && p.parts > 0 && p.slot_offset >= 256 && p.slot_offset % 16 == 0,
                 "needs rows, parts > 0 and a 16-byte aligned slot behind the header");
  Regions regions;
  LLMOPT_REQUIRE(collect_regions(args, p.ranks, (size_t)p.slot_offset + (size_t)p.rows * p.parts * 8, &regions),
                 "a region is too short or misaligned");
  LLMOPT_REQUIRE(args.lengths[p.ranks] >= (size_t)p.rows * 4, "token id buffer is too short");
  launch_kernel(args, exchange_argmax_kernel, dim3(p.rows), dim3(256), 0, regions, (uint32_t*)args.buffers[p.ranks], p,
                context_device_error(args.ctx));
  return check_launch(args);
}

}  // namespace llmopt
