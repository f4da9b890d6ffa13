// Decode batches (9..64 rows) of the W4A16 group-64 product on tcgen05, with the operands swapped
// relative to the prefill kernel: the WEIGHT tile is the M side of the MMA (128 rows, converted to
// fp16 in shared memory) and the activations are the N side (the batch, padded to 32 or 64), so
// the tensor work is proportional to the batch and the kernel is bound by the weight stream from
// HBM, like the single-row GEMV, instead of by a 128-row activation tile that is mostly padding.
//   D^T[weight row, batch row] = W[weight row, :] . X[batch row, :]      per 64-wide k-block
// Roles per CTA (one 128-row weight tile; gate and up tiles together in the dual form):
//   warp 0        TMA: X tile [NB x 64] fp16, 128-byte swizzle, 4-deep ring
//   warp 1        tcgen05.mma 128 x NB x 16, four per k-block and matrix; accumulators in tensor memory
//   warps 2-9     each streams ITS rows' packed weights with cp.async in groups of four k-blocks (128
//                 bytes per row, three groups deep, private to the warp: no barrier on the weight
//                 stream) and converts them: int4 -> fp16 (q * scale) rows of the A tile, 128-byte
//                 swizzled, 3-deep ring.  Eight warps issuing loads keep enough requests in flight
//                 for HBM; one or two producer warps (or the TMA unit) reach about 10 GB/s per SM.
// K is split over CTAs when there are few weight tiles (narrow projections); the last CTA of a tile
// adds the parked fp32 partials in split order and writes the result.  All waits are bounded.
// Output is transposed on the way out: a thread owns one weight row = one output column.
#include <atomic>
#include <cstdlib>

#include "w4a16_tc_device.cuh"

namespace llmopt {
using namespace gemv;
using namespace tc;

uint32_t* context_device_error(Context* ctx);
void* context_split_scratch(Context* ctx, size_t zeroed_bytes, size_t bytes, cudaStream_t stream, std::string* error);

namespace {

constexpr int kRows = 128;  // weight rows per matrix and CTA
constexpr int kBK = 64, kGroupBlocks = 4;
constexpr int kXStages = 4, kWStages = 3, kRawStages = 3;
constexpr int kConvertWarps = 8;
constexpr int kThreads = (2 + kConvertWarps) * 32;
constexpr uint32_t kSplitCounterTiles = 1u << 14;

enum BatchEpilogue { kBatchLinear = 0, kBatchDualSwiglu = 1 };

struct BatchProblem {
  uint32_t m, n, k;
  const uint8_t* packed[2];
  const __half* scale[2];
  __half* out;
  const __half* aux;  // bias (row stride 0) or residual (row stride n)
  uint32_t aux_row_stride, has_aux;
  uint32_t splits;
  float* partials;     // [tiles][splits][matrices * 128 rows][NB]
  uint32_t* counters;  // [tiles], zero between launches
};

template <int NMAT, int NB>
struct Layout {
  static constexpr int kXTile = NB * 128;             // NB batch rows x 64 halves
  static constexpr int kWTile = NMAT * kRows * 128;   // converted rows of one k-block
  static constexpr int kRawTile = NMAT * kRows * 128; // packed rows of one group (4 k-blocks)
  static constexpr int kOffsetX = 0;
  static constexpr int kOffsetW = kOffsetX + kXStages * ((kXTile + 1023) / 1024 * 1024);
  static constexpr int kOffsetRaw = kOffsetW + kWStages * kWTile;
  static constexpr int kOffsetBarriers = kOffsetRaw + kRawStages * kRawTile;
  static constexpr int kBarriers = 2 * kXStages + 2 * kWStages + 1;
  static constexpr int kOffsetHolder = kOffsetBarriers + kBarriers * 8;
  static constexpr int kBytes = kOffsetHolder + 16 + 1024;
  static constexpr uint32_t kColumns = NMAT * NB < 32 ? 32 : NMAT * NB;  // tensor-memory columns (power of two)
};

__device__ uint32_t g_abandoned_batch_launch = 0;

template <int EPI, int NB>
__global__ void __launch_bounds__(kThreads, 1)
w4a16_gemm_tc_batch_kernel(const __grid_constant__ CUtensorMap map_x, const BatchProblem p, uint32_t* error_word,
                           uint32_t launch_id) {
  constexpr int NMAT = EPI == kBatchDualSwiglu ? 2 : 1;
  using L = Layout<NMAT, NB>;
  constexpr int kXStride = (L::kXTile + 1023) / 1024 * 1024;
  extern __shared__ unsigned char shared_raw[];
  grid_chain_prologue();
  if (*reinterpret_cast<volatile uint32_t*>(&g_abandoned_batch_launch) == launch_id) return;
  const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
  unsigned char* base_pointer = shared_raw + (base - smem_u32(shared_raw));
  const uint32_t x_full = base + L::kOffsetBarriers, x_empty = x_full + kXStages * 8;
  const uint32_t w_full = x_empty + kXStages * 8, w_empty = w_full + kWStages * 8;
  const uint32_t accumulator_full = w_empty + kWStages * 8;
  volatile uint32_t* holder = reinterpret_cast<volatile uint32_t*>(base_pointer + L::kOffsetHolder);  // [tmem, abort, last]

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t tile = blockIdx.x, split = blockIdx.y, n0 = tile * kRows;
  const uint32_t all_k_blocks = p.k / kBK, all_groups = (all_k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
  const uint32_t group_begin = (uint32_t)((uint64_t)all_groups * split / p.splits);
  const uint32_t group_end = (uint32_t)((uint64_t)all_groups * (split + 1u) / p.splits);
  const uint32_t kb_begin = group_begin * kGroupBlocks;
  const uint32_t k_blocks = min(group_end * kGroupBlocks, all_k_blocks) - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kXStages; ++s) {
      barrier_init(x_full + s * 8, 1);
      barrier_init(x_empty + s * 8, 1);
    }
    for (int s = 0; s < kWStages; ++s) {
      barrier_init(w_full + s * 8, kConvertWarps);
      barrier_init(w_empty + s * 8, 1);
    }
    barrier_init(accumulator_full, 1);
    holder[1] = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + L::kOffsetHolder),
                 "r"(L::kColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = holder[0];
  volatile uint32_t* abort_flag = holder + 1;

  auto give_up = [&]() {
    *abort_flag = 1u;
    g_abandoned_batch_launch = launch_id;
    if (error_word) atomicExch(error_word, 1u);
  };

  if (warp == 0) {
    // ------------------------------ X tiles by TMA ------------------------------
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        const uint32_t s = kb % kXStages;
        if (*abort_flag || !barrier_wait(x_empty + s * 8, ((kb / kXStages) & 1u) ^ 1u)) {
          give_up();
          break;
        }
        barrier_expect_tx(x_full + s * 8, L::kXTile);
        tma_load_2d(base + L::kOffsetX + s * kXStride, &map_x, (int32_t)((kb_begin + kb) * kBK), 0, x_full + s * 8);
        issued = kb + 1;
      }
      if (*abort_flag) {
        const uint32_t first = issued > kXStages ? issued - kXStages : 0u;
        for (uint32_t kb = first; kb < issued; ++kb) barrier_wait(x_full + (kb % kXStages) * 8, (kb / kXStages) & 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t instruction = instruction_descriptor(kRows, NB);
      bool ok = true;
      for (uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
        const uint32_t s = kb % kXStages, t = kb % kWStages;
        ok = !*abort_flag && barrier_wait(x_full + s * 8, (kb / kXStages) & 1u) &&
             barrier_wait(w_full + t * 8, (kb / kWStages) & 1u);
        if (!ok) {
          give_up();
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t x_tile = base + L::kOffsetX + s * kXStride, w_tile = base + L::kOffsetW + t * L::kWTile;
#pragma unroll
        for (int a = 0; a < NMAT; ++a)
#pragma unroll
          for (int j = 0; j < kBK / 16; ++j)
            mma_f16(tmem_base + a * NB, operand_descriptor(w_tile + a * (kRows * 128) + j * 32),
                    operand_descriptor(x_tile + j * 32), (kb > 0 || j > 0) ? 1u : 0u, instruction);
        mma_commit(x_empty + s * 8);
        mma_commit(w_empty + t * 8);
      }
      if (ok) mma_commit(accumulator_full);
    }
  } else {
    // ------------------------------ conversion, then epilogue ------------------------------
    constexpr uint32_t kThreadsPerRow = 256 / (NMAT * kRows);  // 1 (dual) or 2
    constexpr uint32_t kWords = 8 / kThreadsPerRow;            // packed words (8 weights each) per thread and k-block
    const uint32_t index = threadIdx.x - 64u;
    const uint32_t row = index / kThreadsPerRow, part = index % kThreadsPerRow;  // row of the stacked tile
    const uint32_t matrix = row / kRows, weight_row = n0 + row % kRows;
    const bool row_present = weight_row < p.n;
    const uint32_t groups = p.k / 64;
    const __half* scale_row = p.scale[NMAT == 2 ? matrix : 0] + (size_t)(row_present ? weight_row : 0u) * groups;
    const uint32_t swizzle = (row & 7u) * 16u;
    bool ok = true;
    // scales of a whole group per load, fetched one group (four k-blocks) ahead
    const bool vector_ok = groups % 4u == 0u && ((uintptr_t)p.scale[NMAT == 2 ? matrix : 0] & 7u) == 0;
    FourHalves group_scales, next_scales = load_four(scale_row, kb_begin, groups, vector_ok, row_present);

    // this warp's private weight stream: its rows, 8 lanes per row (128 contiguous bytes), 4 rows per instruction
    constexpr uint32_t kRowsPerWarp = NMAT * kRows / kConvertWarps;  // 32 (dual) or 16
    const uint32_t first_row = (warp - 2u) * kRowsPerWarp, copy_chunk = lane & 7u, copy_row = lane >> 3;
    const uint32_t row_bytes = p.k / 2, my_groups = (k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
    auto issue_group = [&](uint32_t group) {
      if (group < my_groups) {
        const uint32_t stage = base + L::kOffsetRaw + (group % kRawStages) * L::kRawTile;
        const uint32_t byte_at = (group_begin + group) * (kGroupBlocks * kBK / 2) + copy_chunk * 16u;
        const uint32_t bytes = byte_at < row_bytes ? 16u : 0u;  // beyond the row end: zeros
#pragma unroll
        for (uint32_t pass = 0; pass < kRowsPerWarp / 4; ++pass) {
          const uint32_t tile_row = first_row + pass * 4u + copy_row;
          const uint32_t source_row = min(n0 + tile_row % kRows, p.n - 1u);  // absent rows re-read the last one
          const uint8_t* source =
              p.packed[NMAT == 2 ? tile_row / kRows : 0] + (size_t)source_row * row_bytes + (bytes ? byte_at : 0u);
          const uint32_t target = stage + tile_row * 128u + ((copy_chunk ^ (tile_row & 7u)) * 16u);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(target), "l"(source), "r"(bytes) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll 1
    for (uint32_t group = 0; group + 1u < kRawStages; ++group) issue_group(group);

    for (uint32_t kb = 0; kb < k_blocks; ++kb) {
      const uint32_t t = kb % kWStages, group = kb / kGroupBlocks, quarter_of_group = kb % kGroupBlocks;
      const uint32_t rs = group % kRawStages;
      if (quarter_of_group == 0u) {
        __syncwarp();  // every lane is done with the stage the next copies overwrite
        issue_group(group + kRawStages - 1u);
        asm volatile("cp.async.wait_group %0;" ::"n"(kRawStages - 1) : "memory");  // this group has landed
        __syncwarp();
        group_scales = next_scales;
        next_scales = load_four(scale_row, kb_begin + kb + kGroupBlocks, groups, vector_ok, row_present);
      }
      const __half scale = group_scales.value[quarter_of_group];
      ok = !*abort_flag && barrier_wait(w_empty + t * 8, ((kb / kWStages) & 1u) ^ 1u);
      if (!ok) {
        give_up();
        break;
      }
      const unsigned char* raw = base_pointer + L::kOffsetRaw + rs * L::kRawTile + row * 128u;
      uint32_t words[kWords];
#pragma unroll
      for (uint32_t i = 0; i < kWords / 4; ++i) {
        const uint32_t raw_chunk = 2u * quarter_of_group + (kThreadsPerRow == 2 ? part : i);
        const uint4 data = *reinterpret_cast<const uint4*>(raw + ((raw_chunk * 16u) ^ swizzle));
        words[4 * i] = data.x, words[4 * i + 1] = data.y, words[4 * i + 2] = data.z, words[4 * i + 3] = data.w;
      }
      const __half2 scale_pair = __halves2half2(scale, __hmul(scale, __float2half(0.0625f)));
      const uint32_t scales = *reinterpret_cast<const uint32_t*>(&scale_pair);
      unsigned char* w_row = base_pointer + L::kOffsetW + t * L::kWTile + row * 128u;
#pragma unroll
      for (uint32_t i = 0; i < kWords; ++i) {  // packed word i -> k 8 i .. 8 i + 7 of this thread's part
        uint4 chunk;
        chunk.x = dequant_pair<false, 0>(words[i], scales, 0u);
        chunk.y = dequant_pair<false, 1>(words[i], scales, 0u);
        chunk.z = dequant_pair<false, 2>(words[i], scales, 0u);
        chunk.w = dequant_pair<false, 3>(words[i], scales, 0u);
        const uint32_t out_chunk = part * kWords + i;
        *reinterpret_cast<uint4*>(w_row + ((out_chunk * 16u) ^ swizzle)) = chunk;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) barrier_arrive(w_full + t * 8);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    // epilogue: a thread owns weight row (lane quarter * 32 + lane) = one output column, and half of
    // the batch columns; lanes of a warp are consecutive output columns, so stores coalesce per batch row
    ok = ok && !*abort_flag && barrier_wait(accumulator_full, 0u);
    if (!ok) give_up();
    {
      uint32_t all_ok;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.u32 q, %1, 0;\n\t"
          "bar.red.and.pred p, 1, 256, q;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(all_ok)
          : "r"(ok ? 1u : 0u)
          : "memory");
      ok = all_ok != 0u;
    }
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      constexpr int kHalf = NB / 2;  // batch columns per thread: 16 or 32
      const uint32_t quarter = warp & 3u, half_index = (warp - 2u) >> 2;
      const uint32_t tile_row = quarter * 32u + lane, column = n0 + tile_row;  // output column
      const uint32_t lane_address = tmem_base + ((quarter * 32u) << 16) + half_index * kHalf;
      float values[NMAT][kHalf];
#pragma unroll
      for (int a = 0; a < NMAT; ++a) {
#pragma unroll
        for (int piece = 0; piece < kHalf / 16; ++piece) {
          uint32_t bits[16];
          tmem_load_16(lane_address + a * NB + piece * 16, bits);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 16; ++i) values[a][piece * 16 + i] = __uint_as_float(bits[i]);
        }
      }
      bool finish = true;
      if (p.splits > 1u) {
        // park, count, and go on only as the last split of this tile
        constexpr int kPerTile = NMAT * kRows * NB;
        float* mine = p.partials + ((size_t)tile * p.splits + split) * kPerTile;
#pragma unroll
        for (int a = 0; a < NMAT; ++a)
#pragma unroll
          for (int i = 0; i < kHalf / 4; ++i)
            *reinterpret_cast<float4*>(mine + ((size_t)a * kRows + tile_row) * NB + half_index * kHalf + 4 * i) =
                make_float4(values[a][4 * i], values[a][4 * i + 1], values[a][4 * i + 2], values[a][4 * i + 3]);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 64u) {
          __threadfence();
          const uint32_t before = atomicAdd(p.counters + tile, 1u);
          const bool last = before + 1u == p.splits;
          if (last) p.counters[tile] = 0u;
          holder[2] = last ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        finish = holder[2] != 0u;
        if (finish) {
          __threadfence();
          const float* parts = p.partials + (size_t)tile * p.splits * kPerTile;
#pragma unroll
          for (int a = 0; a < NMAT; ++a)
#pragma unroll
            for (int i = 0; i < kHalf; ++i) values[a][i] = 0.0f;
          for (uint32_t s = 0; s < p.splits; ++s)  // split order: the sum does not depend on who came last
#pragma unroll
            for (int a = 0; a < NMAT; ++a)
#pragma unroll
              for (int i = 0; i < kHalf / 4; ++i) {
                const float4 part = __ldcg(reinterpret_cast<const float4*>(
                    parts + (size_t)s * kPerTile + ((size_t)a * kRows + tile_row) * NB + half_index * kHalf + 4 * i));
                values[a][4 * i] += part.x;
                values[a][4 * i + 1] += part.y;
                values[a][4 * i + 2] += part.z;
                values[a][4 * i + 3] += part.w;
              }
        }
      }
      if (finish && column < p.n) {
#pragma unroll
        for (int i = 0; i < kHalf; ++i) {
          const uint32_t batch_row = half_index * kHalf + i;
          if (batch_row >= p.m) break;
          float value;
          if (EPI == kBatchDualSwiglu) {
            const float g = values[0][i];
            value = (g / (1.0f + __expf(-g))) * values[NMAT - 1][i];  // lib/metal_w4a16_source.ml:571-575
          } else {
            value = values[0][i];
            if (p.has_aux) value += __half2float(p.aux[(size_t)batch_row * p.aux_row_stride + column]);
          }
          p.out[(size_t)batch_row * p.n + column] = __float2half_rn(value);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  }

  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::kColumns) : "memory");
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled function = []() -> EncodeTiled {
    void* pointer = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiled>(pointer);
  }();
  return function;
}

template <int EPI, int NB>
int run_batch(const KernelArgs& args, const CUtensorMap& map_x, BatchProblem p) {
  constexpr int NMAT = EPI == kBatchDualSwiglu ? 2 : 1;
  using L = Layout<NMAT, NB>;
  auto kernel = w4a16_gemm_tc_batch_kernel<EPI, NB>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  const uint32_t tiles = (p.n + kRows - 1) / kRows, sms = (uint32_t)context_sm_count(args.ctx);
  const uint32_t groups = (p.k / kBK + kGroupBlocks - 1u) / kGroupBlocks;
  // one CTA per SM at most (a second wave would double the time); each split keeps at least two groups
  uint32_t splits = sms / tiles;
  if (splits > groups / 2u) splits = groups / 2u;
  if (splits > 16u) splits = 16u;
  if (splits < 1u || tiles > kSplitCounterTiles) splits = 1u;
  p.splits = splits;
  if (splits > 1u) {
    constexpr size_t counter_bytes = kSplitCounterTiles * sizeof(uint32_t);
    const size_t partial_bytes = (size_t)tiles * splits * NMAT * kRows * NB * sizeof(float);
    uint8_t* scratch =
        (uint8_t*)context_split_scratch(args.ctx, counter_bytes, counter_bytes + partial_bytes, args.stream, args.error);
    if (scratch == nullptr) return 1;
    p.counters = reinterpret_cast<uint32_t*>(scratch);
    p.partials = reinterpret_cast<float*>(scratch + counter_bytes);
  }
  static std::atomic<uint32_t> launches{0};
  launch_kernel(args, kernel, dim3(tiles, splits), dim3(kThreads), L::kBytes, map_x, p,
                context_device_error(args.ctx), launches.fetch_add(1) + 1u);
  return check_launch(args);
}

}  // namespace

// Rows from which decode batches take this kernel (below it the small-M GEMV wins);
// LLMOPT_CUDA_TC_BATCH_MIN_ROWS overrides it, 0 disables the kernel.
uint32_t tensor_core_batch_min_rows() {
  static const uint32_t rows = []() -> uint32_t {
    const char* text = getenv("LLMOPT_CUDA_TC_BATCH_MIN_ROWS");
    if (text == nullptr) return 33u;
    const long value = strtol(text, nullptr, 10);
    return value <= 0 ? 0xffffffffu : (uint32_t)value;
  }();
  return rows;
}

// Decode batches up to 64 rows; returns -1 outside its domain (the caller falls back).
int launch_w4a16_gemm_tc_batch(const KernelArgs& args, const GemvProblem& problem, int epilogue) {
  if (args.ctx == nullptr || problem.m < tensor_core_batch_min_rows() || problem.m > 64 || problem.x_rows != problem.m ||
      problem.k % 64 != 0 || problem.norm_weight != nullptr)
    return -1;
  if (epilogue == kEpiQkv) {
    for (uint32_t i = 0; i < problem.matrices; ++i) {
      GemvProblem one = problem;
      one.mat[0] = problem.mat[i];
      one.matrices = 1;
      one.out[0] = problem.out[i];
      one.has_aux = 0;
      const int status = launch_w4a16_gemm_tc_batch(args, one, kEpiLinear);
      if (status != 0) return i == 0 ? status : (status < 0 ? 1 : status);
    }
    return 0;
  }
  if (epilogue != kEpiLinear && epilogue != kEpiDualSwiglu) return -1;
  if (problem.out_f32 != nullptr) return -1;
  const uint32_t matrices = epilogue == kEpiDualSwiglu ? 2u : 1u;
  if (((uintptr_t)problem.x & 15u) != 0 || (problem.k / 2) % 16 != 0) return -1;
  for (uint32_t i = 0; i < matrices; ++i)
    if (((uintptr_t)problem.mat[i].packed & 15u) != 0 || problem.mat[i].n != problem.mat[0].n) return -1;
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return -1;
  const uint32_t padded = problem.m <= 32 ? 32u : 64u;
  CUtensorMap map_x;
  const cuuint64_t dims[2] = {problem.k, problem.m};
  const cuuint64_t strides[1] = {(cuuint64_t)problem.k * 2};
  const cuuint32_t box[2] = {kBK, padded};
  const cuuint32_t element_strides[2] = {1, 1};
  if (encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(problem.x), dims, strides, box,
             element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -1;
  BatchProblem p = {};
  p.m = problem.m;
  p.n = problem.mat[0].n;
  p.k = problem.k;
  for (uint32_t i = 0; i < 2; ++i) {
    p.packed[i] = problem.mat[i < matrices ? i : 0].packed;
    p.scale[i] = problem.mat[i < matrices ? i : 0].scale;
  }
  p.out = problem.out[0];
  p.aux = problem.aux0;
  p.aux_row_stride = problem.aux_row_stride;
  p.has_aux = problem.has_aux;
  if (epilogue == kEpiDualSwiglu)
    return padded == 32 ? run_batch<kBatchDualSwiglu, 32>(args, map_x, p) : run_batch<kBatchDualSwiglu, 64>(args, map_x, p);
  return padded == 32 ? run_batch<kBatchLinear, 32>(args, map_x, p) : run_batch<kBatchLinear, 64>(args, map_x, p);
}

}  // namespace llmopt
