// Decode batches (17..64 rows) and prompts of the W4A16 group-64 product on tcgen05, with the operands swapped
// relative to the prefill kernel: the WEIGHT tile is the M side of the MMA (128 rows) and the
// activations are the N side (the batch, padded to 16, 32 or 64), so the tensor work is
// proportional to the batch and the kernel is bound by the weight stream from HBM, like the
// single-row GEMV, instead of by a 128-row activation tile that is mostly padding.
//   D^T[weight row, batch row] = W[weight row, :] . X[batch row, :]      per 64-wide k-block
// The converted weights never touch shared memory: the A operand of the MMA is read from TENSOR
// MEMORY, where lane = weight row and one 32-bit column = two consecutive k (K-major), which is
// exactly what a thread that converts one weight row holds in registers (tcgen05.st, 32 columns per
// k-block).  Shared memory carries only the packed bytes and the activation tiles.
// Roles per CTA (one 128-row weight tile; gate and up tiles together in the dual form):
//   warp 0        TMA: X tile [NB x 64] fp16, 128-byte swizzle, 4-deep ring
//   warp 1        tcgen05.mma 128 x NB x 16 (A from tensor memory, B = X from shared memory), four per
//                 k-block and matrix; accumulators in tensor memory
//   warps 2-17    warp w owns tensor-memory lanes 32 (w % 4) .. +31, i.e. those 32 weight rows, and of
//                 every group of k-blocks (eight; four per matrix in the dual form) it converts two
//                 consecutive ones: it streams exactly those 64 packed bytes per row with cp.async
//                 (private to the warp: no barrier on the weight stream, several groups deep) and
//                 converts them, int4 -> fp16 (q * scale), one k-block = 32 columns per tcgen05.st,
//                 into a ring of A stages in tensor memory.  The completion of a store is waited
//                 for behind the next k-block's arithmetic: store, wait, publish per k-block made
//                 every k-block cost ~0.7 us whatever else the kernel did (loads, MMAs, conversion
//                 removed one at a time: no change), because every warp took part in every k-block.
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
constexpr int kBK = 64;
constexpr int kConvertWarps = 16;
constexpr int kThreads = (2 + kConvertWarps) * 32;
constexpr uint32_t kSplitCounterTiles = 1u << 14;

// kBatchLinear: one 128-row weight tile per CTA; kBatchDualSwiglu: the gate and the up tile of the same rows;
// kBatchLinearPair: two neighbouring 128-row tiles of ONE matrix (the prompt form: the activation tile is
// read once for 256 output columns); kBatchDualStacked: ONE tile whose lanes 0..63 are 64 gate rows and
// lanes 64..127 the same 64 up rows, so that gate/up prompts also run 256 tokens wide with one accumulator
// (the halves meet in shared memory for silu(gate) * up).
// kBatchSplitF32: one weight tile; the activation rows are fp32 values given as exact hi/lo half pairs in
// 8-row slot tiles [hi0..hi3, lo0..lo3] (the LM head's normalised rows) and the output is the fp32 sum of the
// pair's two accumulator columns.
enum BatchEpilogue { kBatchLinear = 0, kBatchDualSwiglu = 1, kBatchLinearPair = 2, kBatchDualStacked = 3, kBatchSplitF32 = 4 };

struct BatchProblem {
  uint32_t m, n, k;
  const uint8_t* packed[2];
  const __half* scale[2];
  const __half* zero[2];  // zero points of the unsigned-nibble form (AFFINE), else unused
  __half* out;
  float* out_f32;     // kBatchSplitF32: [m, n] fp32
  const __half* aux;  // bias (row stride 0) or residual (row stride n)
  uint32_t aux_row_stride, has_aux;
  uint32_t splits;
  float* partials;     // [tiles][splits][matrices * 128 rows][NB]
  uint32_t* counters;  // [tiles], zero between launches
};

constexpr uint32_t next_power_of_two(uint32_t value) {
  uint32_t power = 32;
  while (power < value) power *= 2;
  return power;
}

template <int NMAT, int NB>
struct Layout {
  // A group is what the conversion warps of a lane quarter share out: every warp converts a PAIR of
  // consecutive k-blocks of it (64 contiguous packed bytes per row).  Single form: four warps per lane
  // quarter, eight k-blocks; dual form: two warps per lane quarter and matrix, four k-blocks.
  // A ring stage (of X in shared memory, of A in tensor memory) is one such pair: the MMA thread pays
  // its waits and its one commit per pair.
  static constexpr int kGroupBlocks = NMAT == 2 ? 4 : 8;
  static constexpr int kRowPitch = kGroupBlocks * 32;  // packed bytes of one row and group
  static constexpr int kXTile = NB * 128;              // NB batch rows x 64 halves
  static constexpr int kXStride = (kXTile + 1023) / 1024 * 1024;
  static constexpr int kXStage = 2 * kXStride;         // the pair's two X tiles
  static constexpr int kRawTile = NMAT * kRows * kRowPitch;  // packed rows of one group
  // Depth of the A ring (tensor memory).  The pairs of a group are produced side by side by different warps
  // and consumed in order, and the waits tell ring phases apart by parity alone: a warp must never be two
  // uses of a stage ahead of the commits, which holds when the ring has at least as many stages as a group
  // has pairs (a warp's previous pair then vouches for the commit two uses back).
  static constexpr int kStages = NMAT == 2 ? (NB > 64 ? 2 : 3) : (NB > 64 ? 4 : 6);
  static_assert(kStages >= kGroupBlocks / 2, "ring phases would alias");
  // Depth of the X ring (shared memory): the same, with the same barrier, unless the tiles are too large
  static constexpr int kXStages = (NMAT == 1 && NB > 128) ? 2 : kStages;
  // groups of packed bytes in flight per warp: what is left of shared memory beside the X ring
  static constexpr int kRawStages = NB > 64 && NMAT == 1 ? 2 : (NMAT == 1 && NB > 32) ? 3 : 4;  // 32 KB each
  static constexpr int kOffsetX = 0;
  static constexpr int kOffsetRaw = kOffsetX + kXStages * kXStage;
  static constexpr int kOffsetBarriers = kOffsetRaw + kRawStages * kRawTile;
  static constexpr int kBarriers = 2 * kStages + 2 * kXStages + 1;
  static constexpr int kOffsetHolder = kOffsetBarriers + kBarriers * 8;
  static constexpr int kBytes = kOffsetHolder + 16 + 1024;
  // tensor memory: NMAT accumulators of NB fp32 columns, then kStages stages of a converted pair:
  // [k-block of the pair][matrix][32 columns = 64 k]
  static constexpr uint32_t kAccumulatorColumns = (NMAT * NB + 31) / 32 * 32;  // the A ring starts on a 32-column boundary
  static constexpr uint32_t kAColumns = 2 * NMAT * 32;
  static constexpr uint32_t kColumns = next_power_of_two(kAccumulatorColumns + kStages * kAColumns);
  static_assert(kColumns <= 512, "tensor memory has 512 columns");
  static_assert(kBytes <= 227 * 1024, "shared memory of one CTA");
};

// D[tmem] (+)= A[tmem] . B[smem descriptor]: the A operand (128 lanes x 8 columns per k16 step) comes from tensor memory.
__device__ __forceinline__ void mma_f16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t accumulate,
                                               uint32_t instruction) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(instruction), "r"(accumulate), "r"(0u)
      : "memory");
}
// 32 consecutive columns of this thread's lane <- 32 registers.
__device__ __forceinline__ void tmem_store_32(uint32_t address, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

__device__ uint32_t g_abandoned_batch_launch = 0;

template <int EPI, int NB, bool AFFINE = false>
__global__ void __launch_bounds__(kThreads, 1)
w4a16_gemm_tc_batch_kernel(const __grid_constant__ CUtensorMap map_x, const BatchProblem p, uint32_t* error_word,
                           uint32_t launch_id) {
  constexpr bool kStacked = EPI == kBatchDualStacked;
  constexpr int NMAT = (EPI == kBatchLinear || kStacked || EPI == kBatchSplitF32) ? 1 : 2;
  constexpr uint32_t kTileRows = EPI == kBatchLinearPair ? 2 * kRows : kStacked ? kRows / 2 : kRows;  // output columns of one CTA
  using L = Layout<NMAT, NB>;
  constexpr int kRawStages = L::kRawStages, kStages = L::kStages, kXStages = L::kXStages, kGroupBlocks = L::kGroupBlocks;
  extern __shared__ unsigned char shared_raw[];
  grid_chain_prologue();
  if (*reinterpret_cast<volatile uint32_t*>(&g_abandoned_batch_launch) == launch_id) return;
  const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
  unsigned char* base_pointer = shared_raw + (base - smem_u32(shared_raw));
  // per ring stage: X landed (TMA bytes), A converted (one arrival per contributing warp), stage consumed
  // (ONE tcgen05.commit, which both the TMA thread and the conversion warps wait for)
  // (a separate X ring has its own release barrier and costs a second commit per pair)
  const uint32_t x_full = base + L::kOffsetBarriers, a_full = x_full + kXStages * 8, empty = a_full + kStages * 8;
  const uint32_t x_empty = empty + kStages * 8, accumulator_full = x_empty + kXStages * 8;
  constexpr bool kSharedRelease = kXStages == kStages;
  volatile uint32_t* holder = reinterpret_cast<volatile uint32_t*>(base_pointer + L::kOffsetHolder);  // [tmem, abort, last]

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t tile = blockIdx.x, split = blockIdx.y, n0 = tile * kTileRows;
  const uint32_t token0 = blockIdx.z * NB;           // first activation row of this CTA (prompts: several row tiles)
  const uint32_t tile_id = blockIdx.z * gridDim.x + tile;  // index of the output tile for the K-split bookkeeping
  const uint32_t all_k_blocks = p.k / kBK, all_groups = (all_k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
  const uint32_t group_begin = (uint32_t)((uint64_t)all_groups * split / p.splits);
  const uint32_t group_end = (uint32_t)((uint64_t)all_groups * (split + 1u) / p.splits);
  const uint32_t kb_begin = group_begin * kGroupBlocks;
  const uint32_t k_blocks = min(group_end * kGroupBlocks, all_k_blocks) - kb_begin;
  const uint32_t pairs = (k_blocks + 1u) / 2u;  // ring stages this CTA goes through; the last may hold one k-block
  // a pair of A is completed by one warp per lane quarter (and matrix)
  constexpr uint32_t kWarpsPerStage = 4 * NMAT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      barrier_init(a_full + s * 8, kWarpsPerStage);
      barrier_init(empty + s * 8, 1);
    }
    for (int s = 0; s < kXStages; ++s) {
      barrier_init(x_full + s * 8, 1);
      barrier_init(x_empty + s * 8, 1);
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
  const uint32_t tmem_a_ring = tmem_base + L::kAccumulatorColumns;
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
      for (uint32_t pair = 0; pair < pairs; ++pair) {
        const uint32_t s = pair % kXStages;
        if (*abort_flag || !barrier_wait((kSharedRelease ? empty : x_empty) + s * 8, ((pair / kXStages) & 1u) ^ 1u)) {
          give_up();
          break;
        }
        const bool both = 2u * pair + 1u < k_blocks;
        barrier_expect_tx(x_full + s * 8, both ? 2 * L::kXTile : L::kXTile);
        const uint32_t target = base + L::kOffsetX + s * L::kXStage;  // s: stage of the X ring
        tma_load_2d(target, &map_x, (int32_t)((kb_begin + 2u * pair) * kBK), (int32_t)token0, x_full + s * 8);
        if (both) tma_load_2d(target + L::kXStride, &map_x, (int32_t)((kb_begin + 2u * pair + 1u) * kBK), (int32_t)token0, x_full + s * 8);
        issued = pair + 1;
      }
      if (*abort_flag) {
        const uint32_t first = issued > kXStages ? issued - kXStages : 0u;
        for (uint32_t pair = first; pair < issued; ++pair) barrier_wait(x_full + (pair % kXStages) * 8, (pair / kXStages) & 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // One thread issues everything, so its instruction stream is part of the critical path: descriptors
    // are advanced by adding constants (never rebuilt), and the stage is released by a single commit.
    if (lane == 0) {
      constexpr uint32_t instruction = instruction_descriptor(kRows, NB);
      const uint64_t x_descriptor_0 = operand_descriptor(base + L::kOffsetX);
      bool ok = true;
      uint32_t accumulate = 0u;
      for (uint32_t pair = 0; pair < pairs && ok; ++pair) {
        const uint32_t s = pair % kStages, phase = (pair / kStages) & 1u, sx = pair % kXStages;
        ok = !*abort_flag && barrier_wait(x_full + sx * 8, (pair / kXStages) & 1u) && barrier_wait(a_full + s * 8, phase);
        if (!ok) {
          give_up();
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_stage = tmem_a_ring + s * L::kAColumns;
        const uint64_t x_descriptor = x_descriptor_0 + (uint64_t)(sx * (L::kXStage >> 4));
        const uint32_t members = 2u * pair + 1u < k_blocks ? 2u : 1u;
#pragma unroll
        for (uint32_t which = 0; which < 2; ++which) {
          if (which < members) {
#pragma unroll
            for (int a = 0; a < NMAT; ++a)
#pragma unroll
              for (int j = 0; j < kBK / 16; ++j) {  // 16 k = 32 bytes further along the swizzled rows: + 2 in the address field
                mma_f16_tmem_a(tmem_base + a * NB, a_stage + which * (NMAT * 32) + a * 32 + j * 8,
                               x_descriptor + (uint64_t)(which * (L::kXStride >> 4) + 2 * j), j == 0 ? accumulate : 1u,
                               instruction);
              }
            accumulate = 1u;
          }
        }
        mma_commit(empty + s * 8);
        if (!kSharedRelease) mma_commit(x_empty + sx * 8);
      }
      if (ok) mma_commit(accumulator_full);
    }
  } else {
    // ------------------------------ conversion, then epilogue ------------------------------
    // a warp reaches the tensor-memory lanes 32 (warp % 4) .. +31 only: those are its weight rows
    const uint32_t quarter = warp & 3u, sub = (warp - 2u) >> 2;  // sub = 0..3: this warp among its lane quarter's four
    const uint32_t tile_row = quarter * 32u + lane;               // row of the weight tile = tensor-memory lane
    const uint32_t matrix = NMAT == 2 ? sub >> 1 : 0u;  // which of the CTA's two weight tiles
    const uint32_t duo = NMAT == 2 ? (sub & 1u) : sub;  // this warp converts k-blocks 2 duo and 2 duo + 1 of every group
    // the matrix this warp's rows come from, the tile's first row there, and the row of a tile row
    const uint32_t source = EPI == kBatchDualSwiglu ? matrix : kStacked ? quarter >> 1 : 0u;
    const uint32_t tile_first_row = n0 + (EPI == kBatchLinearPair ? matrix * kRows : 0u);
    auto row_in_source = [&](uint32_t row) { return kStacked ? (row & (kRows / 2 - 1u)) : row; };
    const uint32_t weight_row = tile_first_row + row_in_source(tile_row);
    const bool row_present = weight_row < p.n;
    const uint32_t groups = p.k / 64;
    const __half* scale_row = p.scale[source] + (size_t)(row_present ? weight_row : 0u) * groups;
    const uint32_t swizzle = (tile_row & 7u) * 16u;
    const uint32_t lane_base = (quarter * 32u) << 16;     // lane field of this warp's tensor-memory addresses
    bool ok = true;
    // the two group scales of this warp's k-blocks, fetched one group ahead (one 4-byte load where aligned)
    const bool pair_ok = groups % 2u == 0u && ((uintptr_t)p.scale[source] & 3u) == 0;
    auto load_scales = [&](uint32_t group) -> __half2 {
      const uint32_t first = kb_begin + group * kGroupBlocks + 2u * duo;
      if (!row_present || first >= groups) return __float2half2_rn(0.0f);
      if (pair_ok) return __ldg(reinterpret_cast<const __half2*>(scale_row + first));
      return __halves2half2(__ldg(scale_row + first), first + 1u < groups ? __ldg(scale_row + first + 1u) : __float2half(0.0f));
    };
    __half2 group_scales = __float2half2_rn(0.0f), next_scales = load_scales(0);
    // zero points of the unsigned-nibble form, fetched like the scales
    const __half* zero_row = AFFINE ? p.zero[source] + (size_t)(row_present ? weight_row : 0u) * groups : nullptr;
    const bool zero_pair_ok = AFFINE && groups % 2u == 0u && ((uintptr_t)p.zero[source] & 3u) == 0;
    auto load_zeros = [&](uint32_t group) -> __half2 {
      const uint32_t first = kb_begin + group * kGroupBlocks + 2u * duo;
      if (!AFFINE || !row_present || first >= groups) return __float2half2_rn(0.0f);
      if (zero_pair_ok) return __ldg(reinterpret_cast<const __half2*>(zero_row + first));
      return __halves2half2(__ldg(zero_row + first), first + 1u < groups ? __ldg(zero_row + first + 1u) : __float2half(0.0f));
    };
    __half2 group_zeros = __float2half2_rn(0.0f), next_zeros = load_zeros(0);

    // This warp's private weight stream: the 64 contiguous bytes per row (chunks 4 duo .. 4 duo + 3 of the
    // row's group) that it converts, four lanes per row, eight rows per instruction.
    const uint32_t copy_row = lane >> 2, copy_chunk = 4u * duo + (lane & 3u);
    const uint32_t row_bytes = p.k / 2, my_groups = (k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
    const uint8_t* packed = p.packed[source];
    auto issue_group = [&](uint32_t group) {
      if (group < my_groups) {
        const uint32_t stage = base + L::kOffsetRaw + (group % kRawStages) * L::kRawTile + matrix * (kRows * L::kRowPitch);
        const uint32_t byte_at = (group_begin + group) * L::kRowPitch + copy_chunk * 16u;
        const uint32_t bytes = byte_at < row_bytes ? 16u : 0u;  // beyond the row end: zeros
#pragma unroll
        for (uint32_t pass = 0; pass < 4; ++pass) {
          const uint32_t row = quarter * 32u + pass * 8u + copy_row;
          const uint32_t source_row = min(tile_first_row + row_in_source(row), p.n - 1u);  // absent rows re-read the last one
          const uint8_t* from = packed + (size_t)source_row * row_bytes + (bytes ? byte_at : 0u);
          const uint32_t target = stage + row * L::kRowPitch + ((copy_chunk ^ (row & 7u)) * 16u);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(target), "l"(from), "r"(bytes) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll 1
    for (uint32_t group = 0; group + 1u < kRawStages; ++group) issue_group(group);

    for (uint32_t group = 0; group < my_groups && ok; ++group) {
      const uint32_t rs = group % kRawStages;
      __syncwarp();  // every lane is done with the stage the next copies overwrite
      issue_group(group + kRawStages - 1u);
      asm volatile("cp.async.wait_group %0;" ::"n"(kRawStages - 1) : "memory");  // this group has landed
      __syncwarp();
      group_scales = next_scales;
      next_scales = load_scales(group + 1u);
      if (AFFINE) {
        group_zeros = next_zeros;
        next_zeros = load_zeros(group + 1u);
      }
      const uint32_t pair = group * (kGroupBlocks / 2) + duo;  // this warp's pair of the group = one ring stage
      if (2u * pair >= k_blocks) continue;
      const uint32_t s = pair % kStages;
      const unsigned char* raw =
          base_pointer + L::kOffsetRaw + rs * L::kRawTile + matrix * (kRows * L::kRowPitch) + tile_row * L::kRowPitch;
#pragma unroll
      for (uint32_t which = 0; which < 2; ++which) {
        if (2u * pair + which >= k_blocks) break;
        const uint32_t in_group = 2u * duo + which;
        const uint4 first = *reinterpret_cast<const uint4*>(raw + (((2u * in_group) * 16u) ^ swizzle));
        const uint4 second = *reinterpret_cast<const uint4*>(raw + (((2u * in_group + 1u) * 16u) ^ swizzle));
        const uint32_t words[8] = {first.x, first.y, first.z, first.w, second.x, second.y, second.z, second.w};
        const __half scale = which == 0 ? __low2half(group_scales) : __high2half(group_scales);
        const __half2 scale_pair = __halves2half2(scale, __hmul(scale, __float2half(0.0625f)));
        const uint32_t scales = *reinterpret_cast<const uint32_t*>(&scale_pair);
        const __half zero = which == 0 ? __low2half(group_zeros) : __high2half(group_zeros);
        const __half2 zero_pair = __halves2half2(zero, __hmul(zero, __float2half(16.0f)));
        const uint32_t zeros = *reinterpret_cast<const uint32_t*>(&zero_pair);
        uint32_t converted[32];  // column c of the k-block = the halves (k = 2c, 2c + 1) of this row
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {  // packed word i -> k 8 i .. 8 i + 7
          converted[4 * i] = dequant_pair<AFFINE, 0>(words[i], scales, zeros);
          converted[4 * i + 1] = dequant_pair<AFFINE, 1>(words[i], scales, zeros);
          converted[4 * i + 2] = dequant_pair<AFFINE, 2>(words[i], scales, zeros);
          converted[4 * i + 3] = dequant_pair<AFFINE, 3>(words[i], scales, zeros);
        }
        if (which == 0) {  // the stage must have been consumed (arithmetic first: the wait is usually over by now)
          ok = !*abort_flag && barrier_wait(empty + s * 8, ((pair / kStages) & 1u) ^ 1u);
          if (!ok) {
            give_up();
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        tmem_store_32(lane_base + tmem_a_ring + s * L::kAColumns + which * (NMAT * 32u) + matrix * 32u, converted);
      }
      if (!ok) break;
      // one completion wait and one arrival per pair (per k-block they cost more than the conversion)
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) barrier_arrive(a_full + s * 8);
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
          "bar.red.and.pred p, 1, 512, q;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(all_ok)
          : "r"(ok ? 1u : 0u)
          : "memory");
      ok = all_ok != 0u;
    }
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      constexpr int kHalf = NB / 4;       // batch columns per thread (the four warps of a lane quarter split them)
      constexpr int kPiece = kHalf < 16 ? kHalf : 16;  // columns handled at a time
      constexpr int kPieces = kHalf / kPiece;
      const uint32_t half_index = sub;
      const uint32_t lane_address = tmem_base + lane_base + half_index * kHalf;
      constexpr int kPerTile = NMAT * kRows * NB;
      auto load_piece = [&](int piece, float (&values)[NMAT][kPiece]) {
#pragma unroll
        for (int a = 0; a < NMAT; ++a) {
          uint32_t bits[16];
          if (kPiece == 16) {
            tmem_load_16(lane_address + a * NB + piece * 16, bits);
          } else if (kPiece == 8) {
            uint32_t eight[8];
            tmem_load_8(lane_address + a * NB, eight);
#pragma unroll
            for (int i = 0; i < 8; ++i) bits[i] = eight[i];
          } else {
            uint32_t four[4];
            tmem_load_4(lane_address + a * NB, four);
#pragma unroll
            for (int i = 0; i < 4; ++i) bits[i] = four[i];
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < kPiece; ++i) values[a][i] = __uint_as_float(bits[i]);
        }
      };
      auto write_piece = [&](int piece, const float (&values)[NMAT][kPiece]) {
#pragma unroll
        for (int a = 0; a < (EPI == kBatchLinearPair ? 2 : 1); ++a) {  // the pair form writes both of its tiles
          const uint32_t column = n0 + a * kRows + tile_row;           // output column
          if (column >= p.n) continue;
#pragma unroll
          for (int i = 0; i < kPiece; ++i) {
            const uint32_t batch_row = token0 + half_index * kHalf + piece * kPiece + i;
            if (batch_row >= p.m) break;
            float value;
            if (EPI == kBatchDualSwiglu) {
              const float g = values[0][i];
              value = (g / (1.0f + __expf(-g))) * values[NMAT - 1][i];  // lib/metal_w4a16_source.ml:571-575
            } else {
              value = values[a][i];
              if (p.has_aux) value += __half2float(p.aux[(size_t)batch_row * p.aux_row_stride + column]);
            }
            if (EPI != kBatchDualSwiglu && p.out_f32 != nullptr)
              p.out_f32[(size_t)batch_row * p.n + column] = value;  // unrounded partial sum of a row-split product
            else
              p.out[(size_t)batch_row * p.n + column] = __float2half_rn(value);
          }
        }
      };
      // stacked gate/up form: the finished values meet in shared memory ([token][tile row], the rings are idle by now)
      float* stash = reinterpret_cast<float*>(base_pointer + L::kOffsetX);
      static_assert(!kStacked || NB * kRows * 4 <= L::kXStages * L::kXStage, "the stash must fit the X ring");
      auto emit = [&](int piece, const float (&values)[NMAT][kPiece]) {
        if (EPI == kBatchSplitF32) {
          // this thread's 16 columns are two slot tiles: token 4 t + w = column 8 t + w (hi) + column 8 t + 4 + w (lo)
          static_assert(EPI != kBatchSplitF32 || kPiece == 16, "hi and lo of a token must sit in one thread's piece");
          const uint32_t column = n0 + tile_row;
          if (column < p.n) {
#pragma unroll
            for (int t = 0; t < kPiece / 8; ++t)
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const uint32_t token = (half_index * kHalf + piece * kPiece) / 2 + 4 * t + w;
                if (token < p.m) p.out_f32[(size_t)token * p.n + column] = values[0][8 * t + w] + values[0][8 * t + 4 + w];
              }
          }
        } else if (kStacked) {
#pragma unroll
          for (int i = 0; i < kPiece; ++i) stash[(half_index * kHalf + piece * kPiece + i) * kRows + tile_row] = values[0][i];
        } else {
          write_piece(piece, values);
        }
      };
      bool finished = true;
      if (p.splits == 1u) {
#pragma unroll 1
        for (int piece = 0; piece < kPieces; ++piece) {
          float values[NMAT][kPiece];
          load_piece(piece, values);
          emit(piece, values);
        }
      } else {
        // park, count, and go on only as the last split of this tile
        float* mine = p.partials + ((size_t)tile_id * p.splits + split) * kPerTile;
#pragma unroll 1
        for (int piece = 0; piece < kPieces; ++piece) {
          float values[NMAT][kPiece];
          load_piece(piece, values);
#pragma unroll
          for (int a = 0; a < NMAT; ++a)
#pragma unroll
            for (int i = 0; i < kPiece / 4; ++i)
              *reinterpret_cast<float4*>(mine + ((size_t)a * kRows + tile_row) * NB + half_index * kHalf + piece * kPiece +
                                         4 * i) =
                  make_float4(values[a][4 * i], values[a][4 * i + 1], values[a][4 * i + 2], values[a][4 * i + 3]);
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        if (threadIdx.x == 64u) {
          __threadfence();
          const uint32_t before = atomicAdd(p.counters + tile_id, 1u);
          const bool last = before + 1u == p.splits;
          if (last) p.counters[tile_id] = 0u;
          holder[2] = last ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        finished = holder[2] != 0u;
        if (finished) {
          __threadfence();
          const float* parts = p.partials + (size_t)tile_id * p.splits * kPerTile;
#pragma unroll 1
          for (int piece = 0; piece < kPieces; ++piece) {
            float values[NMAT][kPiece];
#pragma unroll
            for (int a = 0; a < NMAT; ++a)
#pragma unroll
              for (int i = 0; i < kPiece; ++i) values[a][i] = 0.0f;
            for (uint32_t s = 0; s < p.splits; ++s)  // split order: the sum does not depend on who came last
#pragma unroll
              for (int a = 0; a < NMAT; ++a)
#pragma unroll
                for (int i = 0; i < kPiece / 4; ++i) {
                  const float4 part = __ldcg(reinterpret_cast<const float4*>(
                      parts + (size_t)s * kPerTile + ((size_t)a * kRows + tile_row) * NB + half_index * kHalf +
                      piece * kPiece + 4 * i));
                  values[a][4 * i] += part.x;
                  values[a][4 * i + 1] += part.y;
                  values[a][4 * i + 2] += part.z;
                  values[a][4 * i + 3] += part.w;
                }
            emit(piece, values);
          }
        }
      }
      if (kStacked && finished) {
        asm volatile("bar.sync 1, 512;" ::: "memory");
        // silu(gate) * up for the tile's 64 output columns: consecutive threads = consecutive columns
        const uint32_t first = threadIdx.x - 64u;
        for (uint32_t index = first; index < (kRows / 2) * NB; index += kConvertWarps * 32) {
          const uint32_t token = index / (kRows / 2), local = index % (kRows / 2);
          const uint32_t batch_row = token0 + token, column = n0 + local;
          if (batch_row >= p.m || column >= p.n) continue;
          const float g = stash[token * kRows + local], u = stash[token * kRows + kRows / 2 + local];
          p.out[(size_t)batch_row * p.n + column] = __float2half_rn((g / (1.0f + __expf(-g))) * u);  // lib/metal_w4a16_source.ml:571-575
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

template <int EPI, int NB, bool AFFINE = false>
int run_batch(const KernelArgs& args, const CUtensorMap& map_x, BatchProblem p) {
  constexpr int NMAT = (EPI == kBatchLinear || EPI == kBatchDualStacked || EPI == kBatchSplitF32) ? 1 : 2;
  constexpr uint32_t kTileRows = EPI == kBatchLinearPair ? 2 * kRows : EPI == kBatchDualStacked ? kRows / 2 : kRows;
  using L = Layout<NMAT, NB>;
  auto kernel = w4a16_gemm_tc_batch_kernel<EPI, NB, AFFINE>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  const uint32_t tiles = (p.n + kTileRows - 1) / kTileRows, row_tiles = (p.m + NB - 1) / NB;
  const uint32_t sms = (uint32_t)context_sm_count(args.ctx);
  const uint32_t groups = (p.k / kBK + L::kGroupBlocks - 1u) / L::kGroupBlocks;
  // one CTA per SM at most (a second wave would double the time); each split keeps at least two groups
  uint32_t splits = sms / (tiles * row_tiles);
  if (splits > groups / 2u) splits = groups / 2u;
  if (splits > 16u) splits = 16u;
  if (splits < 1u || tiles * row_tiles > kSplitCounterTiles) splits = 1u;
  p.splits = splits;
  if (splits > 1u) {
    constexpr size_t counter_bytes = kSplitCounterTiles * sizeof(uint32_t);
    const size_t partial_bytes = (size_t)tiles * row_tiles * splits * NMAT * kRows * NB * sizeof(float);
    uint8_t* scratch =
        (uint8_t*)context_split_scratch(args.ctx, counter_bytes, counter_bytes + partial_bytes, args.stream, args.error);
    if (scratch == nullptr) return 1;
    p.counters = reinterpret_cast<uint32_t*>(scratch);
    p.partials = reinterpret_cast<float*>(scratch + counter_bytes);
  }
  static std::atomic<uint32_t> launches{0};
  launch_kernel(args, kernel, dim3(tiles, splits, row_tiles), dim3(kThreads), L::kBytes, map_x, p,
                context_device_error(args.ctx), launches.fetch_add(1) + 1u);
  return check_launch(args);
}

}  // namespace

// Rows from which decode batches take this kernel (below it the small-M GEMV wins);
// LLMOPT_CUDA_TC_BATCH_MIN_ROWS overrides it, 0 disables the kernel.  Measured at the Llama-8B shapes
// (us in a back-to-back run over 32 operand sets, pipelined GEMV -> this kernel): 32 rows: gate/up 54.1 ->
// 36.7, down 35.2 -> 30.4, o_proj 11.2 -> 14.7, QKV (three launches here) 15.4 -> 42; 16 rows: gate/up
// 36.0 -> 35.4, down 17.2 -> 26.6.  So from 17 rows the large matrices take it, the small ones from 33.
uint32_t tensor_core_batch_min_rows() {
  static const uint32_t rows = []() -> uint32_t {
    const char* text = getenv("LLMOPT_CUDA_TC_BATCH_MIN_ROWS");
    if (text == nullptr) return 17u;
    const long value = strtol(text, nullptr, 10);
    return value <= 0 ? 0xffffffffu : (uint32_t)value;
  }();
  return rows;
}

// Rows up to which this kernel is taken (at most 64); LLMOPT_CUDA_TC_BATCH_MAX_ROWS overrides it.
uint32_t tensor_core_batch_max_rows() {
  static const uint32_t rows = []() -> uint32_t {
    const char* text = getenv("LLMOPT_CUDA_TC_BATCH_MAX_ROWS");
    if (text == nullptr) return 64u;
    const long value = strtol(text, nullptr, 10);
    return value <= 0 ? 0u : (value > 64 ? 64u : (uint32_t)value);
  }();
  return rows;
}

// Prompts (more than 64 rows) on this kernel: 128-row activation tiles, two weight tiles per CTA.
// LLMOPT_CUDA_TC_PROMPT_TMEM=0 sends them to the shared-memory-operand GEMM instead.
static bool prompt_rows_enabled() {
  static const bool enabled = []() {
    const char* text = getenv("LLMOPT_CUDA_TC_PROMPT_TMEM");
    return text == nullptr || text[0] != '0';
  }();
  return enabled;
}

// Decode batches (up to 64 rows) and prompts; returns -1 outside its domain (the caller falls back).
int launch_w4a16_gemm_tc_batch(const KernelArgs& args, const GemvProblem& problem, int epilogue, bool affine) {
  if (args.ctx == nullptr || problem.m < tensor_core_batch_min_rows() ||
      (problem.x_rows != problem.m && epilogue != kEpiSplitF32) || problem.k % 64 != 0 || problem.norm_weight != nullptr)
    return -1;
  const bool prompt = problem.m > tensor_core_batch_max_rows();
  if (prompt && (!prompt_rows_enabled() || problem.m <= 64)) return -1;
  // up to 32 rows only large matrices gain (measured: 58 M weights yes, 17 M no; the line is drawn at 24 M, which
  // keeps the halves of a two-way tensor-parallel split on this kernel)
  static const bool forced = getenv("LLMOPT_CUDA_TC_BATCH_MIN_ROWS") != nullptr;
  if (problem.m <= 32 && !forced &&
      (epilogue == kEpiQkv || (uint64_t)problem.mat[0].n * problem.k < (24ull << 20)))
    return -1;
  if (epilogue == kEpiQkv) {
    for (uint32_t i = 0; i < problem.matrices; ++i) {
      GemvProblem one = problem;
      one.mat[0] = problem.mat[i];
      one.matrices = 1;
      one.out[0] = problem.out[i];
      one.has_aux = 0;
      const int status = launch_w4a16_gemm_tc_batch(args, one, kEpiLinear, false);
      if (status != 0) return i == 0 ? status : (status < 0 ? 1 : status);
    }
    return 0;
  }
  if (epilogue == kEpiSplitF32) {
    // the LM head's hi/lo rows: 17..32 rows = up to 64 slot rows, one launch instead of two 16-row passes
    if (affine || prompt || problem.m > 32 || problem.x_rows > 64 || problem.x_rows % 8 != 0 || problem.out_f32 == nullptr ||
        ((uintptr_t)problem.x & 15u) != 0 || (problem.k / 2) % 16 != 0 || ((uintptr_t)problem.mat[0].packed & 15u) != 0)
      return -1;
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return -1;
    CUtensorMap map_x;
    const cuuint64_t dims[2] = {problem.k, problem.x_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)problem.k * 2};
    const cuuint32_t box[2] = {kBK, 64};
    const cuuint32_t element_strides[2] = {1, 1};
    if (encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(problem.x), dims, strides, box,
               element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -1;
    BatchProblem p = {};
    p.m = problem.m;
    p.n = problem.mat[0].n;
    p.k = problem.k;
    p.packed[0] = p.packed[1] = problem.mat[0].packed;
    p.scale[0] = p.scale[1] = problem.mat[0].scale;
    p.out_f32 = problem.out_f32;
    return run_batch<kBatchSplitF32, 64>(args, map_x, p);
  }
  if (epilogue != kEpiLinear && epilogue != kEpiDualSwiglu) return -1;
  if (problem.out_f32 != nullptr && (epilogue != kEpiLinear || problem.has_aux)) return -1;
  // the zero-point form: plain products of prompts only (what the shared-memory-operand GEMM covered)
  if (affine && (epilogue != kEpiLinear || !prompt || problem.mat[0].zero == nullptr)) return -1;
  const uint32_t matrices = epilogue == kEpiDualSwiglu ? 2u : 1u;
  if (((uintptr_t)problem.x & 15u) != 0 || (problem.k / 2) % 16 != 0) return -1;
  for (uint32_t i = 0; i < matrices; ++i)
    if (((uintptr_t)problem.mat[i].packed & 15u) != 0 || problem.mat[i].n != problem.mat[0].n) return -1;
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return -1;
  // prompts of 256 rows and more: 256-token tiles (an MMA with N = 256 runs at the tensor pipe's full rate,
  // narrower ones cost three quarters of that for half the work); LLMOPT_CUDA_TC_PROMPT_WIDE=0 keeps 128
  static const bool wide_prompts = getenv("LLMOPT_CUDA_TC_PROMPT_WIDE") == nullptr || getenv("LLMOPT_CUDA_TC_PROMPT_WIDE")[0] != '0';
  const bool wide = prompt && wide_prompts && problem.m >= 256;
  const uint32_t padded = wide ? 256u : prompt ? 128u : problem.m <= 16 ? 16u : problem.m <= 32 ? 32u : 64u;
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
    p.zero[i] = problem.mat[i < matrices ? i : 0].zero;
  }
  p.out = problem.out[0];
  p.out_f32 = problem.out_f32;
  p.aux = problem.aux0;
  p.aux_row_stride = problem.aux_row_stride;
  p.has_aux = problem.has_aux;
  if (prompt) {
    if (epilogue == kEpiDualSwiglu)
      return padded == 256 ? run_batch<kBatchDualStacked, 256>(args, map_x, p) : run_batch<kBatchDualSwiglu, 128>(args, map_x, p);
    if (affine) {
      if (padded == 256) return run_batch<kBatchLinear, 256, true>(args, map_x, p);
      return p.n > kRows ? run_batch<kBatchLinearPair, 128, true>(args, map_x, p) : run_batch<kBatchLinear, 128, true>(args, map_x, p);
    }
    if (padded == 256) return run_batch<kBatchLinear, 256>(args, map_x, p);
    return p.n > kRows ? run_batch<kBatchLinearPair, 128>(args, map_x, p) : run_batch<kBatchLinear, 128>(args, map_x, p);
  }
  if (epilogue == kEpiDualSwiglu) {
    switch (padded) {
      case 16: return run_batch<kBatchDualSwiglu, 16>(args, map_x, p);
      case 32: return run_batch<kBatchDualSwiglu, 32>(args, map_x, p);
      default: return run_batch<kBatchDualSwiglu, 64>(args, map_x, p);
    }
  }
  switch (padded) {
    case 16: return run_batch<kBatchLinear, 16>(args, map_x, p);
    case 32: return run_batch<kBatchLinear, 32>(args, map_x, p);
    default: return run_batch<kBatchLinear, 64>(args, map_x, p);
  }
}

}  // namespace llmopt
