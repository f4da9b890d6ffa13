// Prefill (M >= 64) W4A16 group-64 product on the 5th-generation tensor cores:
//   Y[M, N] = X[M, K] . dequant(W[N, K])^T, fp32 accumulate in tensor memory, one rounding to half.
// Restates lib/metal_w4a16_source.ml:60-212 (the reference's tiled simdgroup-matrix kernels for
// M > 1: dequantise a weight tile into threadgroup memory, multiply on the matrix units) for sm_100a.
//
// One CTA computes a 128 x 256 output tile (or 128 x 128 of silu(gate) * up in the dual form, the
// 256 tile rows being 128 gate rows and 128 up rows).  Per 64-wide k-block, which is exactly one
// quantisation group:
//   warp 0      TMA: the X tile [128 x 64] fp16 (128-byte swizzle) into a 4-deep ring, completion on an
//               mbarrier by byte count;
//   warps 10-11 the packed weight rows, four k-blocks (128 bytes per row, 32 KB per stage) at a time, by
//               cp.async into a 3-deep ring; completion reaches the stage's mbarrier through
//               cp.async.mbarrier.arrive.  Many threads with copies in flight sustain the HBM rate where
//               one TMA-issuing thread per SM does not;
//   warps 2-9   one thread per weight row: 32 packed bytes -> 64 exact integers in fp16 (PRMT + LOP3
//               + one subtract) -> times the group scale -> the row of the B tile in the canonical
//               K-major 128-byte-swizzled layout (2-deep ring); generic-proxy writes are published
//               to the tensor core with fence.proxy.async;
//   warp 1      one thread issues four tcgen05.mma (128 x 256 x 16, kind::f16) per k-block with the
//               accumulator in tensor memory; tcgen05.commit releases the ring stages.
// With few output tiles the k-blocks are split over grid.z: each split parks its fp32 partial tile, the
// last one to arrive (an atomic counter per tile) adds them in split order and runs the epilogue.
// After the last k-block the eight conversion warps read the accumulator (tcgen05.ld, each warp
// its 32-lane quarter and one column half), apply the epilogue and store halves.
//
// The weight rounding differs from the decode kernels in one place: the B operand is
// half(q * scale) (the tensor core needs fp16 operands), where the decode path scales the fp32
// group sum; the difference is below 2^-11 per weight and averages out over K.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the context's device error
// word and the CTA drains its copies, frees its tensor memory and returns.
#include <cuda.h>

#include <atomic>
#include <cstdlib>

#include "w4a16_tc_device.cuh"

namespace llmopt {
using namespace gemv;
using namespace tc;

uint32_t* context_device_error(Context* ctx);
// Scratch of the K-split protocol: grows on demand, earlier blocks stay valid for captured plans;
// the first `zeroed_bytes` of a new block are cleared on `stream` before its first user.
void* context_split_scratch(Context* ctx, size_t zeroed_bytes, size_t bytes, cudaStream_t stream, std::string* error);

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64;
// Rings: X tiles per k-block; packed weights per GROUP of four k-blocks (128 bytes per weight row and
// TMA request: full DRAM bursts and 96 KiB of weight stream in flight per SM, which is what keeps
// HBM busy when the weights are read once, i.e. for decode batches); converted B tiles per k-block.
constexpr int kAStages = 4, kRawStages = 3, kBStages = 2, kGroupBlocks = 4;
constexpr int kATileBytes = kBM * kBK * 2;                    // 16 KiB
constexpr int kRawTileBytes = kBN * kGroupBlocks * kBK / 2;   // 32 KiB: 256 rows x 128 bytes, 128-byte swizzle
constexpr int kBTileBytes = kBN * kBK * 2;                    // 32 KiB
constexpr int kConvertWarps = 8;
// X producer, MMA issuer, 8 conversion warps, 2 weight-producer warps
constexpr int kWeightProducerWarps = 2;
constexpr int kThreadsTc = (2 + kConvertWarps + kWeightProducerWarps) * 32;
constexpr int kWeightProducerWarp = 2 + kConvertWarps;  // first of them
constexpr uint32_t kTmemColumns = 256;
constexpr uint32_t kSplitCounterTiles = 1u << 14;  // output tiles whose split counters fit the scratch header

constexpr int kOffsetA = 0;
constexpr int kOffsetB = kOffsetA + kAStages * kATileBytes;
constexpr int kOffsetRaw = kOffsetB + kBStages * kBTileBytes;
constexpr int kOffsetBarriers = kOffsetRaw + kRawStages * kRawTileBytes;
constexpr int kBarrierCount = 2 * kAStages + 2 * kRawStages + 2 * kBStages + 1;
constexpr int kOffsetTmemHolder = kOffsetBarriers + kBarrierCount * 8;
constexpr int kOffsetAbort = kOffsetTmemHolder + 4;
constexpr int kOffsetLast = kOffsetAbort + 4;
constexpr int kSharedBytesTc = kOffsetLast + 4 + 1024;  // + slack to align the base to 1024 bytes

enum TcEpilogue { kTcLinear = 0, kTcDualSwiglu = 1, kTcTagged = 2 };

struct TcProblem {
  uint32_t m, n, k;  // n: output columns
  const uint8_t* packed[2];
  const __half* scale[2];
  const __half* zero[2];
  __half* out;
  const __half* aux0;
  const __half* aux1;
  uint32_t aux_row_stride;
  uint32_t has_aux;
  uint32_t tag;
  // K split over grid.z CTAs per output tile (few tiles, long K): every CTA parks its fp32 tile in
  // partials[tile][split], bumps counters[tile]; the last one adds all splits in split order and
  // runs the epilogue.  Nobody waits for anybody.
  uint32_t splits;
  float* partials;     // [tiles][splits][kBM][kBN]
  uint32_t* counters;  // [tiles], zero between launches
};

// Launch id of the last launch in which a bounded wait ran out (0: none).
__device__ uint32_t g_abandoned_launch = 0;

template <int EPI, bool AFFINE>
__global__ void __launch_bounds__(kThreadsTc, 1)
w4a16_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w0,
                     const __grid_constant__ CUtensorMap map_w1, const TcProblem p, uint32_t* error_word,
                     uint32_t launch_id) {
  extern __shared__ unsigned char shared_raw[];
  grid_chain_prologue();
  // A CTA that starts after another one of the same launch has given up does nothing, which
  // keeps a failing grid short.  The mark lives in device memory: the error word is pinned host
  // memory, and polling it from every CTA costs a PCIe round trip per thread.
  if (*reinterpret_cast<volatile uint32_t*>(&g_abandoned_launch) == launch_id) return;
  // 128-byte-swizzled tiles need 1024-byte alignment
  const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
  unsigned char* base_pointer = shared_raw + (base - smem_u32(shared_raw));
  const uint32_t a_full = base + kOffsetBarriers, a_empty = a_full + kAStages * 8;
  const uint32_t raw_full = a_empty + kAStages * 8, raw_empty = raw_full + kRawStages * 8;
  const uint32_t b_full = raw_empty + kRawStages * 8, b_empty = b_full + kBStages * 8;
  const uint32_t accumulator_full = b_empty + kBStages * 8;
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_pointer + kOffsetTmemHolder);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(base_pointer + kOffsetAbort);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  constexpr uint32_t columns_per_tile = EPI == kTcDualSwiglu ? kBN / 2 : kBN;
  const uint32_t n0 = blockIdx.x * columns_per_tile, m0 = blockIdx.y * kBM;
  // this CTA's share of K: whole groups of four k-blocks (the last group of K may be short)
  const uint32_t all_k_blocks = p.k / kBK, all_groups = (all_k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
  const uint32_t split = blockIdx.z;
  const uint32_t group_begin = (uint32_t)((uint64_t)all_groups * split / p.splits);
  const uint32_t group_end = (uint32_t)((uint64_t)all_groups * (split + 1u) / p.splits);
  const uint32_t kb_begin = group_begin * kGroupBlocks;
  const uint32_t k_blocks = min(group_end * kGroupBlocks, all_k_blocks) - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) {
      barrier_init(a_full + s * 8, 1);   // the producer's expect_tx arrival; completes by byte count
      barrier_init(a_empty + s * 8, 1);  // one tcgen05.commit
    }
    for (int s = 0; s < kRawStages; ++s) {
      barrier_init(raw_full + s * 8, kWeightProducerWarps * 32);  // one arrival per producer lane, when its copies land
      barrier_init(raw_empty + s * 8, 1);  // the commit after the group's last k-block
    }
    for (int s = 0; s < kBStages; ++s) {
      barrier_init(b_full + s * 8, kConvertWarps);  // one arrival per conversion warp
      barrier_init(b_empty + s * 8, 1);             // one tcgen05.commit
    }
    barrier_init(accumulator_full, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + kOffsetTmemHolder),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  auto give_up = [&]() {
    *abort_flag = 1u;
    g_abandoned_launch = launch_id;
    if (error_word) atomicExch(error_word, 1u);
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {  // kb counts this CTA's k-blocks
        const uint32_t s = kb % kAStages;
        if (*abort_flag || !barrier_wait(a_empty + s * 8, ((kb / kAStages) & 1u) ^ 1u)) {
          give_up();
          break;
        }
        barrier_expect_tx(a_full + s * 8, kATileBytes);
        tma_load_2d(base + kOffsetA + s * kATileBytes, &map_x, (int32_t)((kb_begin + kb) * kBK), (int32_t)m0, a_full + s * 8);
        issued = kb + 1;
      }
      if (*abort_flag) {
        // the copies already started must land before the shared memory goes away
        const uint32_t first = issued > kAStages ? issued - kAStages : 0u;
        for (uint32_t kb = first; kb < issued; ++kb) barrier_wait(a_full + (kb % kAStages) * 8, (kb / kAStages) & 1u);
      }
    }
  } else if (warp >= kWeightProducerWarp) {
    // ------------------------------ producers of the packed weights ------------------------------
    // 16-byte cp.async from every lane of two warps (one per 128 weight rows) instead of TMA: when the
    // weights are read once (decode batches) they come from HBM, and a TMA unit keeps too few requests
    // in flight for that latency (measured: ~10 GB/s per SM against ~30 needed).  The stream runs up
    // to kRawStages groups (twelve k-blocks) ahead of the math, whatever the depth of the X ring.
    const uint32_t half_index = warp - kWeightProducerWarp;  // rows [0,128) or [128,256) of the tile
    const uint8_t* packed = (EPI == kTcDualSwiglu && half_index == 1u) ? p.packed[1] : p.packed[0];
    const uint32_t first_row = EPI == kTcDualSwiglu ? n0 : n0 + half_index * (kBN / 2);
    const uint32_t row_bytes = p.k / 2;
    const uint32_t groups = (k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
    const uint32_t chunk = lane & 7u, row_in_pass = lane >> 3;  // 8 lanes copy one row's 128 bytes
    uint32_t issued = 0;
    bool ok = true;
    for (uint32_t group = 0; group < groups; ++group) {
      const uint32_t rs = group % kRawStages;
      ok = !*abort_flag && barrier_wait(raw_empty + rs * 8, ((group / kRawStages) & 1u) ^ 1u);
      if (!ok) {
        give_up();
        break;
      }
      const uint32_t stage = base + kOffsetRaw + rs * kRawTileBytes + half_index * (kRawTileBytes / 2);
      const uint32_t byte_at = (group_begin + group) * (kGroupBlocks * kBK / 2) + chunk * 16u;
      const uint32_t bytes = byte_at < row_bytes ? 16u : 0u;  // beyond the row end: zeros (K not a multiple of 256)
#pragma unroll 4
      for (uint32_t pass = 0; pass < (kBN / 2) / 4; ++pass) {
        const uint32_t row = pass * 4u + row_in_pass;                     // row of this half tile
        const uint32_t weight_row = min(first_row + row, p.n - 1u);        // absent rows re-read the last one
        const uint8_t* source = packed + (size_t)weight_row * row_bytes + (bytes ? byte_at : 0u);
        const uint32_t target = stage + row * 128u + ((chunk ^ (row & 7u)) * 16u);  // 128-byte swizzle
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(target), "l"(source), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_full + rs * 8) : "memory");
      issued = group + 1;
    }
    // the copies must have landed before this warp's shared memory can go away
    asm volatile("cp.async.wait_all;" ::: "memory");
    (void)issued;
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      bool ok = true;
      for (uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
        const uint32_t s = kb % kAStages, t = kb % kBStages;
        ok = !*abort_flag && barrier_wait(a_full + s * 8, (kb / kAStages) & 1u) &&
             barrier_wait(b_full + t * 8, (kb / kBStages) & 1u);
        if (!ok) {
          give_up();
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_tile = base + kOffsetA + s * kATileBytes, b_tile = base + kOffsetB + t * kBTileBytes;
#pragma unroll
        for (int j = 0; j < kBK / 16; ++j)
          mma_f16(tmem_base, operand_descriptor(a_tile + j * 32), operand_descriptor(b_tile + j * 32),
                  (kb > 0 || j > 0) ? 1u : 0u);
        mma_commit(a_empty + s * 8);
        mma_commit(b_empty + t * 8);
        // the conversions of a group's last k-block are behind these MMAs: its packed bytes are free
        if (kb % kGroupBlocks == kGroupBlocks - 1u || kb + 1u == k_blocks)
          mma_commit(raw_empty + ((kb / kGroupBlocks) % kRawStages) * 8);
      }
      if (ok) mma_commit(accumulator_full);
    }
  } else {
    // ------------------------------ conversion, then epilogue ------------------------------
    const uint32_t row = threadIdx.x - 64u;  // row of the B tile, 0..255
    const uint32_t matrix = EPI == kTcDualSwiglu ? row / (kBN / 2) : 0u;
    const uint32_t weight_row = EPI == kTcDualSwiglu ? n0 + row % (kBN / 2) : n0 + row;
    const bool row_present = weight_row < p.n;
    const uint32_t groups = p.k / 64;
    const __half* scale_row = p.scale[matrix] + (size_t)(row_present ? weight_row : 0u) * groups;
    const __half* zero_row = AFFINE ? p.zero[matrix] + (size_t)(row_present ? weight_row : 0u) * groups : nullptr;
    const uint32_t swizzle = (row & 7u) * 16u;
    bool ok = true;
    __half next_scale = row_present ? __ldg(scale_row + kb_begin) : __float2half(0.0f);
    __half next_zero = AFFINE && row_present ? __ldg(zero_row + kb_begin) : __float2half(0.0f);
    for (uint32_t kb = 0; kb < k_blocks; ++kb) {
      const uint32_t t = kb % kBStages, group = kb / kGroupBlocks, quarter_of_group = kb % kGroupBlocks;
      const uint32_t rs = group % kRawStages;
      const __half scale = next_scale, zero = next_zero;
      if (kb + 1 < k_blocks && row_present) {
        next_scale = __ldg(scale_row + kb_begin + kb + 1);
        if (AFFINE) next_zero = __ldg(zero_row + kb_begin + kb + 1);
      }
      ok = !*abort_flag && (quarter_of_group != 0u || barrier_wait(raw_full + rs * 8, (group / kRawStages) & 1u)) &&
           barrier_wait(b_empty + t * 8, ((kb / kBStages) & 1u) ^ 1u);
      if (!ok) {
        give_up();
        break;
      }
      // the row's 128 packed bytes of the group sit 128-byte swizzled: 16-byte chunk c at (c ^ (row & 7))
      const unsigned char* raw = base_pointer + kOffsetRaw + rs * kRawTileBytes + row * 128u;
      const uint4 first = *reinterpret_cast<const uint4*>(raw + (((2u * quarter_of_group) * 16u) ^ swizzle));
      const uint4 second = *reinterpret_cast<const uint4*>(raw + (((2u * quarter_of_group + 1u) * 16u) ^ swizzle));
      const uint32_t words[8] = {first.x, first.y, first.z, first.w, second.x, second.y, second.z, second.w};
      const __half2 scale_pair = __halves2half2(scale, __hmul(scale, __float2half(0.0625f)));
      const __half2 zero_pair = __halves2half2(zero, __hmul(zero, __float2half(16.0f)));
      const uint32_t scales = *reinterpret_cast<const uint32_t*>(&scale_pair);
      const uint32_t zeros = *reinterpret_cast<const uint32_t*>(&zero_pair);
      unsigned char* b_row = base_pointer + kOffsetB + t * kBTileBytes + row * 128u;
#pragma unroll
      for (int c = 0; c < 8; ++c) {  // word c = k 8c .. 8c+7 = 16-byte chunk c of the row
        uint4 chunk;
        chunk.x = dequant_pair<AFFINE, 0>(words[c], scales, zeros);
        chunk.y = dequant_pair<AFFINE, 1>(words[c], scales, zeros);
        chunk.z = dequant_pair<AFFINE, 2>(words[c], scales, zeros);
        chunk.w = dequant_pair<AFFINE, 3>(words[c], scales, zeros);
        *reinterpret_cast<uint4*>(b_row + ((c * 16u) ^ swizzle)) = chunk;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // publish to the tensor core's proxy
      __syncwarp();
      if (lane == 0) barrier_arrive(b_full + t * 8);
    }

    // epilogue: this warp reads its lane quarter and one half of the columns
    ok = ok && !*abort_flag && barrier_wait(accumulator_full, 0u);
    if (!ok) give_up();
    {
      // one decision for all eight epilogue warps: the steps below synchronise among them
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
      const uint32_t quarter = warp & 3u, half_index = (warp - 2u) >> 2;
      const uint32_t tile_row = quarter * 32u + lane, out_row = m0 + tile_row;
      const uint32_t lane_address = tmem_base + ((quarter * 32u) << 16);
      bool combine = false;  // sums come from the parked tiles of all splits instead of tensor memory
      const uint32_t tile = blockIdx.y * gridDim.x + blockIdx.x;
      const float* tile_partials = p.partials + (size_t)tile * p.splits * (kBM * kBN);
      if (p.splits > 1u) {
        // park this CTA's fp32 tile (rows that exist only), count it, and go on only as the last split
        float* mine = p.partials + ((size_t)tile * p.splits + split) * (kBM * kBN) + (size_t)tile_row * kBN;
#pragma unroll 1
        for (uint32_t piece = 0; piece < 4; ++piece) {
          const uint32_t column = half_index * 128u + piece * 32u;
          uint32_t values[32];
          tmem_load_32(lane_address + column, values);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (out_row < p.m) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<uint4*>(mine + column)[i] =
                  make_uint4(values[4 * i], values[4 * i + 1], values[4 * i + 2], values[4 * i + 3]);
          }
        }
        volatile uint32_t* last_flag = reinterpret_cast<volatile uint32_t*>(base_pointer + kOffsetLast);
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps
        if (threadIdx.x == 64u) {
          __threadfence();  // publishes the tile the barrier ordered before this thread
          const uint32_t before = atomicAdd(p.counters + tile, 1u);
          const bool last = before + 1u == p.splits;
          if (last) p.counters[tile] = 0u;  // ready for the next launch
          *last_flag = last ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        combine = *last_flag != 0u;
        if (combine) __threadfence();
      }
      // 32 consecutive accumulator columns of this thread's row
      auto load_columns = [&](uint32_t column, uint32_t (&values)[32]) {
        if (!combine) {
          tmem_load_32(lane_address + column, values);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          return;
        }
        float sums[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) sums[i] = 0.0f;
        if (out_row < p.m) {
          for (uint32_t s = 0; s < p.splits; ++s) {  // split order: the sum does not depend on who came last
            const float4* source =
                reinterpret_cast<const float4*>(tile_partials + (size_t)s * (kBM * kBN) + (size_t)tile_row * kBN + column);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 part = __ldcg(source + i);
              sums[4 * i] += part.x;
              sums[4 * i + 1] += part.y;
              sums[4 * i + 2] += part.z;
              sums[4 * i + 3] += part.w;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) values[i] = __float_as_uint(sums[i]);
      };
      if (p.splits > 1u && !combine) {
        // another CTA finishes this tile
      } else if (EPI == kTcDualSwiglu) {
        // columns [0, 128) gate, [128, 256) up; this warp covers 64 output columns
#pragma unroll 1
        for (uint32_t piece = 0; piece < 2; ++piece) {
          const uint32_t column = half_index * 64u + piece * 32u;
          uint32_t gate[32], up[32];
          load_columns(column, gate);
          load_columns(kBN / 2 + column, up);
          if (out_row < p.m) {
            const size_t out_index = (size_t)out_row * p.n + n0 + column;
            __half* target = p.out + out_index;
            // silu in fp32, one rounding of the product: lib/metal_w4a16_source.ml:571-575
            auto gated = [&](int i) {
              const float g = __uint_as_float(gate[i]);
              return (g / (1.0f + __expf(-g))) * __uint_as_float(up[i]);
            };
            if (n0 + column + 32u <= p.n && (out_index & 7u) == 0) {
              uint32_t packed[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const __half2 pair = __floats2half2_rn(gated(2 * i), gated(2 * i + 1));
                packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(target)[i] =
                    make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n0 + column + i < p.n) target[i] = __float2half_rn(gated(i));
            }
          }
        }
      } else {
#pragma unroll 1
        for (uint32_t piece = 0; piece < 4; ++piece) {
          const uint32_t column = half_index * 128u + piece * 32u;
          uint32_t values[32];
          load_columns(column, values);
          if (out_row < p.m) {
            const size_t out_index = (size_t)out_row * p.n + n0 + column;
            const bool whole = n0 + column + 32u <= p.n && (out_index & 7u) == 0;
            if (EPI == kTcLinear && whole && !p.has_aux) {
              uint32_t packed[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const __half2 pair = __floats2half2_rn(__uint_as_float(values[2 * i]), __uint_as_float(values[2 * i + 1]));
                packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
              }
              uint4* target = reinterpret_cast<uint4*>(p.out + out_index);
#pragma unroll
              for (int i = 0; i < 4; ++i) target[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const uint32_t col = n0 + column + i;
                if (col < p.n) {
                  float value = __uint_as_float(values[i]);
                  if (EPI == kTcTagged) {
                    const float first = p.aux0 ? __half2float(p.aux0[col]) : 0.0f;
                    const float second = p.aux1 ? __half2float(p.aux1[col]) : 0.0f;
                    p.out[out_index + i] = __float2half_rn(epilogue_tagged(p.tag, value, first, second));
                  } else {
                    if (p.has_aux) value += __half2float(p.aux0[(size_t)out_row * p.aux_row_stride + col]);
                    p.out[out_index + i] = __float2half_rn(value);
                  }
                }
              }
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  }

  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
  }
}

// cuTensorMapEncodeTiled, resolved through the runtime so that the library does not link libcuda.
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

bool make_map(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t outer,
              uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, type, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI, bool AFFINE>
int run_tc(const KernelArgs& args, const CUtensorMap& map_x, const CUtensorMap& map_w0, const CUtensorMap& map_w1,
           const TcProblem& p) {
  auto kernel = w4a16_gemm_tc_kernel<EPI, AFFINE>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedBytesTc) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  constexpr uint32_t columns_per_tile = EPI == kTcDualSwiglu ? kBN / 2 : kBN;
  dim3 grid((p.n + columns_per_tile - 1) / columns_per_tile, (p.m + kBM - 1) / kBM, 1);
  TcProblem problem = p;
  // Few output tiles and a long K (decode batches, narrow projections): split K over enough CTAs to
  // occupy the machine; every split keeps at least four k-blocks.
  const uint32_t tiles = grid.x * grid.y, sms = (uint32_t)context_sm_count(args.ctx), k_blocks = p.k / kBK;
  problem.splits = 1;
  if (tiles * 2u <= sms) {
    const uint32_t groups = (k_blocks + kGroupBlocks - 1u) / kGroupBlocks;
    uint32_t splits = sms / tiles;
    if (splits > groups / 2u) splits = groups / 2u;  // at least two groups (eight k-blocks) per split
    if (splits > 16u) splits = 16u;
    if (splits > 1u && tiles <= kSplitCounterTiles) problem.splits = splits;
  }
  if (problem.splits > 1u) {
    constexpr size_t counter_bytes = kSplitCounterTiles * sizeof(uint32_t);
    const size_t partial_bytes = (size_t)tiles * problem.splits * kBM * kBN * sizeof(float);
    uint8_t* scratch =
        (uint8_t*)context_split_scratch(args.ctx, counter_bytes, counter_bytes + partial_bytes, args.stream, args.error);
    if (scratch == nullptr) return 1;
    problem.counters = reinterpret_cast<uint32_t*>(scratch);
    problem.partials = reinterpret_cast<float*>(scratch + counter_bytes);
    grid.z = problem.splits;
  }
  static std::atomic<uint32_t> launches{0};
  launch_kernel(args, kernel, grid, dim3(kThreadsTc), kSharedBytesTc, map_x, map_w0, map_w1, problem,
                context_device_error(args.ctx), launches.fetch_add(1) + 1u);
  return check_launch(args);
}

}  // namespace

// Fewest rows that take the tensor-core path.  With one 128-row tile the kernel streams the
// weights once at the rate of the tensor pipe, which beats the small-M kernel well below 64 rows;
// LLMOPT_CUDA_TC_MIN_ROWS overrides the threshold.
uint32_t tensor_core_min_rows() {
  static const uint32_t rows = []() -> uint32_t {
    const char* text = getenv("LLMOPT_CUDA_TC_MIN_ROWS");
    const long value = text ? strtol(text, nullptr, 10) : 0;
    return value > 0 ? (uint32_t)value : 64u;
  }();
  return rows;
}

// Tensor-core path for M >= tensor_core_min_rows(); returns -1 when the shape or the pointers are outside its domain
// (the caller then falls back to passes of the small-M kernel).
int launch_w4a16_gemm_tc(const KernelArgs& args, const GemvProblem& problem, int epilogue, bool affine) {
  if (args.ctx == nullptr || problem.m < tensor_core_min_rows() || problem.k % 64 != 0) return -1;
  if (epilogue == kEpiQkv) {
    // three independent products of the same activations: one launch each
    for (uint32_t i = 0; i < problem.matrices; ++i) {
      GemvProblem one = problem;
      one.mat[0] = problem.mat[i];
      one.matrices = 1;
      one.out[0] = problem.out[i];
      one.has_aux = 0;
      const int status = launch_w4a16_gemm_tc(args, one, kEpiLinear, false);
      if (status != 0) return i == 0 ? status : (status < 0 ? 1 : status);
    }
    return 0;
  }
  if (epilogue != kEpiLinear && epilogue != kEpiDualSwiglu && epilogue != kEpiTagged) return -1;
  if (affine && epilogue != kEpiLinear) return -1;
  const uint32_t matrices = epilogue == kEpiDualSwiglu ? 2u : 1u;
  if (((uintptr_t)problem.x & 15u) != 0) return -1;
  for (uint32_t i = 0; i < matrices; ++i)
    if (((uintptr_t)problem.mat[i].packed & 15u) != 0 || problem.mat[i].n != problem.mat[0].n) return -1;

  CUtensorMap map_x, map_w[2];
  if (!make_map(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, problem.x, problem.k, problem.m, (uint64_t)problem.k * 2, kBK,
                kBM, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  for (uint32_t i = 0; i < 2; ++i) {
    const GemvMatrix& mat = problem.mat[i < matrices ? i : 0];
    if (!make_map(&map_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, mat.packed, problem.k / 2, mat.n, problem.k / 2,
                  kGroupBlocks * kBK / 2, kBN / 2, CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
  }
  TcProblem p = {};
  p.m = problem.m;
  p.n = problem.mat[0].n;
  p.k = problem.k;
  for (uint32_t i = 0; i < 2; ++i) {
    p.packed[i] = problem.mat[i < matrices ? i : 0].packed;
    p.scale[i] = problem.mat[i < matrices ? i : 0].scale;
    p.zero[i] = problem.mat[i < matrices ? i : 0].zero;
  }
  p.out = problem.out[0];
  p.aux0 = problem.aux0;
  p.aux1 = problem.aux1;
  p.aux_row_stride = problem.aux_row_stride;
  p.has_aux = problem.has_aux;
  p.tag = problem.tag;
  if (epilogue == kEpiDualSwiglu) return run_tc<kTcDualSwiglu, false>(args, map_x, map_w[0], map_w[1], p);
  if (epilogue == kEpiTagged) return run_tc<kTcTagged, false>(args, map_x, map_w[0], map_w[1], p);
  return affine ? run_tc<kTcLinear, true>(args, map_x, map_w[0], map_w[1], p)
                : run_tc<kTcLinear, false>(args, map_x, map_w[0], map_w[1], p);
}

}  // namespace llmopt
