// Pipelined W4A16 group-64 decode product: the HBM-bound fast path of
// w4a16_gemv.cu for K a multiple of 512 (same storage contract, same outputs).
//
// Why a second kernel: the direct-load kernel keeps only a few 8-byte loads per
// lane in flight and pays address arithmetic and a nibble-bias subtraction per
// weight; at the Llama FFN shapes it is latency- and issue-bound at a quarter of
// the HBM roofline (the memory system here needs on the order of 100 KB per SM in
// flight to stream at its rate).  This kernel separates the two jobs:
//   * a PRODUCER warp streams the packed weights and scales of 16-column tiles
//     into a deep shared-memory ring with 16-byte asynchronous copies (cp.async,
//     two 256-byte row pieces per warp instruction) whose completion arrives on
//     one mbarrier per ring stage (cp.async.mbarrier.arrive); bytes in flight are bounded by shared memory
//     only, not by registers or by the consumers' progress;
//   * eight CONSUMER warps wait on a stage's "full" barrier, each takes one group
//     of 64 of the stage's 512 k, and release the stage on its "empty" barrier —
//     no CTA-wide barrier and no copy instructions on the math path;
//   * shared rows are padded by 32 bytes, so the 8-byte fragment reads of a
//     half-warp (4 rows x 32 bytes) fall in distinct banks;
//   * for small activation blocks (M*K <= 16 Ki elements) the activations sit in
//     shared memory already in MMA fragment order, and the nibble bias is not
//     subtracted per weight: even nibbles enter the MMA as 1032 + q, odd ones as
//     72 + q (one LOP3 each, exact fp16 integers), and the per-group term
//     1032*sum(x_even) + 72*sum(x_odd), computed once per CTA in fp32, is removed
//     from the group sum before it is scaled — products stay exact, the fp32
//     group sums differ from the unbiased form by fp32 rounding (~1e-5 of the
//     group magnitude);
//   * tiles are dealt round-robin to a grid sized so every CTA gets the same
//     number of tiles; the consumers' partial sums are added in fixed order.
// Every wait on an mbarrier is bounded: after kSpinLimit polls the warp records
// an error word the host checks and goes on without waiting, still taking part in
// every later barrier, so the kernel always terminates.
#include <cstdlib>

#include "w4a16_gemv_device.cuh"

namespace llmopt {
using namespace gemv;

uint32_t* context_device_error(Context* ctx);

namespace {

// A ring stage holds GPW groups of 64 k for each of the 8 consumer warps:
// 512*GPW k of 16 weight rows (+32 bytes of padding per row) and their scales.
// More groups per warp and stage = more independent work per wait (the math of
// one group is a dependent chain) and less per-stage overhead.
template <int GPW> struct Stage {
  static constexpr int kChunkK = 512 * GPW;
  static constexpr int kRowBytes = kChunkK / 2 + 32;
  static constexpr int kWeights = 16 * kRowBytes;
  static constexpr int kScaleRow = 16 * GPW;  // 8*GPW fp16 scales per row
  static constexpr int kBytes = kWeights + 16 * kScaleRow;
};
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr uint32_t kSpinLimit = 1u << 18;    // polls of ~0.1 us: tens of milliseconds at most

__device__ __forceinline__ uint32_t shared_address(const void* pointer) {
  return (uint32_t)__cvta_generic_to_shared(pointer);
}
__device__ __forceinline__ void mbarrier_init(uint32_t barrier, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(barrier), "r"(count));
}
__device__ __forceinline__ void mbarrier_arrive(uint32_t barrier) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barrier) : "memory");
}
__device__ __forceinline__ bool mbarrier_test(uint32_t barrier, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(barrier), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait: false (and an error word) if the phase never completed.
__device__ __forceinline__ bool mbarrier_wait(uint32_t barrier, uint32_t parity, uint32_t* error_word) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
    if (mbarrier_test(barrier, parity)) return true;
  atomicExch(error_word, 1u);
  return false;
}
// 16-byte asynchronous copy global -> shared (bypassing L1), and the arrival on an
// mbarrier that fires once all earlier copies of this thread have landed.
__device__ __forceinline__ void copy_16(uint32_t destination, const void* source) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(destination), "l"(source) : "memory");
}
__device__ __forceinline__ void arrive_when_copied(uint32_t barrier) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(barrier) : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// (word & mask) ^ constant with the exponent of 1024 (even nibbles) or 64 (odd
// nibbles) and bit 3 of the nibble flipped: the halves read 1032 + q and 72 + q.
__device__ __forceinline__ void nibbles_biased(uint32_t word, uint32_t& even_pair, uint32_t& odd_pair) {
  even_pair = lop3_and_xor(word, 0x000F000Fu, 0x64086408u);
  odd_pair = lop3_and_xor(word, 0x00F000F0u, 0x54805480u);
}

// D = A B + C with C in registers of its own (the first MMA of a group takes the group's bias
// term as C, so the sum needs no seeding moves).
__device__ __forceinline__ void mma_16816_from(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

// The GPW consecutive fp16 group scales of one weight row as floats: one shared-memory load.
template <int GPW>
__device__ __forceinline__ void load_scales(const unsigned char* address, float (&scales)[GPW]) {
  if (GPW == 1) {
    scales[0] = __half2float(*reinterpret_cast<const __half*>(address));
  } else if (GPW == 2) {
    const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(address));
    scales[0] = pair.x;
    scales[GPW - 1] = pair.y;
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(address);
    const float2 low = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 high = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    scales[0] = low.x;
    scales[1 % GPW] = low.y;
    scales[2 % GPW] = high.x;
    scales[3 % GPW] = high.y;
  }
}

// The LM-head form (fp32 candidates, tens of tiles per CTA, light epilogue) gains from a fourth
// resident CTA per SM (more warps to hide the LOP3 -> MMA latency: 109 -> 87 us at 128256 x 4096);
// the projections, with two or three tiles per CTA, do not.
// With one batch tile a single warp can finish a tile's reduction quickly enough that the others
// need not wait for it (see the end of the tile loop); wider accumulators keep the CTA-wide form,
// and so does the LM-head form, whose tiles are shorter than its ring (the warps that ran ahead
// would only spin on the reducer).
template <int NT, int EPI> constexpr bool kLazyReduce = NT == 1 && EPI != kEpiSplitF32;

template <int NT, int EPI> constexpr int kDenseResidency = NT == 1 ? (EPI == kEpiSplitF32 ? 4 : 3) : 1;

// RES: resident CTAs per SM the kernel is compiled for (its register budget).  Launches that fill at
// most two CTA slots per SM take the RES = 2 build of the one-batch-tile forms: with up to 112
// registers the compiler keeps several groups' loads and LOP3 -> MMA chains in flight per warp
// (o_proj at 4096 x 4096: 6.8 -> 5.4 us).
//
// ONE: the activation block is a single row (the decode shape).  Only column 0 of every MMA result
// is a real output then, so the kernel keeps two accumulators per matrix instead of four, applies two
// scale FMAs per group instead of four, reads one bias term per group instead of two, and hands
// the bias to the first MMA of a group as its C operand (no register moves to seed the sum).
template <int NT, int NMAT, int EPI, bool SMALLX, int GPW, int RES = kDenseResidency<NT, EPI>, bool ONE = false>
__global__ void __launch_bounds__(kThreads, RES) w4a16_gemv_pipe_kernel(const GemvProblem p, const uint32_t stage_count,
                                                                   uint32_t* error_word) {
  static_assert(!ONE || (SMALLX && NT == 1), "the one-row form is a staged-activation, one-batch-tile form");
  extern __shared__ __align__(16) unsigned char shared[];
  // The next kernel of the stream may start its launch now; the producer warp below
  // streams weights (which no kernel writes) without waiting for the previous kernel,
  // the consumer warps wait for it before they read the activations.
  grid_launch_dependents();
  constexpr int kAcc = NMAT * NT * 4;
  constexpr int kChunkK = Stage<GPW>::kChunkK, kRowBytes = Stage<GPW>::kRowBytes;
  constexpr int kStageWeights = Stage<GPW>::kWeights, kScaleRow = Stage<GPW>::kScaleRow;
  constexpr int kStageBytes = Stage<GPW>::kBytes;
  const uint32_t groups = p.k >> 6;
  // [full barriers | empty barriers | reduction words] [ring] [reduce] [x fragments] [x bias]
  uint64_t* barriers = reinterpret_cast<uint64_t*>(shared);
  // two words after the barriers: arrivals at the current tile's reduction, tiles reduced so far
  volatile uint32_t* reduce_sync = reinterpret_cast<volatile uint32_t*>(shared + stage_count * 16u);
  unsigned char* stages = shared + stage_count * 16u + 16u;
  float* reduce = reinterpret_cast<float*>(stages + stage_count * (NMAT * kStageBytes));  // [8][kAcc][32]
  uint4* x_fragments = reinterpret_cast<uint4*>(reduce + kConsumerWarps * kAcc * 32);     // [groups][2][x_rows][4]
  float* x_bias = reinterpret_cast<float*>(x_fragments + (SMALLX ? groups * 2 * p.x_rows * 4 + 1 : 0));
  const uint32_t full_base = shared_address(barriers);
  const uint32_t empty_base = full_base + stage_count * 8u;

  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t chunks_per_tile = p.k / kChunkK;
  const uint32_t half_k = p.k >> 1;

  uint32_t tiles[3] = {0, 0, 0}, total_tiles = 0;
  if (EPI == kEpiQkv) {
    for (uint32_t i = 0; i < p.matrices; ++i) {
      tiles[i] = (p.mat[i].n + 15u) >> 4;
      total_tiles += tiles[i];
    }
  } else {
    tiles[0] = (p.mat[0].n + 15u) >> 4;
    total_tiles = tiles[0];
  }
  const uint32_t my_tiles = blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;

  auto locate = [&](uint32_t tile, uint32_t& matrix, uint32_t& local_tile) {
    matrix = 0;
    local_tile = tile;
    if (EPI == kEpiQkv) {
      if (local_tile >= tiles[0]) { local_tile -= tiles[0]; matrix = 1; }
      if (matrix == 1 && local_tile >= tiles[1]) { local_tile -= tiles[1]; matrix = 2; }
    }
  };

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < stage_count; ++s) {
      mbarrier_init(full_base + s * 8u, 32);                // one arrival per producer lane, when its copies land
      mbarrier_init(empty_base + s * 8u, kConsumerWarps);   // one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    reduce_sync[0] = 0u;
    reduce_sync[1] = 0u;
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    uint32_t stage = 0, parity = 1;  // a fresh "empty" barrier reads as released
    bool aborted = false;
    for (uint32_t slot = 0; slot < my_tiles; ++slot) {
      uint32_t matrix, local_tile;
      locate(blockIdx.x + slot * gridDim.x, matrix, local_tile);
      for (uint32_t chunk = 0; chunk < chunks_per_tile; ++chunk) {
        if (!aborted) aborted = !mbarrier_wait(empty_base + stage * 8u, parity, error_word);
        const uint32_t full = full_base + stage * 8u;
        if (!aborted) {
          const uint32_t target = shared_address(stages + stage * (NMAT * kStageBytes));
#pragma unroll
          for (int a = 0; a < NMAT; ++a) {
            const GemvMatrix& mat = p.mat[EPI == kEpiQkv ? matrix : a];
            // one warp instruction copies 512 contiguous bytes of one row
            constexpr int kPerRow = kChunkK / 2 / 512;  // instructions per row piece (GPW/2, at least... see below)
            if (kPerRow >= 1) {
#pragma unroll
              for (int row_in_tile = 0; row_in_tile < 16; ++row_in_tile) {
                const uint32_t row = min(local_tile * 16u + row_in_tile, mat.n - 1u);
                const unsigned char* source = mat.packed + (size_t)row * half_k + (size_t)chunk * (kChunkK / 2) + lane * 16;
#pragma unroll
                for (int part = 0; part < (kPerRow >= 1 ? kPerRow : 1); ++part)
                  copy_16(target + a * kStageBytes + row_in_tile * kRowBytes + part * 512 + lane * 16, source + part * 512);
              }
            } else {
              // 256-byte row pieces: two rows per instruction
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const uint32_t row_in_tile = 2 * i + (lane >> 4);
                const uint32_t row = min(local_tile * 16u + row_in_tile, mat.n - 1u);
                copy_16(target + a * kStageBytes + row_in_tile * kRowBytes + (lane & 15u) * 16,
                        mat.packed + (size_t)row * half_k + (size_t)chunk * (kChunkK / 2) + (lane & 15u) * 16);
              }
            }
            // scales: 16 rows x kScaleRow bytes = 16*GPW sixteen-byte pieces
#pragma unroll
            for (int i = 0; i < (16 * GPW + 31) / 32; ++i) {
              const uint32_t piece = i * 32 + lane;
              if (piece < 16u * GPW) {
                const uint32_t row_in_tile = piece / GPW, part = piece % GPW;
                const uint32_t row = min(local_tile * 16u + row_in_tile, mat.n - 1u);
                copy_16(target + a * kStageBytes + kStageWeights + row_in_tile * kScaleRow + part * 16,
                        reinterpret_cast<const unsigned char*>(mat.scale + (size_t)row * groups) +
                            (size_t)chunk * kScaleRow + part * 16);
              }
            }
          }
        }
        arrive_when_copied(full);
        if (++stage == stage_count) {
          stage = 0;
          parity ^= 1u;
        }
      }
    }
    // the copies must have landed before this warp's shared memory can go away
    asm volatile("cp.async.wait_all;" ::: "memory");
    return;
  }

  // ------------------------------ consumers ------------------------------
  grid_dependency_wait();
  const uint32_t r = lane >> 2, c = lane & 3u;
  if (SMALLX) {
    // activations -> shared in MMA fragment order: unit ((g*2 + h)*x_rows + row)*4 + c holds
    // x[row][64g + 16c + 8h + {0,4,1,5,2,6,3,7}]
    const uint32_t units = groups * 2 * p.x_rows * 4;
    const bool single_row = p.x_rows == 1u;
    // A folded RMS norm: warp w owns row w (at most 8 rows here) and leaves 1 / rms in shared memory.
    float* inverse_rms = reinterpret_cast<float*>(reduce);  // free until the first tile is reduced
    if (p.norm_weight != nullptr) {
      if (warp < p.x_rows) {
        float squares = 0.0f;
        for (uint32_t i = lane * 8u; i < p.k; i += 256u) {
          const uint4 raw = *reinterpret_cast<const uint4*>(p.x + (size_t)warp * p.k + i);
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&words[j]));
            squares = fmaf(pair.x, pair.x, squares);
            squares = fmaf(pair.y, pair.y, squares);
          }
        }
        squares = warp_sum(squares);
        if (lane == 0) inverse_rms[warp] = rsqrtf(squares / (float)p.k + p.norm_epsilon);
      }
      consumer_barrier();
    }
    for (uint32_t unit = threadIdx.x; unit < units; unit += kConsumerWarps * 32) {
      const uint32_t cc = unit & 3u, row = (unit >> 2) % p.x_rows, gh = (unit >> 2) / p.x_rows;
      const uint32_t k_at = (gh >> 1) * 64 + cc * 16 + (gh & 1u) * 8;
      uint4 source = *reinterpret_cast<const uint4*>(p.x + (size_t)row * p.k + k_at);
      if (p.norm_weight != nullptr) {
        // half((x inv) w) or half((x w) inv), exactly what the stand-alone norm kernels round to
        const uint4 weights = *reinterpret_cast<const uint4*>(p.norm_weight + k_at);
        const float inverse = inverse_rms[row];
        const uint32_t x_words[4] = {source.x, source.y, source.z, source.w};
        const uint32_t w_words[4] = {weights.x, weights.y, weights.z, weights.w};
        uint32_t y_words[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&x_words[j]));
          const float2 w = __half22float2(*reinterpret_cast<const __half2*>(&w_words[j]));
          const __half2 y = p.norm_weight_first ? __floats2half2_rn((x.x * w.x) * inverse, (x.y * w.y) * inverse)
                                                : __floats2half2_rn((x.x * inverse) * w.x, (x.y * inverse) * w.y);
          y_words[j] = *reinterpret_cast<const uint32_t*>(&y);
        }
        source = make_uint4(y_words[0], y_words[1], y_words[2], y_words[3]);
        if (blockIdx.x == 0 && p.norm_out != nullptr)
          *reinterpret_cast<uint4*>(p.norm_out + (size_t)row * p.k + k_at) = source;
      }
      uint4 permuted;
      permuted.x = prmt(source.x, source.z, 0x5410u);
      permuted.y = prmt(source.x, source.z, 0x7632u);
      permuted.z = prmt(source.y, source.w, 0x5410u);
      permuted.w = prmt(source.y, source.w, 0x7632u);
      x_fragments[unit] = permuted;
      if (single_row) {
        // one row: the eight units of a group sit in eight neighbouring lanes, so the group's
        // bias term is a fixed-order butterfly over them and needs no second pass
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&source.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&source.y));
        const float2 c2 = __half22float2(*reinterpret_cast<const __half2*>(&source.z));
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&source.w));
        float even = (a.x + b.x) + (c2.x + d.x), odd = (a.y + b.y) + (c2.y + d.y);
#pragma unroll
        for (int step = 1; step < 8; step <<= 1) {
          even += __shfl_xor_sync(0xffffffffu, even, step);
          odd += __shfl_xor_sync(0xffffffffu, odd, step);
        }
        if ((unit & 7u) == 0u) x_bias[unit >> 3] = -(1032.0f * even + 72.0f * odd);  // stored negated
      }
    }
    if (!single_row) consumer_barrier();
    // several rows: per (row, group) 1032 * sum of the even-k activations + 72 * sum of the odd-k
    // ones, read back from the fragment units (words x, z hold even k, words y, w odd k), fixed order
    for (uint32_t index = threadIdx.x; !single_row && index < p.x_rows * groups; index += kConsumerWarps * 32) {
      const uint32_t row = index / groups, g = index - row * groups;
      float even = 0.0f, odd = 0.0f;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const uint4 unit_words = x_fragments[((g * 2 + h) * p.x_rows + row) * 4 + cc];
          const float2 e0 = __half22float2(*reinterpret_cast<const __half2*>(&unit_words.x));
          const float2 o0 = __half22float2(*reinterpret_cast<const __half2*>(&unit_words.y));
          const float2 e1 = __half22float2(*reinterpret_cast<const __half2*>(&unit_words.z));
          const float2 o1 = __half22float2(*reinterpret_cast<const __half2*>(&unit_words.w));
          even += (e0.x + e0.y) + (e1.x + e1.y);
          odd += (o0.x + o0.y) + (o1.x + o1.y);
        }
      x_bias[index] = -(1032.0f * even + 72.0f * odd);
    }
    if (threadIdx.x == 0) {
      x_fragments[units] = make_uint4(0u, 0u, 0u, 0u);
      x_bias[p.x_rows * groups] = 0.0f;
    }
    consumer_barrier();
  }

  float acc[NMAT][NT][4];
#pragma unroll
  for (int a = 0; a < NMAT; ++a)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[a][t][j] = 0.0f;

  uint32_t stage_index = 0, parity = 0;
  bool aborted = false;
  // this lane's fragment words inside a stage: rows r and r+8, bytes [group*32 + c*8, +8) of
  // the warp's first group (group index in the stage = warp*GPW + j)
  const uint32_t word_offset = r * kRowBytes + warp * GPW * 32 + c * 8;
  const uint32_t scale_offset = kStageWeights + r * kScaleRow + warp * GPW * 2;
  // SMALLX addressing: fragment unit of (group g, half h, row r, c) is ((g*2 + h)*x_rows + r)*4 + c
  const uint32_t fragment_stride = 2 * p.x_rows * 4, fragment_lane = r * 4 + c;
  // lanes whose batch row does not exist read the zero unit / zero bias: base + g * stride
  // with stride 0 and the base pointing at the zero entry, so no select is needed per group
  const uint32_t zero_unit = groups * fragment_stride, zero_bias = p.x_rows * groups;
  const bool has_row = r < p.x_rows, has_bias0 = 2 * c < p.x_rows, has_bias1 = 2 * c + 1 < p.x_rows;
  const uint4* first_base = x_fragments + (has_row ? fragment_lane : zero_unit);
  const uint4* second_base = x_fragments + (has_row ? fragment_lane + p.x_rows * 4 : zero_unit);
  const uint32_t unit_stride = has_row ? fragment_stride : 0u;
  const float* bias_base0 = x_bias + (has_bias0 ? (2 * c) * groups : zero_bias);
  const float* bias_base1 = x_bias + (has_bias1 ? (2 * c + 1) * groups : zero_bias);
  const uint32_t bias_stride0 = has_bias0 ? 1u : 0u, bias_stride1 = has_bias1 ? 1u : 0u;

  for (uint32_t slot = 0; slot < my_tiles; ++slot) {
    for (uint32_t chunk = 0; chunk < chunks_per_tile; ++chunk) {
      if (!aborted) aborted = !mbarrier_wait(full_base + stage_index * 8u, parity, error_word);
      const unsigned char* stage = stages + stage_index * (NMAT * kStageBytes);
      float stage_scale_a[NMAT][GPW], stage_scale_b[NMAT][GPW];  // ONE: this warp's group scales, rows r and r + 8
      if (ONE) {
#pragma unroll
        for (int a = 0; a < NMAT; ++a) {
          load_scales<GPW>(stage + a * kStageBytes + scale_offset, stage_scale_a[a]);
          load_scales<GPW>(stage + a * kStageBytes + scale_offset + 8 * kScaleRow, stage_scale_b[a]);
        }
      }
#pragma unroll
      for (int jg = 0; jg < GPW; ++jg) {
        const uint32_t g = (chunk * 8 + warp) * GPW + jg;  // one of this warp's groups
        if (ONE) {
          const uint4 first = first_base[g * unit_stride];
          const uint4 second = second_base[g * unit_stride];
          const float bias0 = bias_base0[g * bias_stride0];
#pragma unroll
          for (int a = 0; a < NMAT; ++a) {
            const unsigned char* base = stage + a * kStageBytes;
            const uint2 word_a = *reinterpret_cast<const uint2*>(base + word_offset + jg * 32);
            const uint2 word_b = *reinterpret_cast<const uint2*>(base + word_offset + jg * 32 + 8 * kRowBytes);
            float sum[4];
            uint32_t a_even, a_odd, b_even, b_odd;
            nibbles_biased(word_a.x, a_even, a_odd);
            nibbles_biased(word_b.x, b_even, b_odd);
            mma_16816_from(sum, a_even, b_even, a_odd, b_odd, first.x, first.y, bias0, 0.0f, bias0, 0.0f);
            nibbles_biased(word_a.x >> 8, a_even, a_odd);
            nibbles_biased(word_b.x >> 8, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, first.z, first.w);
            nibbles_biased(word_a.y, a_even, a_odd);
            nibbles_biased(word_b.y, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, second.x, second.y);
            nibbles_biased(word_a.y >> 8, a_even, a_odd);
            nibbles_biased(word_b.y >> 8, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, second.z, second.w);
            acc[a][0][0] = fmaf(stage_scale_a[a][jg], sum[0], acc[a][0][0]);
            acc[a][0][2] = fmaf(stage_scale_b[a][jg], sum[2], acc[a][0][2]);
          }
        } else if (SMALLX) {
          const uint4 first = first_base[g * unit_stride];
          const uint4 second = second_base[g * unit_stride];
          const uint32_t frag[8] = {first.x, first.y, first.z, first.w, second.x, second.y, second.z, second.w};
          const float bias0 = bias_base0[g * bias_stride0];
          const float bias1 = bias_base1[g * bias_stride1];
#pragma unroll
          for (int a = 0; a < NMAT; ++a) {
            const unsigned char* base = stage + a * kStageBytes;
            const uint2 word_a = *reinterpret_cast<const uint2*>(base + word_offset + jg * 32);
            const uint2 word_b = *reinterpret_cast<const uint2*>(base + word_offset + jg * 32 + 8 * kRowBytes);
            const float scale_a = __half2float(*reinterpret_cast<const __half*>(base + scale_offset + jg * 2));
            const float scale_b =
                __half2float(*reinterpret_cast<const __half*>(base + scale_offset + jg * 2 + 8 * kScaleRow));
            // the group's bias term rides in as the accumulator's start value
            float sum[4] = {bias0, bias1, bias0, bias1};  // the table holds the negated term
            uint32_t a_even, a_odd, b_even, b_odd;
            nibbles_biased(word_a.x, a_even, a_odd);
            nibbles_biased(word_b.x, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, frag[0], frag[1]);
            nibbles_biased(word_a.x >> 8, a_even, a_odd);
            nibbles_biased(word_b.x >> 8, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, frag[2], frag[3]);
            nibbles_biased(word_a.y, a_even, a_odd);
            nibbles_biased(word_b.y, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, frag[4], frag[5]);
            nibbles_biased(word_a.y >> 8, a_even, a_odd);
            nibbles_biased(word_b.y >> 8, b_even, b_odd);
            mma_16816(sum, a_even, b_even, a_odd, b_odd, frag[6], frag[7]);
            acc[a][0][0] = fmaf(scale_a, sum[0], acc[a][0][0]);
            acc[a][0][1] = fmaf(scale_a, sum[1], acc[a][0][1]);
            acc[a][0][2] = fmaf(scale_b, sum[2], acc[a][0][2]);
            acc[a][0][3] = fmaf(scale_b, sum[3], acc[a][0][3]);
          }
        } else {
          uint32_t a_frag[NMAT][4][4];
          float scale_a[NMAT], scale_b[NMAT];
#pragma unroll
          for (int a = 0; a < NMAT; ++a) {
            const unsigned char* base = stage + a * kStageBytes;
            const uint2 word_a = *reinterpret_cast<const uint2*>(base + word_offset + jg * 32);
            const uint2 word_b = *reinterpret_cast<const uint2*>(base + word_offset + jg * 32 + 8 * kRowBytes);
            scale_a[a] = __half2float(*reinterpret_cast<const __half*>(base + scale_offset + jg * 2));
            scale_b[a] = __half2float(*reinterpret_cast<const __half*>(base + scale_offset + jg * 2 + 8 * kScaleRow));
#pragma unroll
            for (int w = 0; w < 2; ++w) {
              uint32_t bits_a = w == 0 ? word_a.x : word_a.y;
              uint32_t bits_b = w == 0 ? word_b.x : word_b.y;
#pragma unroll
              for (int step = 0; step < 2; ++step) {
                nibbles_to_half2<true>(bits_a, a_frag[a][w * 2 + step][0], a_frag[a][w * 2 + step][2]);
                nibbles_to_half2<true>(bits_b, a_frag[a][w * 2 + step][1], a_frag[a][w * 2 + step][3]);
                bits_a >>= 8;
                bits_b >>= 8;
              }
            }
          }
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint32_t batch_row = t * 8 + r;
            uint4 first = make_uint4(0u, 0u, 0u, 0u), second = first;
            if (batch_row < p.x_rows) {
              const uint4* source =
                  reinterpret_cast<const uint4*>(p.x + (size_t)batch_row * p.k + (g << 6) + (c << 4));
              first = __ldg(source);
              second = __ldg(source + 1);
            }
            uint32_t frag[8];
            frag[0] = prmt(first.x, first.z, 0x5410u);
            frag[1] = prmt(first.x, first.z, 0x7632u);
            frag[2] = prmt(first.y, first.w, 0x5410u);
            frag[3] = prmt(first.y, first.w, 0x7632u);
            frag[4] = prmt(second.x, second.z, 0x5410u);
            frag[5] = prmt(second.x, second.z, 0x7632u);
            frag[6] = prmt(second.y, second.w, 0x5410u);
            frag[7] = prmt(second.y, second.w, 0x7632u);
#pragma unroll
            for (int a = 0; a < NMAT; ++a) {
              float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
              for (int i = 0; i < 4; ++i)
                mma_16816(sum, a_frag[a][i][0], a_frag[a][i][1], a_frag[a][i][2], a_frag[a][i][3], frag[2 * i],
                          frag[2 * i + 1]);
              acc[a][t][0] = fmaf(scale_a[a], sum[0], acc[a][t][0]);
              acc[a][t][1] = fmaf(scale_a[a], sum[1], acc[a][t][1]);
              acc[a][t][2] = fmaf(scale_b[a], sum[2], acc[a][t][2]);
              acc[a][t][3] = fmaf(scale_b[a], sum[3], acc[a][t][3]);
            }
          }
        }
      }

      // the stage's words are in registers: hand it back to the producer
      __syncwarp();
      if (lane == 0) mbarrier_arrive(empty_base + stage_index * 8u);
      if (++stage_index == stage_count) {
        stage_index = 0;
        parity ^= 1u;
      }
    }

    // tile finished: fixed-order sum of the eight warps' partials, then the writeback
    uint32_t matrix, local_tile;
    locate(blockIdx.x + slot * gridDim.x, matrix, local_tile);
    const uint32_t n = p.mat[EPI == kEpiQkv ? matrix : 0].n;
    if (kLazyReduce<NT, EPI>) {
      // No CTA-wide barrier: every warp leaves its partials and goes on with the next tile; the
      // warp that arrives last adds them (warp order, so the sum does not depend on who that is)
      // and writes the tile.  The buffer is reused once the previous tile's reader has announced
      // that it is done, which the ring's depth all but guarantees; the check is a bounded spin.
      if (slot > 0 && !aborted) {
        uint32_t spin = 0;
        while (reduce_sync[1] < slot && ++spin < kSpinLimit) {
        }
        if (spin >= kSpinLimit) {
          atomicExch(error_word, 1u);
          aborted = true;
        }
      }
#pragma unroll
      for (int a = 0; a < NMAT; ++a)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (ONE && (j & 1)) continue;  // column 1 of the tile does not exist with one row
          reduce[(warp * kAcc + a * 4 + j) * 32 + lane] = acc[a][0][j];
          acc[a][0][j] = 0.0f;
        }
      __threadfence_block();
      __syncwarp();
      uint32_t arrived = 0;
      if (lane == 0) arrived = atomicAdd(const_cast<uint32_t*>(reduce_sync), 1u);
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived == kConsumerWarps - 1) {
        __threadfence_block();
#pragma unroll 1
        for (uint32_t j = 0; j < 4; ++j) {
          // positions whose batch row does not exist are not summed at all
          const bool wanted = EPI == kEpiSplitF32 ? c < 2u : 2u * c + (j & 1u) < p.m;
          if (!wanted) continue;
          float value[NMAT];
#pragma unroll
          for (int a = 0; a < NMAT; ++a) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) sum += reduce[(w * kAcc + a * 4 + j) * 32 + lane];
            value[a] = sum;
          }
          float partner = 0.0f;
          if (EPI == kEpiSplitF32) {
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) partner += reduce[(w * kAcc + j) * 32 + (lane ^ 2u)];
          }
          write_position<NT, NMAT, EPI>(p, value, partner, matrix, local_tile, n, 0u, j, lane);
        }
        __syncwarp();
        if (lane == 0) {
          reduce_sync[0] = 0u;
          __threadfence_block();
          reduce_sync[1] = slot + 1u;
        }
      }
    } else {
      consumer_barrier();  // the previous tile's reader is done with the buffer
#pragma unroll
      for (int a = 0; a < NMAT; ++a)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            reduce[(warp * kAcc + (a * NT + t) * 4 + j) * 32 + lane] = acc[a][t][j];
            acc[a][t][j] = 0.0f;
          }
      consumer_barrier();
      // every consumer thread finishes some accumulator positions: fixed-order sum over the
      // eight warps' partials, then the writeback of that position
      for (uint32_t position = threadIdx.x; position < NT * 4 * 32; position += kConsumerWarps * 32) {
        const uint32_t tj = position >> 5, position_lane = position & 31u;
        float value[NMAT];
#pragma unroll
        for (int a = 0; a < NMAT; ++a) {
          float sum = 0.0f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) sum += reduce[(w * kAcc + a * NT * 4 + tj) * 32 + position_lane];
          value[a] = sum;
        }
        float partner = 0.0f;
        if (EPI == kEpiSplitF32) {
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) partner += reduce[(w * kAcc + tj) * 32 + (position_lane ^ 2u)];
        }
        write_position<NT, NMAT, EPI>(p, value, partner, matrix, local_tile, n, tj >> 2, tj & 3u, position_lane);
      }
    }
  }
}

struct PipePlan {
  size_t shared_bytes;
  uint32_t ctas;
  uint32_t stages;
  uint32_t resident;  // CTAs per SM the plan was sized for
};

// Ring depth and grid: consumer warps are the scarce resource (the math is a chain of
// dependent instructions per group), bytes in flight the second: take the most
// resident CTAs per SM (up to 3; 4 for the LM-head form) whose ring still holds at least three
// stages (two at 4 CTAs), and one CTA per slot.
// CTAs per SM that this instantiation's registers allow (the wide-batch forms use up to 168 per thread).
template <int NT, int NMAT, int EPI, bool SMALLX, int GPW>
uint32_t register_resident_limit() {
  static const uint32_t limit = []() -> uint32_t {
    cudaFuncAttributes attributes;
    if (cudaFuncGetAttributes(&attributes, w4a16_gemv_pipe_kernel<NT, NMAT, EPI, SMALLX, GPW>) != cudaSuccess) {
      cudaGetLastError();
      return 3u;
    }
    const uint32_t per_cta = (uint32_t)((attributes.numRegs + 7) / 8 * 8) * kThreads;
    const uint32_t fit = 65536u / per_cta;
    return fit < 1u ? 1u : fit;
  }();
  return limit;
}

// Wide-batch forms (two and four batch tiles) compiled for two resident CTAs per SM (at most 112
// registers, a few spilled words in the dual form) instead of one CTA with all the registers it
// wants: LLMOPT_CUDA_GEMV_WIDE_RESIDENCY=2 selects it.
inline bool wide_forms_at_two_ctas() {
  static const bool two = []() {
    const char* text = getenv("LLMOPT_CUDA_GEMV_WIDE_RESIDENCY");
    return text != nullptr && text[0] == '2';
  }();
  return two;
}

template <int NT, int NMAT, int EPI, bool SMALLX, int GPW>
bool plan_pipe(const KernelArgs& args, const GemvProblem& p, PipePlan* plan) {
  uint32_t total_tiles = 0;
  const uint32_t matrices = EPI == kEpiQkv ? p.matrices : 1u;
  for (uint32_t i = 0; i < matrices; ++i) total_tiles += (p.mat[i].n + 15u) / 16u;
  const uint32_t groups = p.k / 64;
  size_t fixed_bytes = (size_t)kConsumerWarps * NMAT * NT * 4 * 32 * sizeof(float) + 64;
  if (SMALLX) fixed_bytes += (size_t)groups * 2 * p.x_rows * 4 * 16 + 16 + (size_t)(p.x_rows * groups + 4) * sizeof(float);
  const size_t stage_bytes = (size_t)NMAT * Stage<GPW>::kBytes + 16;
  const uint32_t sms = (uint32_t)context_sm_count(args.ctx);
  constexpr size_t kSharedPerSm = 220 * 1024;  // usable shared memory of one SM
  const uint32_t chunks_per_tile = p.k / Stage<GPW>::kChunkK;
  // a fourth resident CTA only where the kernel was compiled for it and every CTA still gets four tiles
  uint32_t most = kDenseResidency<NT, EPI> == 4 && total_tiles >= 16u * sms ? 4u : 3u;
  // Wide-batch forms on few, short tiles (QKV, o_proj): size grid and ring for the CTAs the registers really
  // let reside (batch 32: QKV 17.8 -> 14.6, o_proj 12.4 -> 10.9 us).  On many or long tiles the oversubscribed
  // grid measured faster (gate/up, down, LM head), so those keep it.
  if (NT > 1 && wide_forms_at_two_ctas())
    most = 2u;
  else if (NT > 1 && total_tiles <= 3u * sms && chunks_per_tile <= 4u &&
           register_resident_limit<NT, NMAT, EPI, SMALLX, GPW>() < most)
    most = register_resident_limit<NT, NMAT, EPI, SMALLX, GPW>();
  for (uint32_t resident = most; resident >= 1; --resident) {
    const size_t per_cta = kSharedPerSm / resident - 1024;
    if (per_cta <= fixed_bytes + 2 * stage_bytes) continue;
    uint32_t stages = (uint32_t)((per_cta - fixed_bytes) / stage_bytes);
    if (stages < (resident == 4 ? 2u : 3u) && resident > 1) continue;
    const uint32_t slots = sms * resident;
    const uint32_t ctas = total_tiles < slots ? total_tiles : slots;
    const uint32_t chunks = ((total_tiles + ctas - 1u) / ctas) * chunks_per_tile;
    if (stages > chunks) stages = chunks < 2 ? 2 : chunks;
    if (stages > 32) stages = 32;
    plan->shared_bytes = fixed_bytes + stages * stage_bytes;
    plan->ctas = ctas == 0 ? 1 : ctas;
    plan->stages = stages;
    plan->resident = resident;
    return true;
  }
  return false;
}

template <int NT, int NMAT, int EPI, bool SMALLX, int GPW>
int run_pipe(const KernelArgs& args, const GemvProblem& p, const PipePlan& plan) {
  constexpr int kDense = kDenseResidency<NT, EPI>;
  constexpr int kSparse = kDense == 3 ? 2 : kDense;  // the build for launches that fill at most two CTA slots per SM
  constexpr bool kOneRow = SMALLX && NT == 1;       // forms that have a single-row build
  const bool sparse = kDense == 3 && plan.ctas <= 2u * (uint32_t)context_sm_count(args.ctx);
  // LLMOPT_CUDA_GEMV_ONE_ROW=0 runs single-row launches on the general build (for comparison)
  static const bool one_row_allowed = getenv("LLMOPT_CUDA_GEMV_ONE_ROW") == nullptr || getenv("LLMOPT_CUDA_GEMV_ONE_ROW")[0] != '0';
  const bool one_row = kOneRow && p.x_rows == 1u && one_row_allowed;
  auto kernel = w4a16_gemv_pipe_kernel<NT, NMAT, EPI, SMALLX, GPW>;
  if (one_row)
    kernel = sparse ? w4a16_gemv_pipe_kernel<NT, NMAT, EPI, SMALLX, GPW, kSparse, kOneRow>
                    : w4a16_gemv_pipe_kernel<NT, NMAT, EPI, SMALLX, GPW, kDense, kOneRow>;
  else if (sparse)
    kernel = w4a16_gemv_pipe_kernel<NT, NMAT, EPI, SMALLX, GPW, kSparse>;
  else if (NT > 1 && wide_forms_at_two_ctas())
    kernel = w4a16_gemv_pipe_kernel<NT, NMAT, EPI, SMALLX, GPW, (NT > 1 ? 2 : kDense)>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.shared_bytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  launch_kernel(args, kernel, dim3(plan.ctas), dim3(kThreads), plan.shared_bytes, p, plan.stages, context_device_error(args.ctx));
  return check_launch(args);
}

// Groups per warp and stage: the most (4, 2, 1) that K allows and that still leaves at
// least two CTAs (18 warps) resident per SM; a fat stage that forces one CTA per SM
// loses more to idle issue slots than it gains from amortised waits.  Four groups only for
// one matrix and one or four batch tiles (measured at the Llama-8B shapes: with two batch
// tiles four groups lose to two; with four tiles they win: batch-32 step 9.22 -> 8.13 ms
// together with two groups for the dual form).
template <int NT, int NMAT, int EPI, bool SMALLX>
int launch_pipe(const KernelArgs& args, const GemvProblem& p) {
  PipePlan plan4 = {}, plan2 = {}, plan1 = {};
  const bool ok4 = (NT == 1 || NT == 4) && NMAT == 1 && p.k % 2048 == 0 && plan_pipe<NT, NMAT, EPI, SMALLX, 4>(args, p, &plan4);
  // (four batch tiles: the fat forms win even at one CTA per SM, which is all their registers allow)
  if (ok4 && (plan4.resident >= 2 || NT == 4)) return run_pipe<NT, NMAT, EPI, SMALLX, 4>(args, p, plan4);
  const bool ok2 = p.k % 1024 == 0 && plan_pipe<NT, NMAT, EPI, SMALLX, 2>(args, p, &plan2);
  if (ok2 && (plan2.resident >= 2 || NT == 4)) return run_pipe<NT, NMAT, EPI, SMALLX, 2>(args, p, plan2);
  const bool ok1 = plan_pipe<NT, NMAT, EPI, SMALLX, 1>(args, p, &plan1);
  if (ok1 && plan1.resident >= 2) return run_pipe<NT, NMAT, EPI, SMALLX, 1>(args, p, plan1);
  if (ok2) return run_pipe<NT, NMAT, EPI, SMALLX, 2>(args, p, plan2);
  if (ok1) return run_pipe<NT, NMAT, EPI, SMALLX, 1>(args, p, plan1);
  if (ok4) return run_pipe<NT, NMAT, EPI, SMALLX, 4>(args, p, plan4);
  return -1;
}

template <int EPI, int NMAT>
int launch_pipe_by_rows(const KernelArgs& args, const GemvProblem& p) {
  const uint32_t rows = p.x_rows;
  const bool small = (size_t)rows * p.k <= 16384 && rows <= 8 && EPI != kEpiSplitF32;
  if (p.norm_weight != nullptr && !small) return -1;  // only the staged-activation form absorbs a norm
  if (rows <= 8) {
    if (small) return launch_pipe<1, NMAT, EPI, true>(args, p);
    return launch_pipe<1, NMAT, EPI, false>(args, p);
  }
  if (rows <= 16) return launch_pipe<2, NMAT, EPI, false>(args, p);
  if (rows <= 32) return launch_pipe<4, NMAT, EPI, false>(args, p);
  return -1;  // 33..64 rows stay on the direct-load kernel
}

}  // namespace

// Returns -1 when the shape is outside this kernel's domain (the caller then
// uses the direct-load kernel), 0 on success, 1 on a launch failure.
int launch_w4a16_gemv_pipe(const KernelArgs& args, const GemvProblem& problem, int epilogue) {
  if (args.ctx == nullptr || problem.k % 512 != 0) return -1;
  const uint32_t matrices = epilogue == kEpiQkv ? problem.matrices : (epilogue == kEpiDualSwiglu ? 2u : 1u);
  for (uint32_t i = 0; i < matrices; ++i) {
    if (((uintptr_t)problem.mat[i].packed & 15u) != 0 || ((uintptr_t)problem.mat[i].scale & 15u) != 0) return -1;
    if (problem.mat[i].n == 0) return -1;
  }
  if (((uintptr_t)problem.x & 15u) != 0) return -1;
  if (problem.norm_weight != nullptr &&
      ((((uintptr_t)problem.norm_weight | (uintptr_t)problem.norm_out) & 15u) != 0 || problem.x_rows > 8))
    return -1;
  switch (epilogue) {
    case kEpiLinear: return launch_pipe_by_rows<kEpiLinear, 1>(args, problem);
    case kEpiQkv: return launch_pipe_by_rows<kEpiQkv, 1>(args, problem);
    case kEpiDualSwiglu: return launch_pipe_by_rows<kEpiDualSwiglu, 2>(args, problem);
    case kEpiTagged: return launch_pipe_by_rows<kEpiTagged, 1>(args, problem);
    case kEpiSplitF32: return launch_pipe_by_rows<kEpiSplitF32, 1>(args, problem);
    default: return -1;
  }
}

}  // namespace llmopt
