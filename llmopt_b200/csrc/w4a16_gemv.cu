// Decode-side W4A16 group-64 products (M <= 64 rows per pass) for sm_100a.
//
// Replaces the reference's SIMD-group GEMV kernels
//   llmopt_w4a16_linear_f16_g64{,_m4,_m8}          lib/metal_w4a16_source.ml:8-194
//   llmopt_w4a16_qkv_linear_f16_g64{,_m4,_m8}      lib/metal_w4a16_source.ml:218-480
//   llmopt_w4a16_dual_swiglu / down_add            lib/metal_w4a16_source.ml:533-966
//   parametric epilogue forms                      lib/metal_parametric_codegen.ml:4-39
// The storage contract is untouched: packed u8 [N, K/2] (low nibble = even k,
// two's complement), fp16 scale [N, K/64].
//
// Shape of the kernel.  HBM traffic is the bound, so the kernel is organised
// around keeping many 8-byte weight loads in flight while spending as few
// issue slots per weight as possible:
//   * a 16-column tile of W is owned by k_warps warps that split K into
//     contiguous runs of groups; lane (r = lane/4, c = lane%4) streams columns
//     r and r+8, 8 bytes (16 nibbles) per group, so a quad covers one whole
//     group of 64 (32 contiguous bytes) and a warp reads 16 rows x 32 B;
//   * nibbles become exact fp16 integers in registers with one LOP3 and one
//     half2 add/fma per pair (no shifts for the low/high nibble of a byte);
//   * the 64-long dot products of one group are done by four
//     mma.sync.m16n8k16 (fp16 x fp16 -> fp32, exact products), with the batch
//     rows in the n dimension, so 1..8 rows cost the same issue slots;
//   * the group's fp32 sum is scaled by the fp32 value of the fp16 scale and
//     added to the running accumulator — the weight is never rounded to half
//     after scaling, as in the reference kernels (lib/metal_w4a16_source.ml:34);
//   * partial sums of the k_warps warps are added in a fixed order in shared
//     memory (deterministic), then the epilogue writes half once.
// The k index inside an MMA is a fixed permutation of the real k (pairs
// (i, i+4) of a byte quad); activations are permuted to match with PRMT.
#include "rms_norm.cuh"
#include "w4a16_gemv_device.cuh"

namespace llmopt {
using namespace gemv;
namespace {

template <int NT, int NMAT, int EPI, bool AFFINE>
__global__ void __launch_bounds__(256, (NT * NMAT >= 8) ? 1 : 2) w4a16_gemv_kernel(const GemvProblem p) {
  grid_chain_prologue();
  // groups whose weight loads are issued together
  constexpr int kUnroll = (NT * NMAT >= 8) ? 2 : 4;
  extern __shared__ float shared[];
  constexpr int kAcc = NMAT * NT * 4;
  float* reduce = shared;                     // [8][kAcc][32]
  float* x_sums = shared + 8 * kAcc * 32;     // AFFINE: [x_rows][groups]

  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t r = lane >> 2, c = lane & 3u;
  const uint32_t k_warps = p.k_warps, slots = 8u / k_warps;
  const uint32_t k_slice = warp % k_warps, slot = warp / k_warps;
  const uint32_t groups = p.k >> 6;
  const uint32_t per_warp = (groups + k_warps - 1u) / k_warps;
  const uint32_t g_begin = min(k_slice * per_warp, groups);
  const uint32_t g_end = min(g_begin + per_warp, groups);
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

  if (AFFINE) {
    // Per (row, group) sums of the activations: the zero point enters as
    // -s (z - 8) sum_k x[k] for each group.
    for (uint32_t index = threadIdx.x; index < p.x_rows * groups; index += 256u) {
      const uint32_t row = index / groups, g = index - row * groups;
      const __half2* source = reinterpret_cast<const __half2*>(p.x + (size_t)row * p.k + (g << 6));
      float sum = 0.0f;
      for (int i = 0; i < 32; ++i) {
        const float2 pair = __half22float2(source[i]);
        sum += pair.x + pair.y;
      }
      x_sums[index] = sum;
    }
    __syncthreads();
  }

  for (uint32_t base = blockIdx.x * slots; base < total_tiles; base += gridDim.x * slots) {
    const uint32_t tile = base + slot;
    const bool active = tile < total_tiles;
    uint32_t matrix = 0, local_tile = tile;
    if (EPI == kEpiQkv) {
      if (local_tile >= tiles[0]) { local_tile -= tiles[0]; matrix = 1; }
      if (matrix == 1 && local_tile >= tiles[1]) { local_tile -= tiles[1]; matrix = 2; }
    }
    float acc[NMAT][NT][4];
#pragma unroll
    for (int a = 0; a < NMAT; ++a)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[a][t][j] = 0.0f;

    const uint32_t n = p.mat[EPI == kEpiQkv ? matrix : 0].n;
    const uint32_t row_a = min(local_tile * 16u + r, n - 1u);
    const uint32_t row_b = min(local_tile * 16u + r + 8u, n - 1u);

    if (active) {
      const uint8_t* weights[NMAT];
      const __half* scales[NMAT];
      const __half* zeros[NMAT];
#pragma unroll
      for (int a = 0; a < NMAT; ++a) {
        const GemvMatrix& mat = p.mat[EPI == kEpiQkv ? matrix : a];
        weights[a] = mat.packed;
        scales[a] = mat.scale;
        zeros[a] = mat.zero;
      }
      for (uint32_t g0 = g_begin; g0 < g_end; g0 += kUnroll) {
        uint2 word_a[NMAT][kUnroll], word_b[NMAT][kUnroll];
        float scale_a[NMAT][kUnroll], scale_b[NMAT][kUnroll];
        float zero_a[NMAT][kUnroll], zero_b[NMAT][kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint32_t g = g0 + u;
          const bool live = g < g_end;
#pragma unroll
          for (int a = 0; a < NMAT; ++a) {
            word_a[a][u] = make_uint2(0u, 0u);
            word_b[a][u] = make_uint2(0u, 0u);
            scale_a[a][u] = 0.0f;
            scale_b[a][u] = 0.0f;
            zero_a[a][u] = 0.0f;
            zero_b[a][u] = 0.0f;
            if (live) {
              word_a[a][u] = __ldg(reinterpret_cast<const uint2*>(
                  weights[a] + (size_t)row_a * half_k + (g << 5) + (c << 3)));
              word_b[a][u] = __ldg(reinterpret_cast<const uint2*>(
                  weights[a] + (size_t)row_b * half_k + (g << 5) + (c << 3)));
              scale_a[a][u] = __half2float(__ldg(scales[a] + (size_t)row_a * groups + g));
              scale_b[a][u] = __half2float(__ldg(scales[a] + (size_t)row_b * groups + g));
              if (AFFINE) {
                zero_a[a][u] = __half2float(__ldg(zeros[a] + (size_t)row_a * groups + g));
                zero_b[a][u] = __half2float(__ldg(zeros[a] + (size_t)row_b * groups + g));
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint32_t g = g0 + u;
          if (g >= g_end) break;
          // Exact fp16 integer fragments of the two weight rows for this group.
          uint32_t a_frag[NMAT][4][4];
#pragma unroll
          for (int a = 0; a < NMAT; ++a)
#pragma unroll
            for (int w = 0; w < 2; ++w) {
              uint32_t bits_a = w == 0 ? word_a[a][u].x : word_a[a][u].y;
              uint32_t bits_b = w == 0 ? word_b[a][u].x : word_b[a][u].y;
#pragma unroll
              for (int step = 0; step < 2; ++step) {
                uint32_t a_low, a_high, b_low, b_high;
                nibbles_to_half2<!AFFINE>(bits_a, a_low, a_high);
                nibbles_to_half2<!AFFINE>(bits_b, b_low, b_high);
                a_frag[a][w * 2 + step][0] = a_low;
                a_frag[a][w * 2 + step][1] = b_low;
                a_frag[a][w * 2 + step][2] = a_high;
                a_frag[a][w * 2 + step][3] = b_high;
                bits_a >>= 8;
                bits_b >>= 8;
              }
            }
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            // Activation fragment: lane (r, c) supplies batch row t*8 + r,
            // k = 64 g + 16 c + [0, 16), paired (i, i+4) like the nibbles.
            const uint32_t batch_row = t * 8 + r;
            uint4 first = make_uint4(0u, 0u, 0u, 0u), second = first;
            if (batch_row < p.x_rows) {
              const uint4* source = reinterpret_cast<const uint4*>(
                  p.x + (size_t)batch_row * p.k + (g << 6) + (c << 4));
              first = __ldg(source);
              second = __ldg(source + 1);
            }
            uint32_t frag[8];
            frag[0] = prmt(first.x, first.z, 0x5410u);    // k0, k4
            frag[1] = prmt(first.x, first.z, 0x7632u);    // k1, k5
            frag[2] = prmt(first.y, first.w, 0x5410u);    // k2, k6
            frag[3] = prmt(first.y, first.w, 0x7632u);    // k3, k7
            frag[4] = prmt(second.x, second.z, 0x5410u);  // k8, k12
            frag[5] = prmt(second.x, second.z, 0x7632u);
            frag[6] = prmt(second.y, second.w, 0x5410u);
            frag[7] = prmt(second.y, second.w, 0x7632u);
#pragma unroll
            for (int a = 0; a < NMAT; ++a) {
              float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
              for (int i = 0; i < 4; ++i)
                mma_16816(sum, a_frag[a][i][0], a_frag[a][i][1], a_frag[a][i][2], a_frag[a][i][3],
                          frag[2 * i], frag[2 * i + 1]);
              acc[a][t][0] = fmaf(scale_a[a][u], sum[0], acc[a][t][0]);
              acc[a][t][1] = fmaf(scale_a[a][u], sum[1], acc[a][t][1]);
              acc[a][t][2] = fmaf(scale_b[a][u], sum[2], acc[a][t][2]);
              acc[a][t][3] = fmaf(scale_b[a][u], sum[3], acc[a][t][3]);
              if (AFFINE) {
                const uint32_t column = t * 8 + 2 * c;
                const float sum0 = column < p.x_rows ? x_sums[column * groups + g] : 0.0f;
                const float sum1 = column + 1 < p.x_rows ? x_sums[(column + 1) * groups + g] : 0.0f;
                const float shift_a = scale_a[a][u] * (zero_a[a][u] - 8.0f);
                const float shift_b = scale_b[a][u] * (zero_b[a][u] - 8.0f);
                acc[a][t][0] = fmaf(-shift_a, sum0, acc[a][t][0]);
                acc[a][t][1] = fmaf(-shift_a, sum1, acc[a][t][1]);
                acc[a][t][2] = fmaf(-shift_b, sum0, acc[a][t][2]);
                acc[a][t][3] = fmaf(-shift_b, sum1, acc[a][t][3]);
              }
            }
          }
        }
      }
    }

    if (k_warps > 1) {
      if (k_slice != 0) {
#pragma unroll
        for (int a = 0; a < NMAT; ++a)
#pragma unroll
          for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reduce[(warp * kAcc + (a * NT + t) * 4 + j) * 32 + lane] = acc[a][t][j];
      }
      __syncthreads();
      if (k_slice == 0) {
        for (uint32_t other = 1; other < k_warps; ++other)
#pragma unroll
          for (int a = 0; a < NMAT; ++a)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                acc[a][t][j] += reduce[((warp + other) * kAcc + (a * NT + t) * 4 + j) * 32 + lane];
      }
    }

    if (active && k_slice == 0) write_tile<NT, NMAT, EPI>(p, acc, matrix, local_tile, n, lane);
    if (k_warps > 1) __syncthreads();
  }
}

template <int NT, int NMAT, int EPI, bool AFFINE>
int launch_one(const KernelArgs& args, const GemvProblem& p) {
  uint32_t total_tiles = 0;
  const uint32_t matrices = EPI == kEpiQkv ? p.matrices : 1u;
  for (uint32_t i = 0; i < matrices; ++i) total_tiles += (p.mat[i].n + 15u) / 16u;
  const uint32_t slots = 8u / p.k_warps;
  const uint32_t wanted = (total_tiles + slots - 1u) / slots;
  size_t shared_bytes = (size_t)8 * NMAT * NT * 4 * 32 * sizeof(float);
  if (AFFINE) shared_bytes += (size_t)p.x_rows * (p.k / 64) * sizeof(float);
  auto kernel = w4a16_gemv_kernel<NT, NMAT, EPI, AFFINE>;
  if (shared_bytes > 48 * 1024) {
    if (shared_bytes > 200 * 1024) return fail(args, "shape needs more shared memory than one CTA has");
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared_bytes);
  }
  const uint32_t resident = (uint32_t)context_sm_count(args.ctx) * 3u;
  const uint32_t ctas = wanted < resident ? wanted : resident;
  launch_kernel(args, kernel, dim3(ctas == 0 ? 1 : ctas), dim3(256), shared_bytes, p);
  return check_launch(args);
}

template <int EPI, int NMAT, bool AFFINE>
int launch_by_rows(const KernelArgs& args, const GemvProblem& p) {
  const uint32_t rows = p.x_rows;
  if (rows <= 8) return launch_one<1, NMAT, EPI, AFFINE>(args, p);
  if (rows <= 16) return launch_one<2, NMAT, EPI, AFFINE>(args, p);
  if (rows <= 32) return launch_one<4, NMAT, EPI, AFFINE>(args, p);
  return launch_one<8, NMAT, EPI, AFFINE>(args, p);
}

uint32_t pick_k_warps(uint32_t k) {
  const uint32_t groups = k / 64;
  if (groups >= 32) return 8;
  if (groups >= 16) return 4;
  if (groups >= 8) return 2;
  return 1;
}

}  // namespace

int launch_w4a16_gemv(const KernelArgs& args, GemvProblem problem, int epilogue, bool affine) {
  LLMOPT_REQUIRE(problem.k > 0 && problem.k % 64 == 0, "K must be a positive multiple of 64");
  LLMOPT_REQUIRE(problem.m > 0, "M must be positive");
  LLMOPT_REQUIRE(((uintptr_t)problem.x & 15u) == 0, "activation buffer must be 16-byte aligned");
  const uint32_t matrices = epilogue == kEpiQkv ? problem.matrices : (epilogue == kEpiDualSwiglu ? 2u : 1u);
  for (uint32_t i = 0; i < matrices; ++i) {
    LLMOPT_REQUIRE(problem.mat[i].n > 0, "N must be positive");
    LLMOPT_REQUIRE(((uintptr_t)problem.mat[i].packed & 7u) == 0, "packed weight must be 8-byte aligned");
  }
  if (problem.k_warps == 0) problem.k_warps = pick_k_warps(problem.k);

  // A norm folded into this product: only the pipelined small-batch kernel stages activations in a
  // form that can absorb it; otherwise run the norm as its own kernel first.
  if (problem.norm_weight != nullptr) {
    const bool absorbs = !affine && problem.x_rows <= 8 && (size_t)problem.x_rows * problem.k <= 16384 &&
                         epilogue != kEpiSplitF32 && problem.k % 512 == 0;
    if (absorbs) {
      const int status = launch_w4a16_gemv_pipe(args, problem, epilogue);
      if (status >= 0) return status;
    }
    if (problem.norm_weight_first)
      launch_rms_norm_rows<__half, true>(args, problem.x, problem.norm_weight, problem.norm_out, problem.x_rows,
                                         problem.k, problem.norm_epsilon);
    else
      launch_rms_norm_rows<__half, false>(args, problem.x, problem.norm_weight, problem.norm_out, problem.x_rows,
                                          problem.k, problem.norm_epsilon);
    if (int status = check_launch(args)) return status;
    problem.x = problem.norm_out;
    problem.norm_weight = nullptr;
    problem.norm_out = nullptr;
  }

  // decode batches from 17 rows and prompts: weights as the M side of the tensor-core product, converted into tensor memory
  {
    const int status = launch_w4a16_gemm_tc_batch(args, problem, epilogue, affine);
    if (status >= 0) return status;
  }

  // 64 rows and more that the kernel above does not cover (tagged epilogues): the GEMM with the converted
  // weights as the shared-memory B operand
  if (problem.m >= tensor_core_min_rows() && problem.x_rows == problem.m) {
    const int status = launch_w4a16_gemm_tc(args, problem, epilogue, affine);
    if (status >= 0) return status;
  }

  // K a multiple of 512 and at most 32 rows: the shared-memory pipelined kernel
  if (!affine && problem.x_rows <= 32) {
    const int status = launch_w4a16_gemv_pipe(args, problem, epilogue);
    if (status >= 0) return status;
  }

  if (epilogue == kEpiSplitF32) {
    LLMOPT_REQUIRE(problem.x_rows <= 64 && problem.x_rows % 8 == 0 && problem.m * 2 <= problem.x_rows,
                   "split activations need 8-row slot tiles and at most 32 rows");
    return launch_by_rows<kEpiSplitF32, 1, false>(args, problem);
  }
  // More than 64 rows: passes of 64 rows over the same weights.
  const uint32_t total_rows = problem.m;
  for (uint32_t row0 = 0; row0 < total_rows; row0 += 64) {
    GemvProblem pass = problem;
    const uint32_t rows = total_rows - row0 < 64 ? total_rows - row0 : 64;
    pass.m = rows;
    pass.x_rows = rows;
    pass.x = problem.x + (size_t)row0 * problem.k;
    for (int i = 0; i < 3; ++i)
      if (problem.out[i]) pass.out[i] = problem.out[i] + (size_t)row0 * problem.mat[epilogue == kEpiQkv ? i : 0].n;
    if (epilogue == kEpiLinear && problem.has_aux)
      pass.aux0 = problem.aux0 + (size_t)row0 * problem.aux_row_stride;
    int status = 0;
    switch (epilogue) {
      case kEpiLinear:
        status = affine ? launch_by_rows<kEpiLinear, 1, true>(args, pass)
                        : launch_by_rows<kEpiLinear, 1, false>(args, pass);
        break;
      case kEpiQkv: status = launch_by_rows<kEpiQkv, 1, false>(args, pass); break;
      case kEpiDualSwiglu: status = launch_by_rows<kEpiDualSwiglu, 2, false>(args, pass); break;
      case kEpiTagged: status = launch_by_rows<kEpiTagged, 1, false>(args, pass); break;
      default: return fail(args, "unknown epilogue");
    }
    if (status != 0) return status;
  }
  return 0;
}

}  // namespace llmopt
