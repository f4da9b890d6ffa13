// Small-M (decode) W4A16 group-64 product: shared problem description.
#pragma once
#include "common.cuh"

namespace llmopt {

// Writeback forms. The arithmetic of each follows the reference:
//  kEpiLinear     half(acc [+ bias[row*stride + col]])   lib/metal_w4a16_source.ml:36-39
//  kEpiQkv        half(acc) into one of three outputs    lib/metal_w4a16_source.ml:262-279
//  kEpiDualSwiglu half(silu(gate) * up)                  lib/metal_w4a16_source.ml:571-575
//  kEpiTagged     lib/epilogue.ml:148-174 (operands indexed by column)
//  kEpiSplitF32   fp32 accumulator out, activations given as hi/lo half pairs
enum GemvEpilogue { kEpiLinear = 0, kEpiQkv = 1, kEpiDualSwiglu = 2, kEpiTagged = 3, kEpiSplitF32 = 4 };

struct GemvMatrix {
  const uint8_t* packed;  // [n, k/2], low nibble = even k
  const __half* scale;    // [n, k/64]
  const __half* zero;     // [n, k/64] or null (affine mode only)
  uint32_t n;
};

struct GemvProblem {
  const __half* x;  // [x_rows, k] row-major
  uint32_t x_rows;  // rows present in x (m, or the hi/lo slot count for kEpiSplitF32)
  uint32_t m;       // logical output rows
  uint32_t k;
  GemvMatrix mat[3];
  uint32_t matrices;  // kEpiQkv: 3 independent; kEpiDualSwiglu: 2 sharing n; else 1
  __half* out[3];
  float* out_f32;
  const __half* aux0;  // bias / residual / up / first epilogue operand
  const __half* aux1;  // second epilogue operand
  uint32_t aux_row_stride;
  uint32_t has_aux;
  uint32_t tag;        // kEpiTagged: lib/epilogue.ml variant index (0..9)
  uint32_t k_warps;    // warps that split K for one 16-column tile (1,2,4,8)
  // Folded RMS norm: x holds the RAW rows; the kernel normalises them with norm_weight while it
  // stages the activations and writes the normalised rows to norm_out (null: no folded norm).
  const __half* norm_weight;
  __half* norm_out;
  float norm_epsilon;
  uint32_t norm_weight_first;
};

// Host entry: validates alignment, picks the tile shape and launches on `stream`.
// Rows beyond 64 are processed in passes of 64.
int launch_w4a16_gemv(const KernelArgs& args, GemvProblem problem, int epilogue, bool affine);

// Tensor-core GEMM for M >= 64 (tcgen05 / tensor memory); returns -1 outside its domain.
int launch_w4a16_gemm_tc(const KernelArgs& args, const GemvProblem& problem, int epilogue, bool affine);
uint32_t tensor_core_min_rows();

// Tensor-core kernel with the converted weights in tensor memory (weights on the M side, rows on the N side):
// decode batches from 17 rows and prompts; returns -1 outside its domain.
int launch_w4a16_gemm_tc_batch(const KernelArgs& args, const GemvProblem& problem, int epilogue, bool affine);

// Pipelined fast path (K % 512 == 0, <= 32 rows); returns -1 if the shape is outside its domain.
int launch_w4a16_gemv_pipe(const KernelArgs& args, const GemvProblem& problem, int epilogue);

}  // namespace llmopt
