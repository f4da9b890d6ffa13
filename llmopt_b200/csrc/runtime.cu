// Runtime behind the C ABI of include/llmopt_cuda.h: contexts, buffers, the
// kernel registry, deferred batches, CUDA-graph "prebaked" plans and the ring
// worker.  It plays the part of native/ocaml_metal_stubs.m in the reference:
// same primitives, same ownership and error rules, CUDA streams and graphs in
// place of Metal command buffers.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/llmopt_cuda.h"
#include "common.cuh"
#include "q8_codec.cuh"

namespace llmopt {

// ---- launchers defined in the kernel translation units --------------------------
int launch_w4a16_linear(const KernelArgs&);
int launch_w4a16_linear_affine(const KernelArgs&);
int launch_w4a16_qkv_linear(const KernelArgs&);
int launch_w4a16_swiglu_rms_f16(const KernelArgs&);
int launch_w4a16_swiglu_rms_f32(const KernelArgs&);
int launch_w4a16_dual_swiglu(const KernelArgs&);
int launch_w4a16_down_add(const KernelArgs&);
template <int TAG> int launch_w4a16_linear_tagged(const KernelArgs&);
template <bool F32, bool EXTRA> int launch_w4a16_lm_head_argmax(const KernelArgs&);
template <bool F32, bool EXTRA> int launch_w4a16_lm_head_stage1(const KernelArgs&);
int launch_w4a16_lm_head_reduce(const KernelArgs&);
int launch_w4a16_linear_partial_f32(const KernelArgs&);
int launch_tp_exchange_sum(const KernelArgs&);
int launch_tp_exchange_argmax(const KernelArgs&);
int launch_tp_exchange_sum_norm(const KernelArgs&);
int launch_tp_exchange_reduce_rows(const KernelArgs&);
int launch_tp_exchange_gather_rows(const KernelArgs&);
int launch_attention_dense(const KernelArgs&);
int launch_q4_0_linear(const KernelArgs&);
int launch_q4_0_gated_linear(const KernelArgs&);
int launch_tile32_affine4_linear(const KernelArgs&);
int launch_cache_pack_tile32_affine8_fwht(const KernelArgs&);
int launch_cache_unpack_tile32_affine8_fwht(const KernelArgs&);
int launch_cache_pack_tile32_affine4_fwht(const KernelArgs&);
int launch_cache_unpack_tile32_affine4_fwht(const KernelArgs&);
int launch_tile32_affine8_linear(const KernelArgs&);
int launch_q4_0_qkv_linear(const KernelArgs&);
int launch_q4_0_dequant(const KernelArgs&);
int launch_cache_pack_attention_q8(const KernelArgs&);
int launch_cache_pack_attention_q8_pair(const KernelArgs&);
int launch_cache_unpack_attention_q8(const KernelArgs&);
int launch_cache_pack_checkpoint_q8(const KernelArgs&);
int launch_cache_unpack_checkpoint_q8(const KernelArgs&);
int launch_attention_q8_paged(const KernelArgs&);
template <bool WEIGHT_F32> int launch_short_conv(const KernelArgs&);
template <bool WEIGHT_F32> int launch_short_conv_silu_tm(const KernelArgs&);
int launch_short_conv_step(const KernelArgs&);
int launch_short_conv_prefill(const KernelArgs&);
template <bool INPUT_F32> int launch_rms_norm(const KernelArgs&);
int launch_rotary_qk(const KernelArgs&);
int launch_rotary_pack_fused(const KernelArgs& rotary, const KernelArgs& pack);
bool paged_attention_takes_rotary_pack(const KernelArgs& attention, const RotaryPackFusion& fusion);
int launch_embedding_f16(const KernelArgs&);
int launch_chain_token_id(const KernelArgs&);
int launch_chain_token_ids(const KernelArgs&);
void launch_argmax_f16(const __half* values, uint32_t count, int* result, cudaStream_t stream);
struct NamedLauncher {
  const char* name;
  Launcher launcher;
};
const NamedLauncher* norm_family_launchers(size_t* count);
struct ExprProgram {
  uint8_t code[192];
  uint32_t length;
  uint32_t operands;
};
const char* validate_expr_program(const uint8_t* code, size_t length, int operand_count);
int launch_w4a16_linear_expr(const KernelArgs&);
int launch_q4_0_linear_expr(const KernelArgs&);
int launch_gated_delta_f32(const KernelArgs&);
int launch_gated_delta_tm_f16(const KernelArgs&);
int launch_triangular_recurrence(const KernelArgs&);

// ---- objects -----------------------------------------------------------------------

struct Context {
  std::atomic<int> references{1};
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  std::string name;
  // scratch blocks are only ever added; captured graphs keep pointing at old ones
  std::vector<void*> scratch_blocks;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  void* split = nullptr;  // K-split scratch of the tensor-core GEMM: [arrival counters | fp32 partials]
  size_t split_bytes = 0;
  size_t split_counter_bytes = 0;  // leading bytes that must read zero between launches
  void* flush_buffer = nullptr;  // L2 flush target for timing
  size_t flush_bytes = 0;
  int* argmax_result = nullptr;  // device int
  // Pinned, device-visible word: kernels whose bounded waits ran out set it; the host
  // reads it after every stream wait.
  uint32_t* device_error = nullptr;
  // Launches may overlap the tail of their predecessor (programmatic dependent launch).
  bool overlap = true;
  // Expression epilogues registered by digest name (llmopt_cuda_register_expr_epilogue).
  std::map<std::string, ExprProgram> expr_programs;
};

struct Allocation {
  std::atomic<int> references{1};
  Context* context = nullptr;
  void* base = nullptr;
  size_t length = 0;
  bool imported = false;  // a peer process's allocation opened through CUDA IPC
};

}  // namespace llmopt

using namespace llmopt;

struct llmopt_cuda_context : Context {};
struct llmopt_cuda_buffer {
  std::atomic<int> references{1};
  Allocation* allocation = nullptr;
  size_t offset = 0;
  size_t length = 0;
  uint8_t* pointer() const { return (uint8_t*)allocation->base + offset; }
};
struct llmopt_cuda_library {
  std::atomic<int> references{1};
  Context* context = nullptr;
  std::map<std::string, Launcher> launchers;
  std::vector<std::string> names;
};

namespace llmopt {

thread_local std::string g_last_error;

static int set_error(int code, const std::string& message) {
  g_last_error = message;
  return code;
}
static int cuda_failure(const char* what, cudaError_t status) {
  return set_error(LLMOPT_CUDA_FAILURE, std::string(what) + ": " + cudaGetErrorString(status));
}
#define CUDA_TRY(expr, what)                                   \
  do {                                                         \
    cudaError_t status__ = (expr);                             \
    if (status__ != cudaSuccess) return cuda_failure(what, status__); \
  } while (0)

static void retain(Context* context) { context->references.fetch_add(1); }
static void release(Context* context) {
  if (context->references.fetch_sub(1) != 1) return;
  cudaSetDevice(context->device);
  if (context->stream) cudaStreamSynchronize(context->stream);
  for (void* block : context->scratch_blocks) cudaFree(block);
  if (context->flush_buffer) cudaFree(context->flush_buffer);
  if (context->argmax_result) cudaFree(context->argmax_result);
  if (context->device_error) cudaFreeHost(context->device_error);
  if (context->stream) cudaStreamDestroy(context->stream);
  delete static_cast<llmopt_cuda_context*>(context);
}
static void release(Allocation* allocation) {
  if (allocation->references.fetch_sub(1) != 1) return;
  cudaSetDevice(allocation->context->device);
  if (allocation->imported) {
    cudaStreamSynchronize(allocation->context->stream);
    cudaIpcCloseMemHandle(allocation->base);
  } else {
    cudaFree(allocation->base);  // cudaFree waits for work that may still use the memory
  }
  release(allocation->context);
  delete allocation;
}

void* context_scratch(Context* context, size_t bytes, std::string* error) {
  if (bytes <= context->scratch_bytes) return context->scratch;
  size_t wanted = context->scratch_bytes ? context->scratch_bytes : (size_t)64 << 20;
  while (wanted < bytes) wanted *= 2;
  void* block = nullptr;
  cudaError_t status = cudaMalloc(&block, wanted);
  if (status != cudaSuccess) {
    if (error) *error = std::string("scratch allocation failed: ") + cudaGetErrorString(status);
    return nullptr;
  }
  context->scratch_blocks.push_back(block);
  context->scratch = block;
  context->scratch_bytes = wanted;
  return block;
}
void* context_split_scratch(Context* context, size_t zeroed_bytes, size_t bytes, cudaStream_t stream,
                            std::string* error) {
  if (bytes <= context->split_bytes) return context->split;
  size_t wanted = context->split_bytes ? context->split_bytes : (size_t)32 << 20;
  while (wanted < bytes) wanted *= 2;
  void* block = nullptr;
  cudaError_t status = cudaMalloc(&block, wanted);
  if (status == cudaSuccess) status = cudaMemsetAsync(block, 0, zeroed_bytes, stream);  // ordered before the first user
  if (status != cudaSuccess) {
    if (error) *error = std::string("scratch allocation failed: ") + cudaGetErrorString(status);
    return nullptr;
  }
  context->scratch_blocks.push_back(block);  // freed with the context; earlier blocks stay valid for captured plans
  context->split = block;
  context->split_bytes = wanted;
  context->split_counter_bytes = zeroed_bytes;
  return block;
}
const ExprProgram* context_expr_program(Context* context, const char* name) {
  auto found = context->expr_programs.find(name ? name : "");
  return found == context->expr_programs.end() ? nullptr : &found->second;
}
int context_sm_count(Context* context) { return context->sm_count; }
bool context_overlap(Context* context) { return context != nullptr && context->overlap; }
uint32_t* context_device_error(Context* context) { return context->device_error; }

static void register_kernels(llmopt_cuda_library* library) {
  auto add = [&](const char* name, Launcher launcher) {
    library->launchers[name] = launcher;
    library->names.push_back(name);
  };
  // W4A16 linear: lib/metal_w4a16_source.ml:196-208 (entries)
  add("llmopt_w4a16_linear_f16_g64", launch_w4a16_linear);
  add("llmopt_w4a16_linear_f16_g64_m4", launch_w4a16_linear);
  add("llmopt_w4a16_linear_f16_g64_m8", launch_w4a16_linear);
  add("llmopt_w4a16_linear_f16_g64_affine", launch_w4a16_linear_affine);
  // dense prefill attention: lib/metal_attention_source.ml (specialised per head size, and generic)
  add("llmopt_attention_f16", launch_attention_dense);
  add("llmopt_attention_f16_simd_h32", launch_attention_dense);
  add("llmopt_attention_f16_simd_h64", launch_attention_dense);
  add("llmopt_attention_f16_simd_h80", launch_attention_dense);
  add("llmopt_attention_f16_simd_h96", launch_attention_dense);
  add("llmopt_attention_f16_simd_h128", launch_attention_dense);
  add("llmopt_attention_f16_simd_h256", launch_attention_dense);
  // Q4_0-block family: every tiling tactic of the reference maps to the same arithmetic
  add("llmopt_dequant_q4_0", launch_q4_0_dequant);
  add("llmopt_q4_0_linear_f16", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_x4", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_x4_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_x8", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_x8_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_x16", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_x16_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m2", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m2_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m4", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m4_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m16", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m16_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m32", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_m32_add", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_simd", launch_q4_0_linear);
  add("llmopt_q4_0_linear_f16_simd_add", launch_q4_0_linear);
  add("llmopt_q4_0_qkv_linear_f16", launch_q4_0_qkv_linear);
  add("llmopt_q4_0_qkv_linear_f16_x8", launch_q4_0_qkv_linear);
  add("llmopt_q4_0_qkv_linear_f16_x16", launch_q4_0_qkv_linear);
  add("llmopt_q4_0_qkv_linear_f16_m4", launch_q4_0_qkv_linear);
  add("llmopt_q4_0_qkv_linear_f16_m16", launch_q4_0_qkv_linear);
  add("llmopt_q4_0_qkv_linear_f16_m32", launch_q4_0_qkv_linear);
  add("llmopt_q4_0_gated_linear_f16_x8", launch_q4_0_gated_linear);
  add("llmopt_q4_0_gated_linear_f16_m4", launch_q4_0_gated_linear);
  add("llmopt_q4_0_gated_linear_f16_m16", launch_q4_0_gated_linear);
  add("llmopt_q4_0_gated_linear_f16_m32", launch_q4_0_gated_linear);
  // tensor-parallel extensions (no reference counterpart)
  add("llmopt_w4a16_linear_partial_f32_g64", launch_w4a16_linear_partial_f32);
  add("llmopt_tp_exchange_sum_f16", launch_tp_exchange_sum);
  add("llmopt_tp_exchange_argmax", launch_tp_exchange_argmax);
  add("llmopt_tp_exchange_sum_rms_f16", launch_tp_exchange_sum_norm);
  add("llmopt_tp_exchange_reduce_rows_f16", launch_tp_exchange_reduce_rows);
  add("llmopt_tp_exchange_gather_rows_f16", launch_tp_exchange_gather_rows);
  add("llmopt_w4a16_qkv_linear_f16_g64", launch_w4a16_qkv_linear);
  add("llmopt_w4a16_qkv_linear_f16_g64_m4", launch_w4a16_qkv_linear);
  add("llmopt_w4a16_qkv_linear_f16_g64_m8", launch_w4a16_qkv_linear);
  add("llmopt_w4a16_swiglu_rms_f16_g64", launch_w4a16_swiglu_rms_f16);
  add("llmopt_w4a16_swiglu_rms_f32_g64", launch_w4a16_swiglu_rms_f32);
  add("llmopt_w4a16_dual_swiglu_f16_g64", launch_w4a16_dual_swiglu);
  add("llmopt_w4a16_dual_swiglu_f16_g64_m4", launch_w4a16_dual_swiglu);
  add("llmopt_w4a16_dual_swiglu_f16_g64_m8", launch_w4a16_dual_swiglu);
  add("llmopt_w4a16_down_add_f16_g64", launch_w4a16_down_add);
  add("llmopt_w4a16_down_add_f16_g64_m4", launch_w4a16_down_add);
  add("llmopt_w4a16_down_add_f16_g64_m8", launch_w4a16_down_add);
  add("llmopt_w4a16_linear_f16_g64_epi_none", launch_w4a16_linear_tagged<0>);
  add("llmopt_w4a16_linear_f16_g64_epi_bias", launch_w4a16_linear_tagged<1>);
  add("llmopt_w4a16_linear_f16_g64_epi_silu", launch_w4a16_linear_tagged<2>);
  add("llmopt_w4a16_linear_f16_g64_epi_gelu", launch_w4a16_linear_tagged<3>);
  add("llmopt_w4a16_linear_f16_g64_epi_silu_mul", launch_w4a16_linear_tagged<4>);
  add("llmopt_w4a16_linear_f16_g64_epi_gelu_mul", launch_w4a16_linear_tagged<5>);
  add("llmopt_w4a16_linear_f16_g64_epi_residual_add", launch_w4a16_linear_tagged<6>);
  add("llmopt_w4a16_linear_f16_g64_epi_bias_residual_add", launch_w4a16_linear_tagged<7>);
  add("llmopt_w4a16_linear_f16_g64_epi_silu_mul_residual_add", launch_w4a16_linear_tagged<8>);
  add("llmopt_w4a16_linear_f16_g64_epi_gelu_mul_residual_add", launch_w4a16_linear_tagged<9>);
  add("llmopt_w4a16_lm_head_argmax_f16", launch_w4a16_lm_head_argmax<false, false>);
  add("llmopt_w4a16_lm_head_argmax_extra_f16", launch_w4a16_lm_head_argmax<false, true>);
  add("llmopt_w4a16_lm_head_argmax_f32", launch_w4a16_lm_head_argmax<true, false>);
  add("llmopt_w4a16_lm_head_argmax_extra_f32", launch_w4a16_lm_head_argmax<true, true>);
  add("llmopt_w4a16_lm_head_argmax_stage1_f16", launch_w4a16_lm_head_stage1<false, false>);
  add("llmopt_w4a16_lm_head_argmax_stage1_extra_f16", launch_w4a16_lm_head_stage1<false, true>);
  add("llmopt_w4a16_lm_head_argmax_stage1_f32", launch_w4a16_lm_head_stage1<true, false>);
  add("llmopt_w4a16_lm_head_argmax_stage1_extra_f32", launch_w4a16_lm_head_stage1<true, true>);
  add("llmopt_w4a16_lm_head_reduce", launch_w4a16_lm_head_reduce);
  // grouped-Q8 cache: lib/metal_cache_source.ml
  add("llmopt_cache_pack_attention_q8", launch_cache_pack_attention_q8);
  add("llmopt_cache_pack_attention_q8_simd", launch_cache_pack_attention_q8);
  add("llmopt_cache_pack_attention_q8_pair_simd", launch_cache_pack_attention_q8_pair);
  add("llmopt_cache_unpack_attention_q8", launch_cache_unpack_attention_q8);
  add("llmopt_cache_unpack_attention_q8_vec4", launch_cache_unpack_attention_q8);
  add("llmopt_cache_pack_checkpoint_q8", launch_cache_pack_checkpoint_q8);
  add("llmopt_cache_pack_checkpoint_q8_simd", launch_cache_pack_checkpoint_q8);
  add("llmopt_cache_unpack_checkpoint_q8", launch_cache_unpack_checkpoint_q8);
  add("llmopt_cache_unpack_checkpoint_q8_vec4", launch_cache_unpack_checkpoint_q8);
  add("llmopt_attention_q8_paged_simd_h64", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_simd_generic", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_simd_h256", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_simd_h512", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_simd_h64_gqa3", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_simd_h64_split8", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_simd_h64_gqa3_split8", launch_attention_q8_paged);
  add("llmopt_attention_q8_paged_batched", launch_attention_q8_paged);
  // recurrent: lib/metal_recurrent_source.ml
  add("llmopt_short_conv_f16", launch_short_conv<false>);
  add("llmopt_short_conv_f16_f32", launch_short_conv<true>);
  add("llmopt_short_conv_silu_tm_f16", launch_short_conv_silu_tm<false>);
  add("llmopt_short_conv_silu_tm_f32", launch_short_conv_silu_tm<true>);
  add("llmopt_short_conv_step_f16", launch_short_conv_step);
  add("llmopt_short_conv_step_fused_f16", launch_short_conv_step);
  add("llmopt_short_conv_prefill_f16", launch_short_conv_prefill);
  add("llmopt_short_conv_prefill_init_f16", launch_short_conv_prefill);
  // glue for whole decode steps
  add("llmopt_rms_norm_f16", launch_rms_norm<false>);
  add("llmopt_rms_norm_f16_simd", launch_rms_norm<false>);
  add("llmopt_rms_norm_f32_f16", launch_rms_norm<true>);
  add("llmopt_rms_norm_f32_f16_simd", launch_rms_norm<true>);
  add("llmopt_rotary_qk_f16_simd_h64", launch_rotary_qk);
  add("llmopt_embedding_f16", launch_embedding_f16);
  add("llmopt_chain_token_id", launch_chain_token_id);
  add("llmopt_chain_token_ids", launch_chain_token_ids);
  add("llmopt_cache_pack_attention_tile32_affine8_fwht_simd", launch_cache_pack_tile32_affine8_fwht);
  add("llmopt_cache_unpack_attention_tile32_affine8_fwht_simd", launch_cache_unpack_tile32_affine8_fwht);
  add("llmopt_cache_pack_attention_tile32_affine4_fwht_simd", launch_cache_pack_tile32_affine4_fwht);
  add("llmopt_cache_unpack_attention_tile32_affine4_fwht_simd", launch_cache_unpack_tile32_affine4_fwht);
  // Tile32 affine linears: every tiling tactic of the format runs the same kernel
  static const char* const kTile32Affine4[] = {
      "llmopt_tile32_affine4_linear_f16_x8",   "llmopt_tile32_affine4_linear_f16_m16",
      "llmopt_tile32_affine4_linear_f16_m32",  "llmopt_tile32_affine4_linear_f16_simd",
      "llmopt_tile32_affine4_linear_f16_m16_add", "llmopt_tile32_affine4_linear_f16_m32_add"};
  static const char* const kTile32Affine8[] = {
      "llmopt_tile32_affine8_linear_f16_x8",   "llmopt_tile32_affine8_linear_f16_m16",
      "llmopt_tile32_affine8_linear_f16_m32",  "llmopt_tile32_affine8_linear_f16_simd",
      "llmopt_tile32_affine8_linear_f16_m16_add", "llmopt_tile32_affine8_linear_f16_m32_add"};
  for (const char* name : kTile32Affine4) add(name, launch_tile32_affine4_linear);
  for (const char* name : kTile32Affine8) add(name, launch_tile32_affine8_linear);
  // gated-delta scan (one name per state width) and the triangular recurrence (gated_delta.cu)
  static const char* const kGatedDeltaF32[] = {
      "llmopt_gated_delta_f32_d32",  "llmopt_gated_delta_f32_d64",  "llmopt_gated_delta_f32_d96",
      "llmopt_gated_delta_f32_d128", "llmopt_gated_delta_f32_d160", "llmopt_gated_delta_f32_d192",
      "llmopt_gated_delta_f32_d224", "llmopt_gated_delta_f32_d256"};
  static const char* const kGatedDeltaF16[] = {
      "llmopt_gated_delta_tm_f16_d32",  "llmopt_gated_delta_tm_f16_d64",  "llmopt_gated_delta_tm_f16_d96",
      "llmopt_gated_delta_tm_f16_d128", "llmopt_gated_delta_tm_f16_d160", "llmopt_gated_delta_tm_f16_d192",
      "llmopt_gated_delta_tm_f16_d224", "llmopt_gated_delta_tm_f16_d256"};
  for (const char* name : kGatedDeltaF32) add(name, launch_gated_delta_f32);
  for (const char* name : kGatedDeltaF16) add(name, launch_gated_delta_tm_f16);
  add("llmopt_triangular_recurrence_f32", launch_triangular_recurrence);
  // norm variants, fused norm + rotary, casts, pointwise (norm_family.cu)
  size_t extra = 0;
  const NamedLauncher* table = norm_family_launchers(&extra);
  for (size_t i = 0; i < extra; ++i) add(table[i].name, table[i].launcher);
}

static bool is_paged_attention_name(const char* name) {
  static const char prefix[] = "llmopt_attention_q8_paged_";  // native/ocaml_metal_stubs.m:145-148
  return strncmp(name, prefix, sizeof(prefix) - 1) == 0;
}
static bool is_checkpoint_pack_name(const char* name) {
  return strcmp(name, "llmopt_cache_pack_checkpoint_q8_simd") == 0;  // :1965
}

// A dispatch with everything owned: buffers retained, parameter bytes copied.
struct OwnedRecord {
  std::string name;
  Launcher launcher = nullptr;
  std::vector<llmopt_cuda_buffer*> buffers;
  std::vector<uint8_t> params;
  uint32_t grid[3] = {1, 1, 1}, group[3] = {1, 1, 1};
  bool is_copy = false;
};

static void retain_buffer(llmopt_cuda_buffer* buffer) { buffer->references.fetch_add(1); }

static void release_record(OwnedRecord& record) {
  for (llmopt_cuda_buffer* buffer : record.buffers) llmopt_cuda_release_buffer(buffer);
  record.buffers.clear();
}

static int own_record(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* record, OwnedRecord* out) {
  if (library == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA library has been finalized");
  if (record == nullptr || record->name == nullptr)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "dispatch record has no kernel name");
  auto found = library->launchers.find(record->name);
  if (found == library->launchers.end())
    return set_error(LLMOPT_CUDA_FAILURE, std::string("CUDA kernel function is missing: ") + record->name);
  if (record->buffer_count < 0 || record->buffer_count > kMaxBuffers)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "a dispatch binds at most 16 buffers");
  if (record->parameter_bytes > (size_t)kMaxParamBytes)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "a dispatch carries at most 256 parameter bytes");
  for (int axis = 0; axis < 3; ++axis) {
    // positive_size, native/ocaml_metal_stubs.m:1161-1168
    if (record->grid[axis] <= 0) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "grid dimensions must be positive");
    if (record->group[axis] <= 0)
      return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "threadgroup dimensions must be positive");
  }
  if ((int64_t)record->group[0] * record->group[1] * record->group[2] > 1024)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "threadgroup exceeds pipeline capacity");
  for (int i = 0; i < record->buffer_count; ++i) {
    if (record->buffers[i] == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
    if (record->buffers[i]->allocation->context != library->context)
      return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "buffer belongs to another context");
  }
  out->name = record->name;
  out->launcher = found->second;
  out->buffers.assign(record->buffers, record->buffers + record->buffer_count);
  for (llmopt_cuda_buffer* buffer : out->buffers) retain_buffer(buffer);
  out->params.assign((const uint8_t*)record->parameters, (const uint8_t*)record->parameters + record->parameter_bytes);
  for (int axis = 0; axis < 3; ++axis) {
    out->grid[axis] = (uint32_t)record->grid[axis];
    out->group[axis] = (uint32_t)record->group[axis];
  }
  return LLMOPT_CUDA_OK;
}

// Plan-level fusion: a row RMS norm whose output is the activation input of the W4A16 product that
// follows it is folded into that product (the product normalises the raw rows while it stages
// them and still writes the normalised tensor).  Recognised by name and by buffer identity:
//   norm    llmopt_rms_norm_f16{,_simd} [x, w, y] {rows, width, eps}      -> (x inv) w
//           llmopt_w4a16_swiglu_rms_f16_g64 [x, w, y] {m, n, k, eps}      -> (x w) inv
//   product llmopt_w4a16_{linear,qkv_linear,dual_swiglu}_f16_g64*  with buffers[0] == y, same rows / k
static bool fold_norm(const OwnedRecord& norm, const OwnedRecord& product, FusedNorm* fused) {
  if (norm.is_copy || product.is_copy || norm.buffers.size() != 3 || product.buffers.empty()) return false;
  uint32_t rows, width;
  float epsilon;
  bool weight_first;
  auto u32 = [](const OwnedRecord& record, size_t index) {
    uint32_t value;
    memcpy(&value, record.params.data() + 4 * index, 4);
    return value;
  };
  if ((norm.name == "llmopt_rms_norm_f16_simd" || norm.name == "llmopt_rms_norm_f16") && norm.params.size() == 12) {
    rows = u32(norm, 0), width = u32(norm, 1), weight_first = false;
    memcpy(&epsilon, norm.params.data() + 8, 4);
  } else if (norm.name == "llmopt_w4a16_swiglu_rms_f16_g64" && norm.params.size() == 16) {
    rows = u32(norm, 0), width = u32(norm, 2), weight_first = true;
    memcpy(&epsilon, norm.params.data() + 12, 4);
  } else {
    return false;
  }
  uint32_t m, k;
  const std::string& name = product.name;
  if (name.rfind("llmopt_w4a16_qkv_linear_f16_g64", 0) == 0 && product.params.size() == 20) {
    m = u32(product, 0), k = u32(product, 1);
  } else if ((name.rfind("llmopt_w4a16_dual_swiglu_f16_g64", 0) == 0 && product.params.size() == 16) ||
             ((name == "llmopt_w4a16_linear_f16_g64" || name == "llmopt_w4a16_linear_f16_g64_m4" ||
               name == "llmopt_w4a16_linear_f16_g64_m8") && product.params.size() == 20)) {
    m = u32(product, 0), k = u32(product, 2);
  } else {
    return false;
  }
  llmopt_cuda_buffer* normalized = norm.buffers[2];
  llmopt_cuda_buffer* consumed = product.buffers[0];
  if (normalized->pointer() != consumed->pointer() || m != rows || k != width || rows == 0 || rows > 8) return false;
  if (normalized->length < (size_t)rows * width * 2 || norm.buffers[0]->length < (size_t)rows * width * 2 ||
      norm.buffers[1]->length < (size_t)width * 2)
    return false;
  // The product reads the raw rows while one of its CTAs writes the normalised ones, and writes its
  // outputs while other CTAs still read the raw rows: the raw rows [input, +rows*width*2) must be
  // disjoint from the normalised rows (no in-place norm, no overlapping views) and from every
  // other buffer the product binds.
  const size_t row_bytes = (size_t)rows * width * 2;
  auto overlaps = [](const uint8_t* a, size_t a_bytes, const uint8_t* b, size_t b_bytes) {
    return a < b + b_bytes && b < a + a_bytes;
  };
  const uint8_t* raw = norm.buffers[0]->pointer();
  if (overlaps(raw, row_bytes, normalized->pointer(), row_bytes)) return false;
  for (llmopt_cuda_buffer* buffer : product.buffers)
    if (buffer != consumed && overlaps(raw, row_bytes, buffer->pointer(), buffer->length)) return false;
  // likewise nothing else the product binds may alias the normalised rows it is about to write
  for (llmopt_cuda_buffer* buffer : product.buffers)
    if (buffer != consumed && overlaps(normalized->pointer(), row_bytes, buffer->pointer(), buffer->length)) return false;
  fused->input = (const __half*)norm.buffers[0]->pointer();
  fused->weight = (const __half*)norm.buffers[1]->pointer();
  fused->normalized = (__half*)normalized->pointer();
  fused->epsilon = epsilon;
  fused->weight_first = weight_first ? 1u : 0u;
  return true;
}

// The per-token values of a replayed plan index device tables the plan captured: row bindings
// read row `past_tokens` of their table, paged attention reads `past_tokens` slot entries per
// sequence.  The smallest of those bounds is the largest past_tokens a replay accepts.
static int64_t plan_token_capacity(const std::vector<OwnedRecord>& records, const llmopt_cuda_row_binding* bindings,
                                   size_t binding_count) {
  int64_t capacity = INT32_MAX;
  for (size_t i = 0; i < binding_count; ++i) {
    const int64_t rows = (int64_t)(bindings[i].table->length / bindings[i].row_bytes);
    capacity = std::min(capacity, rows - 1);
  }
  for (const OwnedRecord& record : records) {
    if (record.is_copy || !is_paged_attention_name(record.name.c_str()) || record.params.size() < 64 ||
        record.buffers.size() < 5)
      continue;
    uint32_t batches = 0, stride = 0;
    memcpy(&batches, record.params.data(), 4);
    if (record.params.size() >= 68) memcpy(&stride, record.params.data() + 64, 4);
    const int64_t entries = (int64_t)(record.buffers[4]->length / 4);
    int64_t per_sequence = entries;
    if (batches > 1) {
      per_sequence = entries - (int64_t)(batches - 1) * stride;
      if (stride > 0) per_sequence = std::min<int64_t>(per_sequence, stride);
    }
    capacity = std::min(capacity, per_sequence);
  }
  return capacity < 0 ? -1 : capacity;
}

static void fill_args(Context* context, const OwnedRecord& record, const uint32_t* past_cell,
                      const uint32_t* checkpoint_cell, KernelArgs* out) {
  KernelArgs& args = *out;
  args.ctx = context;
  args.stream = context->stream;
  args.buffer_count = (int)record.buffers.size();
  for (size_t i = 0; i < record.buffers.size(); ++i) {
    args.buffers[i] = record.buffers[i]->pointer();
    args.lengths[i] = record.buffers[i]->length;
  }
  args.params = record.params.data();
  args.param_bytes = record.params.size();
  for (int axis = 0; axis < 3; ++axis) {
    args.grid[axis] = record.grid[axis];
    args.group[axis] = record.group[axis];
  }
  args.name = record.name.c_str();
  args.past_tokens_cell = is_paged_attention_name(args.name) && record.params.size() >= 16 ? past_cell : nullptr;
  args.checkpoint_cell = is_checkpoint_pack_name(args.name) && record.params.size() >= 4 ? checkpoint_cell : nullptr;
}

static int run_record(Context* context, const OwnedRecord& record, const uint32_t* past_cell,
                      const uint32_t* checkpoint_cell, const FusedNorm* fused_norm = nullptr) {
  if (record.is_copy) {
    CUDA_TRY(cudaMemcpyAsync(record.buffers[1]->pointer(), record.buffers[0]->pointer(), record.buffers[0]->length,
                             cudaMemcpyDeviceToDevice, context->stream),
             "CUDA batch copy failed");
    return LLMOPT_CUDA_OK;
  }
  KernelArgs args = {};
  fill_args(context, record, past_cell, checkpoint_cell, &args);
  args.fused_norm = fused_norm;
  std::string message;
  args.error = &message;
  if (record.launcher(args) != 0) return set_error(LLMOPT_CUDA_FAILURE, message);
  return LLMOPT_CUDA_OK;
}

// Plan-capture peephole: a rotary record directly followed by the pair-pack record of the same
// decode token runs as one kernel.  Returns -1 when the pair does not fit the fused form.
static int run_rotary_pack(Context* context, const OwnedRecord& rotary, const OwnedRecord& pack) {
  if (rotary.is_copy || pack.is_copy || rotary.name != "llmopt_rotary_qk_f16_simd_h64" ||
      pack.name != "llmopt_cache_pack_attention_q8_pair_simd")
    return -1;
  KernelArgs rotary_args = {}, pack_args = {};
  fill_args(context, rotary, nullptr, nullptr, &rotary_args);
  fill_args(context, pack, nullptr, nullptr, &pack_args);
  std::string message;
  rotary_args.error = &message;
  pack_args.error = &message;
  const int status = launch_rotary_pack_fused(rotary_args, pack_args);
  if (status > 0) return set_error(LLMOPT_CUDA_FAILURE, message);
  return status < 0 ? -1 : LLMOPT_CUDA_OK;
}

// Plan-capture peephole: rotary record, pair-pack record and the paged attention of the same decode token as
// ONE attention launch that rotates its query rows itself and hands the rotated rows and the new slot's Q8
// bytes out as warp tasks.  Returns -1 when the three do not fit that form.
static int run_rotary_pack_attention(Context* context, const OwnedRecord& rotary, const OwnedRecord& pack,
                                     const OwnedRecord& attention, const uint32_t* past_cell,
                                     const uint32_t* checkpoint_cell) {
  if (rotary.is_copy || pack.is_copy || attention.is_copy || rotary.name != "llmopt_rotary_qk_f16_simd_h64" ||
      pack.name != "llmopt_cache_pack_attention_q8_pair_simd" ||
      attention.name.rfind("llmopt_attention_q8_paged_", 0) != 0)
    return -1;
  KernelArgs rotary_args = {}, pack_args = {}, attention_args = {};
  fill_args(context, rotary, nullptr, nullptr, &rotary_args);
  fill_args(context, pack, nullptr, nullptr, &pack_args);
  fill_args(context, attention, past_cell, checkpoint_cell, &attention_args);
  RotaryPackFusion fusion;
  if (!make_rotary_pack_fusion(rotary_args, pack_args, &fusion) || !paged_attention_takes_rotary_pack(attention_args, fusion))
    return -1;
  attention_args.rotary_fusion = &fusion;
  std::string message;
  attention_args.error = &message;
  if (attention.launcher(attention_args) != 0) return set_error(LLMOPT_CUDA_FAILURE, message);
  return LLMOPT_CUDA_OK;
}

static int wait_stream(Context* context, const char* what) {
  cudaError_t status = cudaStreamSynchronize(context->stream);
  if (status != cudaSuccess) return cuda_failure(what, status);
  if (context->device_error && *(volatile uint32_t*)context->device_error != 0) {
    *(volatile uint32_t*)context->device_error = 0;
    // A split-K GEMM CTA that gave up never bumped its tile's arrival counter, so the counter was
    // not returned to zero by a last arrival: clear them all, or the next launch would elect its
    // last split too early.
    if (context->split && context->split_counter_bytes) {
      cudaMemsetAsync(context->split, 0, context->split_counter_bytes, context->stream);
      cudaStreamSynchronize(context->stream);
    }
    return set_error(LLMOPT_CUDA_FAILURE, std::string(what) + ": a device-side check failed: a bounded wait ran out or a slot / checkpoint index lay outside its pool (results are invalid)");
  }
  return LLMOPT_CUDA_OK;
}

// ---- prebaked plan ------------------------------------------------------------------

struct PlanCells {       // device resident
  uint32_t past_tokens;  // read by paged attention kernels
  uint32_t checkpoint;   // read by the checkpoint pack kernel
  long long token;       // copied into the token buffer by the prologue
};

struct RowBindingDevice {
  uint8_t* destination;
  const uint8_t* table;
  uint32_t row_bytes;
};
struct RowBindings {
  RowBindingDevice item[8];
  int count;
};

__global__ void plan_prologue_kernel(const PlanCells* cells, long long* token_buffer, RowBindings bindings) {
  grid_chain_prologue();
  if (blockIdx.x == 0 && threadIdx.x == 0 && token_buffer != nullptr) token_buffer[0] = cells->token;
  const uint32_t past = cells->past_tokens;
  for (int b = 0; b < bindings.count; ++b) {
    const RowBindingDevice binding = bindings.item[b];
    const uint8_t* source = binding.table + (size_t)past * binding.row_bytes;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < binding.row_bytes; i += gridDim.x * blockDim.x)
      binding.destination[i] = source[i];
  }
}

// Between chained replays: next token = previous output, one more past token.
__global__ void plan_advance_kernel(PlanCells* cells, const int* output, int* tokens_out, int step) {
  grid_chain_prologue();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const int token = output[0];
    tokens_out[step] = token;
    cells->token = (long long)token;
    cells->past_tokens += 1;
  }
}

}  // namespace llmopt

struct llmopt_cuda_prebaked {
  Context* context = nullptr;
  std::vector<OwnedRecord> records;
  llmopt_cuda_buffer* token_buffer = nullptr;
  llmopt_cuda_buffer* output_buffer = nullptr;
  std::vector<llmopt_cuda_buffer*> binding_buffers;
  PlanCells* cells = nullptr;        // device
  PlanCells* staging = nullptr;      // pinned host, ring of kStaging slots
  int staging_next = 0;
  int* result_host = nullptr;        // pinned host
  int* chained_tokens = nullptr;     // device, grown on demand
  int chained_capacity = 0;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t executable = nullptr;
  int kernel_nodes = 0;
  int folded_norms = 0;  // norm records folded into the product that follows them
  // Largest past_tokens a replay may run with: every row binding must hold row `past_tokens`
  // and every paged-attention slot table `past_tokens` entries per sequence.
  int64_t token_capacity = INT32_MAX;
  static constexpr int kStaging = 16;
};

struct llmopt_cuda_batch {
  llmopt_cuda_library* library = nullptr;
  std::vector<OwnedRecord> pending;
  bool finished = false;
};

struct RingEntry {
  int64_t request_id;
  int64_t token;
  int32_t past_tokens;
  int32_t flags;
};
struct RingCompletion {
  int64_t request_id;
  int32_t token;
  int32_t status;
};
struct llmopt_cuda_ring {
  static constexpr size_t kCapacity = 256;  // native/ocaml_metal_stubs.m:1467
  std::mutex mutex;
  std::condition_variable submitted, completed;
  std::deque<RingEntry> submissions;
  std::deque<RingCompletion> completions;
  std::thread worker;
  llmopt_cuda_prebaked* plan = nullptr;
  bool started = false;
  bool stopping = false;
};

extern "C" {

const char* llmopt_cuda_last_error(void) { return g_last_error.c_str(); }

int llmopt_cuda_create_context(int device, llmopt_cuda_context** out) {
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  int count = 0;
  cudaError_t status = cudaGetDeviceCount(&count);
  if (status != cudaSuccess || count == 0)
    return set_error(LLMOPT_CUDA_FAILURE, std::string("no CUDA device is available: ") + cudaGetErrorString(status));
  if (device < 0) CUDA_TRY(cudaGetDevice(&device), "cudaGetDevice failed");
  if (device >= count) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "CUDA device index is out of range");
  CUDA_TRY(cudaSetDevice(device), "cudaSetDevice failed");
  cudaDeviceProp properties;
  CUDA_TRY(cudaGetDeviceProperties(&properties, device), "cudaGetDeviceProperties failed");
  if (properties.major != 10)
    return set_error(LLMOPT_CUDA_FAILURE, std::string("libllmopt_cuda is built for sm_100a only; device is ") +
                                              properties.name);
  llmopt_cuda_context* context = new llmopt_cuda_context();
  context->device = device;
  context->sm_count = properties.multiProcessorCount;
  if (const char* overlap = getenv("LLMOPT_CUDA_OVERLAP")) context->overlap = overlap[0] != '0';
  context->name = properties.name;
  status = cudaStreamCreateWithFlags(&context->stream, cudaStreamNonBlocking);
  if (status != cudaSuccess) {
    delete context;
    return cuda_failure("cudaStreamCreate failed", status);
  }
  status = cudaMalloc((void**)&context->argmax_result, sizeof(int));
  if (status == cudaSuccess) status = cudaHostAlloc((void**)&context->device_error, sizeof(uint32_t), cudaHostAllocMapped);
  if (status == cudaSuccess) *context->device_error = 0;
  if (status != cudaSuccess) {
    release(context);
    return cuda_failure("context allocation failed", status);
  }
  std::string message;
  if (context_scratch(context, (size_t)64 << 20, &message) == nullptr) {
    release(context);
    return set_error(LLMOPT_CUDA_FAILURE, message);
  }
  *out = context;
  return LLMOPT_CUDA_OK;
}

void llmopt_cuda_release_context(llmopt_cuda_context* context) {
  if (context) release(static_cast<Context*>(context));
}

const char* llmopt_cuda_device_name(llmopt_cuda_context* context) { return context ? context->name.c_str() : ""; }

int llmopt_cuda_load_library(llmopt_cuda_context* context, const char* path, llmopt_cuda_library** out) {
  (void)path;
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  llmopt_cuda_library* library = new llmopt_cuda_library();
  library->context = context;
  retain(context);
  register_kernels(library);
  *out = library;
  return LLMOPT_CUDA_OK;
}

void llmopt_cuda_release_library(llmopt_cuda_library* library) {
  if (library == nullptr || library->references.fetch_sub(1) != 1) return;
  release(library->context);
  delete library;
}

int llmopt_cuda_has_function(llmopt_cuda_library* library, const char* name) {
  return library != nullptr && name != nullptr && library->launchers.count(name) ? 1 : 0;
}

int llmopt_cuda_preload_pipeline(llmopt_cuda_library* library, const char* name) {
  if (library == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA library has been finalized");
  if (!llmopt_cuda_has_function(library, name))
    return set_error(LLMOPT_CUDA_FAILURE, std::string("CUDA kernel function is missing: ") + (name ? name : "(null)"));
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_function_count(llmopt_cuda_library* library) { return library ? (int)library->names.size() : 0; }
const char* llmopt_cuda_function_name(llmopt_cuda_library* library, int index) {
  if (library == nullptr || index < 0 || index >= (int)library->names.size()) return nullptr;
  return library->names[index].c_str();
}

int llmopt_cuda_register_alias(llmopt_cuda_library* library, const char* alias, const char* target) {
  if (library == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA library has been finalized");
  if (alias == nullptr || target == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null kernel name");
  auto found = library->launchers.find(target);
  if (found == library->launchers.end())
    return set_error(LLMOPT_CUDA_FAILURE, std::string("CUDA kernel function is missing: ") + target);
  if (!library->launchers.count(alias)) library->names.push_back(alias);
  library->launchers[alias] = found->second;
  // an expression epilogue is found by the name it is dispatched under: the alias gets the program too
  auto program = library->context->expr_programs.find(target);
  if (program != library->context->expr_programs.end()) library->context->expr_programs[alias] = program->second;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_register_expr_epilogue(llmopt_cuda_library* library, const char* name, const void* program,
                                       size_t program_bytes, int operand_count) {
  if (library == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA library has been finalized");
  if (name == nullptr || name[0] == '\0' || program == nullptr)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "expression epilogue needs a name and a program");
  if (library->launchers.count(name))
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, std::string("kernel name is already taken: ") + name);
  if (const char* problem = validate_expr_program((const uint8_t*)program, program_bytes, operand_count))
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, problem);
  ExprProgram stored = {};
  memcpy(stored.code, program, program_bytes);
  stored.length = (uint32_t)program_bytes;
  stored.operands = (uint32_t)operand_count;
  library->context->expr_programs[name] = stored;
  // the base the digest name extends decides the product and the buffer order
  const bool over_q4_0 = strncmp(name, "llmopt_q4_0_linear_f16", 22) == 0;
  library->launchers[name] = over_q4_0 ? launch_q4_0_linear_expr : launch_w4a16_linear_expr;
  library->names.push_back(name);
  return LLMOPT_CUDA_OK;
}

// ---- buffers ---------------------------------------------------------------------------

static int new_allocation(llmopt_cuda_context* context, size_t length, llmopt_cuda_buffer** out) {
  CUDA_TRY(cudaSetDevice(context->device), "cudaSetDevice failed");
  void* base = nullptr;
  // 256-byte granularity keeps every tensor view of a mapped archive aligned
  const size_t padded = (length + 255) / 256 * 256;
  cudaError_t status = cudaMalloc(&base, padded);
  if (status != cudaSuccess) return cuda_failure("CUDA could not allocate a buffer", status);
  Allocation* allocation = new Allocation();
  allocation->context = context;
  retain(context);
  allocation->base = base;
  allocation->length = length;
  llmopt_cuda_buffer* buffer = new llmopt_cuda_buffer();
  buffer->allocation = allocation;
  buffer->offset = 0;
  buffer->length = length;
  *out = buffer;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_buffer_of_bytes(llmopt_cuda_context* context, const void* bytes, size_t length,
                                llmopt_cuda_buffer** out) {
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  if (out == nullptr || (bytes == nullptr && length > 0))
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null pointer argument");
  const size_t actual = length == 0 ? 16 : length;
  if (int status = new_allocation(context, actual, out)) return status;
  cudaError_t status = cudaMemsetAsync((*out)->pointer(), 0, (actual + 255) / 256 * 256, context->stream);
  if (status == cudaSuccess && length > 0)
    status = cudaMemcpyAsync((*out)->pointer(), bytes, length, cudaMemcpyHostToDevice, context->stream);
  if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
  if (status != cudaSuccess) {
    llmopt_cuda_release_buffer(*out);
    *out = nullptr;
    return cuda_failure("CUDA could not fill a buffer", status);
  }
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_create_buffer(llmopt_cuda_context* context, int64_t length, llmopt_cuda_buffer** out) {
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  const size_t actual = length <= 0 ? 16 : (size_t)length;
  if (int status = new_allocation(context, actual, out)) return status;
  cudaError_t status = cudaMemsetAsync((*out)->pointer(), 0, (actual + 255) / 256 * 256, context->stream);
  if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
  if (status != cudaSuccess) {
    llmopt_cuda_release_buffer(*out);
    *out = nullptr;
    return cuda_failure("CUDA could not clear a buffer", status);
  }
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_map_file(llmopt_cuda_context* context, const char* path, llmopt_cuda_buffer** out) {
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  if (out == nullptr || path == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null pointer argument");
  const int descriptor = open(path, O_RDONLY);
  if (descriptor < 0) return set_error(LLMOPT_CUDA_FAILURE, std::string("could not open ") + path);
  struct stat info;
  if (fstat(descriptor, &info) != 0 || info.st_size <= 0) {
    close(descriptor);
    return set_error(LLMOPT_CUDA_FAILURE, std::string("could not size ") + path);
  }
  void* mapped = mmap(nullptr, (size_t)info.st_size, PROT_READ, MAP_PRIVATE, descriptor, 0);
  close(descriptor);
  if (mapped == MAP_FAILED) return set_error(LLMOPT_CUDA_FAILURE, std::string("could not map ") + path);
  const int status = llmopt_cuda_buffer_of_bytes(context, mapped, (size_t)info.st_size, out);
  munmap(mapped, (size_t)info.st_size);
  return status;
}

int llmopt_cuda_buffer_view(llmopt_cuda_buffer* parent, int64_t offset, int64_t length, llmopt_cuda_buffer** out) {
  if (parent == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  if (offset < 0 || length < 0 || (uint64_t)offset > parent->length ||
      (uint64_t)length > parent->length - (uint64_t)offset)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "CUDA buffer view is outside its parent");
  llmopt_cuda_buffer* view = new llmopt_cuda_buffer();
  view->allocation = parent->allocation;
  parent->allocation->references.fetch_add(1);
  view->offset = parent->offset + (size_t)offset;
  view->length = (size_t)length;
  *out = view;
  return LLMOPT_CUDA_OK;
}

// ---- sharing a buffer with the other ranks of a tensor-parallel group -------------------
int llmopt_cuda_buffer_export(llmopt_cuda_buffer* buffer, void* handle, uint64_t* offset) {
  if (buffer == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (handle == nullptr || offset == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null pointer argument");
  if (buffer->allocation->imported)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "an imported buffer cannot be exported again");
  static_assert(sizeof(cudaIpcMemHandle_t) == LLMOPT_CUDA_EXPORT_HANDLE_BYTES, "handle size");
  CUDA_TRY(cudaSetDevice(buffer->allocation->context->device), "cudaSetDevice failed");
  cudaIpcMemHandle_t ipc;
  CUDA_TRY(cudaIpcGetMemHandle(&ipc, buffer->allocation->base), "CUDA could not export the buffer");
  memcpy(handle, &ipc, sizeof(ipc));
  *offset = buffer->offset;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_buffer_import(llmopt_cuda_context* context, const void* handle, uint64_t offset, uint64_t length,
                              llmopt_cuda_buffer** out) {
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  if (handle == nullptr || out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null pointer argument");
  CUDA_TRY(cudaSetDevice(context->device), "cudaSetDevice failed");
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, sizeof(ipc));
  void* base = nullptr;
  cudaError_t status = cudaIpcOpenMemHandle(&base, ipc, cudaIpcMemLazyEnablePeerAccess);
  if (status != cudaSuccess) return cuda_failure("CUDA could not open a peer's buffer", status);
  Allocation* allocation = new Allocation();
  allocation->context = context;
  retain(context);
  allocation->base = base;
  allocation->length = (size_t)(offset + length);
  allocation->imported = true;
  llmopt_cuda_buffer* buffer = new llmopt_cuda_buffer();
  buffer->allocation = allocation;
  buffer->offset = (size_t)offset;
  buffer->length = (size_t)length;
  *out = buffer;
  return LLMOPT_CUDA_OK;
}

void llmopt_cuda_release_buffer(llmopt_cuda_buffer* buffer) {
  if (buffer == nullptr || buffer->references.fetch_sub(1) != 1) return;
  release(buffer->allocation);
  delete buffer;
}

size_t llmopt_cuda_buffer_length(llmopt_cuda_buffer* buffer) { return buffer ? buffer->length : 0; }

void* llmopt_cuda_buffer_device_pointer(llmopt_cuda_buffer* buffer) { return buffer ? buffer->pointer() : nullptr; }

int llmopt_cuda_buffer_contents(llmopt_cuda_buffer* buffer, void* destination, size_t capacity) {
  if (buffer == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (destination == nullptr || capacity < buffer->length)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "destination is smaller than the buffer");
  Context* context = buffer->allocation->context;
  CUDA_TRY(cudaMemcpyAsync(destination, buffer->pointer(), buffer->length, cudaMemcpyDeviceToHost, context->stream),
           "CUDA buffer readback failed");
  return wait_stream(context, "CUDA buffer readback failed");
}

int llmopt_cuda_buffer_argmax_f16(llmopt_cuda_buffer* buffer, int64_t vocabulary, int64_t* out) {
  if (buffer == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  if (vocabulary <= 0 || (uint64_t)vocabulary * 2 > buffer->length)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "argmax vocabulary is outside the buffer");
  Context* context = buffer->allocation->context;
  const size_t rows = buffer->length / ((size_t)vocabulary * 2);
  const __half* last_row = (const __half*)buffer->pointer() + (rows - 1) * (size_t)vocabulary;
  launch_argmax_f16(last_row, (uint32_t)vocabulary, context->argmax_result, context->stream);
  int result = 0;
  CUDA_TRY(cudaMemcpyAsync(&result, context->argmax_result, sizeof(int), cudaMemcpyDeviceToHost, context->stream),
           "CUDA argmax readback failed");
  if (int status = wait_stream(context, "CUDA argmax failed")) return status;
  *out = result;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_buffer_copy(llmopt_cuda_buffer* source, llmopt_cuda_buffer* destination) {
  if (source == nullptr || destination == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (source->length != destination->length)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "CUDA buffer copy needs equal lengths");
  Context* context = destination->allocation->context;
  CUDA_TRY(cudaMemcpyAsync(destination->pointer(), source->pointer(), source->length, cudaMemcpyDeviceToDevice,
                           context->stream),
           "CUDA buffer copy failed");
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_buffer_write(llmopt_cuda_buffer* buffer, int64_t offset, const void* bytes, size_t length) {
  if (buffer == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (offset < 0 || (uint64_t)offset > buffer->length || length > buffer->length - (uint64_t)offset)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "host write is outside the buffer");
  if (length == 0) return LLMOPT_CUDA_OK;
  if (bytes == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null source pointer");
  Context* context = buffer->allocation->context;
  // pageable source: the runtime stages the bytes before returning, so the caller may reuse them
  CUDA_TRY(cudaMemcpyAsync(buffer->pointer() + offset, bytes, length, cudaMemcpyHostToDevice, context->stream),
           "CUDA host write failed");
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_buffer_set_int64(llmopt_cuda_buffer* buffer, int64_t offset, int64_t value) {
  return llmopt_cuda_buffer_write(buffer, offset, &value, sizeof(value));
}

int llmopt_cuda_buffer_set_u32_array(llmopt_cuda_buffer* buffer, int64_t offset, const uint32_t* values,
                                     size_t count) {
  return llmopt_cuda_buffer_write(buffer, offset, values, count * sizeof(uint32_t));
}

// ---- dispatch ----------------------------------------------------------------------------

int llmopt_cuda_dispatch(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* record) {
  OwnedRecord owned;
  if (int status = own_record(library, record, &owned)) return status;
  int status = run_record(library->context, owned, nullptr, nullptr);
  if (status == LLMOPT_CUDA_OK) status = wait_stream(library->context, "CUDA dispatch failed");
  release_record(owned);
  return status;
}

int llmopt_cuda_begin_batch(llmopt_cuda_library* library, llmopt_cuda_batch** out) {
  if (library == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA library has been finalized");
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  llmopt_cuda_batch* batch = new llmopt_cuda_batch();
  batch->library = library;
  library->references.fetch_add(1);
  *out = batch;
  return LLMOPT_CUDA_OK;
}

static int require_active(llmopt_cuda_batch* batch) {
  if (batch == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA batch has been finalized");
  if (batch->finished) return set_error(LLMOPT_CUDA_FAILURE, "CUDA batch is already finished");
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_batch_dispatch(llmopt_cuda_batch* batch, llmopt_cuda_library* library,
                               const llmopt_cuda_dispatch_record* record) {
  if (int status = require_active(batch)) return status;
  OwnedRecord owned;
  if (int status = own_record(library, record, &owned)) return status;
  batch->pending.push_back(std::move(owned));
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_batch_dispatch_all(llmopt_cuda_batch* batch, llmopt_cuda_library* library,
                                   const llmopt_cuda_dispatch_record* records, size_t count) {
  for (size_t i = 0; i < count; ++i)
    if (int status = llmopt_cuda_batch_dispatch(batch, library, &records[i])) return status;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_batch_copy(llmopt_cuda_batch* batch, llmopt_cuda_buffer* source, llmopt_cuda_buffer* destination) {
  if (int status = require_active(batch)) return status;
  if (source == nullptr || destination == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA buffer has been finalized");
  if (source->length != destination->length)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "CUDA batch copy needs equal lengths");
  if (source->allocation == destination->allocation && source->offset < destination->offset + destination->length &&
      destination->offset < source->offset + source->length)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "CUDA batch copy ranges overlap");
  OwnedRecord record;
  record.name = "copy";
  record.is_copy = true;
  record.buffers = {source, destination};
  retain_buffer(source);
  retain_buffer(destination);
  batch->pending.push_back(std::move(record));
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_batch_barrier(llmopt_cuda_batch* batch) { return require_active(batch); }

static int flush_batch(llmopt_cuda_batch* batch, bool wait) {
  if (int status = require_active(batch)) return status;
  Context* context = batch->library->context;
  int status = LLMOPT_CUDA_OK;
  for (OwnedRecord& record : batch->pending) {
    status = run_record(context, record, nullptr, nullptr);
    if (status != LLMOPT_CUDA_OK) break;
  }
  if (status == LLMOPT_CUDA_OK && wait) status = wait_stream(context, "CUDA batch failed");
  if (status != LLMOPT_CUDA_OK || wait) {
    if (status != LLMOPT_CUDA_OK) cudaStreamSynchronize(context->stream);
    for (OwnedRecord& record : batch->pending) release_record(record);
    batch->pending.clear();
  }
  batch->finished = true;
  return status;
}

int llmopt_cuda_commit_batch(llmopt_cuda_batch* batch) { return flush_batch(batch, true); }
int llmopt_cuda_commit_batch_async(llmopt_cuda_batch* batch) { return flush_batch(batch, false); }

int llmopt_cuda_abort_batch(llmopt_cuda_batch* batch) {
  if (batch == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA batch has been finalized");
  if (!batch->finished) {
    for (OwnedRecord& record : batch->pending) release_record(record);
    batch->pending.clear();
    batch->finished = true;
  }
  return LLMOPT_CUDA_OK;
}

void llmopt_cuda_release_batch(llmopt_cuda_batch* batch) {
  if (batch == nullptr) return;
  if (!batch->pending.empty()) {
    // an async commit keeps its buffers until the stream has drained
    cudaStreamSynchronize(batch->library->context->stream);
    for (OwnedRecord& record : batch->pending) release_record(record);
  }
  llmopt_cuda_release_library(batch->library);
  delete batch;
}

int llmopt_cuda_synchronize(llmopt_cuda_context* context) {
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  return wait_stream(context, "CUDA synchronize failed");
}

// ---- prebaked ------------------------------------------------------------------------------

void llmopt_cuda_release_prebaked(llmopt_cuda_prebaked* plan) {
  if (plan == nullptr) return;
  if (plan->context) {
    cudaSetDevice(plan->context->device);
    cudaStreamSynchronize(plan->context->stream);
  }
  if (plan->executable) cudaGraphExecDestroy(plan->executable);
  if (plan->graph) cudaGraphDestroy(plan->graph);
  if (plan->cells) cudaFree(plan->cells);
  if (plan->chained_tokens) cudaFree(plan->chained_tokens);
  if (plan->staging) cudaFreeHost(plan->staging);
  if (plan->result_host) cudaFreeHost(plan->result_host);
  for (OwnedRecord& record : plan->records) release_record(record);
  if (plan->token_buffer) llmopt_cuda_release_buffer(plan->token_buffer);
  if (plan->output_buffer) llmopt_cuda_release_buffer(plan->output_buffer);
  for (llmopt_cuda_buffer* buffer : plan->binding_buffers) llmopt_cuda_release_buffer(buffer);
  if (plan->context) release(plan->context);
  delete plan;
}

int llmopt_cuda_prebaked_create_bound(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* records,
                                      size_t count, llmopt_cuda_buffer* token_buffer,
                                      llmopt_cuda_buffer* output_buffer, const llmopt_cuda_row_binding* bindings,
                                      size_t binding_count, llmopt_cuda_prebaked** out) {
  if (library == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA library has been finalized");
  if (out == nullptr || (records == nullptr && count > 0))
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null pointer argument");
  if (binding_count > 8) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "a plan takes at most 8 row bindings");
  if (token_buffer && token_buffer->length < 8)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "token buffer is shorter than one int64");
  if (output_buffer && output_buffer->length < 4)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "output buffer is shorter than one int32");
  Context* context = library->context;
  llmopt_cuda_prebaked* plan = new llmopt_cuda_prebaked();
  plan->context = context;
  retain(context);
  plan->records.resize(count);
  for (size_t i = 0; i < count; ++i)
    if (int status = own_record(library, &records[i], &plan->records[i])) {
      llmopt_cuda_release_prebaked(plan);
      return status;
    }
  if (token_buffer) {
    plan->token_buffer = token_buffer;
    retain_buffer(token_buffer);
  }
  if (output_buffer) {
    plan->output_buffer = output_buffer;
    retain_buffer(output_buffer);
  }
  RowBindings device_bindings = {};
  for (size_t i = 0; i < binding_count; ++i) {
    const llmopt_cuda_row_binding& binding = bindings[i];
    if (binding.destination == nullptr || binding.table == nullptr || binding.row_bytes == 0 ||
        binding.destination->length < binding.row_bytes || binding.table->length < binding.row_bytes) {
      llmopt_cuda_release_prebaked(plan);
      return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "row binding is inconsistent");
    }
    retain_buffer(binding.destination);
    retain_buffer(binding.table);
    plan->binding_buffers.push_back(binding.destination);
    plan->binding_buffers.push_back(binding.table);
    device_bindings.item[i] = {binding.destination->pointer(), binding.table->pointer(), (uint32_t)binding.row_bytes};
  }
  device_bindings.count = (int)binding_count;
  plan->token_capacity = plan_token_capacity(plan->records, bindings, binding_count);

  cudaError_t status = cudaMalloc((void**)&plan->cells, sizeof(PlanCells));
  if (status == cudaSuccess) status = cudaMemset(plan->cells, 0, sizeof(PlanCells));
  if (status == cudaSuccess)
    status = cudaHostAlloc((void**)&plan->staging, sizeof(PlanCells) * llmopt_cuda_prebaked::kStaging, cudaHostAllocDefault);
  if (status == cudaSuccess) status = cudaHostAlloc((void**)&plan->result_host, sizeof(int), cudaHostAllocDefault);
  if (status != cudaSuccess) {
    llmopt_cuda_release_prebaked(plan);
    return cuda_failure("prebaked plan allocation failed", status);
  }
  *plan->result_host = 0;

  // Relaxed mode: a launcher may grow the context scratch (cudaMalloc) while the
  // stream is capturing; scratch blocks are never freed before the context.
  status = cudaStreamBeginCapture(context->stream, cudaStreamCaptureModeRelaxed);
  if (status != cudaSuccess) {
    llmopt_cuda_release_prebaked(plan);
    return cuda_failure("CUDA graph capture could not start", status);
  }
  plan_prologue_kernel<<<binding_count ? 4 : 1, 128, 0, context->stream>>>(
      plan->cells, plan->token_buffer ? (long long*)plan->token_buffer->pointer() : nullptr, device_bindings);
  int failure = LLMOPT_CUDA_OK;
  const bool fold = getenv("LLMOPT_CUDA_FOLD_NORMS") == nullptr || getenv("LLMOPT_CUDA_FOLD_NORMS")[0] != '0';
  const bool fuse_pack = getenv("LLMOPT_CUDA_FUSE_ROTARY_PACK") == nullptr || getenv("LLMOPT_CUDA_FUSE_ROTARY_PACK")[0] != '0';
  const bool fuse_attention = fuse_pack && (getenv("LLMOPT_CUDA_FUSE_ROTARY_ATTENTION") == nullptr ||
                                            getenv("LLMOPT_CUDA_FUSE_ROTARY_ATTENTION")[0] != '0');
  for (size_t index = 0; index < plan->records.size(); ++index) {
    FusedNorm fused;
    if (fuse_attention && index + 2 < plan->records.size()) {
      const int fused_status =
          run_rotary_pack_attention(context, plan->records[index], plan->records[index + 1], plan->records[index + 2],
                                    &plan->cells->past_tokens, &plan->cells->checkpoint);
      if (fused_status >= 0) {
        failure = fused_status;
        index += 2;
        if (failure != LLMOPT_CUDA_OK) break;
        continue;
      }
    }
    if (fuse_pack && index + 1 < plan->records.size()) {
      const int fused_status = run_rotary_pack(context, plan->records[index], plan->records[index + 1]);
      if (fused_status >= 0) {
        failure = fused_status;
        ++index;
        if (failure != LLMOPT_CUDA_OK) break;
        continue;
      }
    }
    if (fold && index + 1 < plan->records.size() && fold_norm(plan->records[index], plan->records[index + 1], &fused)) {
      failure = run_record(context, plan->records[index + 1], &plan->cells->past_tokens, &plan->cells->checkpoint, &fused);
      ++index;
      plan->folded_norms += 1;
    } else {
      failure = run_record(context, plan->records[index], &plan->cells->past_tokens, &plan->cells->checkpoint);
    }
    if (failure != LLMOPT_CUDA_OK) break;
  }
  if (failure == LLMOPT_CUDA_OK && plan->output_buffer) {
    status = cudaMemcpyAsync(plan->result_host, plan->output_buffer->pointer(), sizeof(int), cudaMemcpyDeviceToHost,
                             context->stream);
    if (status != cudaSuccess) failure = cuda_failure("prebaked readback could not be captured", status);
  }
  cudaGraph_t graph = nullptr;
  status = cudaStreamEndCapture(context->stream, &graph);
  if (failure != LLMOPT_CUDA_OK) {
    if (graph) cudaGraphDestroy(graph);
    const std::string message = g_last_error;
    llmopt_cuda_release_prebaked(plan);
    return set_error(failure, message);
  }
  if (status != cudaSuccess) {
    llmopt_cuda_release_prebaked(plan);
    return cuda_failure("CUDA graph capture failed", status);
  }
  plan->graph = graph;
  size_t nodes = 0;
  cudaGraphGetNodes(graph, nullptr, &nodes);
  std::vector<cudaGraphNode_t> node_list(nodes);
  if (nodes) cudaGraphGetNodes(graph, node_list.data(), &nodes);
  for (cudaGraphNode_t node : node_list) {
    cudaGraphNodeType type;
    if (cudaGraphNodeGetType(node, &type) == cudaSuccess && type == cudaGraphNodeTypeKernel) plan->kernel_nodes += 1;
  }
  status = cudaGraphInstantiate(&plan->executable, graph, 0);
  if (status != cudaSuccess) {
    llmopt_cuda_release_prebaked(plan);
    return cuda_failure("CUDA graph instantiation failed", status);
  }
  *out = plan;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_prebaked_create(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* records,
                                size_t count, llmopt_cuda_buffer* token_buffer, llmopt_cuda_buffer* output_buffer,
                                llmopt_cuda_prebaked** out) {
  return llmopt_cuda_prebaked_create_bound(library, records, count, token_buffer, output_buffer, nullptr, 0, out);
}

static int check_plan_tokens(llmopt_cuda_prebaked* plan, int64_t last_past_tokens) {
  if (last_past_tokens > plan->token_capacity)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT,
                     "past_tokens " + std::to_string(last_past_tokens) + " exceeds the plan's token capacity " +
                         std::to_string(plan->token_capacity) + " (row-binding tables and slot tables it captured)");
  return LLMOPT_CUDA_OK;
}

static int publish_cells(llmopt_cuda_prebaked* plan, int64_t token, int32_t past_tokens, int32_t checkpoint) {
  PlanCells* slot = &plan->staging[plan->staging_next];
  plan->staging_next = (plan->staging_next + 1) % llmopt_cuda_prebaked::kStaging;
  slot->token = token;
  slot->past_tokens = (uint32_t)past_tokens;
  slot->checkpoint = (uint32_t)checkpoint;
  CUDA_TRY(cudaMemcpyAsync(plan->cells, slot, sizeof(PlanCells), cudaMemcpyHostToDevice, plan->context->stream),
           "prebaked uniform upload failed");
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_prebaked_execute(llmopt_cuda_prebaked* plan, int64_t token, int32_t past_tokens,
                                 int32_t checkpoint, int32_t* next_token) {
  if (plan == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "prebaked plan has been finalized");
  if (past_tokens < 0 || checkpoint < 0) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "negative plan uniform");
  if (int status = check_plan_tokens(plan, past_tokens)) return status;
  if (int status = publish_cells(plan, token, past_tokens, checkpoint)) return status;
  CUDA_TRY(cudaGraphLaunch(plan->executable, plan->context->stream), "Prebaked CUDA batch failed");
  if (int status = wait_stream(plan->context, "Prebaked CUDA batch failed")) return status;
  if (next_token) *next_token = plan->output_buffer ? *plan->result_host : 0;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_prebaked_execute_chained(llmopt_cuda_prebaked* plan, int64_t first_token, int32_t past_tokens,
                                         int32_t checkpoint, int32_t steps, int32_t* tokens_out,
                                         float* elapsed_ms) {
  if (plan == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "prebaked plan has been finalized");
  if (steps <= 0 || tokens_out == nullptr || plan->output_buffer == nullptr)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "chained execution needs steps > 0, a result array and an output buffer");
  if (past_tokens < 0 || checkpoint < 0) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "negative plan uniform");
  if (int status = check_plan_tokens(plan, (int64_t)past_tokens + steps - 1)) return status;
  Context* context = plan->context;
  if (plan->chained_capacity < steps) {
    if (plan->chained_tokens) {
      cudaStreamSynchronize(context->stream);
      cudaFree(plan->chained_tokens);
      plan->chained_tokens = nullptr;
    }
    CUDA_TRY(cudaMalloc((void**)&plan->chained_tokens, sizeof(int) * (size_t)steps), "chained token array allocation failed");
    plan->chained_capacity = steps;
  }
  if (int status = publish_cells(plan, first_token, past_tokens, checkpoint)) return status;
  cudaEvent_t begin = nullptr, end = nullptr;
  if (elapsed_ms) {
    CUDA_TRY(cudaEventCreate(&begin), "cudaEventCreate failed");
    CUDA_TRY(cudaEventCreate(&end), "cudaEventCreate failed");
    CUDA_TRY(cudaEventRecord(begin, context->stream), "cudaEventRecord failed");
  }
  for (int step = 0; step < steps; ++step) {
    CUDA_TRY(cudaGraphLaunch(plan->executable, context->stream), "Prebaked CUDA batch failed");
    plan_advance_kernel<<<1, 32, 0, context->stream>>>(plan->cells, (const int*)plan->output_buffer->pointer(),
                                                       plan->chained_tokens, step);
  }
  if (elapsed_ms) CUDA_TRY(cudaEventRecord(end, context->stream), "cudaEventRecord failed");
  CUDA_TRY(cudaMemcpyAsync(tokens_out, plan->chained_tokens, sizeof(int) * (size_t)steps, cudaMemcpyDeviceToHost,
                           context->stream),
           "chained token readback failed");
  int status = wait_stream(context, "Prebaked CUDA batch failed");
  if (elapsed_ms) {
    if (status == LLMOPT_CUDA_OK) cudaEventElapsedTime(elapsed_ms, begin, end);
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
  }
  return status;
}

int llmopt_cuda_prebaked_kernel_count(llmopt_cuda_prebaked* plan) { return plan ? plan->kernel_nodes : 0; }

int64_t llmopt_cuda_prebaked_token_capacity(llmopt_cuda_prebaked* plan) { return plan ? plan->token_capacity : 0; }

// ---- ring ------------------------------------------------------------------------------------

static void ring_worker(llmopt_cuda_ring* ring) {
  cudaSetDevice(ring->plan->context->device);
  for (;;) {
    RingEntry entry;
    {
      std::unique_lock<std::mutex> lock(ring->mutex);
      ring->submitted.wait(lock, [&] { return !ring->submissions.empty() || ring->stopping; });
      if (ring->submissions.empty()) return;
      entry = ring->submissions.front();
      ring->submissions.pop_front();
    }
    if (entry.flags == 2) return;  // stop request, native/ocaml_metal_stubs.m:1540-1546
    int32_t token = 0;
    const int status = llmopt_cuda_prebaked_execute(ring->plan, entry.token, entry.past_tokens, 0, &token);
    {
      std::lock_guard<std::mutex> lock(ring->mutex);
      ring->completions.push_back({entry.request_id, token, status == LLMOPT_CUDA_OK ? 0 : 1});
    }
    ring->completed.notify_all();
  }
}

int llmopt_cuda_ring_create(llmopt_cuda_ring** out) {
  if (out == nullptr) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "null result pointer");
  *out = new llmopt_cuda_ring();
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_ring_start_worker(llmopt_cuda_ring* ring, llmopt_cuda_library* library,
                                  const llmopt_cuda_dispatch_record* records, size_t count,
                                  llmopt_cuda_buffer* token_buffer, llmopt_cuda_buffer* output_buffer) {
  if (ring == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "ring queue has been destroyed");
  if (ring->started) return set_error(LLMOPT_CUDA_FAILURE, "ring worker is already running");
  if (int status = llmopt_cuda_prebaked_create(library, records, count, token_buffer, output_buffer, &ring->plan))
    return status;
  ring->started = true;
  ring->worker = std::thread(ring_worker, ring);
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_ring_submit(llmopt_cuda_ring* ring, int64_t request_id, int64_t token, int32_t past_tokens,
                            int32_t flags, int* accepted) {
  if (ring == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "ring queue has been destroyed");
  {
    std::lock_guard<std::mutex> lock(ring->mutex);
    if (ring->submissions.size() >= llmopt_cuda_ring::kCapacity) {
      if (accepted) *accepted = 0;
      return LLMOPT_CUDA_OK;
    }
    ring->submissions.push_back({request_id, token, past_tokens, flags});
  }
  ring->submitted.notify_one();
  if (accepted) *accepted = 1;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_ring_wait_completion(llmopt_cuda_ring* ring, int64_t* request_id, int32_t* token, int32_t* status) {
  if (ring == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "ring queue has been destroyed");
  std::unique_lock<std::mutex> lock(ring->mutex);
  if (!ring->started && ring->completions.empty())
    return set_error(LLMOPT_CUDA_FAILURE, "ring worker is not running");
  ring->completed.wait(lock, [&] { return !ring->completions.empty(); });
  const RingCompletion completion = ring->completions.front();
  ring->completions.pop_front();
  if (request_id) *request_id = completion.request_id;
  if (token) *token = completion.token;
  if (status) *status = completion.status;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_ring_poll_completion(llmopt_cuda_ring* ring, int* available, int64_t* request_id, int32_t* token,
                                     int32_t* status) {
  if (ring == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "ring queue has been destroyed");
  std::lock_guard<std::mutex> lock(ring->mutex);
  if (ring->completions.empty()) {
    if (available) *available = 0;
    return LLMOPT_CUDA_OK;
  }
  const RingCompletion completion = ring->completions.front();
  ring->completions.pop_front();
  if (available) *available = 1;
  if (request_id) *request_id = completion.request_id;
  if (token) *token = completion.token;
  if (status) *status = completion.status;
  return LLMOPT_CUDA_OK;
}

int llmopt_cuda_ring_destroy(llmopt_cuda_ring* ring) {
  if (ring == nullptr) return LLMOPT_CUDA_OK;
  if (ring->started) {
    {
      std::lock_guard<std::mutex> lock(ring->mutex);
      ring->stopping = true;
      ring->submissions.push_back({0, 0, 0, 2});
    }
    ring->submitted.notify_all();
    if (ring->worker.joinable()) ring->worker.join();
  }
  if (ring->plan) llmopt_cuda_release_prebaked(ring->plan);
  delete ring;
  return LLMOPT_CUDA_OK;
}

// ---- helpers -----------------------------------------------------------------------------------

int64_t llmopt_cuda_f16_argmax(const void* halves, size_t count) {
  if (halves == nullptr || count == 0) return 0;
  const __half* values = (const __half*)halves;
  float best = __half2float(values[0]);
  size_t index = 0;
  for (size_t i = 1; i < count; ++i) {
    const float value = __half2float(values[i]);
    if (value > best) {
      best = value;
      index = i;
    }
  }
  return (int64_t)index;
}

int llmopt_cuda_w4a16_linear(llmopt_cuda_context* context, const void* input, const void* packed_weight,
                             const void* scale, const void* bias, void* output, int64_t m, int64_t n, int64_t k,
                             void* stream) {
  if (context == nullptr) return set_error(LLMOPT_CUDA_FAILURE, "CUDA context has been finalized");
  // the checks of native/metal_runtime.cpp:58-110
  if (m <= 0 || n <= 0 || k <= 0) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "w4a16_linear dimensions must be positive");
  if (k % 64 != 0) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "w4a16_linear K must be a multiple of 64");
  if (!input || !packed_weight || !scale || !output)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "w4a16_linear received a null tensor");
  uint32_t params[5] = {(uint32_t)m, (uint32_t)n, (uint32_t)k, bias ? 1u : 0u, 0u};
  KernelArgs args = {};
  args.ctx = context;
  args.stream = stream ? (cudaStream_t)stream : context->stream;
  args.buffer_count = 5;
  args.buffers[0] = (void*)input;
  args.lengths[0] = (size_t)m * k * 2;
  args.buffers[1] = (void*)packed_weight;
  args.lengths[1] = (size_t)n * (k / 2);
  args.buffers[2] = (void*)scale;
  args.lengths[2] = (size_t)n * (k / 64) * 2;
  args.buffers[3] = (void*)(bias ? bias : scale);
  args.lengths[3] = bias ? (size_t)n * 2 : args.lengths[2];
  args.buffers[4] = output;
  args.lengths[4] = (size_t)m * n * 2;
  args.params = (const uint8_t*)params;
  args.param_bytes = sizeof(params);
  args.name = "llmopt_w4a16_linear_f16_g64";
  std::string message;
  args.error = &message;
  if (launch_w4a16_linear(args) != 0) return set_error(LLMOPT_CUDA_FAILURE, message);
  return LLMOPT_CUDA_OK;
}

namespace llmopt {
__global__ void flush_kernel(uint4* buffer, size_t count, uint32_t seed) {
  grid_chain_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    buffer[i] = make_uint4(seed, seed + 1, seed + 2, seed + 3);
}
}  // namespace llmopt

int llmopt_cuda_time_dispatch(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* record, int warmup,
                              int iterations, int flush_l2, float* average_ms) {
  if (average_ms == nullptr || iterations <= 0) return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "bad timing request");
  OwnedRecord owned;
  if (int status = own_record(library, record, &owned)) return status;
  Context* context = library->context;
  if (flush_l2 && context->flush_buffer == nullptr) {
    context->flush_bytes = (size_t)256 << 20;  // larger than the 126 MB L2
    cudaError_t status = cudaMalloc(&context->flush_buffer, context->flush_bytes);
    if (status != cudaSuccess) {
      release_record(owned);
      return cuda_failure("flush buffer allocation failed", status);
    }
  }
  cudaEvent_t begin, end;
  cudaEventCreate(&begin);
  cudaEventCreate(&end);
  int status = LLMOPT_CUDA_OK;
  double total = 0.0;
  for (int i = 0; i < warmup + iterations && status == LLMOPT_CUDA_OK; ++i) {
    if (flush_l2)
      flush_kernel<<<context->sm_count * 4, 256, 0, context->stream>>>((uint4*)context->flush_buffer,
                                                                         context->flush_bytes / 16, (uint32_t)i);
    cudaEventRecord(begin, context->stream);
    status = run_record(context, owned, nullptr, nullptr);
    cudaEventRecord(end, context->stream);
    if (status == LLMOPT_CUDA_OK) status = wait_stream(context, "timed dispatch failed");
    if (status == LLMOPT_CUDA_OK && i >= warmup) {
      float elapsed = 0.0f;
      cudaEventElapsedTime(&elapsed, begin, end);
      total += elapsed;
    }
  }
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  release_record(owned);
  if (status == LLMOPT_CUDA_OK) *average_ms = (float)(total / iterations);
  return status;
}

int llmopt_cuda_time_dispatches(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* records,
                                size_t count, int warmup, int iterations, float* average_ms_per_dispatch) {
  if (average_ms_per_dispatch == nullptr || iterations <= 0 || count == 0 || records == nullptr)
    return set_error(LLMOPT_CUDA_INVALID_ARGUMENT, "bad timing request");
  std::vector<OwnedRecord> owned(count);
  for (size_t i = 0; i < count; ++i)
    if (int status = own_record(library, &records[i], &owned[i])) {
      for (size_t j = 0; j < i; ++j) release_record(owned[j]);
      return status;
    }
  Context* context = library->context;
  cudaEvent_t begin, end;
  cudaEventCreate(&begin);
  cudaEventCreate(&end);
  int status = LLMOPT_CUDA_OK;
  double total = 0.0;
  for (int i = 0; i < warmup + iterations && status == LLMOPT_CUDA_OK; ++i) {
    cudaEventRecord(begin, context->stream);
    for (size_t j = 0; j < count && status == LLMOPT_CUDA_OK; ++j) status = run_record(context, owned[j], nullptr, nullptr);
    cudaEventRecord(end, context->stream);
    if (status == LLMOPT_CUDA_OK) status = wait_stream(context, "timed dispatches failed");
    if (status == LLMOPT_CUDA_OK && i >= warmup) {
      float elapsed = 0.0f;
      cudaEventElapsedTime(&elapsed, begin, end);
      total += elapsed;
    }
  }
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  for (OwnedRecord& record : owned) release_record(record);
  if (status == LLMOPT_CUDA_OK) *average_ms_per_dispatch = (float)(total / iterations / (double)count);
  return status;
}

}  // extern "C"
