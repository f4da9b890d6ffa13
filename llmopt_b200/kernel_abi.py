"""Mirror of the reference's ``Kernel_abi`` surface for the hot path
(lib/kernel_abi.ml:1-151): operation wire names and the kernel ``Entry`` record,
plus the entry table of the kernels libllmopt_cuda.so provides.  The wire
strings and entry names are the reference's; packages refer to kernels by them."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

# Kernel_abi.Operation.to_string, lib/kernel_abi.ml:36-70 (hot-path subset)
LINEAR = "linear"
GATED_LINEAR = "gated-linear"
FUSED_LINEAR = "fused-linear"
W4A16_LINEAR = "w4a16-linear-g64"
W4A16_QKV_LINEAR = "w4a16-qkv-linear-g64"
W4A16_SWIGLU_FFN = "w4a16-swiglu-ffn-g64"
W4A16_LM_HEAD_ARGMAX = "w4a16-lm-head-argmax"
RMS_NORM = "rms-norm"
RMS_ROPE = "rms-rope"
RMS_ROPE_QK = "rms-rope-qk"
ROTARY_QK = "rotary-qk"
CAST = "cast"
POINTWISE = "pointwise"
GATED_DELTA = "gated-delta"
TRIANGULAR_RECURRENCE = "triangular-recurrence"
SHORT_CONV = "short-conv"
SHORT_CONV_STEP = "short-conv-step"
SHORT_CONV_PREFILL = "short-conv-prefill"
ATTENTION = "attention"
EMBEDDING = "embedding"
CACHE = "cache"

OPERATIONS = (
    LINEAR, GATED_LINEAR, FUSED_LINEAR, W4A16_LINEAR, W4A16_QKV_LINEAR, W4A16_SWIGLU_FFN, W4A16_LM_HEAD_ARGMAX, RMS_NORM, ROTARY_QK, SHORT_CONV,
    SHORT_CONV_STEP, SHORT_CONV_PREFILL, ATTENTION, EMBEDDING, CACHE, RMS_ROPE, RMS_ROPE_QK, CAST, POINTWISE,
    GATED_DELTA, TRIANGULAR_RECURRENCE,
)


@dataclass(frozen=True)
class Entry:
    """``Kernel_abi.Entry.t`` (lib/kernel_abi.ml:110-118)."""

    name: str
    operation: str
    input_dtype: str
    output_dtype: str
    threadgroup: tuple = (256, 1, 1)
    tile: Optional[tuple] = None

    def __post_init__(self):
        # Entry.make, lib/kernel_abi.ml:120-133
        if not self.name.strip():
            raise ValueError("kernel entry-point name cannot be empty")
        if any(v <= 0 for v in self.threadgroup):
            raise ValueError("kernel threadgroup dimensions must be positive")
        if self.tile is not None and (any(v <= 0 for v in self.tile) or self.tile[2] % 4 != 0):
            raise ValueError("kernel tile dimensions must be positive and tile_k must be divisible by four")


def _entries() -> list[Entry]:
    f16, f32, u8, i64 = "float16", "float32", "uint8", "int64"
    table = []

    def add(name, operation, input_dtype=f16, output_dtype=f16, threadgroup=(256, 1, 1)):
        table.append(Entry(name, operation, input_dtype, output_dtype, threadgroup))

    for suffix in ("", "_m4", "_m8"):  # lib/metal_w4a16_source.ml:196-208
        add("llmopt_w4a16_linear_f16_g64" + suffix, W4A16_LINEAR)
        add("llmopt_w4a16_qkv_linear_f16_g64" + suffix, W4A16_QKV_LINEAR)
        add("llmopt_w4a16_dual_swiglu_f16_g64" + suffix, W4A16_SWIGLU_FFN)
        add("llmopt_w4a16_down_add_f16_g64" + suffix, W4A16_SWIGLU_FFN)
    add("llmopt_w4a16_linear_f16_g64_affine", W4A16_LINEAR)
    # Q4_0-block family: input dtype is the quantised storage (Ir.Dtype.Quant Q4_0)
    add("llmopt_dequant_q4_0", LINEAR, "q4_0", f16, threadgroup=(256, 1, 1))
    for tactic in ("", "_x4", "_x8", "_x16", "_m2", "_m4", "_m16", "_m32", "_simd"):
        add("llmopt_q4_0_linear_f16" + tactic, LINEAR, "q4_0", f16)
        add("llmopt_q4_0_linear_f16" + tactic + "_add", LINEAR, "q4_0", f16)
    for tactic in ("", "_x8", "_x16", "_m4", "_m16", "_m32"):
        add("llmopt_q4_0_qkv_linear_f16" + tactic, FUSED_LINEAR, "q4_0", f16)
    for tactic in ("_x8", "_m4", "_m16", "_m32"):
        add("llmopt_q4_0_gated_linear_f16" + tactic, GATED_LINEAR, "q4_0", f16)
    for bits in (4, 8):  # lib/metal_block_codegen.ml:144-722; input dtype is the quantised storage
        for tactic in ("_x8", "_m16", "_m32", "_simd", "_m16_add", "_m32_add"):
            add(f"llmopt_tile32_affine{bits}_linear_f16{tactic}", LINEAR, f"tile32_affine{bits}", f16)
        add(f"llmopt_cache_pack_attention_tile32_affine{bits}_fwht_simd", CACHE, f16, f"tile32_affine{bits}")
        add(f"llmopt_cache_unpack_attention_tile32_affine{bits}_fwht_simd", CACHE, f"tile32_affine{bits}", f16)
    add("llmopt_w4a16_swiglu_rms_f16_g64", W4A16_SWIGLU_FFN)
    add("llmopt_w4a16_swiglu_rms_f32_g64", W4A16_SWIGLU_FFN, f32, f16)
    for stem in ("llmopt_w4a16_lm_head_argmax", "llmopt_w4a16_lm_head_argmax_extra",
                 "llmopt_w4a16_lm_head_argmax_stage1", "llmopt_w4a16_lm_head_argmax_stage1_extra"):
        add(stem + "_f16", W4A16_LM_HEAD_ARGMAX, f16, "int32")
        add(stem + "_f32", W4A16_LM_HEAD_ARGMAX, f32, "int32")
    add("llmopt_w4a16_lm_head_reduce", W4A16_LM_HEAD_ARGMAX, "int32", "int32")
    for name in ("llmopt_cache_pack_attention_q8", "llmopt_cache_pack_attention_q8_simd",
                 "llmopt_cache_pack_attention_q8_pair_simd", "llmopt_cache_pack_checkpoint_q8",
                 "llmopt_cache_pack_checkpoint_q8_simd"):
        add(name, CACHE, f16, u8)
    for name in ("llmopt_cache_unpack_attention_q8", "llmopt_cache_unpack_attention_q8_vec4",
                 "llmopt_cache_unpack_checkpoint_q8", "llmopt_cache_unpack_checkpoint_q8_vec4"):
        add(name, CACHE, u8, f16)
    for name in ("llmopt_attention_q8_paged_simd_h64", "llmopt_attention_q8_paged_simd_generic",
                 "llmopt_attention_q8_paged_simd_h64_gqa3", "llmopt_attention_q8_paged_simd_h64_split8",
                 "llmopt_attention_q8_paged_simd_h64_gqa3_split8", "llmopt_attention_q8_paged_batched"):
        add(name, ATTENTION)
    for name in ("llmopt_attention_f16", "llmopt_attention_f16_simd_h32", "llmopt_attention_f16_simd_h64",
                 "llmopt_attention_f16_simd_h80", "llmopt_attention_f16_simd_h96", "llmopt_attention_f16_simd_h128",
                 "llmopt_attention_f16_simd_h256"):
        add(name, ATTENTION, threadgroup=(128, 1, 1) if "simd" in name else (1, 1, 1))
    add("llmopt_attention_q8_paged_simd_h256", ATTENTION, threadgroup=(32, 1, 1))
    add("llmopt_attention_q8_paged_simd_h512", ATTENTION, threadgroup=(32, 1, 1))
    add("llmopt_short_conv_f16", SHORT_CONV)
    add("llmopt_short_conv_f16_f32", SHORT_CONV, f32, f16)
    add("llmopt_short_conv_silu_tm_f16", SHORT_CONV)
    add("llmopt_short_conv_silu_tm_f32", SHORT_CONV, f32, f16)
    add("llmopt_short_conv_step_f16", SHORT_CONV_STEP)
    add("llmopt_short_conv_step_fused_f16", SHORT_CONV_STEP)
    add("llmopt_short_conv_prefill_f16", SHORT_CONV_PREFILL)
    add("llmopt_short_conv_prefill_init_f16", SHORT_CONV_PREFILL)
    add("llmopt_rms_norm_f16", RMS_NORM)
    add("llmopt_rms_norm_f16_simd", RMS_NORM)
    add("llmopt_rms_norm_f32_f16", RMS_NORM, f32, f16)
    add("llmopt_rms_norm_f32_f16_simd", RMS_NORM, f32, f16)
    # lib/metal_normalization_source.ml:449-516 (entries of the norm variants), :586-590, :660-668, :737-757
    for name in ("llmopt_rms_norm_f16_wf32_simd", "llmopt_rms_norm_f16_wf32_wide", "llmopt_rms_norm_add_f16_wf32_simd",
                 "llmopt_rms_norm_add_f16_wf32_wide", "llmopt_rms_norm_scale_f16_wf32_simd",
                 "llmopt_rms_norm_scale_f16_wf32_wide", "llmopt_rms_norm_add_scale_f16_wf32_simd",
                 "llmopt_rms_norm_add_scale_f16_wf32_wide", "llmopt_rms_norm_unweighted_f16_simd",
                 "llmopt_rms_norm_unweighted_f16_wide", "llmopt_rms_norm_unweighted_add_f16_simd",
                 "llmopt_rms_norm_unweighted_add_f16_wide", "llmopt_l2_norm_f16_simd", "llmopt_l2_norm_slice_f16_simd"):
        add(name, RMS_NORM)
    add("llmopt_rms_norm_f32_f16_wf32_simd", RMS_NORM, f32, f16)
    add("llmopt_rms_rope_f16_simd_h64", RMS_ROPE)
    add("llmopt_rms_rope_f16_wf32_simd", RMS_ROPE)
    add("llmopt_rms_rope_qk_f16_simd_h64", RMS_ROPE_QK)
    add("llmopt_rms_rope_qk_f16_wf32_simd", RMS_ROPE_QK)
    add("llmopt_cast_f16_f32", CAST, f16, f32)   # lib/metal_tensor_source.ml:928-938
    add("llmopt_cast_f32_f16", CAST, f32, f16)
    add("llmopt_cast_i64_f32", CAST, i64, f32)
    for name in ("llmopt_add_f16", "llmopt_mul_f16", "llmopt_div_f16", "llmopt_silu_mul_f16", "llmopt_gelu_mul_f16",
                 "llmopt_sigmoid_mul_f16", "llmopt_neg_f16", "llmopt_silu_f16", "llmopt_sigmoid_f16", "llmopt_tanh_f16",
                 "llmopt_rsqrt_f16", "llmopt_mul_f32_f16_f16"):
        add(name, POINTWISE)
    for name in ("llmopt_add_f32", "llmopt_sub_f32", "llmopt_mul_f32", "llmopt_neg_f32", "llmopt_silu_f32",
                 "llmopt_exp_f32", "llmopt_rsqrt_f32", "llmopt_cos_f32", "llmopt_sin_f32", "llmopt_softplus_f32"):
        add(name, POINTWISE, f32, f32)
    add("llmopt_mul_f16_f32", POINTWISE, f16, f32)
    add("llmopt_mul_f16_f32_f16", POINTWISE, f16, f16)
    add("llmopt_rotary_qk_f16_simd_h64", ROTARY_QK)
    for width in range(32, 257, 32):  # lib/metal_recurrent_source.ml:309-327, 400-410
        add(f"llmopt_gated_delta_f32_d{width}", GATED_DELTA, f32, f16, threadgroup=(128, 1, 1))
        add(f"llmopt_gated_delta_tm_f16_d{width}", GATED_DELTA, f16, f16, threadgroup=(128, 1, 1))
    add("llmopt_triangular_recurrence_f32", TRIANGULAR_RECURRENCE, f32, f32, threadgroup=(64, 1, 1))
    add("llmopt_embedding_f16", EMBEDDING, i64, f16)
    add("llmopt_chain_token_id", EMBEDDING, i64, i64, (32, 1, 1))
    add("llmopt_chain_token_ids", EMBEDDING, "int32", i64, (128, 1, 1))
    return table


ENTRIES: tuple = tuple(_entries())


def find_entry(*, operation: str, input_dtype: str, output_dtype: str, name: Optional[str] = None) -> Entry:
    """``Metal_native.kernel_entry`` lookup rule (lib/metal_native.ml:461-487):
    exactly one entry must match the operation, both dtypes and, if given, the name."""
    if operation not in OPERATIONS:
        raise ValueError(f"unsupported kernel operation: {operation}")
    matches = [e for e in ENTRIES if e.operation == operation and e.input_dtype == input_dtype
               and e.output_dtype == output_dtype and (name is None or e.name == name)]
    if not matches:
        raise LookupError(f"package declares no kernel for operation {operation}" + (f" named {name}" if name else ""))
    if len(matches) > 1:
        raise LookupError(f"package declares multiple kernels for operation {operation}")
    return matches[0]
