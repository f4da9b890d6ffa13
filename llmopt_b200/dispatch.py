"""Host-side dispatchers: they choose the kernel NAME, the buffer ORDER, the
parameter BYTES and the Metal-style GRID exactly as the reference's
``Metal_dispatch_linear`` / ``Metal_dispatch_attention`` /
``Metal_dispatch_recurrent`` / ``Metal_cache`` modules do, and hand the record
to ``cuda_native`` (immediately, or into a batch whose ``pending`` list a
prebaked plan is built from).  Shape, dtype and guard checks and their error
strings follow the reference; ``reference_guards=False`` lifts the size guards
that exist only because of Metal threadgroup-memory limits (k <= 2048,
n <= 8192), which the CUDA kernels do not have.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

from . import kernel_abi, parameters
from .cuda_native import Batch, Buffer, Runtime
from .kv_cache import Layout


@dataclass
class Tensor:
    """A device value: buffer + logical shape + dtype name (the reference's Ir.Value
    bound to a Metal buffer in Metal_execution_state)."""

    buffer: Buffer
    shape: tuple
    dtype: str = "float16"

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


@dataclass
class ExecutionBatch:
    """Scratch kept per batch (Metal_execution_state.Execution_batch,
    lib/metal_execution_state.ml:26-49): reused when large enough."""

    swiglu_normalized: Optional[Buffer] = None
    swiglu_product: Optional[Buffer] = None
    candidates_buffer: Optional[Buffer] = None
    resources: list = field(default_factory=list)


@dataclass
class Context:
    """Metal_execution_state.context: runtime, optional command batch, scratch."""

    runtime: Runtime
    batch: Optional[Batch] = None
    execution_batch: ExecutionBatch = field(default_factory=ExecutionBatch)
    decode_uniforms_past_tokens: Optional[int] = None


class DispatchError(ValueError):
    """The reference's ``Error msg`` results from its dispatchers."""


def round_up(value: int, multiple: int) -> int:  # lib/metal_dispatch_common.ml:59-62
    return (value + multiple - 1) // multiple * multiple


def linear_f16_grid(columns: int) -> int:  # lib/metal_dispatch_common.ml:64-70
    return round_up(columns, 8) * 32


def simd_rows_grid(rows: int) -> int:
    return round_up(rows, 8) * 32


def _scratch(context: Context, field_name: str, nbytes: int) -> Buffer:
    current = getattr(context.execution_batch, field_name)
    if current is not None and current.byte_length() >= nbytes:
        return current
    buffer = Buffer.create(context.runtime, nbytes)
    setattr(context.execution_batch, field_name, buffer)
    context.execution_batch.resources.append(buffer)
    return buffer


def _run(context: Context, entry, buffers, params, grid) -> str:
    return context.runtime.dispatch(entry, buffers=buffers, parameters=params, grid=grid, batch=context.batch)


# ---- W4A16 linear family ---------------------------------------------------------------

def dispatch_w4a16_linear(context: Context, *, input: Tensor, weight: Tensor, scale: Tensor, output: Tensor,
                          bias: Optional[Tensor] = None, bias_row_stride: int = 0) -> list:
    """dispatch_w4a16_linear, lib/metal_dispatch_linear.ml:938-982. ``bias`` with
    ``bias_row_stride`` = n is the fused residual form
    (lib/metal_dispatch_assignment.ml:416-453)."""
    k = input.shape[-1]
    m = input.numel // k
    n = weight.shape[0]
    if (input.dtype != "float16" or weight.dtype != "uint8" or scale.dtype != "float16"
            or output.dtype != "float16" or (bias is not None and bias.dtype != "float16")):
        raise DispatchError("W4A16 linear expects f16 input/scale/bias/output and uint8 packed weight")
    if k % 64 != 0 or tuple(weight.shape) != (n, k // 2) or tuple(scale.shape) != (n, k // 64):
        raise DispatchError("W4A16 linear weight metadata is inconsistent")
    if output.numel != m * n:
        raise DispatchError("W4A16 linear output shape is inconsistent")
    params = parameters.w4a16_linear(m=m, n=n, k=k, has_bias=bias is not None, bias_row_stride=bias_row_stride)
    bias_buffer = bias.buffer if bias is not None else scale.buffer
    if m == 1:
        name, grid = "llmopt_w4a16_linear_f16_g64", linear_f16_grid(m * n)
    else:
        name, grid = "llmopt_w4a16_linear_f16_g64_m4", linear_f16_grid(((m + 3) // 4) * n)
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.W4A16_LINEAR, input_dtype="float16",
                                         output_dtype="float16")
    return [_run(context, entry, [input.buffer, weight.buffer, scale.buffer, bias_buffer, output.buffer], params,
                 (grid, 1, 1))]


def dispatch_w4a16_linear_affine(context: Context, *, input: Tensor, weight: Tensor, scale: Tensor, zero: Tensor,
                                 output: Tensor, bias: Optional[Tensor] = None) -> list:
    """Unsigned nibbles with fp16 zero points, w = (u - z) s: no reference dispatcher;
    the algebra is Tile32_Affine4's (lib/block_schema.ml:706-741) at group 64."""
    k = input.shape[-1]
    m = input.numel // k
    n = weight.shape[0]
    if k % 64 != 0 or tuple(weight.shape) != (n, k // 2) or tuple(scale.shape) != (n, k // 64) \
            or tuple(zero.shape) != (n, k // 64):
        raise DispatchError("W4A16 linear weight metadata is inconsistent")
    params = parameters.w4a16_linear(m=m, n=n, k=k, has_bias=bias is not None, bias_row_stride=0)
    entry = context.runtime.kernel_entry(name="llmopt_w4a16_linear_f16_g64_affine",
                                         operation=kernel_abi.W4A16_LINEAR, input_dtype="float16",
                                         output_dtype="float16")
    bias_buffer = bias.buffer if bias is not None else scale.buffer
    grid = linear_f16_grid(m * n) if m == 1 else linear_f16_grid(((m + 3) // 4) * n)  # as the contract form
    return [_run(context, entry,
                 [input.buffer, weight.buffer, scale.buffer, zero.buffer, bias_buffer, output.buffer], params,
                 (grid, 1, 1))]


def dispatch_w4a16_qkv_linear_command(context: Context, *, input: Tensor, q_weight: Tensor, q_scale: Tensor,
                                      k_weight: Tensor, k_scale: Tensor, v_weight: Tensor, v_scale: Tensor,
                                      q_output: Tensor, k_output: Tensor, v_output: Tensor) -> list:
    """dispatch_w4a16_qkv_linear_command, lib/metal_dispatch_linear.ml:398-455."""
    k = input.shape[-1]
    m = input.numel // k
    n_q, n_k, n_v = q_weight.shape[0], k_weight.shape[0], v_weight.shape[0]
    for weight, scale, n in ((q_weight, q_scale, n_q), (k_weight, k_scale, n_k), (v_weight, v_scale, n_v)):
        if tuple(weight.shape) != (n, k // 2) or tuple(scale.shape) != (n, k // 64) or k % 64 != 0:
            raise DispatchError("W4A16 QKV linear command has inconsistent inputs")
    params = parameters.w4a16_qkv_linear(m=m, k=k, n_q=n_q, n_k=n_k, n_v=n_v)
    total = n_q + n_k + n_v
    if m == 1:
        name, grid = "llmopt_w4a16_qkv_linear_f16_g64", linear_f16_grid(m * total)
    else:
        name, grid = "llmopt_w4a16_qkv_linear_f16_g64_m4", linear_f16_grid(((m + 3) // 4) * total)
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.W4A16_QKV_LINEAR, input_dtype="float16",
                                         output_dtype="float16")
    buffers = [input.buffer, q_weight.buffer, q_scale.buffer, k_weight.buffer, k_scale.buffer, v_weight.buffer,
               v_scale.buffer, q_output.buffer, k_output.buffer, v_output.buffer]
    return [_run(context, entry, buffers, params, (grid, 1, 1))]


def dispatch_w4a16_swiglu_ffn_command(context: Context, *, m: int, n: int, k: int, epsilon: float,
                                      activation: Tensor, residual: Tensor, gate_weight: Tensor,
                                      gate_scale: Tensor, up_weight: Tensor, up_scale: Tensor,
                                      down_weight: Tensor, down_scale: Tensor, norm_weight: Tensor, output: Tensor,
                                      reference_guards: bool = True) -> list:
    """dispatch_w4a16_swiglu_ffn_command, lib/metal_dispatch_linear.ml:252-396:
    rms -> dual gate/up SwiGLU -> down + residual, three launches."""
    guards_ok = (k <= 2048 and n <= 8192) or not reference_guards
    consistent = (
        math.isfinite(epsilon) and epsilon > 0.0 and m > 0 and n > 0 and k > 0 and n % 64 == 0 and k % 64 == 0
        and guards_ok and activation.dtype in ("float16", "float32") and residual.dtype == "float16"
        and gate_weight.dtype == "uint8" and gate_scale.dtype == "float16" and up_weight.dtype == "uint8"
        and up_scale.dtype == "float16" and down_weight.dtype == "uint8" and down_scale.dtype == "float16"
        and norm_weight.dtype == "float16" and output.dtype == "float16" and activation.numel == m * k
        and tuple(residual.shape) == tuple(output.shape) and output.numel == m * k
        and tuple(gate_weight.shape) == (n, k // 2) and tuple(gate_scale.shape) == (n, k // 64)
        and tuple(up_weight.shape) == (n, k // 2) and tuple(up_scale.shape) == (n, k // 64)
        and tuple(down_weight.shape) == (k, n // 2) and tuple(down_scale.shape) == (k, n // 64)
        and tuple(norm_weight.shape) == (k,))
    if not consistent:
        raise DispatchError("W4A16 SwiGLU input metadata is inconsistent")
    runtime = context.runtime
    rms_name = "llmopt_w4a16_swiglu_rms_f16_g64" if activation.dtype == "float16" else "llmopt_w4a16_swiglu_rms_f32_g64"
    rms_entry = runtime.kernel_entry(name=rms_name, operation=kernel_abi.W4A16_SWIGLU_FFN,
                                     input_dtype=activation.dtype, output_dtype="float16")
    suffix = "" if m == 1 else "_m4"
    dual_entry = runtime.kernel_entry(name="llmopt_w4a16_dual_swiglu_f16_g64" + suffix,
                                      operation=kernel_abi.W4A16_SWIGLU_FFN, input_dtype="float16",
                                      output_dtype="float16")
    down_entry = runtime.kernel_entry(name="llmopt_w4a16_down_add_f16_g64" + suffix,
                                      operation=kernel_abi.W4A16_SWIGLU_FFN, input_dtype="float16",
                                      output_dtype="float16")
    normalized = _scratch(context, "swiglu_normalized", m * k * 2)
    product = _scratch(context, "swiglu_product", m * n * 2)
    params = parameters.w4a16_swiglu_ffn(m=m, n=n, k=k, epsilon=epsilon)
    rows = m if m == 1 else (m + 3) // 4
    kernels = [
        _run(context, rms_entry, [activation.buffer, norm_weight.buffer, normalized], params, (m * 256, 1, 1)),
        _run(context, dual_entry,
             [normalized, gate_weight.buffer, gate_scale.buffer, up_weight.buffer, up_scale.buffer, product], params,
             (linear_f16_grid(rows * n), 1, 1)),
        _run(context, down_entry, [product, down_weight.buffer, down_scale.buffer, residual.buffer, output.buffer],
             params, (linear_f16_grid(rows * k), 1, 1)),
    ]
    return kernels


def dispatch_w4a16_lm_head_argmax_command(context: Context, *, m: int, n: int, k: int, epsilon: float,
                                          input: Tensor, norm_weight: Tensor, weight: Tensor, scale: Tensor,
                                          output: Tensor, logits: Optional[Tensor] = None,
                                          reference_guards: bool = True, two_stage: bool = True) -> list:
    """dispatch_w4a16_lm_head_argmax_command, lib/metal_dispatch_linear.ml:570-721:
    the two-stage form (stage 1 + reduce over 256 candidates per row) when both
    entries exist, else the single-pass kernel."""
    guards_ok = k <= 2048 or not reference_guards
    consistent = (
        math.isfinite(epsilon) and epsilon > 0.0 and m > 0 and n > 0 and k > 0 and k % 64 == 0 and guards_ok
        and input.dtype in ("float16", "float32") and norm_weight.dtype == "float16" and weight.dtype == "uint8"
        and scale.dtype == "float16" and output.dtype == "int32" and input.numel == m * k
        and tuple(norm_weight.shape) == (k,) and tuple(weight.shape) == (n, k // 2)
        and tuple(scale.shape) == (n, k // 64) and output.numel == m
        and (logits is None or (logits.dtype == "float16" and tuple(logits.shape) == (m, n))))
    if not consistent:
        raise DispatchError("W4A16 LM-head argmax input metadata is inconsistent")
    runtime = context.runtime
    suffix = "_f16" if input.dtype == "float16" else "_f32"
    extra = "_extra" if logits is not None else ""
    params = parameters.w4a16_lm_head_argmax(m=m, n=n, k=k, epsilon=epsilon)
    tail = [logits.buffer] if logits is not None else []
    if two_stage:
        entry1 = runtime.kernel_entry(name="llmopt_w4a16_lm_head_argmax_stage1" + extra + suffix,
                                      operation=kernel_abi.W4A16_LM_HEAD_ARGMAX, input_dtype=input.dtype,
                                      output_dtype="int32")
        entry2 = runtime.kernel_entry(name="llmopt_w4a16_lm_head_reduce", operation=kernel_abi.W4A16_LM_HEAD_ARGMAX,
                                      input_dtype="int32", output_dtype="int32")
        candidates = _scratch(context, "candidates_buffer", m * 256 * 8)
        return [
            _run(context, entry1, [input.buffer, norm_weight.buffer, weight.buffer, scale.buffer, candidates] + tail,
                 params, (256 * 256, m, 1)),
            _run(context, entry2, [candidates, output.buffer], parameters.u32s([m]), (m * 256, 1, 1)),
        ]
    entry = runtime.kernel_entry(name="llmopt_w4a16_lm_head_argmax" + extra + suffix,
                                 operation=kernel_abi.W4A16_LM_HEAD_ARGMAX, input_dtype=input.dtype,
                                 output_dtype="int32")
    return [_run(context, entry, [input.buffer, norm_weight.buffer, weight.buffer, scale.buffer, output.buffer] + tail,
                 params, (m * 256, 1, 1))]


# ---- attention ----------------------------------------------------------------------------

@dataclass(frozen=True)
class PagedAttentionConfig:
    """Ir.Paged_attention_q8 (lib/ir.ml:472-540)."""

    token_elements: int
    key_offset: int
    value_offset: int
    group_size: int
    token_stride: int
    scale: float
    window: Optional[int] = None


def paged_attention_kernel_name(*, split8: bool, experimental_gqa3_split8: bool, query_heads: int, kv_heads: int,
                                head_dimension: int) -> str:
    """Paged_attention_tactic.kernel_name, lib/metal_dispatch_common.ml:41-57."""
    gqa3 = head_dimension == 64 and query_heads == 3 * kv_heads
    if head_dimension == 64:
        if split8:
            return ("llmopt_attention_q8_paged_simd_h64_gqa3_split8" if gqa3 and experimental_gqa3_split8
                    else "llmopt_attention_q8_paged_simd_h64_split8")
        return "llmopt_attention_q8_paged_simd_h64_gqa3" if gqa3 else "llmopt_attention_q8_paged_simd_h64"
    if head_dimension == 256:
        return "llmopt_attention_q8_paged_simd_h256"
    if head_dimension == 512:
        return "llmopt_attention_q8_paged_simd_h512"
    return "llmopt_attention_q8_paged_simd_generic"


# ---- Q4_0-block linears --------------------------------------------------------------------

def _q4_0_weight_ok(weight: Tensor, n: int, k: int) -> bool:
    return weight.dtype == "uint8" and k % 32 == 0 and weight.numel == n * (k // 32) * 18


def dispatch_quant_linear(context: Context, *, m: int, n: int, k: int, input: Tensor, weight: Tensor,
                          output: Tensor, additive: Optional[Tensor] = None, epilogue_mode: int = 0) -> list:
    """dispatch_quant_linear for Q4_0 storage, lib/metal_dispatch_common.ml:299-420: buffers
    [input, weight, additive, output], params {m, n, k, epilogue_mode} (0 none, 1 bias, 2 residual
    add, which selects the ``_add`` entry).  The tactic is chosen by the row count like the
    reference's costed selection; every tactic computes the same values."""
    if epilogue_mode not in (0, 1, 2) or (epilogue_mode != 0) != (additive is not None):
        raise DispatchError("quantized Linear epilogue mode and additive operand are inconsistent")
    if not (m > 0 and n > 0 and input.dtype == "float16" and output.dtype == "float16" and input.numel == m * k
            and output.numel == m * n and _q4_0_weight_ok(weight, n, k)):
        raise DispatchError("quantized Linear input metadata is inconsistent")
    tactic = "" if m == 1 else "_m2" if m == 2 else "_m4" if m <= 8 else "_m16" if m <= 16 else "_m32"
    name = "llmopt_q4_0_linear_f16" + tactic + ("_add" if epilogue_mode == 2 else "")
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.LINEAR, input_dtype="q4_0",
                                         output_dtype="float16")
    extra = additive.buffer if additive is not None else input.buffer
    return [_run(context, entry, [input.buffer, weight.buffer, extra, output.buffer],
                 parameters.u32s([m, n, k, epilogue_mode]), (linear_f16_grid(m * n), 1, 1))]


def dispatch_quant_qkv_linear(context: Context, *, m: int, k: int, input: Tensor, q_weight: Tensor, k_weight: Tensor,
                              v_weight: Tensor, q_output: Tensor, k_output: Tensor, v_output: Tensor) -> list:
    """Fused Q4_0 QKV (lib/metal_quant_qkv_source.ml:17-170): 7 buffers, params {m, k, n_q, n_k, n_v}."""
    n_q, n_k, n_v = q_output.numel // m, k_output.numel // m, v_output.numel // m
    if not (m > 0 and input.numel == m * k and _q4_0_weight_ok(q_weight, n_q, k) and _q4_0_weight_ok(k_weight, n_k, k)
            and _q4_0_weight_ok(v_weight, n_v, k)):
        raise DispatchError("quantized QKV Linear input metadata is inconsistent")
    name = "llmopt_q4_0_qkv_linear_f16" + ("" if m == 1 else "_m4" if m <= 8 else "_m16" if m <= 16 else "_m32")
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.FUSED_LINEAR, input_dtype="q4_0",
                                         output_dtype="float16")
    buffers = [input.buffer, q_weight.buffer, k_weight.buffer, v_weight.buffer, q_output.buffer, k_output.buffer,
               v_output.buffer]
    return [_run(context, entry, buffers, parameters.w4a16_qkv_linear(m=m, k=k, n_q=n_q, n_k=n_k, n_v=n_v),
                 (linear_f16_grid(m * (n_q + n_k + n_v)), 1, 1))]


def dispatch_quant_gated_linear(context: Context, *, m: int, n: int, k: int, input: Tensor, gate_weight: Tensor,
                                up_weight: Tensor, product: Tensor, activation: str = "silu") -> list:
    """Q4_0 gated product (lib/metal_q4_0_source.ml:26-150, llmopt_gated_product): buffers
    [input, gate, up, product], params {m, n, k, activation} with 0 silu, 1 gelu, 2 sigmoid."""
    codes = {"silu": 0, "gelu": 1, "sigmoid": 2}
    if activation not in codes:
        raise DispatchError(f"gated Linear activation {activation} is unsupported")
    if not (m > 0 and input.numel == m * k and product.numel == m * n and _q4_0_weight_ok(gate_weight, n, k)
            and _q4_0_weight_ok(up_weight, n, k)):
        raise DispatchError("quantized gated Linear input metadata is inconsistent")
    name = "llmopt_q4_0_gated_linear_f16" + ("_x8" if m == 1 else "_m4" if m <= 8 else "_m16" if m <= 16 else "_m32")
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.GATED_LINEAR, input_dtype="q4_0",
                                         output_dtype="float16")
    return [_run(context, entry, [input.buffer, gate_weight.buffer, up_weight.buffer, product.buffer],
                 parameters.u32s([m, n, k, codes[activation]]), (linear_f16_grid(m * n), 1, 1))]


def dispatch_attention(context: Context, *, causal: bool, scale: float, query: Tensor, key: Tensor, value: Tensor,
                       output: Tensor, mask: Optional[Tensor] = None) -> list:
    """dispatch_attention, lib/metal_dispatch_attention.ml:6-102: dense fp16 attention (prefill).
    query [b,h,q,d]; key [b,kvh,k,d]; value [b,kvh,k,d] or token-first [b,k,kvh,d]; output
    [b,h,q,d], or token-first when its shape is [b,q,h*d] or [b,q,h,d]."""
    if len(query.shape) != 4:
        raise DispatchError("attention query must have rank four")
    batches, heads, query_length, head_dimension = query.shape
    if len(key.shape) != 4:
        raise DispatchError("attention key must have rank four")
    kv_heads, key_length = key.shape[1], key.shape[2]
    if tuple(value.shape) == (batches, kv_heads, key_length, head_dimension):
        token_first_value = 0
    elif tuple(value.shape) == (batches, key_length, kv_heads, head_dimension):
        token_first_value = 1
    else:
        raise DispatchError("attention value must match key in head-major or token-major layout")
    if mask is not None:
        if len(mask.shape) != 4:
            raise DispatchError("attention mask must have rank four")
        if mask.dtype == "bool":
            mask_dtype = 1
        elif mask.dtype == "float16":
            mask_dtype = 2
        else:
            raise DispatchError(f"attention mask dtype {mask.dtype} is unsupported")
        mask_batches, mask_heads, mask_buffer = mask.shape[0], mask.shape[1], mask.buffer
    else:
        mask_batches, mask_heads, mask_dtype, mask_buffer = 0, 0, 0, query.buffer
    token_first_output = 1 if tuple(output.shape) in ((batches, query_length, heads * head_dimension),
                                                      (batches, query_length, heads, head_dimension)) else 0
    params = parameters.attention(
        batches=batches, heads=heads, query_length=query_length, key_length=key_length,
        head_dimension=head_dimension, mask_batches=mask_batches, mask_heads=mask_heads, causal=causal, scale=scale,
        kv_heads=kv_heads, token_first_output=token_first_output, past_length=max(0, key_length - query_length),
        token_first_value=token_first_value, mask_dtype=mask_dtype)
    entry, simd = None, False
    candidates = [(f"llmopt_attention_f16_simd_h{head_dimension}", True)] if head_dimension % 8 == 0 else []
    for name, is_simd in candidates + [("llmopt_attention_f16", False)]:
        try:
            entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.ATTENTION, input_dtype=query.dtype,
                                                 output_dtype=output.dtype)
            simd = is_simd
            break
        except (LookupError, RuntimeError):  # no such entry, or the library lacks the function
            continue
    if entry is None:
        raise DispatchError(f"serving package has no attention kernel for {query.dtype} -> {output.dtype}")
    rows = batches * heads * query_length
    grid_x = batches * heads * ((query_length + 31) // 32) * 128 if simd else rows
    return [_run(context, entry, [query.buffer, key.buffer, value.buffer, mask_buffer, output.buffer], params,
                 (grid_x, 1, 1))]


def dispatch_paged_attention_q8(context: Context, *, config: PagedAttentionConfig, query: Tensor,
                                current_key: Tensor, current_value: Tensor, pool: Tensor, slots: Tensor,
                                output: Tensor, mask: Optional[Tensor] = None,
                                slot_batch_stride: Optional[int] = None) -> list:
    """dispatch_paged_attention_q8, lib/metal_dispatch_attention.ml:104-217.
    ``slot_batch_stride`` (not None) selects the batched-decode extension: slots is
    [batches, stride] and the 72-byte parameter block is used."""
    if len(query.shape) != 4:
        raise DispatchError("paged Q8 attention query must have shape [b,h,q,d]")
    batches, query_heads, query_length, head_dimension = query.shape
    if len(current_key.shape) != 4 or current_key.shape[2] != query_length:
        raise DispatchError("paged Q8 attention current key must match query tokens")
    kv_heads = current_key.shape[1]
    if context.decode_uniforms_past_tokens is not None:
        past_length = context.decode_uniforms_past_tokens
    elif slot_batch_stride is not None:
        past_length = slots.shape[-1] if len(slots.shape) == 2 else None
        if past_length is None:
            raise DispatchError("batched paged Q8 attention slots must have rank two")
    else:
        if len(slots.shape) != 1:
            raise DispatchError("paged Q8 attention slots must have rank one")
        past_length = slots.shape[0]
    if mask is None:
        if query_length != 1:
            raise DispatchError("maskless paged Q8 attention requires one query token")
        mask_batches, mask_heads, mask_dtype, mask_buffer = 0, 0, 0, slots.buffer
    else:
        if len(mask.shape) != 4 or mask.shape[2] not in (query_length, 1):
            raise DispatchError("paged Q8 attention mask must have rank four")
        if mask.dtype == "bool":
            mask_dtype = 1
        elif mask.dtype == "float16":
            mask_dtype = 2
        else:
            raise DispatchError(f"paged Q8 attention mask dtype {mask.dtype} is unsupported")
        mask_batches, mask_heads, mask_buffer = mask.shape[0], mask.shape[1], mask.buffer
    fields = dict(batches=batches, query_heads=query_heads, kv_heads=kv_heads, past_length=past_length,
                  head_dimension=head_dimension, mask_batches=mask_batches, mask_heads=mask_heads,
                  token_elements=config.token_elements, key_offset=config.key_offset,
                  value_offset=config.value_offset, group_size=config.group_size, token_stride=config.token_stride,
                  scale=config.scale, mask_dtype=mask_dtype, query_length=query_length, window=config.window or 0)
    if slot_batch_stride is not None:
        params = parameters.paged_attention_q8_batched(slot_batch_stride=slot_batch_stride, **fields)
        name = "llmopt_attention_q8_paged_batched"
    else:
        params = parameters.paged_attention_q8(**fields)
        name = paged_attention_kernel_name(split8=False, experimental_gqa3_split8=False, query_heads=query_heads,
                                           kv_heads=kv_heads, head_dimension=head_dimension)
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.ATTENTION, input_dtype="float16",
                                         output_dtype=output.dtype)
    by_kv_head = name.endswith("_gqa3") or name.endswith("_gqa3_split8")
    rows = batches * (kv_heads if by_kv_head else query_heads) * query_length
    buffers = [query.buffer, current_key.buffer, current_value.buffer, pool.buffer, slots.buffer, mask_buffer,
               output.buffer]
    return [_run(context, entry, buffers, params, (simd_rows_grid(rows), 1, 1))]


# ---- recurrent ---------------------------------------------------------------------------------

def dispatch_short_conv_step(context: Context, *, in_proj: Tensor, conv_state: Tensor, conv_weight: Tensor,
                             output: Tensor) -> list:
    """lib/metal_dispatch_recurrent.ml:91-113; conv_state [1,C,3] is updated in place."""
    channels = output.shape[-1]
    if in_proj.numel != 3 * channels or conv_state.numel != 3 * channels or conv_weight.numel != 3 * channels:
        raise DispatchError("short conv step shapes are inconsistent")
    entry = context.runtime.kernel_entry(name="llmopt_short_conv_step_f16", operation=kernel_abi.SHORT_CONV_STEP,
                                         input_dtype="float16", output_dtype="float16")
    return [_run(context, entry, [in_proj.buffer, conv_state.buffer, conv_weight.buffer, output.buffer],
                 parameters.short_conv_step(channels=channels), (channels, 1, 1))]


def dispatch_short_conv_prefill(context: Context, *, in_proj: Tensor, conv_weight: Tensor, output: Tensor,
                                conv_state_out: Tensor, conv_state_in: Optional[Tensor] = None) -> list:
    """lib/metal_dispatch_recurrent.ml:115-154; with an initial state the _init
    kernel is chosen and the state is bound as the fifth buffer."""
    tokens, channels = output.shape[-2], output.shape[-1]
    if in_proj.numel != tokens * 3 * channels or conv_weight.numel != 3 * channels:
        raise DispatchError("short conv prefill shapes are inconsistent")
    name = "llmopt_short_conv_prefill_f16" if conv_state_in is None else "llmopt_short_conv_prefill_init_f16"
    entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.SHORT_CONV_PREFILL,
                                         input_dtype="float16", output_dtype="float16")
    buffers = [in_proj.buffer, conv_weight.buffer, output.buffer, conv_state_out.buffer]
    if conv_state_in is not None:
        buffers.append(conv_state_in.buffer)
    params = parameters.short_conv_prefill(tokens=tokens, channels=channels,
                                           has_initial_state=conv_state_in is not None)
    return [_run(context, entry, buffers, params, (channels, 1, 1))]


# ---- physical Q8 cache ------------------------------------------------------------------------------

class Cache:
    """The pack / unpack dispatch half of ``Metal_cache`` (lib/metal_cache.ml:289-608):
    owns the token pool, the checkpoint pool and a slot scratch buffer. Slot
    OWNERSHIP (radix leases) stays with the caller, as in the reference."""

    def __init__(self, runtime: Runtime, layout: Layout, *, token_capacity: int, checkpoint_capacity: int = 0):
        self.runtime = runtime
        self.layout = layout
        self.token_capacity = token_capacity
        self.checkpoint_capacity = checkpoint_capacity
        self.token_pool = Buffer.create(runtime, max(token_capacity * layout.bytes_per_token, 16))
        self.checkpoint_pool = Buffer.create(runtime, max(checkpoint_capacity * layout.bytes_per_checkpoint, 16))

    def _slot_buffer(self, slots: Sequence[int]) -> Buffer:
        for slot in slots:
            if slot < 0 or slot >= self.token_capacity:
                raise DispatchError("physical cache slot is outside the token pool")
        buffer = Buffer.create(self.runtime, max(4 * len(slots), 16))
        if slots:
            buffer.set_u32_array(0, list(slots))
        return buffer

    def _attention_fields(self, layer: int, items: int, source_items: int, source_offset: int) -> dict:
        if layer < 0 or layer >= len(self.layout.attentions):
            raise DispatchError("physical cache attention layer is outside the layout")
        region = self.layout.attentions[layer]
        return dict(items=items, heads=region.geometry.kv_heads, head_dim=region.geometry.head_dim,
                    group_size=self.layout.group_size, token_elements=self.layout.token_elements,
                    token_groups=self.layout.token_groups, token_stride=self.layout.bytes_per_token,
                    source_items=source_items, source_offset=source_offset)

    def pack_attention(self, context: Context, *, layer: int, kind: str, slots, source: Buffer, source_items: int,
                       source_offset: int = 0, slot_buffer: Optional[Buffer] = None) -> list:
        region = self.layout.attentions[layer] if 0 <= layer < len(self.layout.attentions) else None
        fields = self._attention_fields(layer, len(slots), source_items, source_offset)
        segment = region.key_offset if kind == "key" else region.value_offset
        expected = fields["heads"] * source_items * fields["head_dim"] * 2
        if source.byte_length() < expected:
            raise DispatchError("physical cache attention source has an unexpected length")
        params = parameters.cache_attention(segment_offset=segment, **fields)
        entry = context.runtime.kernel_entry(name="llmopt_cache_pack_attention_q8_simd", operation=kernel_abi.CACHE,
                                             input_dtype="float16", output_dtype="uint8")
        groups = len(slots) * fields["heads"] * (fields["head_dim"] // fields["group_size"])
        slot_buffer = slot_buffer or self._slot_buffer(slots)
        context.execution_batch.resources.append(slot_buffer)
        return [_run(context, entry, [source, slot_buffer, self.token_pool], params,
                     (round_up(max(groups, 1), 8) * 32, 1, 1))]

    def pack_attention_pair(self, context: Context, *, layer: int, slots, key_source: Buffer, value_source: Buffer,
                            source_items: int, source_offset: int = 0,
                            slot_buffer: Optional[Buffer] = None) -> list:
        region = self.layout.attentions[layer] if 0 <= layer < len(self.layout.attentions) else None
        fields = self._attention_fields(layer, len(slots), source_items, source_offset)
        params = parameters.cache_attention_pair(key_segment_offset=region.key_offset,
                                                 value_segment_offset=region.value_offset, **fields)
        entry = context.runtime.kernel_entry(name="llmopt_cache_pack_attention_q8_pair_simd",
                                             operation=kernel_abi.CACHE, input_dtype="float16", output_dtype="uint8")
        groups = len(slots) * fields["heads"] * (fields["head_dim"] // fields["group_size"])
        slot_buffer = slot_buffer or self._slot_buffer(slots)
        context.execution_batch.resources.append(slot_buffer)
        return [_run(context, entry, [key_source, value_source, slot_buffer, self.token_pool], params,
                     (round_up(max(groups, 1), 8) * 32, 1, 1))]

    def unpack_attention(self, context: Context, *, layer: int, kind: str, slots, destination: Buffer) -> list:
        region = self.layout.attentions[layer] if 0 <= layer < len(self.layout.attentions) else None
        fields = self._attention_fields(layer, len(slots), len(slots), 0)
        segment = region.key_offset if kind == "key" else region.value_offset
        elements = len(slots) * fields["heads"] * fields["head_dim"]
        if destination.byte_length() != elements * 2:  # exact_buffer_length, lib/metal_cache.ml:249-255
            raise DispatchError("physical cache attention destination has an unexpected length")
        params = parameters.cache_attention(segment_offset=segment, **fields)
        vec4 = elements % 4 == 0 and fields["head_dim"] % 4 == 0
        name = "llmopt_cache_unpack_attention_q8_vec4" if vec4 else "llmopt_cache_unpack_attention_q8"
        entry = context.runtime.kernel_entry(name=name, operation=kernel_abi.CACHE, input_dtype="uint8",
                                             output_dtype="float16")
        slot_buffer = self._slot_buffer(slots)
        context.execution_batch.resources.append(slot_buffer)
        grid = elements // 4 if vec4 else elements
        return [_run(context, entry, [self.token_pool, slot_buffer, destination], params,
                     (round_up(max(grid, 1), 256), 1, 1))]

    def _checkpoint_params(self, layer: int, checkpoint: int) -> bytes:
        if layer < 0 or layer >= self.layout.recurrent_layers:
            raise DispatchError("physical cache recurrent layer is outside the layout")
        if checkpoint < 0 or checkpoint >= self.checkpoint_capacity:
            raise DispatchError("physical cache checkpoint is outside the checkpoint pool")
        return parameters.cache_checkpoint(
            checkpoint=checkpoint, layer=layer, layer_elements=self.layout.recurrent_layer_elements,
            group_size=self.layout.group_size, checkpoint_elements=self.layout.checkpoint_elements,
            checkpoint_groups=self.layout.checkpoint_groups, checkpoint_stride=self.layout.bytes_per_checkpoint)

    def pack_checkpoint(self, context: Context, *, layer: int, checkpoint: int, source: Buffer) -> list:
        params = self._checkpoint_params(layer, checkpoint)
        if source.byte_length() != self.layout.recurrent_layer_elements * 2:
            raise DispatchError("physical cache checkpoint source has an unexpected length")
        entry = context.runtime.kernel_entry(name="llmopt_cache_pack_checkpoint_q8_simd", operation=kernel_abi.CACHE,
                                             input_dtype="float16", output_dtype="uint8")
        groups = self.layout.recurrent_layer_elements // self.layout.group_size
        return [_run(context, entry, [source, self.checkpoint_pool], params, (round_up(groups, 8) * 32, 1, 1))]

    def unpack_checkpoint(self, context: Context, *, layer: int, checkpoint: int, destination: Buffer) -> list:
        params = self._checkpoint_params(layer, checkpoint)
        if destination.byte_length() != self.layout.recurrent_layer_elements * 2:
            raise DispatchError("physical cache checkpoint destination has an unexpected length")
        entry = context.runtime.kernel_entry(name="llmopt_cache_unpack_checkpoint_q8_vec4",
                                             operation=kernel_abi.CACHE, input_dtype="uint8", output_dtype="float16")
        return [_run(context, entry, [self.checkpoint_pool, destination], params,
                     (round_up(self.layout.recurrent_layer_elements // 4, 256), 1, 1))]


def dispatch_gated_delta(context: Context, *, query: Tensor, key: Tensor, value: Tensor, gate: Tensor, beta: Tensor,
                         output: Tensor) -> list:
    """dispatch_gated_delta, lib/metal_dispatch_recurrent.ml:34-89: f32 head-major [b,h,t,w] or f16
    token-major [b,t,h,w] vectors, width a multiple of 32, gate f32, output f16 token-major."""
    if len(query.shape) != 4:
        raise DispatchError("unsupported Metal gated-delta layout or dtype contract")
    if query.dtype == "float32":
        batch, heads, tokens, width = query.shape
        scalar_shape, beta_dtype, stem = (batch, heads, tokens), "float32", "llmopt_gated_delta_f32_d"
    elif query.dtype == "float16":
        batch, tokens, heads, width = query.shape
        scalar_shape, beta_dtype, stem = (batch, tokens, heads), "float16", "llmopt_gated_delta_tm_f16_d"
    else:
        raise DispatchError("unsupported Metal gated-delta layout or dtype contract")
    ok = (width > 0 and width % 32 == 0 and tuple(output.shape) == (batch, tokens, heads, width)
          and key.dtype == query.dtype and value.dtype == query.dtype and gate.dtype == "float32"
          and beta.dtype == beta_dtype and tuple(key.shape) == tuple(query.shape)
          and tuple(value.shape) == tuple(query.shape) and tuple(gate.shape) == scalar_shape
          and tuple(beta.shape) == scalar_shape)
    if not ok:
        raise DispatchError("unsupported Metal gated-delta layout or dtype contract")
    entry = context.runtime.kernel_entry(name=f"{stem}{width}", operation=kernel_abi.GATED_DELTA,
                                         input_dtype=query.dtype, output_dtype="float16")
    grid = round_up(batch * heads * width, 4) * 32  # gated_delta_grid, lib/metal_dispatch_common.ml:80-86
    return [_run(context, entry, [query.buffer, key.buffer, value.buffer, gate.buffer, beta.buffer, output.buffer],
                 parameters.u32s([batch, heads, tokens, width]), (grid, 1, 1))]


def dispatch_triangular_recurrence(context: Context, *, start: int, stop: int, input: Tensor, output: Tensor) -> list:
    """dispatch_triangular_recurrence, lib/metal_dispatch_recurrent.ml:6-32: square matrices up to 64 wide."""
    width, rows = input.shape[-1], input.shape[-2]
    if width > 64 or rows != width:
        raise DispatchError("unsupported Metal triangular recurrence shape")
    outer = input.numel // (width * width)
    entry = context.runtime.kernel_entry(name="llmopt_triangular_recurrence_f32",
                                         operation=kernel_abi.TRIANGULAR_RECURRENCE, input_dtype="float32",
                                         output_dtype="float32")
    return [_run(context, entry, [input.buffer, output.buffer], parameters.u32s([outer, width, start, stop]),
                 (outer * 64, 1, 1))]
