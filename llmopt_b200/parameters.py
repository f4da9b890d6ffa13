"""Byte-exact little-endian parameter blocks, mirroring the reference's
``Metal_parameters`` (lib/metal_parameters.ml) and the ad-hoc ``Parameters.u32s``
blocks built in its dispatchers.  A value that does not fit uint32 raises
``ValueError`` with the reference's message."""

from __future__ import annotations

import struct
from typing import Iterable


def _u32(value: int) -> int:
    if value < 0 or value > 0xFFFFFFFF:
        raise ValueError(f"Metal parameter does not fit uint32: {value}")
    return int(value)


def u32s(values: Iterable[int]) -> bytes:  # lib/metal_parameters.ml:14-22
    values = [_u32(v) for v in values]
    return struct.pack(f"<{len(values)}I", *values)


def rms_norm(*, rows: int, width: int, epsilon: float) -> bytes:  # :24-29
    return struct.pack("<IIf", _u32(rows), _u32(width), epsilon)


def w4a16_lm_head_argmax(*, m: int, n: int, k: int, epsilon: float) -> bytes:  # :38-43
    return struct.pack("<IIIf", _u32(m), _u32(n), _u32(k), epsilon)


def w4a16_swiglu_ffn(*, m: int, n: int, k: int, epsilon: float) -> bytes:  # :45-50
    return struct.pack("<IIIf", _u32(m), _u32(n), _u32(k), epsilon)


def w4a16_linear(*, m: int, n: int, k: int, has_bias: bool, bias_row_stride: int) -> bytes:
    """lib/metal_dispatch_linear.ml:964-967."""
    return u32s([m, n, k, 1 if has_bias else 0, bias_row_stride])


def w4a16_qkv_linear(*, m: int, k: int, n_q: int, n_k: int, n_v: int) -> bytes:  # :423
    return u32s([m, k, n_q, n_k, n_v])


def rotary_qk(*, batches, tokens, q_heads, k_heads, width, half_dimension, trig_batches) -> bytes:  # :77-81
    return u32s([batches, tokens, q_heads, k_heads, width, half_dimension, trig_batches])


def attention(*, batches, heads, query_length, key_length, head_dimension, mask_batches, mask_heads, causal,
              scale, kv_heads=None, token_first_output=0, past_length=0, token_first_value=0,
              mask_dtype=0) -> bytes:  # :95-117, 56 bytes
    kv_heads = heads if kv_heads is None else kv_heads
    return struct.pack(
        "<8If5I", _u32(batches), _u32(heads), _u32(query_length), _u32(key_length), _u32(head_dimension),
        _u32(mask_batches), _u32(mask_heads), 1 if causal else 0, scale, _u32(kv_heads), _u32(token_first_output),
        _u32(past_length), _u32(token_first_value), _u32(mask_dtype))


def paged_attention_q8(*, batches, query_heads, kv_heads, past_length, head_dimension, mask_batches, mask_heads,
                       token_elements, key_offset, value_offset, group_size, token_stride, scale, mask_dtype,
                       query_length=1, window=0) -> bytes:  # :119-140, 64 bytes; past_length at byte 12
    return struct.pack(
        "<12If3I", _u32(batches), _u32(query_heads), _u32(kv_heads), _u32(past_length), _u32(head_dimension),
        _u32(mask_batches), _u32(mask_heads), _u32(token_elements), _u32(key_offset), _u32(value_offset),
        _u32(group_size), _u32(token_stride), scale, _u32(query_length), _u32(mask_dtype), _u32(window))


def paged_attention_q8_batched(*, slot_batch_stride: int, **fields) -> bytes:
    """The 64 standard bytes followed by slot_batch_stride and a reserved word:
    every sequence of the batch reads its own slot table (an extension; the
    reference shares one table, lib/metal_cache_source.ml:382-401)."""
    return paged_attention_q8(**fields) + struct.pack("<II", _u32(slot_batch_stride), 0)


def cache_attention(*, items, segment_offset, heads, head_dim, group_size, token_elements, token_groups,
                    token_stride, source_items, source_offset) -> bytes:  # lib/metal_cache.ml:315-318
    return u32s([items, segment_offset, heads, head_dim, group_size, token_elements, token_groups, token_stride,
                 source_items, source_offset])


def cache_attention_pair(*, items, key_segment_offset, value_segment_offset, heads, head_dim, group_size,
                         token_elements, token_groups, token_stride, source_items,
                         source_offset) -> bytes:  # lib/metal_cache.ml:344-347
    return u32s([items, key_segment_offset, value_segment_offset, heads, head_dim, group_size, token_elements,
                 token_groups, token_stride, source_items, source_offset])


def cache_checkpoint(*, checkpoint, layer, layer_elements, group_size, checkpoint_elements, checkpoint_groups,
                     checkpoint_stride) -> bytes:  # lib/metal_cache.ml:544-547; checkpoint at byte 0
    return u32s([checkpoint, layer, layer_elements, group_size, checkpoint_elements, checkpoint_groups,
                 checkpoint_stride])


def short_conv(*, batches, channels, input_width, output_width, kernel_width, stride, padding,
               dilation) -> bytes:  # lib/metal_dispatch_recurrent.ml:175-180
    return u32s([batches, channels, input_width, output_width, kernel_width, stride, padding, dilation])


def short_conv_silu_tm(*, batches, tokens, channels, kernel_width, stride, padding, dilation,
                       output_start) -> bytes:  # lib/metal_dispatch_recurrent.ml:210-217
    return u32s([batches, tokens, channels, kernel_width, stride, padding, dilation, output_start])


def short_conv_step(*, channels) -> bytes:  # lib/metal_dispatch_recurrent.ml:98
    return u32s([channels])


def short_conv_prefill(*, tokens, channels, has_initial_state) -> bytes:  # :138
    return u32s([tokens, channels, 1 if has_initial_state else 0])


def embedding(*, tokens, vocabulary, width) -> bytes:  # lib/metal_tensor_source.ml:237
    return u32s([tokens, vocabulary, width])


def rms_rope(*, batches, tokens, heads, width, half_dimension, trig_batches, epsilon) -> bytes:  # :52-61, 28 bytes
    return struct.pack("<6If", *[_u32(v) for v in (batches, tokens, heads, width, half_dimension, trig_batches)], epsilon)


def rms_rope_qk(*, batches, tokens, q_heads, k_heads, width, half_dimension, trig_batches, epsilon) -> bytes:  # :63-72
    return struct.pack("<7If", *[_u32(v) for v in (batches, tokens, q_heads, k_heads, width, half_dimension,
                                                   trig_batches)], epsilon)


def l2_norm_slice(*, input_rows, groups, width, input_width, offset, epsilon) -> bytes:
    """L2NormSliceParams, lib/metal_normalization_source.ml:553-556 (24 bytes)."""
    return struct.pack("<5If", *[_u32(v) for v in (input_rows, groups, width, input_width, offset)], epsilon)


def count(*, count) -> bytes:  # CastParams / UnaryParams {count}
    return u32s([count])


def pointwise(*, output_shape, left_shape=None, right_shape=None, left_scalar=None, right_scalar=None) -> bytes:
    """``Metal_parameters.pointwise`` (lib/metal_parameters.ml:331-382), 136 bytes: count, rank, scalar
    flags, the output shape and both operand shapes aligned to it from the right (missing or
    scalar operands are all ones), padded with ones to rank 8, then the scalars as int64 and f32."""
    output_shape = [int(v) for v in output_shape]
    rank = len(output_shape)
    if rank > 8:
        raise ValueError("Metal pointwise kernels support rank at most eight")

    def aligned(shape):
        if shape is None:
            return [1] * rank
        shape = [int(v) for v in shape]
        if len(shape) > rank:
            raise ValueError("pointwise input rank exceeds output rank")
        shape = [1] * (rank - len(shape)) + shape
        if any(i != 1 and i != o for i, o in zip(shape, output_shape)):
            raise ValueError("pointwise input shape is not broadcastable to output")
        return shape

    pad = lambda dims: [_u32(v) for v in dims] + [1] * (8 - rank)
    total = 1
    for v in output_shape:
        total *= v
    block = bytearray(struct.pack("<4I", _u32(total), rank, 1 if left_scalar is not None else 0,
                                  1 if right_scalar is not None else 0))
    for dims in (output_shape, aligned(left_shape), aligned(right_shape)):
        block += struct.pack("<8I", *pad(dims))
    block += struct.pack("<qqff", int(left_scalar or 0), int(right_scalar or 0), float(left_scalar or 0.0),
                         float(right_scalar or 0.0))
    assert len(block) == 136
    return bytes(block)
