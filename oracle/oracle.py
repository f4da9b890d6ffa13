"""ctypes front end of the CPU oracle (oracle/llmopt_oracle.c).

TEST INFRASTRUCTURE ONLY: the oracle is the checker for the CUDA kernels.  Only
tests, the smoke entry and the bench's CPU-baseline leg import this module; the
shipped library never does.

Every function takes and returns numpy arrays.  f16 tensors are ``np.float16``
arrays; packed weights and cache pools are ``np.uint8``.
"""

from __future__ import annotations

import ctypes
import os
import struct
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    source = os.path.join(_HERE, "llmopt_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or (
        os.path.exists(source) and os.path.getmtime(source) > os.path.getmtime(_LIB_PATH)
    )
    if force or stale:
        os.makedirs(os.path.dirname(_LIB_PATH), exist_ok=True)
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-o", _LIB_PATH, source, "-lm"]
        )
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_epilogue_apply.restype = ctypes.c_double
        _lib.orc_epilogue_apply.argtypes = [ctypes.c_int] + [ctypes.c_double] * 3
        _lib.orc_argmax_f16.restype = ctypes.c_int64
    return _lib


def _p(array):
    if array is None:
        return None
    assert array.flags["C_CONTIGUOUS"], "oracle inputs must be contiguous"
    return array.ctypes.data_as(ctypes.c_void_p)


def _f16(array):
    return np.ascontiguousarray(array, dtype=np.float16)


def _u8(array):
    return np.ascontiguousarray(array, dtype=np.uint8)


def _u32(array):
    return np.ascontiguousarray(array, dtype=np.uint32)


I64 = ctypes.c_int64
U32 = ctypes.c_uint32
F32 = ctypes.c_float

EPILOGUE_TAGS = {
    "none": 0,
    "bias": 1,
    "silu": 2,
    "gelu": 3,
    "silu_mul": 4,
    "gelu_mul": 5,
    "residual_add": 6,
    "bias_residual_add": 7,
    "silu_mul_residual_add": 8,
    "gelu_mul_residual_add": 9,
}


def unpack_int4(packed):
    packed = _u8(packed)
    n, half_k = packed.shape
    out = np.empty((n, half_k * 2), dtype=np.int8)
    lib().orc_unpack_int4(_p(packed), _p(out), I64(n), I64(half_k * 2))
    return out


def w4a16_linear(x, packed, scale, bias=None, bias_row_stride=0, zero=None, order="f64"):
    """y[m,n] = half(x . dequant(W)^T (+bias)); order 'f64' follows lib/cpu.ml,
    'msl_m1' the Metal m=1 kernel's fp32 lane order."""
    x, packed, scale = _f16(x), _u8(packed), _f16(scale)
    m, k = x.shape
    n = packed.shape[0]
    assert packed.shape == (n, k // 2) and scale.shape == (n, k // 64)
    y = np.empty((m, n), dtype=np.float16)
    bias_c = None if bias is None else _f16(bias)
    if order == "msl_m1":
        assert zero is None
        lib().orc_w4a16_linear_msl_m1(
            _p(x), _p(packed), _p(scale), _p(bias_c), I64(bias_row_stride), _p(y), I64(m), I64(n), I64(k)
        )
    else:
        zero_c = None if zero is None else _f16(zero)
        lib().orc_w4a16_linear(
            _p(x), _p(packed), _p(scale), _p(zero_c), ctypes.c_int(0 if zero is None else 1),
            _p(bias_c), I64(bias_row_stride), _p(y), I64(m), I64(n), I64(k),
        )
    return y


def w4a16_linear_f64(x, packed, scale, zero=None):
    x, packed, scale = _f16(x), _u8(packed), _f16(scale)
    m, k = x.shape
    n = packed.shape[0]
    y = np.empty((m, n), dtype=np.float64)
    zero_c = None if zero is None else _f16(zero)
    lib().orc_w4a16_linear_f64(
        _p(x), _p(packed), _p(scale), _p(zero_c), ctypes.c_int(0 if zero is None else 1), _p(y),
        I64(m), I64(n), I64(k),
    )
    return y


def set_threads(threads: int) -> int:
    """Sets the OpenMP thread count of the ``_mt`` functions; returns the count in force."""
    lib().orc_set_threads(ctypes.c_int(int(threads)))
    return int(lib().orc_max_threads())


def w4a16_linear_cols_mt(x, packed, scale, col_begin, col_end):
    """Timing helper: reference loop nest over a column range, OpenMP threads."""
    x, packed, scale = _f16(x), _u8(packed), _f16(scale)
    m, k = x.shape
    n = packed.shape[0]
    y = np.zeros((m, n), dtype=np.float16)
    lib().orc_w4a16_linear_cols_mt(
        _p(x), _p(packed), _p(scale), _p(y), I64(m), I64(n), I64(k), I64(col_begin), I64(col_end)
    )
    return y


def w4a16_qkv_linear(x, qw, qs, kw, ks, vw, vs):
    x = _f16(x)
    m, k = x.shape
    qw, kw, vw = _u8(qw), _u8(kw), _u8(vw)
    qs, ks, vs = _f16(qs), _f16(ks), _f16(vs)
    n_q, n_k, n_v = qw.shape[0], kw.shape[0], vw.shape[0]
    q = np.empty((m, n_q), np.float16)
    kk = np.empty((m, n_k), np.float16)
    v = np.empty((m, n_v), np.float16)
    lib().orc_w4a16_qkv_linear(
        _p(x), _p(qw), _p(qs), _p(kw), _p(ks), _p(vw), _p(vs), _p(q), _p(kk), _p(v),
        I64(m), I64(k), I64(n_q), I64(n_k), I64(n_v),
    )
    return q, kk, v


def rms_norm(x, weight, epsilon):
    x = np.ascontiguousarray(x)
    is_f32 = x.dtype == np.float32
    if not is_f32:
        x = _f16(x)
    rows, width = x.shape
    out = np.empty((rows, width), np.float16)
    lib().orc_rms_norm(_p(x), ctypes.c_int(int(is_f32)), _p(_f16(weight)), _p(out), I64(rows), I64(width), F32(epsilon))
    return out


def w4a16_swiglu_ffn(activation, residual, gate_w, gate_s, up_w, up_s, down_w, down_s, norm_w, epsilon):
    """Returns (output, normalized, product); n = intermediate, k = hidden."""
    activation = np.ascontiguousarray(activation)
    is_f32 = activation.dtype == np.float32
    if not is_f32:
        activation = _f16(activation)
    m, k = activation.shape
    n = gate_w.shape[0]
    y = np.empty((m, k), np.float16)
    normalized = np.empty((m, k), np.float16)
    product = np.empty((m, n), np.float16)
    lib().orc_w4a16_swiglu_ffn(
        _p(activation), ctypes.c_int(int(is_f32)), _p(_f16(residual)), _p(_u8(gate_w)), _p(_f16(gate_s)),
        _p(_u8(up_w)), _p(_f16(up_s)), _p(_u8(down_w)), _p(_f16(down_s)), _p(_f16(norm_w)), _p(y),
        _p(normalized), _p(product), I64(m), I64(n), I64(k), F32(epsilon),
    )
    return y, normalized, product


def w4a16_dual_swiglu(x, gate_w, gate_s, up_w, up_s):
    x = _f16(x)
    m, k = x.shape
    n = gate_w.shape[0]
    product = np.empty((m, n), np.float16)
    lib().orc_w4a16_dual_swiglu(
        _p(x), _p(_u8(gate_w)), _p(_f16(gate_s)), _p(_u8(up_w)), _p(_f16(up_s)), _p(product),
        I64(m), I64(n), I64(k),
    )
    return product


def w4a16_linear_epilogue(x, packed, scale, tag, first=None, second=None):
    x, packed, scale = _f16(x), _u8(packed), _f16(scale)
    m, k = x.shape
    n = packed.shape[0]
    y = np.empty((m, n), np.float16)
    lib().orc_w4a16_linear_epilogue(
        _p(x), _p(packed), _p(scale), ctypes.c_int(EPILOGUE_TAGS[tag]),
        _p(None if first is None else _f16(first)), _p(None if second is None else _f16(second)),
        _p(y), I64(m), I64(n), I64(k),
    )
    return y


def w4a16_lm_head_argmax(x, norm_w, weight, scale, epsilon, want_logits=False):
    """Returns (token_ids u32[m], logits f16[m,n] or None, best fp32 values)."""
    x = np.ascontiguousarray(x)
    is_f32 = x.dtype == np.float32
    if not is_f32:
        x = _f16(x)
    m, k = x.shape
    n = weight.shape[0]
    tokens = np.empty((m,), np.uint32)
    logits = np.empty((m, n), np.float16) if want_logits else None
    best = np.empty((m,), np.float32)
    lib().orc_w4a16_lm_head_argmax(
        _p(x), ctypes.c_int(int(is_f32)), _p(_f16(norm_w)), _p(_u8(weight)), _p(_f16(scale)), _p(tokens),
        _p(logits), _p(best), I64(m), I64(n), I64(k), F32(epsilon),
    )
    return tokens, logits, best


def cache_pack_attention_q8(source, slots, pool, *, segment_offset, heads, head_dim, group_size,
                            token_elements, token_stride, source_items, source_offset=0):
    """Packs in place into ``pool`` (np.uint8, 1-D)."""
    source, slots = _f16(source), _u32(slots)
    assert pool.dtype == np.uint8 and pool.flags["C_CONTIGUOUS"]
    lib().orc_cache_pack_attention_q8(
        _p(source), _p(slots), _p(pool), U32(len(slots)), U32(segment_offset), U32(heads), U32(head_dim),
        U32(group_size), U32(token_elements), U32(token_stride), U32(source_items), U32(source_offset),
    )


def cache_unpack_attention_q8(pool, slots, *, segment_offset, heads, head_dim, group_size,
                              token_elements, token_stride):
    slots = _u32(slots)
    out = np.empty((heads, len(slots), head_dim), np.float16)
    lib().orc_cache_unpack_attention_q8(
        _p(_u8(pool)), _p(slots), _p(out), U32(len(slots)), U32(segment_offset), U32(heads), U32(head_dim),
        U32(group_size), U32(token_elements), U32(token_stride),
    )
    return out


def cache_pack_checkpoint_q8(source, pool, *, checkpoint, layer, layer_elements, group_size,
                             checkpoint_elements, checkpoint_stride):
    lib().orc_cache_pack_checkpoint_q8(
        _p(_f16(source)), _p(pool), U32(checkpoint), U32(layer), U32(layer_elements), U32(group_size),
        U32(checkpoint_elements), U32(checkpoint_stride),
    )


def cache_unpack_checkpoint_q8(pool, *, checkpoint, layer, layer_elements, group_size,
                               checkpoint_elements, checkpoint_stride):
    out = np.empty((layer_elements,), np.float16)
    lib().orc_cache_unpack_checkpoint_q8(
        _p(_u8(pool)), _p(out), U32(checkpoint), U32(layer), U32(layer_elements), U32(group_size),
        U32(checkpoint_elements), U32(checkpoint_stride),
    )
    return out


def paged_params_bytes(*, batches, query_heads, kv_heads, past_length, head_dim, mask_batches=0,
                       mask_heads=0, token_elements, key_offset, value_offset, group_size,
                       token_stride, scale, query_length=1, mask_dtype=0, window=0) -> bytes:
    """The 64-byte Q8PagedAttentionParams block (lib/metal_parameters.ml:119-140)."""
    return struct.pack(
        "<12If3I", batches, query_heads, kv_heads, past_length, head_dim, mask_batches, mask_heads,
        token_elements, key_offset, value_offset, group_size, token_stride, scale, query_length,
        mask_dtype, window,
    )


def attention_q8_paged(query, current_key, current_value, pool, slots, mask, params: bytes,
                       slot_batch_stride=0):
    """query [b,hq,q,D] -> output token-first [b,q,hq,D]."""
    query = _f16(query)
    b, hq, q, d = query.shape
    out = np.empty((b, q, hq, d), np.float16)
    mask_c = None if mask is None else np.ascontiguousarray(mask)
    block = ctypes.create_string_buffer(params, 64)
    lib().orc_attention_q8_paged(
        _p(query), _p(_f16(current_key)), _p(_f16(current_value)), _p(_u8(pool)), _p(_u32(slots)),
        _p(mask_c), _p(out), block, U32(slot_batch_stride),
    )
    return out


def attention_dense(q, k, v, mask, *, causal, scale, kv_heads=0, token_first_output=0, past_length=0,
                    token_first_value=0, mask_dtype=0, mask_batches=0, mask_heads=0):
    q, k, v = _f16(q), _f16(k), _f16(v)
    b, h, ql, d = q.shape
    kl = v.shape[1] if token_first_value else k.shape[2]
    kl = k.shape[2]
    out = np.empty((b, ql, h, d) if token_first_output else (b, h, ql, d), np.float16)
    mask_c = None if mask is None else np.ascontiguousarray(mask)
    lib().orc_attention_dense(
        _p(q), _p(k), _p(v), _p(mask_c), _p(out), U32(b), U32(h), U32(ql), U32(kl), U32(d), U32(mask_batches),
        U32(mask_heads), U32(causal), F32(scale), U32(kv_heads), U32(token_first_output), U32(past_length),
        U32(token_first_value), U32(mask_dtype),
    )
    return out


def short_conv(x, weight, *, output_width, stride, padding, dilation):
    x, weight = _f16(x), _f16(weight)
    b, c, w = x.shape
    kw = weight.shape[-1]
    out = np.empty((b, c, output_width), np.float16)
    lib().orc_short_conv(_p(x), _p(weight), _p(out), U32(b), U32(c), U32(w), U32(output_width), U32(kw),
                         U32(stride), U32(padding), U32(dilation))
    return out


def short_conv_silu_tm(x, weight, *, stride=1, padding=0, dilation=1, output_start=0):
    x, weight = _f16(x), _f16(weight)
    b, t, c = x.shape
    kw = weight.shape[-1]
    out = np.empty((b, t, c), np.float16)
    lib().orc_short_conv_silu_tm(_p(x), _p(weight), _p(out), U32(b), U32(t), U32(c), U32(kw), U32(stride),
                                 U32(padding), U32(dilation), U32(output_start))
    return out


def short_conv_step(in_proj, conv_state, conv_weight):
    """Returns (output [C], new_state [C,3]); does not mutate its inputs."""
    in_proj, conv_weight = _f16(in_proj).reshape(-1), _f16(conv_weight)
    channels = in_proj.size // 3
    state = _f16(conv_state).copy()
    out = np.empty((channels,), np.float16)
    lib().orc_short_conv_step(_p(in_proj), _p(state), _p(conv_weight), _p(out), U32(channels))
    return out, state


def short_conv_prefill(in_proj, conv_weight, state_in=None):
    in_proj, conv_weight = _f16(in_proj), _f16(conv_weight)
    tokens = in_proj.shape[-2]
    channels = in_proj.shape[-1] // 3
    out = np.empty((tokens, channels), np.float16)
    state_out = np.empty((channels, 3), np.float16)
    state_c = None if state_in is None else _f16(state_in)
    lib().orc_short_conv_prefill(_p(in_proj), _p(conv_weight), _p(out), _p(state_out), _p(state_c),
                                 U32(tokens), U32(channels), U32(0 if state_in is None else 1))
    return out, state_out


def rotary_qk(q_in, k_in, cosine, sine, *, half_dimension, trig_batches=1):
    """q_in/k_in token-first [b,t,h,w] -> head-major [b,h,t,w]."""
    q_in, k_in = _f16(q_in), _f16(k_in)
    b, t, qh, w = q_in.shape
    kh = k_in.shape[2]
    q_out = np.empty((b, qh, t, w), np.float16)
    k_out = np.empty((b, kh, t, w), np.float16)
    lib().orc_rotary_qk(_p(q_in), _p(k_in), _p(_f16(cosine)), _p(_f16(sine)), _p(q_out), _p(k_out), U32(b),
                        U32(t), U32(qh), U32(kh), U32(w), U32(half_dimension), U32(trig_batches))
    return q_out, k_out


def embedding_f16(indices, table):
    indices = np.ascontiguousarray(indices, dtype=np.int64).reshape(-1)
    table = _f16(table)
    out = np.empty((indices.size, table.shape[1]), np.float16)
    lib().orc_embedding_f16(_p(indices), _p(table), _p(out), U32(indices.size), U32(table.shape[1]),
                            U32(table.shape[0]))
    return out


def add_f16(a, b):
    a, b = _f16(a), _f16(b)
    out = np.empty(a.shape, np.float16)
    lib().orc_add_f16(_p(a), _p(b), _p(out), ctypes.c_uint64(a.size))
    return out


def argmax_f16(values):
    values = _f16(values).reshape(-1)
    return int(lib().orc_argmax_f16(_p(values), I64(values.size)))


# ---- Q4_0 block family (lib/metal_q4_0_source.ml, lib/metal_quant_qkv_source.ml) ----

def q4_0_dequant(blocks):
    blocks = _u8(blocks).reshape(-1)
    total = blocks.size // 18
    out = np.empty((total * 32,), np.float16)
    lib().orc_q4_0_dequant(_p(blocks), _p(out), I64(total))
    return out


def q4_0_linear(x, weight, additive=None, mode=0):
    """weight: uint8 [n, (k/32)*18]; mode 0 none, 1 bias [n], 2 residual [m, n]."""
    x, weight = _f16(x), _u8(weight)
    m, k = x.shape
    n = weight.shape[0]
    y = np.empty((m, n), np.float16)
    lib().orc_q4_0_linear(_p(x), _p(weight), _p(None if additive is None else _f16(additive)), ctypes.c_int(mode),
                          _p(y), I64(m), I64(n), I64(k))
    return y


def q4_0_gated_linear(x, gate_weight, up_weight, activation=0):
    x = _f16(x)
    m, k = x.shape
    n = gate_weight.shape[0]
    product = np.empty((m, n), np.float16)
    lib().orc_q4_0_gated_linear(_p(x), _p(_u8(gate_weight)), _p(_u8(up_weight)), ctypes.c_int(activation),
                                _p(product), I64(m), I64(n), I64(k))
    return product


def sample_f16(logits, *, temperature, top_k, top_p, min_p, seed):
    """Restatement of the reference's host sampler (native/ocaml_metal_stubs.m:2629-2765)."""
    logits = _f16(logits).reshape(-1)
    function = lib().orc_sample_f16
    function.restype = ctypes.c_int64
    return int(function(_p(logits), I64(logits.size), F32(temperature), ctypes.c_int(top_k), F32(top_p), F32(min_p),
                        ctypes.c_uint64(seed)))


def norm_family(x, *, weight=None, residual=None, layer_scalar=None, epsilon, l2=False, groups=1, offset=0, width=None):
    """The RMS / L2 norm variants (lib/metal_normalization_source.ml:92-585): input f16 or f32,
    weight None / f16 / f32, optional half-precision residual add, optional layer scalar;
    ``groups`` / ``offset`` / ``width`` select the slice form."""
    x = np.ascontiguousarray(x)
    is_f32 = x.dtype == np.float32
    if not is_f32:
        x = _f16(x)
    input_rows, input_width = x.shape
    width = input_width if width is None else width
    rows = input_rows * groups
    kind = 0
    if weight is not None:
        weight = np.ascontiguousarray(weight)
        kind = 2 if weight.dtype == np.float32 else 1
        if kind == 1:
            weight = _f16(weight)
    out = np.empty((rows, width), np.float16)
    scalar = None if layer_scalar is None else np.asarray([layer_scalar], np.float32)
    lib().orc_norm_family(_p(x), ctypes.c_int(int(is_f32)), _p(weight), ctypes.c_int(kind),
                          _p(None if residual is None else _f16(residual)), _p(scalar), _p(out), I64(rows), I64(width),
                          F32(epsilon), ctypes.c_int(int(l2)), I64(groups), I64(input_width), I64(offset))
    return out


def rms_rope(x, weight, cosine, sine, *, half_dimension, epsilon, trig_batches=1):
    """x token-first [b,t,h,w] -> head-major [b,h,t,w]; weight f16 or f32 [w]."""
    x = _f16(x)
    b, t, h, w = x.shape
    weight = np.ascontiguousarray(weight)
    is_f32 = weight.dtype == np.float32
    out = np.empty((b, h, t, w), np.float16)
    lib().orc_rms_rope(_p(x), _p(weight if is_f32 else _f16(weight)), ctypes.c_int(int(is_f32)), _p(_f16(cosine)),
                       _p(_f16(sine)), _p(out), U32(b), U32(t), U32(h), U32(w), U32(half_dimension), U32(trig_batches),
                       F32(epsilon))
    return out


def rms_rope_qk(q, q_weight, k, k_weight, cosine, sine, *, half_dimension, epsilon, trig_batches=1):
    q, k = _f16(q), _f16(k)
    b, t, qh, w = q.shape
    kh = k.shape[2]
    q_weight, k_weight = np.ascontiguousarray(q_weight), np.ascontiguousarray(k_weight)
    is_f32 = q_weight.dtype == np.float32
    if not is_f32:
        q_weight, k_weight = _f16(q_weight), _f16(k_weight)
    q_out, k_out = np.empty((b, qh, t, w), np.float16), np.empty((b, kh, t, w), np.float16)
    lib().orc_rms_rope_qk(_p(q), _p(q_weight), _p(k), _p(k_weight), ctypes.c_int(int(is_f32)), _p(_f16(cosine)),
                          _p(_f16(sine)), _p(q_out), _p(k_out), U32(b), U32(t), U32(qh), U32(kh), U32(w),
                          U32(half_dimension), U32(trig_batches), F32(epsilon))
    return q_out, k_out


def gated_delta(query, key, value, gate, beta, *, token_major):
    """Cpu.gated_delta (lib/cpu.ml:909-976). token_major: f16 vectors [b,t,h,w], beta f16 [b,t,h];
    else f32 vectors [b,h,t,w], beta f32 [b,h,t]; gate f32. Output f16 [b,t,h,w]."""
    cast = _f16 if token_major else (lambda a: np.ascontiguousarray(a, dtype=np.float32))
    query, key, value, beta = cast(query), cast(key), cast(value), cast(beta)
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    if token_major:
        b, t, h, w = query.shape
    else:
        b, h, t, w = query.shape
    out = np.empty((b, t, h, w), np.float16)
    lib().orc_gated_delta(_p(query), _p(key), _p(value), _p(gate), _p(beta), _p(out), ctypes.c_int(int(token_major)),
                          I64(b), I64(h), I64(t), I64(w))
    return out


def triangular_recurrence(matrices, *, start, stop):
    """Cpu.triangular_recurrence (lib/cpu.ml:424-460) on f32 [outer, w, w]."""
    matrices = np.ascontiguousarray(matrices, dtype=np.float32)
    outer, width = int(np.prod(matrices.shape[:-2])), matrices.shape[-1]
    out = np.empty_like(matrices)
    lib().orc_triangular_recurrence(_p(matrices), _p(out), I64(outer), I64(width), I64(start), I64(stop))
    return out


def tile32_affine_linear(x, weight, *, bits, additive=None, mode=0):
    """weight: uint8 [n, (k/32) * (20 if bits == 4 else 36)] Tile32 affine blocks."""
    x, weight = _f16(x), _u8(weight)
    m, k = x.shape
    n = weight.shape[0]
    y = np.empty((m, n), np.float16)
    lib().orc_tile32_affine_linear(_p(x), _p(weight), _p(None if additive is None else _f16(additive)), ctypes.c_int(mode),
                                   ctypes.c_int(bits), _p(y), I64(m), I64(n), I64(k))
    return y


def tile32_affine_blocks(weight, *, bits):
    """Quantises fp32 [n, k] to Tile32 affine blocks (scale = range / (2^bits - 1), minimum = min
    of each 32-wide block, both stored as f16): test data in the storage format."""
    weight = np.asarray(weight, np.float32)
    n, k = weight.shape
    blocks = weight.reshape(n, k // 32, 32)
    low = blocks.min(-1).astype(np.float16)
    scale = ((blocks.max(-1) - low.astype(np.float32)) / (2 ** bits - 1)).astype(np.float16)
    safe = np.where(scale.astype(np.float32) > 0, scale.astype(np.float32), 1.0)
    codes = np.clip(np.rint((blocks - low.astype(np.float32)[..., None]) / safe[..., None]), 0, 2 ** bits - 1).astype(np.uint8)
    out = np.zeros((n, k // 32, 36 if bits == 8 else 20), np.uint8)
    out[..., 0:2] = scale.view(np.uint8).reshape(n, k // 32, 2)
    out[..., 2:4] = low.view(np.uint8).reshape(n, k // 32, 2)
    out[..., 4:] = codes if bits == 8 else (codes[..., :16] | (codes[..., 16:] << 4))
    return out.reshape(n, -1)


def cache_pack_attention_fwht(source, slots, pool, *, bits, segment_offset, heads, head_dim, token_stride,
                              source_items, source_offset=0):
    """Packs in place into ``pool`` (np.uint8, 1-D); source [heads, source_items, head_dim] f16."""
    source, slots = _f16(source), _u32(slots)
    lib().orc_cache_pack_attention_fwht(_p(source), _p(slots), _p(pool), ctypes.c_int(bits), U32(len(slots)),
                                        U32(segment_offset), U32(heads), U32(head_dim), U32(token_stride),
                                        U32(source_items), U32(source_offset))


def cache_unpack_attention_fwht(pool, slots, *, bits, segment_offset, heads, head_dim, token_stride):
    slots = _u32(slots)
    out = np.empty((heads, len(slots), head_dim), np.float16)
    lib().orc_cache_unpack_attention_fwht(_p(_u8(pool)), _p(slots), _p(out), ctypes.c_int(bits), U32(len(slots)),
                                          U32(segment_offset), U32(heads), U32(head_dim), U32(token_stride))
    return out
