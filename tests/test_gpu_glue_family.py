"""The non-quantised glue kernels a compiled decode list names around the hot path — RMS / L2 norm
variants, fused RMS norm + rotary, casts, broadcasting pointwise kernels — through the C ABI,
against the CPU oracle (norms, norm + rotary) or the same arithmetic in numpy (casts, pointwise:
one operation per element, each rounded to its storage type)."""

import numpy as np
import pytest

from conftest import assert_close_f16

pytestmark = pytest.mark.gpu


def _buf(runtime, array):
    from llmopt_b200.cuda_native import Buffer

    return Buffer.of_array(runtime, np.ascontiguousarray(array))


def _out(runtime, shape, dtype=np.float16):
    return _buf(runtime, np.full(shape, np.nan, dtype))


@pytest.mark.parametrize("rows,width", [(1, 576), (5, 1024), (3, 4096), (2, 100)])
def test_rms_norm_variants_match_oracle(runtime, oracle, rows, width):
    from llmopt_b200 import parameters

    rng = np.random.default_rng(rows * 1000 + width)
    x = rng.standard_normal((rows, width)).astype(np.float16)
    x32 = rng.standard_normal((rows, width)).astype(np.float32)
    w32 = rng.uniform(0.5, 1.5, size=width).astype(np.float32)
    residual = rng.standard_normal((rows, width)).astype(np.float16)
    scalar = np.array([0.731], np.float32)
    block = parameters.rms_norm(rows=rows, width=width, epsilon=1e-5)
    cases = [
        ("llmopt_rms_norm_f32_f16_wf32_simd", [x32, w32], dict(weight=w32), x32),
        ("llmopt_rms_norm_f16_wf32_simd", [x, w32], dict(weight=w32), x),
        ("llmopt_rms_norm_f16_wf32_wide", [x, w32], dict(weight=w32), x),
        ("llmopt_rms_norm_add_f16_wf32_simd", [x, w32, residual], dict(weight=w32, residual=residual), x),
        ("llmopt_rms_norm_add_f16_wf32_wide", [x, w32, residual], dict(weight=w32, residual=residual), x),
        ("llmopt_rms_norm_scale_f16_wf32_simd", [x, w32, scalar], dict(weight=w32, layer_scalar=scalar[0]), x),
        ("llmopt_rms_norm_add_scale_f16_wf32_wide", [x, w32, residual, scalar],
         dict(weight=w32, residual=residual, layer_scalar=scalar[0]), x),
        ("llmopt_rms_norm_unweighted_f16_simd", [x], dict(), x),
        ("llmopt_rms_norm_unweighted_add_f16_wide", [x, residual], dict(residual=residual), x),
        ("llmopt_l2_norm_f16_simd", [x], dict(l2=True), x),
    ]
    for name, inputs, fields, source in cases:
        assert runtime.has_function(name), name
        out = _out(runtime, (rows, width))
        runtime.dispatch(name, buffers=[_buf(runtime, a) for a in inputs] + [out], parameters=block, grid=(256, 1, 1))
        want = oracle.norm_family(source, epsilon=1e-5, **fields)
        assert_close_f16(out.to_numpy(np.float16, (rows, width)), want, rel=1e-3, label=name)
    # the slice form: two slices of 64 columns starting at column 32 of rows 256 wide
    wide = rng.standard_normal((rows, 256)).astype(np.float16)
    out = _out(runtime, (rows * 2, 64))
    runtime.dispatch("llmopt_l2_norm_slice_f16_simd", buffers=[_buf(runtime, wide), out],
                     parameters=parameters.l2_norm_slice(input_rows=rows, groups=2, width=64, input_width=256, offset=32,
                                                         epsilon=1e-6), grid=(256, 1, 1))
    want = oracle.norm_family(wide, epsilon=1e-6, l2=True, groups=2, offset=32, width=64)
    assert_close_f16(out.to_numpy(np.float16, (rows * 2, 64)), want, rel=1e-3, label="l2 slice")
    with pytest.raises(Exception, match="outside the input row"):
        runtime.dispatch("llmopt_l2_norm_slice_f16_simd", buffers=[_buf(runtime, wide), out],
                         parameters=parameters.l2_norm_slice(input_rows=rows, groups=2, width=128, input_width=256,
                                                             offset=32, epsilon=1e-6), grid=(256, 1, 1))


@pytest.mark.parametrize("weight_dtype", [np.float16, np.float32])
def test_rms_rope_and_rms_rope_qk_match_oracle(runtime, oracle, weight_dtype):
    from llmopt_b200 import parameters

    rng = np.random.default_rng(5)
    b, t, qh, kh, d = 2, 3, 4, 2, 64
    q = rng.standard_normal((b, t, qh, d)).astype(np.float16)
    k = rng.standard_normal((b, t, kh, d)).astype(np.float16)
    qw = rng.uniform(0.5, 1.5, size=d).astype(weight_dtype)
    kw = rng.uniform(0.5, 1.5, size=d).astype(weight_dtype)
    angle = rng.uniform(0, 6.28, size=(1, t, d)).astype(np.float32)
    cos, sin = np.cos(angle).astype(np.float16), np.sin(angle).astype(np.float16)
    suffix = "_simd_h64" if weight_dtype == np.float16 else "_wf32_simd"
    out = _out(runtime, (b, qh, t, d))
    runtime.dispatch("llmopt_rms_rope_f16" + suffix,
                     buffers=[_buf(runtime, q), _buf(runtime, qw), _buf(runtime, cos), _buf(runtime, sin), out],
                     parameters=parameters.rms_rope(batches=b, tokens=t, heads=qh, width=d, half_dimension=d // 2,
                                                    trig_batches=1, epsilon=1e-6), grid=(256, 1, 1))
    want = oracle.rms_rope(q, qw, cos, sin, half_dimension=d // 2, epsilon=1e-6)
    assert_close_f16(out.to_numpy(np.float16, want.shape), want, rel=2e-3, label="rms_rope")
    q_out, k_out = _out(runtime, (b, qh, t, d)), _out(runtime, (b, kh, t, d))
    runtime.dispatch("llmopt_rms_rope_qk_f16" + suffix,
                     buffers=[_buf(runtime, q), _buf(runtime, qw), _buf(runtime, k), _buf(runtime, kw), _buf(runtime, cos),
                              _buf(runtime, sin), q_out, k_out],
                     parameters=parameters.rms_rope_qk(batches=b, tokens=t, q_heads=qh, k_heads=kh, width=d,
                                                       half_dimension=d // 2, trig_batches=1, epsilon=1e-6),
                     grid=(256, 1, 1))
    want_q, want_k = oracle.rms_rope_qk(q, qw, k, kw, cos, sin, half_dimension=d // 2, epsilon=1e-6)
    assert_close_f16(q_out.to_numpy(np.float16, want_q.shape), want_q, rel=2e-3, label="rms_rope_qk q")
    assert_close_f16(k_out.to_numpy(np.float16, want_k.shape), want_k, rel=2e-3, label="rms_rope_qk k")


def test_casts_and_pointwise_kernels(runtime):
    from llmopt_b200 import parameters

    rng = np.random.default_rng(9)
    h = rng.standard_normal(1000).astype(np.float16)
    f = (rng.standard_normal(1000) * 100).astype(np.float32)
    ints = rng.integers(-2 ** 40, 2 ** 40, size=1000)
    for name, source, dtype, want in (("llmopt_cast_f16_f32", h, np.float32, h.astype(np.float32)),
                                      ("llmopt_cast_f32_f16", f, np.float16, f.astype(np.float16)),
                                      ("llmopt_cast_i64_f32", ints, np.float32, ints.astype(np.float32))):
        out = _out(runtime, 1000, dtype)
        runtime.dispatch(name, buffers=[_buf(runtime, source), out], parameters=parameters.count(count=1000),
                         grid=(1000, 1, 1))
        assert np.array_equal(out.to_numpy(dtype), want), name
    # broadcasting binary kernels: [2, 3, 8] op [3, 1] and op scalar, bit-exact in half / float
    left = rng.standard_normal((2, 3, 8)).astype(np.float16)
    right = rng.standard_normal((3, 1)).astype(np.float16)
    f32 = lambda a: a.astype(np.float32)
    silu = lambda a: (f32(a) / (np.float32(1) + np.exp(-f32(a)))).astype(np.float16)
    sigmoid = lambda a: (np.float32(1) / (np.float32(1) + np.exp(-f32(a)))).astype(np.float16)
    expected = {
        "llmopt_add_f16": (left + right, True), "llmopt_mul_f16": (left * right, True),
        "llmopt_div_f16": ((f32(left) / f32(right)).astype(np.float16), True),
        "llmopt_silu_mul_f16": (silu(left) * right, False), "llmopt_sigmoid_mul_f16": (sigmoid(left) * right, False),
    }
    block = parameters.pointwise(output_shape=(2, 3, 8), left_shape=(2, 3, 8), right_shape=(3, 1))
    assert len(block) == 136
    for name, (want, exact) in expected.items():
        out = _out(runtime, (2, 3, 8))
        runtime.dispatch(name, buffers=[_buf(runtime, left), _buf(runtime, right), out], parameters=block, grid=(48, 1, 1))
        got = out.to_numpy(np.float16, (2, 3, 8))
        if exact:
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), name
        else:  # expf differs from numpy's exp by an ulp now and then
            assert_close_f16(got, want, rel=1e-3, label=name)
    out = _out(runtime, (2, 3, 8))
    runtime.dispatch("llmopt_mul_f16", buffers=[_buf(runtime, left), _buf(runtime, left), out],
                     parameters=parameters.pointwise(output_shape=(2, 3, 8), left_shape=(2, 3, 8), right_scalar=0.5),
                     grid=(48, 1, 1))
    assert np.array_equal(out.to_numpy(np.float16, (2, 3, 8)).view(np.uint16), (left * np.float16(0.5)).view(np.uint16))
    a32, b32 = rng.standard_normal((4, 5)).astype(np.float32), rng.standard_normal((1, 5)).astype(np.float32)
    for name, want in (("llmopt_add_f32", a32 + b32), ("llmopt_sub_f32", a32 - b32), ("llmopt_mul_f32", a32 * b32)):
        out = _out(runtime, (4, 5), np.float32)
        runtime.dispatch(name, buffers=[_buf(runtime, a32), _buf(runtime, b32), out],
                         parameters=parameters.pointwise(output_shape=(4, 5), left_shape=(4, 5), right_shape=(1, 5)),
                         grid=(20, 1, 1))
        assert np.array_equal(out.to_numpy(np.float32, (4, 5)), want), name
    # mixed multiplies
    hl = rng.standard_normal((4, 5)).astype(np.float16)
    for name, l, r, dtype, want in (
            ("llmopt_mul_f16_f32", hl, b32, np.float32, f32(hl) * b32),
            ("llmopt_mul_f16_f32_f16", hl, b32, np.float16, (f32(hl) * b32).astype(np.float16)),
            ("llmopt_mul_f32_f16_f16", a32, hl[:1], np.float16, (a32 * f32(hl[:1])).astype(np.float16))):
        out = _out(runtime, (4, 5), dtype)
        runtime.dispatch(name, buffers=[_buf(runtime, l), _buf(runtime, r), out],
                         parameters=parameters.pointwise(output_shape=(4, 5), left_shape=l.shape, right_shape=r.shape),
                         grid=(20, 1, 1))
        assert np.array_equal(out.to_numpy(dtype, (4, 5)), want), name
    # unary
    out = _out(runtime, 1000)
    runtime.dispatch("llmopt_neg_f16", buffers=[_buf(runtime, h), out], parameters=parameters.count(count=1000), grid=(1000, 1, 1))
    assert np.array_equal(out.to_numpy(np.float16).view(np.uint16), (-h).view(np.uint16))
    runtime.dispatch("llmopt_silu_f16", buffers=[_buf(runtime, h), out], parameters=parameters.count(count=1000), grid=(1000, 1, 1))
    assert_close_f16(out.to_numpy(np.float16), silu(h), rel=1e-3, label="silu")
    # a shape that does not broadcast is refused on the host
    with pytest.raises(Exception, match="broadcast"):
        bad = bytearray(block)
        bad[48 + 4:48 + 8] = (2).to_bytes(4, "little")  # left_shape[1] = 2 against output 3
        runtime.dispatch("llmopt_add_f16", buffers=[_buf(runtime, left), _buf(runtime, right), out], parameters=bytes(bad),
                         grid=(48, 1, 1))


@pytest.mark.parametrize("token_major,width,tokens", [(False, 64, 40), (True, 128, 33), (True, 32, 5), (False, 256, 9)])
def test_gated_delta_matches_oracle(runtime, oracle, token_major, width, tokens):
    """Gated-delta scan against the CPU statement (lib/cpu.ml:909-976) in float64: fp16 output,
    fp32 state kept in registers over the whole scan."""
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(width + tokens)
    batch, heads = 2, 3
    dtype, name = (np.float16, "float16") if token_major else (np.float32, "float32")
    shape = (batch, tokens, heads, width) if token_major else (batch, heads, tokens, width)
    scalars = shape[:3]
    # unit-norm keys and queries, decays below one, betas in (0, 1): the regime the scan is used in
    unit = lambda a: a / np.linalg.norm(a, axis=-1, keepdims=True)
    query = unit(rng.standard_normal(shape)).astype(dtype)
    key = unit(rng.standard_normal(shape)).astype(dtype)
    value = rng.standard_normal(shape).astype(dtype)
    gate = -rng.uniform(0.01, 0.5, size=scalars).astype(np.float32)
    beta = rng.uniform(0.1, 0.9, size=scalars).astype(dtype)
    tensor = lambda a, d: dispatch.Tensor(_buf(runtime, a), a.shape, d)
    out = dispatch.Tensor(_out(runtime, (batch, tokens, heads, width)), (batch, tokens, heads, width), "float16")
    names = dispatch.dispatch_gated_delta(dispatch.Context(runtime), query=tensor(query, name), key=tensor(key, name),
                                          value=tensor(value, name), gate=tensor(gate, "float32"),
                                          beta=tensor(beta, name), output=out)
    assert names == [("llmopt_gated_delta_tm_f16_d" if token_major else "llmopt_gated_delta_f32_d") + str(width)]
    want = oracle.gated_delta(query, key, value, gate, beta, token_major=token_major)
    assert_close_f16(out.buffer.to_numpy(np.float16, want.shape), want, rel=2e-3, label=names[0])


def test_triangular_recurrence_is_bit_exact(runtime, oracle):
    """Every product and partial sum of the recurrence is rounded to fp32 on its own, in a fixed
    order, in the reference's CPU statement and kernel alike (lib/cpu.ml:424-460,
    lib/metal_recurrent_source.ml:290-299): results are compared bit for bit."""
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(3)
    for outer, width, start, stop in ((3, 64, 1, 64), (2, 33, 0, 20), (1, 1, 0, 1)):
        matrices = (rng.standard_normal((outer, width, width)) * 0.2).astype(np.float32)
        out = dispatch.Tensor(_out(runtime, matrices.shape, np.float32), matrices.shape, "float32")
        dispatch.dispatch_triangular_recurrence(dispatch.Context(runtime), start=start, stop=stop,
                                                input=dispatch.Tensor(_buf(runtime, matrices), matrices.shape, "float32"),
                                                output=out)
        want = oracle.triangular_recurrence(matrices, start=start, stop=stop)
        assert np.array_equal(out.buffer.to_numpy(np.float32, matrices.shape).view(np.uint32), want.view(np.uint32))


def test_a_package_declaring_every_entry_validates_against_the_library(runtime):
    """Package validation as the reference's loader does it (lib/metal_native.ml:271-285): every
    kernel entry point a package declares must resolve in the loaded library.  The package here
    declares the whole entry table, written and read back through the package.llmopt envelope."""
    from llmopt_b200 import kernel_abi, serving_package as sp

    tagged = [entry for entry in kernel_abi.ENTRIES
              if entry.operation in sp._OPERATION_OF and entry.input_dtype in sp._DTYPE_OF and entry.output_dtype in sp._DTYPE_OF]
    assert len(tagged) > 150
    package = sp.of_bytes(sp.Package("compiled-graph", "model.metallib", tagged).to_bytes())
    package.validate_declared_functions(runtime)
    missing = [entry.name for entry in kernel_abi.ENTRIES if not runtime.has_function(entry.name)]
    assert not missing, missing
    with pytest.raises(sp.PackageError, match="does not define declared kernel"):
        sp.Package("compiled-graph", "model.metallib",
                   [kernel_abi.Entry("llmopt_no_such_kernel", kernel_abi.LINEAR, "float16", "float16")]
                   ).validate_declared_functions(runtime)
