"""GPU parity of the W4A16 group-64 family against the CPU oracle, through the
C ABI (kernel name + buffers + parameter bytes), as the reference dispatches it."""

import numpy as np
import pytest

from conftest import assert_close_f16, f16_bits
from helpers import random_w4

pytestmark = pytest.mark.gpu


def _ctx(runtime):
    from llmopt_b200 import dispatch

    return dispatch.Context(runtime)


def _tensor(runtime, array, dtype=None):
    from llmopt_b200 import dispatch
    from llmopt_b200.cuda_native import Buffer

    array = np.ascontiguousarray(array)
    names = {np.dtype(np.float16): "float16", np.dtype(np.uint8): "uint8", np.dtype(np.float32): "float32",
             np.dtype(np.int32): "int32", np.dtype(np.uint32): "uint32", np.dtype(np.int64): "int64"}
    return dispatch.Tensor(Buffer.of_array(runtime, array), tuple(array.shape), dtype or names[array.dtype])


def _linear(runtime, x, packed, scale, bias=None, stride=0):
    from llmopt_b200 import dispatch

    m, n = x.shape[0], packed.shape[0]
    out = _tensor(runtime, np.full((m, n), np.nan, np.float16))  # NaN sentinel: every element must be written
    dispatch.dispatch_w4a16_linear(_ctx(runtime), input=_tensor(runtime, x), weight=_tensor(runtime, packed),
                                   scale=_tensor(runtime, scale), output=out,
                                   bias=None if bias is None else _tensor(runtime, bias), bias_row_stride=stride)
    return out.buffer.to_numpy(np.float16, (m, n))


def test_reference_fixture_bits(runtime):
    # python/examples/write_w4a16_weight_fixture.py:11-23, bin/ocaml_metal_smoke.ml:184-236
    packed = np.arange(96, dtype=np.uint8).reshape(3, 32).copy()
    packed[0, 0] = 0x78
    scale = np.array([[0.125], [0.25], [0.5]], np.float16)
    bias = np.array([0.5, 1.0, -1.0], np.float16)
    y = _linear(runtime, np.ones((2, 64), np.float16), packed, scale, bias)
    assert y.view(np.uint16).reshape(-1).tolist() == [0x3600, 0x4C40, 0x53E0] * 2


def test_tail_columns_exact(runtime, oracle):
    # python/examples/metal_runtime_smoke.py:28-74: M=3, N=29, K=64, bytes 0x11 / 0xFF, exact equality
    packed = np.empty((29, 32), np.uint8)
    packed[0::2] = 0x11
    packed[1::2] = 0xFF
    scale = np.full((29, 1), 0.5, np.float16)
    x = np.ones((3, 64), np.float16)
    bias = np.arange(29, dtype=np.float16)
    for b in (None, bias):
        got = _linear(runtime, x, packed, scale, b)
        want = oracle.w4a16_linear(x, packed, scale, b, 0)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,k,n", [(1, 576, 1536), (128, 576, 1536), (1, 64, 16), (2, 128, 17), (5, 1024, 333),
                                   (8, 4096, 512), (9, 1536, 576), (17, 2048, 256), (33, 576, 192), (64, 1024, 128),
                                   (70, 256, 96)])
def test_linear_matches_oracle(runtime, oracle, m, k, n):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    got = _linear(runtime, x, packed, scale)
    want = oracle.w4a16_linear(x, packed, scale)
    assert_close_f16(got, want, label=f"linear m={m} k={k} n={n}")


def test_dyadic_inputs_are_bit_exact(runtime, oracle):
    # Dyadic activations and scales make fp32 accumulation order-independent, so the
    # GPU result must equal the float64 oracle bit for bit (the reference's probe method).
    rng = np.random.default_rng(1)
    m, k, n = 4, 1024, 96
    x = (rng.integers(-8, 9, size=(m, k)) / 8.0).astype(np.float16)
    packed, _ = random_w4(rng, n, k)
    scale = (2.0 ** rng.integers(-6, -2, size=(n, k // 64))).astype(np.float16)
    got = _linear(runtime, x, packed, scale)
    want = oracle.w4a16_linear(x, packed, scale)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_bias_and_row_residual(runtime, oracle):
    rng = np.random.default_rng(2)
    m, k, n = 3, 576, 576
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    bias = rng.standard_normal(n).astype(np.float16)
    residual = rng.standard_normal((m, n)).astype(np.float16)
    assert_close_f16(_linear(runtime, x, packed, scale, bias, 0), oracle.w4a16_linear(x, packed, scale, bias, 0))
    assert_close_f16(_linear(runtime, x, packed, scale, residual, n), oracle.w4a16_linear(x, packed, scale, residual, n))


def test_affine_zero_point_mode(runtime, oracle):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(0)
    for m in (1, 128):
        k, n = 576, 1536
        x = rng.standard_normal((m, k)).astype(np.float16)
        packed, scale = random_w4(rng, n, k)
        zero = rng.uniform(6, 9, size=(n, k // 64)).astype(np.float16)
        out = _tensor(runtime, np.full((m, n), np.nan, np.float16))
        dispatch.dispatch_w4a16_linear_affine(_ctx(runtime), input=_tensor(runtime, x), weight=_tensor(runtime, packed),
                                              scale=_tensor(runtime, scale), zero=_tensor(runtime, zero), output=out)
        got = out.buffer.to_numpy(np.float16, (m, n))
        assert_close_f16(got, oracle.w4a16_linear(x, packed, scale, zero=zero), label=f"affine m={m}")


@pytest.mark.parametrize("m,k,nq,nk,nv", [(1, 576, 576, 192, 192), (4, 1024, 1024, 512, 512), (1, 128, 40, 24, 8)])
def test_qkv_matches_oracle(runtime, oracle, m, k, nq, nk, nv):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, k)).astype(np.float16)
    weights = [random_w4(rng, n, k) for n in (nq, nk, nv)]
    outs = [_tensor(runtime, np.full((m, n), np.nan, np.float16)) for n in (nq, nk, nv)]
    dispatch.dispatch_w4a16_qkv_linear_command(
        _ctx(runtime), input=_tensor(runtime, x), q_weight=_tensor(runtime, weights[0][0]),
        q_scale=_tensor(runtime, weights[0][1]), k_weight=_tensor(runtime, weights[1][0]),
        k_scale=_tensor(runtime, weights[1][1]), v_weight=_tensor(runtime, weights[2][0]),
        v_scale=_tensor(runtime, weights[2][1]), q_output=outs[0], k_output=outs[1], v_output=outs[2])
    want = oracle.w4a16_qkv_linear(x, weights[0][0], weights[0][1], weights[1][0], weights[1][1], weights[2][0],
                                   weights[2][1])
    for out, expected, n in zip(outs, want, (nq, nk, nv)):
        assert_close_f16(out.buffer.to_numpy(np.float16, (m, n)), expected, label="qkv")


@pytest.mark.parametrize("m,k,n,f32", [(1, 576, 1536, False), (3, 1024, 4608, False), (1, 576, 1536, True),
                                       (6, 128, 192, False)])
def test_swiglu_ffn_matches_oracle(runtime, oracle, m, k, n, f32):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(4)
    activation = rng.standard_normal((m, k)).astype(np.float32 if f32 else np.float16)
    residual = rng.standard_normal((m, k)).astype(np.float16)
    gate, up, down = random_w4(rng, n, k), random_w4(rng, n, k), random_w4(rng, k, n)
    norm = rng.uniform(0.5, 1.5, size=k).astype(np.float16)
    out = _tensor(runtime, np.full((m, k), np.nan, np.float16))
    context = _ctx(runtime)
    kernels = dispatch.dispatch_w4a16_swiglu_ffn_command(
        context, m=m, n=n, k=k, epsilon=1e-5, activation=_tensor(runtime, activation),
        residual=_tensor(runtime, residual), gate_weight=_tensor(runtime, gate[0]), gate_scale=_tensor(runtime, gate[1]),
        up_weight=_tensor(runtime, up[0]), up_scale=_tensor(runtime, up[1]), down_weight=_tensor(runtime, down[0]),
        down_scale=_tensor(runtime, down[1]), norm_weight=_tensor(runtime, norm), output=out)
    assert len(kernels) == 3 and kernels[0].startswith("llmopt_w4a16_swiglu_rms")
    want, want_normalized, _ = oracle.w4a16_swiglu_ffn(activation, residual, gate[0], gate[1], up[0], up[1], down[0],
                                                       down[1], norm, 1e-5)
    # Stage by stage, each linear against the oracle fed with the rows the GPU gave the stage: the
    # reference's bound of 2e-3 per linear.  The chained triple adds the stages' roundings to half
    # (normalised rows, SwiGLU product) as seen through the next stage, hence the wider end-to-end bound.
    batch = context.execution_batch
    got_normalized = batch.swiglu_normalized.to_numpy(np.float16, (m, k))
    got_product = batch.swiglu_product.to_numpy(np.float16, (m, n))
    got = out.buffer.to_numpy(np.float16, (m, k))
    assert_close_f16(got_normalized, want_normalized, rel=1e-3, label="swiglu ffn: normalised rows")
    assert_close_f16(got_product, oracle.w4a16_dual_swiglu(got_normalized, gate[0], gate[1], up[0], up[1]), rel=2e-3,
                     label="swiglu ffn: gate/up product")
    assert_close_f16(got, oracle.w4a16_linear(got_product, down[0], down[1], residual, k), rel=2e-3,
                     label="swiglu ffn: down + residual")
    assert_close_f16(got, want, rel=3e-3, label="swiglu ffn, chained")


@pytest.mark.parametrize("tag", ["none", "bias", "silu", "gelu", "silu_mul", "gelu_mul", "residual_add",
                                 "bias_residual_add", "silu_mul_residual_add", "gelu_mul_residual_add"])
def test_tagged_epilogues(runtime, oracle, tag):
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer, DispatchItem

    rng = np.random.default_rng(5)
    m, k, n = 1, 576, 320
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    operands = {"none": 0, "silu": 0, "gelu": 0}.get(tag, 2 if tag.count("_") >= 2 and tag != "residual_add" else 1)
    if tag in ("bias_residual_add", "silu_mul_residual_add", "gelu_mul_residual_add"):
        operands = 2
    elif tag in ("bias", "silu_mul", "gelu_mul", "residual_add"):
        operands = 1
    extra = [rng.standard_normal(n).astype(np.float16) for _ in range(operands)]
    out = Buffer.of_array(runtime, np.full((m, n), np.nan, np.float16))
    buffers = [Buffer.of_array(runtime, a) for a in (x, packed, scale, scale)] + [out] + [Buffer.of_array(runtime, e) for e in extra]
    runtime.dispatch("llmopt_w4a16_linear_f16_g64_epi_" + tag, buffers=buffers,
                     parameters=parameters.w4a16_linear(m=m, n=n, k=k, has_bias=False, bias_row_stride=0),
                     grid=(n * 32, 1, 1))
    want = oracle.w4a16_linear_epilogue(x, packed, scale, tag, *(extra + [None, None])[:2])
    assert_close_f16(out.to_numpy(np.float16, (m, n)), want, label=tag)


@pytest.mark.parametrize("m,k,n,f32,two_stage,logits", [(1, 576, 4096, False, True, False), (2, 1024, 3000, False, False, True),
                                                         (1, 576, 49152, True, True, True), (5, 128, 777, False, True, False),
                                                         (32, 1024, 32768, False, True, True), (20, 576, 49152, True, True, False)])  # 17..32 rows: one tensor-core pass
def test_lm_head_argmax(runtime, oracle, m, k, n, f32, two_stage, logits):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(6)
    x = rng.standard_normal((m, k)).astype(np.float32 if f32 else np.float16)
    norm = rng.uniform(0.5, 1.5, size=k).astype(np.float16)
    weight, scale = random_w4(rng, n, k)
    tokens = _tensor(runtime, np.full((m,), -1, np.int32))
    logit_tensor = _tensor(runtime, np.full((m, n), np.nan, np.float16)) if logits else None
    dispatch.dispatch_w4a16_lm_head_argmax_command(
        _ctx(runtime), m=m, n=n, k=k, epsilon=1e-5, input=_tensor(runtime, x), norm_weight=_tensor(runtime, norm),
        weight=_tensor(runtime, weight), scale=_tensor(runtime, scale), output=tokens, logits=logit_tensor,
        two_stage=two_stage)
    want_tokens, want_logits, _ = oracle.w4a16_lm_head_argmax(x, norm, weight, scale, 1e-5, want_logits=True)
    got_tokens = tokens.buffer.to_numpy(np.int32)
    exact = oracle.w4a16_linear_f64(oracle.rms_norm(x, norm, 1e-5), weight, scale)  # only for a tie diagnosis
    for row in range(m):
        if got_tokens[row] != want_tokens[row]:
            gap = abs(float(want_logits[row, got_tokens[row]]) - float(want_logits[row, want_tokens[row]]))
            raise AssertionError(f"row {row}: token {got_tokens[row]} != {want_tokens[row]} (logit gap {gap}, {exact.shape})")
    if logits:
        assert_close_f16(logit_tensor.buffer.to_numpy(np.float16, (m, n)), want_logits, label="lm head logits")


def test_lm_head_tie_breaks_to_lowest_index(runtime):
    from llmopt_b200 import dispatch

    k, n = 64, 512
    x = np.ones((1, k), np.float16)
    norm = np.ones(k, np.float16)
    weight = np.full((n, k // 2), 0x11, np.uint8)  # every column identical -> all logits tie
    scale = np.full((n, 1), 0.5, np.float16)
    tokens = _tensor(runtime, np.full((1,), -1, np.int32))
    dispatch.dispatch_w4a16_lm_head_argmax_command(
        _ctx(runtime), m=1, n=n, k=k, epsilon=1e-5, input=_tensor(runtime, x), norm_weight=_tensor(runtime, norm),
        weight=_tensor(runtime, weight), scale=_tensor(runtime, scale), output=tokens)
    assert tokens.buffer.to_numpy(np.int32)[0] == 0


def test_python_single_op_boundary(runtime, oracle):
    # the native/metal_runtime.cpp entry on raw device pointers
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(7)
    m, k, n = 3, 64, 29
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    bias = rng.standard_normal(n).astype(np.float16)
    bufs = [Buffer.of_array(runtime, a) for a in (x, packed, scale, bias)]
    out = Buffer.of_array(runtime, np.full((m, n), np.nan, np.float16))
    runtime.w4a16_linear_pointers(bufs[0].device_pointer(), bufs[1].device_pointer(), bufs[2].device_pointer(),
                                  bufs[3].device_pointer(), out.device_pointer(), m, n, k)
    runtime.synchronize()
    assert_close_f16(out.to_numpy(np.float16, (m, n)), oracle.w4a16_linear(x, packed, scale, bias, 0))
    with pytest.raises(ValueError):
        runtime.w4a16_linear_pointers(bufs[0].device_pointer(), bufs[1].device_pointer(), bufs[2].device_pointer(),
                                      None, out.device_pointer(), m, n, 65)


def test_dispatch_errors(runtime):
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer, NativeError

    small = Buffer.create(runtime, 64)
    with pytest.raises(NativeError, match="missing"):
        runtime.dispatch("llmopt_no_such_kernel", buffers=[small], parameters=b"", grid=(1, 1, 1))
    with pytest.raises(NativeError, match="too short"):
        runtime.dispatch("llmopt_w4a16_linear_f16_g64", buffers=[small] * 5,
                         parameters=parameters.w4a16_linear(m=1, n=64, k=64, has_bias=False, bias_row_stride=0),
                         grid=(64 * 32, 1, 1))
    with pytest.raises(NativeError, match="parameter bytes"):
        runtime.dispatch("llmopt_w4a16_linear_f16_g64", buffers=[small] * 5, parameters=b"\0" * 8, grid=(32, 1, 1))
    with pytest.raises(ValueError, match="grid"):
        runtime.dispatch("llmopt_w4a16_linear_f16_g64", buffers=[small] * 5, parameters=b"\0" * 20, grid=(0, 1, 1))
    with pytest.raises(ValueError):
        small.view(32, 64)


def test_digest_named_epilogue_kernels(runtime, oracle):
    """A compiled package names an algebraic epilogue kernel by digest
    (base_<8 hex of MD5(dtypes | writeback)>, lib/epilogue.ml:217-229).  epilogue.bind makes such a
    name resolve: to the built-in tagged kernel when the expression is one of the ten forms, else to
    a registered expression program run by the interpreter kernel."""
    from llmopt_b200 import epilogue as ep, parameters
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(21)
    m, k, n = 3, 1024, 200
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    up = rng.standard_normal(n).astype(np.float16)
    ceiling = rng.uniform(0.2, 2.0, size=n).astype(np.float32)
    base = "llmopt_w4a16_linear_f16_g64"
    buffers = [Buffer.of_array(runtime, a) for a in (x, packed, scale)]
    block = parameters.w4a16_linear(m=m, n=n, k=k, has_bias=False, bias_row_stride=0)
    acc = oracle.w4a16_linear_f64(x, packed, scale)

    def run(name, operands):
        out = Buffer.of_array(runtime, np.full((m, n), np.nan, np.float16))
        runtime.dispatch(name, buffers=buffers + [buffers[2], out] + [Buffer.of_array(runtime, a) for a in operands],
                         parameters=block, grid=(256, 1, 1))
        return out.to_numpy(np.float16, (m, n))

    # a tagged form under its digest name: an alias of the built-in kernel, bit-identical to it
    gated = ep.of_expr(ep.Binop("mul", ep.Unop("silu", ep.ACC), ep.Read(ep.Value(17))))
    name = ep.bind(runtime, base, gated)
    assert name == ep.algebraic_kernel_name(base, ep.tagged("silu_mul", ep.Value(0))) and runtime.has_function(name)
    assert np.array_equal(run(name, [up]).view(np.uint16), run(base + "_epi_silu_mul", [up]).view(np.uint16))
    want = (acc / (1 + np.exp(-acc))) * up.astype(np.float64)
    assert_close_f16(run(name, [up]), want, label="digest-named silu_mul")
    # a free-form tree: clamp(silu(acc) * up + 0.5, -1, ceiling) with an fp32 operand
    tree = ep.Triop("clamp", ep.Binop("add", ep.Binop("mul", ep.Unop("silu", ep.ACC), ep.Read(ep.Value(4))), ep.Const(0.5)),
                    ep.Const(-1.0), ep.Read(ep.Value(9, "f32")))
    free = ep.of_expr(tree)
    assert ep.matching_tag(free) is None
    name = ep.bind(runtime, base, free)
    assert runtime.has_function(name) and ep.bind(runtime, base, free) == name  # binding twice is harmless
    want = np.clip(want + 0.5, -1.0, ceiling.astype(np.float64))
    assert_close_f16(run(name, [up, ceiling]), want, label="expression epilogue")
    # a program that pops an empty stack is refused at registration
    with pytest.raises(ValueError, match="empty stack"):
        runtime.register_expr_epilogue("llmopt_w4a16_linear_f16_g64_deadbeef", bytes([20]), 0)
