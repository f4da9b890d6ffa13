"""GPU parity of the prefill (M >= 64) W4A16 product, which runs on the tcgen05 /
tensor-memory path, against the CPU oracle through the same named dispatches."""

import numpy as np
import pytest

from conftest import assert_close_f16
from helpers import random_w4
from test_gpu_w4a16 import _ctx, _linear, _tensor

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n", [(64, 64, 256), (128, 128, 256), (128, 576, 1536), (200, 320, 512),
                                   (128, 256, 320), (65, 192, 40), (512, 1024, 768), (300, 2048, 1000)])
def test_prefill_linear_matches_oracle(runtime, oracle, m, k, n):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    got = _linear(runtime, x, packed, scale)
    want = oracle.w4a16_linear(x, packed, scale)
    assert_close_f16(got, want, label=f"prefill linear m={m} k={k} n={n}")


def test_prefill_dyadic_inputs_are_bit_exact(runtime, oracle):
    # dyadic activations and power-of-two scales: every product and partial sum is exact in
    # fp16 operands / fp32 accumulation, so the result equals the float64 oracle bit for bit
    rng = np.random.default_rng(11)
    m, k, n = 128, 512, 256
    x = (rng.integers(-8, 9, size=(m, k)) / 8.0).astype(np.float16)
    packed, _ = random_w4(rng, n, k)
    scale = (2.0 ** rng.integers(-6, -2, size=(n, k // 64))).astype(np.float16)
    got = _linear(runtime, x, packed, scale)
    want = oracle.w4a16_linear(x, packed, scale)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_prefill_bias_and_row_residual(runtime, oracle):
    rng = np.random.default_rng(12)
    m, k, n = 130, 576, 576
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    bias = rng.standard_normal(n).astype(np.float16)
    residual = rng.standard_normal((m, n)).astype(np.float16)
    assert_close_f16(_linear(runtime, x, packed, scale, bias, 0), oracle.w4a16_linear(x, packed, scale, bias, 0))
    assert_close_f16(_linear(runtime, x, packed, scale, residual, n), oracle.w4a16_linear(x, packed, scale, residual, n))


@pytest.mark.parametrize("m,k,n", [(256, 576, 1536), (100, 1024, 384), (300, 512, 100), (64, 576, 1536)])
def test_prefill_affine_zero_points(runtime, oracle, m, k, n):
    """Unsigned nibbles with fp16 zero points at prompt rows: 256-token tiles, 128-token pairs of weight
    tiles, a single narrow tile, and 64 rows (the shared-memory-operand GEMM)."""
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(13)
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    zero = rng.uniform(6, 9, size=(n, k // 64)).astype(np.float16)
    out = _tensor(runtime, np.full((m, n), np.nan, np.float16))
    dispatch.dispatch_w4a16_linear_affine(_ctx(runtime), input=_tensor(runtime, x), weight=_tensor(runtime, packed),
                                          scale=_tensor(runtime, scale), zero=_tensor(runtime, zero), output=out)
    assert_close_f16(out.buffer.to_numpy(np.float16, (m, n)), oracle.w4a16_linear(x, packed, scale, zero=zero),
                     label="prefill affine")


@pytest.mark.parametrize("m,k,n", [(128, 256, 256), (192, 576, 1536), (64, 128, 192)])
def test_prefill_swiglu_ffn_matches_oracle(runtime, oracle, m, k, n):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(14)
    activation = rng.standard_normal((m, k)).astype(np.float16)
    residual = rng.standard_normal((m, k)).astype(np.float16)
    gate, up, down = random_w4(rng, n, k), random_w4(rng, n, k), random_w4(rng, k, n)
    norm = rng.uniform(0.5, 1.5, size=k).astype(np.float16)
    out = _tensor(runtime, np.full((m, k), np.nan, np.float16))
    dispatch.dispatch_w4a16_swiglu_ffn_command(
        _ctx(runtime), m=m, n=n, k=k, epsilon=1e-5, activation=_tensor(runtime, activation),
        residual=_tensor(runtime, residual), gate_weight=_tensor(runtime, gate[0]), gate_scale=_tensor(runtime, gate[1]),
        up_weight=_tensor(runtime, up[0]), up_scale=_tensor(runtime, up[1]), down_weight=_tensor(runtime, down[0]),
        down_scale=_tensor(runtime, down[1]), norm_weight=_tensor(runtime, norm), output=out, reference_guards=False)
    want, _, _ = oracle.w4a16_swiglu_ffn(activation, residual, gate[0], gate[1], up[0], up[1], down[0], down[1], norm, 1e-5)
    assert_close_f16(out.buffer.to_numpy(np.float16, (m, k)), want, rel=3e-3, label="prefill swiglu ffn")


# ---- decode batches: the tensor-core kernel with the weights on the M side, converted into tensor memory.
# Which rows take it is a library setting (LLMOPT_CUDA_TC_BATCH_MIN_ROWS / _MAX_ROWS); the cases cover
# every padded batch width (16, 32, 64, 128) whichever kernel serves them. ----

@pytest.mark.parametrize("m,k,n", [(33, 128, 128), (36, 64, 40), (40, 1024, 384), (33, 576, 192), (48, 2048, 1000),
                                   (64, 4096, 512), (56, 14336, 256), (9, 1024, 384), (16, 4096, 512), (17, 576, 192),
                                   (32, 4096, 1000), (24, 14336, 256), (100, 2048, 384), (128, 1024, 640),
                                   (32, 4096, 8192), (20, 8192, 4096)])  # 32 M weights: the tensor-core kernel from 17 rows
def test_decode_batch_linear_matches_oracle(runtime, oracle, m, k, n):
    rng = np.random.default_rng(40)
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    residual = rng.standard_normal((m, n)).astype(np.float16)
    assert_close_f16(_linear(runtime, x, packed, scale), oracle.w4a16_linear(x, packed, scale),
                     label=f"decode batch linear m={m} k={k} n={n}")
    assert_close_f16(_linear(runtime, x, packed, scale, residual, n), oracle.w4a16_linear(x, packed, scale, residual, n),
                     label=f"decode batch linear + residual m={m} k={k} n={n}")


def test_decode_batch_dyadic_inputs_are_bit_exact(runtime, oracle):
    rng = np.random.default_rng(41)
    m, k, n = 40, 4096, 256  # few tiles, long K: the K-split path with its split-ordered sum
    x = (rng.integers(-8, 9, size=(m, k)) / 8.0).astype(np.float16)
    packed, _ = random_w4(rng, n, k)
    scale = (2.0 ** rng.integers(-6, -2, size=(n, k // 64))).astype(np.float16)
    got = _linear(runtime, x, packed, scale)
    assert np.array_equal(got.view(np.uint16), oracle.w4a16_linear(x, packed, scale).view(np.uint16))


@pytest.mark.parametrize("m,k,n", [(33, 256, 256), (48, 576, 1536), (40, 1024, 192), (12, 1024, 192), (32, 576, 1536),
                                   (96, 256, 256), (24, 4096, 8192), (300, 512, 1024)])
def test_decode_batch_swiglu_ffn_matches_oracle(runtime, oracle, m, k, n):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(42)
    activation = rng.standard_normal((m, k)).astype(np.float16)
    gate, up, down = random_w4(rng, n, k), random_w4(rng, n, k), random_w4(rng, k, n)
    norm = rng.uniform(0.5, 1.5, size=k).astype(np.float16)
    out = _tensor(runtime, np.full((m, k), np.nan, np.float16))
    dispatch.dispatch_w4a16_swiglu_ffn_command(
        _ctx(runtime), m=m, n=n, k=k, epsilon=1e-5, activation=_tensor(runtime, activation),
        residual=_tensor(runtime, activation), gate_weight=_tensor(runtime, gate[0]), gate_scale=_tensor(runtime, gate[1]),
        up_weight=_tensor(runtime, up[0]), up_scale=_tensor(runtime, up[1]), down_weight=_tensor(runtime, down[0]),
        down_scale=_tensor(runtime, down[1]), norm_weight=_tensor(runtime, norm), output=out, reference_guards=False)
    want, _, _ = oracle.w4a16_swiglu_ffn(activation, activation, gate[0], gate[1], up[0], up[1], down[0], down[1], norm, 1e-5)
    assert_close_f16(out.buffer.to_numpy(np.float16, (m, k)), want, rel=3e-3, label="decode batch swiglu ffn")
