"""GPU parity of the Q4_0-block linear family against the float64 oracle, through the named dispatches."""

import numpy as np
import pytest

from conftest import assert_close_f16
from test_gpu_w4a16 import _ctx, _tensor

pytestmark = pytest.mark.gpu


def _weights(rng, n, k):
    from llmopt_b200.quantize import q4_0_blocks

    scales = rng.uniform(0.005, 0.03, size=(n, k // 32)).astype(np.float16)
    return q4_0_blocks(scales, rng.integers(0, 16, size=(n, k), dtype=np.uint8))


def test_dequant_is_bit_exact(runtime, oracle):
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Batch, Buffer

    rng = np.random.default_rng(30)
    blocks = _weights(rng, 7, 96)  # 21 blocks
    out = Buffer.create(runtime, 21 * 64)
    batch = Batch(runtime)
    batch.dispatch(name="llmopt_dequant_q4_0", buffers=[Buffer.of_array(runtime, blocks), out],
                   parameters=parameters.u32s([21]), grid=(21 * 32, 1, 1), group=(256, 1, 1))
    batch.commit()
    assert np.array_equal(out.to_numpy(np.uint16), oracle.q4_0_dequant(blocks).view(np.uint16))


def test_reference_fixture_block_layout(runtime, oracle):
    # test/test_quant.ml:690-693: d = 1.0, byte i = (i & 15) | ((15 - i) & 15) << 4 -> elements i - 8 and 7 - i
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Batch, Buffer

    block = np.zeros(18, np.uint8)
    block[0:2] = np.array([0x3C00], np.uint16).view(np.uint8)
    for i in range(16):
        block[2 + i] = (i & 15) | (((15 - i) & 15) << 4)
    want = np.array([i - 8 for i in range(16)] + [7 - i for i in range(16)], np.float16)
    assert np.array_equal(oracle.q4_0_dequant(block), want)
    out = Buffer.create(runtime, 64)
    batch = Batch(runtime)
    batch.dispatch(name="llmopt_dequant_q4_0", buffers=[Buffer.of_array(runtime, block), out],
                   parameters=parameters.u32s([1]), grid=(32, 1, 1), group=(256, 1, 1))
    batch.commit()
    assert np.array_equal(out.to_numpy(np.float16), want)


@pytest.mark.parametrize("m,k,n,mode", [(1, 576, 1536, 0), (1, 4096, 512, 2), (2, 1024, 96, 1), (5, 1536, 333, 2),
                                        (16, 256, 40, 0), (37, 96, 17, 2),
                                        # the tensor-core form: two K chunks, a short last chunk, more than 32 rows
                                        (1, 8192, 48, 0), (9, 4352, 32, 1), (33, 512, 64, 2), (8, 14336, 24, 0),
                                        # the stream form with a single half slice of K, and seven rows
                                        (3, 256, 24, 1), (7, 2304, 50, 2)])
def test_linear_matches_oracle(runtime, oracle, m, k, n, mode):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(31)
    x = rng.standard_normal((m, k)).astype(np.float16)
    weight = _weights(rng, n, k)
    additive = None if mode == 0 else rng.standard_normal((n,) if mode == 1 else (m, n)).astype(np.float16)
    out = _tensor(runtime, np.full((m, n), np.nan, np.float16))
    kernels = dispatch.dispatch_quant_linear(
        _ctx(runtime), m=m, n=n, k=k, input=_tensor(runtime, x), weight=_tensor(runtime, weight), output=out,
        additive=None if additive is None else _tensor(runtime, additive), epilogue_mode=mode)
    assert kernels[0].endswith("_add") == (mode == 2)
    assert_close_f16(out.buffer.to_numpy(np.float16, (m, n)), oracle.q4_0_linear(x, weight, additive, mode),
                     label=f"q4_0 linear m={m} k={k} n={n} mode={mode}")


@pytest.mark.parametrize("m,k,nq,nk,nv", [(1, 576, 576, 192, 192), (3, 1024, 256, 64, 64), (2, 512, 40, 24, 8), (12, 768, 48, 16, 40)])
def test_qkv_matches_oracle(runtime, oracle, m, k, nq, nk, nv):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(32)
    x = rng.standard_normal((m, k)).astype(np.float16)
    weights = [_weights(rng, n, k) for n in (nq, nk, nv)]
    outs = [_tensor(runtime, np.full((m, n), np.nan, np.float16)) for n in (nq, nk, nv)]
    dispatch.dispatch_quant_qkv_linear(
        _ctx(runtime), m=m, k=k, input=_tensor(runtime, x), q_weight=_tensor(runtime, weights[0]),
        k_weight=_tensor(runtime, weights[1]), v_weight=_tensor(runtime, weights[2]), q_output=outs[0],
        k_output=outs[1], v_output=outs[2])
    for out, weight, n in zip(outs, weights, (nq, nk, nv)):
        assert_close_f16(out.buffer.to_numpy(np.float16, (m, n)), oracle.q4_0_linear(x, weight), label="q4_0 qkv")


@pytest.mark.parametrize("activation,code", [("silu", 0), ("gelu", 1), ("sigmoid", 2)])
def test_gated_matches_oracle(runtime, oracle, activation, code):
    from llmopt_b200 import dispatch

    rng = np.random.default_rng(33)
    m, k, n = 3, 768, 200
    x = rng.standard_normal((m, k)).astype(np.float16)
    gate, up = _weights(rng, n, k), _weights(rng, n, k)
    product = _tensor(runtime, np.full((m, n), np.nan, np.float16))
    dispatch.dispatch_quant_gated_linear(_ctx(runtime), m=m, n=n, k=k, input=_tensor(runtime, x),
                                         gate_weight=_tensor(runtime, gate), up_weight=_tensor(runtime, up),
                                         product=product, activation=activation)
    assert_close_f16(product.buffer.to_numpy(np.float16, (m, n)), oracle.q4_0_gated_linear(x, gate, up, code),
                     rel=3e-3, label=f"q4_0 gated {activation}")


@pytest.mark.parametrize("m,k,n", [(3, 1024, 200), (2, 96, 40), (11, 512, 64)])
def test_digest_named_epilogue_over_q4_0(runtime, oracle, m, k, n):
    """A Q4_0 linear with an algebraic epilogue is named llmopt_q4_0_linear_f16<tactic>_<digest> and binds
    [input, weight, epilogue inputs .., output] (Writeback.Epilogue, lib/metal_q4_0_epilogue_codegen.ml:7-31).
    epilogue.bind registers the expression's program under that name; the result is the epilogue of the
    unrounded Q4_0 sums, on the tensor-core form (K a multiple of 256) and on the general kernel."""
    from llmopt_b200 import epilogue as ep, parameters
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(41 + k)
    x = rng.standard_normal((m, k)).astype(np.float16)
    blocks = _weights(rng, n, k)
    up = rng.standard_normal(n).astype(np.float16)
    ceiling = rng.uniform(0.2, 2.0, size=n).astype(np.float32)
    # the unrounded sums from the raw blocks: w = d (q - 8), low nibbles first
    raw = blocks.reshape(n, k // 32, 18)
    d = raw[:, :, :2].copy().view(np.float16).astype(np.float64)  # [n, blocks, 1]
    quants = raw[:, :, 2:].astype(np.int32)
    q = np.concatenate([(quants & 15) - 8, (quants >> 4) - 8], axis=2).astype(np.float64)
    acc = x.astype(np.float64) @ (d * q).reshape(n, k).T
    base = "llmopt_q4_0_linear_f16_x8"
    tree = ep.Triop("clamp", ep.Binop("add", ep.Binop("mul", ep.Unop("silu", ep.ACC), ep.Read(ep.Value(4))), ep.Const(0.5)),
                    ep.Const(-1.0), ep.Read(ep.Value(9, "f32")))
    name = ep.bind(runtime, base, ep.of_expr(tree))
    assert name.startswith(base + "_") and runtime.has_function(name)
    out = Buffer.of_array(runtime, np.full((m, n), np.nan, np.float16))
    runtime.dispatch(name, buffers=[Buffer.of_array(runtime, x), Buffer.of_array(runtime, blocks), Buffer.of_array(runtime, up),
                                    Buffer.of_array(runtime, ceiling), out],
                     parameters=parameters.u32s([m, n, k, 0]), grid=(256, 1, 1))
    want = np.clip((acc / (1 + np.exp(-acc))) * up.astype(np.float64) + 0.5, -1.0, ceiling.astype(np.float64))
    assert_close_f16(out.to_numpy(np.float16, (m, n)), want, label=f"q4_0 expression epilogue m={m} k={k}")
    # a tagged form has no built-in kernel over this base: it is a program as well
    gated = ep.bind(runtime, base, ep.tagged("silu_mul", ep.Value(0)))
    out = Buffer.of_array(runtime, np.full((m, n), np.nan, np.float16))
    runtime.dispatch(gated, buffers=[Buffer.of_array(runtime, x), Buffer.of_array(runtime, blocks), Buffer.of_array(runtime, up), out],
                     parameters=parameters.u32s([m, n, k, 0]), grid=(256, 1, 1))
    assert_close_f16(out.to_numpy(np.float16, (m, n)), (acc / (1 + np.exp(-acc))) * up.astype(np.float64),
                     label="q4_0 silu_mul epilogue")
    from llmopt_b200.cuda_native import NativeError

    with pytest.raises(NativeError, match="buffer count"):
        runtime.dispatch(gated, buffers=[out] * 5, parameters=parameters.u32s([m, n, k, 0]), grid=(256, 1, 1))
