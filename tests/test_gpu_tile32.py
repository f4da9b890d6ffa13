"""Tile32 affine formats through the named dispatches: the block-quantised linears
(llmopt_tile32_affine{4,8}_linear_f16_*) against the float64 oracle, and the Hadamard-rotated
Tile32 cache codec (llmopt_cache_{pack,unpack}_attention_tile32_affine{8,4}_fwht_simd), whose fp32
operations are fixed by the reference kernels and are therefore compared byte for byte."""

import numpy as np
import pytest

from conftest import assert_close_f16

pytestmark = pytest.mark.gpu


def _buf(runtime, array):
    from llmopt_b200.cuda_native import Buffer

    return Buffer.of_array(runtime, np.ascontiguousarray(array))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,k,n,mode", [(1, 576, 200, 0), (5, 1024, 96, 1), (9, 128, 33, 2)])
def test_tile32_affine_linear_matches_oracle(runtime, oracle, bits, m, k, n, mode):
    from llmopt_b200 import parameters

    rng = np.random.default_rng(bits * 100 + m)
    weight = oracle.tile32_affine_blocks(rng.standard_normal((n, k)) * 0.05, bits=bits)
    x = rng.standard_normal((m, k)).astype(np.float16)
    additive = {0: None, 1: rng.standard_normal(n).astype(np.float16), 2: rng.standard_normal((m, n)).astype(np.float16)}[mode]
    out = _buf(runtime, np.full((m, n), np.nan, np.float16))
    for tactic in ("_x8", "_simd", "_m16"):
        name = f"llmopt_tile32_affine{bits}_linear_f16{tactic}"
        assert runtime.has_function(name)
        runtime.dispatch(name, buffers=[_buf(runtime, x), _buf(runtime, weight),
                                        _buf(runtime, additive if additive is not None else x), out],
                         parameters=parameters.u32s([m, n, k, mode]), grid=(256, 1, 1))
        want = oracle.tile32_affine_linear(x, weight, bits=bits, additive=additive, mode=mode)
        assert_close_f16(out.to_numpy(np.float16, (m, n)), want, label=name)


@pytest.mark.parametrize("bits", [8, 4])
def test_fwht_cache_codec_is_byte_exact(runtime, oracle, bits):
    from llmopt_b200 import parameters

    rng = np.random.default_rng(40 + bits)
    heads, dim, items, capacity = 3, 128, 4, 9
    tile_bytes = 36 if bits == 8 else 20
    elements = 2 * heads * dim                      # one layer: K then V
    stride = elements // 32 * tile_bytes
    source = rng.standard_normal((heads, items, dim)).astype(np.float16)
    source[1, 2, 32:64] = 0                          # an all-zero tile: scale 0, codes 0
    source[0, 0, :32] = 1.5                          # a constant tile: only the first rotated lane is nonzero
    slots = np.array([7, 0, 3, 5], np.uint32)
    block = parameters.cache_attention(items=items, segment_offset=heads * dim, heads=heads, head_dim=dim, group_size=32,
                                       token_elements=elements, token_groups=elements // 32, token_stride=stride,
                                       source_items=items, source_offset=0)
    pool = _buf(runtime, np.full(capacity * stride, 0xEE, np.uint8))
    runtime.dispatch(f"llmopt_cache_pack_attention_tile32_affine{bits}_fwht_simd",
                     buffers=[_buf(runtime, source), _buf(runtime, slots), pool], parameters=block, grid=(256, 1, 1))
    want_pool = np.full(capacity * stride, 0xEE, np.uint8)
    oracle.cache_pack_attention_fwht(source, slots, want_pool, bits=bits, segment_offset=heads * dim, heads=heads,
                                     head_dim=dim, token_stride=stride, source_items=items)
    got_pool = pool.to_numpy(np.uint8)
    assert np.array_equal(got_pool, want_pool)
    assert not np.array_equal(got_pool, np.full_like(got_pool, 0xEE))
    out = _buf(runtime, np.full((heads, items, dim), np.nan, np.float16))
    runtime.dispatch(f"llmopt_cache_unpack_attention_tile32_affine{bits}_fwht_simd",
                     buffers=[pool, _buf(runtime, slots), out], parameters=block, grid=(256, 1, 1))
    want = oracle.cache_unpack_attention_fwht(want_pool, slots, bits=bits, segment_offset=heads * dim, heads=heads,
                                              head_dim=dim, token_stride=stride)
    got = out.to_numpy(np.float16, (heads, items, dim))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # the codec is lossy but close: 8-bit tiles reproduce the rows to a few thousandths of their range
    error = np.max(np.abs(got.astype(np.float32) - source.astype(np.float32)))
    assert error <= (0.03 if bits == 8 else 0.5)
