"""CPU tests: the oracle against every known-answer vector the reference holds for
this path and against outputs of the reference's own Python implementation
(tests/golden/w4a16_reference.npz, made by tests/golden/make_golden.py)."""

import os

import numpy as np
import pytest

from conftest import f16_bits

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "w4a16_reference.npz")


def bits(array):
    return np.asarray(array, np.float16).view(np.uint16).reshape(-1).tolist()


def test_w4a16_fixture_bits(oracle):
    # python/examples/write_w4a16_weight_fixture.py:11-23 + bin/ocaml_metal_smoke.ml:184-236
    packed = np.arange(96, dtype=np.uint8).reshape(3, 32).copy()
    packed[0, 0] = 0x78
    scale = np.array([[0.125], [0.25], [0.5]], np.float16)
    bias = np.array([0.5, 1.0, -1.0], np.float16)
    x = np.ones((2, 64), np.float16)
    for order in ("f64", "msl_m1"):
        assert bits(oracle.w4a16_linear(x, packed, scale, bias, 0, order=order)) == [0x3600, 0x4C40, 0x53E0] * 2


def test_nibble_order(oracle):
    # python/tests/test_quantization.py:25-31: byte 0x78 -> (-8, +7)
    assert oracle.unpack_int4(np.array([[0x78] * 32], np.uint8))[0, :2].tolist() == [-8, 7]


def test_metal_runtime_smoke_case(oracle):
    # python/examples/metal_runtime_smoke.py:28-74: 0x11 rows give 64, 0xFF rows give -64, times 0.5
    packed = np.empty((29, 32), np.uint8)
    packed[0::2] = 0x11
    packed[1::2] = 0xFF
    scale = np.full((29, 1), 0.5, np.float16)
    x = np.ones((3, 64), np.float16)
    y = oracle.w4a16_linear(x, packed, scale)
    assert np.all(y[:, 0::2] == 32.0) and np.all(y[:, 1::2] == -32.0)
    bias = np.arange(29, dtype=np.float16)
    assert np.array_equal(oracle.w4a16_linear(x, packed, scale, bias, 0), y + bias)


def test_against_reference_python_outputs(oracle):
    from llmopt_b200.quantize import pack_int4_weight, unpack_int4_weight

    golden = np.load(GOLDEN)
    assert golden["nibble_unpacked"][0, :2].tolist() == [-8.0, 7.0]
    # integer decode and dequantised weights: bit-exact
    packed, scale = golden["small_packed"], golden["small_scale"]
    q = oracle.unpack_int4(packed).astype(np.float32)
    assert np.array_equal(q * np.repeat(scale.astype(np.float32), 64, axis=1), golden["small_unpacked"])
    assert np.array_equal(unpack_int4_weight(packed, scale), golden["small_unpacked"])
    rows = np.arange(0, 1536, 97)
    assert np.array_equal(unpack_int4_weight(golden["c1_packed"], golden["c1_scale"])[rows], golden["c1_unpacked_rows"])
    # the numpy quantiser reproduces the reference's bytes and scales
    repacked, rescale = pack_int4_weight(golden["small_weight"])
    assert np.array_equal(repacked, packed) and np.array_equal(rescale.view(np.uint16), scale.view(np.uint16))
    # linear outputs: the reference accumulates in fp32 (torch), the oracle in float64
    for tag, ms in (("c1", (1, 128)), ("small", (3,))):
        for m in ms:
            x = golden[f"{tag}_x{m}"]
            for bias_key, out_key in ((None, f"{tag}_y{m}_nobias"), (f"{tag}_bias{m}", f"{tag}_y{m}")):
                bias = None if bias_key is None else golden[bias_key]
                got = oracle.w4a16_linear(x, golden[f"{tag}_packed"], golden[f"{tag}_scale"], bias, 0).astype(np.float64)
                want = golden[out_key].astype(np.float64)
                scale_of_output = np.max(np.abs(want))
                assert np.max(np.abs(got - want)) <= 1e-3 * scale_of_output
                assert np.mean(got == want) > 0.97  # all but a few last-place roundings agree exactly


def test_q8_round_trip_exact(oracle):
    # bin/ocaml_metal_smoke.ml:45-170
    pattern = np.array([0x57F0, 0xD7F0, 0x3C00, 0xBC00], np.uint16)
    key = np.tile(pattern, 32).view(np.float16).reshape(1, 2, 64)
    pool = np.zeros(4 * 132, np.uint8)
    fields = dict(segment_offset=0, heads=1, head_dim=64, group_size=64, token_elements=128, token_stride=132)
    oracle.cache_pack_attention_q8(key, [2, 0], pool, source_items=2, **fields)
    assert np.array_equal(oracle.cache_unpack_attention_q8(pool, [2, 0], **fields).view(np.uint16), key.view(np.uint16))
    state = np.tile(pattern, 16).view(np.float16)
    cpool = np.zeros(2 * 66, np.uint8)
    cfields = dict(checkpoint=1, layer=0, layer_elements=64, group_size=64, checkpoint_elements=64, checkpoint_stride=66)
    oracle.cache_pack_checkpoint_q8(state, cpool, **cfields)
    assert np.array_equal(oracle.cache_unpack_checkpoint_q8(cpool, **cfields).view(np.uint16), state.view(np.uint16))
    assert cpool[66:66 + 4].view(np.int8).tolist() == [127, -127, 1, -1]


def test_q8_quantiser_rules(oracle):
    # all-zero group -> scale 1.0; round half to even; clamp to +-127
    source = np.zeros((1, 1, 64), np.float16)
    pool = np.zeros(66, np.uint8)
    fields = dict(segment_offset=0, heads=1, head_dim=64, group_size=64, token_elements=64, token_stride=66)
    oracle.cache_pack_attention_q8(source, [0], pool, source_items=1, **fields)
    assert pool[64:66].view(np.uint16)[0] == 0x3C00 and not pool[:64].any()
    source[0, 0, :4] = [127.0, 0.5, 1.5, 2.5]  # scale = 1.0: rint -> 127, 0, 2, 2
    oracle.cache_pack_attention_q8(source, [0], pool, source_items=1, **fields)
    assert pool[:4].view(np.int8).tolist() == [127, 0, 2, 2]


def test_paged_attention_known_answer(oracle):
    # bin/ocaml_metal_primitives_smoke.ml:66-73,238-254,387-390; bin/native_schedule_fixture.ml:296-337
    pool = np.zeros(132, np.uint8)
    pool[64:128] = 2
    pool[128:132] = np.array([0x3C00, 0x3C00], np.uint16).view(np.uint8)
    for heads in (1, 3):
        params = oracle.paged_params_bytes(batches=1, query_heads=heads, kv_heads=1, past_length=1, head_dim=64,
                                           mask_batches=1, mask_heads=1, token_elements=128, key_offset=0,
                                           value_offset=64, group_size=64, token_stride=132, scale=1.0,
                                           query_length=1, mask_dtype=1)
        out = oracle.attention_q8_paged(np.zeros((1, heads, 1, 64), np.float16), np.zeros((1, 1, 1, 64), np.float16),
                                        np.full((1, 1, 1, 64), 4.0, np.float16), pool, [0], np.ones(2, np.uint8), params)
        assert set(bits(out)) == {0x4200}


def test_short_conv_known_answers(oracle):
    # bin/ocaml_metal_primitives_smoke.ml:202-220,371-381
    weight = f16_bits([0x3C00, 0x0000, 0xBC00, 0x3800, 0x3C00, 0x3800]).reshape(2, 3)
    x = f16_bits([0x3C00, 0x4000, 0x4200, 0x4400, 0x4500, 0x4600, 0x4700, 0x4800]).reshape(1, 2, 4)
    assert bits(oracle.short_conv(x, weight, output_width=6, stride=1, padding=2, dilation=1)) == [
        0xBC00, 0xC000, 0xC000, 0xC000, 0x4200, 0x4400, 0x4100, 0x4800, 0x4A00, 0x4B00, 0x49C0, 0x4400]
    out, state = oracle.short_conv_step(f16_bits([0x3C00, 0x3C00, 0x4000, 0x3800, 0x3C00, 0x3C00]),
                                        f16_bits([0x3C00, 0x4000, 0x4200, 0x4400, 0x4500, 0x4600]).reshape(2, 3), weight)
    assert bits(out) == [0x4000, 0x4480] and state.reshape(-1).tolist() == [2, 3, 1, 5, 6, 1]
    out, state = oracle.short_conv_prefill(np.ones((4, 6), np.float16), weight)
    assert bits(out) == [0xBC00, 0x3800, 0xBC00, 0x3E00, 0x0000, 0x4000, 0x0000, 0x4000]
    assert bits(state) == [0x3C00] * 6


def test_dense_attention_known_answer(oracle):
    # bin/ocaml_metal_primitives_smoke.ml:221-229,382-383
    eye = f16_bits([0x3C00, 0, 0, 0x3C00]).reshape(1, 1, 2, 2)
    value = f16_bits([0x4900, 0, 0, 0x4D00]).reshape(1, 1, 2, 2)
    mask = np.array([1, 0, 0, 1], np.uint8)
    out = oracle.attention_dense(eye, eye, value, mask, causal=0, scale=1.0, mask_dtype=1, mask_batches=1, mask_heads=1)
    assert bits(out) == [0x4900, 0, 0, 0x4D00]


def test_epilogue_formulas(oracle):
    # lib/epilogue.ml:148-174
    import math

    lib = oracle.lib()
    acc, first, second = 0.75, -1.25, 2.0
    silu = acc / (1 + math.exp(-acc))
    gelu = 0.5 * acc * (1 + math.tanh(0.7978845608 * (acc + 0.044715 * acc ** 3)))
    expect = {0: acc, 1: acc + first, 2: silu, 3: gelu, 4: silu * first, 5: gelu * first, 6: acc + first,
              7: acc + first + second, 8: silu * first + second, 9: gelu * first + second}
    for tag, want in expect.items():
        assert abs(lib.orc_epilogue_apply(tag, acc, first, second) - want) < 1e-12


def test_lm_head_tie_and_msl_order(oracle):
    rng = np.random.default_rng(0)
    k, n = 128, 40
    weight = np.full((n, k // 2), 0x21, np.uint8)
    scale = np.full((n, 2), 0.25, np.float16)
    x = rng.standard_normal((2, k)).astype(np.float16)
    tokens, logits, _ = oracle.w4a16_lm_head_argmax(x, np.ones(k, np.float16), weight, scale, 1e-5, want_logits=True)
    assert tokens.tolist() == [0, 0] and logits.shape == (2, n)
    # the Metal m=1 evaluation order (fp32) and the float64 loop agree to the parity bound
    packed = rng.integers(0, 256, size=(64, k // 2), dtype=np.uint8)
    a = oracle.w4a16_linear(x, packed, scale[:1].repeat(64, 0)).astype(np.float64)
    b = oracle.w4a16_linear(x, packed, scale[:1].repeat(64, 0), order="msl_m1").astype(np.float64)
    assert np.max(np.abs(a - b)) <= 2e-3 * np.max(np.abs(a))


@pytest.mark.parametrize("hq,hkv,dim,group,past", [(6, 2, 64, 64, 37), (8, 8, 128, 32, 21), (4, 1, 64, 32, 1)])
def test_paged_attention_equals_dense_attention_on_the_unpacked_pool(oracle, hq, hkv, dim, group, past):
    """The reference has no CPU paged attention (lib/cpu.ml:995-996); its dense attention
    (lib/cpu.ml:606-717) on the dequantised cache is the same function.  This pins what the
    degenerate known-answer vector cannot: the K/V dequantisation, the scale index
    segment_offset/group + kv_head*groups_per_head + d/group, the slot indirection and the layer
    offsets of the paged restatement (lib/metal_cache_source.ml:382-489)."""
    from helpers import random_pool
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    rng = np.random.default_rng(hq * 100 + past)
    layout = Layout([AttentionLayer(hkv, dim)] * 3, group_size=group)
    capacity = past + 4
    pool = random_pool(rng, capacity, layout.bytes_per_token, layout.token_elements, group, scale_range=(0.004, 0.03))
    slots = rng.permutation(capacity)[:past].astype(np.uint32)
    region = layout.attentions[1]
    query = (rng.standard_normal((1, hq, 1, dim)) * 2).astype(np.float16)
    current_key = rng.standard_normal((1, hkv, 1, dim)).astype(np.float16)
    current_value = rng.standard_normal((1, hkv, 1, dim)).astype(np.float16)
    scale = float(np.float32(1 / np.sqrt(dim)))
    params = oracle.paged_params_bytes(batches=1, query_heads=hq, kv_heads=hkv, past_length=past, head_dim=dim,
                                       mask_batches=0, mask_heads=0, token_elements=layout.token_elements,
                                       key_offset=region.key_offset, value_offset=region.value_offset,
                                       group_size=group, token_stride=layout.bytes_per_token, scale=scale,
                                       query_length=1, mask_dtype=0)
    paged = oracle.attention_q8_paged(query, current_key, current_value, pool, slots, None, params)
    fields = dict(heads=hkv, head_dim=dim, group_size=group, token_elements=layout.token_elements,
                  token_stride=layout.bytes_per_token)
    keys = oracle.cache_unpack_attention_q8(pool, slots, segment_offset=region.key_offset, **fields)      # [hkv, past, D]
    values = oracle.cache_unpack_attention_q8(pool, slots, segment_offset=region.value_offset, **fields)
    keys = np.concatenate([keys, current_key[0]], axis=1)[None]
    values = np.concatenate([values, current_value[0]], axis=1)[None]
    dense = oracle.attention_dense(query, keys, values, None, causal=0, scale=scale, kv_heads=hkv, token_first_output=1)
    assert paged.shape == dense.shape == (1, 1, hq, dim)
    error = np.max(np.abs(paged.astype(np.float64) - dense.astype(np.float64))) / np.max(np.abs(dense.astype(np.float64)))
    assert error <= 2e-3, error
    # and the cross-check has teeth: another layer's segment gives a different answer
    other = layout.attentions[2]
    wrong = oracle.paged_params_bytes(batches=1, query_heads=hq, kv_heads=hkv, past_length=past, head_dim=dim,
                                      mask_batches=0, mask_heads=0, token_elements=layout.token_elements,
                                      key_offset=other.key_offset, value_offset=other.value_offset,
                                      group_size=group, token_stride=layout.bytes_per_token, scale=scale,
                                      query_length=1, mask_dtype=0)
    assert not np.array_equal(oracle.attention_q8_paged(query, current_key, current_value, pool, slots, None, wrong), paged)
