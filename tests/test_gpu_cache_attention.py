"""GPU parity of the grouped-Q8 cache codec (bit-exact), paged attention and the
recurrent-state kernels against the CPU oracle and the reference's known answers."""

import numpy as np
import pytest

from conftest import assert_close_f16, f16_bits
from helpers import random_pool

pytestmark = pytest.mark.gpu


def _buf(runtime, array):
    from llmopt_b200.cuda_native import Buffer

    return Buffer.of_array(runtime, np.ascontiguousarray(array))


def _tensor(runtime, array, dtype="float16"):
    from llmopt_b200 import dispatch

    return dispatch.Tensor(_buf(runtime, array), tuple(np.shape(array)), dtype)


def test_q8_codec_reference_round_trip(runtime):
    # bin/ocaml_metal_smoke.ml:45-170: values +-127, +-1 survive pack -> unpack byte for byte
    from llmopt_b200 import dispatch
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    layout = Layout([AttentionLayer(1, 64)], recurrent_layers=1, recurrent_width=64, recurrent_window=1)
    cache = dispatch.Cache(runtime, layout, token_capacity=4, checkpoint_capacity=2)
    context = dispatch.Context(runtime)
    pattern = np.array([0x57F0, 0xD7F0, 0x3C00, 0xBC00], np.uint16)
    key = np.tile(pattern, 32).view(np.float16).reshape(1, 2, 64)       # [heads, items, D]
    value = np.tile(pattern[[1, 0, 3, 2]], 32).view(np.float16).reshape(1, 2, 64)
    cache.pack_attention(context, layer=0, kind="key", slots=[2, 0], source=_buf(runtime, key), source_items=2)
    cache.pack_attention(context, layer=0, kind="value", slots=[2, 0], source=_buf(runtime, value), source_items=2)
    for kind, want in (("key", key), ("value", value)):
        out = _buf(runtime, np.full((1, 2, 64), np.nan, np.float16))
        cache.unpack_attention(context, layer=0, kind=kind, slots=[2, 0], destination=out)
        assert np.array_equal(out.to_numpy(np.uint16), want.view(np.uint16).reshape(-1))
    state = np.tile(pattern, 16).view(np.float16)
    cache.pack_checkpoint(context, layer=0, checkpoint=1, source=_buf(runtime, state))
    out = _buf(runtime, np.full((64,), np.nan, np.float16))
    cache.unpack_checkpoint(context, layer=0, checkpoint=1, destination=out)
    assert np.array_equal(out.to_numpy(np.uint16), state.view(np.uint16))


@pytest.mark.parametrize("heads,dim,group,items", [(3, 64, 64, 5), (8, 128, 64, 3), (2, 64, 32, 7), (1, 256, 64, 2)])
def test_q8_pack_bit_exact_vs_oracle(runtime, oracle, heads, dim, group, items):
    from llmopt_b200 import dispatch
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    rng = np.random.default_rng(10)
    layout = Layout([AttentionLayer(heads, dim)] * 2, group_size=group)
    capacity = 16
    cache = dispatch.Cache(runtime, layout, token_capacity=capacity)
    context = dispatch.Context(runtime)
    source_items = items + 2
    key = (rng.standard_normal((heads, source_items, dim)) * rng.uniform(0.01, 30)).astype(np.float16)
    value = rng.standard_normal((heads, source_items, dim)).astype(np.float16)
    key[0, 1, :group] = 0  # an all-zero group stores scale 1.0
    key[0, 2, 0] = np.float16(65504.0)
    slots = rng.permutation(capacity)[:items].tolist()
    cache.pack_attention_pair(context, layer=1, slots=slots, key_source=_buf(runtime, key),
                              value_source=_buf(runtime, value), source_items=source_items, source_offset=1)
    got = cache.token_pool.to_numpy(np.uint8)
    want = np.zeros(capacity * layout.bytes_per_token, np.uint8)
    region = layout.attentions[1]
    for segment, source in ((region.key_offset, key), (region.value_offset, value)):
        oracle.cache_pack_attention_q8(source, slots, want, segment_offset=segment, heads=heads, head_dim=dim,
                                       group_size=group, token_elements=layout.token_elements,
                                       token_stride=layout.bytes_per_token, source_items=source_items,
                                       source_offset=1)
    assert np.array_equal(got, want)
    out = _buf(runtime, np.full((heads, items, dim), np.nan, np.float16))
    cache.unpack_attention(context, layer=1, kind="key", slots=slots, destination=out)
    want_unpacked = oracle.cache_unpack_attention_q8(want, slots, segment_offset=region.key_offset, heads=heads,
                                                     head_dim=dim, group_size=group,
                                                     token_elements=layout.token_elements,
                                                     token_stride=layout.bytes_per_token)
    assert np.array_equal(out.to_numpy(np.uint16), want_unpacked.view(np.uint16).reshape(-1))


def test_checkpoint_codec_bit_exact(runtime, oracle):
    from llmopt_b200 import dispatch
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    rng = np.random.default_rng(11)
    layout = Layout([AttentionLayer(8, 64)], recurrent_layers=10, recurrent_width=1024, recurrent_window=3)
    cache = dispatch.Cache(runtime, layout, token_capacity=1, checkpoint_capacity=3)
    context = dispatch.Context(runtime)
    state = rng.standard_normal(3072).astype(np.float16)
    cache.pack_checkpoint(context, layer=7, checkpoint=2, source=_buf(runtime, state))
    want = np.zeros(3 * layout.bytes_per_checkpoint, np.uint8)
    fields = dict(checkpoint=2, layer=7, layer_elements=3072, group_size=64,
                  checkpoint_elements=layout.checkpoint_elements, checkpoint_stride=layout.bytes_per_checkpoint)
    oracle.cache_pack_checkpoint_q8(state, want, **fields)
    assert np.array_equal(cache.checkpoint_pool.to_numpy(np.uint8), want)
    out = _buf(runtime, np.full((3072,), np.nan, np.float16))
    cache.unpack_checkpoint(context, layer=7, checkpoint=2, destination=out)
    assert np.array_equal(out.to_numpy(np.uint16), oracle.cache_unpack_checkpoint_q8(want, **fields).view(np.uint16))


def _paged(runtime, oracle, *, batches, hq, hkv, dim, group, past, q_len=1, layers=2, layer=1, window=None, mask=None,
           mask_dtype=None, per_sequence=False, seed=0, query_scale=1.0):
    from llmopt_b200 import dispatch
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    rng = np.random.default_rng(seed)
    layout = Layout([AttentionLayer(hkv, dim)] * layers, group_size=group)
    capacity = max(past * (batches if per_sequence else 1), 1) + 3
    pool = random_pool(rng, capacity, layout.bytes_per_token, layout.token_elements, group)
    if per_sequence:
        slots = np.stack([rng.permutation(capacity)[:past] for _ in range(batches)]).astype(np.uint32)
        slots = np.ascontiguousarray(slots.reshape(batches, past))
    else:
        slots = rng.permutation(capacity)[:past].astype(np.uint32)
    query = (rng.standard_normal((batches, hq, q_len, dim)) * query_scale).astype(np.float16)
    current_key = rng.standard_normal((batches, hkv, q_len, dim)).astype(np.float16)
    current_value = rng.standard_normal((batches, hkv, q_len, dim)).astype(np.float16)
    region = layout.attentions[layer]
    config = dispatch.PagedAttentionConfig(token_elements=layout.token_elements, key_offset=region.key_offset,
                                           value_offset=region.value_offset, group_size=group,
                                           token_stride=layout.bytes_per_token, scale=1.0 / np.sqrt(dim), window=window)
    out = _tensor(runtime, np.full((batches, q_len, hq, dim), np.nan, np.float16))
    slots_for_device = slots if slots.size else np.zeros(4, np.uint32)
    slot_tensor = dispatch.Tensor(_buf(runtime, slots_for_device), tuple(slots.shape), "uint32")
    mask_tensor = None
    if mask is not None:
        mask_tensor = dispatch.Tensor(_buf(runtime, mask), tuple(mask.shape), mask_dtype)
    names = dispatch.dispatch_paged_attention_q8(
        dispatch.Context(runtime), config=config, query=_tensor(runtime, query), current_key=_tensor(runtime, current_key),
        current_value=_tensor(runtime, current_value), pool=dispatch.Tensor(_buf(runtime, pool), (pool.size,), "uint8"),
        slots=slot_tensor, output=out, mask=mask_tensor, slot_batch_stride=past if per_sequence else None)
    params = oracle.paged_params_bytes(
        batches=batches, query_heads=hq, kv_heads=hkv, past_length=past, head_dim=dim,
        mask_batches=0 if mask is None else mask.shape[0], mask_heads=0 if mask is None else mask.shape[1],
        token_elements=layout.token_elements, key_offset=region.key_offset, value_offset=region.value_offset,
        group_size=group, token_stride=layout.bytes_per_token, scale=float(np.float32(1.0 / np.sqrt(dim))),
        query_length=q_len, mask_dtype={None: 0, "bool": 1, "float16": 2}[mask_dtype], window=window or 0)
    want = oracle.attention_q8_paged(query, current_key, current_value, pool, slots_for_device, mask, params,
                                     slot_batch_stride=past if per_sequence else 0)
    got = out.buffer.to_numpy(np.float16, (batches, q_len, hq, dim))
    return got, want, names


def test_paged_reference_known_answer(runtime):
    # bin/ocaml_metal_primitives_smoke.ml:66-73,238-254,387-390: every output is 0x4200 (3.0)
    from llmopt_b200 import dispatch

    pool = np.zeros(132, np.uint8)
    pool[64:128] = 2
    pool[128:132] = np.array([0x3C00, 0x3C00], np.uint16).view(np.uint8)
    config = dispatch.PagedAttentionConfig(token_elements=128, key_offset=0, value_offset=64, group_size=64,
                                           token_stride=132, scale=1.0)
    for heads in (1, 3):
        out = _tensor(runtime, np.full((1, 1, heads, 64), np.nan, np.float16))
        mask = np.ones((1, 1, 1, 2), np.uint8)
        for use_mask in (True, False):
            dispatch.dispatch_paged_attention_q8(
                dispatch.Context(runtime), config=config, query=_tensor(runtime, np.zeros((1, heads, 1, 64), np.float16)),
                current_key=_tensor(runtime, np.zeros((1, 1, 1, 64), np.float16)),
                current_value=_tensor(runtime, np.full((1, 1, 1, 64), 4.0, np.float16)),
                pool=dispatch.Tensor(_buf(runtime, pool), (132,), "uint8"),
                slots=dispatch.Tensor(_buf(runtime, np.zeros(4, np.uint32)), (1,), "uint32"), output=out,
                mask=dispatch.Tensor(_buf(runtime, mask), mask.shape, "bool") if use_mask else None)
            assert set(out.buffer.to_numpy(np.uint16).tolist()) == {0x4200}


@pytest.mark.parametrize("batches,hq,hkv,dim,group,past", [
    (1, 9, 3, 64, 64, 512), (1, 16, 8, 64, 64, 1040), (2, 32, 8, 128, 64, 777), (1, 32, 8, 128, 64, 8192),
    (1, 4, 1, 128, 32, 100), (3, 8, 8, 64, 32, 33), (1, 9, 3, 64, 64, 0), (1, 9, 3, 64, 64, 1), (1, 8, 1, 128, 64, 15),
])
def test_paged_decode_matches_oracle(runtime, oracle, batches, hq, hkv, dim, group, past):
    got, want, names = _paged(runtime, oracle, batches=batches, hq=hq, hkv=hkv, dim=dim, group=group, past=past,
                              query_scale=3.0)
    assert_close_f16(got, want, label=f"paged {names}")


def test_paged_per_sequence_slot_tables(runtime, oracle):
    got, want, names = _paged(runtime, oracle, batches=4, hq=32, hkv=8, dim=128, group=64, past=300, per_sequence=True)
    assert names == ["llmopt_attention_q8_paged_batched"]
    assert_close_f16(got, want, label="paged batched")


def test_paged_fallback_shapes(runtime, oracle):
    # q > 1 with a bool / f16 mask, sliding window, other head sizes: the row kernel
    rng = np.random.default_rng(3)
    mask = (rng.random((1, 1, 3, 23)) > 0.3).astype(np.uint8)
    mask[..., 0] = 1
    got, want, _ = _paged(runtime, oracle, batches=1, hq=4, hkv=2, dim=64, group=64, past=20, q_len=3, mask=mask,
                          mask_dtype="bool")
    assert_close_f16(got, want, label="paged bool mask")
    fmask = np.where(rng.random((2, 4, 2, 12)) > 0.4, 0.0, -np.inf).astype(np.float16)
    fmask[..., 0] = 0
    got, want, _ = _paged(runtime, oracle, batches=2, hq=4, hkv=4, dim=64, group=64, past=10, q_len=2, mask=fmask,
                          mask_dtype="float16")
    assert_close_f16(got, want, label="paged f16 mask")
    got, want, _ = _paged(runtime, oracle, batches=1, hq=2, hkv=1, dim=64, group=64, past=50, window=16)
    assert_close_f16(got, want, label="paged window")
    got, want, _ = _paged(runtime, oracle, batches=1, hq=2, hkv=2, dim=256, group=64, past=40)
    assert_close_f16(got, want, label="paged h256")
    got, want, _ = _paged(runtime, oracle, batches=1, hq=1, hkv=1, dim=192, group=64, past=9)
    assert_close_f16(got, want, label="paged generic 192")


def test_short_conv_known_answers(runtime):
    # bin/ocaml_metal_primitives_smoke.ml:202-220,371-381
    from llmopt_b200 import dispatch, parameters

    context = dispatch.Context(runtime)
    weight = f16_bits([0x3C00, 0x0000, 0xBC00, 0x3800, 0x3C00, 0x3800])
    # generic conv: [1,2,4], stride 1, pad 2, dilation 1 -> [1,2,6]
    out = _buf(runtime, np.full(12, np.nan, np.float16))
    runtime.dispatch("llmopt_short_conv_f16",
                     buffers=[_buf(runtime, f16_bits([0x3C00, 0x4000, 0x4200, 0x4400, 0x4500, 0x4600, 0x4700, 0x4800])),
                              _buf(runtime, weight), out],
                     parameters=parameters.short_conv(batches=1, channels=2, input_width=4, output_width=6,
                                                      kernel_width=3, stride=1, padding=2, dilation=1),
                     grid=(256, 1, 1))
    assert out.to_numpy(np.uint16).tolist() == [0xBC00, 0xC000, 0xC000, 0xC000, 0x4200, 0x4400, 0x4100, 0x4800,
                                                0x4A00, 0x4B00, 0x49C0, 0x4400]
    # step
    state = dispatch.Tensor(_buf(runtime, f16_bits([0x3C00, 0x4000, 0x4200, 0x4400, 0x4500, 0x4600])), (1, 2, 3))
    step_out = dispatch.Tensor(_buf(runtime, np.full(2, np.nan, np.float16)), (1, 1, 2))
    dispatch.dispatch_short_conv_step(
        context, in_proj=dispatch.Tensor(_buf(runtime, f16_bits([0x3C00, 0x3C00, 0x4000, 0x3800, 0x3C00, 0x3C00])), (1, 1, 6)),
        conv_state=state, conv_weight=dispatch.Tensor(_buf(runtime, weight), (2, 1, 3)), output=step_out)
    assert step_out.buffer.to_numpy(np.uint16).tolist() == [0x4000, 0x4480]
    assert state.buffer.to_numpy(np.float16).tolist() == [2, 3, 1, 5, 6, 1]
    # prefill
    pre_out = dispatch.Tensor(_buf(runtime, np.full(8, np.nan, np.float16)), (1, 4, 2))
    state_out = dispatch.Tensor(_buf(runtime, np.zeros(6, np.float16)), (1, 2, 3))
    dispatch.dispatch_short_conv_prefill(
        context, in_proj=dispatch.Tensor(_buf(runtime, np.ones(24, np.float16)), (1, 4, 6)),
        conv_weight=dispatch.Tensor(_buf(runtime, weight), (2, 1, 3)), output=pre_out, conv_state_out=state_out)
    assert pre_out.buffer.to_numpy(np.uint16).tolist() == [0xBC00, 0x3800, 0xBC00, 0x3E00, 0x0000, 0x4000, 0x0000, 0x4000]
    assert state_out.buffer.to_numpy(np.uint16).tolist() == [0x3C00] * 6


def test_short_conv_random_vs_oracle(runtime, oracle):
    from llmopt_b200 import dispatch, parameters

    rng = np.random.default_rng(12)
    context = dispatch.Context(runtime)
    channels, tokens = 1024, 37
    weight = rng.standard_normal((channels, 1, 3)).astype(np.float16)
    in_proj = rng.standard_normal((1, tokens, 3 * channels)).astype(np.float16)
    state_in = rng.standard_normal((1, channels, 3)).astype(np.float16)
    for initial in (None, state_in):
        out = dispatch.Tensor(_buf(runtime, np.full((tokens, channels), np.nan, np.float16)), (1, tokens, channels))
        state_out = dispatch.Tensor(_buf(runtime, np.full((channels, 3), np.nan, np.float16)), (1, channels, 3))
        dispatch.dispatch_short_conv_prefill(
            context, in_proj=dispatch.Tensor(_buf(runtime, in_proj), in_proj.shape),
            conv_weight=dispatch.Tensor(_buf(runtime, weight), weight.shape), output=out, conv_state_out=state_out,
            conv_state_in=None if initial is None else dispatch.Tensor(_buf(runtime, initial), initial.shape))
        want, want_state = oracle.short_conv_prefill(in_proj[0], weight.reshape(channels, 3),
                                                     None if initial is None else initial[0])
        assert_close_f16(out.buffer.to_numpy(np.float16, (tokens, channels)), want, rel=1e-3, label="conv prefill")
        assert np.array_equal(state_out.buffer.to_numpy(np.uint16), want_state.view(np.uint16).reshape(-1))
    # one decode step continues the prefill state
    step_in = rng.standard_normal((3 * channels,)).astype(np.float16)
    state = dispatch.Tensor(_buf(runtime, want_state), (1, channels, 3))
    step_out = dispatch.Tensor(_buf(runtime, np.full(channels, np.nan, np.float16)), (1, 1, channels))
    dispatch.dispatch_short_conv_step(context, in_proj=dispatch.Tensor(_buf(runtime, step_in), (1, 1, 3 * channels)),
                                      conv_state=state, conv_weight=dispatch.Tensor(_buf(runtime, weight), weight.shape),
                                      output=step_out)
    want_out, want_next = oracle.short_conv_step(step_in, want_state, weight.reshape(channels, 3))
    assert_close_f16(step_out.buffer.to_numpy(np.float16), want_out, rel=1e-3, label="conv step")
    assert np.array_equal(state.buffer.to_numpy(np.uint16), want_next.view(np.uint16).reshape(-1))
    # token-major conv + SiLU
    x = rng.standard_normal((2, 9, 64)).astype(np.float16)
    w = rng.standard_normal((64, 3)).astype(np.float16)
    out = _buf(runtime, np.full(x.shape, np.nan, np.float16))
    runtime.dispatch("llmopt_short_conv_silu_tm_f16", buffers=[_buf(runtime, x), _buf(runtime, w), out],
                     parameters=parameters.short_conv_silu_tm(batches=2, tokens=9, channels=64, kernel_width=3,
                                                              stride=1, padding=2, dilation=1, output_start=0),
                     grid=(x.size, 1, 1))
    assert_close_f16(out.to_numpy(np.float16, x.shape),
                     oracle.short_conv_silu_tm(x, w, stride=1, padding=2, dilation=1), rel=1.5e-3, label="conv silu")


def test_glue_kernels(runtime, oracle):
    from llmopt_b200 import parameters

    rng = np.random.default_rng(13)
    rows, width = 5, 576
    x = rng.standard_normal((rows, width)).astype(np.float16)
    w = rng.uniform(0.5, 1.5, size=width).astype(np.float16)
    out = _buf(runtime, np.full((rows, width), np.nan, np.float16))
    runtime.dispatch("llmopt_rms_norm_f16_simd", buffers=[_buf(runtime, x), _buf(runtime, w), out],
                     parameters=parameters.rms_norm(rows=rows, width=width, epsilon=1e-5), grid=(256, 1, 1))
    assert_close_f16(out.to_numpy(np.float16, (rows, width)), oracle.rms_norm(x, w, 1e-5), rel=1e-3, label="rms")
    # rotary: token-first in, head-major out, half-precision arithmetic -> bit exact
    b, t, qh, kh, d = 2, 3, 4, 2, 64
    q = rng.standard_normal((b, t, qh, d)).astype(np.float16)
    k = rng.standard_normal((b, t, kh, d)).astype(np.float16)
    angle = rng.uniform(0, 6.28, size=(1, t, d)).astype(np.float32)
    cos, sin = np.cos(angle).astype(np.float16), np.sin(angle).astype(np.float16)
    q_out = _buf(runtime, np.full((b, qh, t, d), np.nan, np.float16))
    k_out = _buf(runtime, np.full((b, kh, t, d), np.nan, np.float16))
    runtime.dispatch("llmopt_rotary_qk_f16_simd_h64",
                     buffers=[_buf(runtime, q), _buf(runtime, k), _buf(runtime, cos), _buf(runtime, sin), q_out, k_out],
                     parameters=parameters.rotary_qk(batches=b, tokens=t, q_heads=qh, k_heads=kh, width=d,
                                                     half_dimension=d // 2, trig_batches=1), grid=(256, 1, 1))
    want_q, want_k = oracle.rotary_qk(q, k, cos, sin, half_dimension=d // 2)
    assert np.array_equal(q_out.to_numpy(np.uint16), want_q.view(np.uint16).reshape(-1))
    assert np.array_equal(k_out.to_numpy(np.uint16), want_k.view(np.uint16).reshape(-1))
    # embedding with an out-of-range id
    table = rng.standard_normal((100, 64)).astype(np.float16)
    ids = np.array([3, 99, 100, -1, 0], np.int64)
    out = _buf(runtime, np.full((5, 64), np.nan, np.float16))
    runtime.dispatch("llmopt_embedding_f16", buffers=[_buf(runtime, ids), _buf(runtime, table), out],
                     parameters=parameters.embedding(tokens=5, vocabulary=100, width=64), grid=(5 * 64, 1, 1))
    assert np.array_equal(out.to_numpy(np.uint16), oracle.embedding_f16(ids, table).view(np.uint16).reshape(-1))
    # last-row argmax, first maximum wins
    logits = np.zeros((2, 50), np.float16)
    logits[1, 7] = logits[1, 30] = 5.0
    assert _buf(runtime, logits).argmax_f16(50) == 7


def test_buffers_batches_and_prebaked(runtime):
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Batch, Buffer, DispatchItem, NativeError, Prebaked

    zero = Buffer.create(runtime, 0)
    assert zero.byte_length() == 16 and zero.contents() == b"\0" * 16
    parent = Buffer.of_bytes(runtime, bytes(range(64)))
    view = parent.view(16, 8)
    assert view.contents() == bytes(range(16, 24))
    view.set_int64(0, -2)
    assert parent.contents()[16:24] == (-2).to_bytes(8, "little", signed=True)
    parent.set_u32_array(0, [7, 9])
    assert np.frombuffer(parent.contents()[:8], np.uint32).tolist() == [7, 9]
    with pytest.raises(ValueError):
        parent.copy_to(view)
    # a batch defers work until commit; abort drops it
    table = np.arange(40, dtype=np.float16).reshape(10, 4)
    out = Buffer.of_array(runtime, np.full((1, 4), np.nan, np.float16))
    ids = Buffer.of_array(runtime, np.array([6], np.int64))
    item = dict(name="llmopt_embedding_f16", buffers=[ids, Buffer.of_array(runtime, table), out],
                parameters=parameters.embedding(tokens=1, vocabulary=10, width=4), grid=(4, 1, 1), group=(256, 1, 1))
    batch = Batch(runtime)
    batch.dispatch(**item)
    batch.abort()
    assert np.isnan(out.to_numpy(np.float16)).all()
    batch = Batch(runtime)
    batch.dispatch(**item)
    with pytest.raises(ValueError, match="overlap"):
        batch.copy(source=parent.view(0, 16), destination=parent.view(8, 16))
    batch.commit()
    assert out.to_numpy(np.float16).tolist() == [24, 25, 26, 27]
    with pytest.raises(NativeError, match="finished"):
        batch.commit()
    # prebaked: token written as int64, row binding gathers row `past_tokens`, output read as int32
    token_buffer = Buffer.create(runtime, 8)
    emb_out = Buffer.create(runtime, 8)
    result = Buffer.create(runtime, 4)
    rows = Buffer.of_array(runtime, np.arange(12, dtype=np.uint32))
    plan = Prebaked(runtime, [
        DispatchItem("llmopt_embedding_f16", [token_buffer, Buffer.of_array(runtime, table), emb_out],
                     parameters.embedding(tokens=1, vocabulary=10, width=4), (4, 1, 1), (256, 1, 1)),
    ], token_buffer, result, row_bindings=[(result, rows, 4)])
    assert plan.execute(token=3, past_tokens=5) == 5
    assert emb_out.to_numpy(np.float16).tolist() == [12, 13, 14, 15]
    assert plan.execute(token=9, past_tokens=11) == 11
    assert emb_out.to_numpy(np.float16).tolist() == [36, 37, 38, 39]
    assert plan.kernel_count() >= 2


@pytest.mark.parametrize("batch,q_heads,k_heads,dim,group", [(1, 8, 2, 128, 64), (3, 4, 4, 64, 32), (2, 6, 2, 128, 64)])
def test_plan_fuses_rotary_and_pair_pack_byte_for_byte(runtime, monkeypatch, batch, q_heads, k_heads, dim, group):
    """A plan runs a rotary record followed by the pair pack of the same token as one kernel; its
    outputs (rotated Q and K, cache bytes and scales) equal the two kernels' bit for bit."""
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer, DispatchItem, Prebaked

    rng = np.random.default_rng(70 + batch)
    q = rng.standard_normal((batch, 1, q_heads, dim)).astype(np.float16)
    k = rng.standard_normal((batch, 1, k_heads, dim)).astype(np.float16)
    v = rng.standard_normal((batch, k_heads, 1, dim)).astype(np.float16)
    v[0, 0, 0, :group] = 0  # an all-zero group takes the scale 1
    angle = rng.uniform(0, 6.28, size=(1, 1, dim))
    cos, sin = np.cos(angle).astype(np.float16), np.sin(angle).astype(np.float16)
    segment = k_heads * dim
    token_elements = 4 * segment  # two layers' K and V; this record packs the second layer
    token_groups = token_elements // group
    token_stride = token_elements + 2 * token_groups
    capacity = 8
    slots = np.array([5, 2, 7][:batch], np.uint32)

    def run(fuse: bool):
        monkeypatch.setenv("LLMOPT_CUDA_FUSE_ROTARY_PACK", "1" if fuse else "0")
        pool = Buffer.of_array(runtime, np.full(capacity * token_stride, 0x55, np.uint8))
        q_out = Buffer.of_array(runtime, np.full(q.shape, np.nan, np.float16))
        k_out = Buffer.of_array(runtime, np.full(k.shape, np.nan, np.float16))
        records = [
            DispatchItem("llmopt_rotary_qk_f16_simd_h64",
                         [Buffer.of_array(runtime, q), Buffer.of_array(runtime, k), Buffer.of_array(runtime, cos),
                          Buffer.of_array(runtime, sin), q_out, k_out],
                         parameters.rotary_qk(batches=batch, tokens=1, q_heads=q_heads, k_heads=k_heads, width=dim,
                                              half_dimension=dim // 2, trig_batches=1),
                         (32 * batch * (q_heads + k_heads), 1, 1), (256, 1, 1)),
            DispatchItem("llmopt_cache_pack_attention_q8_pair_simd",
                         [k_out, Buffer.of_array(runtime, v), Buffer.of_array(runtime, slots), pool],
                         parameters.cache_attention_pair(
                             items=batch, key_segment_offset=2 * segment, value_segment_offset=3 * segment, heads=1,
                             head_dim=segment, group_size=group, token_elements=token_elements,
                             token_groups=token_groups, token_stride=token_stride, source_items=batch, source_offset=0),
                         (32 * batch * segment // group, 1, 1), (256, 1, 1)),
        ]
        plan = Prebaked(runtime, records, None, None)
        plan.execute(token=0, past_tokens=0)
        return plan.kernel_count(), q_out.to_numpy(np.float16), k_out.to_numpy(np.float16), pool.to_numpy(np.uint8)

    fused_kernels, fused_q, fused_k, fused_pool = run(True)
    plain_kernels, plain_q, plain_k, plain_pool = run(False)
    assert fused_kernels == plain_kernels - 1
    assert np.array_equal(fused_q.view(np.uint16), plain_q.view(np.uint16))
    assert np.array_equal(fused_k.view(np.uint16), plain_k.view(np.uint16))
    assert np.array_equal(fused_pool, plain_pool)
    assert not np.array_equal(plain_pool, np.full_like(plain_pool, 0x55))


@pytest.mark.parametrize("batch,q_heads,k_heads,dim,group,past", [(1, 32, 8, 128, 64, 700), (3, 8, 2, 128, 64, 90),
                                                                  (2, 16, 8, 64, 32, 333), (1, 4, 1, 64, 64, 0)])
def test_plan_hands_rotary_and_pack_to_the_attention_byte_for_byte(runtime, monkeypatch, batch, q_heads, k_heads, dim, group, past):
    """Rotary record, pair-pack record and the paged attention of the same token run as one attention launch
    (+ merge): rotated Q and K, the new slot's bytes and scales and the attention output equal what the
    separate kernels write, bit for bit, and the plan is one kernel shorter."""
    from llmopt_b200 import dispatch, parameters
    from llmopt_b200.cuda_native import Batch, Buffer, DispatchItem, Prebaked
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    rng = np.random.default_rng(80 + batch)
    layout = Layout([AttentionLayer(k_heads, dim)] * 2, group_size=group)
    region = layout.attentions[1]
    capacity = past + 5
    q = rng.standard_normal((batch, 1, q_heads, dim)).astype(np.float16)
    k = rng.standard_normal((batch, 1, k_heads, dim)).astype(np.float16)
    v = rng.standard_normal((batch, k_heads, 1, dim)).astype(np.float16)
    angle = rng.uniform(0, 6.28, size=(1, 1, dim))
    cos, sin = np.cos(angle).astype(np.float16), np.sin(angle).astype(np.float16)
    pool_bytes = random_pool(rng, batch * capacity, layout.bytes_per_token, layout.token_elements, group)
    slot_table = np.stack([b * capacity + rng.permutation(capacity) for b in range(batch)]).astype(np.uint32)
    new_slots = np.ascontiguousarray(slot_table[:, past])
    segment = k_heads * dim

    def run(fuse: bool):
        monkeypatch.setenv("LLMOPT_CUDA_FUSE_ROTARY_ATTENTION", "1" if fuse else "0")
        pool = Buffer.of_array(runtime, pool_bytes)
        q_out = Buffer.of_array(runtime, np.full(q.shape, np.nan, np.float16))
        k_out = Buffer.of_array(runtime, np.full(k.shape, np.nan, np.float16))
        v_in = Buffer.of_array(runtime, v)
        out = Buffer.of_array(runtime, np.full((batch, 1, q_heads, dim), np.nan, np.float16))
        commands = Batch(runtime)
        dispatch.dispatch_paged_attention_q8(
            dispatch.Context(runtime, batch=commands),
            config=dispatch.PagedAttentionConfig(token_elements=layout.token_elements, key_offset=region.key_offset,
                                                 value_offset=region.value_offset, group_size=group,
                                                 token_stride=layout.bytes_per_token, scale=1.0 / np.sqrt(dim)),
            query=dispatch.Tensor(q_out, (batch, q_heads, 1, dim)), current_key=dispatch.Tensor(k_out, (batch, k_heads, 1, dim)),
            current_value=dispatch.Tensor(v_in, (batch, k_heads, 1, dim)),
            pool=dispatch.Tensor(pool, (pool_bytes.size,), "uint8"),
            slots=dispatch.Tensor(Buffer.of_array(runtime, np.ascontiguousarray(slot_table[:, :max(past, 1)])),
                                  (batch, past), "uint32"),
            output=dispatch.Tensor(out, (batch, 1, q_heads, dim)), slot_batch_stride=max(past, 1))
        attention = commands.pending[0]
        commands.abort()
        records = [
            DispatchItem("llmopt_rotary_qk_f16_simd_h64",
                         [Buffer.of_array(runtime, q), Buffer.of_array(runtime, k), Buffer.of_array(runtime, cos),
                          Buffer.of_array(runtime, sin), q_out, k_out],
                         parameters.rotary_qk(batches=batch, tokens=1, q_heads=q_heads, k_heads=k_heads, width=dim,
                                              half_dimension=dim // 2, trig_batches=1),
                         (32 * batch * (q_heads + k_heads), 1, 1), (256, 1, 1)),
            DispatchItem("llmopt_cache_pack_attention_q8_pair_simd",
                         [k_out, v_in, Buffer.of_array(runtime, new_slots), pool],
                         parameters.cache_attention_pair(
                             items=batch, key_segment_offset=region.key_offset, value_segment_offset=region.value_offset,
                             heads=1, head_dim=segment, group_size=group, token_elements=layout.token_elements,
                             token_groups=layout.token_groups, token_stride=layout.bytes_per_token, source_items=batch,
                             source_offset=0),
                         (32 * batch * segment // group, 1, 1), (256, 1, 1)),
            attention,
        ]
        plan = Prebaked(runtime, records, None, None)
        plan.execute(token=0, past_tokens=past)
        return (plan.kernel_count(), q_out.to_numpy(np.uint16), k_out.to_numpy(np.uint16), pool.to_numpy(np.uint8),
                out.to_numpy(np.uint16))

    fused, plain = run(True), run(False)
    assert fused[0] == plain[0] - 1
    for index, label in ((1, "rotated query"), (2, "rotated key"), (3, "pool"), (4, "attention output")):
        assert np.array_equal(fused[index], plain[index]), label
    assert not np.array_equal(plain[3], pool_bytes)
    assert not np.any(np.isnan(plain[4].view(np.float16)))


def test_plan_refuses_tokens_beyond_its_tables(runtime):
    """A replayed plan indexes device tables with the per-token values it is given: a row binding
    reads row ``past_tokens``, paged attention reads ``past_tokens`` slot entries.  Values beyond
    the captured tables are refused on the host instead of read on the device."""
    from llmopt_b200 import dispatch, parameters
    from llmopt_b200.cuda_native import Batch, Buffer, DispatchItem, Prebaked

    table = np.arange(40, dtype=np.float16).reshape(10, 4)
    token_buffer, emb_out, result = Buffer.create(runtime, 8), Buffer.create(runtime, 8), Buffer.create(runtime, 4)
    rows = Buffer.of_array(runtime, np.arange(12, dtype=np.uint32))
    plan = Prebaked(runtime, [
        DispatchItem("llmopt_embedding_f16", [token_buffer, Buffer.of_array(runtime, table), emb_out],
                     parameters.embedding(tokens=1, vocabulary=10, width=4), (4, 1, 1), (256, 1, 1)),
    ], token_buffer, result, row_bindings=[(result, rows, 4)])
    assert plan.token_capacity() == 11
    assert plan.execute(token=3, past_tokens=11) == 11
    with pytest.raises(ValueError, match="token capacity"):
        plan.execute(token=3, past_tokens=12)
    with pytest.raises(ValueError, match="token capacity"):
        plan.execute_chained(token=3, past_tokens=10, steps=3)
    with pytest.raises(ValueError, match="negative"):
        plan.execute(token=3, past_tokens=-1)
    # a paged-attention record bounds the plan by its slot table: 2 sequences x 20 entries
    pool = random_pool(np.random.default_rng(0), 64, 132, 128, 64)
    config = dispatch.PagedAttentionConfig(token_elements=128, key_offset=0, value_offset=64, group_size=64,
                                           token_stride=132, scale=1.0)
    commands = Batch(runtime)
    context = dispatch.Context(runtime, batch=commands, decode_uniforms_past_tokens=4)
    slots = np.arange(40, dtype=np.uint32).reshape(2, 20)
    out = _tensor(runtime, np.zeros((2, 1, 2, 64), np.float16))
    dispatch.dispatch_paged_attention_q8(
        context, config=config, query=_tensor(runtime, np.ones((2, 2, 1, 64), np.float16)),
        current_key=_tensor(runtime, np.ones((2, 1, 1, 64), np.float16)),
        current_value=_tensor(runtime, np.ones((2, 1, 1, 64), np.float16)),
        pool=dispatch.Tensor(_buf(runtime, pool), (pool.size,), "uint8"),
        slots=dispatch.Tensor(_buf(runtime, slots), slots.shape, "uint32"), output=out, slot_batch_stride=20)
    records = list(commands.pending)
    commands.abort()
    plan = Prebaked(runtime, records, None, None)
    assert plan.token_capacity() == 20
    plan.execute(token=0, past_tokens=20)
    with pytest.raises(ValueError, match="token capacity"):
        plan.execute(token=0, past_tokens=21)


def test_slots_outside_the_pool_are_refused_on_the_device(runtime):
    """A slot value beyond the pool's rows is never dereferenced: the pack skips the item, the
    attention reads nothing outside the pool, and the next stream wait reports the error; the
    context stays usable."""
    from llmopt_b200 import dispatch, parameters
    from llmopt_b200.cuda_native import Buffer, NativeError

    rng = np.random.default_rng(5)
    capacity = 8
    pool_bytes = np.full(capacity * 132, 0x11, np.uint8)
    pool = Buffer.of_array(runtime, pool_bytes)
    key = Buffer.of_array(runtime, rng.standard_normal((2, 64)).astype(np.float16))
    value = Buffer.of_array(runtime, rng.standard_normal((2, 64)).astype(np.float16))
    pair = parameters.cache_attention_pair(items=2, key_segment_offset=0, value_segment_offset=64, heads=1, head_dim=64,
                                           group_size=64, token_elements=128, token_groups=2, token_stride=132,
                                           source_items=2, source_offset=0)
    with pytest.raises(NativeError, match="outside its pool"):
        runtime.dispatch("llmopt_cache_pack_attention_q8_pair_simd",
                         buffers=[key, value, Buffer.of_array(runtime, np.array([3, capacity], np.uint32)), pool],
                         parameters=pair, grid=(64, 1, 1))
    after = pool.to_numpy(np.uint8).reshape(capacity, 132)
    assert not np.array_equal(after[3], pool_bytes[:132])           # the valid item was packed
    assert np.array_equal(np.delete(after, 3, axis=0).reshape(-1), np.delete(pool_bytes.reshape(capacity, 132), 3, axis=0).reshape(-1))
    # a segment that does not fit the token row is refused before any launch
    bad = parameters.cache_attention_pair(items=1, key_segment_offset=64, value_segment_offset=128, heads=1, head_dim=64,
                                          group_size=64, token_elements=128, token_groups=2, token_stride=132,
                                          source_items=1, source_offset=0)
    with pytest.raises(NativeError, match="outside the token row"):
        runtime.dispatch("llmopt_cache_pack_attention_q8_pair_simd",
                         buffers=[key, value, Buffer.of_array(runtime, np.array([0], np.uint32)), pool],
                         parameters=bad, grid=(64, 1, 1))
    # attention (split path and row path) with a slot beyond the pool
    real_pool = random_pool(rng, capacity, 132, 128, 64)
    config = dispatch.PagedAttentionConfig(token_elements=128, key_offset=0, value_offset=64, group_size=64,
                                           token_stride=132, scale=0.125)
    for window in (None, 64):
        slots = np.array([0, 1, 2] + [3] * 38 + [capacity + 5] + [4] * 38, np.uint32)  # the bad slot lies inside the window
        out = _tensor(runtime, np.full((1, 1, 2, 64), np.nan, np.float16))
        with pytest.raises(NativeError, match="outside its pool"):
            dispatch.dispatch_paged_attention_q8(
                dispatch.Context(runtime), config=dispatch.PagedAttentionConfig(**{**config.__dict__, "window": window}),
                query=_tensor(runtime, rng.standard_normal((1, 2, 1, 64)).astype(np.float16)),
                current_key=_tensor(runtime, rng.standard_normal((1, 1, 1, 64)).astype(np.float16)),
                current_value=_tensor(runtime, rng.standard_normal((1, 1, 1, 64)).astype(np.float16)),
                pool=dispatch.Tensor(_buf(runtime, real_pool), (real_pool.size,), "uint8"),
                slots=dispatch.Tensor(_buf(runtime, slots), slots.shape, "uint32"), output=out)
            runtime.synchronize()
        assert np.all(np.isfinite(out.buffer.to_numpy(np.float16)))
    runtime.synchronize()  # the context is still usable


@pytest.mark.parametrize("in_place", [False, True])
def test_plan_folds_only_norms_whose_rows_do_not_alias(runtime, monkeypatch, in_place):
    """An RMS norm is folded into the W4A16 product that consumes it only when the raw rows and the
    normalised rows are different memory; an in-place norm (or overlapping views) keeps its own
    kernel.  Either way the plan's buffers equal the unfolded plan's byte for byte."""
    from helpers import random_w4
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer, DispatchItem, Prebaked

    rng = np.random.default_rng(31)
    rows, k, n = 2, 1024, 320
    x = rng.standard_normal((rows, k)).astype(np.float16)
    weight = rng.uniform(0.5, 1.5, size=k).astype(np.float16)
    packed, scale = random_w4(rng, n, k)

    def run(fold: bool):
        monkeypatch.setenv("LLMOPT_CUDA_FOLD_NORMS", "1" if fold else "0")
        raw = Buffer.of_array(runtime, x)
        normed = raw if in_place else Buffer.create(runtime, rows * k * 2)
        out = Buffer.of_array(runtime, np.full((rows, n), np.nan, np.float16))
        scales = Buffer.of_array(runtime, scale)
        records = [
            DispatchItem("llmopt_rms_norm_f16_simd", [raw, Buffer.of_array(runtime, weight), normed],
                         parameters.rms_norm(rows=rows, width=k, epsilon=1e-5), (256, 1, 1), (256, 1, 1)),
            DispatchItem("llmopt_w4a16_linear_f16_g64_m4",
                         [normed, Buffer.of_array(runtime, packed), scales, scales, out],
                         parameters.u32s([rows, n, k, 0, 0]), (256, 1, 1), (256, 1, 1)),
        ]
        plan = Prebaked(runtime, records, None, None)
        plan.execute(token=0, past_tokens=0)
        return plan.kernel_count(), normed.to_numpy(np.uint16), out.to_numpy(np.uint16)

    folded_kernels, folded_rows, folded_out = run(True)
    plain_kernels, plain_rows, plain_out = run(False)
    assert folded_kernels == (plain_kernels if in_place else plain_kernels - 1)
    assert np.array_equal(folded_rows, plain_rows)
    assert np.array_equal(folded_out, plain_out)
    assert not np.any(np.isnan(plain_out.view(np.float16)))
