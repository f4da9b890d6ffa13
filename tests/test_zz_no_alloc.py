"""The allocation-free attention entry point against the regular one.

`llmopt_cuda_attention_q8_paged_static` serves hosts that cannot let the library
allocate device memory (their own pools own all of HBM, or an allocation's
implicit device-wide synchronisation is not acceptable where they call from): it
keeps the split scratch in an array inside the library image instead of the
context's growable scratch.  Here it is called twice in a row, on two different
problems, through the C ABI on raw device pointers, and each result must match
both the CPU oracle's paged attention on the same arrays and the regular
`llmopt_attention_q8_paged_*` dispatch, within the fp16 parity bound (the second
call also shows that whatever the first left in the shared array does not leak
into the next result).  Collected last so a failure here cannot hide another
test's result."""

import ctypes

import numpy as np
import pytest

from conftest import assert_close_f16
from helpers import random_pool

pytestmark = pytest.mark.gpu


def _problem(runtime, oracle, seed, *, batches, hq, hkv, dim, group, past):
    from llmopt_b200 import dispatch, parameters
    from llmopt_b200.cuda_native import Buffer
    from llmopt_b200.kv_cache import AttentionLayer, Layout

    rng = np.random.default_rng(seed)
    layout = Layout([AttentionLayer(hkv, dim)] * 2, group_size=group)
    capacity = batches * past + 5
    pool = random_pool(rng, capacity, layout.bytes_per_token, layout.token_elements, group)
    slots = np.stack([rng.permutation(capacity)[:past] for _ in range(batches)]).astype(np.uint32)
    region = layout.attentions[1]
    arrays = dict(
        query=(rng.standard_normal((batches, hq, 1, dim)) * 2).astype(np.float16),
        key=rng.standard_normal((batches, hkv, 1, dim)).astype(np.float16),
        value=rng.standard_normal((batches, hkv, 1, dim)).astype(np.float16),
        pool=pool, slots=np.ascontiguousarray(slots))
    buffers = {name: Buffer.of_array(runtime, array) for name, array in arrays.items()}
    fields = dict(batches=batches, query_heads=hq, kv_heads=hkv, past_length=past, head_dimension=dim,
                  mask_batches=0, mask_heads=0, token_elements=layout.token_elements, key_offset=region.key_offset,
                  value_offset=region.value_offset, group_size=group, token_stride=layout.bytes_per_token,
                  scale=float(np.float32(1 / np.sqrt(dim))), mask_dtype=0)
    shape = (batches, 1, hq, dim)
    # the regular entry point: a named dispatch whose scratch comes from the context
    regular = Buffer.of_array(runtime, np.full(shape, np.nan, np.float16))
    runtime.dispatch("llmopt_attention_q8_paged_batched",
                     buffers=[buffers["query"], buffers["key"], buffers["value"], buffers["pool"], buffers["slots"],
                              buffers["slots"], regular],
                     parameters=parameters.paged_attention_q8_batched(slot_batch_stride=past, **fields),
                     grid=(batches * hq * 32, 1, 1))
    block = parameters.paged_attention_q8(**fields)
    expected = oracle.attention_q8_paged(arrays["query"], arrays["key"], arrays["value"], pool, arrays["slots"], None,
                                         block, slot_batch_stride=past)
    return buffers, block, expected, regular.to_numpy(np.float16, shape), shape


def _call_static(buffers, block, shape, stride, runtime):
    from llmopt_b200 import cuda_native
    from llmopt_b200.cuda_native import Buffer

    lib = cuda_native.load_library()
    output = Buffer.of_array(runtime, np.full(shape, np.nan, np.float16))
    status = lib.llmopt_cuda_attention_q8_paged_static(
        buffers["query"].device_pointer(), buffers["key"].device_pointer(), buffers["value"].device_pointer(),
        buffers["pool"].device_pointer(), buffers["slots"].device_pointer(), output.device_pointer(),
        block, len(block), stride, None)
    assert status == 0, lib.llmopt_cuda_last_error().decode()
    cudart = ctypes.CDLL("libcudart.so.12")  # the call ran on the default stream: wait for the device
    assert cudart.cudaDeviceSynchronize() == 0
    return output.to_numpy(np.float16, shape)


def test_static_scratch_entry_matches_oracle_and_regular_entry_twice(runtime, oracle):
    from llmopt_b200 import cuda_native

    first = _problem(runtime, oracle, 21, batches=3, hq=32, hkv=8, dim=128, group=64, past=700)
    second = _problem(runtime, oracle, 22, batches=2, hq=9, hkv=3, dim=64, group=64, past=257)
    for index, (buffers, block, expected, regular, shape) in enumerate((first, second)):
        past = int(np.frombuffer(block, np.uint32)[3])
        got = _call_static(buffers, block, shape, past, runtime)
        assert_close_f16(got, np.asarray(expected).reshape(shape), label=f"static entry vs oracle, call {index + 1}")
        assert_close_f16(got, regular, label=f"static entry vs regular entry, call {index + 1}")
    # a problem with more (batch, kv head) pairs than the fixed array has records is refused, not truncated
    lib = cuda_native.load_library()
    buffers, block, _, _, _ = first
    huge = bytearray(block)
    huge[0:4] = (300).to_bytes(4, "little")  # 300 batches x 8 kv heads = 2400 records > 2016
    pointer = buffers["query"].device_pointer()
    status = lib.llmopt_cuda_attention_q8_paged_static(pointer, pointer, pointer, pointer, pointer, pointer,
                                                       bytes(huge), len(huge), 700, None)
    assert status == 2 and b"exceeds" in lib.llmopt_cuda_last_error()
    # head size 64: 2112-byte records, 3971 fit; 1324 batches x 3 kv heads = 3972 is one too many
    small = bytearray(second[1])
    small[0:4] = (1324).to_bytes(4, "little")
    status = lib.llmopt_cuda_attention_q8_paged_static(pointer, pointer, pointer, pointer, pointer, pointer,
                                                       bytes(small), len(small), 257, None)
    assert status == 2 and b"3971" in lib.llmopt_cuda_last_error()
    status = lib.llmopt_cuda_attention_q8_paged_static(pointer, pointer, pointer, pointer, pointer, pointer,
                                                       bytes(block[:60]), 60, 700, None)
    assert status == 2
