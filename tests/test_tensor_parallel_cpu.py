"""Host-side logic of the tensor-parallel path, without a GPU: the slot plan, the weight
sharding, and -- as two gloo ranks on CPU -- that the sharded products, exchanged the way the
exchange kernels combine them, reproduce the unsharded oracle result."""

import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from helpers import random_w4
from llmopt_b200 import tensor_parallel
from llmopt_b200.model import LLAMA3_8B, LFM25_350M, SMOLLM2_135M, random_weights, tiny_config


def test_slot_plan_never_reuses_a_slot_in_adjacent_exchanges():
    for exchanges in range(2, 400):
        count, slots = tensor_parallel.plan_slots(exchanges)
        assert len(slots) == exchanges and 3 <= count <= 7 and max(slots) < count
        assert tensor_parallel.check_slot_plan(slots), exchanges
    assert tensor_parallel.plan_slots(0) == (0, [])
    with pytest.raises(ValueError):
        tensor_parallel.plan_slots(1)
    assert tensor_parallel.plan_slots(65)[0] == 3 and tensor_parallel.plan_slots(64)[0] == 4  # 64 % 3 == 1
    assert not tensor_parallel.check_slot_plan([0, 1, 2, 0])  # wraps 0 -> 0


def test_prompt_slot_order_fits_between_decode_steps():
    for slot_count in (3, 4, 5, 7):
        for layers in (1, 2, 16, 32):
            decode_count, decode = tensor_parallel.plan_slots(2 * layers + 1)
            if decode_count > slot_count:
                continue
            slots = tensor_parallel.plan_prompt_slots(slot_count, 4 * layers + 1, decode)
            assert len(slots) == 4 * layers + 1 and max(slots) < slot_count
            sequence = list(decode) + slots + list(decode)  # a step, the prompt, a step
            assert all(a != b for a, b in zip(sequence, sequence[1:])), (slot_count, layers)
    with pytest.raises(ValueError):
        tensor_parallel.plan_prompt_slots(2, 9, [0, 1])


class _FakeBuffer:
    pass


def test_prompt_row_shares_cover_the_rows_once():
    for rows in (1, 2, 5, 8, 70, 512):
        for world in (1, 2, 4, 8):
            shares = [tensor_parallel.prompt_row_share(rows, world, rank) for rank in range(world)]
            assert shares[0][0] == 0 and shares[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(shares, shares[1:]))
            assert max(hi - lo for lo, hi in shares) == (rows + world - 1) // world


def test_prompt_row_exchange_records():
    import struct

    regions = [_FakeBuffer() for _ in range(4)]
    group = tensor_parallel.ExchangeGroup(1, 4, 8 * 4096 * 4, 3, regions)
    seen = []
    record = lambda **item: seen.append(item) or item
    residual, output = _FakeBuffer(), _FakeBuffer()
    first, second = group.sum_rows_records(record, slot=2, slice_slot=0, rows=8, width=4096, residual=residual, output=output)
    assert [item["name"] for item in seen] == ["llmopt_tp_exchange_reduce_rows_f16", "llmopt_tp_exchange_gather_rows_f16"]
    assert first["buffers"] == regions + [residual, output] and second["buffers"] == regions + [output]
    assert first["parameters"] == second["parameters"] and len(first["parameters"]) == 28
    assert struct.unpack("<7I", first["parameters"]) == (4, 1, 8, 4096, group.slot_offset(2), 1, group.slot_offset(0))
    without = group.sum_rows_records(record, slot=1, slice_slot=2, rows=3, width=64, residual=None, output=output)[0]
    assert struct.unpack("<7I", without["parameters"])[5] == 0 and without["buffers"][-2:] == [output, output]
    with pytest.raises(ValueError):
        group.sum_rows_records(record, slot=1, slice_slot=1, rows=8, width=4096, residual=None, output=output)
    with pytest.raises(ValueError):
        group.sum_rows_records(record, slot=0, slice_slot=1, rows=9, width=4096, residual=None, output=output)
    with pytest.raises(ValueError):
        group.slot_offset(3)


def test_which_models_shard():
    assert all(tensor_parallel.shards(LLAMA3_8B, world) for world in (1, 2, 4, 8))
    assert not tensor_parallel.shards(LLAMA3_8B, 3) and not tensor_parallel.shards(LLAMA3_8B, 16)
    assert tensor_parallel.shards(SMOLLM2_135M, 1) and not tensor_parallel.shards(SMOLLM2_135M, 2)  # 3 KV heads
    assert not tensor_parallel.shards(LFM25_350M, 2)  # conv blocks are not sharded
    local = tensor_parallel.local_config(LLAMA3_8B, 8)
    assert (local.query_heads, local.kv_heads, local.intermediate, local.vocabulary) == (4, 1, 1792, 16032)
    with pytest.raises(ValueError):
        tensor_parallel.local_config(SMOLLM2_135M, 2)


def test_shards_reassemble_to_the_whole_model():
    config = tiny_config(layers=("attention",) * 2, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                         vocabulary=512)
    weights = random_weights(config, seed=1)
    world = 2
    parts = [tensor_parallel.shard_weights(config, weights, rank, world) for rank in range(world)]
    for name in ("q", "k", "v", "gate", "up"):  # column split: rows concatenate
        for i in range(2):
            whole = np.concatenate([p["layer0"][name][i] for p in parts], axis=0)
            assert np.array_equal(whole, weights["layer0"][name][i])
    for name in ("o", "down"):  # row split: K slices concatenate
        for i in range(2):
            whole = np.concatenate([p["layer1"][name][i] for p in parts], axis=1)
            assert np.array_equal(whole, weights["layer1"][name][i])
    assert np.array_equal(np.concatenate([p["lm_head"][0] for p in parts]), weights["lm_head"][0])
    assert parts[0]["embedding"] is weights["embedding"]


def test_row_split_partials_sum_to_the_whole_product(oracle):
    rng = np.random.default_rng(5)
    m, k, n, world = 3, 512, 96, 4
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    residual = rng.standard_normal((m, n)).astype(np.float16)
    total = np.zeros((m, n), np.float32)
    for rank in range(world):
        lo, hi = rank * k // world, (rank + 1) * k // world
        part = oracle.w4a16_linear_f64(np.ascontiguousarray(x[:, lo:hi]), np.ascontiguousarray(packed[:, lo // 2:hi // 2]),
                                       np.ascontiguousarray(scale[:, lo // 64:hi // 64]))
        total += part.astype(np.float32)  # the exchange adds fp32 partials in rank order
    got = (total + residual.astype(np.float32)).astype(np.float16)
    want = oracle.w4a16_linear(x, packed, scale, residual, n)
    error = np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / np.max(np.abs(want.astype(np.float64)))
    assert error <= 2e-3


def _free_port() -> int:
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def test_two_gloo_ranks_reproduce_the_unsharded_layer(tmp_path):
    """world_size 2 on CPU: each rank computes its shard of one decoder layer's linears with the
    oracle, the exchanges are a gloo all_reduce (sum of fp32 partials) and all_gather (argmax
    candidates); both ranks must end with the oracle's unsharded hidden state and token."""
    worker = os.path.join(os.path.dirname(__file__), "tp_gloo_worker.py")
    port = _free_port()
    processes = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TP_OUT=str(tmp_path / f"rank{rank}.npz"))
        processes.append(subprocess.Popen([sys.executable, worker], env=env, stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT))
    outputs = [p.communicate(timeout=240)[0].decode() for p in processes]
    assert all(p.returncode == 0 for p in processes), "\n".join(outputs)
    results = [np.load(tmp_path / f"rank{rank}.npz") for rank in range(2)]
    assert np.array_equal(results[0]["hidden"], results[1]["hidden"])  # same bits on every rank
    assert int(results[0]["token"]) == int(results[1]["token"]) == int(results[0]["want_token"])
    # prompt rows through the reduce-scatter / all-gather form of the exchange: same bits on both ranks, oracle's result
    assert np.array_equal(results[0]["rows"].view(np.uint16), results[1]["rows"].view(np.uint16))
    assert float(results[0]["rows_error"]) <= 2e-3
    error = float(results[0]["error"])
    assert error <= 2e-3, error
