"""Tensor-parallel exchange kernels and plan on the GPU.

On one GPU the peers cannot run (kernels that wait on one another must not share a GPU), so the
single-GPU cases stage the peer's contribution and flag from the host before this rank's kernel
is launched: the kernel finds the peer already announced and never waits on another kernel.
The two-rank case runs as two processes on two GPUs when the box has them."""

import os
import socket
import struct
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HEADER = 256
FLAGS = 64


def _dispatch(runtime, name, buffers, params):
    from llmopt_b200.cuda_native import Batch

    batch = Batch(runtime)
    batch.dispatch(name=name, buffers=buffers, parameters=params, grid=(256, 1, 1), group=(256, 1, 1))
    batch.commit()


def test_exchange_sum_two_ranks_staged_peer(runtime):
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(0)
    rows, width, slot_bytes = 3, 512, 8192
    regions = [Buffer.create(runtime, HEADER + 2 * slot_bytes) for _ in range(2)]  # rank 0 = "this" rank
    residual = rng.standard_normal((rows, width)).astype(np.float16)
    residual_buffer = Buffer.of_array(runtime, residual)
    output = Buffer.create(runtime, rows * width * 2)
    for epoch, slot in ((1, 0), (2, 1)):  # two exchanges in a row: the epoch advances on the device
        mine = rng.standard_normal((rows, width)).astype(np.float32)
        theirs = rng.standard_normal((rows, width)).astype(np.float32)
        offset = HEADER + slot * slot_bytes
        regions[0].write(offset, mine)
        regions[1].write(offset, theirs)
        regions[0].write(FLAGS + 4, np.array([epoch], np.uint32))  # the peer (rank 1) has announced `epoch`
        _dispatch(runtime, "llmopt_tp_exchange_sum_f16", regions + [residual_buffer, output],
                  parameters.u32s([2, 0, rows, width, offset, 1]))
        got = output.to_numpy(np.float16, (rows, width))
        want = ((mine + theirs) + residual.astype(np.float32)).astype(np.float16)  # rank order 0, 1, then residual
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
        header0 = regions[0].view(0, HEADER).to_numpy(np.uint32)
        header1 = regions[1].view(0, HEADER).to_numpy(np.uint32)
        assert header0[0] == epoch and header0[1] == 0  # epoch published, arrival counter back to zero
        assert header0[FLAGS // 4] == epoch and header1[FLAGS // 4] == epoch  # rank 0 announced to both regions


def test_exchange_rows_reduce_then_gather_staged_peer(runtime):
    """Prompt rows: rank 0 of two reduces ITS rows from both partials (reduce-scatter), then copies the
    peer's rows from the peer's fp16 share (all-gather); the peer's contribution, share and flags are staged."""
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(5)
    rows, width = 7, 256  # shares: rows 0..3 (rank 0), 4..6 (rank 1)
    slot_bytes = rows * width * 4
    regions = [Buffer.create(runtime, HEADER + 2 * slot_bytes) for _ in range(2)]
    residual = rng.standard_normal((rows, width)).astype(np.float16)
    mine = rng.standard_normal((rows, width)).astype(np.float32)
    theirs = rng.standard_normal((rows, width)).astype(np.float32)
    total = ((mine + theirs) + residual.astype(np.float32)).astype(np.float16)
    partial_offset, share_offset = HEADER, HEADER + slot_bytes
    regions[0].write(partial_offset, mine)
    regions[1].write(partial_offset, theirs)
    peer_share = np.zeros((rows, width), np.float16)
    peer_share[4:] = total[4:]  # what rank 1's reduce step leaves in its own region
    regions[1].write(share_offset, peer_share)
    output = Buffer.of_array(runtime, np.full((rows, width), np.nan, np.float16))
    params = parameters.u32s([2, 0, rows, width, partial_offset, 1, share_offset])
    regions[0].write(FLAGS + 4, np.array([1], np.uint32))  # the peer has announced exchange 1 (partials written)
    _dispatch(runtime, "llmopt_tp_exchange_reduce_rows_f16", regions + [Buffer.of_array(runtime, residual), output], params)
    got = output.to_numpy(np.float16, (rows, width))
    assert np.array_equal(got[:4].view(np.uint16), total[:4].view(np.uint16))
    assert np.all(np.isnan(got[4:]))  # the peer's rows are not this step's
    own_share = regions[0].view(share_offset, rows * width * 2).to_numpy(np.float16, (rows, width))
    assert np.array_equal(own_share[:4].view(np.uint16), total[:4].view(np.uint16))
    regions[0].write(FLAGS + 4, np.array([2], np.uint32))  # the peer has announced exchange 2 (its share written)
    _dispatch(runtime, "llmopt_tp_exchange_gather_rows_f16", regions + [output], params)
    got = output.to_numpy(np.float16, (rows, width))
    assert np.array_equal(got.view(np.uint16), total.view(np.uint16))
    header0 = regions[0].view(0, HEADER).to_numpy(np.uint32)
    assert header0[0] == 2 and header0[1] == 0


def test_exchange_argmax_two_ranks_staged_peer(runtime):
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(1)
    rows, parts, shard = 2, 256, 1000
    regions = [Buffer.create(runtime, HEADER + rows * parts * 8) for _ in range(2)]
    candidates = []
    for rank in range(2):
        values = rng.standard_normal((rows, parts)).astype(np.float32)
        indices = rng.integers(0, shard, size=(rows, parts)).astype(np.uint32)
        candidates.append((values, indices))
    # row 0: the peer holds the maximum; row 1: an exact tie, the lower global index (rank 0) wins
    candidates[1][0][0, 17] = 9.0
    candidates[1][1][0, 17] = 123
    candidates[0][0][1, 5] = 7.5
    candidates[0][1][1, 5] = 900
    candidates[1][0][1, 200] = 7.5
    candidates[1][1][1, 200] = 3
    for rank in range(2):
        packed = np.empty((rows, parts, 2), np.uint32)
        packed[..., 0] = candidates[rank][0].view(np.uint32)
        packed[..., 1] = candidates[rank][1]
        regions[rank].write(HEADER, packed)
    regions[0].write(FLAGS + 4, np.array([1], np.uint32))
    tokens = Buffer.create(runtime, rows * 4)
    _dispatch(runtime, "llmopt_tp_exchange_argmax", regions + [tokens], parameters.u32s([2, 0, rows, parts, HEADER, shard]))
    assert tokens.to_numpy(np.uint32).tolist() == [shard + 123, 900]


def test_exchange_reports_a_peer_that_never_arrives(runtime):
    """The wait on a peer is bounded (about two seconds): a flag that nothing sets ends the kernel
    with the context's error raised at the next stream wait, and the context stays usable."""
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer, NativeError

    regions = [Buffer.create(runtime, HEADER + 4096) for _ in range(2)]
    output = Buffer.create(runtime, 4 * 64 * 2)
    with pytest.raises(NativeError):
        _dispatch(runtime, "llmopt_tp_exchange_sum_f16", regions + [output, output], parameters.u32s([2, 0, 4, 64, HEADER, 0]))
        runtime.synchronize()
    # the context still works: a group of one needs no peer
    single = Buffer.create(runtime, HEADER + 4096)
    single.write(HEADER, np.ones((4, 64), np.float32))
    _dispatch(runtime, "llmopt_tp_exchange_sum_f16", [single, output, output], parameters.u32s([1, 0, 4, 64, HEADER, 0]))
    assert np.all(output.to_numpy(np.float16) == 1.0)


def test_partial_f32_linear_matches_oracle(runtime, oracle):
    from helpers import random_w4
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer

    rng = np.random.default_rng(2)
    m, k, n = 2, 1024, 320
    x = rng.standard_normal((m, k)).astype(np.float16)
    packed, scale = random_w4(rng, n, k)
    out = Buffer.create(runtime, m * n * 4)
    _dispatch(runtime, "llmopt_w4a16_linear_partial_f32_g64",
              [Buffer.of_array(runtime, x), Buffer.of_array(runtime, packed), Buffer.of_array(runtime, scale), out],
              parameters.u32s([m, n, k]))
    got = out.to_numpy(np.float32, (m, n)).astype(np.float64)
    want = oracle.w4a16_linear_f64(x, packed, scale)
    assert np.max(np.abs(got - want)) <= 1e-4 * np.max(np.abs(want))  # fp32 accumulation against float64


def test_single_rank_plan_through_the_exchange_kernels(runtime):
    """The tensor-parallel record list with a group of one: partial fp32 products, exchange sums and
    the exchange argmax reproduce the oracle's greedy tokens like the plain plan does."""
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights, tiny_config
    from llmopt_b200.tensor_parallel import CANDIDATE_PARTS, ExchangeGroup
    from oracle_model import OracleDecoder

    config = tiny_config(layers=("attention",) * 2, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                         vocabulary=1024)
    weights = random_weights(config, seed=4, std=0.05)
    steps, prompt = 24, [5, 77, 301, 12]
    group = ExchangeGroup.create(runtime, 0, 1, max(config.hidden * 4, CANDIDATE_PARTS * 8), 7)
    engine = DecodeEngine(runtime, config, weights, batch=1, capacity=len(prompt) + steps + 1, group=group)
    cpu = OracleDecoder(config, weights, len(prompt) + steps + 1)
    got, want = [], []
    token_gpu = token_cpu = None
    for position, token in enumerate(prompt):
        token_gpu = engine.step([token], position)[0]
        token_cpu, _ = cpu.step(token)
    for step in range(steps):
        got.append(token_gpu)
        want.append(token_cpu)
        token_gpu = engine.step([token_gpu], len(prompt) + step)[0]
        token_cpu, _ = cpu.step(token_cpu)
    assert got == want
    assert any(record.name == "llmopt_tp_exchange_sum_f16" for record in engine.records)


def test_single_rank_prefill_through_the_exchange_kernels(runtime):
    """The tensor-parallel prompt pass with a group of one: fp32 partial products of all prompt rows,
    exchange sums over rows x hidden slots and the exchange argmax, then decode over the cache the prompt left:
    the oracle's dense-prefill route."""
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights, tiny_config
    from llmopt_b200.tensor_parallel import CANDIDATE_PARTS, ExchangeGroup
    from oracle_model import OracleDecoder

    config = tiny_config(layers=("attention",) * 2, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                         vocabulary=1024)
    weights = random_weights(config, seed=4, std=0.05)
    prompt = np.random.default_rng(9).integers(0, config.vocabulary, size=70).tolist()
    steps, capacity = 16, len(prompt) + 17
    group = ExchangeGroup.create(runtime, 0, 1, max(len(prompt) * config.hidden * 4, CANDIDATE_PARTS * 8), 7)
    engine = DecodeEngine(runtime, config, weights, batch=1, capacity=capacity, group=group)
    cpu = OracleDecoder(config, weights, capacity)
    want, _ = cpu.prefill_dense(prompt)
    got = engine.prefill(prompt)
    assert got == want
    for step in range(steps):
        got = engine.step([want], len(prompt) + step)[0]
        want_next, logits = cpu.step(want, want_logits=True)
        if got != want_next:
            row = logits[0].astype(np.float64)
            gap = abs(row[want_next] - row[got]) / max(np.max(np.abs(row)), 1e-6)
            assert gap <= 5e-3, f"step {step}: {got} != {want_next}, logit gap {gap:.3e}"
        want = want_next


def _free_port() -> int:
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def _device_count() -> int:
    try:
        output = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
    except (OSError, subprocess.TimeoutExpired):
        return 0
    return sum(1 for line in output.splitlines() if line.startswith("GPU "))


@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus_match_the_single_gpu_tokens(tmp_path):
    """Two processes, one GPU each: the sharded decode produces the oracle's tokens on both ranks."""
    worker = os.path.join(os.path.dirname(__file__), "tp_gpu_worker.py")
    port = _free_port()
    processes = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), TP_OUT=str(tmp_path / f"rank{rank}.npz"), NCCL_NVLS_ENABLE="0")
        processes.append(subprocess.Popen([sys.executable, worker], env=env, stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT))
    outputs = [p.communicate(timeout=600)[0].decode() for p in processes]
    assert all(p.returncode == 0 for p in processes), "\n".join(outputs)
    results = [np.load(tmp_path / f"rank{rank}.npz") for rank in range(2)]
    assert results[0]["tokens"].tolist() == results[1]["tokens"].tolist() == results[0]["want"].tolist()
    # the sharded prompt pass (rows x hidden partial sums exchanged) and the decode after it
    assert results[0]["prompt_tokens"].tolist() == results[1]["prompt_tokens"].tolist()
    assert results[0]["prompt_tokens"].tolist() == results[0]["prompt_want"].tolist()
