"""Whole-token greedy decode on the GPU against the CPU oracle executing the same
op sequence: token-identical output, host-driven and device-chained."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(runtime, config, prompt_length, steps, batch=1, seed=0):
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights
    from oracle_model import OracleDecoder

    weights = random_weights(config, seed=seed, std=0.05)
    rng = np.random.default_rng(seed)
    prompts = rng.integers(0, config.vocabulary, size=(batch, prompt_length))
    capacity = prompt_length + steps + 1
    engine = DecodeEngine(runtime, config, weights, batch=batch, capacity=capacity)
    gpu_tokens = [[] for _ in range(batch)]
    nxt = None
    for position in range(prompt_length):  # the prompt goes through the decode path token by token
        nxt = engine.step(prompts[:, position].tolist(), position)
    for step in range(steps):
        for b in range(batch):
            gpu_tokens[b].append(nxt[b])
        nxt = engine.step(nxt, prompt_length + step)
    want = []
    gaps = []
    for b in range(batch):
        cpu = OracleDecoder(config, weights, capacity)
        token = None
        for position in range(prompt_length):
            token, _ = cpu.step(int(prompts[b, position]))
        sequence = []
        for step in range(steps):
            sequence.append(token)
            token, logits = cpu.step(token, want_logits=True)
            top = np.sort(logits[0].astype(np.float64))[-2:]
            gaps.append(top[1] - top[0])
        want.append(sequence)
    return engine, gpu_tokens, want, prompts, min(gaps)


def test_llama_shaped_greedy_tokens_match_oracle(runtime):
    from llmopt_b200.model import tiny_config

    config = tiny_config(layers=("attention",) * 3, hidden=192, heads=3, kv_heads=1, head_dim=64, intermediate=384,
                         vocabulary=1024)
    engine, got, want, prompts, gap = _run(runtime, config, prompt_length=24, steps=128)
    assert got == want, f"token streams differ (smallest oracle top-2 logit gap {gap})"
    # the device-chained replay reproduces the host-driven stream
    prompt_length = 24
    engine2_tokens, elapsed = engine.generate_chained([got[0][0]], prompt_length, 32)
    assert engine2_tokens[:31] == got[0][1:32]
    assert elapsed > 0


def test_hybrid_conv_attention_batched_teacher_forced(runtime):
    """Conv + attention blocks, three sequences per step. Both sides consume the
    oracle's token stream; every GPU pick must be the oracle's pick, or — when the
    oracle's two best logits are closer than the parity bound (2e-3 of the logit
    scale) — one of the tied candidates."""
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights, tiny_config
    from oracle_model import OracleDecoder

    config = tiny_config(layers=("conv", "attention", "conv", "attention"), hidden=256, heads=4, kv_heads=2,
                         head_dim=64, intermediate=512, vocabulary=2048)
    batch, prompt_length, steps = 3, 9, 40
    weights = random_weights(config, seed=1, std=0.05)
    rng = np.random.default_rng(1)
    prompts = rng.integers(0, config.vocabulary, size=(batch, prompt_length))
    capacity = prompt_length + steps + 1
    engine = DecodeEngine(runtime, config, weights, batch=batch, capacity=capacity)
    oracles = [OracleDecoder(config, weights, capacity) for _ in range(batch)]
    mismatches = 0
    tokens = prompts[:, 0].tolist()
    for position in range(prompt_length + steps):
        got = engine.step(tokens, position)
        results = [oracles[b].step(int(tokens[b]), want_logits=True) for b in range(batch)]
        for b, (want, logits) in enumerate(results):
            if got[b] != want:
                row = logits[0].astype(np.float64)
                gap = abs(row[want] - row[got[b]]) / max(np.max(np.abs(row)), 1e-6)
                assert gap <= 2e-3, f"step {position} sequence {b}: {got[b]} != {want}, logit gap {gap:.3e}"
                mismatches += 1
        tokens = [prompts[b, position + 1] if position + 1 < prompt_length else results[b][0] for b in range(batch)]
    assert mismatches <= 3, f"{mismatches} near-tie picks differ"


@pytest.mark.parametrize("layers,prompt_length", [(("attention",) * 3, 70), (("conv", "attention", "conv", "attention"), 130)])
def test_prefill_path_then_decode_matches_oracle(runtime, layers, prompt_length):
    """The prompt in one pass (one row per token through every linear — the tcgen05 kernels from
    17 rows on — dense causal attention, bulk cache pack, short-conv prefill), then greedy decode
    over the cache the prefill left: the first token, the last prompt row's hidden state and the
    following decode tokens equal the oracle's dense-prefill route."""
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights, tiny_config
    from oracle_model import OracleDecoder

    config = tiny_config(layers=layers, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512, vocabulary=2048)
    weights = random_weights(config, seed=3, std=0.05)
    prompt = np.random.default_rng(3).integers(0, config.vocabulary, size=prompt_length).tolist()
    steps, capacity = 24, prompt_length + 25
    engine = DecodeEngine(runtime, config, weights, batch=1, capacity=capacity)
    cpu = OracleDecoder(config, weights, capacity)
    want, _ = cpu.prefill_dense(prompt)
    got = engine.prefill(prompt)
    hidden = engine.prefill_hidden.buffer.to_numpy(np.float16, (prompt_length, config.hidden)).astype(np.float64)
    reference = cpu.last_hidden.astype(np.float64)
    drift = np.max(np.abs(hidden - reference)) / np.max(np.abs(reference))
    assert drift <= 5e-3, f"prefill hidden rows differ by {drift:.3e} of their scale"
    assert got == want
    mismatches = 0
    for step in range(steps):
        got = engine.step([want], prompt_length + step)[0]
        want_next, logits = cpu.step(want, want_logits=True)
        if got != want_next:
            row = logits[0].astype(np.float64)
            gap = abs(row[want_next] - row[got]) / max(np.max(np.abs(row)), 1e-6)
            assert gap <= 5e-3, f"step {step}: {got} != {want_next}, logit gap {gap:.3e}"
            mismatches += 1
        want = want_next
    assert mismatches <= 1, f"{mismatches} near-tie picks differ"


def test_a_replayed_prompt_plan_equals_a_fresh_pass(runtime):
    """A second prompt of a length seen before replays the recorded dispatch list with new ids: first
    token, hidden rows and the decode that follows are bit-identical to a fresh engine's pass over that
    prompt (every buffer of the pass is fully rewritten)."""
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights, tiny_config

    config = tiny_config(layers=("conv", "attention", "attention"), hidden=256, heads=4, kv_heads=2, head_dim=64,
                         intermediate=512, vocabulary=2048)
    weights = random_weights(config, seed=8, std=0.05)
    length, steps = 90, 12
    rng = np.random.default_rng(8)
    first, second = (rng.integers(0, config.vocabulary, size=length).tolist() for _ in range(2))

    def run(engine, prompt):
        token = engine.prefill(prompt)
        hidden = engine.prefill_hidden.buffer.to_numpy(np.float16, (length, config.hidden)).copy()
        stream = [token]
        for step in range(steps):
            stream.append(engine.step([stream[-1]], length + step)[0])
        return stream, hidden

    reused = DecodeEngine(runtime, config, weights, batch=1, capacity=length + steps + 1)
    run(reused, first)
    recorded = reused.prefill_seconds[0]
    stream, hidden = run(reused, second)  # the plan of `first`, the ids of `second`
    assert reused.prefill_seconds[0] < recorded, "the second pass recorded its dispatches again"
    fresh = DecodeEngine(runtime, config, weights, batch=1, capacity=length + steps + 1)
    want_stream, want_hidden = run(fresh, second)
    assert stream == want_stream
    assert np.array_equal(hidden.view(np.uint16), want_hidden.view(np.uint16))


def test_prefill_path_on_the_smollm2_shape_gives_the_stream_of_the_stepped_route(runtime):
    """SmolLM2-135M shape, 512-token prompt: prefill in one pass + 32 decode steps produce the token
    stream the oracle produced feeding the prompt token by token (tests/golden/decode_streams.npz):
    the two routes differ only in how the prompt's keys and values were read (fp16 versus the Q8
    cache), which the picks of this stream tolerate (their smallest top-2 gap is 8.5e-2)."""
    import os

    from llmopt_b200 import model
    from llmopt_b200.decode_engine import DecodeEngine

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "decode_streams.npz"))
    prompts, picks = data["smollm2_prompts"], data["smollm2_picks"]
    config = model.SMOLLM2_135M
    engine = DecodeEngine(runtime, config, model.random_weights(config, seed=0), batch=1, capacity=600)
    token = engine.prefill(prompts[0].tolist())
    stream = [token]
    for step in range(32):
        token = engine.step([token], 512 + step)[0]
        stream.append(token)
    assert stream == picks[0, :33].tolist()
    assert engine.prefill_kernels < 16 * 30
