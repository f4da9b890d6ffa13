"""Generates tests/golden/decode_streams.npz: the CPU oracle's greedy token streams on the
model shapes the headline configurations name, so the GPU parity tests can check the full-size
configurations without spending minutes of oracle time beside the GPU.

    python tests/golden/make_decode_golden.py [case ...]      # cases: smollm2 lfm25 lfm25_batch16

Everything is seeded: weights = ``model.random_weights(config, seed=0)`` (N(0, 0.02) quantised
W4A16 group-64 by the numpy restatement of the reference quantiser, tied LM head), prompts are
uniform random ids from ``numpy.random.default_rng(seed)``.  Per case the file holds the
prompts, the oracle's pick after the prompt and after every further step (teacher-forced on its
own picks = free-running greedy decode), the eight best candidates of every pick with their
logits relative to the largest |logit| of the step (what a near-tie analysis needs),
and the hidden state that entered the LM head at the last step (the accumulated rounding
difference of the whole stack shows there before any argmax hides it).

  smollm2         SmolLM2-135M shape, 512-token prompt, 128 steps, one sequence
  lfm25           LFM2.5-350M shape (10 gated short-conv + 6 attention blocks), 1024-token prompt,
                  256 steps, one sequence
  lfm25_batch16   the same model, 16 sequences side by side: 32-token prompts, 32 steps each
                  (the full 1024 + 256 of all 16 sequences is hours of oracle time)
"""

import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

CASES = {
    "smollm2": dict(model="SMOLLM2_135M", sequences=1, prompt=512, steps=128, seed=0),
    "lfm25": dict(model="LFM25_350M", sequences=1, prompt=1024, steps=256, seed=0),
    "lfm25_batch16": dict(model="LFM25_350M", sequences=16, prompt=32, steps=32, seed=1),
}
OUTPUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_streams.npz")


def run_case(name: str, case: dict) -> dict:
    from llmopt_b200 import model
    from oracle_model import OracleDecoder

    config = getattr(model, case["model"])
    weights = model.random_weights(config, seed=0)
    rng = np.random.default_rng(case["seed"])
    sequences, prompt_length, steps = case["sequences"], case["prompt"], case["steps"]
    prompts = rng.integers(0, config.vocabulary, size=(sequences, prompt_length))
    oracle = OracleDecoder(config, weights, prompt_length + steps + 1, sequences=sequences)
    start = time.time()
    picks = np.zeros((sequences, steps + 1), np.int64)      # picks[:, 0]: after the prompt
    top_ids = np.zeros((sequences, steps + 1, 8), np.int64)  # the eight largest logits, best first
    top_gap = np.zeros((sequences, steps + 1, 8), np.float64)  # (logit of the pick - logit) / max |logit|
    gap = np.zeros((sequences, steps + 1), np.float64)       # to the best candidate that is not the pick

    def record(column, chosen, logits):
        for s in range(sequences):
            row = logits[s].astype(np.float64)
            scale = max(np.max(np.abs(row)), 1e-9)
            order = np.argsort(-row, kind="stable")[:8]
            picks[s, column] = chosen[s]
            top_ids[s, column] = order
            top_gap[s, column] = (row[chosen[s]] - row[order]) / scale
            others = [index for index in order if index != chosen[s]]
            gap[s, column] = (row[chosen[s]] - row[others[0]]) / scale

    # the prompt: every sequence's rows in one call, picks wanted for each sequence's last row
    rows = [(s, int(prompts[s, t])) for s in range(sequences) for t in range(prompt_length)]
    emit = [s * prompt_length + prompt_length - 1 for s in range(sequences)]
    chosen, logits = oracle.forward(rows, emit, want_logits=True)
    record(0, chosen, logits)
    print(f"{name}: prompt done in {time.time() - start:.0f} s", flush=True)
    for step in range(steps):
        chosen, logits = oracle.step_all(chosen, want_logits=True)
        record(step + 1, chosen, logits)
    print(f"{name}: {steps} steps done in {time.time() - start:.0f} s; smallest top-2 gap {gap.min():.3e}", flush=True)
    return {f"{name}_prompts": prompts, f"{name}_picks": picks, f"{name}_top_ids": top_ids, f"{name}_top_gap": top_gap,
            f"{name}_gap": gap,
            f"{name}_last_hidden": oracle.last_hidden.copy()}


def main(names) -> None:
    data = dict(np.load(OUTPUT)) if os.path.exists(OUTPUT) else {}
    for name in names or list(CASES):
        data.update(run_case(name, CASES[name]))
        np.savez_compressed(OUTPUT, **data)
    print("wrote", OUTPUT)


if __name__ == "__main__":
    main(sys.argv[1:])
