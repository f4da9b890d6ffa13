"""One gloo rank of test_tensor_parallel_cpu.test_two_gloo_ranks_reproduce_the_unsharded_layer."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from llmopt_b200 import tensor_parallel  # noqa: E402
from llmopt_b200.model import random_weights, tiny_config  # noqa: E402
from oracle import oracle  # noqa: E402


def main() -> None:
    dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
    rank, world = dist.get_rank(), dist.get_world_size()
    config = tiny_config(layers=("attention",), hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                         vocabulary=512)
    weights = random_weights(config, seed=3, std=0.05)
    mine = tensor_parallel.shard_weights(config, weights, rank, world)
    local = tensor_parallel.local_config(config, world)
    rng = np.random.default_rng(7)
    hidden = rng.standard_normal((2, config.hidden)).astype(np.float16)
    layer, whole = mine["layer0"], weights["layer0"]

    def all_reduce_f32(partial):
        tensor = torch.from_numpy(np.ascontiguousarray(partial.astype(np.float32)))
        gathered = [torch.empty_like(tensor) for _ in range(world)]
        dist.all_gather(gathered, tensor)
        total = np.zeros_like(partial, dtype=np.float32)
        for part in gathered:  # rank order, like the exchange kernel
            total += part.numpy()
        return total

    # FFN of one layer: rms (replicated) -> gate/up on local columns -> down on the local K slice -> exchange
    want, normed, _ = oracle.w4a16_swiglu_ffn(hidden, hidden, whole["gate"][0], whole["gate"][1], whole["up"][0],
                                              whole["up"][1], whole["down"][0], whole["down"][1], whole["ffn_norm"],
                                              config.epsilon)
    product = oracle.w4a16_dual_swiglu(normed, layer["gate"][0], layer["gate"][1], layer["up"][0], layer["up"][1])
    partial = oracle.w4a16_linear_f64(product, layer["down"][0], layer["down"][1])
    out = (all_reduce_f32(partial) + hidden.astype(np.float32)).astype(np.float16)
    error = np.max(np.abs(out.astype(np.float64) - want.astype(np.float64))) / np.max(np.abs(want.astype(np.float64)))

    # LM head: local argmax over the vocabulary shard, then the best over the ranks (ties: lowest index)
    token, _, best_value = oracle.w4a16_lm_head_argmax(out[:1], weights["final_norm"], mine["lm_head"][0],
                                                       mine["lm_head"][1], config.epsilon)
    candidate = torch.tensor([float(best_value[0]), float(int(token[0]) + rank * local.vocabulary)],
                             dtype=torch.float64)
    gathered = [torch.empty_like(candidate) for _ in range(world)]
    dist.all_gather(gathered, candidate)
    best = max(gathered, key=lambda c: (float(c[0]), -float(c[1])))
    want_token, _, _ = oracle.w4a16_lm_head_argmax(out[:1], weights["final_norm"], weights["lm_head"][0],
                                                   weights["lm_head"][1], config.epsilon)
    # Prompt rows: the same row split as a reduce-scatter (this rank sums ITS share of the rows over every
    # rank's fp32 partial, rank order, residual, one rounding) and an all-gather of the fp16 shares
    rows = 5
    prompt = rng.standard_normal((rows, config.hidden)).astype(np.float16)
    want_rows, normed_rows, _ = oracle.w4a16_swiglu_ffn(prompt, prompt, whole["gate"][0], whole["gate"][1], whole["up"][0],
                                                        whole["up"][1], whole["down"][0], whole["down"][1],
                                                        whole["ffn_norm"], config.epsilon)
    product_rows = oracle.w4a16_dual_swiglu(normed_rows, layer["gate"][0], layer["gate"][1], layer["up"][0], layer["up"][1])
    partial_rows = torch.from_numpy(np.ascontiguousarray(
        oracle.w4a16_linear_f64(product_rows, layer["down"][0], layer["down"][1]).astype(np.float32)))
    partials = [torch.empty_like(partial_rows) for _ in range(world)]
    dist.all_gather(partials, partial_rows)  # stands for the peer reads of the slot
    first, last = tensor_parallel.prompt_row_share(rows, world, rank)
    total = np.zeros((last - first, config.hidden), np.float32)
    for part in partials:
        total += part.numpy()[first:last]
    # (the fp16 bits travel as int32: gloo has no 16-bit integer)
    share = torch.from_numpy((total + prompt[first:last].astype(np.float32)).astype(np.float16).view(np.uint16).astype(np.int32))
    padded = torch.zeros(((rows + world - 1) // world, config.hidden), dtype=torch.int32)
    padded[:last - first] = share
    shares = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(shares, padded)  # the gather exchange
    out_rows = np.zeros((rows, config.hidden), np.float16)
    for peer, piece in enumerate(shares):
        lo, hi = tensor_parallel.prompt_row_share(rows, world, peer)
        out_rows[lo:hi] = piece.numpy().astype(np.uint16).view(np.float16)[:hi - lo]
    rows_error = (np.max(np.abs(out_rows.astype(np.float64) - want_rows.astype(np.float64))) /
                  np.max(np.abs(want_rows.astype(np.float64))))
    np.savez(os.environ["TP_OUT"], hidden=out, token=int(best[1]), want_token=int(want_token[0]), error=error,
             rows=out_rows, rows_error=rows_error)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
