"""One rank of test_gpu_tensor_parallel.test_two_ranks_on_two_gpus_match_the_single_gpu_tokens."""

import os
import sys

import numpy as np
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from llmopt_b200 import cuda_native, tensor_parallel  # noqa: E402
from llmopt_b200.decode_engine import DecodeEngine  # noqa: E402
from llmopt_b200.model import random_weights, tiny_config  # noqa: E402


def main() -> None:
    dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
    rank, world = dist.get_rank(), dist.get_world_size()
    runtime = cuda_native.Runtime(int(os.environ["LOCAL_RANK"]))
    config = tiny_config(layers=("attention",) * 2, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                         vocabulary=1024)
    weights = random_weights(config, seed=4, std=0.05)
    steps, prompt = 24, [5, 77, 301, 12]
    long_prompt = np.random.default_rng(9).integers(0, config.vocabulary, size=70).tolist()
    group = tensor_parallel.ExchangeGroup.create(
        runtime, rank, world, max(len(long_prompt) * config.hidden * 4, tensor_parallel.CANDIDATE_PARTS * 8), 7,
        tensor_parallel.torch_all_gather())
    engine = DecodeEngine(runtime, tensor_parallel.local_config(config, world),
                          tensor_parallel.shard_weights(config, weights, rank, world), batch=1,
                          capacity=len(prompt) + steps + 1, group=group)
    tokens, token = [], None
    for position, value in enumerate(prompt):
        token = engine.step([value], position)[0]
    for step in range(steps):
        tokens.append(token)
        token = engine.step([token], len(prompt) + step)[0]
    want = []
    if rank == 0:
        from oracle_model import OracleDecoder

        cpu = OracleDecoder(config, weights, len(prompt) + steps + 1)
        reference = None
        for value in prompt:
            reference, _ = cpu.step(value)
        for _ in range(steps):
            want.append(reference)
            reference, _ = cpu.step(reference)
    # second part: the prompt in one sharded pass, then decode over the cache it left
    dist.barrier()  # no exchange of the stepped part is in flight on any rank
    second = DecodeEngine(runtime, tensor_parallel.local_config(config, world),
                          tensor_parallel.shard_weights(config, weights, rank, world), batch=1,
                          capacity=len(long_prompt) + steps + 1, group=group)
    token = second.prefill(long_prompt)
    prompt_tokens = [token]
    for step in range(steps):
        token = second.step([token], len(long_prompt) + step)[0]
        prompt_tokens.append(token)
    prompt_want = []
    if rank == 0:
        cpu = OracleDecoder(config, weights, len(long_prompt) + steps + 1)
        reference, _ = cpu.prefill_dense(long_prompt)
        prompt_want.append(reference)
        for _ in range(steps):
            reference, _ = cpu.step(reference)
            prompt_want.append(reference)
    np.savez(os.environ["TP_OUT"], tokens=np.array(tokens), want=np.array(want), prompt_tokens=np.array(prompt_tokens),
             prompt_want=np.array(prompt_want))
    dist.barrier()  # no rank unmaps its region while a peer may still read it
    runtime.synchronize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
