#!/usr/bin/env python
"""Decode benchmark of the W4A16 / grouped-Q8 hot path on B200.

One "step" is one decode token for every sequence of the batch through the
prebaked plan (all linears, attention over the pre-filled Q8 context, cache pack,
LM-head argmax).  Inputs are synthetic: random-init weights of the named shape,
a context of random Q8 K/V with valid scales, random token ids.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llama3-8b|smollm2-135m|lfm2.5-350m]
                  [--batch B] [--context C] [--impl reference]

Prints ONE JSON line (rank 0).  `value` is device-timed (CUDA events around K
chained graph replays, inputs resident in HBM); `e2e` is the same metric through
the host-driven `Prebaked.execute` call with host<->device copies every step.
`--impl reference` times the CPU restatement of the reference's own loop nest
(oracle/) on a bounded sample of the same workload; it is the only place this
file executes the oracle apart from the `cpu_baseline` leg.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {"llama3-8b": "LLAMA3_8B", "smollm2-135m": "SMOLLM2_135M", "lfm2.5-350m": "LFM25_350M"}
DEFAULT_CONTEXT = {"llama3-8b": 8192, "smollm2-135m": 512, "lfm2.5-350m": 1024}
METRIC = "decode_tokens_per_s"


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            peaks = json.load(handle)
        return {"hbm_gbs": float(peaks["hbm_gbs"]), "bf16_tflops": float(peaks.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(peaks.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(device_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 9:
                continue
            try:
                clocks.append(float(fields[1]))
                maxima.append(float(fields[2]))
            except ValueError:
                continue
            for name, value in zip(names, fields[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(clocks)[len(clocks) // 2:]  # the upper half is the part under load
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(maxima), "samples": len(clocks),
                "reasons": sorted(reasons)}


def distributed_setup(gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    group = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        group = dist
    return rank, world, local, group


def cpu_reference_rate(config, batch: int, seconds: float = 12.0) -> dict:
    """Tokens/s of the reference's CPU loop nest (lib/cpu.ml:128-152, restated in
    oracle/llmopt_oracle.c) on a bounded sample: a column slice of one gate
    projection, all host threads, extrapolated by weight elements per token."""
    from oracle import oracle

    hidden, inter = config.hidden, config.intermediate
    rng = np.random.default_rng(0)
    cores = os.cpu_count() or 1
    columns = min(inter, 64 * cores)
    packed = rng.integers(0, 256, size=(columns, hidden // 2), dtype=np.uint8)
    scale = rng.uniform(0.005, 0.02, size=(columns, hidden // 64)).astype(np.float16)
    x = rng.standard_normal((batch, hidden)).astype(np.float16)
    oracle.w4a16_linear_cols_mt(x, packed, scale, 0, min(columns, 8))  # warm up the thread pool
    elapsed, repeats = 0.0, 0
    while elapsed < seconds and repeats < 2000:
        start = time.perf_counter()
        oracle.w4a16_linear_cols_mt(x, packed, scale, 0, columns)
        elapsed += time.perf_counter() - start
        repeats += 1
    per_sample = elapsed / repeats
    sample_elements = columns * hidden
    total_elements = 0
    dim = config.head_dim
    for kind in config.layers:
        if kind == "attention":
            total_elements += (config.query_heads + 2 * config.kv_heads) * dim * hidden + hidden * config.query_heads * dim
        else:
            total_elements += 4 * hidden * hidden
        total_elements += 3 * inter * hidden
    total_elements += config.vocabulary * hidden
    seconds_per_step = per_sample * total_elements / sample_elements
    return {
        "value": batch / seconds_per_step, "unit": "tokens/s", "cores": cores, "kind": "port",
        "sample": (f"{columns} columns of one gate projection (K={hidden}, M={batch}) x{repeats} repeats, "
                   f"{per_sample * 1e3:.2f} ms each, scaled by weight elements per token "
                   f"({total_elements / sample_elements:.0f}x); linears only, attention not included"),
        "seconds_per_step": seconds_per_step,
    }


def run_reference(args, config) -> dict:
    baseline = cpu_reference_rate(config, args.batch, seconds=max(4.0, min(30.0, 0.4 * (args.steps + args.warmup))))
    return {
        "impl": "reference", "metric": METRIC, "value": baseline["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": baseline["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.gpus > 1 else "strong", "vs_baseline": None,
        "dtype": "f64 accumulate (CPU loop nest)",
        "data": "synthetic", "config": workload_config(args, config),
        "cpu_baseline": {k: baseline[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": baseline["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def workload_config(args, config) -> dict:
    return {
        "workload": f"{config.name} greedy decode, batch {args.batch}, context {args.context} tokens of Q8 KV "
                    f"(group {config.kv_group_size}), W4A16 group-64 linears",
        "batch": args.batch, "context": args.context,
        "parallelism": parallelism_label(args, config),
        "l2": "every step streams its weights and KV once; the working set per step is far larger than the "
              "126 MB L2, so nothing is flushed between steps",
    }


def tensor_parallel_run(args, config) -> bool:
    from llmopt_b200 import tensor_parallel

    return args.gpus > 1 and args.parallel == "tp" and tensor_parallel.shards(config, args.gpus)


def parallelism_label(args, config) -> str:
    if args.gpus <= 1:
        return "single"
    if tensor_parallel_run(args, config):
        return (f"tp{args.gpus}: column-split QKV / gate / up / LM head, row-split o_proj / down with fp32 partial sums "
                f"reduced over peer memory (NVLink), attention split by KV head; one sequence set for all GPUs")
    return f"{args.gpus} independent replicas (one per GPU, no exchange)"


def time_kernels(engine, runtime) -> dict:
    """Device time of each W4A16 / attention dispatch of one token, measured the way a
    replayed plan runs it: the same dispatch over every layer's own weights / cache
    region, launched back to back between one pair of CUDA events (operands far
    larger than the L2, so every launch reads cold data). Algorithmic bytes from the shapes."""
    config, batch = engine.config, engine.batch
    hidden, dim = config.hidden, config.head_dim
    groups = {}

    def linear_bytes(n, k, matrices=1, extra=0):
        return matrices * (n * k // 2 + n * (k // 64) * 2) + batch * k * 2 + matrices * batch * n * 2 + extra

    for item in engine.records:
        name = item.name
        if name.startswith("llmopt_w4a16_qkv"):
            n = (config.query_heads + 2 * config.kv_heads) * dim
            nbytes, label = linear_bytes(n, hidden), "qkv"
        elif name.startswith("llmopt_w4a16_dual_swiglu"):
            nbytes = 2 * (config.intermediate * hidden // 2 + config.intermediate * (hidden // 64) * 2) \
                + batch * hidden * 2 + batch * config.intermediate * 2
            label = "gate_up_swiglu"
        elif name.startswith("llmopt_w4a16_down_add"):
            nbytes, label = linear_bytes(hidden, config.intermediate, extra=batch * hidden * 2), "down_add"
        elif name.startswith("llmopt_w4a16_linear_partial_f32"):  # row-split product of a tensor-parallel rank
            params = np.frombuffer(bytes(item.parameters), np.uint32)
            n, k = int(params[1]), int(params[2])
            nbytes = n * k // 2 + n * (k // 64) * 2 + batch * k * 2 + batch * n * 4
            label = f"linear_partial_n{n}_k{k}"
        elif name.startswith("llmopt_w4a16_linear"):
            params = np.frombuffer(bytes(item.parameters), np.uint32)
            nbytes = linear_bytes(int(params[1]), int(params[2]), extra=batch * int(params[1]) * 2 if params[3] else 0)
            label = f"linear_n{int(params[1])}_k{int(params[2])}"
        elif name.startswith("llmopt_w4a16_lm_head"):
            rows_here = int(np.frombuffer(bytes(item.parameters[:4]), np.uint32)[0])
            nbytes = config.vocabulary * hidden // 2 + config.vocabulary * (hidden // 64) * 2 + rows_here * hidden * 2 + rows_here * 4
            label = "lm_head_argmax"
        elif name.startswith("llmopt_attention_q8_paged"):
            past = engine._context.decode_uniforms_past_tokens
            per_key = 2 * config.kv_heads * dim + 4 * config.kv_heads * dim // config.kv_group_size + 4
            nbytes = batch * (past * per_key + 2 * config.query_heads * dim * 2 + 2 * config.kv_heads * dim * 2)
            label = "paged_attention_q8"
        else:
            continue
        groups.setdefault(label, {"name": name, "bytes": nbytes, "items": []})["items"].append(item)
    table = {}
    for label, group in groups.items():
        items = group["items"]
        while len(items) * group["bytes"] < (1 << 30) and len(items) < 64:  # cover >= 1 GB so the L2 cannot help
            items = items + group["items"]
        milliseconds = runtime.time_dispatches(items, warmup=2, iterations=5)
        table[label] = {"kernel": label, "name": group["name"], "ms": milliseconds, "bytes": group["bytes"],
                        "launches_timed": len(items), "gbs": group["bytes"] / milliseconds / 1e6}
    return table


# DRAM bytes per launch (ncu: dram__bytes_read.sum + dram__bytes_write.sum) over the algorithmic
# bytes of the same launch, from the captures summarised under profiles/ (GEMV: batch 1 gate/up;
# attention: batch 8, 8192 tokens; both grow in proportion to the units processed).
TRAFFIC_RATIO = {
    "gate_up_swiglu": (62_625_536 / 62_427_136, "profiles/w4a16_gemv_pipe_m1_llama3_8b.md"),
    "paged_attention_q8": (147_036_160 / 138_838_016, "profiles/paged_attention_q8_split_llama3_8b.md"),
}


def time_prefill_gemm(engine, runtime, peaks) -> dict:
    """The prefill side of the path: the gate/up projection of the first layers at M = 2048 rows
    (one prefill chunk) on the tcgen05 GEMM, device-timed back to back; dense-equivalent FLOPs."""
    from llmopt_b200 import dispatch
    from llmopt_b200.cuda_native import Batch, Buffer

    config = engine.config
    m, k, n = 2048, config.hidden, config.intermediate
    rng = np.random.default_rng(1)
    x = dispatch.Tensor(Buffer.of_array(runtime, rng.standard_normal((m, k)).astype(np.float16)), (m, k))
    residual = dispatch.Tensor(Buffer.create(runtime, m * k * 2), (m, k))
    output = dispatch.Tensor(Buffer.create(runtime, m * k * 2), (m, k))
    commands = Batch(runtime)
    context = dispatch.Context(runtime, batch=commands)
    items = []
    for layer in engine.layers[:4]:
        dispatch.dispatch_w4a16_swiglu_ffn_command(
            context, m=m, n=n, k=k, epsilon=config.epsilon, activation=x, residual=residual,
            gate_weight=layer["gate"][0], gate_scale=layer["gate"][1], up_weight=layer["up"][0],
            up_scale=layer["up"][1], down_weight=layer["down"][0], down_scale=layer["down"][1],
            norm_weight=layer["ffn_norm"], output=output, reference_guards=False)
    items = [item for item in commands.pending if item.name.startswith("llmopt_w4a16_dual_swiglu")]
    name = items[0].name
    milliseconds = runtime.time_dispatches(items, warmup=1, iterations=3)
    commands.abort()
    tflops = 2.0 * 2 * m * k * n / milliseconds / 1e9
    return {"kernel": name, "m": m, "k": k, "n": n, "products": 2, "ms": milliseconds, "bound": "tensor",
            "achieved": tflops, "unit": "TFLOP/s", "peak": peaks["bf16_tflops"], "frac": tflops / peaks["bf16_tflops"],
            "peak_sustained": peaks.get("bf16_tflops_sustained"), "peak_source": peaks["source"]}


def run_native(args, config, rank: int, world: int, local: int, group) -> dict:
    from llmopt_b200 import cuda_native
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import decode_bytes_per_token, random_weights

    # N > 1: tensor parallel when the model splits over N ranks (every rank decodes the same
    # sequences with its share of every layer), else one independent replica of the whole model
    # per GPU (no exchange on the data path).
    runtime = cuda_native.Runtime(local)
    whole_config = config
    fast = config.hidden >= 2048
    weights = random_weights(config, seed=0, fast=fast)
    capacity = args.context + args.steps * 2 + args.warmup * 2 + 16
    tensor_parallel_mode = tensor_parallel_run(args, config)
    if tensor_parallel_mode:
        from llmopt_b200 import tensor_parallel

        exchange_group = tensor_parallel.ExchangeGroup.create(
            runtime, rank, world, max(args.batch * config.hidden * 4, min(args.batch, 32) * 256 * 8), 7,
            tensor_parallel.torch_all_gather())
        shard = tensor_parallel.shard_weights(config, weights, rank, world)
        del weights
        weights = shard
        config = tensor_parallel.local_config(config, world)
        engine = DecodeEngine(runtime, config, weights, batch=args.batch, capacity=capacity, group=exchange_group)
    else:
        engine = DecodeEngine(runtime, config, weights, batch=args.batch, capacity=capacity)
    del weights
    engine.fill_cache_random(args.context, seed=0)
    engine.build(args.context)
    rng = np.random.default_rng(0)
    first = rng.integers(0, config.vocabulary, size=args.batch).tolist()

    # device-timed region: K chained replays, CUDA events on the launching stream
    engine.generate_chained(first, args.context, max(args.warmup, 3))
    sampler = ClockSampler(local)
    if group is not None:
        group.barrier()
    runtime.synchronize()
    _, elapsed_ms = engine.generate_chained(first, args.context, args.steps)
    runtime.synchronize()
    if group is not None:
        import torch

        slowest = torch.tensor([elapsed_ms], dtype=torch.float64)
        group.all_reduce(slowest, op=group.ReduceOp.MAX)  # device-timed on every rank, max over ranks
        elapsed_ms = float(slowest.item())
        group.barrier()
    clocks = sampler.stop()
    ms_per_step = elapsed_ms / args.steps
    jobs = 1 if tensor_parallel_mode else world  # tensor parallel: all GPUs decode the same sequences
    value = jobs * args.batch * 1000.0 / ms_per_step

    # end to end: the host drives every token (token id in, H2D; next id out, D2H)
    tokens = first
    for step in range(max(args.warmup, 3)):
        tokens = engine.step(tokens, args.context + step)
    runtime.synchronize()
    start = time.perf_counter()
    for step in range(args.steps):
        tokens = engine.step(tokens, args.context + step)
    runtime.synchronize()
    e2e_seconds = time.perf_counter() - start
    if group is not None:
        import torch

        slowest = torch.tensor([e2e_seconds], dtype=torch.float64)
        group.all_reduce(slowest, op=group.ReduceOp.MAX)
        e2e_seconds = float(slowest.item())
    e2e_value = jobs * args.batch * args.steps / e2e_seconds
    h2d = 16 + (8 * args.batch if args.batch > 1 else 0)
    d2h = 4 + (4 * args.batch if args.batch > 1 else 0)

    peaks = measured_peaks()
    kernels = time_kernels(engine, runtime)
    dominant = kernels.get("gate_up_swiglu") or next(iter(kernels.values()))
    if args.batch >= 8 and "paged_attention_q8" in kernels:
        attention_ms = kernels["paged_attention_q8"]["ms"] * config.attention_layers
        if attention_ms > dominant["ms"] * len(config.layers):
            dominant = kernels["paged_attention_q8"]
    step_bytes = decode_bytes_per_token(config, args.batch, args.context)
    result = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak" if world > 1 and not tensor_parallel_mode else "strong",
        "vs_baseline": None, "dtype": "w4a16 (int4 weights, f16 activations, f32 accumulate); q8 KV",
        "data": "synthetic", "config": workload_config(args, whole_config),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": (engine.plan.kernel_count() + 1) * args.steps,
        "kernels_per_step": engine.plan.kernel_count(),
        "clocks": clocks,
        "roofline": {
            "bound": "hbm", "kernel": dominant["name"], "achieved": dominant["gbs"], "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": dominant["gbs"] / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "frac_of_spec_8000": dominant["gbs"] / 8000.0,
            "traffic": round(dominant["bytes"] * TRAFFIC_RATIO[dominant["kernel"]][0])
            if dominant["kernel"] in TRAFFIC_RATIO else None,
            "traffic_source": TRAFFIC_RATIO.get(dominant["kernel"], (None, None))[1],
            "bytes_per_launch": dominant["bytes"], "ms_per_launch": dominant["ms"],
        },
        "step_roofline": {
            "algorithmic_bytes_per_step": step_bytes["total"], "weights": step_bytes["weights"],
            "attention": step_bytes["attention"], "achieved_gbs": step_bytes["total"] / ms_per_step / 1e6,
            "frac": step_bytes["total"] / ms_per_step / 1e6 / peaks["hbm_gbs"],
        },
        "kernels": {k: {"ms": round(v["ms"], 5), "gbs": round(v["gbs"], 1), "frac": round(v["gbs"] / peaks["hbm_gbs"], 3)}
                    for k, v in kernels.items()},
    }
    if config.hidden >= 2048 and world == 1:
        result["prefill_gemm"] = time_prefill_gemm(engine, runtime, peaks)
    if group is not None:
        group.barrier()  # no rank leaves (and unmaps its exchange region) while a peer still runs
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        baseline = cpu_reference_rate(config, args.batch)
        result["cpu_baseline"] = {k: baseline[k] for k in ("value", "unit", "cores", "kind", "sample")}
    return result


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--workload", default="llama3-8b", choices=sorted(WORKLOADS))
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--context", type=int, default=None)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--parallel", default="tp", choices=["tp", "replicas"],
                        help="with --gpus N > 1: tensor parallel (when the model splits over N) or N replicas")
    args = parser.parse_args()
    from llmopt_b200 import model

    config = getattr(model, WORKLOADS[args.workload])
    if args.context is None:
        args.context = DEFAULT_CONTEXT[args.workload]
    if args.impl == "reference":
        # rank 0 alone measures; the other ranks of a torchrun launch leave at once
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(run_reference(args, config)), flush=True)
        return
    rank, world, local, group = distributed_setup(args.gpus)
    result = run_native(args, config, rank, world, local, group)
    if rank == 0:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
