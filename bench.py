#!/usr/bin/env python
"""Decode benchmark of the W4A16 / grouped-Q8 hot path on B200.

One "step" is one decode token for every sequence of the batch through the
prebaked plan (all linears, attention over the pre-filled Q8 context, cache pack,
LM-head argmax).  Inputs are synthetic: random-init weights of the named shape,
a context of random Q8 K/V with valid scales, random token ids.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llama3-8b|smollm2-135m|lfm2.5-350m]
                  [--batch B] [--context C] [--impl reference] [--no-extra-legs]

Prints ONE JSON line (rank 0).  `value` is device-timed (CUDA events around K
chained graph replays, inputs resident in HBM; the median of several repetitions
of the K steps); `e2e` is the same metric through the host-driven
`Prebaked.execute` call with host<->device copies every step.  The headline is
batch 1; the same line carries the batch-32 leg (`batch32`), the small-model
legs (`smollm2_135m`, `lfm25_350m`), the prefill GEMM sweep (`prefill_gemm`,
`prefill_gemm_c5`), timings of the zero-point / group-32 input mode
(`baseline_mode`) and, at N > 1, a correctness check of the tensor-parallel
run (`tp_check`).  `--impl reference` times the CPU restatement of the
reference's own loop nest (oracle/) on a bounded sample of the same workload; it
is the only place this file executes the oracle apart from the `cpu_baseline` leg.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {"llama3-8b": "LLAMA3_8B", "smollm2-135m": "SMOLLM2_135M", "lfm2.5-350m": "LFM25_350M"}
DEFAULT_CONTEXT = {"llama3-8b": 8192, "smollm2-135m": 512, "lfm2.5-350m": 1024}
METRIC = "decode_tokens_per_s"
REPETITIONS = 5  # the K timed steps are repeated this often; the median repetition is reported


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            peaks = json.load(handle)
        return {"hbm_gbs": float(peaks["hbm_gbs"]), "bf16_tflops": float(peaks.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(peaks.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def profile_traffic(relative_path: str, heading_key: str):
    """(algorithmic bytes, DRAM bytes read + written) of one captured launch, read from the
    section of a profile summary under profiles/ whose heading contains ``heading_key``."""
    path = os.path.join(ROOT, relative_path)
    if not os.path.exists(path):
        return None
    algorithmic = read = written = None
    inside = False
    with open(path) as handle:
        for line in handle:
            if line.startswith("## "):
                if inside:
                    break
                inside = heading_key in line
                if inside:
                    found = re.search(r"([\d,]+) algorithmic bytes", line)
                    algorithmic = int(found.group(1).replace(",", "")) if found else None
                continue
            if not inside:
                continue
            cells = [cell.strip() for cell in line.split("|")]
            if len(cells) >= 3 and cells[1] == "dram__bytes_read.sum":
                read = int(cells[2])
            if len(cells) >= 3 and cells[1] == "dram__bytes_write.sum":
                written = int(cells[2])
    if algorithmic is None or read is None or written is None:
        return None
    return algorithmic, read + written


# kernel label -> (profile summary, heading of the capture that matches this batch size best)
TRAFFIC_SOURCES = {
    "gate_up_swiglu": ("profiles/w4a16_gemv_pipe_m1_llama3_8b.md", "gate/up"),
    "down_add": ("profiles/w4a16_gemv_pipe_m1_llama3_8b.md", "down + residual"),
    "qkv": ("profiles/w4a16_gemv_pipe_m1_llama3_8b.md", "fused QKV"),
    "lm_head_argmax": ("profiles/w4a16_gemv_pipe_m1_llama3_8b.md", "LM head"),
    "paged_attention_q8": ("profiles/paged_attention_q8_split_llama3_8b.md", "batch 8"),
}


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


# ---- the reference's CPU path ------------------------------------------------------------------

def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def weight_elements_per_token(config) -> int:
    hidden, inter, dim = config.hidden, config.intermediate, config.head_dim
    total = 0
    for kind in config.layers:
        if kind == "attention":
            total += (config.query_heads + 2 * config.kv_heads) * dim * hidden + hidden * config.query_heads * dim
        else:
            total += 4 * hidden * hidden
        total += 3 * inter * hidden
    return total + config.vocabulary * hidden


def cpu_reference_rate(config, batch: int, context: int, seconds: float = 12.0) -> dict:
    """Tokens/s of the reference's CPU path on a bounded sample of the decode step: the
    Cpu.w4a16_linear loop nest (lib/cpu.ml:128-152, restated in oracle/llmopt_oracle.c) over a
    column slice of one gate projection, once on one thread (the reference interpreter is single
    threaded) and once with OpenMP over all host threads, plus one layer of paged Q8 attention
    over the context (one thread); each scaled to a whole token by the units it stands for."""
    from oracle import oracle

    hidden, inter, dim = config.hidden, config.intermediate, config.head_dim
    rng = np.random.default_rng(0)
    threads = host_threads()
    columns = min(inter, 64 * threads)
    packed = rng.integers(0, 256, size=(columns, hidden // 2), dtype=np.uint8)
    scale = rng.uniform(0.005, 0.02, size=(columns, hidden // 64)).astype(np.float16)
    x = rng.standard_normal((batch, hidden)).astype(np.float16)
    total_elements = weight_elements_per_token(config)

    def timed(columns_used: int, budget: float):
        oracle.w4a16_linear_cols_mt(x, packed, scale, 0, min(columns_used, 8))  # warm up the thread pool
        elapsed, repeats = 0.0, 0
        while elapsed < budget and repeats < 2000:
            start = time.perf_counter()
            oracle.w4a16_linear_cols_mt(x, packed, scale, 0, columns_used)
            elapsed += time.perf_counter() - start
            repeats += 1
        return elapsed / repeats, repeats

    oracle.set_threads(1)
    single_columns = min(columns, 64)
    single_sample, single_repeats = timed(single_columns, min(3.0, seconds / 4))
    used = oracle.set_threads(threads)
    per_sample, repeats = timed(columns, seconds)
    linear_seconds = per_sample * total_elements / (columns * hidden)
    linear_seconds_single = single_sample * total_elements / (single_columns * hidden)

    # one layer of paged attention over the context for one sequence, single thread
    attention_seconds = 0.0
    attention_note = "no attention layers"
    if config.attention_layers:
        from llmopt_b200.kv_cache import AttentionLayer, Layout

        layout = Layout([AttentionLayer(config.kv_heads, dim)], group_size=config.kv_group_size)
        keys = min(context, 2048)
        pool = np.zeros((keys, layout.bytes_per_token), np.uint8)
        pool[:, :layout.token_elements] = rng.integers(-127, 128, size=(keys, layout.token_elements),
                                                       dtype=np.int8).view(np.uint8)
        pool[:, layout.token_elements:] = rng.uniform(0.004, 0.02, size=(keys, layout.token_groups)).astype(
            np.float16).view(np.uint8).reshape(keys, -1)
        region = layout.attentions[0]
        params = oracle.paged_params_bytes(
            batches=1, query_heads=config.query_heads, kv_heads=config.kv_heads, past_length=keys, head_dim=dim,
            token_elements=layout.token_elements, key_offset=region.key_offset, value_offset=region.value_offset,
            group_size=layout.group_size, token_stride=layout.bytes_per_token, scale=float(1.0 / np.sqrt(dim)))
        query = rng.standard_normal((1, config.query_heads, 1, dim)).astype(np.float16)
        current = rng.standard_normal((1, config.kv_heads, 1, dim)).astype(np.float16)
        start = time.perf_counter()
        oracle.attention_q8_paged(query, current, current, pool.reshape(-1), np.arange(keys, dtype=np.uint32), None, params)
        layer_seconds = (time.perf_counter() - start) * context / keys
        attention_seconds = layer_seconds * config.attention_layers * batch
        attention_note = (f"paged Q8 attention of one layer over {keys} keys on one thread ({layer_seconds * 1e3:.0f} ms "
                          f"scaled to {context} keys), x{config.attention_layers} layers x{batch} sequences")
    seconds_per_step = linear_seconds + attention_seconds
    return {
        "value": batch / seconds_per_step, "unit": "tokens/s", "cores": used, "kind": "port",
        "sample": (f"{columns} columns of one gate projection (K={hidden}, M={batch}) x{repeats} repeats on {used} OpenMP "
                   f"threads, {per_sample * 1e3:.2f} ms each, scaled by weight elements per token "
                   f"({total_elements / (columns * hidden):.0f}x); {attention_note}"),
        "single_thread": {
            "value": batch / (linear_seconds_single + attention_seconds), "unit": "tokens/s", "cores": 1,
            "sample": f"{single_columns} columns x{single_repeats} repeats on one thread (the reference interpreter's "
                      f"own loop order), {single_sample * 1e3:.2f} ms each; same attention sample"},
        "linears_only": {"value": batch / linear_seconds, "unit": "tokens/s",
                         "note": "the same all-thread linear sample without the attention term"},
        "seconds_per_step": seconds_per_step, "seconds_per_sample": per_sample,
        "linear_seconds": linear_seconds, "attention_seconds": attention_seconds,
    }


def run_reference(args, config) -> dict:
    budget = max(4.0, min(30.0, 0.4 * (args.steps + args.warmup)))
    baseline = cpu_reference_rate(config, args.batch, args.context, seconds=budget)
    return {
        "impl": "reference", "metric": METRIC, "value": baseline["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # each "step" of this arm is one bounded sample (a column slice of one projection); a whole token is
        # `seconds_per_token` of such work
        "ms_per_step": baseline["seconds_per_sample"] * 1e3, "seconds_per_token": baseline["seconds_per_step"],
        "higher_is_better": True, "scaling": scaling_label(args, config), "vs_baseline": None,
        "dtype": "f64 accumulate (CPU loop nest)",
        "data": "synthetic", "config": workload_config(args, config),
        "cpu_baseline": {k: baseline[k] for k in ("value", "unit", "cores", "kind", "sample", "single_thread", "linears_only")},
        "e2e": {"value": baseline["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def workload_config(args, config, batch=None, context=None) -> dict:
    batch = args.batch if batch is None else batch
    context = args.context if context is None else context
    return {
        "workload": f"{config.name} greedy decode, batch {batch}, context {context} tokens of Q8 KV "
                    f"(group {config.kv_group_size}), W4A16 group-64 linears",
        "batch": batch, "context": context,
        "parallelism": parallelism_label(args, config),
        "l2": "every step streams its weights and KV once; the working set per step is far larger than the "
              "126 MB L2, so nothing is flushed between steps",
    }


def tensor_parallel_run(args, config) -> bool:
    from llmopt_b200 import tensor_parallel

    return args.gpus > 1 and args.parallel == "tp" and tensor_parallel.shards(config, args.gpus)


def scaling_label(args, config) -> str:
    return "weak" if args.gpus > 1 and not tensor_parallel_run(args, config) else "strong"


def parallelism_label(args, config) -> str:
    if args.gpus <= 1:
        return "single"
    if tensor_parallel_run(args, config):
        return (f"tp{args.gpus}: column-split QKV / gate / up / LM head, row-split o_proj / down with fp32 partial sums "
                f"reduced over peer memory (NVLink), attention split by KV head; one sequence set for all GPUs")
    return f"{args.gpus} independent replicas (one per GPU, no exchange)"


# ---- per-kernel timing ----------------------------------------------------------------------------

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


def roofline_entry(kernel: dict, peaks: dict) -> dict:
    entry = {
        "bound": "hbm", "kernel": kernel["name"], "achieved": kernel["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": kernel["gbs"] / peaks["hbm_gbs"], "peak_source": peaks["source"],
        "frac_of_spec_8000": kernel["gbs"] / 8000.0, "traffic": None, "traffic_source": None,
        "bytes_per_launch": kernel["bytes"], "ms_per_launch": kernel["ms"],
    }
    source = TRAFFIC_SOURCES.get(kernel["kernel"])
    captured = profile_traffic(*source) if source else None
    if captured:
        algorithmic, dram = captured
        # the captured launch's DRAM bytes, scaled to this launch by the algorithmic bytes (traffic grows in
        # proportion to the units processed)
        entry["traffic"] = round(kernel["bytes"] * dram / algorithmic)
        entry["traffic_source"] = f"{source[0]} ({source[1]}: {dram} DRAM bytes for {algorithmic} algorithmic)"
    return entry


def time_prefill_gemm(runtime, peaks, *, m, k, n, form, weights=None) -> dict:
    """One prefill product on the tcgen05 GEMM, device-timed back to back over distinct weights.
    ``form`` = "dual" (gate and up with the SwiGLU epilogue, two products), "affine" (unsigned
    nibbles with fp16 zero points, w = (u - z) s) or "linear"."""
    from llmopt_b200 import dispatch
    from llmopt_b200.cuda_native import Batch, Buffer

    rng = np.random.default_rng(1)
    x = dispatch.Tensor(Buffer.of_array(runtime, rng.standard_normal((m, k)).astype(np.float16)), (m, k))
    commands = Batch(runtime)
    context = dispatch.Context(runtime, batch=commands)

    def w4(rows, cols, low, high, zero=False):
        packed = dispatch.Tensor(Buffer.of_array(runtime, rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)),
                                 (rows, cols // 2), "uint8")
        scale = dispatch.Tensor(Buffer.of_array(runtime, rng.uniform(low, high, size=(rows, cols // 64)).astype(np.float16)),
                                (rows, cols // 64))
        if not zero:
            return packed, scale
        zeros = dispatch.Tensor(Buffer.of_array(runtime, rng.uniform(6, 9, size=(rows, cols // 64)).astype(np.float16)),
                                (rows, cols // 64))
        return packed, scale, zeros

    copies = max(2, min(4, (256 << 20) // max(n * k // 2, 1)))  # distinct weights so the L2 holds none of them
    products = 1
    if form == "dual":
        products = 2
        output = dispatch.Tensor(Buffer.create(runtime, m * k * 2), (m, k))
        for index in range(copies):
            layer = weights[index] if weights else None
            gate = layer["gate"] if layer else w4(n, k, 0.005, 0.02)
            up = layer["up"] if layer else w4(n, k, 0.005, 0.02)
            down = layer["down"] if layer else w4(k, n, 0.005, 0.02)
            norm = layer["ffn_norm"] if layer else dispatch.Tensor(Buffer.of_array(runtime, np.ones(k, np.float16)), (k,))
            dispatch.dispatch_w4a16_swiglu_ffn_command(
                context, m=m, n=n, k=k, epsilon=1e-5, activation=x, residual=x, gate_weight=gate[0], gate_scale=gate[1],
                up_weight=up[0], up_scale=up[1], down_weight=down[0], down_scale=down[1], norm_weight=norm,
                output=output, reference_guards=False)
        items = [item for item in commands.pending if item.name.startswith("llmopt_w4a16_dual_swiglu")]
    else:
        output = dispatch.Tensor(Buffer.create(runtime, m * n * 2), (m, n))
        for _ in range(copies):
            if form == "affine":
                packed, scale, zeros = w4(n, k, 0.002, 0.01, zero=True)
                dispatch.dispatch_w4a16_linear_affine(context, input=x, weight=packed, scale=scale, zero=zeros, output=output)
            else:
                packed, scale = w4(n, k, 0.002, 0.01)
                dispatch.dispatch_w4a16_linear(context, input=x, weight=packed, scale=scale, output=output)
        items = list(commands.pending)
    name = items[0].name
    milliseconds = runtime.time_dispatches(items, warmup=1, iterations=3)
    commands.abort()
    tflops = 2.0 * products * m * k * n / milliseconds / 1e9
    return {"kernel": name, "form": form, "m": m, "k": k, "n": n, "products": products, "ms": milliseconds,
            "bound": "tensor", "achieved": tflops, "unit": "TFLOP/s", "peak": peaks["bf16_tflops"],
            "frac": tflops / peaks["bf16_tflops"], "peak_sustained": peaks.get("bf16_tflops_sustained"),
            "frac_of_sustained": tflops / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"]}


def time_ffn_tensor_parallel(runtime, peaks, rank: int, world: int, group) -> list:
    """The 70B-shape SwiGLU FFN (hidden 8192, intermediate 28672) of a prompt, split over the ranks: every rank runs
    the RMS norm, gate and up with the SwiGLU epilogue on its 28672 / N intermediate columns and the down projection
    on the matching rows of K as an fp32 partial of all prompt rows, then the partials are added over peer memory
    (reduce-scatter + all-gather of the rows).  Device-timed back to back on every rank, max over ranks."""
    import torch
    import torch.distributed as dist

    from llmopt_b200 import dispatch, parameters, tensor_parallel
    from llmopt_b200.cuda_native import Batch, Buffer

    hidden, intermediate = 8192, 28672
    columns = intermediate // world
    rows_most = 8192
    rng = np.random.default_rng(11)  # the same whole matrices on every rank; a rank uploads its share
    exchange = tensor_parallel.ExchangeGroup.create(runtime, rank, world, rows_most * hidden * 4, 2,
                                                    tensor_parallel.torch_all_gather())

    def whole(rows, cols):
        return (rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8),
                rng.uniform(0.002, 0.01, size=(rows, cols // 64)).astype(np.float16))

    def upload(pair):
        return tuple(Buffer.of_array(runtime, np.ascontiguousarray(part)) for part in pair)

    whole_gate, whole_up, whole_down = whole(intermediate, hidden), whole(intermediate, hidden), whole(hidden, intermediate)
    mine = slice(rank * columns, (rank + 1) * columns)
    gate = upload((whole_gate[0][mine], whole_gate[1][mine]))   # this rank's intermediate columns: rows of gate / up
    up = upload((whole_up[0][mine], whole_up[1][mine]))
    down = upload((whole_down[0][:, rank * columns // 2:(rank + 1) * columns // 2],  # the matching stretch of K
                   whole_down[1][:, rank * columns // 64:(rank + 1) * columns // 64]))
    norm = Buffer.of_array(runtime, np.ones(hidden, np.float16))
    out = []
    check = None
    for m in (512, 2048, 8192):
        x = Buffer.of_array(runtime, np.random.default_rng(5).standard_normal((m, hidden)).astype(np.float16))
        normed, result = Buffer.create(runtime, m * hidden * 2), Buffer.create(runtime, m * hidden * 2)
        product = Buffer.create(runtime, m * columns * 2)
        commands = Batch(runtime)
        ffn = parameters.w4a16_swiglu_ffn(m=m, n=columns, k=hidden, epsilon=1e-5)
        commands.dispatch(name="llmopt_w4a16_swiglu_rms_f16_g64", buffers=[x, norm, normed], parameters=ffn,
                          grid=(m * 256, 1, 1), group=(256, 1, 1))
        commands.dispatch(name="llmopt_w4a16_dual_swiglu_f16_g64_m4",
                          buffers=[normed, gate[0], gate[1], up[0], up[1], product], parameters=ffn,
                          grid=(1, 1, 1), group=(256, 1, 1))
        commands.dispatch(name="llmopt_w4a16_linear_partial_f32_g64",
                          buffers=[product, down[0], down[1], exchange.slot_view(0, m * hidden * 4)],
                          parameters=parameters.u32s([m, hidden, columns]), grid=(1, 1, 1), group=(256, 1, 1))
        exchange.sum_rows_records(commands.dispatch, slot=0, slice_slot=1, rows=m, width=hidden, residual=x, output=result)
        items = list(commands.pending)
        dist.barrier()
        milliseconds = runtime.time_dispatches(items, warmup=2, iterations=5) * len(items)  # per FFN, not per launch
        commands.abort()
        if check is None:
            # the same layer unsplit, on rank 0 alone, against the exchanged result (every rank holds the same one)
            check = {"m": m, "bound": 2e-3}
            if rank == 0:
                single = Batch(runtime)
                context = dispatch.Context(runtime, batch=single)
                tensors = []
                for pair in (whole_gate, whole_up, whole_down):
                    packed, scale = upload(pair)
                    tensors.append((dispatch.Tensor(packed, pair[0].shape, "uint8"), dispatch.Tensor(scale, pair[1].shape)))
                expected = dispatch.Tensor(Buffer.create(runtime, m * hidden * 2), (m, hidden))
                activation = dispatch.Tensor(x, (m, hidden))
                dispatch.dispatch_w4a16_swiglu_ffn_command(
                    context, m=m, n=intermediate, k=hidden, epsilon=1e-5, activation=activation, residual=activation,
                    gate_weight=tensors[0][0], gate_scale=tensors[0][1], up_weight=tensors[1][0], up_scale=tensors[1][1],
                    down_weight=tensors[2][0], down_scale=tensors[2][1],
                    norm_weight=dispatch.Tensor(norm, (hidden,)), output=expected, reference_guards=False)
                single.commit()
                want = expected.buffer.to_numpy(np.float16, (m, hidden)).astype(np.float32)
                got = result.to_numpy(np.float16, (m, hidden)).astype(np.float32)
                check["max_error_over_scale"] = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
                check["equal_to_one_gpu"] = bool(check["max_error_over_scale"] <= check["bound"])
                del tensors, expected
            dist.barrier()
        worst = torch.tensor([milliseconds], dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        milliseconds = float(worst.item())
        tflops = 3 * 2.0 * m * hidden * intermediate / milliseconds / 1e9
        out.append({"m": m, "k": hidden, "n": intermediate, "parallelism": f"tp{world}", "ms": round(milliseconds, 4),
                    "tflops": round(tflops, 1), "tflops_per_gpu": round(tflops / world, 1),
                    "frac_of_measured_bf16_per_gpu": round(tflops / world / peaks["bf16_tflops"], 3),
                    "launches": len(items), "exchange_bytes_per_gpu": m * hidden * (4 + 2) * (world - 1) // world,
                    "data": "synthetic"})
        del x, normed, result, product
    dist.barrier()  # no rank unmaps its region while a peer may still read it
    runtime.synchronize()
    if check is not None:
        out[0]["check_against_one_gpu"] = check
    return out


def time_baseline_mode(runtime, peaks) -> dict:
    """The zero-point / group-32 input mode of the stated configurations, timed alone: the decode
    GEMV on unsigned nibbles with fp16 zero points (w = (u - z) s) at the gate shape, and the
    paged attention over a Q8 cache with one scale per 32 elements."""
    from llmopt_b200 import kernel_bench

    out = {}
    for label, fields in (
            ("gemv_affine_m1", dict(op="linear_affine", m=1, k=4096, n=14336)),
            ("gemv_contract_m1", dict(op="linear", m=1, k=4096, n=14336)),
            ("attention_group32_b8", dict(op="attention", m=8, group=32, layers=32)),
            ("attention_group64_b8", dict(op="attention", m=8, group=64, layers=32))):
        options = types.SimpleNamespace(op="linear", m=1, k=4096, n=14336, heads=32, kv_heads=8, dim=128, group=64,
                                        layers=2, past=8192)
        options.__dict__.update(fields)
        item, nbytes, keep = kernel_bench.build_item(runtime, options)
        milliseconds = runtime.time_dispatch(item, warmup=3, iterations=20, flush_l2=True)
        out[label] = {"kernel": item.name, "ms": round(milliseconds, 5), "bytes": nbytes,
                      "gbs": round(nbytes / milliseconds / 1e6, 1),
                      "frac": round(nbytes / milliseconds / 1e6 / peaks["hbm_gbs"], 3),
                      "mode": "isolated launch, L2 flushed before each"}
        del keep
    return out


def time_other_kernels(runtime, peaks) -> dict:
    """Kernels of the path that no leg above times: the Q4_0-block GEMV (GGUF blocks, 18 bytes per 32
    weights) at the gate shape against the HBM peak, and the dense causal prefill attention
    (mma.sync flash-attention forward) at 2048 tokens of the Llama-8B head geometry against the
    tensor peak."""
    from llmopt_b200 import kernel_bench

    out = {}
    options = types.SimpleNamespace(op="q4_0", m=1, k=4096, n=14336, heads=32, kv_heads=8, dim=128, group=64, layers=2,
                                    past=8192)
    # like the W4A16 kernels above: the same dispatch over distinct weights back to back (cold operands, the
    # launches' programmatic overlap as inside a plan), 8 x 33 MB against 126 MB of L2
    items, keeps, nbytes = [], [], 0
    for _ in range(8):
        item, nbytes, keep = kernel_bench.build_item(runtime, options)
        items.append(item)
        keeps.append(keep)
    milliseconds = runtime.time_dispatches(items, warmup=2, iterations=10)
    out["q4_0_gemv_m1"] = {"kernel": items[0].name, "ms": round(milliseconds, 5), "bytes": nbytes, "bound": "hbm",
                           "gbs": round(nbytes / milliseconds / 1e6, 1),
                           "frac": round(nbytes / milliseconds / 1e6 / peaks["hbm_gbs"], 3),
                           "mode": "8 distinct operand sets back to back"}
    milliseconds = runtime.time_dispatch(items[0], warmup=3, iterations=20, flush_l2=True)
    out["q4_0_gemv_m1"]["isolated_cold_launch_ms"] = round(milliseconds, 5)
    del items, keeps
    tokens = 2048
    options = types.SimpleNamespace(op="dense_attention", m=tokens, k=0, n=0, heads=32, kv_heads=8, dim=128, group=64,
                                    layers=2, past=0)
    item, nbytes, keep = kernel_bench.build_item(runtime, options)
    milliseconds = runtime.time_dispatch(item, warmup=3, iterations=10, flush_l2=True)
    flops = 2.0 * tokens * tokens * 128 * 32  # causal: half of the square, two products per head
    out["dense_attention_causal_2048"] = {
        "kernel": item.name, "ms": round(milliseconds, 5), "bound": "tensor", "tflops": round(flops / milliseconds / 1e9, 1),
        "frac": round(flops / milliseconds / 1e9 / peaks["bf16_tflops"], 3),
        "note": "legacy tensor path (mma.sync), fp16, 32 query / 8 KV heads of 128", "mode": "isolated launch"}
    del keep
    return out


# ---- decode measurement ---------------------------------------------------------------------------

def measure_decode(engine, runtime, args, group, *, context: int, jobs: int, device_index: int, peaks: dict) -> dict:
    """Device-timed chained decode (median of REPETITIONS x K steps, max over ranks), the host-driven
    end-to-end loop, the per-kernel table and the roofline of the dominant kernel."""
    batch, config = engine.batch, engine.config
    rng = np.random.default_rng(0)
    first = rng.integers(0, config.vocabulary, size=batch).tolist()
    warmup = max(args.warmup, 3)
    engine.generate_chained(first, context, warmup)
    sampler = ClockSampler(device_index)
    repetitions = []
    token_streams = []
    for _ in range(REPETITIONS):
        if group is not None:
            group.barrier()
        runtime.synchronize()
        tokens, elapsed_ms = engine.generate_chained(first, context, args.steps)
        runtime.synchronize()
        if group is not None:
            import torch

            slowest = torch.tensor([elapsed_ms], dtype=torch.float64)
            group.all_reduce(slowest, op=group.ReduceOp.MAX)  # device-timed on every rank, max over ranks
            elapsed_ms = float(slowest.item())
        repetitions.append(elapsed_ms)
        token_streams.append(tokens)
    if group is not None:
        group.barrier()
    clocks = sampler.stop()
    elapsed_ms = statistics.median(repetitions)
    ms_per_step = elapsed_ms / args.steps
    value = jobs * batch * 1000.0 / ms_per_step

    # end to end: the host drives every token (token id in, H2D; next id out, D2H)
    tokens = first
    for step in range(warmup):
        tokens = engine.step(tokens, context + step)
    runtime.synchronize()
    start = time.perf_counter()
    for step in range(args.steps):
        tokens = engine.step(tokens, context + step)
    runtime.synchronize()
    e2e_seconds = time.perf_counter() - start
    if group is not None:
        import torch

        slowest = torch.tensor([e2e_seconds], dtype=torch.float64)
        group.all_reduce(slowest, op=group.ReduceOp.MAX)
        e2e_seconds = float(slowest.item())
    e2e_value = jobs * batch * args.steps / e2e_seconds
    h2d = 16 + (8 * batch if batch > 1 else 0)
    d2h = 4 + (4 * batch if batch > 1 else 0)

    kernels = time_kernels(engine, runtime)
    dominant = kernels.get("gate_up_swiglu") or next(iter(kernels.values()))
    if batch >= 8 and "paged_attention_q8" in kernels:
        attention_ms = kernels["paged_attention_q8"]["ms"] * config.attention_layers
        if attention_ms > dominant["ms"] * len(config.layers):
            dominant = kernels["paged_attention_q8"]
    from llmopt_b200.model import decode_bytes_per_token

    step_bytes = decode_bytes_per_token(config, batch, context)
    return {
        "value": value, "unit": "tokens/s", "ms_per_step": ms_per_step, "batch": batch, "context": context,
        "repetitions_ms": [round(v, 4) for v in repetitions],
        "tokens_identical_across_repetitions": all(stream == token_streams[0] for stream in token_streams),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": (engine.plan.kernel_count() + 1) * args.steps,
        "kernels_per_step": engine.plan.kernel_count(),
        "clocks": clocks,
        "roofline": roofline_entry(dominant, peaks),
        "step_roofline": {
            "algorithmic_bytes_per_step": step_bytes["total"], "weights": step_bytes["weights"],
            "attention": step_bytes["attention"], "achieved_gbs": step_bytes["total"] / ms_per_step / 1e6,
            "frac": step_bytes["total"] / ms_per_step / 1e6 / peaks["hbm_gbs"],
        },
        "kernels": {k: {"ms": round(v["ms"], 5), "gbs": round(v["gbs"], 1), "frac": round(v["gbs"] / peaks["hbm_gbs"], 3)}
                    for k, v in kernels.items()},
        "_tokens": token_streams[0],
    }


def small_model_leg(runtime, args, name: str, peaks: dict, batch: int = 1) -> dict:
    """A launch-latency-bound model of the stated configurations: tokens/s next to the floor the
    launches alone set (the same plan's kernel count times the measured cost of an empty dependent
    launch is not separable on the device, so the floor reported is bytes / HBM peak)."""
    from llmopt_b200 import model
    from llmopt_b200.decode_engine import DecodeEngine

    config = getattr(model, WORKLOADS[name])
    context = DEFAULT_CONTEXT[name]
    weights = model.random_weights(config, seed=0, fast=True)
    engine = DecodeEngine(runtime, config, weights, batch=batch, capacity=context + 8 * (args.steps + args.warmup) + 64)
    del weights
    engine.fill_cache_random(context, seed=0)
    engine.build(context)
    first = np.random.default_rng(0).integers(0, config.vocabulary, size=batch).tolist()
    engine.generate_chained(first, context, max(args.warmup, 3))
    times = []
    for _ in range(REPETITIONS):
        _, elapsed = engine.generate_chained(first, context, args.steps)
        times.append(elapsed / args.steps)
    ms_per_step = statistics.median(times)
    step_bytes = model.decode_bytes_per_token(config, batch, context)
    return {
        "workload": f"{config.name}, batch {batch}, context {context}", "value": batch * 1000.0 / ms_per_step,
        "unit": "tokens/s", "ms_per_step": ms_per_step, "kernels_per_step": engine.plan.kernel_count(),
        "us_per_kernel": 1000.0 * ms_per_step / engine.plan.kernel_count(),
        "algorithmic_bytes_per_step": step_bytes["total"],
        "hbm_floor_ms": step_bytes["total"] / peaks["hbm_gbs"] / 1e6,
        "frac_of_hbm": step_bytes["total"] / ms_per_step / 1e6 / peaks["hbm_gbs"],
        "bound": "launch latency: the whole step moves less than the L2 holds per launch",
    }


PREFILL_TOKENS = 512


def time_prefill(engine, runtime, tokens: int, group=None) -> dict:
    """Time to first token through the prefill path: the whole prompt in one pass (one row per
    token through every linear, dense causal attention, bulk cache pack), wall clock around the
    call that returns the first generated token; the prompt ids go host to device, the token comes back."""
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, engine.config.vocabulary, size=tokens).tolist()
    engine.prefill(prompt)  # warm-up (scratch growth, first-use kernel loads); it also records the pass for this length
    first_record = engine.prefill_seconds[0]
    runtime.synchronize()
    samples = []
    for _ in range(3):
        if group is not None:
            group.barrier()  # every rank has finished the previous prompt's exchanges
        start = time.perf_counter()
        engine.prefill(prompt)
        samples.append((time.perf_counter() - start, *engine.prefill_seconds))
    seconds, record, execute = sorted(samples)[1]
    return {"prompt_tokens": tokens, "ttft_ms": seconds * 1e3, "prompt_tokens_per_s": tokens / seconds,
            "record_ms": record * 1e3, "execute_ms": execute * 1e3, "execute_tokens_per_s": tokens / execute,
            "first_record_ms": first_record * 1e3,
            "kernels": engine.prefill_kernels, "h2d_bytes": 8 * tokens, "d2h_bytes": 4,
            "note": "median of 3, empty KV cache; a prompt length seen before replays its recorded dispatch list "
                    "(record = upload of the ids and hand-over of the list; first_record = the host side building the "
                    "list the first time, Python); execute = commit of the list until the first token is back on the host"}


def tensor_parallel_check(args, whole_config, whole_weights, runtime, rank, world, group, timed_tokens) -> dict:
    """Correctness of the tensor-parallel run on real peers: (1) every rank produced the same token
    stream in the timed run; (2) a short decode from an empty cache gives, on every rank, the same
    tokens, and its final hidden state equals an unsharded single-GPU run of the same seeded
    weights (rank 0) within 2e-3 of the state's scale."""
    from llmopt_b200 import tensor_parallel
    from llmopt_b200.decode_engine import DecodeEngine

    gathered = [None] * world
    group.all_gather_object(gathered, list(timed_tokens))
    ranks_identical = all(stream == gathered[0] for stream in gathered)

    steps, batch = 16, 1
    exchange_group = tensor_parallel.ExchangeGroup.create(
        runtime, rank, world, max(batch * whole_config.hidden * 4, 256 * 8), 7, tensor_parallel.torch_all_gather())
    shard = tensor_parallel.shard_weights(whole_config, whole_weights, rank, world)
    engine = DecodeEngine(runtime, tensor_parallel.local_config(whole_config, world), shard, batch=batch, capacity=64,
                          group=exchange_group)
    del shard
    engine.build(0)
    first = [int(np.random.default_rng(7).integers(0, whole_config.vocabulary))]
    sharded_tokens, hidden_states = [], []
    tokens = first
    for step in range(steps):
        tokens = engine.step(tokens, step)
        sharded_tokens.append(int(tokens[0]))
        hidden_states.append(engine.final_hidden.buffer.to_numpy(np.float16).astype(np.float64))
    group.barrier()
    streams = [None] * world
    group.all_gather_object(streams, sharded_tokens)
    result = {"timed_tokens_identical_across_ranks": ranks_identical,
              "short_run_tokens_identical_across_ranks": all(stream == streams[0] for stream in streams),
              "steps": steps}
    if rank == 0:
        single = DecodeEngine(runtime, whole_config, whole_weights, batch=batch, capacity=64)
        single.build(0)
        tokens, equal_prefix, worst = first, 0, 0.0
        diverged = False
        for step in range(steps):
            # teacher-forced with the sharded run's tokens so every step compares the same input
            tokens = single.step(first if step == 0 else [sharded_tokens[step - 1]], step)
            reference_hidden = single.final_hidden.buffer.to_numpy(np.float16).astype(np.float64)
            scale = max(float(np.max(np.abs(reference_hidden))), 1e-6)
            worst = max(worst, float(np.max(np.abs(hidden_states[step] - reference_hidden))) / scale)
            if not diverged and int(tokens[0]) == sharded_tokens[step]:
                equal_prefix += 1
            else:
                diverged = True
        result.update({"hidden_max_rel_err_vs_single_gpu": worst, "hidden_tolerance": 2e-3,
                       "tokens_equal_to_single_gpu": equal_prefix, "hidden_within_tolerance": worst <= 2e-3})
        del single
    group.barrier()
    result["tokens_match"] = bool(result["timed_tokens_identical_across_ranks"]
                                  and result["short_run_tokens_identical_across_ranks"]
                                  and result.get("hidden_within_tolerance", True))
    return result


def run_native(args, config, rank: int, world: int, local: int, group) -> dict:
    from llmopt_b200 import cuda_native
    from llmopt_b200.decode_engine import DecodeEngine
    from llmopt_b200.model import random_weights

    # N > 1: tensor parallel when the model splits over N ranks (every rank decodes the same
    # sequences with its share of every layer), else one independent replica of the whole model
    # per GPU (no exchange on the data path).
    runtime = cuda_native.Runtime(local)
    whole_config = config
    fast = config.hidden >= 2048
    whole_weights = random_weights(config, seed=0, fast=fast)
    weights = whole_weights
    # the repetitions and the end-to-end loop restart at `context`; only the longest run matters
    capacity = args.context + max(args.steps, args.warmup, 3) + 16
    tensor_parallel_mode = tensor_parallel_run(args, config)
    peaks = measured_peaks()
    extra_legs = not args.no_extra_legs and args.workload == "llama3-8b" and args.batch == 1

    def make_engine(batch, share=None):
        if tensor_parallel_mode:
            from llmopt_b200 import tensor_parallel

            # slots of the first engine also hold the fp32 partial sums of a 512-token prompt (the prefill leg)
            rows = max(batch, PREFILL_TOKENS if share is None and extra_legs else batch)
            exchange_group = tensor_parallel.ExchangeGroup.create(
                runtime, rank, world, max(rows * whole_config.hidden * 4, min(batch, 32) * 256 * 8), 7,
                tensor_parallel.torch_all_gather())
            local_weights = None if share is not None else tensor_parallel.shard_weights(whole_config, whole_weights, rank, world)
            return DecodeEngine(runtime, tensor_parallel.local_config(whole_config, world), local_weights, batch=batch,
                                capacity=capacity, group=exchange_group, share_weights_of=share)
        return DecodeEngine(runtime, whole_config, None if share is not None else weights, batch=batch,
                            capacity=capacity, share_weights_of=share)

    engine = make_engine(args.batch)
    engine.fill_cache_random(args.context, seed=0)
    engine.build(args.context)
    jobs = 1 if tensor_parallel_mode else world  # tensor parallel: all GPUs decode the same sequences
    head = measure_decode(engine, runtime, args, group, context=args.context, jobs=jobs, device_index=local, peaks=peaks)
    timed_tokens = head.pop("_tokens")
    result = {
        "metric": METRIC, "value": head["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
        "scaling": scaling_label(args, whole_config),
        "vs_baseline": None, "dtype": "w4a16 (int4 weights, f16 activations, f32 accumulate); q8 KV",
        "data": "synthetic", "config": workload_config(args, whole_config),
        "repetitions": REPETITIONS, "timing": f"median of {REPETITIONS} repetitions of the {args.steps} steps",
    }
    for key in ("e2e", "gpu_launches", "kernels_per_step", "clocks", "roofline", "step_roofline", "kernels",
                "repetitions_ms", "tokens_identical_across_repetitions"):
        result[key] = head[key]

    if extra_legs:
        # the metric's second batch size, same weights, same process
        wide = make_engine(32, share=engine)
        wide.fill_cache_random(args.context, seed=0)
        wide.build(args.context)
        leg = measure_decode(wide, runtime, args, group, context=args.context, jobs=jobs, device_index=local, peaks=peaks)
        leg.pop("_tokens")
        leg["config"] = workload_config(args, whole_config, batch=32)
        result["batch32"] = leg
        result["gpu_launches"] += leg["gpu_launches"]
        del wide
        if world == 1:
            # the stated configuration's other batch sizes, in short: same weights, same process
            for other_batch in (8, 64):
                other = make_engine(other_batch, share=engine)
                other.fill_cache_random(args.context, seed=0)
                other.build(args.context)
                leg = measure_decode(other, runtime, args, group, context=args.context, jobs=jobs, device_index=local,
                                     peaks=peaks)
                result[f"batch{other_batch}"] = {key: leg[key] for key in (
                    "value", "unit", "ms_per_step", "e2e", "kernels_per_step", "gpu_launches", "repetitions_ms",
                    "tokens_identical_across_repetitions", "clocks") if key in leg}
                result["gpu_launches"] += leg["gpu_launches"]
                del other

    if tensor_parallel_mode:
        result["tp_check"] = tensor_parallel_check(args, whole_config, whole_weights, runtime, rank, world, group, timed_tokens)
        result["tokens_match"] = result["tp_check"]["tokens_match"]
    del whole_weights, weights

    if extra_legs:
        if group is not None:
            group.barrier()  # no exchange of the decode legs is in flight on any rank when the prompt starts
        result["prefill"] = time_prefill(engine, runtime, PREFILL_TOKENS, group)
        if tensor_parallel_mode:
            result["prefill"]["parallelism"] = f"tp{world}: the same pass on every rank's heads and columns, o_proj and down as row splits with their fp32 partial sums added over peer memory"
    if tensor_parallel_mode and extra_legs:
        result["prefill_ffn_c5"] = time_ffn_tensor_parallel(runtime, peaks, rank, world, group)
    if world == 1 and config.hidden >= 2048:
        result["prefill_gemm"] = time_prefill_gemm(runtime, peaks, m=2048, k=config.hidden, n=config.intermediate,
                                                   form="dual", weights=engine.layers[:4])
    if world == 1 and extra_legs:
        del engine
        sweep = []
        for m in (512, 2048, 8192):
            sweep.append(time_prefill_gemm(runtime, peaks, m=m, k=8192, n=28672, form="affine"))   # gate or up
            sweep.append(time_prefill_gemm(runtime, peaks, m=m, k=28672, n=8192, form="affine"))   # down
        sweep.append(time_prefill_gemm(runtime, peaks, m=2048, k=8192, n=28672, form="linear"))
        result["prefill_gemm_c5"] = sweep
        result["baseline_mode"] = time_baseline_mode(runtime, peaks)
        result["other_kernels"] = time_other_kernels(runtime, peaks)
        result["smollm2_135m"] = small_model_leg(runtime, args, "smollm2-135m", peaks)
        result["lfm25_350m"] = small_model_leg(runtime, args, "lfm2.5-350m", peaks)
        result["lfm25_350m_batch16"] = small_model_leg(runtime, args, "lfm2.5-350m", peaks, batch=16)
    if group is not None:
        group.barrier()  # no rank leaves (and unmaps its exchange region) while a peer still runs
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        baseline = cpu_reference_rate(whole_config, args.batch, args.context)
        result["cpu_baseline"] = {k: baseline[k] for k in ("value", "unit", "cores", "kind", "sample", "single_thread", "linears_only")}
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
    parser.add_argument("--no-extra-legs", action="store_true",
                        help="only the headline batch: no batch-32, small-model, prefill-sweep or input-mode legs")
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
