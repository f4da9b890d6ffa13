"""Shapes and synthetic weights of the decoder families the hot path serves:
Llama-style blocks (RMSNorm, fused QKV, RoPE, GQA attention over the Q8 cache,
SwiGLU FFN) and LFM-style gated short-conv blocks (lib/lfm25.ml:18-34).  The
weights are random-init and quantised W4A16 group-64; there is no checkpoint
loader here — a compiled package brings its own tensors."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

from .quantize import pack_int4_weight


@dataclass(frozen=True)
class ModelConfig:
    name: str
    hidden: int
    layers: Sequence[str]          # "attention" or "conv" per block
    query_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocabulary: int
    epsilon: float = 1e-5
    rope_theta: float = 1e5
    kv_group_size: int = 64

    @property
    def attention_layers(self) -> int:
        return sum(1 for kind in self.layers if kind == "attention")

    @property
    def conv_layers(self) -> int:
        return sum(1 for kind in self.layers if kind == "conv")


SMOLLM2_135M = ModelConfig("smollm2-135m-shaped", 576, ("attention",) * 30, 9, 3, 64, 1536, 49152, 1e-5, 1e5)
# lib/lfm25.ml:30-33: conv and attention blocks interleaved, 10 conv + 6 attention
LFM25_350M = ModelConfig(
    "lfm2.5-350m-shaped", 1024,
    ("conv", "conv", "attention", "conv", "conv", "attention", "conv", "conv", "attention", "conv", "attention",
     "conv", "attention", "conv", "attention", "conv"),
    16, 8, 64, 4608, 65536, 1e-5, 1e6)
LLAMA3_8B = ModelConfig("llama-3-8b-shaped", 4096, ("attention",) * 32, 32, 8, 128, 14336, 128256, 1e-5, 5e5)


def tiny_config(layers=("attention", "attention"), hidden=192, heads=3, kv_heads=1, head_dim=64, intermediate=384,
                vocabulary=1024) -> ModelConfig:
    return ModelConfig("tiny", hidden, tuple(layers), heads, kv_heads, head_dim, intermediate, vocabulary, 1e-5, 1e5)


def _quantized(rng, n, k, std, fast):
    if fast:
        # uniform random nibbles and scales: same bytes-per-weight, no host quantisation pass
        packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
        scale = rng.uniform(0.5 * std / 7 * 3, 1.5 * std / 7 * 3, size=(n, k // 64)).astype(np.float16)
        return packed, scale
    return pack_int4_weight((rng.standard_normal((n, k)) * std).astype(np.float32))


def random_weights(config: ModelConfig, seed: int = 0, std: float = 0.02, fast: bool = False) -> dict:
    """Random-init N(0, std) weights quantised with the reference quantiser.
    ``fast`` draws packed bytes and scales directly (for multi-GB models)."""
    rng = np.random.default_rng(seed)
    hidden, dim = config.hidden, config.head_dim
    weights = {}
    embedding = (rng.standard_normal((config.vocabulary, hidden)) * std).astype(np.float32)
    weights["embedding"] = embedding.astype(np.float16)
    if fast:
        weights["lm_head"] = _quantized(rng, config.vocabulary, hidden, std, True)
    else:
        weights["lm_head"] = pack_int4_weight(embedding)  # tied embeddings: W4 copy of the table
    weights["final_norm"] = np.ones(hidden, np.float16)
    for index, kind in enumerate(config.layers):
        layer = {"input_norm": np.ones(hidden, np.float16), "ffn_norm": np.ones(hidden, np.float16)}
        if kind == "attention":
            layer["q"] = _quantized(rng, config.query_heads * dim, hidden, std, fast)
            layer["k"] = _quantized(rng, config.kv_heads * dim, hidden, std, fast)
            layer["v"] = _quantized(rng, config.kv_heads * dim, hidden, std, fast)
            layer["o"] = _quantized(rng, hidden, config.query_heads * dim, std, fast)
        else:
            layer["in_proj"] = _quantized(rng, 3 * hidden, hidden, std, fast)
            layer["conv"] = (rng.standard_normal((hidden, 1, 3)) * 0.5).astype(np.float16)
            layer["out_proj"] = _quantized(rng, hidden, hidden, std, fast)
        layer["gate"] = _quantized(rng, config.intermediate, hidden, std, fast)
        layer["up"] = _quantized(rng, config.intermediate, hidden, std, fast)
        layer["down"] = _quantized(rng, hidden, config.intermediate, std, fast)
        weights[f"layer{index}"] = layer
    return weights


def decode_bytes_per_token(config: ModelConfig, batch: int, past: int) -> dict:
    """Algorithmic bytes one decode step must move: every weight matrix and scale
    once, the KV of every sequence once, activations negligible but counted for
    the linears (x once, y once per op)."""
    hidden, dim = config.hidden, config.head_dim

    def linear(n, k):
        return n * k // 2 + n * (k // 64) * 2 + batch * k * 2 + batch * n * 2

    weights = 0
    for kind in config.layers:
        if kind == "attention":
            weights += linear((config.query_heads + 2 * config.kv_heads) * dim, hidden)
            weights += linear(hidden, config.query_heads * dim)
        else:
            weights += linear(3 * hidden, hidden) + linear(hidden, hidden)
        weights += 2 * linear(config.intermediate, hidden) + linear(hidden, config.intermediate)
    weights += linear(config.vocabulary, hidden)
    kv_per_token = 2 * config.kv_heads * dim + 2 * 2 * config.kv_heads * dim // config.kv_group_size
    attention = config.attention_layers * batch * (past * (kv_per_token + 4))
    return {"weights": weights, "attention": attention, "total": weights + attention + hidden * 2 * batch}
