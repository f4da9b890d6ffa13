"""Shared builders of seeded synthetic inputs for the parity tests."""

import numpy as np


def random_w4(rng, n, k, scale_range=(0.005, 0.02)):
    """Uniform nibbles 0..15 packed low-nibble-first, fp16 group-64 scales."""
    codes = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    scale = rng.uniform(*scale_range, size=(n, k // 64)).astype(np.float16)
    return packed, scale


def random_pool(rng, capacity, layout_bytes, token_elements, group_size, scale_range=(0.004, 0.02)):
    """A token pool with random int8 payload (-127..127) and valid fp16 scales."""
    pool = np.zeros((capacity, layout_bytes), dtype=np.uint8)
    pool[:, :token_elements] = rng.integers(-127, 128, size=(capacity, token_elements), dtype=np.int8).view(np.uint8)
    groups = (layout_bytes - token_elements) // 2
    scales = rng.uniform(*scale_range, size=(capacity, groups)).astype(np.float16)
    pool[:, token_elements:] = scales.view(np.uint8).reshape(capacity, groups * 2)
    return pool.reshape(-1)
