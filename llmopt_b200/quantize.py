"""W4A16 weight packing in numpy: the reference's ``pack_int4_weight`` /
``unpack_int4_weight`` (python/llmopt_backend/quantization.py:63-121) and the
serving RoPE tables (lib/serving_rope_table.ml:147-175).  Used to prepare
weights on the host; nothing here runs per token."""

from __future__ import annotations

import numpy as np

GROUP_SIZE = 64
_QMIN, _QMAX = -8, 7


def pack_int4_weight(weight: np.ndarray):
    """fp [N, K] -> (packed u8 [N, K/2], scale f16 [N, K/64]): symmetric per
    group of 64, scale = max(amax, eps) / 7 in fp32, q = clamp(round(w / scale)),
    two's-complement nibbles, low nibble = even k."""
    if weight.ndim != 2:
        raise ValueError(f"W4 weight must be 2-D, got shape {tuple(weight.shape)}")
    n, k = weight.shape
    if n <= 0 or k <= 0:
        raise ValueError("W4 weight dimensions must be positive")
    if k % GROUP_SIZE != 0:
        raise ValueError(f"W4 weight K dimension must be a multiple of {GROUP_SIZE}, got {k}")
    source = weight.astype(np.float32).reshape(n, k // GROUP_SIZE, GROUP_SIZE)
    scale = np.maximum(np.abs(source).max(axis=-1), np.finfo(np.float32).eps).astype(np.float32) / np.float32(_QMAX)
    quantized = np.clip(np.rint(source / scale[..., None]), _QMIN, _QMAX).astype(np.int16)
    nibbles = np.remainder(quantized, 16).astype(np.uint8)
    packed = (nibbles[..., 0::2] | (nibbles[..., 1::2] << 4)).reshape(n, k // 2)
    return np.ascontiguousarray(packed), np.ascontiguousarray(scale.astype(np.float16))


def unpack_int4_weight(packed: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """(packed, scale) -> fp32 [N, K]."""
    if packed.dtype != np.uint8:
        raise TypeError(f"packed W4 weight storage must be uint8, got {packed.dtype}")
    if scale.dtype != np.float16:
        raise TypeError(f"W4 scales must be float16, got {scale.dtype}")
    n, half_k = packed.shape
    groups = half_k * 2 // GROUP_SIZE
    if scale.shape != (n, groups):
        raise ValueError(f"W4 scales must have shape [{n}, {groups}], got {list(scale.shape)}")
    nibbles = np.stack((packed & 0x0F, (packed >> 4) & 0x0F), axis=-1).reshape(n, groups, GROUP_SIZE).astype(np.int16)
    signed = np.where(nibbles < 8, nibbles, nibbles - 16)
    return (signed.astype(np.float32) * scale.astype(np.float32)[..., None]).reshape(n, half_k * 2)


def rope_tables(positions: int, head_dim: int, theta: float):
    """cos / sin tables f16 [positions, head_dim] with duplicated halves: fp32
    inv_freq * position -> fp32 cos / sin -> f16 (lib/serving_rope_table.ml:157-172)."""
    half = head_dim // 2
    inv_freq = (1.0 / (np.float64(theta) ** (np.arange(half, dtype=np.float64) * 2.0 / head_dim))).astype(np.float32)
    frequency = (inv_freq[None, :] * np.arange(positions, dtype=np.float32)[:, None]).astype(np.float32)
    cosine = np.cos(frequency.astype(np.float64)).astype(np.float32).astype(np.float16)
    sine = np.sin(frequency.astype(np.float64)).astype(np.float32).astype(np.float16)
    return np.concatenate([cosine, cosine], axis=1), np.concatenate([sine, sine], axis=1)


def q4_0_blocks(scales, nibbles):
    """Q4_0 weight rows from fp16 block scales [n, k/32] and nibbles 0..15 [n, k]
    (element i of a block in the low nibble of byte i for i < 16, in the high nibble of
    byte i - 16 otherwise; bin/ocaml_metal_primitives_smoke.ml:39-52): uint8 [n, (k/32)*18]."""
    import numpy as np

    scales = np.ascontiguousarray(scales, dtype=np.float16)
    nibbles = np.ascontiguousarray(nibbles, dtype=np.uint8)
    n, blocks = scales.shape
    grouped = nibbles.reshape(n, blocks, 32)
    out = np.empty((n, blocks, 18), np.uint8)
    out[:, :, 0:2] = scales.view(np.uint8).reshape(n, blocks, 2)
    out[:, :, 2:18] = grouped[:, :, :16] | (grouped[:, :, 16:] << 4)
    return out.reshape(n, blocks * 18)
