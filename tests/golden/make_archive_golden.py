"""Writes tests/golden/tiny_weights.llmoptwt with the reference's own exporter
(python/llmopt_backend/tensor_archive.py, imported from the reference checkout), so the reader is
pinned against bytes the reference produced.  Run once, in a container that has the reference:

    python tests/golden/make_archive_golden.py /path/to/reference
"""

import os
import sys

import numpy as np


def tensors():
    """Seeded payloads: a W4A16 weight + scales, a Q4_0 tensor, an fp16 norm weight, an int64 table."""
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
    from llmopt_b200.quantize import q4_0_blocks

    rng = np.random.default_rng(123)
    packed = rng.integers(0, 256, size=(16, 64), dtype=np.uint8)               # W4A16 [16, 128/2]
    scale = rng.uniform(0.005, 0.02, size=(16, 2)).astype(np.float16)           # [16, 128/64]
    q4 = q4_0_blocks(rng.uniform(0.01, 0.03, size=(8, 2)).astype(np.float16),
                     rng.integers(0, 16, size=(8, 64), dtype=np.uint8))         # Q4_0 [8, 64] = 16 blocks
    norm = rng.uniform(0.5, 1.5, size=(128,)).astype(np.float16)
    table = np.arange(5, dtype=np.int64) * 7
    return {
        "layers.0.ffn_norm.weight": ("float16", (128,), norm.tobytes()),
        "layers.0.gate.packed": ("uint8", (16, 64), packed.tobytes()),
        "layers.0.gate.scale": ("float16", (16, 2), scale.tobytes()),
        "layers.0.q.weight": ("Q4_0", (8, 64), q4.tobytes()),
        "positions": ("int64", (5,), table.tobytes()),
    }


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: make_archive_golden.py /path/to/reference")
    reference = sys.argv[1]
    sys.path.insert(0, os.path.join(reference, "python"))
    from llmopt_backend import tensor_archive

    payloads = tensors()
    specs = [tensor_archive.TensorSpec(name, tensor_archive.DTYPE_TAGS[dtype], shape, len(data))
             for name, (dtype, shape, data) in payloads.items()]
    destination = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_weights.llmoptwt")
    summary = tensor_archive.write_payloads(specs, destination, lambda name: (payloads[name][2],))
    print(summary)


if __name__ == "__main__":
    main()
