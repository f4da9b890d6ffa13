"""Generates tests/golden/w4a16_reference.npz by running the REFERENCE's own
Python implementation of the W4A16 path (python/llmopt_backend/quantization.py:
pack_int4_weight, unpack_int4_weight, the fp32-accumulate `w4a16_linear`
fallback and the W4A16Linear module) on seeded inputs.  Run where the reference
checkout is mounted:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The fixture travels with the repository; the tests never import the reference.
"""

import sys

import numpy as np
import torch


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root + "/python")
    from llmopt_backend import quantization as q

    torch.manual_seed(0)
    out = {}
    # pack / unpack on random-init weights at the reference runtime test's own shape and a ragged one
    for tag, (n, k) in {"c1": (1536, 576), "small": (29, 128)}.items():
        weight = torch.randn(n, k) * 0.02
        packed, scale = q.pack_int4_weight(weight)
        out[f"{tag}_packed"] = packed.numpy()
        out[f"{tag}_scale"] = scale.numpy()
        if tag == "small":  # the fp32 originals are kept for the small case only (fixture size)
            out[f"{tag}_weight"] = weight.numpy()
            out[f"{tag}_unpacked"] = q.unpack_int4_weight(packed, scale).numpy()
        else:
            rows = torch.arange(0, n, 97)
            out[f"{tag}_unpacked_rows"] = q.unpack_int4_weight(packed, scale)[rows].numpy()
        for m in (1, 128) if tag == "c1" else (3,):
            x = torch.randn(m, k).half()
            bias = torch.randn(n).half()
            module = q.W4A16Linear(packed, scale, bias)
            out[f"{tag}_x{m}"] = x.numpy()
            out[f"{tag}_bias{m}"] = bias.numpy()
            out[f"{tag}_y{m}"] = module(x).detach().numpy()
            out[f"{tag}_y{m}_nobias"] = q.W4A16Linear(packed, scale, None)(x).detach().numpy()
    # nibble order pin (python/tests/test_quantization.py:25-31)
    packed = torch.tensor([[0x78] * 32], dtype=torch.uint8)
    out["nibble_unpacked"] = q.unpack_int4_weight(packed, torch.ones(1, 1).half()).numpy()
    np.savez_compressed(__file__.rsplit("/", 1)[0] + "/w4a16_reference.npz", **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1])
