"""The LLMOPTWT reader against an archive written by the reference's own exporter
(tests/golden/tiny_weights.llmoptwt, made by tests/golden/make_archive_golden.py), and the
validation rules of lib/weight_archive.ml on corrupted copies."""

import os
import struct
import sys

import numpy as np
import pytest

from llmopt_b200 import weight_archive

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_weights.llmoptwt")


def _expected():
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from make_archive_golden import tensors

    return tensors()


def test_reference_written_archive_reads_back():
    archive = weight_archive.Archive(GOLDEN)
    expected = _expected()
    assert [t.name for t in archive.tensors] == sorted(expected)  # strictly sorted names
    assert archive.index_bytes == 512 and archive.file_size == 2600
    names = {"float16": "F16", "uint8": "U8", "int64": "I64", "Q4_0": "Q4_0"}
    for name, (dtype, shape, data) in expected.items():
        tensor = archive.find(name)
        assert tensor.dtype == names[dtype] and tensor.shape == tuple(shape)
        assert tensor.offset % 256 == 0 and tensor.byte_length == len(data)
        assert archive.read(name) == data
    assert archive.find("missing") is None
    assert archive.find("layers.0.q.weight").byte_length == 8 * 64 // 32 * 18  # Q4_0: 18 bytes per 32 weights


def _corrupt(tmp_path, edit):
    data = bytearray(open(GOLDEN, "rb").read())
    edit(data)
    path = tmp_path / "bad.llmoptwt"
    path.write_bytes(bytes(data))
    return str(path)


@pytest.mark.parametrize("edit,message", [
    (lambda d: d.__setitem__(0, ord("X")), "invalid weight-archive magic"),
    (lambda d: d.__setitem__(slice(8, 10), struct.pack("<H", 2)), "unsupported weight-archive version"),
    (lambda d: d.__setitem__(slice(10, 12), struct.pack("<H", 1)), "unsupported weight-archive flags"),
    (lambda d: d.__setitem__(slice(12, 16), struct.pack("<I", 0)), "contains no tensors"),
    (lambda d: d.__setitem__(24 + 6, 1), "reserved field is non-zero"),
    (lambda d: d.__setitem__(24 + 4, 99), "unknown weight-archive dtype tag"),
    (lambda d: d.__setitem__(500, 1), "index padding contains non-zero bytes"),
    (lambda d: d.extend(b"\\0"), "trailing or missing payload bytes"),
])
def test_validation_rules(tmp_path, edit, message):
    with pytest.raises(weight_archive.ArchiveError, match=message):
        weight_archive.Archive(_corrupt(tmp_path, edit))


def test_names_must_be_sorted_and_lengths_consistent(tmp_path):
    # swap the first two characters of the second name so that it sorts before the first
    def unsort(data):
        first_name_length = struct.unpack_from("<I", data, 24)[0]
        second = 24 + 8 + first_name_length + 8 * 1 + 16  # first tensor has rank 1
        start = second + 8
        data[start:start + 1] = b"a"

    with pytest.raises(weight_archive.ArchiveError, match="not strictly sorted"):
        weight_archive.Archive(_corrupt(tmp_path, unsort))

    def wrong_length(data):
        first_name_length = struct.unpack_from("<I", data, 24)[0]
        length_at = 24 + 8 + first_name_length + 8 + 8
        data[length_at:length_at + 8] = struct.pack("<Q", 250)

    with pytest.raises(weight_archive.ArchiveError, match="byte length disagrees"):
        weight_archive.Archive(_corrupt(tmp_path, wrong_length))


@pytest.mark.gpu
def test_archive_tensors_feed_the_kernels(runtime, oracle):
    """Upload once, bind views: a W4A16 linear straight from the archive's buffer."""
    from llmopt_b200 import dispatch

    archive = weight_archive.Archive(GOLDEN)
    packed, scale = archive.view(runtime, "layers.0.gate.packed"), archive.view(runtime, "layers.0.gate.scale")
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2, 128)).astype(np.float16)
    from llmopt_b200.cuda_native import Buffer

    out = dispatch.Tensor(Buffer.create(runtime, 2 * 16 * 2), (2, 16))
    dispatch.dispatch_w4a16_linear(
        dispatch.Context(runtime), input=dispatch.Tensor(Buffer.of_array(runtime, x), (2, 128)),
        weight=dispatch.Tensor(packed, (16, 64), "uint8"), scale=dispatch.Tensor(scale, (16, 2)), output=out)
    expected = _expected()
    want = oracle.w4a16_linear(x, np.frombuffer(expected["layers.0.gate.packed"][2], np.uint8).reshape(16, 64),
                               np.frombuffer(expected["layers.0.gate.scale"][2], np.float16).reshape(16, 2))
    got = out.buffer.to_numpy(np.float16, (2, 16))
    assert np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) <= 2e-3 * np.max(np.abs(want.astype(np.float64)))
