"""Reader of the ``LLMOPTWT`` weight archive (ABI v1): binary index + 256-byte aligned payloads.

Mirrors ``Weight_archive`` (lib/weight_archive.ml:3-330) and the Python exporter's layout
(python/llmopt_backend/tensor_archive.py:19-118):

    prefix  "<8sHHIQ"  magic "LLMOPTWT", version 1, flags 0, tensor count, index bytes (= data start)
    entry   "<IBBH"    name length, dtype tag, rank, reserved 0; name (utf-8, strictly sorted);
                       rank x u64 dimensions; u64 payload offset; u64 payload byte length
    index padded with zeros to a multiple of 256; payloads in entry order, each at the next
    multiple of 256 after the previous one; nothing after the last payload.

``Archive.upload`` puts the whole file into one device buffer (``Buffer.map_file``); tensors are
views at their payload offsets, which keeps every view 256-byte aligned as the kernels expect."""

from __future__ import annotations

import os
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

MAGIC = b"LLMOPTWT"
VERSION = 1
ALIGNMENT = 256
_PREFIX = struct.Struct("<8sHHIQ")
_ENTRY = struct.Struct("<IBBH")

# Dtype.of_tag, lib/weight_archive.ml:67-87: name, bytes per element or (block elements, block bytes)
DTYPES = (
    ("F32", 4), ("F16", 2), ("BF16", 2), ("I64", 8), ("I32", 4), ("I8", 1), ("BOOL", 1), ("U8", 1),
    ("Q8_0", (32, 34)), ("Q4_K", (256, 144)), ("Q5_K", (256, 176)), ("Q6_K", (256, 210)), ("Q5_0", (32, 22)),
    ("Q4_0", (32, 18)), ("IQ4_XS", (256, 136)), ("Tile32_Affine4", (32, 20)), ("Tile32_Affine8", (32, 36)),
    ("EXL3_4", (256, 128)),
)


class ArchiveError(ValueError):
    """The reference reports these as ``Error "weight archive ..."`` strings."""


@dataclass(frozen=True)
class Tensor:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    offset: int
    byte_length: int


def _align(value: int) -> int:
    return (value + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT


def expected_bytes(dtype_tag: int, shape: Tuple[int, ...], name: str) -> int:
    elements = 1
    for dimension in shape:
        elements *= dimension
    width = DTYPES[dtype_tag][1]
    if isinstance(width, tuple):
        block, block_bytes = width
        if elements % block:
            raise ArchiveError(f"weight archive tensor {name} element count {elements} is not a multiple of quant "
                               f"block size {block}")
        return elements // block * block_bytes
    return elements * width


def parse(data: bytes, file_size: int) -> Tuple[int, Tuple[Tensor, ...]]:
    """(index bytes, tensors) from the first ``index_bytes`` of the file; raises ArchiveError."""
    if len(data) < _PREFIX.size:
        raise ArchiveError("weight archive is shorter than its prefix")
    magic, version, flags, count, index_bytes = _PREFIX.unpack_from(data, 0)
    if magic != MAGIC:
        raise ArchiveError("invalid weight-archive magic")
    if version != VERSION:
        raise ArchiveError(f"unsupported weight-archive version: {version}")
    if flags != 0:
        raise ArchiveError(f"unsupported weight-archive flags: {flags}")
    if count == 0:
        raise ArchiveError("weight archive contains no tensors")
    if index_bytes > len(data) or index_bytes % ALIGNMENT:
        raise ArchiveError("weight archive index length is inconsistent")
    cursor = _PREFIX.size
    tensors, previous = [], None
    for _ in range(count):
        if cursor + _ENTRY.size > index_bytes:
            raise ArchiveError("weight archive index is truncated")
        name_length, dtype_tag, rank, reserved = _ENTRY.unpack_from(data, cursor)
        cursor += _ENTRY.size
        if dtype_tag >= len(DTYPES):
            raise ArchiveError(f"unknown weight-archive dtype tag: {dtype_tag}")
        if cursor + name_length + 8 * rank + 16 > index_bytes:
            raise ArchiveError("weight archive index is truncated")
        raw_name = data[cursor:cursor + name_length]
        cursor += name_length
        if reserved != 0:
            raise ArchiveError("weight archive tensor reserved field is non-zero")
        if not raw_name:
            raise ArchiveError("weight archive tensor name cannot be empty")
        if b"\x00" in raw_name:
            raise ArchiveError("weight archive tensor name contains a NUL byte")
        if previous is not None and previous >= raw_name:  # String.compare: byte order
            raise ArchiveError("weight archive tensor names are not strictly sorted")
        previous = raw_name
        name = raw_name.decode("utf-8")
        shape = struct.unpack_from(f"<{rank}Q", data, cursor)
        cursor += 8 * rank
        offset, byte_length = struct.unpack_from("<QQ", data, cursor)
        cursor += 16
        elements = 1
        for dimension in shape:
            elements *= dimension
        if elements == 0 or byte_length == 0:
            raise ArchiveError(f"weight archive tensor {name} is empty")
        if byte_length != expected_bytes(dtype_tag, shape, name):
            raise ArchiveError(f"weight archive tensor {name} byte length disagrees with its dtype and shape")
        if offset % ALIGNMENT:
            raise ArchiveError(f"weight archive tensor {name} offset is not aligned")
        tensors.append(Tensor(name, DTYPES[dtype_tag][0], tuple(int(d) for d in shape), int(offset), int(byte_length)))
    if any(data[cursor:index_bytes]):
        raise ArchiveError("weight archive index padding contains non-zero bytes")
    position = index_bytes
    for tensor in tensors:
        position = _align(position)
        if tensor.offset != position:
            raise ArchiveError(f"weight archive tensor {tensor.name} has an unexpected payload offset")
        if position > file_size or tensor.byte_length > file_size - position:
            raise ArchiveError(f"weight archive tensor {tensor.name} exceeds the file")
        position += tensor.byte_length
    if position != file_size:
        raise ArchiveError("weight archive file has trailing or missing payload bytes")
    return int(index_bytes), tuple(tensors)


class Archive:
    """``Weight_archive.t``: the parsed index of one file."""

    def __init__(self, path: str):
        self.path = path
        self.file_size = os.path.getsize(path)
        with open(path, "rb") as source:
            prefix = source.read(_PREFIX.size)
            if len(prefix) < _PREFIX.size:
                raise ArchiveError("weight archive is shorter than its prefix")
            index_bytes = _PREFIX.unpack(prefix)[4]
            if prefix[:8] != MAGIC:
                raise ArchiveError("invalid weight-archive magic")
            if index_bytes > self.file_size:
                raise ArchiveError("weight archive index exceeds the file")
            source.seek(0)
            data = source.read(index_bytes)
        self.index_bytes, self.tensors = parse(data, self.file_size)
        self.index: Dict[str, Tensor] = {tensor.name: tensor for tensor in self.tensors}
        self._buffer = None

    def find(self, name: str):
        return self.index.get(name)

    def read(self, name: str) -> bytes:
        """Payload bytes of one tensor, from the file."""
        tensor = self.index[name]
        with open(self.path, "rb") as source:
            source.seek(tensor.offset)
            return source.read(tensor.byte_length)

    def upload(self, runtime):
        """The whole archive as one device buffer (``Metal_native.Buffer.map_file``)."""
        from .cuda_native import Buffer

        if self._buffer is None:
            self._buffer = Buffer.map_file(runtime, self.path)
        return self._buffer

    def view(self, runtime, name: str):
        """Device view of one tensor's payload (shares the archive's buffer, 256-byte aligned)."""
        tensor = self.index[name]
        return self.upload(runtime).view(tensor.offset, tensor.byte_length)
