"""Reader (and writer, for fixtures) of the reference's ``package.llmopt`` envelope
(lib/serving_package.ml:303-373): magic ``LLMOPTPK``, ABI version, stage, target, model name, the
kernel-library artifact, the declared kernel entry points (``Kernel_abi.Entry``: name, operation
tag, dtype tags, threadgroup), the tensor-store artifact, the radix-cache page size, then two
length-prefixed blobs — the serving schedule and its memory plan.

What this gives the CUDA layer is the reference's package validation: every kernel a compiled
package declares must resolve in the loaded library (``validate_declared_functions``,
lib/metal_native.ml:271-277), with the operation and dtypes the entry states.  The schedule and
memory-plan blobs are carried opaquely: decoding the schedule's op encoding
(lib/serving_schedule_codec.ml) is not part of this layer — the OCaml engine does that and hands the
native layer plain dispatches.

All integers are little endian; a string is u32 length + bytes, a blob is u64 length + bytes, an
option is a u8 tag (0 none, 1 some) followed by the value (lib/binary.ml)."""

from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Optional

from . import kernel_abi

MAGIC = b"LLMOPTPK"
CURRENT_ABI_VERSION = 27  # lib/serving_package.ml:76
STAGES = ("compiled-graph", "serving")

# lib/serving_package.ml:150-183 (operation tags) and :222-240 (dtype tags); only wire names this layer knows
OPERATION_TAGS = {
    0: "matmul", 1: kernel_abi.FUSED_LINEAR, 2: kernel_abi.LINEAR, 5: kernel_abi.RMS_NORM, 6: kernel_abi.SHORT_CONV,
    7: kernel_abi.ATTENTION, 8: kernel_abi.EMBEDDING, 9: "arange", 10: "diff", 11: "cumsum", 12: "fill", 13: "gather2",
    14: kernel_abi.CAST, 15: kernel_abi.POINTWISE, 16: "movement", 17: "reduction", 18: "update-slice",
    19: kernel_abi.CACHE, 23: kernel_abi.RMS_ROPE, 24: kernel_abi.SHORT_CONV_STEP, 25: kernel_abi.SHORT_CONV_PREFILL,
    26: kernel_abi.W4A16_LM_HEAD_ARGMAX, 27: kernel_abi.W4A16_LINEAR, 28: kernel_abi.W4A16_SWIGLU_FFN,
    29: kernel_abi.W4A16_QKV_LINEAR, 30: kernel_abi.RMS_ROPE_QK, 31: kernel_abi.TRIANGULAR_RECURRENCE, 32: "eye",
    33: "batched-matmul", 34: kernel_abi.GATED_DELTA, 35: kernel_abi.GATED_LINEAR, 36: kernel_abi.ROTARY_QK,
    37: "moe-swiglu-ffn",
}
DTYPE_TAGS = {0: "float32", 1: "float16", 2: "bfloat16", 3: "int64", 4: "int32", 5: "int8", 6: "bool", 7: "uint8",
              8: "q8_0", 9: "q4_k", 10: "q5_k", 11: "q6_k", 12: "q5_0", 13: "q4_0", 14: "iq4_xs", 15: "tile32_affine4",
              16: "tile32_affine8", 17: "exl3_4"}
_OPERATION_OF = {name: tag for tag, name in OPERATION_TAGS.items()}
_DTYPE_OF = {name: tag for tag, name in DTYPE_TAGS.items()}


class PackageError(ValueError):
    """An ``Error msg`` of the reference's reader (same messages)."""


def _artifact(path: str) -> str:
    """``Artifact.create`` (lib/serving_package.ml:14-28): a canonical relative path."""
    path = path.strip()
    if path == "":
        raise PackageError("serving-package artifact path cannot be empty")
    if path.startswith("/"):
        raise PackageError("serving-package artifact path must be relative: " + path)
    if "\0" in path:
        raise PackageError("serving-package artifact path contains a NUL byte")
    if any(component in ("", ".", "..") for component in path.split("/")):
        raise PackageError("serving-package artifact path is not canonical: " + path)
    return path


@dataclass
class Package:
    stage: str
    kernel_library: str
    kernels: List[kernel_abi.Entry]
    schedule: bytes = b""
    memory_plan: bytes = b""
    model: Optional[str] = None
    tensor_store: Optional[str] = None
    page_size: int = 1
    abi_version: int = CURRENT_ABI_VERSION

    def validate(self) -> None:
        """The envelope-level rules of ``Serving_package.validate`` (lib/serving_package.ml:78-96);
        the rule about tensor-store inputs of the schedule needs the decoded schedule and is the
        engine's."""
        names = [entry.name for entry in self.kernels]
        if self.model is not None and self.model.strip() == "":
            raise PackageError("serving-package model identifier cannot be empty")
        if not self.kernels:
            raise PackageError("serving-package must declare at least one kernel")
        if len(names) != len(set(names)):
            raise PackageError("serving-package kernel entry-point names must be unique")
        if self.stage == "compiled-graph" and self.tensor_store is not None:
            raise PackageError("compiled-graph package cannot declare a tensor store")
        if self.stage == "serving" and self.tensor_store is None:
            raise PackageError("serving-stage package must declare a tensor store")
        if self.page_size <= 0:
            raise PackageError("serving-package radix page_size must be positive")

    def validate_declared_functions(self, runtime) -> None:
        """``validate_declared_functions`` + ``preload_declared_pipelines``
        (lib/metal_native.ml:271-285): every declared kernel resolves in the library."""
        for entry in self.kernels:
            if not runtime.has_function(entry.name):
                raise PackageError("CUDA library does not define declared kernel: " + entry.name)
            runtime.preload_pipeline(entry.name)

    def to_bytes(self) -> bytes:
        out = bytearray(MAGIC)
        out += struct.pack("<HBB", self.abi_version, STAGES.index(self.stage), 0)
        _write_option(out, self.model, _write_string)
        _write_string(out, self.kernel_library)
        out += struct.pack("<H", len(self.kernels))
        for entry in self.kernels:
            _write_string(out, entry.name)
            out += struct.pack("<BBB3I", _OPERATION_OF[entry.operation], _DTYPE_OF[entry.input_dtype],
                               _DTYPE_OF[entry.output_dtype], *entry.threadgroup)
        _write_option(out, self.tensor_store, lambda buffer, path: (buffer.append(0), _write_string(buffer, path)))
        out += struct.pack("<I", self.page_size)
        for blob in (self.schedule, self.memory_plan):
            out += struct.pack("<Q", len(blob)) + blob
        return bytes(out)


def _write_string(out: bytearray, value: str) -> None:
    data = value.encode()
    out += struct.pack("<I", len(data)) + data


def _write_option(out: bytearray, value, write) -> None:
    if value is None:
        out.append(0)
    else:
        out.append(1)
        write(out, value)


class _Reader:
    def __init__(self, data: bytes):
        self.data, self.offset = bytes(data), 0

    def take(self, length: int) -> bytes:
        remaining = len(self.data) - self.offset
        if length > remaining:
            raise PackageError(f"truncated binary input at byte {self.offset}: need {length} bytes, have {remaining}")
        value = self.data[self.offset:self.offset + length]
        self.offset += length
        return value

    def unpack(self, layout: str):
        values = struct.unpack("<" + layout, self.take(struct.calcsize("<" + layout)))
        return values[0] if len(values) == 1 else values

    def string(self) -> str:
        return self.take(self.unpack("I")).decode()

    def blob(self) -> bytes:
        return self.take(self.unpack("Q"))

    def option(self, read):
        tag = self.unpack("B")
        if tag == 0:
            return None
        if tag == 1:
            return read()
        raise PackageError(f"unknown serving-package option tag: {tag}")


def of_bytes(data: bytes) -> Package:
    """``Serving_package.of_bytes`` (lib/serving_package.ml:325-373) up to the two blobs."""
    reader = _Reader(data)
    if reader.take(len(MAGIC)) != MAGIC:
        raise PackageError("invalid serving-package magic")
    version = reader.unpack("H")
    if version != CURRENT_ABI_VERSION:
        raise PackageError(f"unsupported serving-package version: {version}")
    stage_tag = reader.unpack("B")
    if stage_tag >= len(STAGES):
        raise PackageError(f"unknown serving-package stage tag: {stage_tag}")
    target = reader.unpack("B")
    if target != 0:
        raise PackageError(f"unsupported serving-package target tag: {target}")
    model = reader.option(reader.string)
    library = _artifact(reader.string())
    kernels = []
    for _ in range(reader.unpack("H")):
        name = reader.string()
        operation_tag, input_tag, output_tag, x, y, z = reader.unpack("BBB3I")
        if operation_tag not in OPERATION_TAGS:
            raise PackageError(f"unknown kernel operation tag: {operation_tag}")
        for tag in (input_tag, output_tag):
            if tag not in DTYPE_TAGS:
                raise PackageError(f"unknown kernel dtype tag: {tag}")
        kernels.append(kernel_abi.Entry(name, OPERATION_TAGS[operation_tag], DTYPE_TAGS[input_tag], DTYPE_TAGS[output_tag],
                                        (x, y, z)))

    def tensor_store():
        tag = reader.unpack("B")
        if tag != 0:
            raise PackageError(f"unknown tensor-store tag: {tag}")
        return _artifact(reader.string())

    store = reader.option(tensor_store)
    page_size = reader.unpack("I")
    schedule, memory_plan = reader.blob(), reader.blob()
    if reader.offset != len(reader.data):
        raise PackageError(f"trailing binary input: {len(reader.data) - reader.offset} bytes")
    package = Package(STAGES[stage_tag], library, kernels, schedule, memory_plan, model, store, page_size, version)
    package.validate()
    return package


def of_file(path: str) -> Package:
    with open(path, "rb") as handle:
        return of_bytes(handle.read())
