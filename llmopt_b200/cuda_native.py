"""Host-side mirror of the reference's ``Metal_native`` module over libllmopt_cuda.so.

The reference binds its native layer from OCaml (lib/metal_native.ml:8-124,
signature lib/metal_native.mli:1-142).  An OCaml toolchain is not part of this
build, so the same surface is bound here with ctypes: ``Runtime`` (context +
library), ``Buffer``, ``Batch``, ``Prebaked``, ``RingQueue``, ``kernel_entry``
and ``dispatch`` keep the reference's names, argument meaning and error
behaviour — a native failure surfaces as ``NativeError`` (the reference's
``Error msg`` result), an argument problem as ``ValueError``
(``Invalid_argument``).

There is no CPU fallback: importing works anywhere, but creating a ``Runtime``
needs the compiled library and a B200; otherwise it raises.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

from . import kernel_abi

_LIBRARY_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libllmopt_cuda.so")
_lib: Optional[ctypes.CDLL] = None


class NativeError(RuntimeError):
    """A failure reported by the native layer (reference: ``Failure msg``)."""


class _Record(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char_p),
        ("buffers", ctypes.POINTER(ctypes.c_void_p)),
        ("buffer_count", ctypes.c_int),
        ("parameters", ctypes.c_void_p),
        ("parameter_bytes", ctypes.c_size_t),
        ("grid", ctypes.c_int * 3),
        ("group", ctypes.c_int * 3),
        ("barrier_before", ctypes.c_int),
    ]


class _RowBinding(ctypes.Structure):
    _fields_ = [("destination", ctypes.c_void_p), ("table", ctypes.c_void_p), ("row_bytes", ctypes.c_size_t)]


# name -> (restype, argtypes); every symbol include/llmopt_cuda.h declares
_P = ctypes.c_void_p
_PP = ctypes.POINTER(ctypes.c_void_p)
_I = ctypes.c_int
_I32 = ctypes.c_int32
_I64 = ctypes.c_int64
_SZ = ctypes.c_size_t
_REC = ctypes.POINTER(_Record)
SIGNATURES = {
    "llmopt_cuda_last_error": (ctypes.c_char_p, []),
    "llmopt_cuda_create_context": (_I, [_I, _PP]),
    "llmopt_cuda_release_context": (None, [_P]),
    "llmopt_cuda_device_name": (ctypes.c_char_p, [_P]),
    "llmopt_cuda_load_library": (_I, [_P, ctypes.c_char_p, _PP]),
    "llmopt_cuda_release_library": (None, [_P]),
    "llmopt_cuda_has_function": (_I, [_P, ctypes.c_char_p]),
    "llmopt_cuda_preload_pipeline": (_I, [_P, ctypes.c_char_p]),
    "llmopt_cuda_function_count": (_I, [_P]),
    "llmopt_cuda_function_name": (ctypes.c_char_p, [_P, _I]),
    "llmopt_cuda_register_alias": (_I, [_P, ctypes.c_char_p, ctypes.c_char_p]),
    "llmopt_cuda_register_expr_epilogue": (_I, [_P, ctypes.c_char_p, _P, _SZ, _I]),
    "llmopt_cuda_buffer_of_bytes": (_I, [_P, _P, _SZ, _PP]),
    "llmopt_cuda_create_buffer": (_I, [_P, _I64, _PP]),
    "llmopt_cuda_map_file": (_I, [_P, ctypes.c_char_p, _PP]),
    "llmopt_cuda_buffer_view": (_I, [_P, _I64, _I64, _PP]),
    "llmopt_cuda_release_buffer": (None, [_P]),
    "llmopt_cuda_buffer_export": (_I, [_P, _P, ctypes.POINTER(ctypes.c_uint64)]),
    "llmopt_cuda_buffer_import": (_I, [_P, _P, ctypes.c_uint64, ctypes.c_uint64, _PP]),
    "llmopt_cuda_buffer_length": (_SZ, [_P]),
    "llmopt_cuda_buffer_contents": (_I, [_P, _P, _SZ]),
    "llmopt_cuda_buffer_argmax_f16": (_I, [_P, _I64, ctypes.POINTER(_I64)]),
    "llmopt_cuda_buffer_copy": (_I, [_P, _P]),
    "llmopt_cuda_buffer_set_int64": (_I, [_P, _I64, _I64]),
    "llmopt_cuda_buffer_set_u32_array": (_I, [_P, _I64, _P, _SZ]),
    "llmopt_cuda_buffer_write": (_I, [_P, _I64, _P, _SZ]),
    "llmopt_cuda_buffer_device_pointer": (_P, [_P]),
    "llmopt_cuda_dispatch": (_I, [_P, _REC]),
    "llmopt_cuda_begin_batch": (_I, [_P, _PP]),
    "llmopt_cuda_batch_dispatch": (_I, [_P, _P, _REC]),
    "llmopt_cuda_batch_dispatch_all": (_I, [_P, _P, _REC, _SZ]),
    "llmopt_cuda_batch_copy": (_I, [_P, _P, _P]),
    "llmopt_cuda_batch_barrier": (_I, [_P]),
    "llmopt_cuda_commit_batch": (_I, [_P]),
    "llmopt_cuda_commit_batch_async": (_I, [_P]),
    "llmopt_cuda_abort_batch": (_I, [_P]),
    "llmopt_cuda_release_batch": (None, [_P]),
    "llmopt_cuda_synchronize": (_I, [_P]),
    "llmopt_cuda_prebaked_create": (_I, [_P, _REC, _SZ, _P, _P, _PP]),
    "llmopt_cuda_prebaked_create_bound": (_I, [_P, _REC, _SZ, _P, _P, ctypes.POINTER(_RowBinding), _SZ, _PP]),
    "llmopt_cuda_prebaked_execute": (_I, [_P, _I64, _I32, _I32, ctypes.POINTER(_I32)]),
    "llmopt_cuda_prebaked_execute_chained": (
        _I, [_P, _I64, _I32, _I32, _I32, ctypes.POINTER(_I32), ctypes.POINTER(ctypes.c_float)]),
    "llmopt_cuda_prebaked_kernel_count": (_I, [_P]),
    "llmopt_cuda_prebaked_token_capacity": (_I64, [_P]),
    "llmopt_cuda_release_prebaked": (None, [_P]),
    "llmopt_cuda_ring_create": (_I, [_PP]),
    "llmopt_cuda_ring_start_worker": (_I, [_P, _P, _REC, _SZ, _P, _P]),
    "llmopt_cuda_ring_submit": (_I, [_P, _I64, _I64, _I32, _I32, ctypes.POINTER(_I)]),
    "llmopt_cuda_ring_wait_completion": (_I, [_P, ctypes.POINTER(_I64), ctypes.POINTER(_I32), ctypes.POINTER(_I32)]),
    "llmopt_cuda_ring_poll_completion": (
        _I, [_P, ctypes.POINTER(_I), ctypes.POINTER(_I64), ctypes.POINTER(_I32), ctypes.POINTER(_I32)]),
    "llmopt_cuda_ring_destroy": (_I, [_P]),
    "llmopt_cuda_f16_argmax": (_I64, [_P, _SZ]),
    "llmopt_cuda_sample_f16": (_I, [_P, _SZ, ctypes.c_double, _I, ctypes.c_double, ctypes.c_double, ctypes.c_uint64,
                                   ctypes.POINTER(_I64)]),
    "llmopt_cuda_measure_hardware": (_I, [_I, _I, _I, _I64, ctypes.c_char_p, _SZ, ctypes.POINTER(_I),
                                         ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]),
    "llmopt_cuda_w4a16_linear": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "llmopt_cuda_attention_q8_paged_static": (_I, [_P, _P, _P, _P, _P, _P, _P, _SZ, ctypes.c_uint32, _P]),
    "llmopt_cuda_time_dispatch": (_I, [_P, _REC, _I, _I, _I, ctypes.POINTER(ctypes.c_float)]),
    "llmopt_cuda_time_dispatches": (_I, [_P, _REC, _SZ, _I, _I, ctypes.POINTER(ctypes.c_float)]),
}


def library_path() -> str:
    return _LIBRARY_PATH


def load_library() -> ctypes.CDLL:
    """Loads libllmopt_cuda.so and types every entry point. Raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIBRARY_PATH):
            raise NativeError(
                f"{_LIBRARY_PATH} is missing: build it with `python -m llmopt_b200._build` (nvcc, sm_100a)"
            )
        lib = ctypes.CDLL(_LIBRARY_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(lib, name)
            function.restype = restype
            function.argtypes = argtypes
        _lib = lib
    return _lib


def _check(status: int) -> None:
    if status == 0:
        return
    message = load_library().llmopt_cuda_last_error().decode("utf-8", "replace")
    if status == 2:
        raise ValueError(message)
    raise NativeError(message)


class Buffer:
    """``Metal_native.Buffer`` (lib/metal_native.mli:26-38): a device allocation or a view."""

    def __init__(self, handle: int, runtime: "Runtime"):
        self._handle = ctypes.c_void_p(handle)
        self._runtime = runtime  # keeps the context alive

    @classmethod
    def of_bytes(cls, runtime: "Runtime", data) -> "Buffer":
        data = bytes(data) if not isinstance(data, (bytes, bytearray)) else data
        out = ctypes.c_void_p()
        source = (ctypes.c_char * len(data)).from_buffer_copy(data) if len(data) else None
        _check(load_library().llmopt_cuda_buffer_of_bytes(runtime._context, source, len(data), ctypes.byref(out)))
        return cls(out.value, runtime)

    @classmethod
    def of_array(cls, runtime: "Runtime", array) -> "Buffer":
        """Uploads a contiguous numpy array without an intermediate bytes copy."""
        import numpy as np

        array = np.ascontiguousarray(array)
        out = ctypes.c_void_p()
        _check(load_library().llmopt_cuda_buffer_of_bytes(
            runtime._context, array.ctypes.data_as(ctypes.c_void_p), array.nbytes, ctypes.byref(out)))
        return cls(out.value, runtime)

    @classmethod
    def create(cls, runtime: "Runtime", nbytes: int) -> "Buffer":
        out = ctypes.c_void_p()
        _check(load_library().llmopt_cuda_create_buffer(runtime._context, int(nbytes), ctypes.byref(out)))
        return cls(out.value, runtime)

    @classmethod
    def map_file(cls, runtime: "Runtime", path: str) -> "Buffer":
        out = ctypes.c_void_p()
        _check(load_library().llmopt_cuda_map_file(runtime._context, os.fsencode(path), ctypes.byref(out)))
        return cls(out.value, runtime)

    def view(self, offset: int, nbytes: int) -> "Buffer":
        out = ctypes.c_void_p()
        _check(load_library().llmopt_cuda_buffer_view(self._handle, int(offset), int(nbytes), ctypes.byref(out)))
        return Buffer(out.value, self._runtime)

    def export_handle(self) -> tuple:
        """(opaque 64 bytes, offset, length): what a peer process needs to map this buffer."""
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_uint64()
        _check(load_library().llmopt_cuda_buffer_export(self._handle, handle, ctypes.byref(offset)))
        return handle.raw, int(offset.value), self.byte_length()

    @classmethod
    def import_handle(cls, runtime: "Runtime", exported: tuple) -> "Buffer":
        """Maps a buffer another process exported with ``export_handle``."""
        handle, offset, length = exported
        out = ctypes.c_void_p()
        _check(load_library().llmopt_cuda_buffer_import(
            runtime._context, ctypes.create_string_buffer(bytes(handle), 64), int(offset), int(length), ctypes.byref(out)))
        return cls(out.value, runtime)

    def byte_length(self) -> int:
        return int(load_library().llmopt_cuda_buffer_length(self._handle))

    def contents(self) -> bytes:
        length = self.byte_length()
        destination = ctypes.create_string_buffer(length)
        _check(load_library().llmopt_cuda_buffer_contents(self._handle, destination, length))
        return destination.raw

    def to_numpy(self, dtype, shape=None):
        import numpy as np

        array = np.empty(self.byte_length() // np.dtype(dtype).itemsize, dtype=dtype)
        _check(load_library().llmopt_cuda_buffer_contents(
            self._handle, array.ctypes.data_as(ctypes.c_void_p), array.nbytes))
        return array if shape is None else array.reshape(shape)

    def argmax_f16(self, vocabulary: int) -> int:
        out = ctypes.c_int64()
        _check(load_library().llmopt_cuda_buffer_argmax_f16(self._handle, int(vocabulary), ctypes.byref(out)))
        return int(out.value)

    def copy_to(self, destination: "Buffer") -> None:
        _check(load_library().llmopt_cuda_buffer_copy(self._handle, destination._handle))

    def set_int64(self, offset: int, value: int) -> None:
        _check(load_library().llmopt_cuda_buffer_set_int64(self._handle, int(offset), int(value)))

    def set_u32_array(self, offset: int, values: Sequence[int]) -> None:
        array = (ctypes.c_uint32 * len(values))(*values)
        _check(load_library().llmopt_cuda_buffer_set_u32_array(self._handle, int(offset), array, len(values)))

    def write(self, offset: int, data) -> None:
        import numpy as np

        array = np.ascontiguousarray(data) if not isinstance(data, (bytes, bytearray)) else np.frombuffer(data, np.uint8)
        _check(load_library().llmopt_cuda_buffer_write(
            self._handle, int(offset), array.ctypes.data_as(ctypes.c_void_p), array.nbytes))

    def device_pointer(self) -> int:
        return int(load_library().llmopt_cuda_buffer_device_pointer(self._handle) or 0)

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and _lib is not None:
            _lib.llmopt_cuda_release_buffer(handle)


@dataclass
class DispatchItem:
    """``Metal_native.Batch.dispatch_item`` (lib/metal_native.mli:40-51)."""

    name: str
    buffers: Sequence[Buffer]
    parameters: bytes
    grid: tuple = (1, 1, 1)
    group: tuple = (1, 1, 1)
    barrier_before: bool = False


class _RecordArray:
    """Packs DispatchItems into a C array and keeps every referenced object alive."""

    def __init__(self, items: Sequence[DispatchItem]):
        self.items = list(items)
        self.array = (_Record * max(len(self.items), 1))()
        self._keep = []
        for record, item in zip(self.array, self.items):
            name = item.name.encode()
            handles = (ctypes.c_void_p * max(len(item.buffers), 1))(*[b._handle for b in item.buffers])
            params = ctypes.create_string_buffer(bytes(item.parameters), max(len(item.parameters), 1))
            self._keep.extend([name, handles, params])
            record.name = name
            record.buffers = ctypes.cast(handles, ctypes.POINTER(ctypes.c_void_p))
            record.buffer_count = len(item.buffers)
            record.parameters = ctypes.cast(params, ctypes.c_void_p)
            record.parameter_bytes = len(item.parameters)
            if any(int(v) > 0x7FFFFFFF for v in tuple(item.grid) + tuple(item.group)):
                raise ValueError(f"{item.name}: grid dimension overflows the 32-bit record field")
            record.grid = (ctypes.c_int * 3)(*[int(v) for v in item.grid])
            record.group = (ctypes.c_int * 3)(*[int(v) for v in item.group])
            record.barrier_before = int(item.barrier_before)

    def __len__(self):
        return len(self.items)


def pack_records(items: Sequence[DispatchItem]) -> _RecordArray:
    """The C array of a dispatch list, for ``Batch.dispatch_recorded``; it keeps the list's buffers alive."""
    return _RecordArray(items)


class Runtime:
    """``Metal_native.t``: one context + the kernel library (lib/metal_native.mli:10-17)."""

    def __init__(self, device: int = -1):
        lib = load_library()
        self._context = ctypes.c_void_p()
        self._library = ctypes.c_void_p()
        _check(lib.llmopt_cuda_create_context(int(device), ctypes.byref(self._context)))
        _check(lib.llmopt_cuda_load_library(self._context, b"", ctypes.byref(self._library)))

    def device_name(self) -> str:
        return load_library().llmopt_cuda_device_name(self._context).decode()

    def has_function(self, name: str) -> bool:
        return bool(load_library().llmopt_cuda_has_function(self._library, name.encode()))

    def preload_pipeline(self, name: str) -> None:
        _check(load_library().llmopt_cuda_preload_pipeline(self._library, name.encode()))

    def function_names(self) -> list[str]:
        lib = load_library()
        return [lib.llmopt_cuda_function_name(self._library, i).decode()
                for i in range(lib.llmopt_cuda_function_count(self._library))]

    def register_alias(self, alias: str, target: str) -> None:
        _check(load_library().llmopt_cuda_register_alias(self._library, alias.encode(), target.encode()))

    def register_expr_epilogue(self, name: str, program: bytes, operand_count: int) -> None:
        """Registers a digest-named W4A16 linear with an expression epilogue (``epilogue.bind``)."""
        code = ctypes.create_string_buffer(bytes(program), max(len(program), 1))
        _check(load_library().llmopt_cuda_register_expr_epilogue(
            self._library, name.encode(), code, len(program), int(operand_count)))

    def synchronize(self) -> None:
        _check(load_library().llmopt_cuda_synchronize(self._context))

    def kernel_entry(self, *, operation: str, input_dtype: str, output_dtype: str,
                     name: Optional[str] = None) -> kernel_abi.Entry:
        """``Metal_native.kernel_entry`` (lib/metal_native.ml:461-487): exactly one
        entry must match (name, operation, dtypes), and its function must exist."""
        entry = kernel_abi.find_entry(operation=operation, input_dtype=input_dtype,
                                      output_dtype=output_dtype, name=name)
        if not self.has_function(entry.name):
            raise NativeError(f"CUDA kernel function is missing: {entry.name}")
        return entry

    def dispatch(self, entry, *, buffers: Sequence[Buffer], parameters: bytes, grid=(1, 1, 1),
                 batch: Optional["Batch"] = None) -> str:
        """``Metal_native.dispatch`` (lib/metal_native.ml:489-512): immediate (waits)
        or appended to ``batch``. Returns the kernel name."""
        name = entry.name if isinstance(entry, kernel_abi.Entry) else str(entry)
        group = entry.threadgroup if isinstance(entry, kernel_abi.Entry) else (256, 1, 1)
        item = DispatchItem(name, list(buffers), bytes(parameters), tuple(grid), tuple(group))
        if batch is not None:
            batch.dispatch_item(item)
        else:
            records = _RecordArray([item])
            _check(load_library().llmopt_cuda_dispatch(self._library, records.array))
        return name

    def time_dispatch(self, item: DispatchItem, *, warmup: int = 3, iterations: int = 20,
                      flush_l2: bool = True) -> float:
        """Average device milliseconds of one dispatch (CUDA events on the context stream)."""
        records = _RecordArray([item])
        out = ctypes.c_float()
        _check(load_library().llmopt_cuda_time_dispatch(
            self._library, records.array, warmup, iterations, int(flush_l2), ctypes.byref(out)))
        return float(out.value)

    def time_dispatches(self, items: Sequence[DispatchItem], *, warmup: int = 2, iterations: int = 5) -> float:
        """Average device milliseconds per dispatch of a list run back to back (one
        pair of CUDA events around the list)."""
        records = _RecordArray(items)
        out = ctypes.c_float()
        _check(load_library().llmopt_cuda_time_dispatches(
            self._library, records.array, len(records), warmup, iterations, ctypes.byref(out)))
        return float(out.value)

    def w4a16_linear_pointers(self, x_ptr: int, packed_ptr: int, scale_ptr: int, bias_ptr: Optional[int],
                              out_ptr: int, m: int, n: int, k: int, stream: int = 0) -> None:
        """The Python single-op boundary (native/metal_runtime.cpp:58-136) on raw device pointers."""
        _check(load_library().llmopt_cuda_w4a16_linear(
            self._context, x_ptr, packed_ptr, scale_ptr, bias_ptr or None, out_ptr, m, n, k, stream or None))

    def __del__(self):
        lib = _lib
        if lib is None:
            return
        library, self._library = getattr(self, "_library", None), None
        context, self._context = getattr(self, "_context", None), None
        if library:
            lib.llmopt_cuda_release_library(library)
        if context:
            lib.llmopt_cuda_release_context(context)


class Batch:
    """``Metal_native.Batch`` (lib/metal_native.mli:40-80): dispatches are kept in
    ``pending`` on the host and pushed to the native batch by ``flush``."""

    def __init__(self, runtime: Runtime):
        self.runtime = runtime
        self.pending: list[DispatchItem] = []
        self.next_dispatch_barrier = False
        self._handle = ctypes.c_void_p()
        self._keep = []
        _check(load_library().llmopt_cuda_begin_batch(runtime._library, ctypes.byref(self._handle)))

    def dispatch_item(self, item: DispatchItem) -> None:
        item.barrier_before = self.next_dispatch_barrier
        self.next_dispatch_barrier = False
        self.pending.append(item)

    def dispatch(self, *, name: str, buffers: Sequence[Buffer], parameters: bytes, grid, group) -> None:
        self.dispatch_item(DispatchItem(name, list(buffers), bytes(parameters), tuple(grid), tuple(group)))

    def mark_barrier(self) -> None:
        self.next_dispatch_barrier = True

    def flush(self) -> None:
        if not self.pending:
            return
        records = _RecordArray(self.pending)
        self._keep.append(records)
        self.pending = []
        _check(load_library().llmopt_cuda_batch_dispatch_all(
            self._handle, self.runtime._library, records.array, len(records)))

    def dispatch_recorded(self, records: "_RecordArray") -> None:
        """Appends a list packed earlier with ``pack_records`` (a dispatch list recorded once and
        replayed, e.g. the prompt pass of a known length): no per-dispatch host work."""
        self.flush()
        self._keep.append(records)
        _check(load_library().llmopt_cuda_batch_dispatch_all(
            self._handle, self.runtime._library, records.array, len(records)))

    def copy(self, *, source: Buffer, destination: Buffer) -> None:
        self.flush()
        _check(load_library().llmopt_cuda_batch_copy(self._handle, source._handle, destination._handle))

    def barrier(self) -> None:
        self.flush()
        _check(load_library().llmopt_cuda_batch_barrier(self._handle))

    def commit(self) -> None:
        self.flush()
        _check(load_library().llmopt_cuda_commit_batch(self._handle))

    def commit_async(self) -> None:
        self.flush()
        _check(load_library().llmopt_cuda_commit_batch_async(self._handle))

    def abort(self) -> None:
        self.pending = []
        _check(load_library().llmopt_cuda_abort_batch(self._handle))

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and _lib is not None:
            _lib.llmopt_cuda_release_batch(handle)


class Prebaked:
    """``Metal_native.Prebaked`` (lib/metal_native.mli:128-142): a recorded per-token
    dispatch list replayed as one CUDA graph."""

    def __init__(self, runtime: Runtime, dispatches: Sequence[DispatchItem], token_buffer: Optional[Buffer],
                 output_buffer: Optional[Buffer], row_bindings: Iterable[tuple] = ()):
        self.runtime = runtime
        self._records = _RecordArray(dispatches)
        self._buffers = (token_buffer, output_buffer)
        bindings = list(row_bindings)
        self._bindings = bindings
        array = (_RowBinding * max(len(bindings), 1))()
        for slot, (destination, table, row_bytes) in zip(array, bindings):
            slot.destination = destination._handle
            slot.table = table._handle
            slot.row_bytes = int(row_bytes)
        self._handle = ctypes.c_void_p()
        _check(load_library().llmopt_cuda_prebaked_create_bound(
            runtime._library, self._records.array, len(self._records),
            token_buffer._handle if token_buffer else None, output_buffer._handle if output_buffer else None,
            array, len(bindings), ctypes.byref(self._handle)))

    def execute(self, *, token: int, past_tokens: int, checkpoint: int = 0) -> int:
        out = ctypes.c_int32()
        _check(load_library().llmopt_cuda_prebaked_execute(
            self._handle, int(token), int(past_tokens), int(checkpoint), ctypes.byref(out)))
        return int(out.value)

    def execute_chained(self, *, token: int, past_tokens: int, steps: int, checkpoint: int = 0):
        """Returns (token ids, device milliseconds) of ``steps`` chained replays."""
        tokens = (ctypes.c_int32 * steps)()
        elapsed = ctypes.c_float()
        _check(load_library().llmopt_cuda_prebaked_execute_chained(
            self._handle, int(token), int(past_tokens), int(checkpoint), int(steps), tokens, ctypes.byref(elapsed)))
        return list(tokens), float(elapsed.value)

    def kernel_count(self) -> int:
        return int(load_library().llmopt_cuda_prebaked_kernel_count(self._handle))

    def token_capacity(self) -> int:
        """Largest ``past_tokens`` a replay accepts (bounded by the row-binding tables and the
        paged-attention slot tables the plan captured)."""
        return int(load_library().llmopt_cuda_prebaked_token_capacity(self._handle))

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and _lib is not None:
            _lib.llmopt_cuda_release_prebaked(handle)


class RingQueue:
    """``Metal_native.Ring_queue`` (lib/metal_native.mli:100-126)."""

    default_pipeline_depth = 2

    def __init__(self):
        self._handle = ctypes.c_void_p()
        self._keep = None
        _check(load_library().llmopt_cuda_ring_create(ctypes.byref(self._handle)))

    def start_worker(self, runtime: Runtime, dispatches: Sequence[DispatchItem], token_buffer: Buffer,
                     output_buffer: Buffer) -> None:
        records = _RecordArray(dispatches)
        self._keep = (records, token_buffer, output_buffer, runtime)
        _check(load_library().llmopt_cuda_ring_start_worker(
            self._handle, runtime._library, records.array, len(records), token_buffer._handle,
            output_buffer._handle))

    def submit(self, *, request_id: int, token: int, past_tokens: int, flags: int = 0) -> bool:
        accepted = ctypes.c_int()
        _check(load_library().llmopt_cuda_ring_submit(
            self._handle, request_id, token, past_tokens, flags, ctypes.byref(accepted)))
        return bool(accepted.value)

    def wait_completion(self) -> tuple:
        request, token, status = ctypes.c_int64(), ctypes.c_int32(), ctypes.c_int32()
        _check(load_library().llmopt_cuda_ring_wait_completion(
            self._handle, ctypes.byref(request), ctypes.byref(token), ctypes.byref(status)))
        return int(request.value), int(token.value), int(status.value)

    def poll_completion(self) -> Optional[tuple]:
        available = ctypes.c_int()
        request, token, status = ctypes.c_int64(), ctypes.c_int32(), ctypes.c_int32()
        _check(load_library().llmopt_cuda_ring_poll_completion(
            self._handle, ctypes.byref(available), ctypes.byref(request), ctypes.byref(token),
            ctypes.byref(status)))
        return (int(request.value), int(token.value), int(status.value)) if available.value else None

    def destroy(self) -> None:
        handle, self._handle = self._handle, None
        if handle and _lib is not None:
            _check(_lib.llmopt_cuda_ring_destroy(handle))

    def __del__(self):
        if getattr(self, "_handle", None):
            self.destroy()


def f16_argmax(data: bytes, count: int) -> int:
    """``caml_llmopt_f16_argmax``: first maximum of ``count`` halves held on the host."""
    buffer = ctypes.create_string_buffer(bytes(data), max(len(data), 1))
    return int(load_library().llmopt_cuda_f16_argmax(buffer, count))


def sample_f16(data: bytes, count: int, *, temperature: float, top_k: int, top_p: float, min_p: float,
               seed: int) -> int:
    """``Sampling.f16_sample_native`` (lib/sampling.ml:192-194): one token from ``count`` fp16
    logits held on the host."""
    buffer = ctypes.create_string_buffer(bytes(data), max(len(data), 1))
    out = ctypes.c_int64()
    _check(load_library().llmopt_cuda_sample_f16(buffer, count, float(temperature), int(top_k), float(top_p),
                                                 float(min_p), int(seed) & 0xFFFFFFFFFFFFFFFF, ctypes.byref(out)))
    return int(out.value)


def measure_hardware(*, warmup: int, repeats: int, nbytes: int, device: int = -1) -> tuple:
    """``caml_llmopt_metal_measure_hardware`` (bin/hardware_probe.ml:9-11): (device name, largest
    thread block, median empty-dispatch seconds, median copy bandwidth in GB/s)."""
    name = ctypes.create_string_buffer(256)
    threads, seconds, bandwidth = ctypes.c_int(), ctypes.c_double(), ctypes.c_double()
    _check(load_library().llmopt_cuda_measure_hardware(int(device), int(warmup), int(repeats), int(nbytes), name, 256,
                                                       ctypes.byref(threads), ctypes.byref(seconds),
                                                       ctypes.byref(bandwidth)))
    return name.value.decode(), int(threads.value), float(seconds.value), float(bandwidth.value)
