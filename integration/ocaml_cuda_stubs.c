/*
 * ocaml_cuda_stubs.c — the OCaml side of the native boundary on top of libllmopt_cuda.so.
 *
 * One CAMLprim per external of lib/metal_native.ml:8-124, lib/sampling.ml:192-194 and
 * bin/hardware_probe.ml:9-11, with the reference's argument and result shapes, each calling the
 * entry of include/llmopt_cuda.h that replaces it.  Drop this file next to
 * native/ocaml_metal_stubs.m, build it with the OCaml headers on the include path and link
 * -lllmopt_cuda -lcudart; lib/cuda_native.ml (beside this file) binds these names behind the
 * unchanged signature of lib/metal_native.mli.
 *
 * Conventions carried over from the reference stubs:
 *   - every handle is an OCaml custom block holding one pointer; the finalizer drops one
 *     reference (views keep their parent alive inside the library);
 *   - errors raise Failure / Invalid_argument with the library's message
 *     (Metal_native.protect turns both into Error msg, lib/metal_native.ml:126-129);
 *   - the runtime lock is released around every call that waits for the GPU;
 *   - the ring worker is a thread of the library and never touches OCaml values.
 *
 * This translation unit needs <caml/...> and is therefore not compiled by the CUDA build of
 * this repository (which has no OCaml toolchain); it is written against the OCaml 5 C API the
 * reference's own stubs use.
 */
#include <stdint.h>
#include <string.h>

#include <caml/alloc.h>
#include <caml/custom.h>
#include <caml/fail.h>
#include <caml/memory.h>
#include <caml/mlvalues.h>
#include <caml/threads.h>

#include "llmopt_cuda.h"

/* ---- errors and handles ---------------------------------------------------------------- */

static void check(int status) {
  if (status == LLMOPT_CUDA_OK) return;
  if (status == LLMOPT_CUDA_INVALID_ARGUMENT) caml_invalid_argument(llmopt_cuda_last_error());
  caml_failwith(llmopt_cuda_last_error());
}

#define HANDLE(name, type, release)                                                              \
  static void finalize_##name(value v) {                                                         \
    type *p = *(type **)Data_custom_val(v);                                                      \
    if (p != NULL) release(p);                                                                   \
  }                                                                                              \
  static struct custom_operations name##_ops = {                                                 \
      "llmopt.cuda." #name,       finalize_##name,          custom_compare_default,              \
      custom_hash_default,        custom_serialize_default, custom_deserialize_default,          \
      custom_compare_ext_default, custom_fixed_length_default};                                  \
  static value alloc_##name(type *p) {                                                           \
    value v = caml_alloc_custom(&name##_ops, sizeof(type *), 0, 1);                              \
    *(type **)Data_custom_val(v) = p;                                                            \
    return v;                                                                                    \
  }                                                                                              \
  static type *name##_val(value v) { return *(type **)Data_custom_val(v); }

static void release_ring(llmopt_cuda_ring *ring) { llmopt_cuda_ring_destroy(ring); }

HANDLE(context, llmopt_cuda_context, llmopt_cuda_release_context)
HANDLE(library, llmopt_cuda_library, llmopt_cuda_release_library)
HANDLE(buffer, llmopt_cuda_buffer, llmopt_cuda_release_buffer)
HANDLE(batch, llmopt_cuda_batch, llmopt_cuda_release_batch)
HANDLE(plan, llmopt_cuda_prebaked, llmopt_cuda_release_prebaked)
HANDLE(ring, llmopt_cuda_ring, release_ring)

/* ---- context, library -------------------------------------------------------------------- */

CAMLprim value caml_llmopt_cuda_create_context(value unit) {
  CAMLparam1(unit);
  llmopt_cuda_context *context = NULL;
  check(llmopt_cuda_create_context(-1, &context));
  CAMLreturn(alloc_context(context));
}

CAMLprim value caml_llmopt_cuda_device_name(value v_context) {
  CAMLparam1(v_context);
  CAMLreturn(caml_copy_string(llmopt_cuda_device_name(context_val(v_context))));
}

CAMLprim value caml_llmopt_cuda_load_library(value v_context, value v_path) {
  CAMLparam2(v_context, v_path);
  llmopt_cuda_library *library = NULL;
  check(llmopt_cuda_load_library(context_val(v_context), String_val(v_path), &library));
  CAMLreturn(alloc_library(library));
}

CAMLprim value caml_llmopt_cuda_has_function(value v_library, value v_name) {
  CAMLparam2(v_library, v_name);
  CAMLreturn(Val_bool(llmopt_cuda_has_function(library_val(v_library), String_val(v_name))));
}

CAMLprim value caml_llmopt_cuda_preload_pipeline(value v_library, value v_name) {
  CAMLparam2(v_library, v_name);
  check(llmopt_cuda_preload_pipeline(library_val(v_library), String_val(v_name)));
  CAMLreturn(Val_unit);
}

/* ---- buffers ---------------------------------------------------------------------------- */

CAMLprim value caml_llmopt_cuda_buffer_of_bytes(value v_context, value v_bytes) {
  CAMLparam2(v_context, v_bytes);
  llmopt_cuda_buffer *buffer = NULL;
  check(llmopt_cuda_buffer_of_bytes(context_val(v_context), Bytes_val(v_bytes), caml_string_length(v_bytes), &buffer));
  CAMLreturn(alloc_buffer(buffer));
}

CAMLprim value caml_llmopt_cuda_create_buffer(value v_context, value v_bytes) {
  CAMLparam2(v_context, v_bytes);
  llmopt_cuda_buffer *buffer = NULL;
  check(llmopt_cuda_create_buffer(context_val(v_context), (int64_t)Long_val(v_bytes), &buffer));
  CAMLreturn(alloc_buffer(buffer));
}

CAMLprim value caml_llmopt_cuda_map_file(value v_context, value v_path) {
  CAMLparam2(v_context, v_path);
  llmopt_cuda_buffer *buffer = NULL;
  check(llmopt_cuda_map_file(context_val(v_context), String_val(v_path), &buffer));
  CAMLreturn(alloc_buffer(buffer));
}

CAMLprim value caml_llmopt_cuda_buffer_view(value v_parent, value v_offset, value v_length) {
  CAMLparam3(v_parent, v_offset, v_length);
  llmopt_cuda_buffer *buffer = NULL;
  check(llmopt_cuda_buffer_view(buffer_val(v_parent), (int64_t)Long_val(v_offset), (int64_t)Long_val(v_length), &buffer));
  CAMLreturn(alloc_buffer(buffer));
}

CAMLprim value caml_llmopt_cuda_buffer_contents(value v_buffer) {
  CAMLparam1(v_buffer);
  CAMLlocal1(v_bytes);
  llmopt_cuda_buffer *buffer = buffer_val(v_buffer);
  size_t length = llmopt_cuda_buffer_length(buffer);
  v_bytes = caml_alloc_string(length);
  /* the copy waits for queued work; the destination is an OCaml block, so the lock stays held */
  check(llmopt_cuda_buffer_contents(buffer, Bytes_val(v_bytes), length));
  CAMLreturn(v_bytes);
}

CAMLprim value caml_llmopt_cuda_buffer_argmax_f16(value v_buffer, value v_vocabulary) {
  CAMLparam2(v_buffer, v_vocabulary);
  int64_t index = 0;
  check(llmopt_cuda_buffer_argmax_f16(buffer_val(v_buffer), (int64_t)Long_val(v_vocabulary), &index));
  CAMLreturn(Val_long(index));
}

CAMLprim value caml_llmopt_cuda_buffer_length(value v_buffer) {
  CAMLparam1(v_buffer);
  CAMLreturn(Val_long((intnat)llmopt_cuda_buffer_length(buffer_val(v_buffer))));
}

CAMLprim value caml_llmopt_cuda_buffer_copy(value v_source, value v_destination) {
  CAMLparam2(v_source, v_destination);
  check(llmopt_cuda_buffer_copy(buffer_val(v_source), buffer_val(v_destination)));
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_buffer_set_int64(value v_buffer, value v_offset, value v_value) {
  CAMLparam3(v_buffer, v_offset, v_value);
  check(llmopt_cuda_buffer_set_int64(buffer_val(v_buffer), (int64_t)Long_val(v_offset), Int64_val(v_value)));
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_buffer_set_u32_array(value v_buffer, value v_offset, value v_values) {
  CAMLparam3(v_buffer, v_offset, v_values);
  mlsize_t count = Wosize_val(v_values);
  uint32_t stack[256];
  uint32_t *values = count <= 256 ? stack : (uint32_t *)caml_stat_alloc(count * sizeof(uint32_t));
  for (mlsize_t i = 0; i < count; ++i) values[i] = (uint32_t)Long_val(Field(v_values, i));
  int status = llmopt_cuda_buffer_set_u32_array(buffer_val(v_buffer), (int64_t)Long_val(v_offset), values, count);
  if (values != stack) caml_stat_free(values);
  check(status);
  CAMLreturn(Val_unit);
}

/* ---- dispatch records -------------------------------------------------------------------- */

/* An OCaml dispatch tuple (name, buffers, parameters, gx, gy, gz, tx, ty, tz[, barrier]) as a
 * record.  The library copies names and parameter bytes and retains the buffers before the call
 * returns, so pointers into OCaml blocks are only used while no allocation can move them. */
typedef struct {
  llmopt_cuda_dispatch_record record;
  llmopt_cuda_buffer *slots[16];
} stub_record;

static void fill_record(value item, int has_barrier, stub_record *out) {
  int count = 0;
  for (value list = Field(item, 1); list != Val_emptylist; list = Field(list, 1)) {
    if (count == 16) caml_invalid_argument("a dispatch binds at most 16 buffers");
    out->slots[count++] = buffer_val(Field(list, 0));
  }
  out->record.name = String_val(Field(item, 0));
  out->record.buffers = out->slots;
  out->record.buffer_count = count;
  out->record.parameters = Bytes_val(Field(item, 2));
  out->record.parameter_bytes = caml_string_length(Field(item, 2));
  for (int axis = 0; axis < 3; ++axis) {
    out->record.grid[axis] = (int)Long_val(Field(item, 3 + axis));
    out->record.group[axis] = (int)Long_val(Field(item, 6 + axis));
  }
  out->record.barrier_before = has_barrier ? Bool_val(Field(item, 9)) : 0;
}

/* the records of a whole array, heap allocated (freed by the caller) */
static stub_record *fill_records(value items, int has_barrier, llmopt_cuda_dispatch_record **flat) {
  mlsize_t count = Wosize_val(items);
  stub_record *records = (stub_record *)caml_stat_alloc((count ? count : 1) * sizeof(stub_record));
  *flat = (llmopt_cuda_dispatch_record *)caml_stat_alloc((count ? count : 1) * sizeof(llmopt_cuda_dispatch_record));
  for (mlsize_t i = 0; i < count; ++i) {
    fill_record(Field(items, i), has_barrier, &records[i]);
    (*flat)[i] = records[i].record;
  }
  return records;
}

/* (library, name, buffers, parameters, gx, gy, gz, tx, ty, tz): one tuple argument */
CAMLprim value caml_llmopt_cuda_dispatch(value v_tuple) {
  CAMLparam1(v_tuple);
  stub_record item;
  /* fields 1.. of the tuple are laid out like a dispatch item shifted by one */
  int count = 0;
  for (value list = Field(v_tuple, 2); list != Val_emptylist; list = Field(list, 1)) {
    if (count == 16) caml_invalid_argument("a dispatch binds at most 16 buffers");
    item.slots[count++] = buffer_val(Field(list, 0));
  }
  item.record.name = String_val(Field(v_tuple, 1));
  item.record.buffers = item.slots;
  item.record.buffer_count = count;
  item.record.parameters = Bytes_val(Field(v_tuple, 3));
  item.record.parameter_bytes = caml_string_length(Field(v_tuple, 3));
  for (int axis = 0; axis < 3; ++axis) {
    item.record.grid[axis] = (int)Long_val(Field(v_tuple, 4 + axis));
    item.record.group[axis] = (int)Long_val(Field(v_tuple, 7 + axis));
  }
  item.record.barrier_before = 0;
  /* synchronous: the call returns when the kernel has finished (the name and parameter bytes are
   * read before the wait, so the lock is kept; a dispatch is microseconds) */
  check(llmopt_cuda_dispatch(library_val(Field(v_tuple, 0)), &item.record));
  CAMLreturn(Val_unit);
}

/* ---- batches ------------------------------------------------------------------------------ */

CAMLprim value caml_llmopt_cuda_begin_batch(value v_library) {
  CAMLparam1(v_library);
  llmopt_cuda_batch *batch = NULL;
  check(llmopt_cuda_begin_batch(library_val(v_library), &batch));
  CAMLreturn(alloc_batch(batch));
}

/* (batch, library, name, buffers, parameters, gx, gy, gz, tx, ty, tz): one tuple argument */
CAMLprim value caml_llmopt_cuda_batch_dispatch(value v_tuple) {
  CAMLparam1(v_tuple);
  stub_record item;
  int count = 0;
  for (value list = Field(v_tuple, 3); list != Val_emptylist; list = Field(list, 1)) {
    if (count == 16) caml_invalid_argument("a dispatch binds at most 16 buffers");
    item.slots[count++] = buffer_val(Field(list, 0));
  }
  item.record.name = String_val(Field(v_tuple, 2));
  item.record.buffers = item.slots;
  item.record.buffer_count = count;
  item.record.parameters = Bytes_val(Field(v_tuple, 4));
  item.record.parameter_bytes = caml_string_length(Field(v_tuple, 4));
  for (int axis = 0; axis < 3; ++axis) {
    item.record.grid[axis] = (int)Long_val(Field(v_tuple, 5 + axis));
    item.record.group[axis] = (int)Long_val(Field(v_tuple, 8 + axis));
  }
  item.record.barrier_before = 0;
  check(llmopt_cuda_batch_dispatch(batch_val(Field(v_tuple, 0)), library_val(Field(v_tuple, 1)), &item.record));
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_batch_dispatch_all(value v_batch, value v_library, value v_items) {
  CAMLparam3(v_batch, v_library, v_items);
  llmopt_cuda_dispatch_record *flat = NULL;
  stub_record *records = fill_records(v_items, 0, &flat);
  int status = llmopt_cuda_batch_dispatch_all(batch_val(v_batch), library_val(v_library), flat, Wosize_val(v_items));
  caml_stat_free(flat);
  caml_stat_free(records);
  check(status);
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_batch_copy(value v_batch, value v_source, value v_destination) {
  CAMLparam3(v_batch, v_source, v_destination);
  check(llmopt_cuda_batch_copy(batch_val(v_batch), buffer_val(v_source), buffer_val(v_destination)));
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_batch_barrier(value v_batch) {
  CAMLparam1(v_batch);
  check(llmopt_cuda_batch_barrier(batch_val(v_batch)));
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_commit_batch(value v_batch) {
  CAMLparam1(v_batch);
  llmopt_cuda_batch *batch = batch_val(v_batch);
  caml_enter_blocking_section(); /* waits for the GPU */
  int status = llmopt_cuda_commit_batch(batch);
  caml_leave_blocking_section();
  check(status);
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_commit_batch_async(value v_batch) {
  CAMLparam1(v_batch);
  check(llmopt_cuda_commit_batch_async(batch_val(v_batch)));
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_abort_batch(value v_batch) {
  CAMLparam1(v_batch);
  check(llmopt_cuda_abort_batch(batch_val(v_batch)));
  CAMLreturn(Val_unit);
}

/* ---- ring queue ---------------------------------------------------------------------------- */

CAMLprim value caml_llmopt_cuda_ring_create(value unit) {
  CAMLparam1(unit);
  llmopt_cuda_ring *ring = NULL;
  check(llmopt_cuda_ring_create(&ring));
  CAMLreturn(alloc_ring(ring));
}

CAMLprim value caml_llmopt_cuda_ring_submit(value v_ring, value v_request, value v_token, value v_past, value v_flags) {
  CAMLparam5(v_ring, v_request, v_token, v_past, v_flags);
  int accepted = 0;
  check(llmopt_cuda_ring_submit(ring_val(v_ring), (int64_t)Long_val(v_request), (int64_t)Long_val(v_token),
                                (int32_t)Long_val(v_past), (int32_t)Long_val(v_flags), &accepted));
  CAMLreturn(Val_bool(accepted));
}

static value completion_tuple(int64_t request, int32_t token, int32_t status) {
  CAMLparam0();
  CAMLlocal1(v_tuple);
  v_tuple = caml_alloc_tuple(3);
  Store_field(v_tuple, 0, Val_long(request));
  Store_field(v_tuple, 1, Val_long(token));
  Store_field(v_tuple, 2, Val_long(status));
  CAMLreturn(v_tuple);
}

CAMLprim value caml_llmopt_cuda_ring_wait_completion(value v_ring) {
  CAMLparam1(v_ring);
  llmopt_cuda_ring *ring = ring_val(v_ring);
  int64_t request = 0;
  int32_t token = 0, status = 0;
  caml_enter_blocking_section(); /* sleeps until the worker posts a completion */
  int outcome = llmopt_cuda_ring_wait_completion(ring, &request, &token, &status);
  caml_leave_blocking_section();
  check(outcome);
  CAMLreturn(completion_tuple(request, token, status));
}

CAMLprim value caml_llmopt_cuda_ring_poll_completion(value v_ring) {
  CAMLparam1(v_ring);
  CAMLlocal2(v_tuple, v_some);
  int available = 0;
  int64_t request = 0;
  int32_t token = 0, status = 0;
  check(llmopt_cuda_ring_poll_completion(ring_val(v_ring), &available, &request, &token, &status));
  if (!available) CAMLreturn(Val_none);
  v_tuple = completion_tuple(request, token, status);
  v_some = caml_alloc_some(v_tuple);
  CAMLreturn(v_some);
}

CAMLprim value caml_llmopt_cuda_ring_start_worker(value v_ring, value v_library, value v_items, value v_token_buffer,
                                                   value v_output_buffer) {
  CAMLparam5(v_ring, v_library, v_items, v_token_buffer, v_output_buffer);
  llmopt_cuda_dispatch_record *flat = NULL;
  stub_record *records = fill_records(v_items, 1, &flat);
  int status = llmopt_cuda_ring_start_worker(ring_val(v_ring), library_val(v_library), flat, Wosize_val(v_items),
                                             buffer_val(v_token_buffer), buffer_val(v_output_buffer));
  caml_stat_free(flat);
  caml_stat_free(records);
  check(status);
  CAMLreturn(Val_unit);
}

CAMLprim value caml_llmopt_cuda_ring_destroy(value v_ring) {
  CAMLparam1(v_ring);
  llmopt_cuda_ring *ring = ring_val(v_ring);
  *(llmopt_cuda_ring **)Data_custom_val(v_ring) = NULL; /* the finalizer must not destroy it twice */
  if (ring != NULL) {
    caml_enter_blocking_section(); /* joins the worker thread */
    int status = llmopt_cuda_ring_destroy(ring);
    caml_leave_blocking_section();
    check(status);
  }
  CAMLreturn(Val_unit);
}

/* ---- prebaked plan ------------------------------------------------------------------------- */

CAMLprim value caml_llmopt_cuda_prebaked_create(value v_library, value v_items, value v_token_buffer,
                                                 value v_output_buffer) {
  CAMLparam4(v_library, v_items, v_token_buffer, v_output_buffer);
  llmopt_cuda_dispatch_record *flat = NULL;
  stub_record *records = fill_records(v_items, 1, &flat);
  llmopt_cuda_prebaked *plan = NULL;
  int status = llmopt_cuda_prebaked_create(library_val(v_library), flat, Wosize_val(v_items),
                                           buffer_val(v_token_buffer), buffer_val(v_output_buffer), &plan);
  caml_stat_free(flat);
  caml_stat_free(records);
  check(status);
  CAMLreturn(alloc_plan(plan));
}

CAMLprim value caml_llmopt_cuda_prebaked_execute(value v_plan, value v_token, value v_past, value v_checkpoint) {
  CAMLparam4(v_plan, v_token, v_past, v_checkpoint);
  llmopt_cuda_prebaked *plan = plan_val(v_plan);
  int64_t token = (int64_t)Long_val(v_token);
  int32_t past = (int32_t)Long_val(v_past), checkpoint = (int32_t)Long_val(v_checkpoint), next = 0;
  caml_enter_blocking_section(); /* replays the graph and waits for the token */
  int status = llmopt_cuda_prebaked_execute(plan, token, past, checkpoint, &next);
  caml_leave_blocking_section();
  check(status);
  CAMLreturn(Val_long(next));
}

/* ---- host helpers ---------------------------------------------------------------------------- */

CAMLprim value caml_llmopt_cuda_f16_argmax(value v_bytes, value v_count) {
  CAMLparam2(v_bytes, v_count);
  CAMLreturn(Val_long(llmopt_cuda_f16_argmax(Bytes_val(v_bytes), (size_t)Long_val(v_count))));
}

CAMLprim value caml_llmopt_cuda_sample_f16_native(value v_bytes, value v_count, value v_temperature, value v_top_k,
                                                   value v_top_p, value v_min_p, value v_seed) {
  CAMLparam5(v_bytes, v_count, v_temperature, v_top_k, v_top_p);
  CAMLxparam2(v_min_p, v_seed);
  int64_t token = 0;
  check(llmopt_cuda_sample_f16(Bytes_val(v_bytes), (size_t)Long_val(v_count), Double_val(v_temperature),
                               (int)Long_val(v_top_k), Double_val(v_top_p), Double_val(v_min_p),
                               (uint64_t)Long_val(v_seed), &token));
  CAMLreturn(Val_long(token));
}

CAMLprim value caml_llmopt_cuda_sample_f16_bytecode(value *argv, int argn) {
  (void)argn;
  return caml_llmopt_cuda_sample_f16_native(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6]);
}

/* (warmup, repeats, bytes) -> (device name, largest thread block, dispatch seconds, copy GB/s) */
CAMLprim value caml_llmopt_cuda_measure_hardware(value v_warmup, value v_repeats, value v_bytes) {
  CAMLparam3(v_warmup, v_repeats, v_bytes);
  CAMLlocal1(v_result);
  char name[256];
  int threads = 0;
  double seconds = 0.0, bandwidth = 0.0;
  int warmup = Int_val(v_warmup), repeats = Int_val(v_repeats);
  int64_t bytes = (int64_t)Long_val(v_bytes);
  caml_enter_blocking_section();
  int status = llmopt_cuda_measure_hardware(-1, warmup, repeats, bytes, name, sizeof name, &threads, &seconds, &bandwidth);
  caml_leave_blocking_section();
  check(status);
  v_result = caml_alloc_tuple(4);
  Store_field(v_result, 0, caml_copy_string(name));
  Store_field(v_result, 1, Val_int(threads));
  Store_field(v_result, 2, caml_copy_double(seconds));
  Store_field(v_result, 3, caml_copy_double(bandwidth));
  CAMLreturn(v_result);
}
