/*
 * llmopt_cuda.h — C ABI of libllmopt_cuda.so, the B200 (sm_100a) replacement
 * for the native layer behind llmopt's `Metal_native` module.
 *
 * Every entry point below stands in for one `caml_llmopt_metal_*` /
 * `caml_llmopt_ring_*` / `caml_llmopt_prebaked_*` primitive of the reference
 * (native/ocaml_metal_stubs.m, bound in lib/metal_native.ml:8-124).  The
 * calling convention of a kernel is the reference's: a kernel NAME, the buffers
 * in binding order, the packed little-endian parameter bytes of
 * lib/metal_parameters.ml, and a Metal-style grid in threads plus threadgroup
 * size.  The CUDA launchers size their own grids; the Metal grid is accepted
 * and ignored.
 *
 * Conventions
 *   - plain C types only: opaque handles, pointers, sizes;
 *   - every function that can fail returns an int: 0 success,
 *     LLMOPT_CUDA_FAILURE (reference: `Failure msg`) or
 *     LLMOPT_CUDA_INVALID_ARGUMENT (reference: `Invalid_argument msg`); the
 *     message is kept per thread and read with llmopt_cuda_last_error();
 *   - nothing here aborts or exits the process;
 *   - handles are reference counted; *_release drops one reference, views keep
 *     their parent alive (native/ocaml_metal_stubs.m:945-970);
 *   - one context = one device + one stream; calls on one context must come
 *     from one thread at a time (the OCaml runtime lock gives that), the ring
 *     worker is the only internal thread.
 */
#ifndef LLMOPT_CUDA_H
#define LLMOPT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Only the entry points declared here are exported by the shared library. */
#pragma GCC visibility push(default)

#define LLMOPT_CUDA_OK 0
#define LLMOPT_CUDA_FAILURE 1
#define LLMOPT_CUDA_INVALID_ARGUMENT 2

typedef struct llmopt_cuda_context llmopt_cuda_context;
typedef struct llmopt_cuda_library llmopt_cuda_library;
typedef struct llmopt_cuda_buffer llmopt_cuda_buffer;
typedef struct llmopt_cuda_batch llmopt_cuda_batch;
typedef struct llmopt_cuda_prebaked llmopt_cuda_prebaked;
typedef struct llmopt_cuda_ring llmopt_cuda_ring;

/* One recorded dispatch: the tuple (name, buffers, parameters, grid, group,
 * barrier_before) of Metal_native.Batch.dispatch_item (lib/metal_native.mli:40-51). */
typedef struct llmopt_cuda_dispatch_record {
  const char* name;
  llmopt_cuda_buffer* const* buffers;
  int buffer_count;          /* <= 16 */
  const void* parameters;
  size_t parameter_bytes;    /* <= 256 */
  int grid[3];
  int group[3];
  int barrier_before;
} llmopt_cuda_dispatch_record;

/* Message of the last failed call on this thread ("" if none). */
const char* llmopt_cuda_last_error(void);

/* ---- context, library ------------------------------------------------------ */

/* caml_llmopt_metal_create_context (native/ocaml_metal_stubs.m:410-475).
 * `device` < 0 selects the current CUDA device. */
int llmopt_cuda_create_context(int device, llmopt_cuda_context** out);
void llmopt_cuda_release_context(llmopt_cuda_context* context);
/* caml_llmopt_metal_device_name */
const char* llmopt_cuda_device_name(llmopt_cuda_context* context);
/* caml_llmopt_metal_load_library (:614-700): opens the built-in kernel registry;
 * `path` is accepted for signature compatibility and not read. */
int llmopt_cuda_load_library(llmopt_cuda_context* context, const char* path, llmopt_cuda_library** out);
void llmopt_cuda_release_library(llmopt_cuda_library* library);
/* caml_llmopt_metal_has_function: 1 if `name` resolves to a launcher, else 0. */
int llmopt_cuda_has_function(llmopt_cuda_library* library, const char* name);
/* caml_llmopt_metal_preload_pipeline: fails if the name does not resolve. */
int llmopt_cuda_preload_pipeline(llmopt_cuda_library* library, const char* name);
/* Number of kernel names in the registry and the i-th name (for package validation). */
int llmopt_cuda_function_count(llmopt_cuda_library* library);
const char* llmopt_cuda_function_name(llmopt_cuda_library* library, int index);
/* Registers `alias` (for example a digest-named epilogue kernel,
 * lib/epilogue.ml:217-229) as another name of the existing kernel `target`. */
int llmopt_cuda_register_alias(llmopt_cuda_library* library, const char* alias, const char* target);
/* Registers `name` (a digest name, lib/epilogue.ml:217-229) as a group-64 W4A16 linear whose
 * writeback is a free-form expression over the accumulator (Epilogue.Expr, lib/epilogue.ml:16;
 * lib/metal_parametric_codegen.ml:4-39 compiles one Metal kernel per expression).  `program`
 * is the expression in postfix form, one byte per operation: 1 accumulator, 2 constant (+ 4
 * bytes f32), 3 operand read (+ operand index, + 0 f16 / 1 f32; read at the output column),
 * 10 neg, 11 abs, 12 silu, 13 gelu, 14 exp, 15 log, 16 rsqrt, 17 round-to-half, 20 add, 21 sub,
 * 22 mul, 23 div, 24 min, 25 max, 30 clamp(x, lo, hi), 31 where(c, a, b); at most 192 bytes, 8
 * operands, 12 stack slots.  A dispatch of `name` binds [input, weight, scale, bias_or_scale,
 * output, operand 0 ...] with the 20-byte linear parameter block and computes
 * half(expression) in fp32, like the generated kernel.  llmopt_b200/epilogue.py derives names
 * and programs from expression trees.  A name that extends llmopt_q4_0_linear_f16* binds the same program over the
 * Q4_0-block product instead, with the buffer order of lib/metal_q4_0_epilogue_codegen.ml:7-31 ([input, weight,
 * operand 0 .., output], the 16-byte quant-linear parameter block). */
int llmopt_cuda_register_expr_epilogue(llmopt_cuda_library* library, const char* name, const void* program,
                                       size_t program_bytes, int operand_count);

/* ---- buffers ---------------------------------------------------------------- */

/* caml_llmopt_metal_buffer_of_bytes (:702-724) */
int llmopt_cuda_buffer_of_bytes(llmopt_cuda_context* context, const void* bytes, size_t length,
                                llmopt_cuda_buffer** out);
/* caml_llmopt_metal_create_buffer (:726-745): zero filled; length <= 0 gives 16 bytes. */
int llmopt_cuda_create_buffer(llmopt_cuda_context* context, int64_t length, llmopt_cuda_buffer** out);
/* caml_llmopt_metal_map_file (:747-785): the whole file as one device buffer. */
int llmopt_cuda_map_file(llmopt_cuda_context* context, const char* path, llmopt_cuda_buffer** out);
/* caml_llmopt_metal_buffer_view (:945-970): bounds checked, shares storage. */
int llmopt_cuda_buffer_view(llmopt_cuda_buffer* parent, int64_t offset, int64_t length, llmopt_cuda_buffer** out);
void llmopt_cuda_release_buffer(llmopt_cuda_buffer* buffer);
/* No counterpart in the reference (which is single-device): lets the other ranks of a
 * tensor-parallel group (one process per GPU) map this buffer.  `handle` receives
 * LLMOPT_CUDA_EXPORT_HANDLE_BYTES opaque bytes and `offset` the buffer's offset inside its
 * allocation; a peer process passes both, with the length, to llmopt_cuda_buffer_import and gets
 * a buffer it may bind to the llmopt_tp_exchange_* kernels.  The exporter must outlive every
 * import.  Exchange kernels wait on peers with a bound (about two seconds) and report a
 * time-out through the usual error path of the next stream wait. */
#define LLMOPT_CUDA_EXPORT_HANDLE_BYTES 64
int llmopt_cuda_buffer_export(llmopt_cuda_buffer* buffer, void* handle, uint64_t* offset);
int llmopt_cuda_buffer_import(llmopt_cuda_context* context, const void* handle, uint64_t offset, uint64_t length,
                              llmopt_cuda_buffer** out);
/* caml_llmopt_metal_buffer_length */
size_t llmopt_cuda_buffer_length(llmopt_cuda_buffer* buffer);
/* caml_llmopt_metal_buffer_contents: copies the whole buffer to `destination`
 * (`capacity` >= buffer length) after all queued work on the context finished. */
int llmopt_cuda_buffer_contents(llmopt_cuda_buffer* buffer, void* destination, size_t capacity);
/* caml_llmopt_metal_buffer_argmax_f16 (:787-810): argmax of the LAST row of
 * `vocabulary` halves, first maximum wins. */
int llmopt_cuda_buffer_argmax_f16(llmopt_cuda_buffer* buffer, int64_t vocabulary, int64_t* out);
/* caml_llmopt_metal_buffer_copy: equal lengths required. */
int llmopt_cuda_buffer_copy(llmopt_cuda_buffer* source, llmopt_cuda_buffer* destination);
/* caml_llmopt_metal_buffer_set_int64 / _set_u32_array: host writes, ordered
 * after the work already queued on the context's stream. */
int llmopt_cuda_buffer_set_int64(llmopt_cuda_buffer* buffer, int64_t offset, int64_t value);
int llmopt_cuda_buffer_set_u32_array(llmopt_cuda_buffer* buffer, int64_t offset, const uint32_t* values,
                                     size_t count);
/* Host write of arbitrary bytes (Metal buffers are host-visible; CUDA needs a copy). */
int llmopt_cuda_buffer_write(llmopt_cuda_buffer* buffer, int64_t offset, const void* bytes, size_t length);
/* Raw device address of the buffer (for callers that own other CUDA code). */
void* llmopt_cuda_buffer_device_pointer(llmopt_cuda_buffer* buffer);

/* ---- dispatch ---------------------------------------------------------------- */

/* caml_llmopt_metal_dispatch (:1384-1454): runs one kernel and waits for it. */
int llmopt_cuda_dispatch(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* record);

/* caml_llmopt_metal_begin_batch .. abort_batch (:1132-1382). A batch defers its
 * dispatches until commit, as a Metal command buffer does; abort drops them. */
int llmopt_cuda_begin_batch(llmopt_cuda_library* library, llmopt_cuda_batch** out);
int llmopt_cuda_batch_dispatch(llmopt_cuda_batch* batch, llmopt_cuda_library* library,
                               const llmopt_cuda_dispatch_record* record);
int llmopt_cuda_batch_dispatch_all(llmopt_cuda_batch* batch, llmopt_cuda_library* library,
                                   const llmopt_cuda_dispatch_record* records, size_t count);
/* rejects overlapping ranges of one allocation and unequal lengths */
int llmopt_cuda_batch_copy(llmopt_cuda_batch* batch, llmopt_cuda_buffer* source, llmopt_cuda_buffer* destination);
int llmopt_cuda_batch_barrier(llmopt_cuda_batch* batch); /* no-op: one in-order stream */
int llmopt_cuda_commit_batch(llmopt_cuda_batch* batch);       /* runs everything, blocks */
int llmopt_cuda_commit_batch_async(llmopt_cuda_batch* batch); /* runs everything, returns */
int llmopt_cuda_abort_batch(llmopt_cuda_batch* batch);
void llmopt_cuda_release_batch(llmopt_cuda_batch* batch);
/* Waits for all work queued on the context. */
int llmopt_cuda_synchronize(llmopt_cuda_context* context);

/* ---- prebaked per-token plan -------------------------------------------------- */

/* A row binding: before every replay, row `past_tokens` of `table` (rows of
 * `row_bytes`) is copied on the device into `destination`. It replaces the host
 * writes the reference engine does between tokens (RoPE row, cache slot). */
typedef struct llmopt_cuda_row_binding {
  llmopt_cuda_buffer* destination;
  llmopt_cuda_buffer* table;
  size_t row_bytes;
} llmopt_cuda_row_binding;

/* caml_llmopt_prebaked_create (:1879-2135): records are captured once into a CUDA
 * graph. Records whose name starts with "llmopt_attention_q8_paged_" read
 * past_tokens from a device cell instead of parameter byte 12; the record named
 * "llmopt_cache_pack_checkpoint_q8_simd" reads `checkpoint` instead of byte 0. */
int llmopt_cuda_prebaked_create(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* records,
                                size_t count, llmopt_cuda_buffer* token_buffer, llmopt_cuda_buffer* output_buffer,
                                llmopt_cuda_prebaked** out);
int llmopt_cuda_prebaked_create_bound(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* records,
                                      size_t count, llmopt_cuda_buffer* token_buffer,
                                      llmopt_cuda_buffer* output_buffer, const llmopt_cuda_row_binding* bindings,
                                      size_t binding_count, llmopt_cuda_prebaked** out);
/* caml_llmopt_prebaked_execute (:2167-2563): writes the token id (int64) into the
 * token buffer, publishes past_tokens / checkpoint, replays, waits, returns the
 * int32 at the start of the output buffer. */
int llmopt_cuda_prebaked_execute(llmopt_cuda_prebaked* plan, int64_t token, int32_t past_tokens,
                                 int32_t checkpoint, int32_t* next_token);
/* Device-chained decode (the ring worker's llmopt_chain_token_id path,
 * native/ocaml_metal_stubs.m:1568-1577): `steps` replays back to back, each
 * feeding its output token to the next and advancing past_tokens by one, with no
 * host round trip in between. `tokens_out` receives `steps` ids; `elapsed_ms`
 * (may be NULL) the device time of the replays measured with CUDA events. */
int llmopt_cuda_prebaked_execute_chained(llmopt_cuda_prebaked* plan, int64_t first_token, int32_t past_tokens,
                                         int32_t checkpoint, int32_t steps, int32_t* tokens_out,
                                         float* elapsed_ms);
/* Number of kernel nodes in the captured graph. */
int llmopt_cuda_prebaked_kernel_count(llmopt_cuda_prebaked* plan);
/* Largest past_tokens a replay of this plan accepts: every row-binding table must
 * hold row `past_tokens` and every paged-attention slot table `past_tokens` entries
 * per sequence. execute / execute_chained / the ring refuse larger values with
 * LLMOPT_CUDA_INVALID_ARGUMENT instead of reading past a table (the reference
 * patches byte 12 unchecked, native/ocaml_metal_stubs.m:2182-2185). */
int64_t llmopt_cuda_prebaked_token_capacity(llmopt_cuda_prebaked* plan);
void llmopt_cuda_release_prebaked(llmopt_cuda_prebaked* plan);

/* ---- ring queue ------------------------------------------------------------------ */

/* caml_llmopt_ring_* (:1465-1877): submission / completion queues of 256 entries
 * served by one worker thread that replays a prebaked plan per request. */
int llmopt_cuda_ring_create(llmopt_cuda_ring** out);
int llmopt_cuda_ring_start_worker(llmopt_cuda_ring* ring, llmopt_cuda_library* library,
                                  const llmopt_cuda_dispatch_record* records, size_t count,
                                  llmopt_cuda_buffer* token_buffer, llmopt_cuda_buffer* output_buffer);
/* `accepted` = 0 when the submission queue is full. flags == 2 stops the worker. */
int llmopt_cuda_ring_submit(llmopt_cuda_ring* ring, int64_t request_id, int64_t token, int32_t past_tokens,
                            int32_t flags, int* accepted);
int llmopt_cuda_ring_wait_completion(llmopt_cuda_ring* ring, int64_t* request_id, int32_t* token, int32_t* status);
int llmopt_cuda_ring_poll_completion(llmopt_cuda_ring* ring, int* available, int64_t* request_id, int32_t* token,
                                     int32_t* status);
int llmopt_cuda_ring_destroy(llmopt_cuda_ring* ring);

/* ---- host-side helpers ------------------------------------------------------------ */

/* caml_llmopt_f16_argmax (:2565-2579): argmax over `count` halves in host memory. */
int64_t llmopt_cuda_f16_argmax(const void* halves, size_t count);

/* caml_llmopt_sample_f16_native / _bytecode (:2629-2771, bound at lib/sampling.ml:192-194):
 * samples one token from `count` fp16 logits in HOST memory.  temperature <= 1e-4 or
 * top_k == 1 is greedy (first maximum).  Otherwise the top_k largest logits (64 when
 * top_k <= 0, at most 256) are weighted by exp((logit - max) / temperature) in fp32, cut by
 * min_p (tail below min_p times the best probability) and then by top_p (shortest prefix
 * whose probability reaches top_p), and one xoroshiro128+ draw seeded from `seed` picks
 * among them; seed 0 takes a clock value.  The same seed gives the same token as the
 * reference's sampler. */
int llmopt_cuda_sample_f16(const void* halves, size_t count, double temperature, int top_k, double top_p,
                           double min_p, uint64_t seed, int64_t* token);

/* caml_llmopt_metal_measure_hardware (:477-611, bound at bin/hardware_probe.ml:11): device
 * name, the largest thread block, the median launch-to-completion time of an empty kernel
 * (host clock, seconds) and the median bandwidth of a device-to-device copy of `bytes`
 * bytes (2 * bytes / device time, GB/s) over `repeats` samples after `warmup`.  Requires
 * warmup >= 0, repeats > 0, bytes >= 4096 and a multiple of 16 (else
 * LLMOPT_CUDA_INVALID_ARGUMENT).  `device` < 0 probes the current device.  Only queries and
 * two small kernels: no device setting is read-modified or changed. */
int llmopt_cuda_measure_hardware(int device, int warmup, int repeats, int64_t bytes, char* name,
                                 size_t name_capacity, int* max_threads_per_block, double* dispatch_seconds,
                                 double* bandwidth_gbps);

/* ---- second boundary: the Python single-op entry ------------------------------------ */

/* native/metal_runtime.cpp:58-136 `w4a16_linear(input, packed_weight, scale, bias)`
 * on raw device pointers: input [m,k] f16, packed [n,k/2] u8, scale [n,k/64] f16,
 * bias [n] f16 or NULL, output [m,n] f16; runs on `stream` (a cudaStream_t, may
 * be NULL for the default stream) and does not synchronise. */
int llmopt_cuda_w4a16_linear(llmopt_cuda_context* context, const void* input, const void* packed_weight,
                             const void* scale, const void* bias, void* output, int64_t m, int64_t n, int64_t k,
                             void* stream);

/* ---- entry point that allocates nothing ---------------------------------------------- */

/* No counterpart in the reference. For hosts that cannot let the library allocate
 * device memory (all HBM already owned by the host's own pools, a fixed memory
 * budget, or a path where an allocation's implicit device synchronisation is not
 * acceptable): the split-K paged Q8 decode attention of
 * llmopt_attention_q8_paged_* with its split scratch in an 8 MiB array that is
 * part of the library image (held on every GPU that loads the library until the
 * process exits). No context is needed; the CURRENT device is used and all
 * pointers are raw device pointers on it:
 *   query [b, hq, 1, D] f16, current_key / current_value [b, hkv, 1, D] f16,
 *   pool u8, slots u32 ([past] shared, or [b, slot_batch_stride] with a nonzero
 *   stride), output [b, 1, hq, D] f16, parameters = the 64-byte paged-attention
 *   block (lib/metal_parameters.ml:119-140).
 * Decode shape only (one query token, no mask, no window, D 64 or 128, group 32 or
 * 64, <= 8 query heads per KV head); batches x kv_heads may not exceed 2016
 * (D = 128) or 3971 (D = 64) — larger problems are rejected with
 * LLMOPT_CUDA_INVALID_ARGUMENT. Runs on `stream` (a cudaStream_t; NULL = default
 * stream) without synchronising. The first call on each device resolves the
 * array's device address; make it before any stream capture begins. Calls share
 * the array, which keeps the previous call's contents; nothing needs clearing,
 * but calls that overlap on the GPU race on it and must be serialised. */
int llmopt_cuda_attention_q8_paged_static(const void* query, const void* current_key, const void* current_value,
                                          const void* pool, const void* slots, void* output,
                                          const void* parameters, size_t parameter_bytes,
                                          uint32_t slot_batch_stride, void* stream);

/* ---- measurement ---------------------------------------------------------------------- */

/* Average device time in milliseconds of one dispatch, measured with CUDA
 * events on the context's stream over `iterations` launches after `warmup`;
 * with flush_l2 != 0 a buffer larger than L2 is rewritten before every timed
 * launch (outside the timed interval). */
int llmopt_cuda_time_dispatch(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* record, int warmup,
                              int iterations, int flush_l2, float* average_ms);

/* The same for a LIST of dispatches run back to back between one pair of events
 * (for example one kernel over the distinct weights of every layer): returns the
 * average milliseconds per dispatch. With a list whose operands exceed the L2
 * many times over no flush is needed, and the launch-to-launch overhead is the
 * one a replayed plan sees rather than that of an isolated launch. */
int llmopt_cuda_time_dispatches(llmopt_cuda_library* library, const llmopt_cuda_dispatch_record* records,
                                size_t count, int warmup, int iterations, float* average_ms_per_dispatch);

#pragma GCC visibility pop

#ifdef __cplusplus
}
#endif
#endif /* LLMOPT_CUDA_H */
