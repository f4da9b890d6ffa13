(* cuda_native.ml — the B200 counterpart of lib/metal_native.ml.

   Same signature as lib/metal_native.mli:1-142 (use that file unchanged as cuda_native.mli), so
   Metal_dispatch_*, Metal_cache, Metal_execution_state, Metal_schedule_executor and
   Serving_engine compile against it untouched: select it with a dune (select ...) clause or pass
   it where a native-layer module is expected.  Every external below is implemented in
   integration/ocaml_cuda_stubs.c on top of libllmopt_cuda.so; argument and result shapes are the
   ones the reference's externals have (lib/metal_native.ml:8-124).

   Differences a caller can observe:
   - [load_library] ignores the metallib path: the kernel registry is built into the shared
     library, and [has_function] answers from it (package validation, :271-277, still runs);
   - [Prebaked.execute] and the ring refuse a [past_tokens] beyond the slot tables the plan
     captured with [Error] instead of reading past them. *)

type context_handle
type library_handle
type buffer_handle
type batch_handle
type ring_handle
type prebaked_handle

let ( let* ) = Result.bind

(* a dispatch as the stubs take it: name, buffers, parameter bytes, grid, threadgroup *)
type raw_dispatch = string * buffer_handle list * bytes * int * int * int * int * int * int
type raw_recorded = string * buffer_handle list * bytes * int * int * int * int * int * int * bool

module Stub = struct
  external create_context : unit -> context_handle = "caml_llmopt_cuda_create_context"
  external device_name : context_handle -> string = "caml_llmopt_cuda_device_name"
  external load_library : context_handle -> string -> library_handle = "caml_llmopt_cuda_load_library"
  external has_function : library_handle -> string -> bool = "caml_llmopt_cuda_has_function"
  external preload_pipeline : library_handle -> string -> unit = "caml_llmopt_cuda_preload_pipeline"
  external buffer_of_bytes : context_handle -> bytes -> buffer_handle = "caml_llmopt_cuda_buffer_of_bytes"
  external create_buffer : context_handle -> int -> buffer_handle = "caml_llmopt_cuda_create_buffer"
  external map_file : context_handle -> string -> buffer_handle = "caml_llmopt_cuda_map_file"
  external buffer_view : buffer_handle -> int -> int -> buffer_handle = "caml_llmopt_cuda_buffer_view"
  external buffer_contents : buffer_handle -> bytes = "caml_llmopt_cuda_buffer_contents"
  external buffer_argmax_f16 : buffer_handle -> int -> int = "caml_llmopt_cuda_buffer_argmax_f16"
  external buffer_length : buffer_handle -> int = "caml_llmopt_cuda_buffer_length"
  external buffer_copy : buffer_handle -> buffer_handle -> unit = "caml_llmopt_cuda_buffer_copy"
  external buffer_set_int64 : buffer_handle -> int -> int64 -> unit = "caml_llmopt_cuda_buffer_set_int64"
  external buffer_set_u32_array : buffer_handle -> int -> int array -> unit
    = "caml_llmopt_cuda_buffer_set_u32_array"
  external dispatch :
    library_handle * string * buffer_handle list * bytes * int * int * int * int * int * int -> unit
    = "caml_llmopt_cuda_dispatch"
  external begin_batch : library_handle -> batch_handle = "caml_llmopt_cuda_begin_batch"
  external batch_dispatch :
    batch_handle * library_handle * string * buffer_handle list * bytes * int * int * int * int * int * int -> unit
    = "caml_llmopt_cuda_batch_dispatch"
  external batch_dispatch_all : batch_handle -> library_handle -> raw_dispatch array -> unit
    = "caml_llmopt_cuda_batch_dispatch_all"
  external batch_copy : batch_handle -> buffer_handle -> buffer_handle -> unit = "caml_llmopt_cuda_batch_copy"
  external batch_barrier : batch_handle -> unit = "caml_llmopt_cuda_batch_barrier"
  external commit_batch : batch_handle -> unit = "caml_llmopt_cuda_commit_batch"
  external commit_batch_async : batch_handle -> unit = "caml_llmopt_cuda_commit_batch_async"
  external abort_batch : batch_handle -> unit = "caml_llmopt_cuda_abort_batch"
  external ring_create : unit -> ring_handle = "caml_llmopt_cuda_ring_create"
  external ring_submit : ring_handle -> int -> int -> int -> int -> bool = "caml_llmopt_cuda_ring_submit"
  external ring_wait_completion : ring_handle -> int * int * int = "caml_llmopt_cuda_ring_wait_completion"
  external ring_poll_completion : ring_handle -> (int * int * int) option
    = "caml_llmopt_cuda_ring_poll_completion"
  external ring_start_worker :
    ring_handle -> library_handle -> raw_recorded array -> buffer_handle -> buffer_handle -> unit
    = "caml_llmopt_cuda_ring_start_worker"
  external ring_destroy : ring_handle -> unit = "caml_llmopt_cuda_ring_destroy"
  external prebaked_create :
    library_handle -> raw_recorded array -> buffer_handle -> buffer_handle -> prebaked_handle
    = "caml_llmopt_cuda_prebaked_create"
  external prebaked_execute : prebaked_handle -> int -> int -> int -> int = "caml_llmopt_cuda_prebaked_execute"
end

(* Failure / Invalid_argument from a stub become [Error msg] (lib/metal_native.ml:126-129). *)
let protect operation =
  match operation () with
  | result -> Ok result
  | exception Failure message -> Error message
  | exception Invalid_argument message -> Error message

type t = {
  context : context_handle;
  library : library_handle;
  package : Serving_package.t;
  tensor_store : (Weight_archive.t * buffer_handle) option;
}

type runtime = t

module Decode_uniforms = struct
  type t = { past_tokens : int }

  let create ~past_tokens =
    if past_tokens > 0 then Ok { past_tokens } else Error "decode past_tokens must be positive"

  let past_tokens { past_tokens } = past_tokens
end

module Buffer = struct
  type t = buffer_handle

  let of_bytes ~runtime contents = protect (fun () -> Stub.buffer_of_bytes runtime.context contents)
  let create ~runtime ~bytes = protect (fun () -> Stub.create_buffer runtime.context bytes)
  let view ~parent ~offset ~bytes = protect (fun () -> Stub.buffer_view parent offset bytes)
  let contents buffer = protect (fun () -> Stub.buffer_contents buffer)
  let argmax_f16 buffer ~vocabulary = protect (fun () -> Stub.buffer_argmax_f16 buffer vocabulary)
  let byte_length = Stub.buffer_length
  let copy ~source ~destination = protect (fun () -> Stub.buffer_copy source destination)
  let set_int64 buffer ~offset value = protect (fun () -> Stub.buffer_set_int64 buffer offset value)
  let set_u32_array buffer ~offset values = protect (fun () -> Stub.buffer_set_u32_array buffer offset values)
end

module Batch = struct
  type dispatch_item = {
    name : string;
    buffers : buffer_handle list;
    parameters : bytes;
    grid_x : int;
    grid_y : int;
    grid_z : int;
    group_x : int;
    group_y : int;
    group_z : int;
    barrier_before : bool;
  }

  type t = {
    handle : batch_handle;
    context : context_handle;
    mutable pending : (library_handle * dispatch_item) list;  (* newest first *)
    mutable next_dispatch_barrier : bool;
  }

  let create (runtime : runtime) =
    let* handle = protect (fun () -> Stub.begin_batch runtime.library) in
    Ok { handle; context = runtime.context; pending = []; next_dispatch_barrier = false }

  let raw item : raw_dispatch =
    ( item.name, item.buffers, item.parameters, item.grid_x, item.grid_y, item.grid_z, item.group_x,
      item.group_y, item.group_z )

  (* Pending dispatches go to the native batch in recording order, one call per run of items that
     share a library (a batch may interleave the libraries of several packages). *)
  let flush batch =
    let oldest_first = List.rev batch.pending in
    batch.pending <- [];
    let rec send = function
      | [] -> Ok ()
      | (library, _) :: _ as items ->
          let same, others = List.partition (fun (other, _) -> other == library) items in
          let records = same |> List.map (fun (_, item) -> raw item) |> Array.of_list in
          let* () = protect (fun () -> Stub.batch_dispatch_all batch.handle library records) in
          send others
    in
    send oldest_first

  let dispatch batch ~(runtime : runtime) ~name ~buffers ~parameters ~grid:(grid_x, grid_y, grid_z)
      ~group:(group_x, group_y, group_z) =
    if batch.context != runtime.context then
      Error "CUDA batch and dispatch runtime use different device contexts"
    else begin
      let item =
        { name; buffers; parameters; grid_x; grid_y; grid_z; group_x; group_y; group_z;
          barrier_before = batch.next_dispatch_barrier }
      in
      batch.pending <- (runtime.library, item) :: batch.pending;
      batch.next_dispatch_barrier <- false;
      Ok ()
    end

  let mark_barrier batch = batch.next_dispatch_barrier <- true

  let after_flush batch operation =
    let* () = flush batch in
    protect operation

  let copy batch ~source ~destination =
    after_flush batch (fun () -> Stub.batch_copy batch.handle source destination)

  let barrier batch = after_flush batch (fun () -> Stub.batch_barrier batch.handle)
  let commit batch = after_flush batch (fun () -> Stub.commit_batch batch.handle)
  let commit_async batch = after_flush batch (fun () -> Stub.commit_batch_async batch.handle)

  let abort batch =
    batch.pending <- [];
    batch.next_dispatch_barrier <- false;
    protect (fun () -> Stub.abort_batch batch.handle)
end

(* ---- package loading: the same checks as the Metal layer, against the built-in registry ---- *)

let declared_kernels package = Serving_package.kernels package |> List.map Kernel_abi.Entry.name

let check_declared library names =
  match List.find_opt (fun name -> not (Stub.has_function library name)) names with
  | Some missing -> Error ("CUDA library does not define declared kernel: " ^ missing)
  | None ->
      List.fold_left
        (fun state name ->
          let* () = state in
          protect (fun () -> Stub.preload_pipeline library name))
        (Ok ()) names

let open_archive ~root package =
  match Serving_package.tensor_store package with
  | None -> Ok None
  | Some store ->
      let path =
        store |> Serving_package.Tensor_store.file |> Serving_package.Artifact.path |> Filename.concat root
      in
      (match Weight_archive.of_file path with
       | Ok archive -> Ok (Some archive)
       | Error _ -> (
           match Gguf.of_file_as_archive path with
           | Ok archive -> Ok (Some archive)
           | Error message -> Error ("cannot load weight store: " ^ message)))

let file_identity path =
  match Unix.stat path with
  | stats -> Ok (stats.Unix.st_dev, stats.Unix.st_ino)
  | exception Unix.Unix_error (error, operation, target) ->
      Error (Printf.sprintf "%s %s: %s" operation target (Unix.error_message error))

let load_packages sources =
  (* validate every package before any device work, as the Metal layer does *)
  let rec validated acc = function
    | [] -> Ok (List.rev acc)
    | (root, package) :: rest ->
        let* () = Serving_package.validate_files ~root package in
        let* archive = open_archive ~root package in
        let* () = Serving_validation.validate ~package ~archive in
        validated ((root, package, archive) :: acc) rest
  in
  let* prepared = validated [] sources in
  if prepared = [] then Error "cannot load an empty serving-package set"
  else
    let* context = protect Stub.create_context in
    (* one device mapping per weight file, shared by the packages that name it *)
    let mapped = Hashtbl.create 4 in
    let map_archive archive =
      let path = Weight_archive.path archive in
      let* identity = file_identity path in
      match Hashtbl.find_opt mapped identity with
      | Some buffer -> Ok buffer
      | None ->
          let* buffer = protect (fun () -> Stub.map_file context path) in
          Hashtbl.add mapped identity buffer;
          Ok buffer
    in
    let rec load acc = function
      | [] -> Ok (List.rev acc)
      | (root, package, archive) :: rest ->
          let library_path =
            Serving_package.files package |> Serving_package.Files.metal_library
            |> Serving_package.Artifact.path |> Filename.concat root
          in
          let* library = protect (fun () -> Stub.load_library context library_path) in
          let* tensor_store =
            match archive with
            | None -> Ok None
            | Some archive ->
                let* buffer = map_archive archive in
                Ok (Some (archive, buffer))
          in
          let* () = check_declared library (declared_kernels package) in
          load ({ context; library; package; tensor_store } :: acc) rest
    in
    load [] prepared

let load_package ~root package =
  let* runtimes = load_packages [ (root, package) ] in
  match runtimes with
  | [ runtime ] -> Ok runtime
  | _ -> Error "single serving-package load returned an invalid runtime count"

let device_name runtime = Stub.device_name runtime.context
let package runtime = runtime.package

let tensor runtime ~name =
  match runtime.tensor_store with
  | None -> Error "serving package has no tensor store"
  | Some (archive, mapped) -> (
      match Weight_archive.find archive name with
      | None -> Error ("tensor store does not contain tensor: " ^ name)
      | Some tensor ->
          let* view =
            protect (fun () ->
                Stub.buffer_view mapped (Weight_archive.Tensor.offset tensor)
                  (Weight_archive.Tensor.byte_length tensor))
          in
          Ok (view, tensor))

(* exactly one entry of the package must match (operation, dtypes[, name]) *)
let kernel_entry ?name runtime ~operation ~input_dtype ~output_dtype =
  let wanted entry =
    Kernel_abi.Entry.operation entry = operation
    && Kernel_abi.Entry.input_dtype entry = input_dtype
    && Kernel_abi.Entry.output_dtype entry = output_dtype
    && (match name with None -> true | Some expected -> Kernel_abi.Entry.name entry = expected)
  in
  let describe () =
    Printf.sprintf "%s -> %s" (Ir.Dtype.to_string input_dtype) (Ir.Dtype.to_string output_dtype)
  in
  match List.filter wanted (Serving_package.kernels runtime.package) with
  | [ entry ] -> Ok entry
  | [] ->
      Error
        (Printf.sprintf "serving package has no %s%s kernel for %s"
           (Kernel_abi.Operation.to_string operation)
           (match name with None -> "" | Some value -> " " ^ value)
           (describe ()))
  | several ->
      Error
        (Printf.sprintf "serving package has ambiguous %s kernel selection for %s: %s"
           (Kernel_abi.Operation.to_string operation) (describe ())
           (several |> List.map Kernel_abi.Entry.name |> String.concat ", "))

let dispatch ?batch runtime entry ~buffers ~parameters ~grid:(grid_x, grid_y, grid_z) =
  let name = Kernel_abi.Entry.name entry in
  let group_x, group_y, group_z = Kernel_abi.Entry.threadgroup entry in
  let* () =
    match batch with
    | Some batch ->
        Batch.dispatch batch ~runtime ~name ~buffers ~parameters ~grid:(grid_x, grid_y, grid_z)
          ~group:(group_x, group_y, group_z)
    | None ->
        protect (fun () ->
            Stub.dispatch
              (runtime.library, name, buffers, parameters, grid_x, grid_y, grid_z, group_x, group_y, group_z))
  in
  Ok name

module Ring_queue = struct
  type t = ring_handle

  let default_pipeline_depth = 1

  let pipeline_depth () =
    match Option.bind (Sys.getenv_opt "LLMOPT_QUEUE_DEPTH") int_of_string_opt with
    | Some depth when depth >= 1 -> depth
    | _ -> default_pipeline_depth

  let create () = protect Stub.ring_create

  let submit ring ~request_id ~token ~past_tokens ~flags =
    protect (fun () -> Stub.ring_submit ring request_id token past_tokens flags)

  let wait_completion ring = protect (fun () -> Stub.ring_wait_completion ring)
  let poll_completion ring = protect (fun () -> Stub.ring_poll_completion ring)

  let start_worker ring ~(runtime : runtime) ~dispatches ~token_buffer ~output_buffer =
    protect (fun () -> Stub.ring_start_worker ring runtime.library dispatches token_buffer output_buffer)

  let destroy ring = protect (fun () -> Stub.ring_destroy ring)
end

module Prebaked = struct
  type t = prebaked_handle

  let create ~(runtime : runtime) ~dispatches ~token_buffer ~output_buffer =
    protect (fun () -> Stub.prebaked_create runtime.library dispatches token_buffer output_buffer)

  let execute plan ~token ~past_tokens ~checkpoint =
    protect (fun () -> Stub.prebaked_execute plan token past_tokens checkpoint)
end
