/* C ABI over the tt::runtime API of the B200 target: the drop-in boundary for host languages.
 *
 * In tt-mlir the callers of the hot path (ttrt, tools/builder, tt-xla's PJRT plugin) reach
 * tt::runtime through the nanobind module runtime/python/runtime/runtime.cpp and
 * runtime/python/binary/binary.cpp.  Each function below flattens one of the C++ entry points
 * those bindings wrap (runtime/include/tt/runtime/runtime.h) into plain C so that any FFI --
 * ctypes, cffi, nanobind, JNI -- can bind the same surface.  The citation beside a
 * declaration is the reference function it stands for.
 *
 * Conventions: every function returns 0 or a non-zero status and never throws;
 * ttrt_last_error() returns the message of the calling thread's last failure (the text the
 * C++ API would have thrown as std::runtime_error).  Handles are opaque pointers owned by
 * the caller and released with the matching *_free.  `dtype` values are tt::target::DataType
 * (include/ttmlir/Target/Common/types.fbs:19-42).
 */
#ifndef TTB_RUNTIME_H
#define TTB_RUNTIME_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TTRT_API __attribute__((visibility("default")))
#define TTRT_MAX_RANK 8

typedef void *ttrt_binary_t;
typedef void *ttrt_device_t;
typedef void *ttrt_tensor_t;
typedef void *ttrt_layout_t;
typedef void *ttrt_tensor_ref_t;

TTRT_API const char *ttrt_last_error(void);
TTRT_API void ttrt_free_string(char *s);

/* ---- Binary (runtime/include/tt/runtime/types.h:336-386, runtime/lib/binary.cpp) ---------- */
TTRT_API int ttrt_binary_load_from_path(const char *path, ttrt_binary_t *out);   /* Binary::loadFromPath */
TTRT_API int ttrt_binary_load_from_memory(const void *mem, size_t size, ttrt_binary_t *out);
TTRT_API void ttrt_binary_free(ttrt_binary_t bin);
TTRT_API int ttrt_binary_store(ttrt_binary_t bin, const char *path);              /* Flatbuffer::store */
TTRT_API int ttrt_binary_file_identifier(ttrt_binary_t bin, char out[5]);         /* getFileIdentifier */
TTRT_API int ttrt_binary_version(ttrt_binary_t bin, char *out, size_t cap);       /* getVersion */
TTRT_API int ttrt_binary_check_schema_hash(ttrt_binary_t bin, int *ok);           /* checkSchemaHash */
TTRT_API int ttrt_binary_as_json(ttrt_binary_t bin, char **out);                  /* asJson; free with ttrt_free_string */
TTRT_API int ttrt_binary_num_programs(ttrt_binary_t bin, uint32_t *n);            /* getNumPrograms */
TTRT_API int ttrt_binary_program_name(ttrt_binary_t bin, uint32_t program, char *out, size_t cap);
TTRT_API int ttrt_binary_is_program_private(ttrt_binary_t bin, uint32_t program, int *priv);
TTRT_API int ttrt_binary_num_program_inputs(ttrt_binary_t bin, uint32_t program, uint32_t *n);
TTRT_API int ttrt_binary_num_program_outputs(ttrt_binary_t bin, uint32_t program, uint32_t *n);
/* getProgramInputs / getProgramOutputs: descriptor `index` of the inputs (is_output = 0) or outputs. */
TTRT_API int ttrt_binary_program_io_desc(ttrt_binary_t bin, uint32_t program, int is_output, uint32_t index,
                                         uint32_t *rank, uint32_t shape[TTRT_MAX_RANK], int *dtype);
TTRT_API int ttrt_binary_program_mesh_shape(ttrt_binary_t bin, uint32_t program, uint32_t *y, uint32_t *x);
TTRT_API int ttrt_binary_program_ops_as_json(ttrt_binary_t bin, uint32_t program, char **out);
/* The remaining string views of a Binary (runtime/lib/binary.cpp): getProgramInputsAsJson, getProgramOutputsAsJson,
 * getMlirAsJson, getSystemDescAsJson, getSchemaHash, getTTMLIRGitHash.  `program` is ignored where it does
 * not apply.  Free the result with ttrt_free_string. */
enum { TTRT_Q_PROGRAM_INPUTS_JSON = 0, TTRT_Q_PROGRAM_OUTPUTS_JSON = 1, TTRT_Q_MLIR_JSON = 2, TTRT_Q_SYSTEM_DESC_JSON = 3,
       TTRT_Q_SCHEMA_HASH = 4, TTRT_Q_TTMLIR_GIT_HASH = 5 };
TTRT_API int ttrt_binary_query_string(ttrt_binary_t bin, int what, uint32_t program, char **out);

/* ---- runtime selection, devices (runtime.h:35-38,160-171) --------------------------------- */
TTRT_API int ttrt_set_compatible_device_runtime(ttrt_binary_t bin);               /* setCompatibleDeviceRuntime */
TTRT_API int ttrt_get_num_available_devices(size_t *n);                           /* getNumAvailableDevices */
/* 128 bytes shared by all processes of a one-process-per-GPU mesh (no reference counterpart:
 * the reference drives a whole mesh from one process). */
TTRT_API int ttrt_get_nccl_unique_id(char id128[128]);
/* openMeshDevice(MeshDeviceOptions).  device_ids may be null (device i backs coordinate i).
 * process_count <= 1: this process owns every coordinate.  Otherwise it owns coordinate
 * process_rank only, on CUDA device device_ids[0] (or 0), and nccl_id128 must be set. */
TTRT_API int ttrt_open_mesh_device(uint32_t mesh_y, uint32_t mesh_x, const int *device_ids, uint32_t n_device_ids,
                                   uint32_t process_rank, uint32_t process_count, const char *nccl_id128,
                                   ttrt_device_t *out);
TTRT_API int ttrt_close_mesh_device(ttrt_device_t dev);                           /* closeMeshDevice */
TTRT_API void ttrt_device_free(ttrt_device_t dev);
TTRT_API int ttrt_device_mesh_shape(ttrt_device_t dev, uint32_t *y, uint32_t *x); /* getMeshShape */
TTRT_API int ttrt_device_num_local(ttrt_device_t dev, uint32_t *n);
/* The CUDA stream (cudaStream_t) and device ordinal behind local coordinate `index`, for
 * callers that time with events on the launching stream. */
TTRT_API int ttrt_device_stream(ttrt_device_t dev, uint32_t index, void **stream, int *cuda_device);

/* ---- tensors (runtime.h:51-157) ------------------------------------------------------------ */
TTRT_API int ttrt_create_borrowed_host_tensor(void *data, const uint32_t *shape, const int64_t *stride, uint32_t rank,
                                              uint32_t itemsize, int dtype, ttrt_tensor_t *out);
TTRT_API int ttrt_create_owned_host_tensor(const void *data, const uint32_t *shape, const int64_t *stride,
                                           uint32_t rank, uint32_t itemsize, int dtype, ttrt_tensor_t *out);
/* createMultiDeviceHostTensor(shards, strategy, meshShape) */
TTRT_API int ttrt_create_multi_device_host_tensor(const ttrt_tensor_t *shards, uint32_t n_shards, uint32_t mesh_y,
                                                  uint32_t mesh_x, ttrt_tensor_t *out);
TTRT_API void ttrt_tensor_free(ttrt_tensor_t t);
/* getTensorShape / getTensorDataType / storage (0 host, 1 device) / shard count / isTensorAllocated */
TTRT_API int ttrt_tensor_info(ttrt_tensor_t t, uint32_t *rank, uint32_t shape[TTRT_MAX_RANK], int *dtype,
                              int *storage, uint32_t *n_shards, int *allocated);
TTRT_API int ttrt_tensor_get_retain(ttrt_tensor_t t, int *retain);                /* getTensorRetain */
TTRT_API int ttrt_tensor_set_retain(ttrt_tensor_t t, int retain);                 /* setTensorRetain */
TTRT_API int ttrt_deallocate_tensor(ttrt_tensor_t t, int force);                  /* deallocateTensor */

/* ---- layouts and movement (runtime.h:196-227) ------------------------------------------------ */
TTRT_API int ttrt_get_layout(ttrt_binary_t bin, uint32_t program, uint32_t input, ttrt_layout_t *out); /* getLayout */
TTRT_API void ttrt_layout_free(ttrt_layout_t l);
/* toLayout(tensor, device, layout, retain): retain < 0 means "not given". */
TTRT_API int ttrt_to_layout(ttrt_tensor_t t, ttrt_device_t dev, ttrt_layout_t layout, int retain, ttrt_tensor_t *out);
TTRT_API int ttrt_has_layout(ttrt_tensor_t t, ttrt_layout_t layout, int *yes);    /* hasLayout */
/* toHost(tensor, untilize, blocking) -> one host tensor per shard. */
TTRT_API int ttrt_to_host(ttrt_tensor_t t, int untilize, int blocking, ttrt_tensor_t *out, uint32_t cap, uint32_t *n);
/* memcpy(void*, Tensor, targetDataType): target_dtype < 0 keeps the tensor's type. */
TTRT_API int ttrt_memcpy_to_ptr(void *dst, ttrt_tensor_t src, int target_dtype);
TTRT_API int ttrt_memcpy_tensor(ttrt_tensor_t dst, ttrt_tensor_t src);            /* memcpy(Tensor, Tensor) */
TTRT_API int ttrt_wait_tensor(ttrt_tensor_t t);                                   /* wait(Tensor) */
/* Address of a host tensor's data (Tensor::data of runtime/include/tt/runtime/types.h): a view, valid
 * while the tensor lives.  After a non-blocking toHost, call ttrt_wait_tensor before reading. */
TTRT_API int ttrt_tensor_host_ptr(ttrt_tensor_t t, void **ptr);

/* ---- execution (runtime.h:299-301) ----------------------------------------------------------- */
/* submit(device, binary, programIndex, inputs) -> outputs */
TTRT_API int ttrt_submit(ttrt_device_t dev, ttrt_binary_t bin, uint32_t program, const ttrt_tensor_t *inputs,
                         uint32_t n_inputs, ttrt_tensor_t *outputs, uint32_t cap, uint32_t *n_outputs);

/* ---- sub-program state: traces, const-eval cache, counters ---------------------------------- */
TTRT_API int ttrt_binary_id(ttrt_binary_t bin, uint64_t *id);                     /* Binary::id */
/* releaseTrace(device, binaryId, mainProgramId), runtime.h:182-183 */
TTRT_API int ttrt_release_trace(ttrt_device_t dev, uint64_t binary_id, size_t main_program);
/* GlobalTensorCache::size / clear (detail/ttnn/types/global_tensor_cache.h:77-93) */
TTRT_API int ttrt_const_eval_cache_size(size_t *n);
TTRT_API int ttrt_const_eval_cache_clear(void);
/* debug::Stats::getStat / clear (debug.h:175-208).  Counters kept by this runtime: ConstEvalCacheHit,
 * ConstEvalCacheMiss, TraceCacheMiss, CapturedTrace, ExecutedTrace. */
TTRT_API int ttrt_stat_get(const char *name, int64_t *value);
TTRT_API int ttrt_stats_clear(void);

/* ---- debug hooks (runtime/include/tt/runtime/debug.h:77-158, runtime.h:229-283) -------------- */
typedef void (*ttrt_op_callback_t)(ttrt_binary_t bin, void *program_ctx, void *op_ctx, void *user);
TTRT_API int ttrt_register_op_hooks(ttrt_op_callback_t pre, ttrt_op_callback_t post, void *user); /* Hooks::get(pre, post) */
TTRT_API int ttrt_unregister_hooks(void);                                                           /* unregisterHooks */
TTRT_API int ttrt_op_loc_info(void *op_ctx, char *out, size_t cap);               /* getOpLocInfo */
TTRT_API int ttrt_op_debug_string(void *op_ctx, char *out, size_t cap);           /* getOpDebugString */
/* getOpOutputTensor: host copy of the op's (first) output on this process' first coordinate;
 * *out = NULL when the op has no live output. */
TTRT_API int ttrt_op_output_tensor(void *op_ctx, void *program_ctx, ttrt_tensor_t *out);
TTRT_API int ttrt_program_index(void *program_ctx, size_t *index);                /* getProgramIndex */

/* getOpInputRefs / getOpOutputRefs (runtime.h:262-263): handles to the tensors an op reads / writes,
 * for callbacks that fetch or overwrite intermediates.  Free each with ttrt_tensor_ref_free. */
TTRT_API int ttrt_op_input_refs(void *op_ctx, ttrt_tensor_ref_t *out, uint32_t cap, uint32_t *n);
TTRT_API int ttrt_op_output_refs(void *op_ctx, ttrt_tensor_ref_t *out, uint32_t cap, uint32_t *n);
TTRT_API void ttrt_tensor_ref_free(ttrt_tensor_ref_t ref);
TTRT_API int ttrt_tensor_ref_info(ttrt_tensor_ref_t ref, uint32_t *rank, uint32_t shape[TTRT_MAX_RANK], int *dtype); /* getTensorRefShape / DataType */
/* retrieveTensorFromPool (runtime.h:266-268): host copy of a live tensor, *out = NULL when it is not live. */
TTRT_API int ttrt_retrieve_tensor_from_pool(void *program_ctx, ttrt_tensor_ref_t ref, int untilize, ttrt_tensor_t *out);
/* updateTensorInPool (runtime.h:269-270): overwrite a live tensor with a host tensor of the same shape. */
TTRT_API int ttrt_update_tensor_in_pool(void *program_ctx, ttrt_tensor_ref_t ref, ttrt_tensor_t src);

/* ---- system descriptor, sub-meshes, embedded goldens ----------------------------------------- */
/* getCurrentSystemDesc (runtime.h:45-47): a "TTSY" flatbuffer describing the visible GPUs (or the devices of
 * `dev`) in the reference's schema; the handle supports the ttrt_binary_* calls that do not need
 * programs (as_json, store, file_identifier, version, free). */
TTRT_API int ttrt_get_current_system_desc(ttrt_device_t dev, ttrt_binary_t *out);
/* createSubMeshDevice / releaseSubMeshDevice / reshapeMeshDevice / getDeviceIds (runtime.h:163-171). */
TTRT_API int ttrt_create_sub_mesh_device(ttrt_device_t parent, uint32_t mesh_y, uint32_t mesh_x, int has_offset,
                                         uint32_t off_y, uint32_t off_x, ttrt_device_t *out);
TTRT_API int ttrt_release_sub_mesh_device(ttrt_device_t sub);
TTRT_API int ttrt_reshape_mesh_device(ttrt_device_t dev, uint32_t mesh_y, uint32_t mesh_x);
TTRT_API int ttrt_device_ids(ttrt_device_t dev, int *ids, uint32_t cap, uint32_t *n);
/* Binary::getDebugInfoGolden (runtime/lib/binary.cpp:233-253): the golden tensors the compiler embedded
 * under a location string, one per device id.  `data` points into the binary (valid while it lives). */
TTRT_API int ttrt_binary_golden_devices(ttrt_binary_t bin, const char *loc, uint32_t *devices, uint32_t cap, uint32_t *n);
TTRT_API int ttrt_binary_golden_tensor(ttrt_binary_t bin, const char *loc, uint32_t device, uint32_t *rank,
                                       int64_t shape[TTRT_MAX_RANK], int64_t stride[TTRT_MAX_RANK], int *dtype,
                                       const void **data, size_t *size);

/* ---- perf::Env (runtime/include/tt/runtime/perf.h:13-53) -----------------------------------------
 * ttrt_perf_env_get = perf::Env::get(dumpDeviceRate, enablePerfTrace, tracyProgramMetadata): the first call
 * fixes the settings; *enabled reports whether tracing is on (also switched on by
 * TT_RUNTIME_ENABLE_PERF_TRACE=1).  While it is on, submit emits per op the reference's messages
 * ("MLIR_OP_LOCATION;<loc>", "MLIR_CONST_EVAL_OP;<bool>", "MLIR_PROGRAM_METADATA;<text>") as NVTX marks and an
 * NVTX range "<OpType> <loc>" around the op's launches.  ttrt_perf_message emits one message by hand
 * (tag 0 tracyLogOpLocation, 1 tracyLogConstEvalProgram, 2 tracyLogProgramMetadata,
 * 3 tracyLogInputLayoutConversion; 4 = setProgramMetadata).  ttrt_perf_emitted counts marks and ranges
 * emitted so far (NVTX has no read-back; tests use this). */
TTRT_API int ttrt_perf_env_get(uint32_t dump_device_rate, int enable_perf_trace, const char *program_metadata, int *enabled);
TTRT_API int ttrt_perf_message(int tag, const char *text);
TTRT_API uint64_t ttrt_perf_emitted(void);

#ifdef __cplusplus
}
#endif

#endif /* TTB_RUNTIME_H */
