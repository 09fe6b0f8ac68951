/*
 * Artifact / session C ABI of libdinoml_b200_gguf.so: the `dino_*` entry points the reference's Python
 * loader binds with ctypes (src/dinoml/runtime.py:735-832), at runtime ABI version 7
 * (runtime/include/dinoml/abi.h:12).  In the reference these live in a generated, per-model
 * module.so (src/dinoml/templates/gpu_module.cu.j2); here one prebuilt library interprets the
 * artifact's `module_plan.txt` launch plan, so an artifact's module.so is a link to that library.
 *
 * Every function returns 0 on success; on failure it returns non-zero and leaves a message for the
 * calling thread in dino_get_last_error() (runtime/src/runtime_common.cpp:5-20).
 */
#ifndef DINOML_B200_RUNTIME_H_
#define DINOML_B200_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#include "dinoml_b200_gguf.h"

#ifdef __cplusplus
extern "C" {
#endif

#define DINO_RUNTIME_ABI_VERSION 7

/* runtime/include/dinoml/abi.h:14-33 */
enum DinoDtype {
  DINO_DTYPE_FLOAT16 = 1, DINO_DTYPE_FLOAT32 = 2, DINO_DTYPE_INT32 = 3, DINO_DTYPE_INT64 = 4,
  DINO_DTYPE_BOOL = 5, DINO_DTYPE_BFLOAT16 = 6, DINO_DTYPE_FLOAT8_E4M3 = 7, DINO_DTYPE_FLOAT8_E5M2 = 8,
};
enum DinoDeviceType { DINO_DEVICE_CPU = 0, DINO_DEVICE_CUDA = 1, DINO_DEVICE_ROCM = 2 };
enum DinoTensorFlags { DINO_TENSOR_FLAG_CONTIGUOUS = 1 << 0 };

/* Field-for-field the reference's DinoTensor (runtime/include/dinoml/abi.h:36-57; ctypes mirror
 * src/dinoml/runtime.py:33-45).  `shape` / `strides` are HOST arrays owned by the caller for the
 * duration of the call; tensors must be contiguous. */
struct DinoTensor {
  void* data;
  const int64_t* shape;
  size_t ndim;
  int dtype;
  const int64_t* strides;
  size_t byte_offset;
  size_t nbytes;
  int device_type;
  uint32_t flags;
  size_t alignment;
};

struct DinoModule;
struct DinoSession;

/* runtime/include/dinoml/abi.h:63-66, runtime/include/dinoml/runtime.h:9-26 */
DINOML_B200_API int dino_runtime_fail(const char* message);
DINOML_B200_API int dino_abi_version(void);
DINOML_B200_API int dino_device_malloc(void** out, size_t nbytes);
DINOML_B200_API int dino_device_free(void* ptr);
DINOML_B200_API int dino_copy_host_to_device(void* dst, const void* src, size_t nbytes);
DINOML_B200_API int dino_copy_device_to_host(void* dst, const void* src, size_t nbytes);
DINOML_B200_API int dino_copy_device_to_device(void* dst, const void* src, size_t nbytes);

/* src/dinoml/templates/gpu_module.cu.j2:394 (eager constants) and :418 (deferred; what Python uses) */
DINOML_B200_API int dino_module_load(const char* artifact_dir, struct DinoModule** out);
DINOML_B200_API int dino_module_load_deferred(const char* artifact_dir, struct DinoModule** out);
/* gpu_module.cu.j2:267 / :302.  Encoded constants whose residency is manual_runtime_load are skipped by
 * load_constants, as in the reference (:295-297); unload synchronizes the device first. */
DINOML_B200_API int dino_module_load_constants(struct DinoModule* module, const char* constants_path);
DINOML_B200_API int dino_module_unload_constants(struct DinoModule* module);
/* gpu_module.cu.j2:318 - device-to-device copy into the module's own buffer; rejects encoded constants. */
DINOML_B200_API int dino_module_set_constant(struct DinoModule* module, const char* name, const struct DinoTensor* tensor);
/* gpu_module.cu.j2:362-391 - exact-size check, allocate once, device-to-device copy of raw GGUF bytes. */
DINOML_B200_API int dino_module_set_encoded_constant(struct DinoModule* module, const char* name, const void* device_bytes,
                                                     size_t nbytes);
/* Host-resident encoded constants - the residency policies the reference declares (src/dinoml/constant_sources.py:17-34:
 * cpu_until_first_use, sequential_offload, grouped_offload) and leaves "future".  The module copies `host_bytes` into pinned
 * host memory of its own.  cpu_until_first_use: uploaded on the stream of the first run that needs the constant, on the device
 * from then on.  sequential_offload / grouped_offload: never resident; a run copies each offload group (`group` >= 0; give
 * every constant its own group for sequential) into one of two device slots just ahead of its launches, the next group on
 * a second stream while the current one computes - device memory held is twice the largest group.  One session at a time
 * may run a module that streams constants.  Optional symbols, like the reference's set_temp_arena_policy pair. */
DINOML_B200_API int dino_module_set_offloaded_encoded_constant(struct DinoModule* module, const char* name, const void* host_bytes,
                                                               size_t nbytes, int group);
/* Bytes of encoded constants resident on the device, bytes of the two offload slots, pinned host bytes held, and the number /
 * bytes of host-to-device uploads made so far by runs.  Any pointer may be NULL. */
DINOML_B200_API int dino_module_get_residency_stats(struct DinoModule* module, size_t* device_resident_bytes, size_t* device_slot_bytes,
                                                    size_t* pinned_host_bytes, size_t* uploads, size_t* upload_bytes);
DINOML_B200_API int dino_module_free(struct DinoModule* module);                       /* :436 */
DINOML_B200_API const char* dino_module_get_metadata_json(struct DinoModule* module);  /* :449 */

/* gpu_module.cu.j2:458-524 / :526 - a session owns a non-blocking stream and its intermediates. */
DINOML_B200_API int dino_session_create(struct DinoModule* module, struct DinoSession** out);
DINOML_B200_API int dino_session_destroy(struct DinoSession* session);
/* :618 - NULL restores the owned stream; an external stream disables the post-run synchronize. */
DINOML_B200_API int dino_session_set_stream(struct DinoSession* session, void* stream);
/* :630 - shape of output `output_index` as of the last run. */
DINOML_B200_API int dino_session_get_output_shape(struct DinoSession* session, size_t output_index, int64_t* out_shape,
                                                  size_t* inout_ndim);
/* Steady-state replay for dino_session_run (off by default; no counterpart in the reference, whose per-run path re-validates
 * and re-launches every time, gpu_module.cu.j2:706-993): with it on, the launch sequence of a combination of input shapes and
 * input / output device pointers is captured into a CUDA graph the second time the combination is seen and replayed from
 * then on (validation ran at capture).  Callers keep their buffers stable (Session.run_numpy's arenas are).  Modules that
 * stream constants from the host and DINOML_PROFILE_RUN runs always take the ordinary path. */
/* Optional entries of the reference's module (gpu_module.cu.j2:589-615, 662-678).  No per-session temporary arena exists here
 * (no dense dequant scratch) and these graphs have no state tensors: the arena calls check their arguments (policy 0..2)
 * and succeed, every state index is invalid. */
DINOML_B200_API int dino_session_set_temp_arena_policy(struct DinoSession* session, int policy);
DINOML_B200_API int dino_session_release_temp_arena(struct DinoSession* session);
DINOML_B200_API int dino_session_get_state_pointer(struct DinoSession* session, size_t state_index, void** out_data);
DINOML_B200_API int dino_session_set_graph_replay(struct DinoSession* session, int enabled);
DINOML_B200_API int dino_session_get_graph_stats(struct DinoSession* session, size_t* cached_graphs, size_t* graph_launches);
/* :995 / :706-993 - validates every tensor, then launches the plan on the session stream.  With DINOML_PROFILE_RUN set every
 * launch is bracketed by events and "[dinoml_profile] ..." lines go to stderr (DINOML_PROFILE_RUN_VERBOSE: one line per launch;
 * DINOML_PROFILE_RUN_SECTIONS=name:first:last,...: elapsed time of launch ranges), as gpu_module.cu.j2:785-983. */
DINOML_B200_API int dino_session_run(struct DinoSession* session, const struct DinoTensor* inputs, size_t num_inputs,
                                     struct DinoTensor* outputs, size_t num_outputs);
/* dino_session_run with host staging in one call: copies `in_bytes` from pinned host memory `host_in` to `device_in` on the
 * session stream, runs (`inputs` / `outputs` describe tensors inside the two device arenas), copies `out_bytes` from
 * `device_out` to pinned `host_out`, and waits once.  What Session.run_numpy does per call; the reference's loader issues
 * the copies from Python (src/dinoml/runtime.py:1371-1431). */
DINOML_B200_API int dino_session_run_staged(struct DinoSession* session, const void* host_in, void* device_in, size_t in_bytes,
                                            const struct DinoTensor* inputs, size_t num_inputs, struct DinoTensor* outputs,
                                            size_t num_outputs, const void* device_out, void* host_out, size_t out_bytes);
/* The same with this call's stream (null = the session's) and graph-replay setting as arguments, so that a host needs one
 * call per run; the session's own stream and setting are untouched.  `outputs` may point into mapped pinned host memory
 * (then pass out_bytes = 0): the kernels' epilogues store over the bus and no device-to-host copy is issued - worth it for
 * decode-sized results. */
DINOML_B200_API int dino_session_run_staged_on(struct DinoSession* session, void* stream, int graph_replay, const void* host_in,
                                               void* device_in, size_t in_bytes, const struct DinoTensor* inputs, size_t num_inputs,
                                               struct DinoTensor* outputs, size_t num_outputs, const void* device_out, void* host_out,
                                               size_t out_bytes);
/* Host-side float32 <-> bfloat16 conversion (round to nearest even as src/dinoml/ir.py:68-73; numpy has no bfloat16). */
DINOML_B200_API void dino_convert_f32_to_bf16(const float* src, uint16_t* dst, size_t count);
DINOML_B200_API void dino_convert_bf16_to_f32(const uint16_t* src, float* dst, size_t count);
/* :1011-1170 - warm-ups, CUDA-graph capture of one run on the owned stream, then per-iteration
 * event / graph launch / event; elapsed milliseconds per measured run are written to out_elapsed_ms. */
DINOML_B200_API int dino_session_benchmark(struct DinoSession* session, const struct DinoTensor* inputs, size_t num_inputs,
                                           struct DinoTensor* outputs, size_t num_outputs, size_t warmup_runs,
                                           size_t measured_runs, double* out_elapsed_ms, size_t out_elapsed_count);

#ifdef __cplusplus
}
#endif
#endif /* DINOML_B200_RUNTIME_H_ */
