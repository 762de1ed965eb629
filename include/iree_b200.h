/* C ABI of libiree_b200.so: the B200 (sm_100a) drop-in for IREE's contraction dispatches.
 *
 * Two layers, both plain C (pointers and sizes only):
 *
 *  1. A mirror of the slice of the HAL C API that a compiled IREE program drives when it
 *     runs a dispatch that carries an external CUDA object: executable creation from an
 *     `ExecutableDef` flatbuffer, push constants, descriptor sets, dispatch (cuLaunchKernel
 *     with "bindings first, then one 32-bit parameter per constant"), transfers, and the
 *     collective channel. Function names follow the reference's with the driver infix
 *     `b200`; every declaration cites the reference interface it stands in for. Paths are
 *     relative to the reference checkout.
 *
 *  2. Operator-level entry points, one per contraction dispatch family, that perform what the
 *     compiler plugin's rewritten host program performs for that dispatch (pick the export,
 *     fill the push constants, bind the buffers, dispatch). These are what a foreign-function
 *     binding would call.
 *
 * Errors: every function returns an `iree_b200_status_t` whose values are the reference's
 * `iree_status_code_t` (runtime/src/iree/base/status.h:79-125); 0 is OK. The message of the
 * most recent failure on the calling thread is available from iree_b200_last_error().
 * There is no CPU fallback anywhere: without a CUDA device every compute call fails with
 * IREE_B200_STATUS_UNAVAILABLE.
 */
#ifndef IREE_B200_H_
#define IREE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t iree_b200_status_t;
enum {
  IREE_B200_STATUS_OK = 0,
  IREE_B200_STATUS_UNKNOWN = 2,
  IREE_B200_STATUS_INVALID_ARGUMENT = 3,
  IREE_B200_STATUS_DEADLINE_EXCEEDED = 4,
  IREE_B200_STATUS_NOT_FOUND = 5,
  IREE_B200_STATUS_PERMISSION_DENIED = 7,
  IREE_B200_STATUS_RESOURCE_EXHAUSTED = 8,
  IREE_B200_STATUS_FAILED_PRECONDITION = 9,
  IREE_B200_STATUS_OUT_OF_RANGE = 11,
  IREE_B200_STATUS_UNIMPLEMENTED = 12,
  IREE_B200_STATUS_INTERNAL = 13,
  IREE_B200_STATUS_UNAVAILABLE = 14,
  IREE_B200_STATUS_DATA_LOSS = 15,
};

/* Message of the last non-OK status returned on this thread ("" if none). */
const char* iree_b200_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Limits of the CUDA HAL driver's pipeline layout
 * (runtime/src/iree/hal/drivers/cuda/pipeline_layout.h:19-28).
 * ---------------------------------------------------------------------------------------- */
#define IREE_HAL_B200_MAX_DESCRIPTOR_SET_COUNT 4
#define IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT 16
#define IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT 64

typedef struct iree_hal_b200_device_t iree_hal_b200_device_t;
typedef struct iree_hal_b200_executable_t iree_hal_b200_executable_t;
typedef struct iree_hal_b200_command_buffer_t iree_hal_b200_command_buffer_t;
typedef struct iree_hal_b200_channel_t iree_hal_b200_channel_t;
typedef struct iree_hal_b200_graph_t iree_hal_b200_graph_t;
typedef struct iree_hal_b200_descriptor_set_layout_t iree_hal_b200_descriptor_set_layout_t;
typedef struct iree_hal_b200_pipeline_layout_t iree_hal_b200_pipeline_layout_t;
typedef struct iree_hal_b200_semaphore_t iree_hal_b200_semaphore_t;

/* ---- device -------------------------------------------------------------------------------
 * Stands in for iree_hal_cuda_driver_create + device creation
 * (runtime/src/iree/hal/drivers/cuda/api.h:59-125, cuda_device.c). Loads libcuda.so at run
 * time like cuda_dynamic_symbols.c, retains the device's primary context (so pointers from
 * other libraries in the process are usable) and creates the dispatch stream. */
iree_b200_status_t iree_hal_b200_device_create(int32_t ordinal, iree_hal_b200_device_t** out_device);
void iree_hal_b200_device_release(iree_hal_b200_device_t* device);
/* Name, SM count, compute capability (major*10+minor) and opt-in shared memory per block. */
iree_b200_status_t iree_hal_b200_device_query(iree_hal_b200_device_t* device, char* name, size_t name_capacity,
                                              int32_t* out_sm_count, int32_t* out_compute_capability,
                                              int32_t* out_max_shared_memory);
/* Blocks until everything queued on the dispatch stream has finished
 * (the fence wait of runtime/src/iree/tooling/run_module.c:251-297). */
iree_b200_status_t iree_hal_b200_device_synchronize(iree_hal_b200_device_t* device);
/* The dispatch CUstream, for callers that interleave their own work (graph capture, NCCL). */
void* iree_hal_b200_device_stream(iree_hal_b200_device_t* device);

/* ---- timing events --------------------------------------------------------------------------
 * CUevent pairs recorded on the dispatch stream, what the driver's tracing context wraps around
 * each dispatch (runtime/src/iree/hal/drivers/cuda/tracing.h; stream_command_buffer.c:519-524).
 * elapsed_ms waits for `end`. */
iree_b200_status_t iree_hal_b200_event_create(iree_hal_b200_device_t* device, void** out_event);
void iree_hal_b200_event_release(iree_hal_b200_device_t* device, void* event);
iree_b200_status_t iree_hal_b200_event_record(iree_hal_b200_device_t* device, void* event);
iree_b200_status_t iree_hal_b200_event_elapsed_ms(iree_hal_b200_device_t* device, void* start, void* end,
                                                  float* out_ms);

/* ---- buffers ------------------------------------------------------------------------------
 * iree_hal_allocator_allocate_buffer / iree_hal_device_transfer_h2d / _d2h
 * (runtime/src/iree/hal/drivers/cuda/cuda_allocator.c; hal/device.h). Buffers are raw device
 * pointers, which is what the driver resolves bindings to before a launch
 * (stream_command_buffer.c:488-491). Transfers are queued on the dispatch stream. */
iree_b200_status_t iree_hal_b200_buffer_allocate(iree_hal_b200_device_t* device, size_t byte_length,
                                                 void** out_device_ptr);
iree_b200_status_t iree_hal_b200_buffer_free(iree_hal_b200_device_t* device, void* device_ptr);
iree_b200_status_t iree_hal_b200_host_allocate(iree_hal_b200_device_t* device, size_t byte_length,
                                               void** out_pinned_host_ptr);
iree_b200_status_t iree_hal_b200_host_free(iree_hal_b200_device_t* device, void* pinned_host_ptr);
iree_b200_status_t iree_hal_b200_transfer_h2d(iree_hal_b200_device_t* device, const void* source,
                                              void* target_device_ptr, size_t byte_length);
iree_b200_status_t iree_hal_b200_transfer_d2h(iree_hal_b200_device_t* device, const void* source_device_ptr,
                                              void* target, size_t byte_length);
iree_b200_status_t iree_hal_b200_fill_buffer(iree_hal_b200_device_t* device, void* device_ptr, size_t byte_length,
                                             uint8_t pattern);

/* ---- executable container -------------------------------------------------------------------
 * Writer for the `ExecutableDef` flatbuffer (file identifier "CUDA",
 * runtime/src/iree/schemas/cuda_executable_def.fbs:10-50), i.e. what
 * CUDATargetBackend::serializeExecutable emits for an external object
 * (compiler/plugins/target/CUDA/CUDATarget.cpp:523-550,665-699): entry names taken verbatim,
 * one block size and one dynamic shared-memory size per entry, the cubin bytes as `ptx_image`.
 * Call with out_data == NULL to query the size. */
iree_b200_status_t iree_b200_executable_def_build(int32_t entry_count, const char* const* entry_names,
                                                  const uint32_t* block_sizes_xyz,
                                                  const uint32_t* shared_memory_sizes, const void* image,
                                                  size_t image_size, void* out_data, size_t out_capacity,
                                                  size_t* out_size);

/* The ExecutableDef of the contraction cubin: every export of the file with the block size and
 * dynamic shared-memory size its kernel needs (what the compiler plugin records per
 * hal.executable.export). Needs no GPU. Call with out_data == NULL to query the size. */
iree_b200_status_t iree_b200_contraction_executable_def(const char* cubin_path, void* out_data, size_t out_capacity,
                                                        size_t* out_size);

/* iree_hal_executable_cache_prepare_executable for format "PTXE"
 * (runtime/src/iree/hal/drivers/cuda/nop_executable_cache.c:76-93,
 * native_executable.c:55-272): verifies the flatbuffer (non-empty entry names, as many block
 * sizes as entries, non-empty image), loads the image with cuModuleLoadDataEx, resolves every
 * entry and raises its dynamic shared-memory limit, rejecting sizes above the device maximum. */
iree_b200_status_t iree_hal_b200_executable_create(iree_hal_b200_device_t* device, const char* executable_format,
                                                   const void* executable_data, size_t executable_data_size,
                                                   iree_hal_b200_executable_t** out_executable);
void iree_hal_b200_executable_release(iree_hal_b200_executable_t* executable);
int32_t iree_hal_b200_executable_entry_count(const iree_hal_b200_executable_t* executable);
/* Ordinal of the named entry point, or -1. */
int32_t iree_hal_b200_executable_lookup(const iree_hal_b200_executable_t* executable, const char* entry_name);

/* ---- command buffer (stream mode) --------------------------------------------------------------
 * iree_hal_command_buffer_{create,push_constants,push_descriptor_set,dispatch,
 * execution_barrier,collective} as implemented by the CUDA stream command buffer
 * (runtime/src/iree/hal/command_buffer.h:658-710;
 * runtime/src/iree/hal/drivers/cuda/stream_command_buffer.c:427-610). Commands execute on the
 * device's dispatch stream in recording order. A command buffer is recorded by one thread
 * at a time. */
typedef struct {
  uint32_t binding;   /* slot within the set */
  void* device_ptr;   /* already offset, as the driver passes it */
} iree_hal_b200_descriptor_set_binding_t;

iree_b200_status_t iree_hal_b200_command_buffer_create(iree_hal_b200_device_t* device,
                                                       iree_hal_b200_command_buffer_t** out_command_buffer);
void iree_hal_b200_command_buffer_release(iree_hal_b200_command_buffer_t* command_buffer);
/* offset and values_length are in bytes and must be multiples of 4. */
iree_b200_status_t iree_hal_b200_command_buffer_push_constants(iree_hal_b200_command_buffer_t* command_buffer,
                                                               size_t offset, const void* values,
                                                               size_t values_length);
iree_b200_status_t iree_hal_b200_command_buffer_push_descriptor_set(
    iree_hal_b200_command_buffer_t* command_buffer, uint32_t set, size_t binding_count,
    const iree_hal_b200_descriptor_set_binding_t* bindings);
/* Launches entry_point with kernel parameters = the bound pointers of set 0 (slots
 * 0..binding_count-1), then constant_count 32-bit constants, each a separate parameter. */
iree_b200_status_t iree_hal_b200_command_buffer_dispatch(iree_hal_b200_command_buffer_t* command_buffer,
                                                         iree_hal_b200_executable_t* executable, int32_t entry_point,
                                                         uint32_t binding_count, uint32_t constant_count,
                                                         uint32_t workgroup_x, uint32_t workgroup_y,
                                                         uint32_t workgroup_z);
/* iree_hal_command_buffer_begin / _end (runtime/src/iree/hal/command_buffer.h:532-540): bracket a
 * recording. Optional here (the other commands do not require them); FAILED_PRECONDITION when
 * unpaired. */
iree_b200_status_t iree_hal_b200_command_buffer_begin(iree_hal_b200_command_buffer_t* command_buffer);
iree_b200_status_t iree_hal_b200_command_buffer_end(iree_hal_b200_command_buffer_t* command_buffer);
/* iree_hal_command_buffer_execution_barrier (command_buffer.h:563-571; the CUDA driver's is a no-op
 * on its in-order stream, stream_command_buffer.c:234-250, and a plain dependency between graph
 * nodes). Commands here already execute in recording order; what the barrier adds is that the dispatch
 * after it is not launched early under set_dispatch_overlap. The masks and flags are accepted and
 * ignored, as the reference's driver does; memory / buffer barrier lists are not taken. */
iree_b200_status_t iree_hal_b200_command_buffer_execution_barrier(iree_hal_b200_command_buffer_t* command_buffer,
                                                                  uint32_t source_stage_mask, uint32_t target_stage_mask,
                                                                  uint32_t flags);
/* iree_hal_command_buffer_fill_buffer (command_buffer.h:623-627; stream_command_buffer.c:300-340):
 * pattern_length 1, 2 or 4; offset and length aligned to it. Stream mode: cuMemsetD{8,16,32}Async;
 * graph mode: a memset node. */
iree_b200_status_t iree_hal_b200_command_buffer_fill_buffer(iree_hal_b200_command_buffer_t* command_buffer,
                                                            void* target_device_ptr, size_t target_offset, size_t length,
                                                            const void* pattern, size_t pattern_length);
/* iree_hal_command_buffer_copy_buffer (command_buffer.h:650-654; stream_command_buffer.c:396-425),
 * device to device; the ranges must not overlap. Stream mode: cuMemcpyDtoDAsync; graph mode: a memcpy
 * node. */
iree_b200_status_t iree_hal_b200_command_buffer_copy_buffer(iree_hal_b200_command_buffer_t* command_buffer,
                                                            const void* source_device_ptr, size_t source_offset,
                                                            void* target_device_ptr, size_t target_offset, size_t length);
/* Descriptor-set and pipeline layouts (runtime/src/iree/hal/drivers/cuda/pipeline_layout.c:47-80 and
 * :145-190): a set layout is its binding count; a pipeline layout records every set's count -- the
 * kernel parameters of a dispatch are the bindings of set 0, then of set 1, ..., each set starting at
 * the running sum of the counts before it -- and the push constant count, whose parameters follow the
 * last set. The pipeline layout copies the counts; set layouts may be released after it was created. */
iree_b200_status_t iree_hal_b200_descriptor_set_layout_create(iree_hal_b200_device_t* device, uint32_t binding_count,
                                                              iree_hal_b200_descriptor_set_layout_t** out_layout);
void iree_hal_b200_descriptor_set_layout_release(iree_hal_b200_descriptor_set_layout_t* layout);
iree_b200_status_t iree_hal_b200_pipeline_layout_create(iree_hal_b200_device_t* device, uint32_t push_constant_count,
                                                        uint32_t set_layout_count,
                                                        iree_hal_b200_descriptor_set_layout_t* const* set_layouts,
                                                        iree_hal_b200_pipeline_layout_t** out_layout);
void iree_hal_b200_pipeline_layout_release(iree_hal_b200_pipeline_layout_t* layout);
/* iree_hal_command_buffer_dispatch with the executable's pipeline layout (stream_command_buffer.c:530-603):
 * parameters = every set's bound pointers in set order, then the layout's push constants. */
iree_b200_status_t iree_hal_b200_command_buffer_dispatch_with_layout(iree_hal_b200_command_buffer_t* command_buffer,
                                                                     iree_hal_b200_executable_t* executable,
                                                                     int32_t entry_point,
                                                                     const iree_hal_b200_pipeline_layout_t* layout,
                                                                     uint32_t workgroup_x, uint32_t workgroup_y,
                                                                     uint32_t workgroup_z);
/* Number of kernel launches this command buffer has issued (for launch accounting). */
uint64_t iree_hal_b200_command_buffer_launch_count(const iree_hal_b200_command_buffer_t* command_buffer);
/* Dispatch overlap (programmatic dependent launch; no counterpart in the reference's CUDA driver,
 * which serialises dispatches of a stream, stream_command_buffer.c:500-610). While enabled, a
 * dispatch is launched (stream mode) or recorded (graph mode) so that the device may start it
 * before the dispatch ahead of it has finished. Only exports that order themselves on the device
 * may be dispatched this way: they call griddepcontrol.wait before reading anything an earlier
 * kernel may write and before writing anything. Of this library's exports those are
 * b200_w4a16_decode_m8 / _m16, which prefetch weight tiles ahead of the wait: the caller vouches
 * that weights and scales are not written by the dispatch ahead. UNAVAILABLE when the driver
 * lacks the feature. */
iree_b200_status_t iree_hal_b200_command_buffer_set_dispatch_overlap(iree_hal_b200_command_buffer_t* command_buffer,
                                                                     int32_t enable);

/* ---- graph mode ------------------------------------------------------------------------------------
 * The CUDA-graph command buffer of the reference (--cuda_use_streams=false,
 * runtime/src/iree/hal/drivers/cuda/graph_command_buffer.c:747-829): between begin_graph and
 * end_graph every dispatch is recorded as a kernel node (same parameter packing), each node
 * depending on the previous one; graph_execute replays the whole recording on the dispatch stream
 * with one cuGraphLaunch. Collectives are not recordable here. */
iree_b200_status_t iree_hal_b200_command_buffer_begin_graph(iree_hal_b200_command_buffer_t* command_buffer);
iree_b200_status_t iree_hal_b200_command_buffer_end_graph(iree_hal_b200_command_buffer_t* command_buffer,
                                                          iree_hal_b200_graph_t** out_graph);
iree_b200_status_t iree_hal_b200_graph_execute(iree_hal_b200_command_buffer_t* command_buffer,
                                               iree_hal_b200_graph_t* graph);
void iree_hal_b200_graph_release(iree_hal_b200_graph_t* graph);

/* ---- resources, semaphores, queue submission --------------------------------------------------------
 * Executables, command buffers, channels and semaphores are reference counted like the reference's
 * iree_hal_resource_t (runtime/src/iree/hal/resource.h; drivers/cuda/native_executable.c:21-25): created
 * with one reference, `retain` adds one, `release` drops one and destroys the object with the last. */
void iree_hal_b200_executable_retain(iree_hal_b200_executable_t* executable);
void iree_hal_b200_command_buffer_retain(iree_hal_b200_command_buffer_t* command_buffer);
void iree_hal_b200_channel_retain(iree_hal_b200_channel_t* channel);
/* Timeline semaphores (runtime/src/iree/hal/semaphore.h:60-140): a 64-bit payload that only grows, advanced
 * by the host (`signal`; OUT_OF_RANGE unless the value grows) or by the device when it passes the point
 * behind which queue_execute queued the signal. `wait` returns OK once the payload is at least `value`,
 * DEADLINE_EXCEEDED after timeout_ms (negative: no limit). */
iree_b200_status_t iree_hal_b200_semaphore_create(iree_hal_b200_device_t* device, uint64_t initial_value,
                                                  iree_hal_b200_semaphore_t** out_semaphore);
void iree_hal_b200_semaphore_retain(iree_hal_b200_semaphore_t* semaphore);
void iree_hal_b200_semaphore_release(iree_hal_b200_semaphore_t* semaphore);
iree_b200_status_t iree_hal_b200_semaphore_query(iree_hal_b200_semaphore_t* semaphore, uint64_t* out_value);
iree_b200_status_t iree_hal_b200_semaphore_signal(iree_hal_b200_semaphore_t* semaphore, uint64_t new_value);
iree_b200_status_t iree_hal_b200_semaphore_wait(iree_hal_b200_semaphore_t* semaphore, uint64_t value, int64_t timeout_ms);
/* iree_hal_device_queue_execute (runtime/src/iree/hal/device.h; drivers/cuda/cuda_device.c): once every wait
 * semaphore has reached its value, the recorded graphs run in order on the dispatch stream, then every
 * signal semaphore is advanced to its value. A wait on a value that a queued device signal will reach
 * costs the host nothing (the stream waits for it); a wait only a later host signal can satisfy holds this
 * call, for ten seconds at most (DEADLINE_EXCEEDED). With no graphs this is a queue barrier. */
iree_b200_status_t iree_hal_b200_device_queue_execute(iree_hal_b200_device_t* device, size_t wait_count,
                                                      iree_hal_b200_semaphore_t* const* wait_semaphores,
                                                      const uint64_t* wait_values, size_t signal_count,
                                                      iree_hal_b200_semaphore_t* const* signal_semaphores,
                                                      const uint64_t* signal_values, size_t graph_count,
                                                      iree_hal_b200_graph_t* const* graphs);

/* ---- collective channel -------------------------------------------------------------------------
 * iree_hal_channel_create with explicit {id, rank, count}
 * (runtime/src/iree/hal/channel.h:40-108; cuda_device.c:439-530; nccl_channel.c:94-160) over
 * NCCL loaded at run time (nccl_dynamic_symbols.c). One process drives one device per rank. */
#define IREE_HAL_B200_CHANNEL_ID_SIZE 128
iree_b200_status_t iree_hal_b200_channel_create_id(void* out_id, size_t id_capacity); /* ncclGetUniqueId */
iree_b200_status_t iree_hal_b200_channel_create(iree_hal_b200_device_t* device, const void* id, size_t id_size,
                                                int32_t rank, int32_t count,
                                                iree_hal_b200_channel_t** out_channel);
void iree_hal_b200_channel_release(iree_hal_b200_channel_t* channel);
/* iree_hal_channel_split (runtime/src/iree/hal/channel.h:85-96; drivers/cuda/nccl_channel.c:176-215, ncclCommSplit):
 * every rank of base_channel calls it; ranks with the same non-negative color form a channel, ordered
 * by key. A negative color (IREE_HAL_CHANNEL_NO_COLOR) takes part in the call and yields *out_channel
 * = NULL. UNAVAILABLE with an NCCL older than 2.18. */
iree_b200_status_t iree_hal_b200_channel_split(iree_hal_b200_channel_t* base_channel, int32_t color, int32_t key,
                                               iree_hal_b200_channel_t** out_channel);
int32_t iree_hal_b200_channel_rank(const iree_hal_b200_channel_t* channel);
int32_t iree_hal_b200_channel_count(const iree_hal_b200_channel_t* channel);

enum { /* element types the contraction path gathers (hal/command_buffer.h collective element types) */
  IREE_HAL_B200_ELEMENT_TYPE_I8 = 0,
  IREE_HAL_B200_ELEMENT_TYPE_F16 = 1,
  IREE_HAL_B200_ELEMENT_TYPE_I32 = 2,
  IREE_HAL_B200_ELEMENT_TYPE_F32 = 3,
  IREE_HAL_B200_ELEMENT_TYPE_BF16 = 4,
};
/* IREE_HAL_COLLECTIVE_KIND_ALL_GATHER through iree_hal_command_buffer_collective
 * (hal/command_buffer.h:658-663; nccl_channel.c:342-359): every rank contributes element_count
 * elements; recv holds count * element_count, ordered by rank. */
iree_b200_status_t iree_hal_b200_command_buffer_all_gather(iree_hal_b200_command_buffer_t* command_buffer,
                                                           iree_hal_b200_channel_t* channel, int32_t element_type,
                                                           const void* send_device_ptr, void* recv_device_ptr,
                                                           size_t element_count);

/* iree_hal_command_buffer_collective for the other kinds (hal/command_buffer.h:215-335; submitted as
 * the reference's NCCL channel does, drivers/cuda/nccl_channel.c:327-500). `kind` and `reduction` take the
 * reference's enum values. `param`: the root rank (BROADCAST, REDUCE), the peer (SEND, RECV), or for
 * SEND_RECV the rank to send to in the low and the rank to receive from in the high 16 bits. element_count:
 * per rank for ALL_GATHER and REDUCE_SCATTER (what a rank contributes / receives), the whole buffer for
 * ALL_REDUCE, ALL_TO_ALL (count / ranks elements per peer), BROADCAST, REDUCE, SEND, RECV. Not recordable
 * into a graph. */
enum {
  IREE_HAL_B200_COLLECTIVE_ALL_GATHER = 0,
  IREE_HAL_B200_COLLECTIVE_ALL_REDUCE = 1,
  IREE_HAL_B200_COLLECTIVE_ALL_TO_ALL = 2,
  IREE_HAL_B200_COLLECTIVE_BROADCAST = 3,
  IREE_HAL_B200_COLLECTIVE_REDUCE = 4,
  IREE_HAL_B200_COLLECTIVE_REDUCE_SCATTER = 5,
  IREE_HAL_B200_COLLECTIVE_SEND = 6,
  IREE_HAL_B200_COLLECTIVE_RECV = 7,
  IREE_HAL_B200_COLLECTIVE_SEND_RECV = 8,
};
enum {
  IREE_HAL_B200_REDUCTION_NONE = 0,
  IREE_HAL_B200_REDUCTION_SUM = 1,
  IREE_HAL_B200_REDUCTION_PRODUCT = 2,
  IREE_HAL_B200_REDUCTION_MINIMUM = 3,
  IREE_HAL_B200_REDUCTION_MAXIMUM = 4,
  IREE_HAL_B200_REDUCTION_AVERAGE = 5,
};
iree_b200_status_t iree_hal_b200_command_buffer_collective(iree_hal_b200_command_buffer_t* command_buffer,
                                                           iree_hal_b200_channel_t* channel, int32_t kind,
                                                           int32_t reduction, int32_t element_type, uint32_t param,
                                                           const void* send_device_ptr, void* recv_device_ptr,
                                                           size_t element_count);

/* Device memory of other ranks (processes) of the same node. `export` yields an opaque
 * IREE_HAL_B200_PEER_HANDLE_SIZE-byte handle for a buffer allocated here; the owner ships it to
 * its peers by any means and they `import` it, which gives a device pointer valid in the
 * importing process (NVLink / NVSwitch peer access), to be released with `unimport` before the
 * owner frees the buffer. (The reference has no counterpart: its collectives go through NCCL only,
 * runtime/src/iree/hal/drivers/cuda/nccl_channel.c.) */
#define IREE_HAL_B200_PEER_HANDLE_SIZE 64
iree_b200_status_t iree_hal_b200_buffer_export(iree_hal_b200_device_t* device, void* device_ptr, void* out_handle);
iree_b200_status_t iree_hal_b200_buffer_import(iree_hal_b200_device_t* device, const void* handle, void** out_device_ptr);
iree_b200_status_t iree_hal_b200_buffer_unimport(iree_hal_b200_device_t* device, void* device_ptr);
/* All-gather by peer copies: this rank's `byte_count` bytes go into slot `rank` of every rank's
 * receive buffer (recv_device_ptrs[p] = rank p's buffer as imported here; the entry of this rank
 * is its own buffer) through the copy engines, on the collective stream, after everything
 * recorded on the dispatch stream so far; a channel barrier follows on the same stream, so that
 * iree_hal_b200_command_buffer_join_collectives() orders the dispatch stream after the arrival
 * of every rank's block in this rank's buffer. No SM takes part, which is what lets it run
 * beside the persistent dispatches. */
iree_b200_status_t iree_hal_b200_command_buffer_all_gather_peer_copies(iree_hal_b200_command_buffer_t* command_buffer,
                                                                        iree_hal_b200_channel_t* channel,
                                                                        const void* send_device_ptr, size_t byte_count,
                                                                        void* const* recv_device_ptrs);
/* The same collective on the device's second stream: it starts when everything recorded before it
 * has run, and dispatches recorded after it do not wait for it (the reference keeps a second
 * stream beside the dispatch stream as well, cuda_device.c). join_collectives makes the dispatch
 * stream wait for every overlapped collective issued so far; call it before a buffer that a
 * collective reads or writes is reused, and before reading results. */
iree_b200_status_t iree_hal_b200_command_buffer_all_gather_overlapped(iree_hal_b200_command_buffer_t* command_buffer,
                                                                      iree_hal_b200_channel_t* channel,
                                                                      int32_t element_type, const void* send_device_ptr,
                                                                      void* recv_device_ptr, size_t element_count);
iree_b200_status_t iree_hal_b200_command_buffer_join_collectives(iree_hal_b200_command_buffer_t* command_buffer);

/* ------------------------------------------------------------------------------------------
 * Operator level: the contraction dispatches.
 * ---------------------------------------------------------------------------------------- */
typedef struct iree_b200_context_t iree_b200_context_t;

/* Creates the device, loads the contraction executable (an ExecutableDef wrapped around the
 * sm_100a cubin found at cubin_path) and a command buffer. */
iree_b200_status_t iree_b200_context_create(int32_t device_ordinal, const char* cubin_path,
                                            iree_b200_context_t** out_context);
void iree_b200_context_release(iree_b200_context_t* context);
iree_hal_b200_device_t* iree_b200_context_device(iree_b200_context_t* context);
iree_hal_b200_executable_t* iree_b200_context_executable(iree_b200_context_t* context);
iree_hal_b200_command_buffer_t* iree_b200_context_command_buffer(iree_b200_context_t* context);

enum { IREE_B200_KIND_F16 = 0, IREE_B200_KIND_BF16 = 1, IREE_B200_KIND_I8 = 2 };
enum {
  IREE_B200_EPILOGUE_CAST = 0,        /* accumulator -> input element type (f16 / bf16): truncf consumer */
  IREE_B200_EPILOGUE_ACCUMULATOR = 1, /* raw f32 / i32 accumulator */
  IREE_B200_EPILOGUE_REQUANT_F16 = 2, /* i8 only: f16(f32(acc) * row_scale[m] * col_scale[n]) */
};
enum {
  IREE_B200_RHS_KN = 0, /* rhs is [batch, K, N] row-major: linalg.matmul / batch_matmul */
  IREE_B200_RHS_NK = 1, /* rhs is [batch, N, K] row-major: matmul_transpose_b / mmt */
};
enum {
  IREE_B200_FLAG_FORCE_GENERIC = 1,      /* use the shape-agnostic SIMT kernel */
  IREE_B200_FLAG_DEVICE_TENSORMAPS = 2,  /* build the tensor maps with the b200_encode_tensormaps dispatch */
  IREE_B200_FLAG_PAIR_CTAS = 4,          /* force the CTA-pair kernels (256-row tiles, cta_group::2) */
  IREE_B200_FLAG_SINGLE_CTA = 8,         /* force the single-CTA kernels (128-row tiles) */
  IREE_B200_FLAG_SPLIT_K = 16,           /* the workspace has iree_b200_matmul_workspace_bytes() bytes: a product of
                                            few rows (M <= 32) cuts every tile's K range into the number of work
                                            items given in bits 8..11 (1..15; 0 = no split, which is the faster
                                            choice on every shape measured so far) */
};
#define IREE_B200_WORKSPACE_BYTES 512

typedef struct {
  int32_t kind;      /* IREE_B200_KIND_* */
  int32_t epilogue;  /* IREE_B200_EPILOGUE_* */
  int32_t M, N, K, batch;
  int32_t rhs_layout; /* IREE_B200_RHS_* */
  int32_t tile_n;     /* 0 = choose */
  int32_t flags;
} iree_b200_matmul_params_t;

/* linalg.matmul / linalg.batch_matmul dispatch (fill + contraction + elementwise consumer, as
 * formed by compiler/src/iree/compiler/Dialect/Flow/Transforms/FormDispatchRegions.cpp:224-246,
 * 534-620); on the reference's CPU path this is pack + iree_uk_mmt4d + unpack
 * (runtime/src/iree/builtins/ukernel/mmt4d.h:14-21). All pointers are device pointers;
 * `workspace` is IREE_B200_WORKSPACE_BYTES of device memory, 128-byte aligned, owned by the
 * caller and not shared between dispatches in flight. Queues work and returns. */
iree_b200_status_t iree_b200_matmul(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                    const void* lhs, const void* rhs, void* out, const float* row_scale,
                                    const float* col_scale, void* workspace);
/* Bytes of workspace a product needs: IREE_B200_WORKSPACE_BYTES, or more when
 * IREE_B200_FLAG_SPLIT_K is set and the product qualifies (tile counters and one partial
 * accumulator per tile and split behind the header). */
size_t iree_b200_matmul_workspace_bytes(iree_b200_context_t* context, const iree_b200_matmul_params_t* params);
/* The same in two steps: prepare() writes the tensor maps and clears the status words (and the
 * tile counters of a split product); run() only dispatches the kernel and may be repeated while
 * operands stay in place. With a split, out_tile_n carries the number of splits minus one in its
 * upper 16 bits; run() wants it back as it is. */
iree_b200_status_t iree_b200_matmul_prepare(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                            const void* lhs, const void* rhs, void* workspace, int32_t* out_tile_n);
iree_b200_status_t iree_b200_matmul_run(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                        const void* lhs, const void* rhs, void* out, const float* row_scale,
                                        const float* col_scale, void* workspace, int32_t tile_n);
/* Synchronises and returns the device-side status words of a workspace: DEADLINE_EXCEEDED if a
 * bounded wait inside the kernel ran out, INVALID_ARGUMENT if the kernel refused its arguments. */
iree_b200_status_t iree_b200_workspace_status(iree_b200_context_t* context, const void* workspace);

/* Host-buffer form of the same dispatch: copies operands in, runs, copies the result out and
 * waits, i.e. what iree-run-module does around one invocation
 * (runtime/src/iree/tooling/run_module.c:199-322). */
iree_b200_status_t iree_b200_matmul_host(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                         const void* lhs, const void* rhs, void* out, const float* row_scale,
                                         const float* col_scale);

/* Host-side tensor-map encoding (cuTensorMapEncodeTiled) for a rank-3 row-major tensor
 * [dim2, dim1, dim0] with 128-byte swizzle; writes 128 bytes to out_map (host memory). */
iree_b200_status_t iree_b200_encode_tensor_map(iree_b200_context_t* context, int32_t elem_bytes, int32_t is_bf16,
                                               const void* device_ptr, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                               uint32_t box0, uint32_t box1, void* out_map);

/* The tensor-map templates the device-side builders start from (exports b200_encode_tensormaps and
 * b200_encode_tensormap): one 128-byte map per kind, each fixing element type, rank, swizzle and fill
 * mode; the builders patch address, extents, strides and box. A stock runtime never calls
 * cuTensorMapEncodeTiled (runtime/src/iree/hal/drivers/cuda/cuda_dynamic_symbol_table.h), so the
 * compiler plugin embeds these bytes as a constant. Writes IREE_B200_TEMPLATE_COUNT * 128 bytes. */
enum {
  IREE_B200_TEMPLATE_F16_SWIZZLE128_RANK3 = 0,  /* f16 operands of the tcgen05 kernels */
  IREE_B200_TEMPLATE_BF16_SWIZZLE128_RANK3 = 1,
  IREE_B200_TEMPLATE_U8_SWIZZLE128_RANK3 = 2,   /* i8 operands */
  IREE_B200_TEMPLATE_U8_SWIZZLE64_RANK3 = 3,    /* raw int4 weight tiles of the W4A16 tensor-core kernels */
  IREE_B200_TEMPLATE_F16_PLAIN_RANK2 = 4,       /* result tiles stored by b200_w4a16_gemm_wt */
  IREE_B200_TEMPLATE_U64_PLAIN_RANK2 = 5,       /* int4 weight rows of the decode kernels when K > 4096 */
  IREE_B200_TEMPLATE_COUNT = 6,
};
iree_b200_status_t iree_b200_tensormap_templates(iree_b200_context_t* context, void* out_templates);

/* ---- fused int4 dequant + matmul (W4A16) -------------------------------------------------------
 * The dispatch that dispatch formation builds by cloning the dequantisation generic into its
 * consumer contraction (compiler/src/iree/compiler/Dialect/Flow/Transforms/RegionOpUtils.cpp:530-610,
 * pinned by Dialect/Flow/Transforms/test/pipeline_tests.mlir:53-99): group-wise scaled int4
 * weights [N, K/2] bytes (element 2i in the low nibble of byte i,
 * runtime/src/iree/builtins/ukernel/mmt4d_tile_generic.c:35-44), f16 scales [N, K/group], f16
 * activations [M, K], f16 result. The result is written at out[m * ldo + n_offset + n], so a rank
 * that owns a slice of N writes into the full-width buffer (ldo = N, n_offset = 0 otherwise). */
enum {
  IREE_B200_W4A16_AUTO = 0,
  IREE_B200_W4A16_DECODE = 1,  /* M <= 16, N % 16 == 0, K % 256 == 0, K <= 16384, group 128, and `a`, `wq`,
                                  `scales` on 16-byte boundaries (INVALID_ARGUMENT otherwise; AUTO then
                                  picks another variant): weight streaming */
  IREE_B200_W4A16_GEMM = 2,    /* group 128, K % 128 == 0: tcgen05 with in-kernel dequantisation */
  IREE_B200_W4A16_GENERIC = 3, /* anything else */
  IREE_B200_W4A16_GEMM_WT = 4, /* GEMM's preconditions, M >= 256, result base and pitch on 16-byte boundaries,
                                  n_offset % 8 == 0: tcgen05 with the dequantised weights as the tensor-memory
                                  operand, results leave through TMA stores */
  IREE_B200_W4A16_DECODE_TC = 5, /* M <= 16, K % 256 == 0, group 128, `a` and `wq` on 16-byte and `scales` on
                                  4-byte boundaries: weight streaming through the tensor cores (weights
                                  expanded into tensor memory, work dealt to the SMs in equal ranges of
                                  128-row x 256-K units); needs prepare() */
};
typedef struct {
  int32_t M, N, K;
  int32_t group_size;
  int32_t ldo;       /* output row pitch in elements */
  int32_t n_offset;  /* first output column */
  int32_t variant;   /* IREE_B200_W4A16_* */
  int32_t tile_n;    /* 0 = choose (tensor-core kernel only; else a multiple of 16 up to 128) */
} iree_b200_w4a16_params_t;
/* prepare() is what makes a workspace usable for run(): it writes the tensor maps of the tensor-core
 * variants and, for DECODE with K > 4096, the map over the weights together with a note of which
 * weights it describes; a DECODE dispatch on a workspace without that note (or with a note for other
 * weights) computes nothing and iree_b200_workspace_status reports INVALID_ARGUMENT. DECODE with
 * K <= 4096 and GENERIC need no prepare().
 * Device workspace the dispatch needs for an N-column weight matrix: tensor maps, status words
 * and the scratch the decode kernel uses when K > 4096 (a counter per 16-row tile and an f32
 * partial tile per tile and 4096-wide K slice). It must be zero-filled once after allocation;
 * the kernels leave the counters at zero. One workspace serves one dispatch in flight. */
size_t iree_b200_w4a16_workspace_bytes(int32_t N);
iree_b200_status_t iree_b200_w4a16(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                   const void* a, const void* wq, const void* scales, void* out, void* workspace);
iree_b200_status_t iree_b200_w4a16_prepare(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                           const void* a, const void* wq, const void* scales, const void* out,
                                           void* workspace, int32_t* out_variant, int32_t* out_tile_n);
iree_b200_status_t iree_b200_w4a16_run(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                       const void* a, const void* wq, const void* scales, void* out, void* workspace,
                                       int32_t variant, int32_t tile_n);
/* N-sharded form of the dispatch for the ranks of one channel (no counterpart in the reference, whose
 * programs follow the sharded dispatch with an all-gather collective,
 * runtime/src/iree/hal/drivers/cuda/nccl_channel.c:342-359): rank `rank` of `world` owns weight rows
 * [n_offset, n_offset + N) and its kernel stores its column block into EVERY rank's full-width
 * [M, ldo] result from its epilogue, so that no collective follows the dispatch.
 *   results[p]  rank p's result buffer as mapped into this process (iree_hal_b200_buffer_import; the
 *               entry of this rank is its own buffer); 16-byte aligned, ldo * 2 a multiple of 16;
 *   flags[p]    rank p's arrival words, `world` uint32 each, zero-filled once (mapped the same way);
 *   epoch       a value that grows with every use of this set of result buffers, starting at 1.
 * prepare_push writes the workspace (tensor maps of every destination, flag pointers); run_push
 * dispatches the kernel, which raises word `rank` of every rank's flags to `epoch` once all of its
 * stores have completed; wait_arrivals enqueues the consumer side on this rank: a small kernel that
 * returns when all `world` words of this rank's own flags have reached `epoch`. Its wait is bounded
 * (about two seconds): iree_b200_workspace_status(workspace) then reports DEADLINE_EXCEEDED.
 * Reuse rule: a rank may start the dispatch that overwrites a result buffer only after its own
 * wait_arrivals for the previous use of that buffer, and whatever reads a result on a rank must be
 * ordered on that rank's stream before its next dispatch into another buffer of the rotation (two
 * buffers in rotation are enough). Needs M >= 256 and the GEMM_WT preconditions. */
iree_b200_status_t iree_b200_w4a16_prepare_push(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                                const void* a, const void* wq, const void* scales,
                                                void* const* results, void* const* flags, int32_t world,
                                                int32_t rank, void* workspace);
iree_b200_status_t iree_b200_w4a16_run_push(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                            const void* scales, void* result, void* workspace, int32_t world,
                                            int32_t rank, int32_t epoch);
iree_b200_status_t iree_b200_w4a16_wait_arrivals(iree_b200_context_t* context, const void* own_flags, void* workspace,
                                                 int32_t world, int32_t epoch);
/* Host-buffer form (copies in, runs, copies out, waits). With ldo != N the existing contents of
 * `out` are uploaded first so that columns outside the slice survive. A many-rows product of tens of
 * megabytes (variant AUTO, M >= 256, N >= 2048 and a multiple of 8, group 128, ldo == N, weights +
 * result >= 32 MB) is run as up to 11 dispatches that follow the operands' arrival, with uploads,
 * kernels and pitched readbacks on three streams; the result is bit-identical to the single
 * dispatch's. Page-locked host buffers (iree_hal_b200_host_allocate) make the copies asynchronous. The
 * host-buffer calls copy and wait themselves: FAILED_PRECONDITION while a graph is being recorded. */
iree_b200_status_t iree_b200_w4a16_host(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                        const void* a, const void* wq, const void* scales, void* out);
/* The dispatches iree_b200_w4a16_host cuts `params` into (needs no device): writes up to `capacity` records
 * {row0, rows, col0, cols, uploads_rows, uploads_cols} - the rectangle of the result a dispatch computes and
 * which operand block goes up before it - and returns their number; 0 when the product runs as one dispatch,
 * -1 for invalid params. No counterpart in the reference (its HAL leaves transfers to the program). */
int32_t iree_b200_w4a16_host_plan(const iree_b200_w4a16_params_t* params, int32_t* out_units, int32_t capacity);

/* ---- sequences of dispatches ----------------------------------------------------------------------
 * `count` dispatches over rotating operand sets issued by one call, i.e. what the reference does
 * when a queue action replays a command buffer that holds that many dispatches
 * (runtime/src/iree/hal/drivers/cuda/pending_queue_actions.c:729-742). Step i uses set
 * (first + i) % set_count; every array has set_count entries (scale arrays may be NULL). */
iree_b200_status_t iree_b200_matmul_run_sequence(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                                 int32_t set_count, const void* const* lhs, const void* const* rhs,
                                                 void* const* out, const float* const* row_scale,
                                                 const float* const* col_scale, void* const* workspace,
                                                 int32_t tile_n, int32_t first, int32_t count);
iree_b200_status_t iree_b200_w4a16_run_sequence(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                                int32_t set_count, const void* const* a, const void* const* wq,
                                                const void* const* scales, void* const* out, void* const* workspace,
                                                int32_t variant, int32_t tile_n, int32_t first, int32_t count);

/* Operator-level switch for the above: while enabled, the operator entry points dispatch the
 * exports that order themselves on the device with overlap, and every other export normally.
 * Off by default. */
iree_b200_status_t iree_b200_context_set_dispatch_overlap(iree_b200_context_t* context, int32_t enable);
/* The kernels are persistent: a dispatch fills every SM with one block for its whole duration, so
 * a collective enqueued on another stream (iree_hal_b200_command_buffer_all_gather_overlapped)
 * would only get SMs when the dispatch ends. Reserving `count` SMs makes the operator entry
 * points size their grids (and choose tiles) for the remaining ones, so that the collective's
 * blocks run beside the dispatch. 0 (the default) uses every SM. */
iree_b200_status_t iree_b200_context_set_reserved_sms(iree_b200_context_t* context, int32_t count);

/* ---- data-tiled entry points: pack / unpack / mmt4d -------------------------------------------
 *
 * The GPU counterparts of the three micro kernels llvm-cpu's data-tiled matmul is made of. The
 * argument lists are the reference's (runtime/src/iree/builtins/ukernel/pack.h:26-34,
 * unpack.h:17-25, mmt4d.h:14-21) with a context in front instead of `cpu_data` behind; buffers
 * are device pointers, sizes / strides / offsets are in elements, flags carry the reference's
 * bit values (exported_bits.h:29-83). Work is enqueued on the context's stream. */
#define IREE_B200_UK_FLAG_MMT4D_TYPE_MASK 0xFF
#define IREE_B200_UK_FLAG_MMT4D_TYPE_F32F32F32 0x01
#define IREE_B200_UK_FLAG_MMT4D_TYPE_S8S8S32 0x02
#define IREE_B200_UK_FLAG_MMT4D_TYPE_F16F16F32 0x03
#define IREE_B200_UK_FLAG_MMT4D_TYPE_F16F16F16 0x04
#define IREE_B200_UK_FLAG_MMT4D_TYPE_BF16BF16F32 0x05
#define IREE_B200_UK_FLAG_MMT4D_TYPE_BF16BF16BF16 0x06
#define IREE_B200_UK_FLAG_MMT4D_TYPE_S16S16S32 0x07
#define IREE_B200_UK_FLAG_MMT4D_TYPE_S16U4S32 0x08
#define IREE_B200_UK_FLAG_MMT4D_TYPE_S16S8S32 0x09
#define IREE_B200_UK_FLAG_MMT4D_TYPE_S8S4S32 0x0A
#define IREE_B200_UK_FLAG_MMT4D_ACCUMULATE 0x100
/* No counterpart in the reference: take the path that brings both operands back to row-major first
 * (un-tile, row-major contraction, re-tile) even where the kernel that reads tiled operands applies. */
#define IREE_B200_UK_FLAG_MMT4D_UNTILE 0x10000
#define IREE_B200_UK_FLAG_PACK_TYPE_MASK 0xFF
#define IREE_B200_UK_FLAG_PACK_TYPE_F32F32 0x01
#define IREE_B200_UK_FLAG_PACK_TYPE_I8I8 0x02
#define IREE_B200_UK_FLAG_PACK_TYPE_I32I32 0x03
#define IREE_B200_UK_FLAG_PACK_TYPE_F16F16 0x04
#define IREE_B200_UK_FLAG_PACK_TYPE_BF16BF16 0x05
#define IREE_B200_UK_FLAG_PACK_TRANSPOSE_INNER 0x100
#define IREE_B200_UK_FLAG_PACK_TRANSPOSE_OUTER 0x200
/* No counterpart in the reference (pack and unpack): take the kernels that stage regions in shared
 * memory even where the shape allows the copy to be done by the TMA unit alone. */
#define IREE_B200_UK_FLAG_PACK_NO_TMA 0x40000
/* iree_uk_pack: row-major [in_size0, in_size1] -> tiled [out_size0..3], ragged edge filled with
 * the low bytes of padding_value. out_stride1 must equal out_size2 * out_size3 (pack.c:72).
 * Kernels, chosen from shape and alignment (results are the same bytes on every path): a copy done
 * by the TMA unit alone when no element moves inside a 16-byte piece (no inner transpose, or a
 * transposed tile one row high; tile rows of whole 16-byte pieces; a matrix the tiles cover exactly;
 * 16-byte aligned addresses and pitches), in both directions; TMA box in / bulk copies out with a
 * byte interleave or gather in shared memory for tiles of sixteen rows x two bytes (the int8 16x2
 * right-hand side with both transposes, the int8 16x2 and f16 / bf16 16x1 left-hand sides; zero
 * padding only); regions staged in shared memory for everything else. */
iree_b200_status_t iree_b200_uk_pack(iree_b200_context_t* context, const void* in_buffer, int64_t in_offset,
                                     int64_t in_stride0, int64_t in_stride1, void* out_buffer, int64_t out_offset,
                                     int64_t out_stride0, int64_t out_stride1, int64_t in_size0, int64_t in_size1,
                                     int64_t out_size0, int64_t out_size1, int64_t out_size2, int64_t out_size3,
                                     uint64_t padding_value, uint32_t flags);
/* iree_uk_unpack: the inverse; in_stride1 must equal in_size2 * in_size3 (unpack.c:49). The type
 * flags are the pack ones (I8I8 is accepted here although the reference's unpack has no user
 * for it). */
iree_b200_status_t iree_b200_uk_unpack(iree_b200_context_t* context, const void* in_buffer, int64_t in_offset,
                                       int64_t in_stride0, int64_t in_stride1, void* out_buffer, int64_t out_offset,
                                       int64_t out_stride0, int64_t out_stride1, int64_t in_size0, int64_t in_size1,
                                       int64_t in_size2, int64_t in_size3, int64_t out_size0, int64_t out_size1,
                                       uint32_t flags);
/* pack and unpack take no workspace, so the kernels among them that wait on copies of their own (the
 * TMA paths) report into a status word the context owns: after the device has been synchronised this
 * returns OK, INVALID_ARGUMENT (a kernel rejected shape or alignment) or DEADLINE_EXCEEDED (a bounded wait
 * ran out; the destination of that call is incomplete), and clears the word. No counterpart in the
 * reference, whose ukernels run on the calling thread. */
iree_b200_status_t iree_b200_uk_status(iree_b200_context_t* context);

/* iree_uk_mmt4d: out[M,N,M0,N0] (+)= lhs[M,K,M0,K0] x rhs[N,K,N0,K0]
 * (runtime/src/iree/builtins/ukernel/mmt4d.c:55-141). Tiles whose rows are 32 bytes in both operands
 * (i8 16x16x2, the x86-64 VNNI tile; f16 / bf16 16x16x1), at 16-byte aligned operand addresses and
 * pitches and 32-byte aligned results, are multiplied as they are by one kernel: 16-byte asynchronous
 * copies land the tiled operands in shared memory in a layout the tensor core reads directly, and the
 * epilogue writes whole [M0,N0] tiles with ACCUMULATE folded in. Other tile shapes are brought to row-major by the
 * unpack kernel, multiplied by the row-major contraction kernel, and the accumulator is tiled (and
 * added, with ACCUMULATE) by the pack kernel. `workspace` is a zero-filled device buffer of
 * iree_b200_uk_mmt4d_workspace_bytes() bytes, 256-byte aligned.
 * Types: S8S8S32 (bit-exact), F16F16F32, BF16BF16F32, F16F16F16, BF16BF16BF16 (f32 accumulation
 * in tensor-core order; ACCUMULATE only with 32-bit outputs) on the tensor cores; F32F32F32, S16S16S32,
 * S16U4S32, S16S8S32, S8S4S32 through a one-thread-per-element kernel in the order of the reference's
 * generic tile functions (integer types bit-exact; offsets and strides in elements of each operand's
 * type, a 4-bit element being half a byte; K0 even for the 4-bit right-hand sides; no workspace needed). The
 * 16-bit-output types always accumulate in f32 and round once at the end, i.e. they behave as the
 * reference does with IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS (0x400) set, whether or not
 * the caller passes that flag (without it the reference's generic tile rounds to the narrow type
 * after every K0 step, mmt4d_tile_generic.c). */
size_t iree_b200_uk_mmt4d_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t M0, int32_t N0, int32_t K0,
                                          uint32_t flags);
iree_b200_status_t iree_b200_uk_mmt4d(iree_b200_context_t* context, const void* lhs_buffer, int64_t lhs_offset,
                                      int64_t lhs_stride0, const void* rhs_buffer, int64_t rhs_offset,
                                      int64_t rhs_stride0, void* out_buffer, int64_t out_offset, int64_t out_stride0,
                                      int64_t M, int64_t N, int64_t K, int32_t M0, int32_t N0, int32_t K0,
                                      uint32_t flags, void* workspace);

/* ---- parameter archives (.irpa): weights from files -------------------------------------------
 *
 * Index, parser, writer and loader for the reference's parameter archive format
 * (runtime/src/iree/schemas/parameter_archive.h). The index is iree_io_parameter_index_t
 * (runtime/src/iree/io/parameter_index.h:23-90), parsing is iree_io_parse_irpa_index
 * (io/formats/irpa/irpa_parser.h) with its checks and status codes, writing lays the file out
 * exactly as iree_io_parameter_archive_builder_write does (io/formats/irpa/irpa_builder.c), and
 * iree_b200_parameter_load is what the parameter provider's load / gather does for one device
 * buffer (io/parameter_index_provider.c). */
typedef struct iree_b200_parameter_index_t iree_b200_parameter_index_t;
enum {
  IREE_B200_PARAMETER_STORAGE_SPLAT = 0, /* IREE_IO_PARAMETER_INDEX_ENTRY_STORAGE_TYPE_SPLAT */
  IREE_B200_PARAMETER_STORAGE_FILE = 1,  /* IREE_IO_PARAMETER_INDEX_ENTRY_STORAGE_TYPE_FILE */
};
typedef struct iree_b200_parameter_entry_t {
  const char* key; /* not NUL-terminated; owned by the index */
  uint64_t key_length;
  const char* metadata;
  uint64_t metadata_length;
  uint64_t length; /* bytes of the parameter */
  int32_t storage_type;
  uint8_t pattern_length; /* splats */
  uint8_t pattern[16];
  uint64_t file_offset; /* file-backed entries: absolute offset in the archive */
} iree_b200_parameter_entry_t;
/* One parameter handed to the writer. A data entry takes its bytes from `data`, or repeats
 * `pattern` when data is NULL (all zeros when pattern_length is 0 too). */
typedef struct iree_b200_parameter_source_t {
  const char* key; /* NUL-terminated */
  const void* metadata;
  uint64_t metadata_length;
  int32_t storage_type;
  uint64_t length;
  const void* data;
  uint8_t pattern_length;
  uint8_t pattern[16];
  uint64_t alignment; /* data entries; 0 = 64 */
} iree_b200_parameter_source_t;
/* Maps the file and indexes every header of its chain. */
iree_b200_status_t iree_b200_parameter_index_open(const char* path, iree_b200_parameter_index_t** out_index);
/* The same over a buffer the caller keeps alive for the index's lifetime. */
iree_b200_status_t iree_b200_parameter_index_parse(const void* data, size_t size,
                                                   iree_b200_parameter_index_t** out_index);
void iree_b200_parameter_index_release(iree_b200_parameter_index_t* index);
int64_t iree_b200_parameter_index_count(const iree_b200_parameter_index_t* index);
iree_b200_status_t iree_b200_parameter_index_get(const iree_b200_parameter_index_t* index, int64_t i,
                                                 iree_b200_parameter_entry_t* out_entry);
/* NOT_FOUND when the key is absent. */
iree_b200_status_t iree_b200_parameter_index_lookup(const iree_b200_parameter_index_t* index, const char* key,
                                                    iree_b200_parameter_entry_t* out_entry);
/* Bytes [parameter_offset, parameter_offset + length) of a parameter into host / device memory
 * (splats are expanded); the call returns when the bytes are in place. */
iree_b200_status_t iree_b200_parameter_read(const iree_b200_parameter_index_t* index, const char* key,
                                            uint64_t parameter_offset, void* host_ptr, uint64_t length);
iree_b200_status_t iree_b200_parameter_load(iree_b200_context_t* context, const iree_b200_parameter_index_t* index,
                                            const char* key, uint64_t parameter_offset, void* device_ptr,
                                            uint64_t length);
/* Writes an archive holding the entries in the order given. */
iree_b200_status_t iree_b200_parameter_archive_write(const char* path, int64_t entry_count,
                                                     const iree_b200_parameter_source_t* entries);

/* ---- W4A16 decode without any allocation ---------------------------------------------------------
 * No counterpart in the reference: added for hosts that cannot allocate device memory where
 * they dispatch (inside a stream capture, after handing all memory to their own pool, or on a
 * path that must not take the driver's allocation lock). Same arithmetic and the same kernel
 * body as IREE_B200_W4A16_DECODE, but the K > 4096 scratch is a fixed array inside the
 * library's device image, so only inputs and outputs are passed; nothing is allocated or freed,
 * here or in any library this calls.
 *   - runs on the CUDA device that is current on the calling thread, on `stream` (a
 *     cudaStream_t; NULL = the default stream); all pointers are device pointers; `a`, `wq` and
 *     `scales` must start on 16-byte boundaries (INVALID_ARGUMENT otherwise: the kernel reads
 *     them with 16-byte loads and bulk copies);
 *   - 1 <= M <= 16; N a multiple of 16 and at most IREE_B200_NOALLOC_MAX_N; K a multiple of 256
 *     and at most 16384; group size 128. K runs in slices of 4096 and the built-in scratch holds
 *     N * slices <= 2 * IREE_B200_NOALLOC_MAX_N, i.e. the full N up to K = 8192 and half of it
 *     at K = 16384 (OUT_OF_RANGE beyond either limit); out[m * ldo + n_offset + n] receives the
 *     result;
 *   - the first call on each device looks up the scratch array's address; make that first call
 *     before starting any stream capture;
 *   - every call on a device shares the one scratch array (about 4 MiB, held by every GPU that
 *     loads the library until the process exits): calls that overlap on the GPU race, so keep
 *     them on one stream or order them yourself;
 *   - a bounded wait that runs out inside the kernel leaves the result partly unwritten and is
 *     reported by iree_b200_w4a16_decode_noalloc_status(), to be called once the stream has been
 *     synchronised: DEADLINE_EXCEEDED (and the record is cleared), else OK. */
#define IREE_B200_NOALLOC_MAX_N 32768
iree_b200_status_t iree_b200_w4a16_decode_noalloc(const void* a, const void* wq, const void* scales, void* out,
                                                  int32_t M, int32_t N, int32_t K, int32_t ldo, int32_t n_offset,
                                                  void* stream);
iree_b200_status_t iree_b200_w4a16_decode_noalloc_status(void);

#ifdef __cplusplus
}
#endif
#endif /* IREE_B200_H_ */
