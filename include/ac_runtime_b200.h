/*
 * C ABI of the B200 runtime library (libac_runtime_b200.so): the opaque-handle runtime interface of
 * uno-km/ameva-compute (include/ac_runtime.h, include/ac_base.h, include/ac_error.h, ABI 2.3) served by a CUDA backend.
 *
 * A host built against the reference's own headers links or dlopens this library unchanged: every struct below has the
 * field order, sizes and offsets of docs/abi/ac_runtime_layout.txt, every enumerator the reference's value, every
 * function the reference's name and signature. Differences, all additive (ABI minor 2.4):
 *   - AC_BACKEND_CUDA (3) is the only backend kind this library creates contexts for; Vulkan / OpenCL kinds are refused
 *     with AC_ERR_BACKEND_UNAVAILABLE;
 *   - kernels are built in: ac_runtime_kernel_create / _create_from_source resolve metadata->kernel_name in the
 *     library's registry and ignore the SPIR-V / OpenCL C blob; an unknown name is AC_ERR_KERNEL_NOT_FOUND (there is no
 *     fallback of any kind); ac_runtime_kernel_create_builtin is the short form;
 *   - buffers are device memory (cudaMalloc): host access only through ac_runtime_buffer_write / read / fill, exactly
 *     like the reference's OpenCL backend (mapped-pointer calls return AC_ERR_BUFFER_NOT_MAPPED);
 *   - dispatches of a context run in recording order on one CUDA stream, so batch barriers are implied.
 * Each declaration cites the reference interface it replaces (file:line inside uno-km/ameva-compute).
 */
#ifndef AC_RUNTIME_B200_H
#define AC_RUNTIME_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- versioning: include/ac_base.h:28-46 ------------------------------------------------------------------------- */
#define AC_ABI_VERSION_MAJOR 2u
#define AC_ABI_VERSION_MINOR 4u /* 2.4 = 2.3 + AC_BACKEND_CUDA + ac_runtime_kernel_create_builtin + ac_b200_* */
#define AC_ABI_VERSION_PATCH 0u
#define AC_ABI_VERSION 0x00020400u
#define AC_ABI_MIN_MINOR 1u
#define AC_ABI_COMPATIBLE(v)                                                                                      \
    ((((v) >> 16) == AC_ABI_VERSION_MAJOR) && ((((v) >> 8) & 0xFFu) >= AC_ABI_MIN_MINOR) &&                       \
     ((((v) >> 8) & 0xFFu) <= AC_ABI_VERSION_MINOR) && (((v)&0xFFu) == 0u))

/* ---- backend kinds: include/ac_base.h:51-55 ---------------------------------------------------------------------- */
typedef uint32_t AcBackendKind;
#define AC_BACKEND_UNKNOWN ((AcBackendKind)0u)
#define AC_BACKEND_VULKAN ((AcBackendKind)1u)
#define AC_BACKEND_OPENCL ((AcBackendKind)2u)
#define AC_BACKEND_CUDA ((AcBackendKind)3u)

/* ---- result codes: include/ac_base.h:92-139 (values are ABI) ----------------------------------------------------- */
typedef enum {
    AC_SUCCESS = 0,
    AC_ERR_INVALID_CONTEXT = -101,
    AC_ERR_DRIVER_NOT_FOUND = -102,
    AC_ERR_DRIVER_SYMBOL_MISSING = -103,
    AC_ERR_DEVICE_NOT_SUPPORTED = -104,
    AC_ERR_DRIVER_INIT_FAILED = -105,
    AC_ERR_INVALID_ARGUMENT = -106,
    AC_ERR_CONTEXT_MISMATCH = -107,
    AC_ERR_FEATURE_NOT_SUPPORTED = -108,
    AC_ERR_INVALID_SHAPE = -109,
    AC_ERR_ABI_MISMATCH = -110,
    AC_ERR_BACKEND_UNAVAILABLE = -111,
    AC_ERR_OUT_OF_HOST_MEMORY = -201,
    AC_ERR_OUT_OF_DEVICE_MEMORY = -202,
    AC_ERR_BUFFER_ALIGNMENT_INVALID = -203,
    AC_ERR_BUFFER_NOT_MAPPED = -204,
    AC_ERR_NULL_POINTER = -205,
    AC_ERR_INVALID_BUFFER_SIZE = -206,
    AC_ERR_KERNEL_BUILD_FAILED = -301,
    AC_ERR_KERNEL_NOT_FOUND = -302,
    AC_ERR_KERNEL_ARG_INVALID = -303,
    AC_ERR_BINARY_CORRUPTED = -304,
    AC_ERR_INVALID_WORK_GROUP_SIZE = -401,
    AC_ERR_INVALID_WORK_ITEM_DIMS = -402,
    AC_ERR_MALI_INFINITE_LOOP_DETECTED = -403,
    AC_ERR_ADRENO_UNSAFE_SUBGROUP_OP = -404,
    AC_ERR_LAUNCH_TIMEOUT = -405,
    AC_ERR_DEVICE_BUSY = -406,
    AC_ERR_RESOURCE_IN_USE = -407,
    AC_ERR_NAN_OR_INF_DETECTED = -501,
    AC_ERR_NUMERICAL_OVERFLOW = -502,
    AC_ERR_DRIVER_CRASH_OR_LOST = -601,
    AC_ERR_OS_PROCESS_KILL_SIGNAL = -602,
    AC_ERR_THERMAL_THROTTLING_TRIPPED = -603
} AcResult;

/* ---- small shared types: include/ac_base.h:60-84, 165-169 -------------------------------------------------------- */
typedef struct { uint32_t x, y, z; } AcDim3;
typedef uint32_t AcSpecConstantType;
typedef struct { uint32_t constant_id; AcSpecConstantType type; uint32_t value_bits; } AcSpecConstant;
typedef struct {
    uint32_t constant_id;
    AcSpecConstantType type;
    uint32_t default_value_bits, min_value_bits, max_value_bits;
    uint32_t overrides_local_size_axis;
} AcSpecConstantSchemaEntry;

/* ---- opaque handles: include/ac_runtime.h:42-45, 389 ------------------------------------------------------------- */
typedef struct AcContext AcContext;
typedef struct AcBuffer AcBuffer;
typedef struct AcKernel AcKernel;
typedef struct AcEvent AcEvent;
typedef struct AcCommandBatch AcCommandBatch;

/* ---- flags: include/ac_runtime.h:54-71, 458-465, 638 ------------------------------------------------------------- */
typedef uint32_t AcBufferUsageFlags;
#define AC_BUFFER_USAGE_STORAGE (1u << 0)
#define AC_BUFFER_USAGE_TRANSFER_SRC (1u << 1)
#define AC_BUFFER_USAGE_TRANSFER_DST (1u << 2)
#define AC_BUFFER_USAGE_UNIFORM (1u << 3)
typedef uint32_t AcShaderStage;
#define AC_STAGE_COMPUTE ((AcShaderStage)(1u << 5))
typedef uint32_t AcRuntimeBindingType;
#define AC_RUNTIME_BINDING_STORAGE_BUFFER ((AcRuntimeBindingType)0u)
#define AC_RUNTIME_BINDING_UNIFORM_BUFFER ((AcRuntimeBindingType)1u)
#define AC_BATCH_MAX_DISPATCHES 65536u
#define AC_BATCH_FLAG_EXPLICIT_BARRIERS (1u << 0)
#define AC_BATCH_FLAG_TIMESTAMPS (1u << 1)
#define AC_BATCH_FLAG_DISPATCH_TIMESTAMPS (1u << 2)
#define AC_KERNEL_SOURCE_BINDING_RANGES (1u << 0)
#define AC_PIPELINE_IDENTITY_SHA256_HEX_SIZE 65u

/* ---- descriptors: include/ac_runtime.h:76-149, 467-515, 640-648 -------------------------------------------------- */
typedef struct { uint32_t binding_index; AcRuntimeBindingType binding_type; AcShaderStage stage_flags; } AcRuntimeBindingDesc;

typedef struct {
    const char* kernel_name; /* the registry key on this backend */
    const char* entry_point;
    uint32_t binding_count;
    const AcRuntimeBindingDesc* bindings;
    size_t push_constant_size;
    AcDim3 local_size;
    uint32_t required_features;
    const char* expected_spirv_sha256; /* not used by this backend */
    uint32_t specialization_schema_count;
    const AcSpecConstantSchemaEntry* specialization_schemas;
} AcKernelRuntimeMetadata;

typedef struct { uint32_t abi_version, struct_size; AcBackendKind backend_kind; uint32_t flags; } AcContextDesc;

typedef struct {
    uint32_t abi_version, struct_size;
    size_t size_bytes;
    AcBufferUsageFlags usage;
    uint32_t force_non_coherent;
} AcBufferDesc;

typedef struct {
    uint32_t abi_version, struct_size;
    const uint32_t* spirv_code; /* ignored (may be NULL) */
    size_t code_size_bytes;     /* ignored */
    const AcKernelRuntimeMetadata* metadata;
    uint32_t specialization_count;
    const AcSpecConstant* specializations;
} AcKernelDesc;

typedef struct {
    uint32_t abi_version, struct_size;
    const char* source; /* ignored (may be NULL) */
    size_t source_size;
    const char* build_options;
    const AcKernelRuntimeMetadata* metadata;
    uint32_t flags;
} AcKernelSourceDesc;

typedef struct {
    uint32_t abi_version, struct_size;
    AcKernel* kernel;
    AcBuffer** buffers;
    uint32_t buffer_count;
    const void* push_constants;
    size_t push_constants_size;
    AcDim3 grid_dim;
} AcLaunchDesc;

typedef struct { uint32_t abi_version, struct_size, max_dispatches, flags; } AcBatchDesc;
typedef struct { AcBuffer* buffer; uint64_t offset, range; } AcBufferBinding;

typedef struct {
    uint32_t abi_version, struct_size;
    uint32_t dispatches, barriers, elided_barriers, flushes;
    uint64_t descriptor_cache_hits, descriptor_cache_misses;
} AcBatchStats;

typedef struct {
    uint32_t abi_version, struct_size;
    uint64_t max_storage_buffer_range;
    uint64_t min_storage_buffer_offset_alignment;
    uint64_t max_memory_allocation_size;
    uint32_t max_compute_workgroup_count[3];
    uint32_t max_compute_workgroup_size[3];
    uint32_t max_compute_workgroup_invocations;
    uint32_t max_compute_shared_memory_size;
    uint32_t max_push_constants_size;
    uint32_t subgroup_size;
    uint32_t timestamps_supported;
    float timestamp_period_ns;
    uint32_t integer_dot_product;             /* appended in 2.3: filled only when struct_size covers them */
    uint32_t integer_dot_product_accelerated;
} AcDeviceLimits;

/* ---- error state: include/ac_error.h:26-49 ----------------------------------------------------------------------- */
typedef enum AmevaBackendOpKind {
    AMEVA_BACKEND_OP_NONE = 0,
    AMEVA_BACKEND_OP_BUFFER_ALLOC,
    AMEVA_BACKEND_OP_BUFFER_FREE,
    AMEVA_BACKEND_OP_BUFFER_MAP,
    AMEVA_BACKEND_OP_BUFFER_UNMAP,
    AMEVA_BACKEND_OP_COPY_HTOD,
    AMEVA_BACKEND_OP_COPY_DTOH,
    AMEVA_BACKEND_OP_DISPATCH,
    AMEVA_BACKEND_OP_SYNC
} AmevaBackendOpKind;

typedef struct AmevaBackendErrorState {
    uint64_t generation;
    int32_t first_error;
    AmevaBackendOpKind operation;
    size_t offset, requested_bytes, capacity_bytes;
} AmevaBackendErrorState;
#define AC_GLOBAL_CONTEXT_ID 0ULL

/* ================================================================================================================== */
/* Entry points. Every out-pointer is NULLed on entry and assigned only on success (include/ac_runtime.h:14).        */
/* ================================================================================================================== */

/* include/ac_runtime.h:612 */
uint32_t ac_runtime_abi_version(void);

/* contexts — include/ac_runtime.h:162-186, 536-539, 651; destroy refuses with AC_ERR_RESOURCE_IN_USE while buffers,
 * kernels, events or batches live (src/runtime/ac_runtime.cpp:161-172). One CUDA device + one stream per context; the
 * device is cudaGetDevice() of the calling thread at creation (a rank selects its GPU before creating the context). */
AcResult ac_runtime_context_create(const AcContextDesc* desc, AcContext** out_ctx);
AcResult ac_runtime_context_destroy(AcContext* ctx);
AcResult ac_runtime_context_get_device_name(const AcContext* ctx, char* out_name, size_t max_len);
AcResult ac_runtime_context_get_limits(const AcContext* ctx, AcDeviceLimits* out_limits);
AcResult ac_runtime_context_get_backend_kind(const AcContext* ctx, AcBackendKind* out_kind);

/* buffers — include/ac_runtime.h:200-264, 663-675 */
AcResult ac_runtime_buffer_create(AcContext* ctx, const AcBufferDesc* desc, AcBuffer** out_buf);
AcResult ac_runtime_buffer_destroy(AcBuffer* buf);
AcResult ac_runtime_buffer_get_mapped_ptr(const AcBuffer* buf, void** out_ptr); /* AC_ERR_BUFFER_NOT_MAPPED */
AcResult ac_runtime_buffer_get_size(const AcBuffer* buf, size_t* out_size);
AcResult ac_runtime_buffer_get_allocation_size(const AcBuffer* buf, size_t* out_alloc_size);
AcResult ac_runtime_buffer_is_coherent(const AcBuffer* buf, uint32_t* out_is_coherent); /* AC_ERR_BUFFER_NOT_MAPPED */
AcResult ac_runtime_buffer_flush(AcBuffer* buf, size_t offset, size_t size_bytes);      /* AC_ERR_BUFFER_NOT_MAPPED */
AcResult ac_runtime_buffer_invalidate(AcBuffer* buf, size_t offset, size_t size_bytes); /* AC_ERR_BUFFER_NOT_MAPPED */
AcResult ac_runtime_buffer_write(AcBuffer* buf, size_t offset, const void* src, size_t size_bytes);
AcResult ac_runtime_buffer_read(AcBuffer* buf, size_t offset, void* dst, size_t size_bytes);
AcResult ac_runtime_buffer_fill(AcBuffer* buf, size_t offset, size_t size_bytes, uint8_t value);
AcResult ac_runtime_buffer_get_address(const AcBuffer* buf, void** out_address); /* the device address */

/* kernels — include/ac_runtime.h:278-332, 657. Validation kept from src/runtime/ac_runtime.cpp:586-660: non-empty
 * kernel_name and entry_point, non-zero local size, push <= 128 B, <= 16 bindings of compute stage and storage/uniform
 * type with distinct indices; plus binding_count and push size must match the registry entry
 * (AC_ERR_KERNEL_ARG_INVALID). */
AcResult ac_runtime_kernel_create(AcContext* ctx, const AcKernelDesc* desc, AcKernel** out_kernel);
AcResult ac_runtime_kernel_create_from_source(AcContext* ctx, const AcKernelSourceDesc* desc, AcKernel** out_kernel);
AcResult ac_runtime_kernel_destroy(AcKernel* kernel);
AcResult ac_runtime_kernel_get_pipeline_identity(const AcKernel* kernel, char* out_hex, size_t out_hex_size);
AcResult ac_runtime_kernel_get_effective_local_size(const AcKernel* kernel, AcDim3* out_local_size);
AcResult ac_runtime_kernel_get_push_constant_size(const AcKernel* kernel, size_t* out_size);

/* dispatch and events — include/ac_runtime.h:348-383. out_event == NULL blocks until the GPU finished. */
AcResult ac_runtime_dispatch(AcContext* ctx, const AcLaunchDesc* desc, AcEvent** out_event);
AcResult ac_runtime_event_wait(AcEvent* event, uint64_t timeout_ns); /* AC_ERR_LAUNCH_TIMEOUT when the deadline passes */
AcResult ac_runtime_event_get_timing(AcEvent* event, uint64_t* out_wall_latency_ns, uint64_t* out_gpu_duration_ns);
AcResult ac_runtime_event_destroy(AcEvent* event);

/* batches — include/ac_runtime.h:398-451, 544-602 */
AcResult ac_runtime_batch_begin(AcContext* context, AcCommandBatch** out_batch);
AcResult ac_runtime_batch_begin_ex(AcContext* context, const AcBatchDesc* desc, AcCommandBatch** out_batch);
AcResult ac_runtime_batch_dispatch(AcCommandBatch* batch, AcKernel* kernel, const AcLaunchDesc* launch,
                                   AcEvent** out_event);
AcResult ac_runtime_batch_dispatch_bindings(AcCommandBatch* batch, AcKernel* kernel, const AcBufferBinding* bindings,
                                            uint32_t binding_count, const void* push_constants,
                                            size_t push_constants_size, AcDim3 grid_dim);
AcResult ac_runtime_batch_barrier(AcCommandBatch* batch);
AcResult ac_runtime_batch_flush(AcCommandBatch* batch);
AcResult ac_runtime_batch_submit(AcCommandBatch* batch, AcEvent** out_completion_event);
AcResult ac_runtime_batch_abort(AcCommandBatch* batch);
void ac_runtime_batch_destroy(AcCommandBatch* batch);
AcResult ac_runtime_batch_get_dispatch_times(const AcCommandBatch* batch, uint64_t* out_ns, uint32_t capacity,
                                             uint32_t* out_count);
AcResult ac_runtime_batch_get_stats(const AcCommandBatch* batch, AcBatchStats* out_stats);

/* pipeline cache — include/ac_runtime.h:524-531. Kernels are precompiled: the cache is empty (size 0), merge accepts
 * only an empty blob. */
AcResult ac_runtime_pipeline_cache_merge(AcContext* ctx, const void* data, size_t size);
AcResult ac_runtime_pipeline_cache_get_data(AcContext* ctx, void* data, size_t* inout_size);

/* error state — include/ac_error.h:55-82, semantics of src/runtime/ac_error.cpp:30-93 (first error wins per generation) */
void ac_runtime_set_error(int32_t error_code, AmevaBackendOpKind op, size_t offset, size_t requested_bytes,
                          size_t capacity_bytes);
AmevaBackendErrorState ac_runtime_get_error_state(void);
int32_t ac_runtime_consume_error(void);
uint64_t ac_runtime_advance_generation(void);
uint64_t ac_runtime_get_generation(void);
void ac_runtime_reset_error_state(void);
void ac_runtime_set_error_ctx(uint64_t context_id, int32_t error_code, AmevaBackendOpKind op, size_t offset,
                              size_t requested_bytes, size_t capacity_bytes);
AmevaBackendErrorState ac_runtime_get_error_state_ctx(uint64_t context_id);
int32_t ac_runtime_consume_error_ctx(uint64_t context_id);
uint64_t ac_runtime_advance_generation_ctx(uint64_t context_id);
uint64_t ac_runtime_get_generation_ctx(uint64_t context_id);
void ac_runtime_reset_error_state_ctx(uint64_t context_id);

/* ================================================================================================================== */
/* 2.4 additions (no counterpart in the reference unless a citation says which code they stand in for)               */
/* ================================================================================================================== */

/* Short form of kernel creation: the registry entry supplies binding count, push size and local size. */
AcResult ac_runtime_kernel_create_builtin(AcContext* ctx, const char* kernel_name, AcKernel** out_kernel);
/* Registry enumeration: number of built-in kernels and the name of entry i (NULL when out of range). */
uint32_t ac_b200_kernel_count(void);
const char* ac_b200_kernel_name(uint32_t index);
/* Launch switches of the tensor-core GEMM kernels ameva_mmtc_<type>[_mp] and bitnet_gemm_i2_s (their last-but-one /
 * fifth push word; 0 = the default schedule).
 *   ONE_TILE_PER_UNIT  every CTA (pair) computes whole output tiles, as many waves as it takes. The default schedule
 *                      cuts K ranges across tiles and has units wait (bounded, about a second, then
 *                      AC_ERR_LAUNCH_TIMEOUT) for partial sums of other units of the same launch, which assumes the
 *                      launch has the whole GPU: a host that shares the device with other contexts or streams sets this.
 *   ONE_ACCUMULATOR    keep launches of more than 256 token rows on the kernel with one accumulator per CTA pair.
 *   TWO_ACCUMULATORS   take the kernel with two accumulators per CTA pair (weights converted once per 512 token rows)
 *                      for every launch of more than 256 token rows; by default only where every CTA pair gets at
 *                      least two whole 256 x 512 output tiles. */
#define AC_B200_GEMM_ONE_TILE_PER_UNIT 64u
#define AC_B200_GEMM_ONE_ACCUMULATOR 128u
#define AC_B200_GEMM_TWO_ACCUMULATORS 256u
/* Upload of a weight tensor with the ggml -> device-regions permutation done on the device: the caller's ggml blocks
 * (rows x k weights of `type`, ggml_nbytes bytes) are copied through two pinned staging chunks of the context (created
 * by the first upload: 2 x 32 MB pinned + 2 x 32 MB device) and permuted by a kernel while the CPU fills the other
 * chunk; returns when the regions at byte `offset` (a multiple of 64) of `buf` are complete. Same bytes as
 * ac_b200_repack_to_device + ac_runtime_buffer_write (the reference repacks on the CPU while uploading,
 * adapters/llama/ggml-ameva/ggml-ameva-buffer.cpp:300-330), so ac_b200_repack_from_device still returns the uploaded
 * blocks exactly. */
AcResult ac_b200_weight_upload(AcBuffer* buf, size_t offset, uint32_t type, const void* ggml_blocks, uint64_t rows,
                               uint64_t k);
/* A host's own kernel under a name of its choosing, dispatched like the built-in ones (batches, replay, events). The
 * reference takes caller kernels as SPIR-V / OpenCL source in AcKernelCreateInfo (ac_runtime.h:560-600); here the caller
 * brings a compiled launcher. fn runs on the recording thread with the device current, must only enqueue work on
 * `stream` (it may be in graph capture) and returns AC_SUCCESS or the error the dispatch reports. `ptr[i]` is binding
 * i's device address with its offset applied, `range[i]` the bytes available there; `push` holds push_bytes / 4 words
 * (zero-filled past what the dispatch supplied). Names are unique for the life of the process (built-in names
 * included): AC_ERR_RESOURCE_IN_USE for a duplicate. 1..16 bindings, push_constant_size <= 128 and a multiple of 4. */
typedef struct AcB200Launch {
    void* stream; /* cudaStream_t */
    uint32_t binding_count;
    void* const* ptr;
    const uint64_t* range;
    const uint32_t* push;
    uint32_t push_bytes;
    int32_t sm_count;
    AcDim3 grid; /* as given by the dispatch; the launcher is free to size its own grid */
} AcB200Launch;
typedef AcResult (*AcB200LaunchFn)(const AcB200Launch* launch);
AcResult ac_b200_kernel_register(const char* name, uint32_t binding_count, uint32_t push_constant_size, AcB200LaunchFn fn);
/* The context's CUDA stream (a cudaStream_t), for callers that time or order their own work against it. */
AcResult ac_b200_context_get_stream(const AcContext* ctx, void** out_stream);
/* Wrap device memory owned by the caller (e.g. a framework allocator) as a buffer; destroy does not free it. */
AcResult ac_b200_buffer_import(AcContext* ctx, void* device_ptr, size_t size_bytes, AcBuffer** out_buf);
/* Sharing a buffer between the ranks of one box (one process per GPU): the owner exports a 64-byte handle
 * (cudaIpcMemHandle_t), a peer opens it and gets a buffer backed by the owner's device memory, reached over NVLink.
 * Used for the fused output exchange of the row-sharded mul_mat (every rank stores its rows into every rank's output).
 * No counterpart in the reference, which is single-device (adapters/llama/ggml-ameva/ggml-ameva-device.cpp:367-370). */
AcResult ac_b200_buffer_export_ipc(AcBuffer* buf, void* out_handle64);
AcResult ac_b200_buffer_open_ipc(AcContext* ctx, const void* handle64, size_t size_bytes, AcBuffer** out_buf);
/* Asynchronous host->device / device->host copies on the context's stream (pinned host memory for true overlap);
 * ordered with the context's dispatches, complete after ac_b200_context_synchronize or a later event wait. */
AcResult ac_b200_buffer_write_async(AcBuffer* buf, size_t offset, const void* src, size_t size_bytes);
AcResult ac_b200_buffer_read_async(AcBuffer* buf, size_t offset, void* dst, size_t size_bytes);
AcResult ac_b200_context_synchronize(AcContext* ctx);

/* Replayable batches. The reference's command batches are one-shot (include/ac_runtime.h:820-880); these two calls have
 * no reference counterpart. ac_b200_batch_instantiate takes a batch that is recording and not yet flushed (without the
 * timestamp flags) and turns its dispatches into an instantiated CUDA graph: every launcher runs once under stream
 * capture, so argument checks and errors are those of a normal flush, and nothing executes yet. ac_b200_batch_replay
 * enqueues the graph on the context's stream (any number of times, in stream order with everything else) and returns a
 * completion event with GPU timing, or blocks when out_completion_event is NULL. The buffers and kernels of the batch
 * stay retained until ac_runtime_batch_destroy. */
AcResult ac_b200_batch_instantiate(AcCommandBatch* batch);
AcResult ac_b200_batch_replay(AcCommandBatch* batch, AcEvent** out_completion_event);

/* Weight codec: ggml block bytes <-> the device region layout the kernels read. Stands in for the reference's CPU
 * repack codec (adapters/llama/ggml-ameva/ggml-ameva-repack.cpp:82-247, ggml-ameva-buffer.cpp:300-330). type is the
 * ggml type id (2 = Q4_0, 8 = Q8_0, 12 = Q4_K, 36 = I2_S). The device layout is the quant payloads of all blocks, padded
 * to a multiple of 64 bytes, then the scale fields of all blocks; ac_b200_device_layout reports its total size and the
 * byte offset of the scale region (I2_S: rows*k/4 bytes, copied unchanged, scale offset = end of payload). Host-side,
 * pure functions. */
AcResult ac_b200_device_layout(uint32_t ggml_type, uint64_t rows, uint64_t k, uint64_t* out_total_bytes,
                               uint64_t* out_scale_offset);
AcResult ac_b200_repack_to_device(uint32_t ggml_type, const void* ggml_blocks, uint64_t rows, uint64_t k, void* dst);
/* Q5_0 (6) and IQ4_NL (20) are accepted by the layout, repack, upload, exponent and plan functions as well: their weights
 * are d * (an int8), so they are kept as Q8_0 regions (the payload decoded exactly at upload, re-encoded exactly at
 * read-back) and served by the Q8_0 kernels: ac_b200_device_type answers which type's kernels and regions serve a
 * weight type (the type itself, 8 for these two, 0 when the type is not built). The reference's repacked family lists
 * both (adapters/llama/ggml-ameva/ggml-ameva-repack.cpp:21-28). Q6_K (14) is accepted too: its payload region holds
 * the 6-bit weights decoded to int8 (q - 32, 256 bytes per block, element order), its scale region the block's 16 int8
 * sub-block scales and fp16 d as they are (18 bytes per block); kernel ameva_mmvqb_q6_K, any M in chunks of 8 rows
 * (ac_b200_mul_mat_plan answers AC_B200_PATH_GEMV). Q5_K (13) likewise: q5 (0..31) as 256 bytes per block, the block's
 * first 16 bytes (d, dmin, packed scales) as its scale record; kernel ameva_mmvqb_q5_K. IQ4_XS (23): kvalues_iq4nl[q4]
 * as 256 int8 per block, the block's first 8 bytes (d, scales_h, scales_l) as its scale record; ameva_mmvqb_iq4_xs.
 * Q4_1 (3) / Q5_1 (7): q as 32 bytes per block, (d, m) as a 4-byte record; ameva_mmvq_q4_1 / ameva_mmvq_q5_1.
 * Q3_K (11): q3 (-4..3) as 256 int8 per block, scales[12] + d as a 14-byte record; ameva_mmvqb_q3_K. Q2_K (10): q2 (0..3)
 * as 256 bytes per block, scales[16] + d + dmin as a 20-byte record; ameva_mmvqb_q2_K.
 * More than 8 activation rows of these seven types (K % 256 == 0): ac_b200_mul_mat_plan answers AC_B200_PATH_GEMM_TC,
 * which for them is ameva_mmtc_scales (scale records -> fp16 (scale, offset) per 16 weights) + ameva_mmtc_b8. */
uint32_t ac_b200_device_type(uint32_t ggml_type);
AcResult ac_b200_repack_from_device(uint32_t ggml_type, const void* device_layout, uint64_t rows, uint64_t k,
                                    void* ggml_blocks);

/* The kernel family a quantized MUL_MAT of a given shape runs on: the one policy every host of this library follows (what
 * the reference decides in mul_mat_qmm_reason / ameva_mmq_plan / ameva_qmv_choice, adapters/llama/ggml-ameva/
 * ggml-ameva.cpp:1326-1377, 2486-2503, 2986). ggml_type as above; M activation rows, N weight rows, K. Shapes outside the
 * contract answer AC_ERR_INVALID_SHAPE / AC_ERR_FEATURE_NOT_SUPPORTED with *out_path = AC_B200_PATH_NONE: there is no
 * other implementation to fall to. Pure host function. */
#define AC_B200_PATH_NONE 0u
#define AC_B200_PATH_GEMV 1u          /* ameva_mmvq_* / ameva_mmvqb_* / bitnet_gemv_i2_s_*; M > 8 in chunks of 8 rows */
#define AC_B200_PATH_GEMV_FQ 2u       /* ameva_mmv*_fq: one activation row quantized inside the GEMV launch */
#define AC_B200_PATH_GEMV_STREAMED 3u /* ameva_mmvs_*: weight rows staged in shared memory by bulk copies */
#define AC_B200_PATH_GEMV_MMA 4u      /* ameva_mmvm_q4_K: up to 8 rows on the integer tensor instruction */
#define AC_B200_PATH_GEMM_TC 5u       /* ameva_mmtc_* / bitnet_gemm_i2_s: tcgen05 GEMM */
#define AC_B200_PLAN_EXACT 1u         /* the caller needs the exact per-block integer sums at every M */
#define AC_B200_PLAN_HOST_LAUNCH 2u   /* kernels are launched one by one from the host (not replayed batches) */
#define AC_B200_PLAN_PEERS 4u         /* the kernel also stores to other ranks' outputs */
#define AC_B200_PLAN_WEIGHT_RANGE 8u  /* AC_B200_WEIGHT_RANGE_EXTREME holds for the weight tensor: integer kernels only */
AcResult ac_b200_mul_mat_plan(uint32_t ggml_type, uint64_t M, uint64_t N, uint64_t K, uint32_t flags, uint32_t* out_path);

/* The magnitude of a weight tensor given as ggml blocks, as a power of two: 2^w_exp brings an upper bound of its largest
 * |w| into [1, 2) (-30..30; 0 for I2_S). The tensor-core GEMM dequantizes weights to fp16; a tensor whose largest
 * magnitude is below 2^-7 or at least 2^14 would lose its small weights to fp16 subnormals or overflow, so hosts compute
 * this once per tensor at upload and pass AC_B200_PLAN_WEIGHT_RANGE for such tensors (they then run on the integer
 * kernels at every M, which are scale-invariant). Host function. */
#define AC_B200_WEIGHT_RANGE_EXTREME(w_exp) ((w_exp) > 7 || (w_exp) < -13)
AcResult ac_b200_weight_exponent(uint32_t ggml_type, const void* ggml_blocks, uint64_t rows, uint64_t k,
                                 int32_t* out_w_exp);

/* Decode mul_mat for callers that cannot allocate. No counterpart in the reference.
 * Q4_0 weights (device layout: w_payload 16 bytes and w_scales one fp16 per 32 weights, row-major over [N][K/32]) times
 * fp32 activations x[M][K], quantized per 32 values on the fly, into dst[M][N] (fp32). The scratch for the quantized
 * activations is a fixed array inside the library's GPU module, so the call performs no device allocation of any kind:
 * meant for hosts that must not allocate where they call from (real-time callbacks, fixed-budget plugins, sandboxes
 * that forbid allocation after start-up). Limits: M <= 8 and K <= 32768, otherwise AC_ERR_INVALID_SHAPE; the array
 * (294 912 bytes) stays resident on every GPU that loads the library. All pointers are device addresses on the current
 * device (the one `stream` belongs to: the scratch used is the array of the device current at the call); x and
 * w_payload must be 16-byte aligned, w_scales 2-byte and dst 4-byte aligned, otherwise the call is refused with
 * AC_ERR_BUFFER_ALIGNMENT_INVALID and nothing is launched. The work is enqueued on `stream` (cudaStream_t, NULL = default
 * stream) and not waited for. The first call on a device also looks the array up and should come before any stream capture. Every call reuses the same array, so calls
 * whose GPU work may overlap must be serialised by the caller. */
AcResult ac_b200_mul_mat_q4_0_static(void* stream, const void* w_payload, const void* w_scales, const float* x,
                                     uint32_t x_stride, float* dst, uint32_t dst_stride, uint32_t M, uint32_t N,
                                     uint32_t K, uint32_t round_mode);

#ifdef __cplusplus
}
#endif
#endif /* AC_RUNTIME_B200_H */
