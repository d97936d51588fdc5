/* Legacy "amuda" host API of uno-km/ameva-compute, served by CUDA on B200: libamuda_b200.so.
 *
 * This is the second boundary of the quantized mul_mat path: the 15 host functions of the reference's include/amuda.h
 * (:76-150) and the one operator of include/amuda_ops.h that lies on the path, ac_ops_bitnet_gemv_i2_s_exact (:73-81).
 * The structs are transparent in the reference and read by its callers (ctx->device_name, buf->host_ptr,
 * tests/test_amuda_bitnet_exact.c:119-127), so their field order and sizes follow include/ac_types.h:41-91 (restated
 * here, checked by the tests against the offsets that header produces on LP64). The type names collide with the opaque
 * handles of the ac_runtime ABI on purpose, as in the reference: a translation unit includes one header or the other.
 *
 * What differs from the reference (OpenCL zero-copy on a UMA phone):
 *   - host_ptr is pinned host memory and native_mem a device allocation of the same size; ac_buffer_sync_to_device /
 *     _to_host are real copies (the reference's are cache maintenance). Callers that follow the reference's protocol
 *     (write host_ptr, sync_to_device or call an ac_ops_*, sync_to_host, read host_ptr) see the same values.
 *   - kernels are resolved by func_name in a built-in table; the OpenCL C source or SPIR-V blob is ignored. Only
 *     "bitnet_gemv_i2_s_exact" exists; any other name is AC_ERR_KERNEL_NOT_FOUND (no silent fallback).
 *   - the other ac_ops_* operators of amuda_ops.h (gemm_fp32, bitnet_gemv_i2, rmsnorm, swiglu, rope) are not part of
 *     this path and are not exported. */
#ifndef AMUDA_B200_H
#define AMUDA_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* include/ac_base.h:92-139 (the values this library can return) */
typedef enum AcResult {
    AC_SUCCESS = 0,
    AC_ERR_INVALID_CONTEXT = -101,
    AC_ERR_DEVICE_NOT_SUPPORTED = -104,
    AC_ERR_DRIVER_INIT_FAILED = -105,
    AC_ERR_INVALID_ARGUMENT = -106,
    AC_ERR_OUT_OF_HOST_MEMORY = -201,
    AC_ERR_OUT_OF_DEVICE_MEMORY = -202,
    AC_ERR_BUFFER_ALIGNMENT_INVALID = -203,
    AC_ERR_NULL_POINTER = -205,
    AC_ERR_INVALID_BUFFER_SIZE = -206,
    AC_ERR_KERNEL_NOT_FOUND = -302,
    AC_ERR_KERNEL_ARG_INVALID = -303,
    AC_ERR_INVALID_WORK_GROUP_SIZE = -401,
    AC_ERR_INVALID_WORK_ITEM_DIMS = -402,
    AC_ERR_LAUNCH_TIMEOUT = -405,
    AC_ERR_NUMERICAL_OVERFLOW = -502,
    AC_ERR_DRIVER_CRASH_OR_LOST = -601
} AcResult;

typedef struct AcDim3 {
    uint32_t x, y, z;
} AcDim3;

/* include/ac_types.h:41-58. On this backend: driver_handle = NULL, platform_id = NULL, device_id = the CUDA device
 * ordinal, context = NULL, command_queue = the cudaStream_t every call of the context runs on. */
typedef struct {
    void* driver_handle;
    void* platform_id;
    void* device_id;
    void* context;
    void* command_queue;
    char device_name[128];
    char vendor_name[64];
    uint32_t vendor_id;
    uint32_t max_compute_units;
    uint64_t max_work_group_size;
    uint64_t max_work_item_sizes[3];
    uint64_t global_mem_size;
    uint64_t local_mem_size;
    uint32_t active_quirks;
    bool is_uma_supported;
} AcContext;

/* include/ac_types.h:63-70. host_ptr: pinned, 64-byte aligned, zero-filled; native_mem: device pointer. */
typedef struct {
    void* host_ptr;
    void* native_mem;
    size_t size_bytes;
    uint32_t flags;
    bool is_mapped;
    bool is_user_allocated;
} AcBuffer;

/* include/ac_types.h:75-81 */
typedef struct {
    void* program;
    void* kernel;
    char kernel_name[64];
    uint64_t work_group_size;
    bool is_builtin;
} AcKernel;

/* include/ac_types.h:86-92 */
typedef struct {
    void* native_event;
    uint64_t submit_time_ns;
    uint64_t start_time_ns;
    uint64_t end_time_ns;
    uint64_t duration_us;
} AcEvent;

/* include/amuda.h:76-150 */
AcResult ac_init(AcContext** out_ctx);
AcResult ac_destroy(AcContext* ctx);
AcResult ac_buffer_alloc(AcContext* ctx, size_t size_bytes, AcBuffer** out_buf);
AcResult ac_buffer_from_host(AcContext* ctx, void* aligned_ptr, size_t size_bytes, AcBuffer** out_buf);
AcResult ac_buffer_sync_to_device(AcContext* ctx, AcBuffer* buf);
AcResult ac_buffer_sync_to_host(AcContext* ctx, AcBuffer* buf);
AcResult ac_buffer_free(AcContext* ctx, AcBuffer* buf);
AcResult ac_kernel_load_source(AcContext* ctx, const char* source_code, const char* func_name, AcKernel** out_kernel);
AcResult ac_kernel_load_binary(AcContext* ctx, const void* binary_data, size_t binary_size, const char* func_name,
                               AcKernel** out_kernel);
AcResult ac_kernel_free(AcContext* ctx, AcKernel* kernel);
/* Validation order and codes of src/amuda/amuda_dispatch.c:278-340: *out_event = NULL first; NULL ctx ->
 * AC_ERR_INVALID_CONTEXT; NULL kernel -> AC_ERR_NULL_POINTER; a zero grid axis -> AC_ERR_INVALID_WORK_ITEM_DIMS; a zero
 * block axis or more than max_work_group_size threads -> AC_ERR_INVALID_WORK_GROUP_SIZE; grid x block over 2^32 - 1 on an
 * axis -> AC_ERR_NUMERICAL_OVERFLOW. Arguments of "bitnet_gemv_i2_s_exact" (src/amuda/amuda_ops.c:334-343): int M, int K,
 * x (pointer to native_mem), W_packed (pointer to native_mem), float tensor_scale, y (pointer to native_mem); any other
 * count or size is AC_ERR_KERNEL_ARG_INVALID. The grid and block the caller passes only have to be valid: the launch
 * geometry is the kernel's own. */
AcResult ac_launch(AcContext* ctx, AcKernel* kernel, AcDim3 grid, AcDim3 block, uint32_t argc, void** argv,
                   size_t* arg_sizes, AcEvent** out_event);
AcResult ac_event_wait(AcContext* ctx, AcEvent* event);
uint64_t ac_event_get_duration_us(AcEvent* event);
AcResult ac_event_free(AcContext* ctx, AcEvent* event);

static inline AcDim3 ac_dim3(uint32_t x, uint32_t y, uint32_t z) {
    AcDim3 d;
    d.x = x;
    d.y = y;
    d.z = z;
    return d;
}
static inline AcDim3 ac_dim1(uint32_t x) { return ac_dim3(x, 1, 1); }

/* include/amuda_ops.h:73-81, src/amuda/amuda_ops.c:299-352: y[m] = tensor_scale * sum_k w[m][k] * x[k] with fp32 x
 * (no activation quantization on this legacy operator) and ternary w decoded from the I2_S packing (code 3 decodes to 0,
 * as the reference's map2bit). M = output rows, K % 128 == 0. Gates in the reference's order: *out_event = NULL; NULL
 * pointer -> AC_ERR_NULL_POINTER; M <= 0, K <= 0 or K % 128 -> AC_ERR_KERNEL_ARG_INVALID; undersized buffer ->
 * AC_ERR_INVALID_BUFFER_SIZE. Like the reference it uploads x, W_packed and y before the launch; the caller downloads y
 * with ac_buffer_sync_to_host. The per-row sum is formed by one warp (lane partials, then a shuffle tree), not in the
 * reference's sequential order, so it agrees with it to fp32 summation error (the reference's own test gate is 1e-3). */
AcResult ac_ops_bitnet_gemv_i2_s_exact(AcContext* ctx, int M, int K, AcBuffer* x, AcBuffer* W_packed, float tensor_scale,
                                       AcBuffer* y, AcEvent** out_event);

#ifdef __cplusplus
}
#endif

#endif /* AMUDA_B200_H */
