// libamuda_b200.so: the reference's legacy "amuda" host API (include/amuda.h:76-150) and the one legacy operator on the
// quantized mul_mat path (ac_ops_bitnet_gemv_i2_s_exact, src/amuda/amuda_ops.c:299-352) on CUDA.
//
// The reference implements these over OpenCL with unified memory; here a buffer is a pinned host allocation plus a
// device allocation and the two sync calls copy on the context's stream. Kernels are looked up by name in a built-in
// table (one entry); the launch contract of ac_launch is the reference's (src/amuda/amuda_dispatch.c:278-400).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>

#include "../../include/amuda_b200.h"

namespace {

constexpr uint32_t kMagicEvent = 0x414D4556u;   // native_event points at one of these

struct NativeEvent {
    uint32_t magic;
    cudaEvent_t start, end;
};

struct DeviceGuard {
    int prev;
    explicit DeviceGuard(int dev) {
        prev = -1;
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int device_of(const AcContext* ctx) { return (int)(intptr_t)ctx->device_id; }
cudaStream_t stream_of(const AcContext* ctx) { return (cudaStream_t)ctx->command_queue; }

// y[row] = scale * sum_k w[row][k] * x[k]; one warp per row. A 128-weight block is 32 bytes: byte g holds the weights
// g, 32+g, 64+g, 96+g in bits 7-6, 5-4, 3-2, 1-0; codes 0, 1, 2 are -1, 0, +1 and code 3 is 0. Per step the warp covers
// four blocks: lane l takes word l % 8 (bytes 4 (l % 8) .. +3) of block 4 step + l / 8 and the four float4 of x that
// meet it.
__global__ void __launch_bounds__(256) i2s_exact_kernel(int M, int K, const float* __restrict__ x,
                                                        const uint8_t* __restrict__ W, float scale,
                                                        float* __restrict__ y) {
    const int row = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= M) return;
    const int blocks = K >> 7;
    const uint32_t* wrow = reinterpret_cast<const uint32_t*>(W + (size_t)row * (K >> 2));
    float acc = 0.0f;
    for (int b = lane >> 3; b < blocks; b += 4) {
        const uint32_t w = __ldg(wrow + b * 8 + (lane & 7));
        const float* xb = x + b * 128 + 4 * (lane & 7);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const float4 xv = __ldg(reinterpret_cast<const float4*>(xb + 32 * g));
            const uint32_t codes = (w >> (6 - 2 * g)) & 0x03030303u;   // one code per byte
            const float xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t c = (codes >> (8 * j)) & 3u;
                acc += c == 0u ? -xs[j] : (c == 2u ? xs[j] : 0.0f);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[row] = acc * scale;
}

const char kExactName[] = "bitnet_gemv_i2_s_exact";

AcResult make_event(AcContext* ctx, NativeEvent** out) {
    NativeEvent* n = new (std::nothrow) NativeEvent();
    if (!n) return AC_ERR_OUT_OF_HOST_MEMORY;
    n->magic = kMagicEvent;
    n->start = n->end = nullptr;
    if (cudaEventCreate(&n->start) != cudaSuccess || cudaEventCreate(&n->end) != cudaSuccess) {
        if (n->start) cudaEventDestroy(n->start);
        cudaGetLastError();
        delete n;
        return AC_ERR_OUT_OF_HOST_MEMORY;
    }
    (void)ctx;
    *out = n;
    return AC_SUCCESS;
}

// Launch of the built-in kernel between two events; fills *out_event when asked, else waits.
AcResult launch_exact(AcContext* ctx, int M, int K, const float* x, const uint8_t* W, float scale, float* y,
                      AcEvent** out_event) {
    NativeEvent* n = nullptr;
    const AcResult r = make_event(ctx, &n);
    if (r != AC_SUCCESS) return r;
    cudaStream_t st = stream_of(ctx);
    cudaEventRecord(n->start, st);
    i2s_exact_kernel<<<(unsigned)((M + 7) / 8), 256, 0, st>>>(M, K, x, W, scale, y);
    const cudaError_t e = cudaGetLastError();
    cudaEventRecord(n->end, st);
    if (e != cudaSuccess) {
        cudaEventDestroy(n->start);
        cudaEventDestroy(n->end);
        delete n;
        return AC_ERR_DRIVER_CRASH_OR_LOST;
    }
    if (out_event) {
        AcEvent* ev = (AcEvent*)calloc(1, sizeof(AcEvent));
        if (!ev) {
            cudaEventSynchronize(n->end);
            cudaEventDestroy(n->start);
            cudaEventDestroy(n->end);
            delete n;
            return AC_ERR_OUT_OF_HOST_MEMORY;
        }
        ev->native_event = n;
        *out_event = ev;
        return AC_SUCCESS;
    }
    const cudaError_t w = cudaEventSynchronize(n->end);   // synchronous contract when no event is requested
    cudaEventDestroy(n->start);
    cudaEventDestroy(n->end);
    delete n;
    return w == cudaSuccess ? AC_SUCCESS : AC_ERR_DRIVER_CRASH_OR_LOST;
}

}  // namespace

extern "C" {

AcResult ac_init(AcContext** out_ctx) {
    if (!out_ctx) return AC_ERR_NULL_POINTER;
    *out_ctx = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_DRIVER_INIT_FAILED;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_DRIVER_INIT_FAILED;
    }
    if (prop.major != 10) return AC_ERR_DEVICE_NOT_SUPPORTED;   // the kernels are sm_100a binaries
    AcContext* c = (AcContext*)calloc(1, sizeof(AcContext));
    if (!c) return AC_ERR_OUT_OF_HOST_MEMORY;
    cudaStream_t st = nullptr;
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        free(c);
        return AC_ERR_DRIVER_INIT_FAILED;
    }
    c->device_id = (void*)(intptr_t)dev;
    c->command_queue = st;
    strncpy(c->device_name, prop.name, sizeof(c->device_name) - 1);
    strncpy(c->vendor_name, "NVIDIA Corporation", sizeof(c->vendor_name) - 1);
    c->vendor_id = 0x10DEu;
    c->max_compute_units = (uint32_t)prop.multiProcessorCount;
    c->max_work_group_size = (uint64_t)prop.maxThreadsPerBlock;
    for (int i = 0; i < 3; ++i) c->max_work_item_sizes[i] = (uint64_t)prop.maxThreadsDim[i];
    c->global_mem_size = (uint64_t)prop.totalGlobalMem;
    c->local_mem_size = (uint64_t)prop.sharedMemPerBlockOptin;
    c->active_quirks = 0;
    c->is_uma_supported = false;
    *out_ctx = c;
    return AC_SUCCESS;
}

AcResult ac_destroy(AcContext* ctx) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    DeviceGuard g(device_of(ctx));
    cudaStreamSynchronize(stream_of(ctx));
    cudaStreamDestroy(stream_of(ctx));
    free(ctx);
    return AC_SUCCESS;
}

AcResult ac_buffer_alloc(AcContext* ctx, size_t size_bytes, AcBuffer** out_buf) {
    if (out_buf) *out_buf = nullptr;
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!out_buf) return AC_ERR_NULL_POINTER;
    if (size_bytes == 0) return AC_ERR_INVALID_BUFFER_SIZE;
    DeviceGuard g(device_of(ctx));
    AcBuffer* b = (AcBuffer*)calloc(1, sizeof(AcBuffer));
    if (!b) return AC_ERR_OUT_OF_HOST_MEMORY;
    if (cudaMallocHost(&b->host_ptr, size_bytes) != cudaSuccess) {   // page-aligned, hence 64-byte aligned
        cudaGetLastError();
        free(b);
        return AC_ERR_OUT_OF_HOST_MEMORY;
    }
    if (cudaMalloc(&b->native_mem, size_bytes) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeHost(b->host_ptr);
        free(b);
        return AC_ERR_OUT_OF_DEVICE_MEMORY;
    }
    memset(b->host_ptr, 0, size_bytes);
    cudaMemsetAsync(b->native_mem, 0, size_bytes, stream_of(ctx));
    b->size_bytes = size_bytes;
    b->is_mapped = true;
    *out_buf = b;
    return AC_SUCCESS;
}

AcResult ac_buffer_from_host(AcContext* ctx, void* aligned_ptr, size_t size_bytes, AcBuffer** out_buf) {
    if (out_buf) *out_buf = nullptr;
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!out_buf || !aligned_ptr) return AC_ERR_NULL_POINTER;
    if (size_bytes == 0) return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)aligned_ptr & 63u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    DeviceGuard g(device_of(ctx));
    AcBuffer* b = (AcBuffer*)calloc(1, sizeof(AcBuffer));
    if (!b) return AC_ERR_OUT_OF_HOST_MEMORY;
    if (cudaMalloc(&b->native_mem, size_bytes) != cudaSuccess) {
        cudaGetLastError();
        free(b);
        return AC_ERR_OUT_OF_DEVICE_MEMORY;
    }
    b->host_ptr = aligned_ptr;   // pageable: the sync copies are staged by the driver
    b->size_bytes = size_bytes;
    b->is_mapped = true;
    b->is_user_allocated = true;
    *out_buf = b;
    return AC_SUCCESS;
}

AcResult ac_buffer_sync_to_device(AcContext* ctx, AcBuffer* buf) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!buf || !buf->host_ptr || !buf->native_mem) return AC_ERR_NULL_POINTER;
    DeviceGuard g(device_of(ctx));
    if (cudaMemcpyAsync(buf->native_mem, buf->host_ptr, buf->size_bytes, cudaMemcpyHostToDevice, stream_of(ctx)) !=
        cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_DRIVER_CRASH_OR_LOST;
    }
    // the host may rewrite host_ptr as soon as this returns
    return cudaStreamSynchronize(stream_of(ctx)) == cudaSuccess ? AC_SUCCESS : AC_ERR_DRIVER_CRASH_OR_LOST;
}

AcResult ac_buffer_sync_to_host(AcContext* ctx, AcBuffer* buf) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!buf || !buf->host_ptr || !buf->native_mem) return AC_ERR_NULL_POINTER;
    DeviceGuard g(device_of(ctx));
    if (cudaMemcpyAsync(buf->host_ptr, buf->native_mem, buf->size_bytes, cudaMemcpyDeviceToHost, stream_of(ctx)) !=
        cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_DRIVER_CRASH_OR_LOST;
    }
    return cudaStreamSynchronize(stream_of(ctx)) == cudaSuccess ? AC_SUCCESS : AC_ERR_DRIVER_CRASH_OR_LOST;
}

AcResult ac_buffer_free(AcContext* ctx, AcBuffer* buf) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!buf) return AC_ERR_NULL_POINTER;
    DeviceGuard g(device_of(ctx));
    cudaStreamSynchronize(stream_of(ctx));
    if (buf->native_mem) cudaFree(buf->native_mem);
    if (buf->host_ptr && !buf->is_user_allocated) cudaFreeHost(buf->host_ptr);
    free(buf);
    return AC_SUCCESS;
}

static AcResult load_builtin(AcContext* ctx, const char* func_name, AcKernel** out_kernel) {
    if (out_kernel) *out_kernel = nullptr;
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!func_name || !out_kernel) return AC_ERR_NULL_POINTER;
    if (strcmp(func_name, kExactName) != 0) return AC_ERR_KERNEL_NOT_FOUND;
    AcKernel* k = (AcKernel*)calloc(1, sizeof(AcKernel));
    if (!k) return AC_ERR_OUT_OF_HOST_MEMORY;
    k->kernel = (void*)kExactName;   // non-NULL marks a loaded kernel, as the reference's launch checks
    strncpy(k->kernel_name, func_name, sizeof(k->kernel_name) - 1);
    k->work_group_size = 256;
    k->is_builtin = true;
    *out_kernel = k;
    return AC_SUCCESS;
}

AcResult ac_kernel_load_source(AcContext* ctx, const char* source_code, const char* func_name, AcKernel** out_kernel) {
    (void)source_code;   // OpenCL C of the reference: ignored, the name selects the precompiled kernel
    return load_builtin(ctx, func_name, out_kernel);
}

AcResult ac_kernel_load_binary(AcContext* ctx, const void* binary_data, size_t binary_size, const char* func_name,
                               AcKernel** out_kernel) {
    (void)binary_data;
    (void)binary_size;
    return load_builtin(ctx, func_name, out_kernel);
}

AcResult ac_kernel_free(AcContext* ctx, AcKernel* kernel) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!kernel) return AC_ERR_NULL_POINTER;
    free(kernel);
    return AC_SUCCESS;
}

AcResult ac_launch(AcContext* ctx, AcKernel* kernel, AcDim3 grid, AcDim3 block, uint32_t argc, void** argv,
                   size_t* arg_sizes, AcEvent** out_event) {
    if (out_event) *out_event = nullptr;
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!kernel || !kernel->kernel) return AC_ERR_NULL_POINTER;
    if (grid.x == 0 || grid.y == 0 || grid.z == 0) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    if (block.x == 0 || block.y == 0 || block.z == 0) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    const uint64_t threads = (uint64_t)block.x * block.y * block.z;
    if (threads == 0 || threads > ctx->max_work_group_size) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    if (block.x > ctx->max_work_item_sizes[0] || block.y > ctx->max_work_item_sizes[1] ||
        block.z > ctx->max_work_item_sizes[2])
        return AC_ERR_INVALID_WORK_ITEM_DIMS;
    // argument contract of the built-in kernel
    if (strcmp(kernel->kernel_name, kExactName) != 0) return AC_ERR_KERNEL_NOT_FOUND;
    static const size_t want[6] = {sizeof(int), sizeof(int), sizeof(void*), sizeof(void*), sizeof(float), sizeof(void*)};
    if (argc != 6 || !argv || !arg_sizes) return AC_ERR_KERNEL_ARG_INVALID;
    for (uint32_t i = 0; i < 6; ++i)
        if (!argv[i] || arg_sizes[i] != want[i]) return AC_ERR_KERNEL_ARG_INVALID;
    if ((uint64_t)grid.x * block.x > UINT32_MAX || (uint64_t)grid.y * block.y > UINT32_MAX ||
        (uint64_t)grid.z * block.z > UINT32_MAX)
        return AC_ERR_NUMERICAL_OVERFLOW;
    const int M = *(const int*)argv[0], K = *(const int*)argv[1];
    const float* x = *(const float* const*)argv[2];
    const uint8_t* W = *(const uint8_t* const*)argv[3];
    const float scale = *(const float*)argv[4];
    float* y = *(float* const*)argv[5];
    if (M <= 0 || K <= 0 || (K % 128) != 0 || !x || !W || !y) return AC_ERR_KERNEL_ARG_INVALID;
    if (((uintptr_t)x & 15u) || ((uintptr_t)W & 3u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    DeviceGuard g(device_of(ctx));
    return launch_exact(ctx, M, K, x, W, scale, y, out_event);
}

AcResult ac_event_wait(AcContext* ctx, AcEvent* event) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!event || !event->native_event) return AC_ERR_NULL_POINTER;
    NativeEvent* n = (NativeEvent*)event->native_event;
    if (n->magic != kMagicEvent) return AC_ERR_INVALID_ARGUMENT;
    DeviceGuard g(device_of(ctx));
    if (cudaEventSynchronize(n->end) != cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_DRIVER_CRASH_OR_LOST;
    }
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, n->start, n->end) == cudaSuccess) {
        event->duration_us = (uint64_t)(ms * 1000.0f + 0.5f);
        event->end_time_ns = event->start_time_ns + (uint64_t)((double)ms * 1e6);
    }
    return AC_SUCCESS;
}

uint64_t ac_event_get_duration_us(AcEvent* event) { return event ? event->duration_us : 0; }

AcResult ac_event_free(AcContext* ctx, AcEvent* event) {
    if (!ctx) return AC_ERR_INVALID_CONTEXT;
    if (!event) return AC_ERR_NULL_POINTER;
    NativeEvent* n = (NativeEvent*)event->native_event;
    if (n && n->magic == kMagicEvent) {
        DeviceGuard g(device_of(ctx));
        cudaEventSynchronize(n->end);
        cudaEventDestroy(n->start);
        cudaEventDestroy(n->end);
        n->magic = 0;
        delete n;
    }
    free(event);
    return AC_SUCCESS;
}

AcResult ac_ops_bitnet_gemv_i2_s_exact(AcContext* ctx, int M, int K, AcBuffer* x, AcBuffer* W_packed, float tensor_scale,
                                       AcBuffer* y, AcEvent** out_event) {
    if (out_event) *out_event = nullptr;
    if (!ctx || !x || !W_packed || !y) return AC_ERR_NULL_POINTER;
    if (M <= 0 || K <= 0) return AC_ERR_KERNEL_ARG_INVALID;
    if (K % 128 != 0) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t req_x = (uint64_t)K * sizeof(float), req_w = (uint64_t)M * ((uint64_t)K / 4),
                   req_y = (uint64_t)M * sizeof(float);
    if (x->size_bytes < req_x || W_packed->size_bytes < req_w || y->size_bytes < req_y) return AC_ERR_INVALID_BUFFER_SIZE;
    AcResult r = ac_buffer_sync_to_device(ctx, x);
    if (r == AC_SUCCESS) r = ac_buffer_sync_to_device(ctx, W_packed);
    if (r == AC_SUCCESS) r = ac_buffer_sync_to_device(ctx, y);
    if (r != AC_SUCCESS) return r;
    DeviceGuard g(device_of(ctx));
    return launch_exact(ctx, M, K, (const float*)x->native_mem, (const uint8_t*)W_packed->native_mem, tensor_scale,
                        (float*)y->native_mem, out_event);
}

}  // extern "C"
