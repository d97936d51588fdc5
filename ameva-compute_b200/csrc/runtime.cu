// CUDA backend of the ac_runtime C ABI (include/ac_runtime_b200.h).
//
// Semantics kept from the reference runtime (src/runtime/ac_runtime.cpp of uno-km/ameva-compute): descriptor
// validation by abi_version / struct_size, out-pointers NULLed on entry, magic-tagged opaque handles, child counting
// with refusal to destroy a context that still owns objects, cross-context rejection, grid and binding validation,
// bounded event waits, and the generation-based first-error-wins error state (src/runtime/ac_error.cpp:30-93).
// The execution model is the one the reference's OpenCL backend documents (include/ac_runtime.h:614-630): one in-order
// queue per context (here a CUDA stream), batches that run at flush/submit, host access through write/read/fill only.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.cuh"

using namespace amv;

namespace {

constexpr uint32_t kMagicCtx = 0x41435831u, kMagicBuf = 0x41434255u, kMagicKer = 0x41434B52u, kMagicEvt = 0x41434556u,
                   kMagicBat = 0x41434254u, kMagicDead = 0xDEADACACu;
constexpr uint64_t kOffsetAlign = 64;
constexpr uint32_t kMaxGroupsAxis = 1u << 20, kMaxGroupsTotal = 1u << 24;  // include/ac_dispatch.h:45-56
constexpr uint64_t kBlockingWaitNs = 120ull * 1000000000ull;

uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

}  // namespace

struct AcContext {
    uint32_t magic;
    int device;
    cudaStream_t stream;
    cudaDeviceProp prop;
    uint32_t* status_host;  // mapped pinned memory, 4 words
    uint32_t* status_dev;
    uint32_t* workspace;    // kWorkspaceBytes of zeroed device memory for the kernels' cross-CTA flags
    uint32_t live_buffers, live_kernels, live_events, live_batches;
    uint64_t id;
    SideQueues side;        // copy queues beside the stream, created by the first launcher that needs them
    // weight upload (ac_b200_weight_upload): two pinned host chunks and two device chunks, created by the first upload
    void* up_pinned[2];
    void* up_dev[2];
    cudaEvent_t up_done[2];
    bool up_used[2], up_ready;
};

struct AcBuffer {
    uint32_t magic;
    AcContext* ctx;
    void* dptr;
    size_t size, alloc_size;
    bool owned;
    bool ipc;   // opened from another process's allocation: closed, not freed, on destroy
    uint32_t retained;  // recorded in batches that have not completed
};

struct AcKernel {
    uint32_t magic;
    AcContext* ctx;
    const KernelEntry* entry;
    size_t push_size;
    uint32_t retained;
};

struct AcEvent {
    uint32_t magic;
    AcContext* ctx;
    cudaEvent_t start, end;
    uint64_t wall_submit_ns, wall_done_ns;
    bool signaled;
    AcResult result;
};

struct BatchRecord {
    AcKernel* kernel;
    uint32_t nbind;
    AcBuffer* buf[16];
    uint64_t offset[16], range[16];
    uint32_t push[32];
    AcDim3 grid;
};

struct AcCommandBatch {
    uint32_t magic;
    AcContext* ctx;
    enum State { RECORDING, SUBMITTED, ABORTED, REPLAYABLE } state;
    cudaGraphExec_t exec;   // REPLAYABLE: the recorded launches as an instantiated CUDA graph
    uint32_t max_dispatches, flags;
    std::vector<BatchRecord> records;
    size_t flushed;  // records already launched
    AcBatchStats stats;
    cudaEvent_t t_begin;
    std::vector<cudaEvent_t> t_after;  // one per dispatch with AC_BATCH_FLAG_DISPATCH_TIMESTAMPS
    cudaEvent_t t_end;
    bool started, completed;
};

namespace {

std::mutex g_id_mutex;
uint64_t g_next_ctx_id = 1;

bool ctx_ok(const AcContext* c) { return c && c->magic == kMagicCtx; }
bool buf_ok(const AcBuffer* b) { return b && b->magic == kMagicBuf; }
bool ker_ok(const AcKernel* k) { return k && k->magic == kMagicKer; }
bool evt_ok(const AcEvent* e) { return e && e->magic == kMagicEvt; }
bool bat_ok(const AcCommandBatch* b) { return b && b->magic == kMagicBat; }

struct DeviceGuard {
    int prev;
    explicit DeviceGuard(int dev) {
        prev = -1;
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

AcResult fail(AcContext* ctx, AcResult r, AmevaBackendOpKind op, size_t off = 0, size_t req = 0, size_t cap = 0) {
    if (r != AC_SUCCESS) {
        ac_runtime_set_error((int32_t)r, op, off, req, cap);
        if (ctx) ac_runtime_set_error_ctx(ctx->id, (int32_t)r, op, off, req, cap);
    }
    return r;
}

constexpr size_t kWorkspaceBytes = 1u << 20;

AcResult validate_grid(AcDim3 g) {
    if (g.x == 0 || g.y == 0 || g.z == 0) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    if (g.x > kMaxGroupsAxis || g.y > kMaxGroupsAxis || g.z > kMaxGroupsAxis) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    if ((uint64_t)g.x * g.y * g.z > kMaxGroupsTotal) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    return AC_SUCCESS;
}

// Reads and clears the device status words after the stream reached a known point.
AcResult take_device_status(AcContext* ctx) {
    volatile uint32_t* s = ctx->status_host;
    const uint32_t code = s[0];
    if (code == DEV_STATUS_OK) return AC_SUCCESS;
    s[0] = 0;
    s[1] = 0;
    // a kernel that gave up may have left sequence flags behind: clear them before the next launch
    cudaMemsetAsync(ctx->workspace, 0, kWorkspaceBytes, ctx->stream);
    return code == DEV_STATUS_WAIT_TIMEOUT ? AC_ERR_LAUNCH_TIMEOUT : AC_ERR_KERNEL_ARG_INVALID;
}

AcResult wait_cuda_event(AcContext* ctx, cudaEvent_t ev, uint64_t timeout_ns) {
    const uint64_t t0 = now_ns();
    uint32_t spins = 0;
    for (;;) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return AC_SUCCESS;
        if (q != cudaErrorNotReady) {   // the CUDA error code travels in the error state's offset field
            fprintf(stderr, "ac_runtime_b200: device error while waiting: %s\n", cudaGetErrorName(q));
            cudaGetLastError();
            return fail(ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_SYNC, (size_t)q);
        }
        if (now_ns() - t0 >= timeout_ns) return AC_ERR_LAUNCH_TIMEOUT;
        if (++spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
}

AcResult launch_record(AcContext* ctx, const KernelEntry* e, uint32_t nbind, void* const* ptrs, const uint64_t* ranges,
                       const uint32_t* push, AcDim3 grid) {
    if (!e->launch) {   // a registered kernel: the public form of the same arguments
        AcB200Launch l;
        l.stream = ctx->stream;
        l.binding_count = nbind;
        l.ptr = ptrs;
        l.range = ranges;
        l.push = push;
        l.push_bytes = e->push_bytes;
        l.sm_count = ctx->prop.multiProcessorCount;
        l.grid = grid;
        return e->ext(&l);
    }
    LaunchArgs a;
    memset(&a, 0, sizeof(a));
    a.stream = ctx->stream;
    a.binding_count = nbind;
    for (uint32_t i = 0; i < nbind; ++i) {
        a.ptr[i] = ptrs[i];
        a.range[i] = ranges[i];
    }
    memcpy(a.push, push, sizeof(a.push));
    a.grid = grid;
    a.status = ctx->status_dev;
    a.sm_count = ctx->prop.multiProcessorCount;
    a.workspace = ctx->workspace;
    a.workspace_bytes = kWorkspaceBytes;
    a.side = &ctx->side;
    return e->launch(a);
}

bool abi_ok(uint32_t abi_version, uint32_t struct_size, size_t expect) {
    return AC_ABI_COMPATIBLE(abi_version) && struct_size == expect;
}

AcResult make_event(AcContext* ctx, bool timing, AcEvent** out) {
    AcEvent* e = new (std::nothrow) AcEvent();
    if (!e) return AC_ERR_OUT_OF_HOST_MEMORY;
    e->magic = kMagicEvt;
    e->ctx = ctx;
    e->start = nullptr;
    e->end = nullptr;
    e->signaled = false;
    e->result = AC_SUCCESS;
    e->wall_submit_ns = now_ns();
    e->wall_done_ns = 0;
    const unsigned flags = timing ? cudaEventDefault : cudaEventDisableTiming;
    if ((timing && cudaEventCreateWithFlags(&e->start, flags) != cudaSuccess) ||
        cudaEventCreateWithFlags(&e->end, flags) != cudaSuccess) {
        if (e->start) cudaEventDestroy(e->start);
        delete e;
        return AC_ERR_OUT_OF_HOST_MEMORY;
    }
    ctx->live_events++;
    *out = e;
    return AC_SUCCESS;
}

void free_event(AcEvent* e) {
    if (e->start) cudaEventDestroy(e->start);
    if (e->end) cudaEventDestroy(e->end);
    e->ctx->live_events--;
    e->magic = kMagicDead;
    delete e;
}

AcResult validate_metadata(const AcKernelRuntimeMetadata* md) {
    if (!md) return AC_ERR_NULL_POINTER;
    if (!md->kernel_name || !md->kernel_name[0] || !md->entry_point || !md->entry_point[0])
        return AC_ERR_INVALID_ARGUMENT;
    if (md->local_size.x == 0 || md->local_size.y == 0 || md->local_size.z == 0) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    if (md->push_constant_size > 128) return AC_ERR_INVALID_ARGUMENT;
    if (md->binding_count > 16) return AC_ERR_INVALID_ARGUMENT;
    if (md->binding_count && !md->bindings) return AC_ERR_NULL_POINTER;
    uint32_t seen = 0;
    for (uint32_t i = 0; i < md->binding_count; ++i) {
        const AcRuntimeBindingDesc& b = md->bindings[i];
        if (b.stage_flags != AC_STAGE_COMPUTE) return AC_ERR_INVALID_ARGUMENT;
        if (b.binding_type != AC_RUNTIME_BINDING_STORAGE_BUFFER && b.binding_type != AC_RUNTIME_BINDING_UNIFORM_BUFFER)
            return AC_ERR_INVALID_ARGUMENT;
        if (b.binding_index >= 32 || (seen & (1u << b.binding_index))) return AC_ERR_INVALID_ARGUMENT;
        seen |= 1u << b.binding_index;
    }
    return AC_SUCCESS;
}

AcResult create_kernel(AcContext* ctx, const char* name, const AcKernelRuntimeMetadata* md, AcKernel** out) {
    const KernelEntry* e = find_kernel(name);
    if (!e) return fail(ctx, AC_ERR_KERNEL_NOT_FOUND, AMEVA_BACKEND_OP_DISPATCH);
    size_t push = e->push_bytes;
    if (md) {
        // a host may declare fewer push bytes than the entry knows (the remainder reads as zero), never more
        if (md->binding_count != e->binding_count || md->push_constant_size > e->push_bytes)
            return fail(ctx, AC_ERR_KERNEL_ARG_INVALID, AMEVA_BACKEND_OP_DISPATCH);
        push = md->push_constant_size;
    }
    AcKernel* k = new (std::nothrow) AcKernel();
    if (!k) return AC_ERR_OUT_OF_HOST_MEMORY;
    k->magic = kMagicKer;
    k->ctx = ctx;
    k->entry = e;
    k->push_size = push;
    k->retained = 0;
    ctx->live_kernels++;
    *out = k;
    return AC_SUCCESS;
}

void release_records(AcCommandBatch* b) {
    for (BatchRecord& r : b->records) {
        if (r.kernel) {
            r.kernel->retained--;
            for (uint32_t i = 0; i < r.nbind; ++i) r.buf[i]->retained--;
            r.kernel = nullptr;
        }
    }
}

AcResult flush_batch(AcCommandBatch* b) {
    AcContext* ctx = b->ctx;
    DeviceGuard g(ctx->device);
    const bool ts = (b->flags & (AC_BATCH_FLAG_TIMESTAMPS | AC_BATCH_FLAG_DISPATCH_TIMESTAMPS)) != 0;
    if (!b->started) {
        b->started = true;
        if (ts) {
            if (cudaEventCreate(&b->t_begin) != cudaSuccess) return AC_ERR_OUT_OF_HOST_MEMORY;
            cudaEventRecord(b->t_begin, ctx->stream);
        }
    }
    for (; b->flushed < b->records.size(); ++b->flushed) {
        BatchRecord& r = b->records[b->flushed];
        void* ptrs[16];
        for (uint32_t i = 0; i < r.nbind; ++i) ptrs[i] = (char*)r.buf[i]->dptr + r.offset[i];
        const AcResult rc = launch_record(ctx, r.kernel->entry, r.nbind, ptrs, r.range, r.push, r.grid);
        if (rc != AC_SUCCESS) return fail(ctx, rc, AMEVA_BACKEND_OP_DISPATCH);
        if (b->flags & AC_BATCH_FLAG_DISPATCH_TIMESTAMPS) {
            cudaEvent_t ev;
            if (cudaEventCreate(&ev) != cudaSuccess) return AC_ERR_OUT_OF_HOST_MEMORY;
            cudaEventRecord(ev, ctx->stream);
            b->t_after.push_back(ev);
        }
    }
    return AC_SUCCESS;
}

void destroy_batch_events(AcCommandBatch* b) {
    if (b->t_begin) cudaEventDestroy(b->t_begin);
    if (b->t_end) cudaEventDestroy(b->t_end);
    for (cudaEvent_t e : b->t_after) cudaEventDestroy(e);
    b->t_begin = b->t_end = nullptr;
    b->t_after.clear();
}

}  // namespace

extern "C" {

uint32_t ac_runtime_abi_version(void) { return AC_ABI_VERSION; }

// ---- contexts --------------------------------------------------------------------------------------------------------
AcResult ac_runtime_context_create(const AcContextDesc* desc, AcContext** out_ctx) {
    if (!out_ctx) return AC_ERR_NULL_POINTER;
    *out_ctx = nullptr;
    if (!desc) return AC_ERR_NULL_POINTER;
    if (!abi_ok(desc->abi_version, desc->struct_size, sizeof(AcContextDesc))) return AC_ERR_INVALID_ARGUMENT;
    if (desc->flags != 0) return AC_ERR_INVALID_ARGUMENT;
    if (desc->backend_kind != AC_BACKEND_CUDA) return AC_ERR_BACKEND_UNAVAILABLE;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(nullptr, AC_ERR_DRIVER_NOT_FOUND, AMEVA_BACKEND_OP_NONE);
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(nullptr, AC_ERR_DRIVER_INIT_FAILED, AMEVA_BACKEND_OP_NONE);
    AcContext* c = new (std::nothrow) AcContext();
    if (!c) return AC_ERR_OUT_OF_HOST_MEMORY;
    memset(c, 0, sizeof(*c));
    c->device = dev;
    if (cudaGetDeviceProperties(&c->prop, dev) != cudaSuccess) {
        delete c;
        return fail(nullptr, AC_ERR_DRIVER_INIT_FAILED, AMEVA_BACKEND_OP_NONE);
    }
    if (c->prop.major != 10) {  // the kernels are sm_100a binaries: anything else cannot run them
        delete c;
        return fail(nullptr, AC_ERR_DEVICE_NOT_SUPPORTED, AMEVA_BACKEND_OP_NONE);
    }
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaHostAlloc((void**)&c->status_host, 16, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0) != cudaSuccess ||
        cudaMalloc((void**)&c->workspace, kWorkspaceBytes) != cudaSuccess ||
        cudaMemset(c->workspace, 0, kWorkspaceBytes) != cudaSuccess) {
        cudaGetLastError();
        if (c->workspace) cudaFree(c->workspace);
        if (c->stream) cudaStreamDestroy(c->stream);
        if (c->status_host) cudaFreeHost(c->status_host);
        delete c;
        return fail(nullptr, AC_ERR_DRIVER_INIT_FAILED, AMEVA_BACKEND_OP_NONE);
    }
    memset(c->status_host, 0, 16);
    {
        std::lock_guard<std::mutex> lock(g_id_mutex);
        c->id = g_next_ctx_id++;
    }
    c->magic = kMagicCtx;
    *out_ctx = c;
    return AC_SUCCESS;
}

AcResult ac_runtime_context_destroy(AcContext* ctx) {
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (ctx->live_buffers || ctx->live_kernels || ctx->live_events || ctx->live_batches) return AC_ERR_RESOURCE_IN_USE;
    DeviceGuard g(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->side.ready) {
        for (int i = 0; i < 8; ++i) {
            cudaStreamSynchronize(ctx->side.stream[i]);
            cudaStreamDestroy(ctx->side.stream[i]);
            cudaEventDestroy(ctx->side.done[i]);
        }
        cudaEventDestroy(ctx->side.fork);
    }
    if (ctx->up_ready) {
        for (int i = 0; i < 2; ++i) {
            cudaFreeHost(ctx->up_pinned[i]);
            cudaFree(ctx->up_dev[i]);
            cudaEventDestroy(ctx->up_done[i]);
        }
    }
    cudaStreamDestroy(ctx->stream);
    cudaFreeHost(ctx->status_host);
    cudaFree(ctx->workspace);
    ctx->magic = kMagicDead;
    delete ctx;
    return AC_SUCCESS;
}

AcResult ac_runtime_context_get_device_name(const AcContext* ctx, char* out_name, size_t max_len) {
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!out_name) return AC_ERR_NULL_POINTER;
    if (max_len == 0) return AC_ERR_INVALID_ARGUMENT;
    snprintf(out_name, max_len, "%s", ctx->prop.name);
    return AC_SUCCESS;
}

AcResult ac_runtime_context_get_backend_kind(const AcContext* ctx, AcBackendKind* out_kind) {
    if (!out_kind) return AC_ERR_NULL_POINTER;
    *out_kind = AC_BACKEND_UNKNOWN;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    *out_kind = AC_BACKEND_CUDA;
    return AC_SUCCESS;
}

AcResult ac_runtime_context_get_limits(const AcContext* ctx, AcDeviceLimits* out) {
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!out) return AC_ERR_NULL_POINTER;
    const size_t base = offsetof(AcDeviceLimits, integer_dot_product);
    if (!AC_ABI_COMPATIBLE(out->abi_version) || out->struct_size < base || out->struct_size > sizeof(AcDeviceLimits))
        return AC_ERR_INVALID_ARGUMENT;
    AcDeviceLimits l;
    memset(&l, 0, sizeof(l));
    l.abi_version = out->abi_version;
    l.struct_size = out->struct_size;
    l.max_memory_allocation_size = ctx->prop.totalGlobalMem;
    l.max_storage_buffer_range = ctx->prop.totalGlobalMem;  // device pointers: a binding may span any allocation
    l.min_storage_buffer_offset_alignment = kOffsetAlign;
    for (int i = 0; i < 3; ++i) {
        l.max_compute_workgroup_count[i] = kMaxGroupsAxis;
        l.max_compute_workgroup_size[i] = (uint32_t)ctx->prop.maxThreadsDim[i];
    }
    l.max_compute_workgroup_invocations = (uint32_t)ctx->prop.maxThreadsPerBlock;
    l.max_compute_shared_memory_size = (uint32_t)ctx->prop.sharedMemPerBlockOptin;
    l.max_push_constants_size = 128;
    l.subgroup_size = 32;
    l.timestamps_supported = 1;
    l.timestamp_period_ns = 1.0f;
    l.integer_dot_product = 1;
    l.integer_dot_product_accelerated = 1;
    memcpy(out, &l, out->struct_size);
    return AC_SUCCESS;
}

// ---- buffers ---------------------------------------------------------------------------------------------------------
AcResult ac_runtime_buffer_create(AcContext* ctx, const AcBufferDesc* desc, AcBuffer** out_buf) {
    if (!out_buf) return AC_ERR_NULL_POINTER;
    *out_buf = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!desc) return AC_ERR_NULL_POINTER;
    if (!abi_ok(desc->abi_version, desc->struct_size, sizeof(AcBufferDesc))) return AC_ERR_INVALID_ARGUMENT;
    if (desc->size_bytes == 0) return AC_ERR_INVALID_BUFFER_SIZE;
    const uint32_t known = AC_BUFFER_USAGE_STORAGE | AC_BUFFER_USAGE_TRANSFER_SRC | AC_BUFFER_USAGE_TRANSFER_DST |
                           AC_BUFFER_USAGE_UNIFORM;
    if (desc->usage == 0 || (desc->usage & ~known) || desc->force_non_coherent > 1) return AC_ERR_INVALID_ARGUMENT;
    DeviceGuard g(ctx->device);
    AcBuffer* b = new (std::nothrow) AcBuffer();
    if (!b) return AC_ERR_OUT_OF_HOST_MEMORY;
    const size_t alloc = (desc->size_bytes + 255) & ~(size_t)255;
    if (cudaMalloc(&b->dptr, alloc) != cudaSuccess) {
        cudaGetLastError();
        delete b;
        return fail(ctx, AC_ERR_OUT_OF_DEVICE_MEMORY, AMEVA_BACKEND_OP_BUFFER_ALLOC, 0, desc->size_bytes, 0);
    }
    b->magic = kMagicBuf;
    b->ctx = ctx;
    b->size = desc->size_bytes;
    b->alloc_size = alloc;
    b->owned = true;
    b->ipc = false;
    b->retained = 0;
    ctx->live_buffers++;
    *out_buf = b;
    return AC_SUCCESS;
}

AcResult ac_b200_buffer_import(AcContext* ctx, void* device_ptr, size_t size_bytes, AcBuffer** out_buf) {
    if (!out_buf) return AC_ERR_NULL_POINTER;
    *out_buf = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!device_ptr) return AC_ERR_NULL_POINTER;
    if (size_bytes == 0) return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)device_ptr % kOffsetAlign) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    AcBuffer* b = new (std::nothrow) AcBuffer();
    if (!b) return AC_ERR_OUT_OF_HOST_MEMORY;
    b->magic = kMagicBuf;
    b->ctx = ctx;
    b->dptr = device_ptr;
    b->size = b->alloc_size = size_bytes;
    b->owned = false;
    b->ipc = false;
    b->retained = 0;
    ctx->live_buffers++;
    *out_buf = b;
    return AC_SUCCESS;
}

// Peer sharing between the ranks of one box (one process per GPU): the owner exports a 64-byte handle, the peers open
// it and get a buffer whose device address is the owner's memory, reachable over NVLink.
AcResult ac_b200_buffer_export_ipc(AcBuffer* buf, void* out_handle64) {
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    if (!out_handle64) return AC_ERR_NULL_POINTER;
    if (!buf->owned) return AC_ERR_FEATURE_NOT_SUPPORTED;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    DeviceGuard g(buf->ctx->device);
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, buf->dptr) != cudaSuccess) {
        cudaGetLastError();
        return fail(buf->ctx, AC_ERR_DRIVER_INIT_FAILED, AMEVA_BACKEND_OP_BUFFER_MAP);
    }
    memcpy(out_handle64, &h, 64);
    return AC_SUCCESS;
}

AcResult ac_b200_buffer_open_ipc(AcContext* ctx, const void* handle64, size_t size_bytes, AcBuffer** out_buf) {
    if (!out_buf) return AC_ERR_NULL_POINTER;
    *out_buf = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!handle64) return AC_ERR_NULL_POINTER;
    if (size_bytes == 0) return AC_ERR_INVALID_BUFFER_SIZE;
    DeviceGuard g(ctx->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !p) {
        cudaGetLastError();
        return fail(ctx, AC_ERR_DRIVER_INIT_FAILED, AMEVA_BACKEND_OP_BUFFER_MAP);
    }
    AcBuffer* b = new (std::nothrow) AcBuffer();
    if (!b) {
        cudaIpcCloseMemHandle(p);
        return AC_ERR_OUT_OF_HOST_MEMORY;
    }
    b->magic = kMagicBuf;
    b->ctx = ctx;
    b->dptr = p;
    b->size = b->alloc_size = size_bytes;
    b->owned = false;
    b->ipc = true;
    b->retained = 0;
    ctx->live_buffers++;
    *out_buf = b;
    return AC_SUCCESS;
}

AcResult ac_runtime_buffer_destroy(AcBuffer* buf) {
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    if (buf->retained) return AC_ERR_RESOURCE_IN_USE;
    AcContext* ctx = buf->ctx;
    DeviceGuard g(ctx->device);
    if (buf->owned) {
        cudaStreamSynchronize(ctx->stream);  // a dispatch still in flight may reference it
        cudaFree(buf->dptr);
    } else if (buf->ipc) {
        cudaStreamSynchronize(ctx->stream);
        cudaIpcCloseMemHandle(buf->dptr);
    }
    ctx->live_buffers--;
    buf->magic = kMagicDead;
    delete buf;
    return AC_SUCCESS;
}

AcResult ac_runtime_buffer_get_mapped_ptr(const AcBuffer* buf, void** out_ptr) {
    if (!out_ptr) return AC_ERR_NULL_POINTER;
    *out_ptr = nullptr;
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    return AC_ERR_BUFFER_NOT_MAPPED;
}
AcResult ac_runtime_buffer_get_size(const AcBuffer* buf, size_t* out_size) {
    if (!out_size) return AC_ERR_NULL_POINTER;
    *out_size = 0;
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    *out_size = buf->size;
    return AC_SUCCESS;
}
AcResult ac_runtime_buffer_get_allocation_size(const AcBuffer* buf, size_t* out_alloc_size) {
    if (!out_alloc_size) return AC_ERR_NULL_POINTER;
    *out_alloc_size = 0;
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    *out_alloc_size = buf->alloc_size;
    return AC_SUCCESS;
}
AcResult ac_runtime_buffer_is_coherent(const AcBuffer* buf, uint32_t* out_is_coherent) {
    if (!out_is_coherent) return AC_ERR_NULL_POINTER;
    *out_is_coherent = 0;
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    return AC_ERR_BUFFER_NOT_MAPPED;
}
AcResult ac_runtime_buffer_flush(AcBuffer* buf, size_t, size_t) {
    return buf_ok(buf) ? AC_ERR_BUFFER_NOT_MAPPED : AC_ERR_INVALID_ARGUMENT;
}
AcResult ac_runtime_buffer_invalidate(AcBuffer* buf, size_t, size_t) {
    return buf_ok(buf) ? AC_ERR_BUFFER_NOT_MAPPED : AC_ERR_INVALID_ARGUMENT;
}
AcResult ac_runtime_buffer_get_address(const AcBuffer* buf, void** out_address) {
    if (!out_address) return AC_ERR_NULL_POINTER;
    *out_address = nullptr;
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    *out_address = buf->dptr;
    return AC_SUCCESS;
}

static AcResult check_span(AcBuffer* buf, size_t offset, size_t n, const void* host, AmevaBackendOpKind op) {
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    if (n == 0) return AC_SUCCESS;
    if (!host) return AC_ERR_NULL_POINTER;
    if (offset > buf->size || n > buf->size - offset)
        return fail(buf->ctx, AC_ERR_INVALID_BUFFER_SIZE, op, offset, n, buf->size);
    return AC_SUCCESS;
}

AcResult ac_runtime_buffer_write(AcBuffer* buf, size_t offset, const void* src, size_t n) {
    const AcResult r = check_span(buf, offset, n, src, AMEVA_BACKEND_OP_COPY_HTOD);
    if (r != AC_SUCCESS || n == 0) return r;
    DeviceGuard g(buf->ctx->device);
    if (cudaMemcpyAsync((char*)buf->dptr + offset, src, n, cudaMemcpyHostToDevice, buf->ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(buf->ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(buf->ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_HTOD, offset, n, buf->size);
    }
    return AC_SUCCESS;
}

AcResult ac_runtime_buffer_read(AcBuffer* buf, size_t offset, void* dst, size_t n) {
    const AcResult r = check_span(buf, offset, n, dst, AMEVA_BACKEND_OP_COPY_DTOH);
    if (r != AC_SUCCESS || n == 0) return r;
    DeviceGuard g(buf->ctx->device);
    if (cudaMemcpyAsync(dst, (char*)buf->dptr + offset, n, cudaMemcpyDeviceToHost, buf->ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(buf->ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(buf->ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_DTOH, offset, n, buf->size);
    }
    return AC_SUCCESS;
}

AcResult ac_b200_buffer_write_async(AcBuffer* buf, size_t offset, const void* src, size_t n) {
    const AcResult r = check_span(buf, offset, n, src, AMEVA_BACKEND_OP_COPY_HTOD);
    if (r != AC_SUCCESS || n == 0) return r;
    DeviceGuard g(buf->ctx->device);
    if (cudaMemcpyAsync((char*)buf->dptr + offset, src, n, cudaMemcpyHostToDevice, buf->ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(buf->ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_HTOD, offset, n, buf->size);
    }
    return AC_SUCCESS;
}

AcResult ac_b200_buffer_read_async(AcBuffer* buf, size_t offset, void* dst, size_t n) {
    const AcResult r = check_span(buf, offset, n, dst, AMEVA_BACKEND_OP_COPY_DTOH);
    if (r != AC_SUCCESS || n == 0) return r;
    DeviceGuard g(buf->ctx->device);
    if (cudaMemcpyAsync(dst, (char*)buf->dptr + offset, n, cudaMemcpyDeviceToHost, buf->ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(buf->ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_DTOH, offset, n, buf->size);
    }
    return AC_SUCCESS;
}

AcResult ac_runtime_buffer_fill(AcBuffer* buf, size_t offset, size_t n, uint8_t value) {
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    if (n == 0) return AC_SUCCESS;
    if (offset > buf->size || n > buf->size - offset)
        return fail(buf->ctx, AC_ERR_INVALID_BUFFER_SIZE, AMEVA_BACKEND_OP_COPY_HTOD, offset, n, buf->size);
    DeviceGuard g(buf->ctx->device);
    if (cudaMemsetAsync((char*)buf->dptr + offset, value, n, buf->ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(buf->ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(buf->ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_HTOD, offset, n, buf->size);
    }
    return AC_SUCCESS;
}

AcResult ac_b200_context_get_stream(const AcContext* ctx, void** out_stream) {
    if (!out_stream) return AC_ERR_NULL_POINTER;
    *out_stream = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    *out_stream = (void*)ctx->stream;
    return AC_SUCCESS;
}

AcResult ac_b200_context_synchronize(AcContext* ctx) {
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    DeviceGuard g(ctx->device);
    cudaEvent_t ev;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return AC_ERR_OUT_OF_HOST_MEMORY;
    cudaEventRecord(ev, ctx->stream);
    AcResult r = wait_cuda_event(ctx, ev, kBlockingWaitNs);
    cudaEventDestroy(ev);
    if (r == AC_SUCCESS) r = take_device_status(ctx);
    return r == AC_SUCCESS ? r : fail(ctx, r, AMEVA_BACKEND_OP_SYNC);
}

// ---- kernels ---------------------------------------------------------------------------------------------------------
AcResult ac_runtime_kernel_create(AcContext* ctx, const AcKernelDesc* desc, AcKernel** out_kernel) {
    if (!out_kernel) return AC_ERR_NULL_POINTER;
    *out_kernel = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!desc) return AC_ERR_NULL_POINTER;
    if (!abi_ok(desc->abi_version, desc->struct_size, sizeof(AcKernelDesc))) return AC_ERR_INVALID_ARGUMENT;
    const AcResult v = validate_metadata(desc->metadata);
    if (v != AC_SUCCESS) return v;
    if (desc->specialization_count && !desc->specializations) return AC_ERR_NULL_POINTER;
    return create_kernel(ctx, desc->metadata->kernel_name, desc->metadata, out_kernel);
}

AcResult ac_runtime_kernel_create_from_source(AcContext* ctx, const AcKernelSourceDesc* desc, AcKernel** out_kernel) {
    if (!out_kernel) return AC_ERR_NULL_POINTER;
    *out_kernel = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!desc) return AC_ERR_NULL_POINTER;
    if (!abi_ok(desc->abi_version, desc->struct_size, sizeof(AcKernelSourceDesc))) return AC_ERR_INVALID_ARGUMENT;
    if (desc->flags & ~AC_KERNEL_SOURCE_BINDING_RANGES) return AC_ERR_INVALID_ARGUMENT;
    const AcResult v = validate_metadata(desc->metadata);
    if (v != AC_SUCCESS) return v;
    return create_kernel(ctx, desc->metadata->kernel_name, desc->metadata, out_kernel);
}

AcResult ac_runtime_kernel_create_builtin(AcContext* ctx, const char* kernel_name, AcKernel** out_kernel) {
    if (!out_kernel) return AC_ERR_NULL_POINTER;
    *out_kernel = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!kernel_name) return AC_ERR_NULL_POINTER;
    if (!kernel_name[0]) return AC_ERR_INVALID_ARGUMENT;
    return create_kernel(ctx, kernel_name, nullptr, out_kernel);
}

AcResult ac_runtime_kernel_destroy(AcKernel* kernel) {
    if (!ker_ok(kernel)) return AC_ERR_INVALID_ARGUMENT;
    if (kernel->retained) return AC_ERR_RESOURCE_IN_USE;
    kernel->ctx->live_kernels--;
    kernel->magic = kMagicDead;
    delete kernel;
    return AC_SUCCESS;
}

AcResult ac_runtime_kernel_get_pipeline_identity(const AcKernel* kernel, char* out_hex, size_t out_hex_size) {
    if (!ker_ok(kernel)) return AC_ERR_INVALID_ARGUMENT;
    if (!out_hex) return AC_ERR_NULL_POINTER;
    if (out_hex_size < AC_PIPELINE_IDENTITY_SHA256_HEX_SIZE) return AC_ERR_INVALID_ARGUMENT;
    // A deterministic 64-hex identity of (name, ABI, bindings, push size): FNV-1a chained four times. It identifies a
    // precompiled registry entry; it is not a SHA-256 of shader code, which this backend does not have.
    std::string key = std::string("b200:") + kernel->entry->name + ":" + std::to_string(AC_ABI_VERSION) + ":" +
                      std::to_string(kernel->entry->binding_count) + ":" + std::to_string(kernel->entry->push_bytes);
    uint64_t h = 1469598103934665603ull;
    for (int part = 0; part < 4; ++part) {
        for (unsigned char ch : key) {
            h ^= ch;
            h *= 1099511628211ull;
        }
        h ^= (uint64_t)part;
        snprintf(out_hex + 16 * part, 17, "%016llx", (unsigned long long)h);
    }
    out_hex[64] = 0;
    return AC_SUCCESS;
}

AcResult ac_runtime_kernel_get_effective_local_size(const AcKernel* kernel, AcDim3* out_local_size) {
    if (!out_local_size) return AC_ERR_NULL_POINTER;
    if (!ker_ok(kernel)) return AC_ERR_INVALID_ARGUMENT;
    *out_local_size = kernel->entry->local_size;
    return AC_SUCCESS;
}

AcResult ac_runtime_kernel_get_push_constant_size(const AcKernel* kernel, size_t* out_size) {
    if (!out_size) return AC_ERR_NULL_POINTER;
    *out_size = 0;
    if (!ker_ok(kernel)) return AC_ERR_INVALID_ARGUMENT;
    *out_size = kernel->push_size;
    return AC_SUCCESS;
}

uint32_t ac_b200_kernel_count(void) { return kernel_count(); }
AcResult ac_b200_kernel_register(const char* name, uint32_t binding_count, uint32_t push_constant_size, AcB200LaunchFn fn) {
    return register_kernel(name, binding_count, push_constant_size, fn);
}
const char* ac_b200_kernel_name(uint32_t index) {
    const KernelEntry* e = kernel_at(index);
    return e ? e->name : nullptr;
}

// ---- weight upload with the repack on the device ----------------------------------------------------------------------
static constexpr size_t kUploadChunk = 32u << 20;   // bytes of ggml blocks per staging chunk

AcResult ac_b200_weight_upload(AcBuffer* buf, size_t offset, uint32_t type, const void* ggml_blocks, uint64_t rows,
                               uint64_t k) {
    if (!buf_ok(buf)) return AC_ERR_INVALID_ARGUMENT;
    if (!ggml_blocks) return AC_ERR_NULL_POINTER;
    uint64_t total = 0, s_off = 0;
    AcResult rc = ac_b200_device_layout(type, rows, k, &total, &s_off);
    if (rc != AC_SUCCESS) return rc;
    if (offset % 64u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    if (offset > buf->size || total > buf->size - offset) return AC_ERR_INVALID_BUFFER_SIZE;
    if (type == 36u) return ac_runtime_buffer_write(buf, offset, ggml_blocks, (size_t)total);   // I2_S: dense already
    const uint32_t blk_bytes = (type == 2u || type == 20u) ? 18u : type == 8u ? 34u : type == 6u ? 22u : type == 3u ? 20u : type == 7u ? 24u : type == 14u ? 210u : type == 13u ? 176u : type == 23u ? 136u : type == 11u ? 110u : type == 10u ? 84u : 144u;
    const uint32_t blk = (type == 12u || type == 13u || type == 14u || type == 23u || type == 10u || type == 11u) ? 256u : 32u;
    const uint64_t nblk = rows * (k / blk);
    AcContext* ctx = buf->ctx;
    DeviceGuard g(ctx->device);
    if (!ctx->up_ready) {
        bool ok = true;
        for (int i = 0; i < 2 && ok; ++i)
            ok = cudaMallocHost(&ctx->up_pinned[i], kUploadChunk) == cudaSuccess &&
                 cudaMalloc(&ctx->up_dev[i], kUploadChunk) == cudaSuccess &&
                 cudaEventCreateWithFlags(&ctx->up_done[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {   // (what was created is released here: the staging either exists whole or not at all)
            cudaGetLastError();
            for (int i = 0; i < 2; ++i) {
                if (ctx->up_pinned[i]) cudaFreeHost(ctx->up_pinned[i]);
                if (ctx->up_dev[i]) cudaFree(ctx->up_dev[i]);
                if (ctx->up_done[i]) cudaEventDestroy(ctx->up_done[i]);
                ctx->up_pinned[i] = ctx->up_dev[i] = nullptr;
                ctx->up_done[i] = nullptr;
            }
            cudaGetLastError();
            return fail(ctx, AC_ERR_OUT_OF_DEVICE_MEMORY, AMEVA_BACKEND_OP_COPY_HTOD, 0, kUploadChunk, 0);
        }
        ctx->up_used[0] = ctx->up_used[1] = false;
        ctx->up_ready = true;
    }
    // whole tiles of 256 blocks per chunk, so every chunk starts where a CTA of the repack kernel starts
    const uint64_t chunk_blocks = (kUploadChunk / blk_bytes) / 256u * 256u;
    char* base = (char*)buf->dptr + offset;
    const char* src = (const char*)ggml_blocks;
    int c = 0;
    for (uint64_t first = 0; first < nblk; first += chunk_blocks, c ^= 1) {
        const uint64_t n = nblk - first < chunk_blocks ? nblk - first : chunk_blocks;
        if (ctx->up_used[c] && cudaEventSynchronize(ctx->up_done[c]) != cudaSuccess) {   // the chunk's last use is over
            cudaGetLastError();
            return fail(ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_HTOD, offset, (size_t)total, buf->size);
        }
        memcpy(ctx->up_pinned[c], src + first * blk_bytes, (size_t)(n * blk_bytes));
        if (cudaMemcpyAsync(ctx->up_dev[c], ctx->up_pinned[c], (size_t)(n * blk_bytes), cudaMemcpyHostToDevice,
                            ctx->stream) != cudaSuccess) {
            cudaGetLastError();
            return fail(ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_HTOD, offset, (size_t)total, buf->size);
        }
        rc = amv::launch_repack(ctx->stream, type, ctx->up_dev[c], base, base + s_off, first, n);
        if (rc != AC_SUCCESS) return rc;
        cudaEventRecord(ctx->up_done[c], ctx->stream);
        ctx->up_used[c] = true;
    }
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_COPY_HTOD, offset, (size_t)total, buf->size);
    }
    return AC_SUCCESS;
}

// ---- dispatch and events --------------------------------------------------------------------------------------------
AcResult ac_runtime_dispatch(AcContext* ctx, const AcLaunchDesc* desc, AcEvent** out_event) {
    if (out_event) *out_event = nullptr;
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!desc) return AC_ERR_NULL_POINTER;
    if (!abi_ok(desc->abi_version, desc->struct_size, sizeof(AcLaunchDesc))) return AC_ERR_INVALID_ARGUMENT;
    if (!ker_ok(desc->kernel)) return AC_ERR_INVALID_ARGUMENT;
    if (desc->kernel->ctx != ctx) return AC_ERR_CONTEXT_MISMATCH;
    AcResult r = validate_grid(desc->grid_dim);
    if (r != AC_SUCCESS) return r;
    const KernelEntry* e = desc->kernel->entry;
    if (desc->buffer_count != e->binding_count) return AC_ERR_KERNEL_ARG_INVALID;
    if (desc->buffer_count && !desc->buffers) return AC_ERR_NULL_POINTER;
    if (desc->push_constants_size > desc->kernel->push_size) return AC_ERR_KERNEL_ARG_INVALID;
    if (desc->push_constants_size && !desc->push_constants) return AC_ERR_NULL_POINTER;
    void* ptrs[16];
    uint64_t ranges[16];
    for (uint32_t i = 0; i < desc->buffer_count; ++i) {
        AcBuffer* b = desc->buffers[i];
        if (!buf_ok(b)) return AC_ERR_INVALID_ARGUMENT;
        if (b->ctx != ctx) return AC_ERR_CONTEXT_MISMATCH;
        ptrs[i] = b->dptr;
        ranges[i] = b->size;
    }
    uint32_t push[32];
    memset(push, 0, sizeof(push));
    if (desc->push_constants_size) memcpy(push, desc->push_constants, desc->push_constants_size);
    DeviceGuard g(ctx->device);
    AcEvent* ev = nullptr;
    r = make_event(ctx, true, &ev);
    if (r != AC_SUCCESS) return r;
    cudaEventRecord(ev->start, ctx->stream);
    r = launch_record(ctx, e, desc->buffer_count, ptrs, ranges, push, desc->grid_dim);
    if (r != AC_SUCCESS) {
        free_event(ev);
        return fail(ctx, r, AMEVA_BACKEND_OP_DISPATCH);
    }
    cudaEventRecord(ev->end, ctx->stream);
    if (out_event) {
        *out_event = ev;
        return AC_SUCCESS;
    }
    r = ac_runtime_event_wait(ev, kBlockingWaitNs);
    free_event(ev);
    return r;
}

AcResult ac_runtime_event_wait(AcEvent* event, uint64_t timeout_ns) {
    if (!evt_ok(event)) return AC_ERR_INVALID_ARGUMENT;
    if (event->signaled) return event->result;
    AcContext* ctx = event->ctx;
    DeviceGuard g(ctx->device);
    AcResult r = wait_cuda_event(ctx, event->end, timeout_ns);
    if (r == AC_ERR_LAUNCH_TIMEOUT) return fail(ctx, r, AMEVA_BACKEND_OP_SYNC);  // may be waited on again
    if (r == AC_SUCCESS) r = take_device_status(ctx);
    event->signaled = true;
    event->wall_done_ns = now_ns();
    event->result = r;
    return r == AC_SUCCESS ? r : fail(ctx, r, AMEVA_BACKEND_OP_SYNC);
}

AcResult ac_runtime_event_get_timing(AcEvent* event, uint64_t* out_wall_latency_ns, uint64_t* out_gpu_duration_ns) {
    if (out_wall_latency_ns) *out_wall_latency_ns = 0;
    if (out_gpu_duration_ns) *out_gpu_duration_ns = 0;
    if (!evt_ok(event)) return AC_ERR_INVALID_ARGUMENT;
    if (!event->signaled) return AC_ERR_DEVICE_BUSY;
    if (out_wall_latency_ns) *out_wall_latency_ns = event->wall_done_ns - event->wall_submit_ns;
    if (out_gpu_duration_ns && event->start) {
        float ms = 0.0f;
        DeviceGuard g(event->ctx->device);
        if (cudaEventElapsedTime(&ms, event->start, event->end) == cudaSuccess)
            *out_gpu_duration_ns = (uint64_t)((double)ms * 1e6);
        else
            cudaGetLastError();
    }
    return AC_SUCCESS;
}

AcResult ac_runtime_event_destroy(AcEvent* event) {
    if (!evt_ok(event)) return AC_ERR_INVALID_ARGUMENT;
    if (!event->signaled) {
        // re-wait briefly and keep the object if the GPU is still busy (src/backend/vulkan/ac_vk_event.cpp:121-158)
        const AcResult r = ac_runtime_event_wait(event, 5ull * 1000000000ull);
        if (r == AC_ERR_LAUNCH_TIMEOUT) return AC_ERR_DEVICE_BUSY;
    }
    DeviceGuard g(event->ctx->device);
    free_event(event);
    return AC_SUCCESS;
}

// ---- batches ---------------------------------------------------------------------------------------------------------
AcResult ac_runtime_batch_begin_ex(AcContext* context, const AcBatchDesc* desc, AcCommandBatch** out_batch) {
    if (!out_batch) return AC_ERR_NULL_POINTER;
    *out_batch = nullptr;
    if (!ctx_ok(context)) return AC_ERR_INVALID_CONTEXT;
    if (!desc) return AC_ERR_NULL_POINTER;
    if (!abi_ok(desc->abi_version, desc->struct_size, sizeof(AcBatchDesc))) return AC_ERR_INVALID_ARGUMENT;
    if (desc->max_dispatches == 0 || desc->max_dispatches > AC_BATCH_MAX_DISPATCHES) return AC_ERR_INVALID_ARGUMENT;
    const uint32_t known = AC_BATCH_FLAG_EXPLICIT_BARRIERS | AC_BATCH_FLAG_TIMESTAMPS | AC_BATCH_FLAG_DISPATCH_TIMESTAMPS;
    if (desc->flags & ~known) return AC_ERR_INVALID_ARGUMENT;
    AcCommandBatch* b = new (std::nothrow) AcCommandBatch();
    if (!b) return AC_ERR_OUT_OF_HOST_MEMORY;
    b->magic = kMagicBat;
    b->ctx = context;
    b->state = AcCommandBatch::RECORDING;
    b->max_dispatches = desc->max_dispatches;
    b->flags = desc->flags;
    b->flushed = 0;
    memset(&b->stats, 0, sizeof(b->stats));
    b->t_begin = b->t_end = nullptr;
    b->started = b->completed = false;
    b->exec = nullptr;
    b->records.reserve(desc->max_dispatches < 256 ? desc->max_dispatches : 256);
    context->live_batches++;
    *out_batch = b;
    return AC_SUCCESS;
}

AcResult ac_runtime_batch_begin(AcContext* context, AcCommandBatch** out_batch) {
    AcBatchDesc d = {AC_ABI_VERSION, (uint32_t)sizeof(AcBatchDesc), 1024u, 0u};
    return ac_runtime_batch_begin_ex(context, &d, out_batch);
}

AcResult ac_runtime_batch_dispatch_bindings(AcCommandBatch* batch, AcKernel* kernel, const AcBufferBinding* bindings,
                                            uint32_t binding_count, const void* push_constants,
                                            size_t push_constants_size, AcDim3 grid_dim) {
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state != AcCommandBatch::RECORDING) return AC_ERR_INVALID_ARGUMENT;
    if (!ker_ok(kernel)) return AC_ERR_INVALID_ARGUMENT;
    if (kernel->ctx != batch->ctx) return AC_ERR_CONTEXT_MISMATCH;
    if (binding_count != kernel->entry->binding_count) return AC_ERR_KERNEL_ARG_INVALID;
    if (binding_count && !bindings) return AC_ERR_NULL_POINTER;
    if (push_constants_size > kernel->push_size) return AC_ERR_KERNEL_ARG_INVALID;
    if (push_constants_size && !push_constants) return AC_ERR_NULL_POINTER;
    const AcResult gr = validate_grid(grid_dim);
    if (gr != AC_SUCCESS) return gr;
    if (batch->records.size() >= batch->max_dispatches) return AC_ERR_INVALID_ARGUMENT;
    BatchRecord r;
    memset(&r, 0, sizeof(r));
    for (uint32_t i = 0; i < binding_count; ++i) {
        AcBuffer* b = bindings[i].buffer;
        if (!buf_ok(b)) return AC_ERR_INVALID_ARGUMENT;
        if (b->ctx != batch->ctx) return AC_ERR_CONTEXT_MISMATCH;
        if (bindings[i].range == 0 || bindings[i].offset > b->size || bindings[i].range > b->size - bindings[i].offset)
            return fail(batch->ctx, AC_ERR_INVALID_BUFFER_SIZE, AMEVA_BACKEND_OP_DISPATCH, bindings[i].offset,
                        bindings[i].range, b->size);
        if (bindings[i].offset % kOffsetAlign) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
        r.buf[i] = b;
        r.offset[i] = bindings[i].offset;
        r.range[i] = bindings[i].range;
    }
    r.kernel = kernel;
    r.nbind = binding_count;
    if (push_constants_size) memcpy(r.push, push_constants, push_constants_size);
    r.grid = grid_dim;
    kernel->retained++;
    for (uint32_t i = 0; i < binding_count; ++i) r.buf[i]->retained++;
    batch->records.push_back(r);
    batch->stats.dispatches++;
    batch->stats.descriptor_cache_hits++;  // no descriptor objects on this backend: every binding is a pointer
    return AC_SUCCESS;
}

AcResult ac_runtime_batch_dispatch(AcCommandBatch* batch, AcKernel* kernel, const AcLaunchDesc* launch,
                                   AcEvent** out_event) {
    if (out_event) *out_event = nullptr;
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (!launch) return AC_ERR_NULL_POINTER;
    if (!abi_ok(launch->abi_version, launch->struct_size, sizeof(AcLaunchDesc))) return AC_ERR_INVALID_ARGUMENT;
    if (launch->kernel && launch->kernel != kernel) return AC_ERR_INVALID_ARGUMENT;
    if (launch->buffer_count > 16) return AC_ERR_KERNEL_ARG_INVALID;
    if (launch->buffer_count && !launch->buffers) return AC_ERR_NULL_POINTER;
    AcBufferBinding bind[16];
    for (uint32_t i = 0; i < launch->buffer_count; ++i) {
        if (!buf_ok(launch->buffers[i])) return AC_ERR_INVALID_ARGUMENT;
        bind[i].buffer = launch->buffers[i];
        bind[i].offset = 0;
        bind[i].range = launch->buffers[i]->size;
    }
    // per-dispatch logical events are not produced: a batch completes as a whole (out_event stays NULL)
    return ac_runtime_batch_dispatch_bindings(batch, kernel, bind, launch->buffer_count, launch->push_constants,
                                              launch->push_constants_size, launch->grid_dim);
}

AcResult ac_runtime_batch_barrier(AcCommandBatch* batch) {
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state != AcCommandBatch::RECORDING) return AC_ERR_INVALID_ARGUMENT;
    batch->stats.barriers++;  // stream order already serialises dependent dispatches
    return AC_SUCCESS;
}

AcResult ac_runtime_batch_flush(AcCommandBatch* batch) {
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state != AcCommandBatch::RECORDING) return AC_ERR_INVALID_ARGUMENT;
    if (batch->flushed == batch->records.size()) return AC_SUCCESS;
    const AcResult r = flush_batch(batch);
    if (r != AC_SUCCESS) {
        batch->state = AcCommandBatch::ABORTED;
        return r;
    }
    batch->stats.flushes++;
    return AC_SUCCESS;
}

AcResult ac_runtime_batch_submit(AcCommandBatch* batch, AcEvent** out_completion_event) {
    if (out_completion_event) *out_completion_event = nullptr;
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state != AcCommandBatch::RECORDING) return AC_ERR_INVALID_ARGUMENT;
    AcContext* ctx = batch->ctx;
    DeviceGuard g(ctx->device);
    AcEvent* ev = nullptr;
    AcResult r = make_event(ctx, true, &ev);
    if (r != AC_SUCCESS) return r;
    cudaEventRecord(ev->start, ctx->stream);
    r = flush_batch(batch);
    if (r != AC_SUCCESS) {
        free_event(ev);
        batch->state = AcCommandBatch::ABORTED;
        return r;
    }
    if (batch->flags & (AC_BATCH_FLAG_TIMESTAMPS | AC_BATCH_FLAG_DISPATCH_TIMESTAMPS)) {
        if (cudaEventCreate(&batch->t_end) == cudaSuccess) cudaEventRecord(batch->t_end, ctx->stream);
    }
    cudaEventRecord(ev->end, ctx->stream);
    batch->state = AcCommandBatch::SUBMITTED;
    if (out_completion_event) {
        *out_completion_event = ev;
        return AC_SUCCESS;
    }
    r = ac_runtime_event_wait(ev, kBlockingWaitNs);
    free_event(ev);
    if (r == AC_SUCCESS) {
        batch->completed = true;
        release_records(batch);
    }
    return r;
}

AcResult ac_runtime_batch_abort(AcCommandBatch* batch) {
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state == AcCommandBatch::SUBMITTED) return AC_ERR_INVALID_ARGUMENT;
    if (batch->flushed) {
        DeviceGuard g(batch->ctx->device);
        cudaStreamSynchronize(batch->ctx->stream);
    }
    release_records(batch);
    batch->state = AcCommandBatch::ABORTED;
    return AC_SUCCESS;
}

// ---- replayable batches (no counterpart in the reference: its command batches are one-shot) ------------------------
// ac_b200_batch_instantiate turns a recorded, not yet flushed batch into a CUDA graph of its launches (stream capture
// of the same launchers, so every argument check still runs once); ac_b200_batch_replay enqueues that graph on the
// context's stream any number of times. Launch-bound step sequences (decode GEMVs of a few microseconds) then cost one
// graph launch instead of one host launch per kernel.
AcResult ac_b200_batch_instantiate(AcCommandBatch* batch) {
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state != AcCommandBatch::RECORDING || batch->flushed || batch->records.empty())
        return AC_ERR_INVALID_ARGUMENT;
    if (batch->flags & (AC_BATCH_FLAG_TIMESTAMPS | AC_BATCH_FLAG_DISPATCH_TIMESTAMPS)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    AcContext* ctx = batch->ctx;
    DeviceGuard g(ctx->device);
    if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, AC_ERR_FEATURE_NOT_SUPPORTED, AMEVA_BACKEND_OP_DISPATCH);
    }
    const AcResult r = flush_batch(batch);
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (r != AC_SUCCESS || e != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        batch->state = AcCommandBatch::ABORTED;
        batch->started = false;   // nothing ran
        return r != AC_SUCCESS ? r : fail(ctx, AC_ERR_FEATURE_NOT_SUPPORTED, AMEVA_BACKEND_OP_DISPATCH);
    }
    const cudaError_t ie = cudaGraphInstantiate(&batch->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        cudaGetLastError();
        batch->exec = nullptr;
        batch->state = AcCommandBatch::ABORTED;
        batch->started = false;
        return fail(ctx, AC_ERR_OUT_OF_DEVICE_MEMORY, AMEVA_BACKEND_OP_DISPATCH);
    }
    batch->state = AcCommandBatch::REPLAYABLE;
    batch->started = false;
    return AC_SUCCESS;
}

AcResult ac_b200_batch_replay(AcCommandBatch* batch, AcEvent** out_completion_event) {
    if (out_completion_event) *out_completion_event = nullptr;
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (batch->state != AcCommandBatch::REPLAYABLE || !batch->exec) return AC_ERR_INVALID_ARGUMENT;
    AcContext* ctx = batch->ctx;
    DeviceGuard g(ctx->device);
    AcEvent* ev = nullptr;
    AcResult r = make_event(ctx, true, &ev);
    if (r != AC_SUCCESS) return r;
    cudaEventRecord(ev->start, ctx->stream);
    if (cudaGraphLaunch(batch->exec, ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        free_event(ev);
        return fail(ctx, AC_ERR_DRIVER_CRASH_OR_LOST, AMEVA_BACKEND_OP_DISPATCH);
    }
    cudaEventRecord(ev->end, ctx->stream);
    batch->started = true;   // work of this batch may be in flight: destroy synchronizes
    batch->stats.flushes++;
    if (out_completion_event) {
        *out_completion_event = ev;
        return AC_SUCCESS;
    }
    r = ac_runtime_event_wait(ev, kBlockingWaitNs);
    free_event(ev);
    return r;
}

void ac_runtime_batch_destroy(AcCommandBatch* batch) {
    if (!bat_ok(batch)) return;
    AcContext* ctx = batch->ctx;
    DeviceGuard g(ctx->device);
    if (batch->started && !batch->completed) cudaStreamSynchronize(ctx->stream);  // launched work may still run
    if (batch->exec) cudaGraphExecDestroy(batch->exec);
    release_records(batch);
    destroy_batch_events(batch);
    ctx->live_batches--;
    batch->magic = kMagicDead;
    delete batch;
}

AcResult ac_runtime_batch_get_dispatch_times(const AcCommandBatch* batch, uint64_t* out_ns, uint32_t capacity,
                                             uint32_t* out_count) {
    if (out_count) *out_count = 0;
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (!out_ns || !out_count) return AC_ERR_NULL_POINTER;
    if (!(batch->flags & AC_BATCH_FLAG_DISPATCH_TIMESTAMPS)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (batch->state != AcCommandBatch::SUBMITTED) return AC_ERR_INVALID_ARGUMENT;
    const uint32_t n = (uint32_t)batch->t_after.size();
    if (capacity < n) return AC_ERR_INVALID_BUFFER_SIZE;
    DeviceGuard g(batch->ctx->device);
    if (n && cudaEventQuery(batch->t_after[n - 1]) != cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_DEVICE_BUSY;
    }
    cudaEvent_t prev = batch->t_begin;
    for (uint32_t i = 0; i < n; ++i) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, prev, batch->t_after[i]);
        out_ns[i] = (uint64_t)((double)ms * 1e6);
        prev = batch->t_after[i];
    }
    *out_count = n;
    return AC_SUCCESS;
}

AcResult ac_runtime_batch_get_stats(const AcCommandBatch* batch, AcBatchStats* out_stats) {
    if (!bat_ok(batch)) return AC_ERR_INVALID_ARGUMENT;
    if (!out_stats) return AC_ERR_NULL_POINTER;
    if (!abi_ok(out_stats->abi_version, out_stats->struct_size, sizeof(AcBatchStats))) return AC_ERR_INVALID_ARGUMENT;
    const uint32_t v = out_stats->abi_version, s = out_stats->struct_size;
    *out_stats = batch->stats;
    out_stats->abi_version = v;
    out_stats->struct_size = s;
    return AC_SUCCESS;
}

// ---- pipeline cache --------------------------------------------------------------------------------------------------
AcResult ac_runtime_pipeline_cache_merge(AcContext* ctx, const void* data, size_t size) {
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (size && !data) return AC_ERR_NULL_POINTER;
    return size == 0 ? AC_SUCCESS : AC_ERR_INVALID_ARGUMENT;
}
AcResult ac_runtime_pipeline_cache_get_data(AcContext* ctx, void*, size_t* inout_size) {
    if (!ctx_ok(ctx)) return AC_ERR_INVALID_CONTEXT;
    if (!inout_size) return AC_ERR_NULL_POINTER;
    *inout_size = 0;
    return AC_SUCCESS;
}

// ---- error state (src/runtime/ac_error.cpp:30-93) --------------------------------------------------------------------
static std::mutex s_err_mutex;
static std::unordered_map<uint64_t, AmevaBackendErrorState> s_err;

static AmevaBackendErrorState& err_state(uint64_t id) {
    auto it = s_err.find(id);
    if (it == s_err.end()) {
        AmevaBackendErrorState init;
        memset(&init, 0, sizeof(init));
        init.generation = 1;
        it = s_err.emplace(id, init).first;
    }
    return it->second;
}
static void err_clear(AmevaBackendErrorState& s) {
    s.first_error = 0;
    s.operation = AMEVA_BACKEND_OP_NONE;
    s.offset = s.requested_bytes = s.capacity_bytes = 0;
}

void ac_runtime_set_error_ctx(uint64_t id, int32_t code, AmevaBackendOpKind op, size_t offset, size_t req, size_t cap) {
    if (code == 0) return;
    std::lock_guard<std::mutex> lock(s_err_mutex);
    AmevaBackendErrorState& s = err_state(id);
    if (s.first_error == 0) {
        s.first_error = code;
        s.operation = op;
        s.offset = offset;
        s.requested_bytes = req;
        s.capacity_bytes = cap;
    }
}
AmevaBackendErrorState ac_runtime_get_error_state_ctx(uint64_t id) {
    std::lock_guard<std::mutex> lock(s_err_mutex);
    return err_state(id);
}
int32_t ac_runtime_consume_error_ctx(uint64_t id) {
    std::lock_guard<std::mutex> lock(s_err_mutex);
    AmevaBackendErrorState& s = err_state(id);
    const int32_t e = s.first_error;
    err_clear(s);
    return e;
}
uint64_t ac_runtime_advance_generation_ctx(uint64_t id) {
    std::lock_guard<std::mutex> lock(s_err_mutex);
    AmevaBackendErrorState& s = err_state(id);
    s.generation++;
    err_clear(s);
    return s.generation;
}
uint64_t ac_runtime_get_generation_ctx(uint64_t id) {
    std::lock_guard<std::mutex> lock(s_err_mutex);
    return err_state(id).generation;
}
void ac_runtime_reset_error_state_ctx(uint64_t id) {
    std::lock_guard<std::mutex> lock(s_err_mutex);
    err_clear(err_state(id));
}
void ac_runtime_set_error(int32_t code, AmevaBackendOpKind op, size_t offset, size_t req, size_t cap) {
    ac_runtime_set_error_ctx(AC_GLOBAL_CONTEXT_ID, code, op, offset, req, cap);
}
AmevaBackendErrorState ac_runtime_get_error_state(void) { return ac_runtime_get_error_state_ctx(AC_GLOBAL_CONTEXT_ID); }
int32_t ac_runtime_consume_error(void) { return ac_runtime_consume_error_ctx(AC_GLOBAL_CONTEXT_ID); }
uint64_t ac_runtime_advance_generation(void) { return ac_runtime_advance_generation_ctx(AC_GLOBAL_CONTEXT_ID); }
uint64_t ac_runtime_get_generation(void) { return ac_runtime_get_generation_ctx(AC_GLOBAL_CONTEXT_ID); }
void ac_runtime_reset_error_state(void) { ac_runtime_reset_error_state_ctx(AC_GLOBAL_CONTEXT_ID); }

}  // extern "C"
