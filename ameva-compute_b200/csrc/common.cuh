// Shared device helpers and the launcher contract of the built-in kernel registry (sm_100a only).
#pragma once
#include <cstring>

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ac_runtime_b200.h"
#include "per_device.h"

namespace amv {

// ---------------------------------------------------------------------------------------------------------------------
// Launcher contract. A dispatch hands the launcher the device address and byte range of every binding (base + offset of
// the bound range), the push constants zero-padded to the kernel's declared size, the caller's grid, and the context's
// device status words. Launchers validate shapes and ranges and return an AcResult: they never fall back to another
// implementation.
// ---------------------------------------------------------------------------------------------------------------------
// Side queues of a context: streams for copy-engine transfers that run beside the context's own stream (the output
// exchange of a row-sharded mul_mat). Created on first use; a launcher forks them off the main stream with `fork`, the
// join launcher makes the main stream wait for every `done` event recorded since.
struct SideQueues {
    cudaStream_t stream[8];
    cudaEvent_t done[8];
    cudaEvent_t fork;
    bool ready;        // streams and events exist
    bool pending[8];   // work was queued on stream i since the last join
};

struct LaunchArgs {
    cudaStream_t stream;
    uint32_t binding_count;
    void* ptr[16];
    uint64_t range[16];
    uint32_t push[32];
    AcDim3 grid;
    uint32_t* status;  // 4 device words owned by the context: [0] error code, [1] detail, [2..3] reserved
    int sm_count;
    uint32_t* workspace;      // device words owned by the context, zero between launches (cross-CTA sequence flags)
    uint64_t workspace_bytes;
    SideQueues* side;         // the context's side queues (copy launchers)
};

typedef AcResult (*LaunchFn)(const LaunchArgs&);

struct KernelEntry {
    const char* name;
    uint32_t binding_count;
    uint32_t push_bytes;
    AcDim3 local_size;
    LaunchFn launch;               // built-in kernels
    AcB200LaunchFn ext = nullptr;  // kernels added by ac_b200_kernel_register (launch is null)
};

const KernelEntry* find_kernel(const char* name);
uint32_t kernel_count();
const KernelEntry* kernel_at(uint32_t i);
AcResult register_kernel(const char* name, uint32_t binding_count, uint32_t push_bytes, AcB200LaunchFn fn);
// repack.cu: the ggml -> device-regions permutation of blocks [first, first + nblk) of a tensor, from staged ggml bytes
AcResult launch_repack(cudaStream_t stream, uint32_t type, const void* src, void* q_region, void* s_region, uint64_t first,
                       uint64_t nblk);

inline AcResult check_launch() {
    return cudaGetLastError() == cudaSuccess ? AC_SUCCESS : AC_ERR_INVALID_WORK_GROUP_SIZE;
}

// Device status codes written by kernels that give up on a bounded wait (never a trap).
enum : uint32_t { DEV_STATUS_OK = 0, DEV_STATUS_WAIT_TIMEOUT = 1, DEV_STATUS_BAD_INDEX = 2 };

inline int current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return dev;
}

#ifdef __CUDACC__
// Raises the dynamic shared-memory limit of `Kernel` on the current device, once per device (the attribute is kept per
// device, so a second GPU used by the same process needs its own call).
template <auto* Kernel>
inline bool ensure_dynamic_smem(int bytes) {
    static PerDeviceOnce once;
    return once.run_once(current_device(), [&]() {
        if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        return true;
    });
}

// ---------------------------------------------------------------------------------------------------------------------
// Timeline build (-DAMV_TRACE=1): thread 0 of the first kTraceCtas CTAs of an instrumented kernel records the global
// nanosecond timer at up to 16 points of each launch (a ring of 64 launches per CTA), read back with
// ac_b200_trace_read_<file> (AMV_TRACE_READER: the stamps are kept per translation unit). Off by default: production
// kernels carry none of it.
#ifndef AMV_TRACE
#define AMV_TRACE 0
#endif
#if AMV_TRACE
constexpr uint32_t kTraceCtas = 256, kTraceLaunches = 64, kTraceStamps = 16;
static __device__ unsigned long long g_trace[kTraceCtas * kTraceLaunches * kTraceStamps];
static __device__ unsigned int g_trace_count[kTraceCtas];
__device__ __forceinline__ uint32_t trace_begin(uint32_t cta) {   // thread 0 only; returns the slot of this launch
    if (cta >= kTraceCtas) return 0xFFFFFFFFu;
    const uint32_t n = g_trace_count[cta];
    g_trace_count[cta] = n + 1u;
    return (cta * kTraceLaunches + (n % kTraceLaunches)) * kTraceStamps;
}
__device__ __forceinline__ void trace_stamp(uint32_t slot, uint32_t i) {
    if (slot == 0xFFFFFFFFu) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_trace[slot + i] = t;
}
#define AMV_TRACE_BEGIN(cta) uint32_t amv_trace_slot = 0xFFFFFFFFu; if (threadIdx.x == 0) amv_trace_slot = trace_begin(cta);
#define AMV_TRACE_STAMP(i) if (threadIdx.x == 0) trace_stamp(amv_trace_slot, i);
// for kernels whose roles live in different threads: thread 0 publishes the slot in shared memory (after a barrier the
// kernel already has), any one thread of a role stamps
#define AMV_TRACE_SHARE(var) if (threadIdx.x == 0) var = amv_trace_slot;
#define AMV_TRACE_STAMP_AT(var, i) trace_stamp(var, i);
// copies the stamps ([cta][launch % 64][16] nanosecond timers) and the per-CTA launch counts of this file's kernels out
#define AMV_TRACE_READER(file)                                                                             \
    extern "C" int ac_b200_trace_read_##file(unsigned long long* stamps, unsigned int* counts) {            \
        if (cudaDeviceSynchronize() != cudaSuccess) return -1;                                              \
        if (cudaMemcpyFromSymbol(stamps, amv::g_trace, sizeof(amv::g_trace)) != cudaSuccess) return -2;     \
        if (cudaMemcpyFromSymbol(counts, amv::g_trace_count, sizeof(amv::g_trace_count)) != cudaSuccess) return -3; \
        return 0;                                                                                           \
    }
#else
#define AMV_TRACE_BEGIN(cta)
#define AMV_TRACE_STAMP(i)
#define AMV_TRACE_SHARE(var)
#define AMV_TRACE_STAMP_AT(var, i)
#define AMV_TRACE_READER(file)
#endif

// Programmatic dependent launch. The quantize and mul_mat kernels are launched with the attribute (launch_pdl) and begin
// with pdl_wait, which returns when the preceding grid of the stream has completed and its writes are visible, followed
// by pdl_trigger, which lets the next kernel of the stream be scheduled once all CTAs of this grid have started. Nothing
// touches memory before its wait, so only launch latency and set-up overlap. After a kernel that never triggers (the
// peer barrier), or a copy, the dependent simply starts when that work is done.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------------------------------------------
// Loads. Weights are streamed exactly once, so they bypass L1 (which is left to the activation vector every warp of the
// SM re-reads).
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
struct __align__(32) u32x8 {
    uint32_t v[8];
};
__device__ __forceinline__ u32x8 ld_stream_u8(const void* p) {  // 256-bit load (sm_100)
    u32x8 r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
                   "=r"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint16_t ld_stream_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached_u4(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
#endif  // __CUDACC__

// Layout constants shared by host packer and kernels.
// Device weight layout ("regions"): the quant payloads of all blocks first (padded to a multiple of 64 bytes), then the
// scale fields of all blocks, both in block order (row-major over [N][K/blk]).
//   Q4_0: Q 16 B/unit, S 2 B/unit (fp16 d)             Q8_0: Q 32 B/unit, S 2 B/unit
//   Q4_K: Q 128 B/block, S 16 B/block (d, dmin, scales[12])   I2_S: unchanged (already dense: K/4 bytes per row)
constexpr int kQ40QBytes = 16, kQ80QBytes = 32, kQ4KQBytes = 128, kQ4KSBytes = 16;
// Quantized-activation scratch:
//   per-32  : AQ int8 [M][K];  AD uint32 [M][K/32]  = fp16 d bits | int16 sum(q) << 16
//   per-256 : AQ int8 [M][K];  AB 48 B  [M][K/256]  = int16 bsums[16] @0, float d @32, 12 B pad
//   per-token: AQ int8 [M][K]; ACT uint32 [M][2]    = bits of 1/scale, sum(q)
constexpr int kABBytes = 48;

}  // namespace amv
