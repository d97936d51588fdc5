// Decode mul_mat (Q4_0 weights x fp32 activations, M <= 8) for callers that cannot allocate device memory.
//
// Some hosts drive the GPU from places where cudaMalloc is off limits: a real-time or interrupt-like callback that must
// not take the allocator's locks, a plugin that was handed a fixed memory budget at load time and nothing after it, a
// sandbox whose policy forbids allocation once inference has started. The regular path needs scratch for the
// quantized activations (int8 values + one scale word per 32 of them) that somebody has to own; here the library owns
// it, as a fixed array that is part of the loaded module. The caller still passes every input and the output.
//
// Cost and limits: the array below (294 912 bytes) stays resident on every GPU that loads this library until the
// process exits. Shapes are capped at kMaxRows token rows and kMaxK elements per row; larger ones are refused with
// AC_ERR_INVALID_SHAPE (and an entry in the runtime's error state giving the requested and the maximum byte counts).
// All calls share the one array and the kernels rewrite it from the start on each call, so nothing has to be cleared
// between calls; two calls whose GPU work overlaps (different streams, or different host threads) race on it and must
// be serialised by the caller.
#include <mutex>

#include "common.cuh"

namespace amv {
AcResult launch_quant_a8(const LaunchArgs&);
AcResult launch_mmvq_q4_0(const LaunchArgs&);
}  // namespace amv

namespace {

constexpr uint32_t kMaxRows = 8;      // activation (token) rows per call
constexpr uint32_t kMaxK = 32768;     // elements per row
constexpr size_t kQuantBytes = (size_t)kMaxRows * kMaxK;              // int8 values
constexpr size_t kScaleBytes = (size_t)kMaxRows * (kMaxK / 32) * 4;   // one word per 32 values
constexpr size_t kScratchBytes = kQuantBytes + kScaleBytes;

// Device-resident scratch. In host code this name is only a handle for the runtime (cudaGetSymbolAddress); it is not
// an address a kernel can be given.
static __device__ __align__(256) uint8_t g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
uint8_t* g_scratch_ptr[kMaxDevices];   // device address of g_static_scratch on each device, once looked up

// Looks the array's device address up once per device, with that device current.
AcResult scratch_for_current_device(uint8_t** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return AC_ERR_INVALID_CONTEXT;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return AC_ERR_DRIVER_INIT_FAILED;
        }
        g_scratch_ptr[dev] = static_cast<uint8_t*>(p);
    }
    *out = g_scratch_ptr[dev];
    return AC_SUCCESS;
}

}  // namespace

// dst[m][n] = sum_k W[n][k] * x[m][k] for Q4_0 weights in the device layout (w_payload: 16 bytes per 32 weights,
// w_scales: one fp16 per 32 weights, both row-major over [N][K/32]), quantizing x per 32 values on the fly exactly as
// the regular path does. All pointers are device addresses on the current device; x rows are x_stride floats apart
// (a multiple of 4), dst rows dst_stride floats apart. The work is enqueued on `stream` (a cudaStream_t; NULL is the
// default stream) and not waited for. The kernels read x and w_payload with 16-byte loads, w_scales with 2-byte loads
// and write dst as floats: x and w_payload must be 16-byte aligned, w_scales 2-byte and dst 4-byte aligned, otherwise
// the call is refused with AC_ERR_BUFFER_ALIGNMENT_INVALID before anything is launched (a misaligned device load would
// be a fault on the GPU, not an error code). The scratch used is the array of the device that is current at the call,
// which must be the device `stream` belongs to.
//
// The first call on each device looks up the scratch array's address (and may load the module): make that call before
// starting any stream capture. The function calls no cudaMalloc, cudaFree or allocating library routine.
extern "C" AcResult ac_b200_mul_mat_q4_0_static(void* stream, const void* w_payload, const void* w_scales,
                                                const float* x, uint32_t x_stride, float* dst, uint32_t dst_stride,
                                                uint32_t M, uint32_t N, uint32_t K, uint32_t round_mode) {
    if (!w_payload || !w_scales || !x || !dst) return AC_ERR_NULL_POINTER;
    if (M == 0 || N == 0 || K == 0 || (K & 31u) || x_stride < K || (x_stride & 3u) || dst_stride < N || round_mode > 1u)
        return AC_ERR_KERNEL_ARG_INVALID;
    if (((uintptr_t)x & 15u) || ((uintptr_t)w_payload & 15u) || ((uintptr_t)w_scales & 1u) || ((uintptr_t)dst & 3u))
        return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    if (M > kMaxRows || K > kMaxK) {
        const size_t want = (size_t)M * K + (size_t)M * (K / 32) * 4;
        ac_runtime_set_error((int32_t)AC_ERR_INVALID_SHAPE, AMEVA_BACKEND_OP_DISPATCH, 0, want, kScratchBytes);
        return AC_ERR_INVALID_SHAPE;
    }
    uint8_t* scratch = nullptr;
    const AcResult sr = scratch_for_current_device(&scratch);
    if (sr != AC_SUCCESS) return sr;
    uint8_t* aq = scratch;                  // int8 [M][K]
    uint8_t* ad = scratch + kQuantBytes;    // uint32 [M][K/32]
    const uint64_t U = K >> 5;

    amv::LaunchArgs a{};
    a.stream = static_cast<cudaStream_t>(stream);
    a.grid = {1, 1, 1};
    a.binding_count = 3;
    a.ptr[0] = const_cast<float*>(x);
    a.range[0] = ((uint64_t)(M - 1) * x_stride + K) * 4u;
    a.ptr[1] = aq;
    a.range[1] = kQuantBytes;
    a.ptr[2] = ad;
    a.range[2] = kScaleBytes;
    a.push[0] = M;
    a.push[1] = K;
    a.push[2] = x_stride;
    a.push[3] = round_mode;
    AcResult r = amv::launch_quant_a8(a);
    if (r != AC_SUCCESS) return r;

    amv::LaunchArgs g{};
    g.stream = a.stream;
    g.grid = {1, 1, 1};
    g.binding_count = 5;
    g.ptr[0] = const_cast<void*>(w_payload);
    g.range[0] = (uint64_t)N * U * 16u;
    g.ptr[1] = const_cast<void*>(w_scales);
    g.range[1] = (uint64_t)N * U * 2u;
    g.ptr[2] = aq;
    g.range[2] = kQuantBytes;
    g.ptr[3] = ad;
    g.range[3] = kScaleBytes;
    g.ptr[4] = dst;
    g.range[4] = ((uint64_t)(M - 1) * dst_stride + N) * 4u;
    g.push[0] = M;
    g.push[1] = N;
    g.push[2] = K;
    g.push[3] = dst_stride;
    return amv::launch_mmvq_q4_0(g);
}
