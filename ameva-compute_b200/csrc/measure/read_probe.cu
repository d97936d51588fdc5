// Read-only streaming probe: how fast can this GPU read a weight region of a given size, with nothing else to do?
//
// The decode GEMV is bounded by reading the packed weights once. A copy benchmark (read + write, seconds long) overstates
// what a read of one weight matrix can reach: a 130 MB read is over in about 30 us, and the ramp and the tail of the
// launch are a fixed part of that. bench.py times this kernel over the same weight regions, in the same way as the
// GEMV, and reports it beside the roofline fraction. The reference has nothing like it. A measurement aid, so it is not
// one of the runtime's kernels: it is built into a library of its own (libac_b200_measure.so) whose one entry point adds
// it to a process's kernel table through ac_b200_kernel_register, under the name "measure_read_probe".
#include "../common.cuh"

namespace amv {

__global__ void __launch_bounds__(256) read_probe_kernel(const uint4* __restrict__ src, size_t n16, uint32_t* sink) {
    pdl_wait();
    pdl_trigger();
    uint32_t acc = 0u;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < n16; i += 2 * stride) {   // two 16-byte loads in flight per thread
        const uint4 a = ld_stream_u4(src + i), b = ld_stream_u4(src + i + stride);
        acc += (a.x ^ a.y ^ a.z ^ a.w) + (b.x ^ b.y ^ b.z ^ b.w);
    }
    if (i < n16) {
        const uint4 a = ld_stream_u4(src + i);
        acc += a.x ^ a.y ^ a.z ^ a.w;
    }
    if (acc == 0x9E3779B9u) sink[0] = acc;   // keeps the loads alive; practically never taken
}

// measure_read_probe: binding 0 the region to read (16-byte aligned), binding 1 a sink of >= 4 bytes; push {bytes as two
// 32-bit halves, low first}: 0 = the whole range of binding 0
static AcResult launch_read_probe(const AcB200Launch* a) {
    size_t bytes = ((size_t)a->push[1] << 32) | a->push[0];
    if (bytes == 0) bytes = a->range[0];
    if (bytes > a->range[0]) return AC_ERR_INVALID_BUFFER_SIZE;
    if (a->range[1] < 4u) return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)a->ptr[0] % 16u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const size_t n16 = bytes / 16u;
    if (n16 == 0) return AC_SUCCESS;
    const unsigned grid = (unsigned)min((size_t)a->sm_count * 8u, (n16 + 255u) / 256u);
    launch_pdl(read_probe_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)a->stream, (const uint4*)a->ptr[0], n16,
               (uint32_t*)a->ptr[1]);
    return check_launch();
}

}  // namespace amv

// Adds the probe to the kernel table of the runtime loaded in this process. Registering twice is not an error.
extern "C" AcResult ac_b200_measure_register(void) {
    const AcResult rc = ac_b200_kernel_register("measure_read_probe", 2, 8, amv::launch_read_probe);
    return rc == AC_ERR_RESOURCE_IN_USE ? AC_SUCCESS : rc;
}
