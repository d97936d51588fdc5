// Cross-GPU barrier for the ranks of one box (one process per GPU), over peer-mapped flag words.
//
// After a row-sharded mul_mat whose epilogue stored its rows into every rank's output buffer, each rank needs to know
// that all the other ranks' stores have landed before it reads its own copy. Every rank launches this kernel in stream
// order after its mul_mat: thread i publishes the epoch into word [rank] of rank i's flag array (a system-scope release
// after a system fence, so the mul_mat's peer stores are visible first), then waits until word [i] of its own array
// reaches the epoch. The wait is bounded (about a second); on expiry the kernel records DEV_STATUS_WAIT_TIMEOUT in the
// context's status words and returns. Ranks run on different GPUs, so the kernels that wait on one another never share
// a device. The reference is single-device and has nothing like it.
#include "common.cuh"

namespace amv {

struct PeerFlags {
    uint32_t* p[8];
};

__global__ void peer_barrier_kernel(const PeerFlags pf, uint32_t rank, uint32_t world, uint32_t epoch,
                                    uint32_t* status) {   // epoch is reassigned below when it is 0
    const uint32_t t = threadIdx.x;
    // epoch 0 = count the uses in word 16 of the own flag array (every rank runs the same sequence of barriers), which
    // lets a recorded step be replayed without re-recording its push constants
    __shared__ uint32_t s_epoch;
    if (t == 0) {
        uint32_t e = epoch;
        if (e == 0u) {
            e = pf.p[rank][16] + 1u;
            pf.p[rank][16] = e;
        }
        s_epoch = e;
    }
    __syncthreads();
    epoch = s_epoch;
    if (t >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.p[t] + rank), "r"(epoch) : "memory");
    const uint32_t* mine = pf.p[rank] + t;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        if (clock64() - t0 > 2000000000ll) {
            if (atomicCAS(status, DEV_STATUS_OK, DEV_STATUS_WAIT_TIMEOUT) == DEV_STATUS_OK) status[1] = 0xB00u | t;
            break;
        }
        __nanosleep(100);
    }
}

// ameva_peer_barrier: bindings 0..7 the flag arrays (>= 128 bytes each, zeroed before the first use) of ranks 0..7 (slot
// `rank` is the local one, unused slots repeat it); push {rank, world (2..8), epoch}: epoch > 0 increasing by one per
// use, or 0 to let the kernel count its uses itself (word 16 of the own array)
AcResult launch_peer_barrier(const LaunchArgs& a) {
    const uint32_t rank = a.push[0], world = a.push[1], epoch = a.push[2];
    if (world < 2u || world > 8u || rank >= world) return AC_ERR_KERNEL_ARG_INVALID;
    PeerFlags pf;
    for (uint32_t i = 0; i < 8u; ++i) {
        if (a.range[i] < 128u) return AC_ERR_INVALID_BUFFER_SIZE;
        pf.p[i] = (uint32_t*)a.ptr[i];
    }
    peer_barrier_kernel<<<1, 32, 0, a.stream>>>(pf, rank, world, epoch, a.status);
    return check_launch();
}

}  // namespace amv
