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

// ---------------------------------------------------------------------------------------------------------------------
// Output exchange of a row-sharded mul_mat, decode sizes (M <= 8): push + barrier in one kernel. CTA j serves peer j: it
// copies this rank's slice of the output (rows m = 0..M-1, `count` floats at `offset` floats into each row) from the
// local output into the same place of peer j's output with 16-byte stores, then publishes the epoch into peer j's flag
// array (system-scope release after a system fence) and waits, bounded, until peer j has published into this rank's:
// when the kernel ends, every peer's slice is in the local output. The GEMV writes only local memory, so its stores
// stay coalesced and nothing of it waits on NVLink. Epoch 0 = CTA j counts its own uses in word 16 + j of the local flag
// array (a recorded step can be replayed).
// ---------------------------------------------------------------------------------------------------------------------
struct PushArgs {
    uint32_t* flags[8];     // flag arrays of ranks 0..7 (slot `rank` = the local one)
    const float* src;       // local output
    float* dst[8];          // outputs of ranks 0..7 (slot `rank` unused)
};

__global__ void __launch_bounds__(256) peer_push_barrier_kernel(const PushArgs pa, uint32_t rank, uint32_t world,
                                                                uint32_t epoch, uint32_t M, uint32_t stride,
                                                                uint32_t offset, uint32_t count, uint32_t* status) {
    const uint32_t peer = blockIdx.x + (blockIdx.x >= rank ? 1u : 0u);   // the j-th other rank
    if (peer >= world) return;
    // the slice, 16 bytes at a time where alignment allows (offset, count and stride multiples of 4 floats)
    const bool vec = ((offset | count | stride) & 3u) == 0u;
    float* dst = pa.dst[peer];
    if (vec) {
        const uint32_t per_row = count >> 2;
        for (uint32_t i = threadIdx.x; i < M * per_row; i += blockDim.x) {
            const uint32_t m = i / per_row, c = i - m * per_row;
            const size_t at = (size_t)m * stride + offset + 4u * c;
            *reinterpret_cast<float4*>(dst + at) = *reinterpret_cast<const float4*>(pa.src + at);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < M * count; i += blockDim.x) {
            const uint32_t m = i / count, c = i - m * count;
            const size_t at = (size_t)m * stride + offset + c;
            dst[at] = pa.src[at];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x != 0) return;
    uint32_t* mine = pa.flags[rank];
    uint32_t e = epoch;
    if (e == 0u) {
        e = mine[16u + peer] + 1u;
        mine[16u + peer] = e;
    }
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pa.flags[peer] + rank), "r"(e) : "memory");
    const uint32_t* wait_on = mine + peer;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_on) : "memory");
        if ((int32_t)(v - e) >= 0) break;
        if (clock64() - t0 > 2000000000ll) {
            if (atomicCAS(status, DEV_STATUS_OK, DEV_STATUS_WAIT_TIMEOUT) == DEV_STATUS_OK) status[1] = 0xB80u | peer;
            break;
        }
        __nanosleep(100);
    }
}

// ameva_peer_push_barrier: bindings 0..7 the flag arrays of ranks 0..7 (>= 128 bytes, zeroed before the first use; slot
// `rank` the local one, unused slots repeat it), 8..15 the outputs of ranks 0..7 (slot `rank` = the local output, the
// source; unused slots repeat it);
// push {rank, world (2..8), epoch (0 = counted by the kernel), M, stride (floats between rows), offset (floats into a
// row where this rank's slice starts), count (floats of the slice per row)}
AcResult launch_peer_push_barrier(const LaunchArgs& a) {
    const uint32_t rank = a.push[0], world = a.push[1], epoch = a.push[2], M = a.push[3], stride = a.push[4],
                   offset = a.push[5], count = a.push[6];
    if (world < 2u || world > 8u || rank >= world || M == 0 || M > 8u || count == 0 || (uint64_t)offset + count > stride)
        return AC_ERR_KERNEL_ARG_INVALID;
    PushArgs pa;
    const uint64_t need = ((uint64_t)(M - 1) * stride + offset + count) * 4u;
    for (uint32_t i = 0; i < 8u; ++i) {
        if (a.range[i] < 128u) return AC_ERR_INVALID_BUFFER_SIZE;
        pa.flags[i] = (uint32_t*)a.ptr[i];
        if (i < world && a.range[8 + i] < need) return AC_ERR_INVALID_BUFFER_SIZE;
        if ((uintptr_t)a.ptr[8 + i] & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
        pa.dst[i] = (float*)a.ptr[8 + i];
    }
    pa.src = (const float*)a.ptr[8 + rank];
    peer_push_barrier_kernel<<<world - 1u, 256, 0, a.stream>>>(pa, rank, world, epoch, M, stride, offset, count, a.status);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// Output exchange, prefill sizes: the copy engines push this rank's column block of a chunk of token rows to every peer
// while the tensor cores work on the next chunk. ameva_peer_copy forks the context's side queues off its stream (one
// per peer) and queues one strided device-to-device copy on each; ameva_peer_join makes the stream wait for all copies
// queued since the last join (ameva_peer_barrier then tells the other ranks, and learns from them, that the data is in
// place). No SM takes part in the transfer.
// ---------------------------------------------------------------------------------------------------------------------
static bool side_ready(SideQueues* sq) {
    if (sq->ready) return true;
    memset(sq, 0, sizeof(*sq));
    bool ok = cudaEventCreateWithFlags(&sq->fork, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 8 && ok; ++i)
        ok = cudaStreamCreateWithFlags(&sq->stream[i], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&sq->done[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        return false;   // (what was created is released with the context)
    }
    sq->ready = true;
    return true;
}

// ameva_peer_copy: bindings 0 the local output (source), 1..7 the same range of up to seven peers' outputs (unused slots
// repeat binding 0); push {rows, width_bytes (of the column block), pitch_bytes (between rows), n_peers}. Binding
// offsets select the first row and the column block (the same offset in every output).
AcResult launch_peer_copy(const LaunchArgs& a) {
    const uint32_t rows = a.push[0], width = a.push[1], pitch = a.push[2], n_peers = a.push[3];
    if (rows == 0 || width == 0 || width > pitch || n_peers == 0 || n_peers > 7u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t need = (uint64_t)(rows - 1) * pitch + width;
    for (uint32_t i = 0; i <= n_peers; ++i)
        if (a.range[i] < need) return AC_ERR_INVALID_BUFFER_SIZE;
    if (!a.side || !side_ready(a.side)) return AC_ERR_DRIVER_INIT_FAILED;
    SideQueues* sq = a.side;
    if (cudaEventRecord(sq->fork, a.stream) != cudaSuccess) return AC_ERR_DRIVER_CRASH_OR_LOST;
    for (uint32_t i = 0; i < n_peers; ++i) {
        if (cudaStreamWaitEvent(sq->stream[i], sq->fork, 0) != cudaSuccess ||
            cudaMemcpy2DAsync(a.ptr[1 + i], pitch, a.ptr[0], pitch, width, rows, cudaMemcpyDeviceToDevice,
                              sq->stream[i]) != cudaSuccess ||
            cudaEventRecord(sq->done[i], sq->stream[i]) != cudaSuccess) {
            cudaGetLastError();
            return AC_ERR_DRIVER_CRASH_OR_LOST;
        }
        sq->pending[i] = true;
    }
    return AC_SUCCESS;
}

// ameva_peer_join: binding 0 any buffer of the context (unused); no push constants.
AcResult launch_peer_join(const LaunchArgs& a) {
    if (!a.side || !a.side->ready) return AC_SUCCESS;   // nothing was ever queued
    for (int i = 0; i < 8; ++i) {
        if (!a.side->pending[i]) continue;
        if (cudaStreamWaitEvent(a.stream, a.side->done[i], 0) != cudaSuccess) {
            cudaGetLastError();
            return AC_ERR_DRIVER_CRASH_OR_LOST;
        }
        a.side->pending[i] = false;
    }
    return AC_SUCCESS;
}

}  // namespace amv
