// Device-side repack of ggml weight blocks into the device regions (payloads first, padded to 64 bytes, then the scale
// fields), fed from pinned staging chunks.
//
// The reference repacks on the CPU while uploading (adapters/llama/ggml-ameva/ggml-ameva-buffer.cpp:300-330 stages
// chunks, ggml-ameva-repack.cpp:82-247 permutes). Here the CPU only copies the caller's ggml bytes into one of two
// pinned chunks; the chunk travels host -> device asynchronously and a kernel does the permutation at memory speed while
// the CPU fills the other chunk. The permutation is a pure byte move (Q5_0 and IQ4_NL: an exactly invertible decode of
// the payload to int8, which makes them Q8_0 blocks), so reading the regions back through ac_b200_repack_from_device
// returns the uploaded bytes exactly.
#include <cstring>

#include "common.cuh"

namespace amv {

struct RepackCodec {
    uint32_t blk_bytes, q_off, q_bytes, s_off, s_bytes;   // placement of the payload / scale fields inside a ggml block
    uint32_t xcode;   // 1 (Q5_0) / 2 (IQ4_NL): the payload is decoded to 32 int8, the block becomes a Q8_0 block
};

// IQ4_NL's sixteen values (ggml's kvalues_iq4nl)
__constant__ int8_t c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// sixteen decoded weights of a Q5_0 / IQ4_NL block: `part` 0 = elements 0..15 (low nibbles), 1 = elements 16..31
__device__ __forceinline__ uint4 decode_piece(uint32_t xcode, const uint8_t* blk, uint32_t part) {
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (xcode == 8u || xcode == 9u) {
        // Q3_K / Q2_K: piece `part` (0..15) = elements 16 part ..: byte qs[32 (part / 8) + 16 (part % 2) + i], shift
        // 2 ((part % 8) / 2); Q3_K subtracts 4 where the hmask bit (part / 2) of hmask[16 (part % 2) + i] is clear
        const uint8_t* qs = blk + (xcode == 8u ? 32u : 16u) + 32u * (part >> 3) + 16u * (part & 1u);
        const uint8_t* hm = blk + 16u * (part & 1u);
        const uint32_t shift = 2u * ((part & 7u) >> 1), bit = part >> 1;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int v = (int)((qs[i] >> shift) & 3u);
            if (xcode == 8u && !((hm[i] >> bit) & 1u)) v -= 4;
            w[i >> 2] |= (uint32_t)(v & 0xFF) << (8 * (i & 3));
        }
    } else if (xcode == 6u || xcode == 7u) {
        // Q4_1 / Q5_1: `part` 0 = elements 0..15 (low nibbles), 1 = elements 16..31 (high nibbles); Q5_1 adds bit 4 from qh
        uint32_t qh = 0;
        const uint8_t* qs = blk + (xcode == 7u ? 8u : 4u);
        if (xcode == 7u) {
            const uint16_t* h = reinterpret_cast<const uint16_t*>(blk + 4);
            qh = (h[0] | ((uint32_t)h[1] << 16)) >> (16u * part);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t nib = part ? (qs[i] >> 4) : (qs[i] & 0x0Fu);
            w[i >> 2] |= (nib | (((qh >> i) & 1u) << 4)) << (8 * (i & 3));
        }
    } else if (xcode == 5u) {
        // IQ4_XS: piece `part` (0..15): sub-block ib = part / 2, low (part even) or high nibbles of qs[16 ib .. 16 ib + 15]
        const uint8_t* qs = blk + 8u + 16u * (part >> 1);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int v = c_iq4nl[(part & 1u) ? (qs[i] >> 4) : (qs[i] & 0x0Fu)];
            w[i >> 2] |= (uint32_t)(v & 0xFF) << (8 * (i & 3));
        }
    } else if (xcode == 4u) {
        // Q5_K: piece `part` (0..15) = elements 16 part .. 16 part + 15: j = part / 4 (64 elements), half = (part / 2) % 2
        // (low or high nibble), l = 16 (part % 2) + i
        const uint32_t j = part >> 2, half = (part >> 1) & 1u, l0 = 16u * (part & 1u);
        const uint8_t* qs = blk + 48u + 32u * j + l0;
        const uint8_t* qh = blk + 16u + l0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t nib = half ? (qs[i] >> 4) : (qs[i] & 0x0Fu);
            const uint32_t v = nib | (((qh[i] >> (2u * j + half)) & 1u) << 4);
            w[i >> 2] |= v << (8 * (i & 3));
        }
    } else if (xcode == 3u) {
        // Q6_K: piece `part` (0..15) = elements 16 part .. 16 part + 15 of the block: half h = part / 8, quarter
        // qr = (part % 8) / 2 (which nibble of which ql byte, which two bits of qh), l = 16 (part % 2) + j
        const uint32_t h = part >> 3, qr = (part & 7u) >> 1, l0 = 16u * (part & 1u);
        const uint8_t* ql = blk + 64u * h + l0 + ((qr & 1u) ? 32u : 0u);
        const uint8_t* qh = blk + 128u + 32u * h + l0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t nib = qr >= 2u ? (ql[j] >> 4) : (ql[j] & 0x0Fu);
            const int v = (int)(nib | (((qh[j] >> (2u * qr)) & 3u) << 4)) - 32;
            w[j >> 2] |= (uint32_t)(v & 0xFF) << (8 * (j & 3));
        }
    } else if (xcode == 1u) {
        const uint16_t* h = reinterpret_cast<const uint16_t*>(blk + 2);
        const uint32_t qh = (h[0] | ((uint32_t)h[1] << 16)) >> (16u * part);
        const uint8_t* qs = blk + 6;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t nib = part ? (qs[j] >> 4) : (qs[j] & 0x0Fu);
            const int v = (int)(nib | (((qh >> j) & 1u) << 4)) - 16;
            w[j >> 2] |= (uint32_t)(v & 0xFF) << (8 * (j & 3));
        }
    } else {
        const uint8_t* qs = blk + 2;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int v = c_iq4nl[part ? (qs[j] >> 4) : (qs[j] & 0x0Fu)];
            w[j >> 2] |= (uint32_t)(v & 0xFF) << (8 * (j & 3));
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

constexpr uint32_t kRepackTile = 256;   // blocks per CTA: 256 x 18, 22, 34, 144 or 210 bytes are whole 16-byte pieces

// One CTA moves kRepackTile consecutive blocks: the tile's bytes are loaded into shared memory with coalesced 16-byte
// loads (a tile starts on a 16-byte boundary of the staging chunk), then every thread assembles 16-byte payload pieces
// (fields sit on 2-byte boundaries inside a block) and 2-byte scale pieces and stores them coalesced.
__global__ void __launch_bounds__(256) repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst_q,
                                                     uint8_t* __restrict__ dst_s, uint64_t nblk, const RepackCodec c) {
    extern __shared__ __align__(16) uint8_t tile[];
    const uint64_t b0 = (uint64_t)blockIdx.x * kRepackTile;
    const uint32_t nb = (uint32_t)min((uint64_t)kRepackTile, nblk - b0);
    const uint32_t bytes = nb * c.blk_bytes;
    const uint8_t* s = src + b0 * c.blk_bytes;
    for (uint32_t i = threadIdx.x * 16u; i < bytes; i += 256u * 16u) {
        if (i + 16u <= bytes) {
            *reinterpret_cast<uint4*>(tile + i) = *reinterpret_cast<const uint4*>(s + i);
        } else {   // the ragged end of the last tile
            for (uint32_t j = i; j < bytes; ++j) tile[j] = s[j];
        }
    }
    __syncthreads();
    const uint32_t q_pieces = nb * (c.q_bytes / 16u), per_blk = c.q_bytes / 16u;
    uint8_t* q = dst_q + b0 * c.q_bytes;
    for (uint32_t p = threadIdx.x; p < q_pieces; p += 256u) {
        const uint32_t blk = p / per_blk, part = p - blk * per_blk;
        uint4 v;
        if (c.xcode) {
            v = decode_piece(c.xcode, tile + blk * c.blk_bytes, part);
        } else {
            const uint16_t* h = reinterpret_cast<const uint16_t*>(tile + blk * c.blk_bytes + c.q_off + part * 16u);
            v.x = h[0] | ((uint32_t)h[1] << 16);
            v.y = h[2] | ((uint32_t)h[3] << 16);
            v.z = h[4] | ((uint32_t)h[5] << 16);
            v.w = h[6] | ((uint32_t)h[7] << 16);
        }
        *reinterpret_cast<uint4*>(q + (size_t)p * 16u) = v;
    }
    const uint32_t s_halves = nb * (c.s_bytes / 2u), per_blk_s = c.s_bytes / 2u;
    uint16_t* sc = reinterpret_cast<uint16_t*>(dst_s + b0 * c.s_bytes);
    for (uint32_t p = threadIdx.x; p < s_halves; p += 256u) {
        const uint32_t blk = p / per_blk_s, part = p - blk * per_blk_s;
        // (Q2_K's record is two slices of the block: scales[16] at its start, d and dmin at bytes 80..83)
        const uint32_t so = (c.xcode == 9u && part >= 8u) ? 64u + part * 2u : c.s_off + part * 2u;
        sc[p] = *reinterpret_cast<const uint16_t*>(tile + blk * c.blk_bytes + so);
    }
}

static bool repack_codec(uint32_t type, RepackCodec* c, uint32_t* blk) {
    switch (type) {
        case 2: *c = {18, 2, 16, 0, 2, 0}; *blk = 32; return true;        // Q4_0: d@0, qs[16]@2
        case 8: *c = {34, 2, 32, 0, 2, 0}; *blk = 32; return true;        // Q8_0: d@0, qs[32]@2
        case 12: *c = {144, 16, 128, 0, 16, 0}; *blk = 256; return true;  // Q4_K: d, dmin, scales[12] @0, qs[128]@16
        case 6: *c = {22, 2, 32, 0, 2, 1}; *blk = 32; return true;        // Q5_0: d@0, qh[4]@2, qs[16]@6, decoded
        case 20: *c = {18, 2, 32, 0, 2, 2}; *blk = 32; return true;       // IQ4_NL: d@0, qs[16]@2, decoded
        case 14: *c = {210, 0, 256, 192, 18, 3}; *blk = 256; return true; // Q6_K: ql, qh decoded to 256 int8; scales[16] + d kept
        case 13: *c = {176, 16, 256, 0, 16, 4}; *blk = 256; return true;  // Q5_K: qh, qs decoded to 256 bytes; d, dmin, scales kept
        case 23: *c = {136, 8, 256, 0, 8, 5}; *blk = 256; return true;    // IQ4_XS: qs decoded to 256 int8; d, scales_h, scales_l kept
        case 11: *c = {110, 0, 256, 96, 14, 8}; *blk = 256; return true;  // Q3_K: hmask, qs decoded to 256 int8; scales[12] + d kept
        case 10: *c = {84, 16, 256, 0, 20, 9}; *blk = 256; return true;   // Q2_K: qs decoded to 256 bytes; scales[16], d, dmin kept
        case 3: *c = {20, 4, 32, 0, 4, 6}; *blk = 32; return true;        // Q4_1: qs decoded to 32 bytes; d, m kept
        case 7: *c = {24, 4, 32, 0, 4, 7}; *blk = 32; return true;        // Q5_1: qh, qs decoded to 32 bytes; d, m kept
        default: return false;
    }
}

// Launches the permutation of `nblk` blocks that start at block `first` of the tensor: src = the staged ggml bytes of
// those blocks (16-byte aligned), q_region / s_region = the start of the tensor's payload / scale regions.
AcResult launch_repack(cudaStream_t stream, uint32_t type, const void* src, void* q_region, void* s_region,
                       uint64_t first, uint64_t nblk) {
    RepackCodec c;
    uint32_t blk;
    if (!repack_codec(type, &c, &blk)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (nblk == 0) return AC_SUCCESS;
    if (((uintptr_t)src & 15u) || ((uintptr_t)q_region & 15u) || ((uintptr_t)s_region & 1u) || (first % kRepackTile))
        return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const uint64_t tiles = (nblk + kRepackTile - 1) / kRepackTile;
    if (tiles > 0x7fffffffull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    if (!ensure_dynamic_smem<repack_kernel>(kRepackTile * 210)) return AC_ERR_INVALID_WORK_GROUP_SIZE;   // (Q6_K tiles: 52.5 KB)
    repack_kernel<<<(unsigned)tiles, 256, kRepackTile * c.blk_bytes, stream>>>(
        (const uint8_t*)src, (uint8_t*)q_region + first * c.q_bytes, (uint8_t*)s_region + first * c.s_bytes, nblk, c);
    return check_launch();
}

}  // namespace amv
