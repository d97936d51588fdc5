// ggml backend plugin over libac_runtime_b200.so: the quantized MUL_MAT of a ggml graph on B200.
//
// Exports ggml_backend_init() / ggml_backend_score() with C linkage, as the reference's plugin does
// (adapters/llama/ggml-ameva/ggml-ameva.cpp:5693-5707), and fills the registry / device / buffer-type / buffer / backend
// tables of ggml's backend interface (ggml-backend-impl.h, API version 2). It is compiled against the ggml headers of the
// host application (llama.cpp b8471 / ggml 0.9.8 is what the reference builds with); none of ggml is part of this
// repository. Behaviour kept from the reference plugin:
//   - buffer type: alignment 64, not host memory (weights live in a device layout), alloc size = the device layout's
//     size for repacked weights, ggml_nbytes otherwise (ggml-ameva-buffer.cpp:662-696);
//   - set_tensor repacks Q4_0 / Q8_0 / Q4_K matrices into the device regions, get_tensor returns the uploaded ggml
//     bytes, partial ranges included (tests/ameva_qmm_check.cpp:184-196); ggml has no error return there, so a failed
//     transfer aborts (ggml-ameva-buffer.cpp:196-219);
//   - supports_buft = the own buffer type only, so the scheduler copies foreign inputs in (ggml-ameva-device.cpp:314-317);
//   - graph_compute checks every node first and returns GGML_STATUS_FAILED without recording anything when one cannot
//     run (ggml-ameva.cpp:5330-5341); it returns after completion (synchronize = NULL); calls are serialised by a mutex;
//   - props: async = false, host_buffer = false, events = false (ggml-ameva-device.cpp:271-281).
// Scope: MUL_MAT with a Q4_0 / Q8_0 / Q4_K src0 (2-D, contiguous) and f32 src1 / dst, plus the no-op view nodes. Other
// ops are reported unsupported, which is how the scheduler keeps them on another backend.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "ggml-backend-impl.h"
#include "ggml-backend.h"
#include "ggml.h"

// The C ABI of libac_runtime_b200.so. (Its header shares no names with ggml's.)
#include "../../include/ac_runtime_b200.h"

namespace {

constexpr size_t kAlign = 64;
char* const kBase = reinterpret_cast<char*>(0x1000);   // tensor->data = kBase + offset inside the device buffer

[[noreturn]] void die(const char* what, AcResult rc) {
    fprintf(stderr, "ggml-ameva-b200: %s failed (AcResult %d)\n", what, (int)rc);
    abort();
}

struct Plugin {                 // one per process
    std::mutex mutex;
    AcContext* ctx = nullptr;
    std::string name;
    ggml_backend_reg reg{};
    ggml_backend_device dev{};
    ggml_backend_buffer_type buft{};
};
Plugin& plugin() {
    static Plugin p;
    return p;
}

AcContext* context() {          // created on first use (the loader probes the registry without touching the device)
    Plugin& p = plugin();
    if (!p.ctx) {
        AcContextDesc d = {AC_ABI_VERSION, (uint32_t)sizeof(AcContextDesc), AC_BACKEND_CUDA, 0};
        const AcResult rc = ac_runtime_context_create(&d, &p.ctx);
        if (rc != AC_SUCCESS) return nullptr;
        char nm[128] = {0};
        ac_runtime_context_get_device_name(p.ctx, nm, sizeof(nm));
        p.name = nm;
    }
    return p.ctx;
}

bool repacked_type(enum ggml_type t) { return t == GGML_TYPE_Q4_0 || t == GGML_TYPE_Q8_0 || t == GGML_TYPE_Q4_K; }

// A weight this backend keeps in its device layout: a supported quantized type, plain 2-D, contiguous, whole 256-blocks
// for Q4_K / whole 32-blocks otherwise (ggml guarantees the latter by construction).
bool is_repacked_weight(const ggml_tensor* t) {
    return t && repacked_type(t->type) && t->ne[2] == 1 && t->ne[3] == 1 && ggml_is_contiguous(t) && t->view_src == nullptr;
}

uint64_t device_bytes(const ggml_tensor* t, uint64_t* s_off) {
    uint64_t total = 0, off = 0;
    const AcResult rc = ac_b200_device_layout((uint32_t)t->type, (uint64_t)t->ne[1], (uint64_t)t->ne[0], &total, &off);
    if (rc != AC_SUCCESS) die("ac_b200_device_layout", rc);
    if (s_off) *s_off = off;
    return total;
}

// ---- buffers ----------------------------------------------------------------------------------------------------------
struct BufferCtx {
    AcBuffer* buf = nullptr;
    size_t size = 0;
    // per repacked weight (by its offset in the buffer): the power of two the tensor-core GEMM scales the weights by
    // while dequantizing them to fp16 (ameva_mmtc_* push word w_exp), computed from the block scales at upload
    std::map<size_t, int> w_exp;
};

float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {   // subnormal: normalise
            int e = -1;
            uint32_t m = man;
            do {
                m <<= 1;
                ++e;
            } while (!(m & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// w_exp of a weight tensor from its ggml blocks: an upper bound of |w| per block from the scale fields alone (Q4_0
// 8 |d|, Q8_0 127 |d|, Q4_K 945 |d| + 63 |dmin|), the largest over the tensor brought into [1, 2); limited to -14..15.
int weight_exponent(enum ggml_type type, const uint8_t* blocks, size_t nbytes) {
    const size_t bb = type == GGML_TYPE_Q4_0 ? 18 : (type == GGML_TYPE_Q8_0 ? 34 : 144);
    float top = 0.0f;
    for (size_t o = 0; o + bb <= nbytes; o += bb) {
        uint16_t h0, h1;
        memcpy(&h0, blocks + o, 2);
        memcpy(&h1, blocks + o + 2, 2);
        const float d = fabsf(half_bits_to_float(h0));
        float bound = type == GGML_TYPE_Q4_0 ? 8.0f * d : (type == GGML_TYPE_Q8_0 ? 127.0f * d
                                                          : 945.0f * d + 63.0f * fabsf(half_bits_to_float(h1)));
        if (bound > top && bound <= 3.0e38f) top = bound;
    }
    if (!(top > 0.0f)) return 0;
    int e = 0;
    frexpf(top, &e);          // top = m * 2^e, m in [0.5, 1)  ->  floor(log2(top)) = e - 1
    const int w = -(e - 1);
    return w < -14 ? -14 : (w > 15 ? 15 : w);
}

size_t tensor_offset(const ggml_tensor* t) { return (size_t)((const char*)t->data - kBase); }

void buffer_free(ggml_backend_buffer_t buffer) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    if (b->buf) ac_runtime_buffer_destroy(b->buf);
    delete b;
}

void* buffer_get_base(ggml_backend_buffer_t) { return kBase; }

void buffer_memset_tensor(ggml_backend_buffer_t buffer, ggml_tensor* tensor, uint8_t value, size_t offset, size_t size) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    // a repacked weight has no byte-for-byte image of a partial range; whole-tensor fills are what ggml issues
    const size_t bytes = is_repacked_weight(tensor) && offset == 0 && size == ggml_nbytes(tensor)
                             ? (size_t)device_bytes(tensor, nullptr) : size;
    const AcResult rc = ac_runtime_buffer_fill(b->buf, tensor_offset(tensor) + offset, bytes, value);
    if (rc != AC_SUCCESS) die("buffer_fill", rc);
}

void buffer_set_tensor(ggml_backend_buffer_t buffer, ggml_tensor* tensor, const void* data, size_t offset, size_t size) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    if (!is_repacked_weight(tensor)) {
        const AcResult rc = ac_runtime_buffer_write(b->buf, tensor_offset(tensor) + offset, data, size);
        if (rc != AC_SUCCESS) die("buffer_write", rc);
        return;
    }
    const size_t nbytes = ggml_nbytes(tensor);
    const uint64_t rows = (uint64_t)tensor->ne[1], k = (uint64_t)tensor->ne[0];
    const uint64_t total = device_bytes(tensor, nullptr);
    std::vector<uint8_t> dev(total), blocks;
    const void* src = data;
    if (offset != 0 || size != nbytes) {   // a partial range: patch the ggml image of what is on the device
        blocks.resize(nbytes);
        AcResult rc = ac_runtime_buffer_read(b->buf, tensor_offset(tensor), dev.data(), total);
        if (rc == AC_SUCCESS) rc = ac_b200_repack_from_device((uint32_t)tensor->type, dev.data(), rows, k, blocks.data());
        if (rc != AC_SUCCESS) die("partial set_tensor read-back", rc);
        memcpy(blocks.data() + offset, data, size);
        src = blocks.data();
    }
    AcResult rc = ac_b200_repack_to_device((uint32_t)tensor->type, src, rows, k, dev.data());
    if (rc == AC_SUCCESS) rc = ac_runtime_buffer_write(b->buf, tensor_offset(tensor), dev.data(), total);
    if (rc != AC_SUCCESS) die("set_tensor", rc);
    b->w_exp[tensor_offset(tensor)] = weight_exponent(tensor->type, (const uint8_t*)src, nbytes);
}

void buffer_get_tensor(ggml_backend_buffer_t buffer, const ggml_tensor* tensor, void* data, size_t offset, size_t size) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    if (!is_repacked_weight(tensor)) {
        const AcResult rc = ac_runtime_buffer_read(b->buf, tensor_offset(tensor) + offset, data, size);
        if (rc != AC_SUCCESS) die("buffer_read", rc);
        return;
    }
    const uint64_t rows = (uint64_t)tensor->ne[1], k = (uint64_t)tensor->ne[0];
    const uint64_t total = device_bytes(tensor, nullptr);
    std::vector<uint8_t> dev(total), blocks(ggml_nbytes(tensor));
    AcResult rc = ac_runtime_buffer_read(b->buf, tensor_offset(tensor), dev.data(), total);
    if (rc == AC_SUCCESS) rc = ac_b200_repack_from_device((uint32_t)tensor->type, dev.data(), rows, k, blocks.data());
    if (rc != AC_SUCCESS) die("get_tensor", rc);
    memcpy(data, blocks.data() + offset, size);
}

void buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    const AcResult rc = ac_runtime_buffer_fill(b->buf, 0, b->size, value);
    if (rc != AC_SUCCESS) die("buffer_clear", rc);
}

ggml_backend_buffer_i buffer_iface() {
    ggml_backend_buffer_i i{};
    i.free_buffer = buffer_free;
    i.get_base = buffer_get_base;
    i.init_tensor = nullptr;
    i.memset_tensor = buffer_memset_tensor;
    i.set_tensor = buffer_set_tensor;
    i.get_tensor = buffer_get_tensor;
    i.cpy_tensor = nullptr;   // copies go through get/set
    i.clear = buffer_clear;
    i.reset = nullptr;
    return i;
}

// ---- buffer type ------------------------------------------------------------------------------------------------------
const char* buft_get_name(ggml_backend_buffer_type_t) { return "AMEVA_B200"; }

ggml_backend_buffer_t buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    std::lock_guard<std::mutex> lock(plugin().mutex);
    AcContext* ctx = context();
    if (!ctx) return nullptr;
    BufferCtx* b = new BufferCtx();
    b->size = size ? size : kAlign;
    AcBufferDesc d = {AC_ABI_VERSION, (uint32_t)sizeof(AcBufferDesc), b->size,
                      AC_BUFFER_USAGE_STORAGE | AC_BUFFER_USAGE_TRANSFER_SRC | AC_BUFFER_USAGE_TRANSFER_DST, 0};
    if (ac_runtime_buffer_create(ctx, &d, &b->buf) != AC_SUCCESS) {
        delete b;
        return nullptr;   // ggml reports the allocation failure
    }
    return ggml_backend_buffer_init(buft, buffer_iface(), b, size);
}

size_t buft_get_alignment(ggml_backend_buffer_type_t) { return kAlign; }

size_t buft_get_max_size(ggml_backend_buffer_type_t) {
    AcContext* ctx = context();
    AcDeviceLimits lim;
    memset(&lim, 0, sizeof(lim));
    lim.abi_version = AC_ABI_VERSION;
    lim.struct_size = (uint32_t)sizeof(lim);
    if (!ctx || ac_runtime_context_get_limits(ctx, &lim) != AC_SUCCESS) return SIZE_MAX;
    return (size_t)lim.max_memory_allocation_size;
}

size_t buft_get_alloc_size(ggml_backend_buffer_type_t, const ggml_tensor* tensor) {
    if (is_repacked_weight(tensor)) {
        const size_t dev = (size_t)device_bytes(tensor, nullptr), nb = ggml_nbytes(tensor);
        return dev > nb ? dev : nb;   // the device layout pads the payload region to 64 bytes
    }
    return ggml_nbytes(tensor);
}

bool buft_is_host(ggml_backend_buffer_type_t) { return false; }

// ---- backend: graph_compute -------------------------------------------------------------------------------------------
struct Backend {
    std::map<std::string, AcKernel*> kernels;
    AcBuffer* aq = nullptr;   // int8 [M][K]
    AcBuffer* ad = nullptr;   // per-block activation scales (u32 per 32 / 48 B per 256)
    AcBuffer* ah = nullptr;   // fp16 [M][K], the tensor-core operand (M > 8)
    AcBuffer* ae = nullptr;   // f32 [M], the per-row range factors of that operand
    size_t aq_bytes = 0, ad_bytes = 0, ah_bytes = 0, ae_bytes = 0;
};

AcKernel* kernel(Backend* be, const char* name) {
    auto it = be->kernels.find(name);
    if (it != be->kernels.end()) return it->second;
    AcKernel* k = nullptr;
    if (ac_runtime_kernel_create_builtin(context(), name, &k) != AC_SUCCESS) return nullptr;
    be->kernels[name] = k;
    return k;
}

// Called before a batch is begun (nothing retains the old buffer then), with the largest need over the graph's nodes, as
// the reference sizes its scratch before recording (ggml-ameva.cpp:5382-5422).
bool grow(AcBuffer** buf, size_t* have, size_t need) {
    if (*have >= need) return true;
    if (*buf) {
        const AcResult rc = ac_runtime_buffer_destroy(*buf);
        if (rc != AC_SUCCESS) {
            fprintf(stderr, "ggml-ameva-b200: scratch buffer still in use (AcResult %d)\n", (int)rc);
            return false;
        }
    }
    *buf = nullptr;
    *have = 0;
    AcBufferDesc d = {AC_ABI_VERSION, (uint32_t)sizeof(AcBufferDesc), need, AC_BUFFER_USAGE_STORAGE, 0};
    if (ac_runtime_buffer_create(context(), &d, buf) != AC_SUCCESS) return false;
    *have = need;
    return true;
}

bool is_view_op(enum ggml_op op) {
    return op == GGML_OP_NONE || op == GGML_OP_RESHAPE || op == GGML_OP_VIEW || op == GGML_OP_PERMUTE ||
           op == GGML_OP_TRANSPOSE;
}

bool own_buffer(const ggml_tensor* t) {
    const ggml_tensor* base = t->view_src ? t->view_src : t;
    return base->buffer && base->buffer->buft == &plugin().buft;
}

// Why a MUL_MAT node cannot run here; NULL when it can (the reference's mul_mat_qmm_reason, ggml-ameva.cpp:1326-1377,
// reduced to this backend's kernels).
const char* mul_mat_reason(const ggml_tensor* node) {
    const ggml_tensor *w = node->src[0], *x = node->src[1];
    if (!w || !x) return "missing operand";
    if (!is_repacked_weight(w)) return "src0 is not a 2-D contiguous Q4_0 / Q8_0 / Q4_K matrix";
    if (!own_buffer(w) || !own_buffer(x) || !own_buffer(node)) return "an operand is not in an AMEVA_B200 buffer";
    if (x->type != GGML_TYPE_F32 || node->type != GGML_TYPE_F32) return "src1 / dst are not f32";
    if (!ggml_is_contiguous(x) || !ggml_is_contiguous(node)) return "src1 / dst are not contiguous";
    if (x->ne[2] != 1 || x->ne[3] != 1 || node->ne[2] != 1 || node->ne[3] != 1) return "batched (3-D / 4-D) operands";
    if (x->ne[0] != w->ne[0] || node->ne[0] != w->ne[1] || node->ne[1] != x->ne[1]) return "shape mismatch";
    if (w->ne[0] % (w->type == GGML_TYPE_Q4_K ? 256 : 32)) return "K is not whole quantization blocks";
    if (tensor_offset(w) % kAlign || tensor_offset(x) % kAlign || tensor_offset(node) % kAlign) return "unaligned tensor";
    // more than 8 activation rows with a K the tensor-core kernel cannot take run as chunks of 8 rows through the GEMV:
    // the chunks' scratch and output offsets (8 K, K, 32 N bytes) must keep the 64-byte binding alignment
    if (x->ne[1] > 8 && w->ne[0] % 256 && (w->ne[0] % 64 || (32 * w->ne[1]) % 64)) return "chunked M > 8 needs K % 64 == 0, N % 2 == 0";
    return nullptr;
}

bool node_supported(const ggml_tensor* node) {
    if (is_view_op(node->op)) return true;
    return node->op == GGML_OP_MUL_MAT && mul_mat_reason(node) == nullptr;
}

AcBufferBinding bind(AcBuffer* b, uint64_t off, uint64_t range) {
    AcBufferBinding r = {b, off, range};
    return r;
}

// Records quantize + mul_mat of one node: the sequence of ameva-compute_b200/qmm.py MulMat.record.
bool record_mul_mat(Backend* be, AcCommandBatch* batch, const ggml_tensor* node) {
    const ggml_tensor *w = node->src[0], *x = node->src[1];
    const uint32_t K = (uint32_t)w->ne[0], N = (uint32_t)w->ne[1], M = (uint32_t)x->ne[1];
    const bool q4k = w->type == GGML_TYPE_Q4_K;
    const char* tname = w->type == GGML_TYPE_Q4_0 ? "q4_0" : (w->type == GGML_TYPE_Q8_0 ? "q8_0" : "q4_K");
    const bool tc = M > 8 && (K % 256) == 0;
    const uint64_t ad_need = q4k ? (uint64_t)M * (K / 256) * 48u : (uint64_t)M * (K / 32) * 4u;
    BufferCtx* wb = (BufferCtx*)w->buffer->context;
    BufferCtx* xb = (BufferCtx*)(x->view_src ? x->view_src : x)->buffer->context;
    BufferCtx* yb = (BufferCtx*)(node->view_src ? node->view_src : node)->buffer->context;
    uint64_t s_off = 0;
    const uint64_t wtotal = device_bytes(w, &s_off);
    const AcDim3 grid = {1, 1, 1};   // the launchers size their own grids

    // One token of a projection small enough to be launch-bound: one launch that quantizes the row inside the GEMV
    // (same bits as the two kernels below; the limits are those of qmm.py's MulMat.record).
    if (M == 1 && K <= 16384u && (uint64_t)N * K <= (64ull << 20) && tensor_offset(x) % 64 == 0 &&
        tensor_offset(node) % 64 == 0) {
        AcKernel* k = kernel(be, (std::string(q4k ? "ameva_mmvqb_" : "ameva_mmvq_") + tname + "_fq").c_str());
        if (!k) return false;
        AcBufferBinding b[4] = {bind(wb->buf, tensor_offset(w), s_off), bind(wb->buf, tensor_offset(w) + s_off, wtotal - s_off),
                                bind(xb->buf, tensor_offset(x), (uint64_t)K * 4),
                                bind(yb->buf, tensor_offset(node), (uint64_t)N * 4)};
        const uint32_t push[3] = {N, K, 0};   // ties-to-even per-32 / ggml's per-256 convention
        return ac_runtime_batch_dispatch_bindings(batch, k, b, 4, push, sizeof(push), grid) == AC_SUCCESS;
    }

    // 1. activation quantization (per-32 for Q4_0 / Q8_0, per-256 for Q4_K; fp16 operand too when M > 8)
    {
        std::string name = q4k ? "ameva_quant_a8b" : "ameva_quant_a8";
        if (tc) name += "_f16";
        AcKernel* k = kernel(be, name.c_str());
        if (!k) return false;
        AcBufferBinding b[5] = {bind(xb->buf, tensor_offset(x), (uint64_t)M * K * 4), bind(be->aq, 0, (uint64_t)M * K),
                                bind(be->ad, 0, ad_need), bind(be->ah, 0, (uint64_t)M * K * 2), bind(be->ae, 0, (uint64_t)M * 4)};
        const uint32_t push[4] = {M, K, K, 0};   // ties-to-even per-32 / ggml's per-256 convention
        if (ac_runtime_batch_dispatch_bindings(batch, k, b, tc ? 5 : 3, push, sizeof(push), grid) != AC_SUCCESS)
            return false;
        ac_runtime_batch_barrier(batch);
    }
    const AcBufferBinding Q = bind(wb->buf, tensor_offset(w), s_off), S = bind(wb->buf, tensor_offset(w) + s_off, wtotal - s_off);
    // 2. the product: tensor-core GEMM for M > 8, streaming GEMV (in chunks of 8 rows when K rules the GEMM out) else
    if (tc) {
        AcKernel* k = kernel(be, (std::string("ameva_mmtc_") + tname).c_str());
        if (!k) return false;
        AcBufferBinding b[5] = {Q, S, bind(be->ah, 0, (uint64_t)M * K * 2),
                                bind(yb->buf, tensor_offset(node), (uint64_t)M * N * 4), bind(be->ae, 0, (uint64_t)M * 4)};
        auto it = wb->w_exp.find(tensor_offset(w));
        const uint32_t push[6] = {M, N, K, N, 0, (uint32_t)(it == wb->w_exp.end() ? 0 : it->second)};
        return ac_runtime_batch_dispatch_bindings(batch, k, b, 5, push, sizeof(push), grid) == AC_SUCCESS;
    }
    // M <= 8 over short weight rows, with several activation rows or a large matrix: the GEMV that stages whole weight
    // rows in shared memory (the choice of qmm.py's MulMat.streamed_pays)
    const uint64_t row_bytes = (uint64_t)(K / 256) * ((w->type == GGML_TYPE_Q8_0 ? 256u : 128u) + 16u);
    if (M <= 8 && (K % 256) == 0 && row_bytes <= 6400u && (M >= 4 || (uint64_t)N * row_bytes >= (64ull << 20))) {
        AcKernel* ks = kernel(be, (std::string("ameva_mmvs_") + tname).c_str());
        if (!ks) return false;
        const AcBufferBinding y = bind(yb->buf, tensor_offset(node), (uint64_t)M * N * 4);
        AcBufferBinding b[12] = {Q, S, bind(be->aq, 0, (uint64_t)M * K), bind(be->ad, 0, ad_need), y, y, y, y, y, y, y, y};
        const uint32_t push[6] = {M, N, K, N, 0, 0};
        return ac_runtime_batch_dispatch_bindings(batch, ks, b, 12, push, sizeof(push), grid) == AC_SUCCESS;
    }
    AcKernel* k = kernel(be, (std::string(q4k ? "ameva_mmvqb_" : "ameva_mmvq_") + tname).c_str());
    if (!k) return false;
    for (uint32_t m0 = 0; m0 < M; m0 += 8) {
        const uint32_t mc = M - m0 < 8 ? M - m0 : 8;
        const uint64_t ad_row = q4k ? (uint64_t)(K / 256) * 48u : (uint64_t)(K / 32) * 4u;
        AcBufferBinding b[5] = {Q, S, bind(be->aq, (uint64_t)m0 * K, (uint64_t)mc * K),
                                bind(be->ad, m0 * ad_row, mc * ad_row),
                                bind(yb->buf, tensor_offset(node) + (uint64_t)m0 * N * 4, (uint64_t)mc * N * 4)};
        const uint32_t push[4] = {mc, N, K, N};
        if (ac_runtime_batch_dispatch_bindings(batch, k, b, 5, push, sizeof(push), grid) != AC_SUCCESS) return false;
    }
    return true;
}

const char* backend_get_name(ggml_backend_t) { return "AMEVA_B200"; }

void backend_free(ggml_backend_t backend) {
    Backend* be = (Backend*)backend->context;
    {
        std::lock_guard<std::mutex> lock(plugin().mutex);
        for (auto& kv : be->kernels) ac_runtime_kernel_destroy(kv.second);
        for (AcBuffer* b : {be->aq, be->ad, be->ah, be->ae})
            if (b) ac_runtime_buffer_destroy(b);
    }
    delete be;
    delete backend;
}

enum ggml_status backend_graph_compute(ggml_backend_t backend, ggml_cgraph* cgraph) {
    Backend* be = (Backend*)backend->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    const int n = ggml_graph_n_nodes(cgraph);
    for (int i = 0; i < n; ++i) {   // every node first: nothing is recorded if one cannot run
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (!node_supported(node)) {
            fprintf(stderr, "ggml-ameva-b200: node %d (%s, %s) cannot run here: %s\n", i, ggml_op_name(node->op), node->name,
                    node->op == GGML_OP_MUL_MAT ? mul_mat_reason(node) : "op not built");
            return GGML_STATUS_FAILED;
        }
    }
    // scratch for the quantized activations: the largest need over all nodes, reserved before anything is recorded
    size_t aq_need = 0, ad_need = 0, ah_need = 0, ae_need = 0;
    for (int i = 0; i < n; ++i) {
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (node->op != GGML_OP_MUL_MAT) continue;
        const ggml_tensor *w = node->src[0], *x = node->src[1];
        const size_t K = (size_t)w->ne[0], M = (size_t)x->ne[1];
        aq_need = std::max(aq_need, M * K);
        ad_need = std::max(ad_need, w->type == GGML_TYPE_Q4_K ? M * (K / 256) * 48u : M * (K / 32) * 4u);
        if (M > 8 && K % 256 == 0) {
            ah_need = std::max(ah_need, M * K * 2);
            ae_need = std::max(ae_need, M * 4);
        }
    }
    if ((aq_need && !grow(&be->aq, &be->aq_bytes, aq_need)) || (ad_need && !grow(&be->ad, &be->ad_bytes, ad_need)) ||
        (ah_need && !grow(&be->ah, &be->ah_bytes, ah_need)) || (ae_need && !grow(&be->ae, &be->ae_bytes, ae_need)))
        return GGML_STATUS_ALLOC_FAILED;
    AcCommandBatch* batch = nullptr;
    AcBatchDesc bd = {AC_ABI_VERSION, (uint32_t)sizeof(AcBatchDesc), 4096u, 0u};
    if (ac_runtime_batch_begin_ex(context(), &bd, &batch) != AC_SUCCESS) return GGML_STATUS_ALLOC_FAILED;
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (node->op == GGML_OP_MUL_MAT) {
            ok = record_mul_mat(be, batch, node);
            ac_runtime_batch_barrier(batch);
        }
    }
    if (ok) ok = ac_runtime_batch_submit(batch, nullptr) == AC_SUCCESS;   // blocks until the GPU finished
    else ac_runtime_batch_abort(batch);
    ac_runtime_batch_destroy(batch);
    return ok ? GGML_STATUS_SUCCESS : GGML_STATUS_FAILED;
}

ggml_guid_t backend_guid() {
    static ggml_guid guid = {0xa3, 0x1e, 0xb2, 0x00, 0x5c, 0x47, 0x4d, 0x0b, 0x91, 0x6a, 0xb2, 0x00, 0xac, 0xde, 0x10, 0x0a};
    return &guid;
}

// ---- device -----------------------------------------------------------------------------------------------------------
const char* dev_get_name(ggml_backend_dev_t) { return "AMEVA_B200_0"; }
const char* dev_get_description(ggml_backend_dev_t) {
    std::lock_guard<std::mutex> lock(plugin().mutex);
    return context() ? plugin().name.c_str() : "NVIDIA B200 (context unavailable)";
}
void dev_get_memory(ggml_backend_dev_t, size_t* free_b, size_t* total_b) {
    std::lock_guard<std::mutex> lock(plugin().mutex);
    AcDeviceLimits lim;
    memset(&lim, 0, sizeof(lim));
    lim.abi_version = AC_ABI_VERSION;
    lim.struct_size = (uint32_t)sizeof(lim);
    size_t v = 0;
    if (context() && ac_runtime_context_get_limits(context(), &lim) == AC_SUCCESS) v = (size_t)lim.max_memory_allocation_size;
    *free_b = v;
    *total_b = v;
}
enum ggml_backend_dev_type dev_get_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_GPU; }
ggml_backend_buffer_type_t dev_get_buffer_type(ggml_backend_dev_t) { return &plugin().buft; }
void dev_get_props(ggml_backend_dev_t dev, ggml_backend_dev_props* props) {
    memset(props, 0, sizeof(*props));
    props->name = dev_get_name(dev);
    props->description = dev_get_description(dev);
    props->type = dev_get_type(dev);
    dev_get_memory(dev, &props->memory_free, &props->memory_total);
    props->caps.async = false;
    props->caps.host_buffer = false;
    props->caps.buffer_from_host_ptr = false;
    props->caps.events = false;
}
ggml_backend_t dev_init_backend(ggml_backend_dev_t dev, const char*) {
    {
        std::lock_guard<std::mutex> lock(plugin().mutex);
        if (!context()) return nullptr;
    }
    ggml_backend* b = new ggml_backend();
    memset(&b->iface, 0, sizeof(b->iface));
    b->guid = backend_guid();
    b->iface.get_name = backend_get_name;
    b->iface.free = backend_free;
    b->iface.synchronize = nullptr;          // graph_compute returns after completion
    b->iface.graph_compute = backend_graph_compute;
    b->device = dev;
    b->context = new Backend();
    return b;
}
bool dev_supports_op(ggml_backend_dev_t, const ggml_tensor* op) {
    if (is_view_op(op->op)) return true;
    if (op->op != GGML_OP_MUL_MAT) return false;
    // at planning time tensors may not be allocated yet: judge types and shapes only
    const ggml_tensor *w = op->src[0], *x = op->src[1];
    return w && x && repacked_type(w->type) && w->ne[2] == 1 && w->ne[3] == 1 && x->type == GGML_TYPE_F32 &&
           op->type == GGML_TYPE_F32 && x->ne[2] == 1 && x->ne[3] == 1 && ggml_is_contiguous(w) && ggml_is_contiguous(x) &&
           w->ne[0] % (w->type == GGML_TYPE_Q4_K ? 256 : 32) == 0;
}
bool dev_supports_buft(ggml_backend_dev_t, ggml_backend_buffer_type_t buft) { return buft == &plugin().buft; }
bool dev_offload_op(ggml_backend_dev_t, const ggml_tensor*) { return false; }

// ---- registry ---------------------------------------------------------------------------------------------------------
const char* reg_get_name(ggml_backend_reg_t) { return "AMEVA_B200"; }
size_t reg_get_device_count(ggml_backend_reg_t) { return 1; }
ggml_backend_dev_t reg_get_device(ggml_backend_reg_t, size_t index) { return index == 0 ? &plugin().dev : nullptr; }
void* reg_get_proc_address(ggml_backend_reg_t, const char*) { return nullptr; }

ggml_backend_reg_t registry() {
    Plugin& p = plugin();
    static std::once_flag once;
    std::call_once(once, [&p] {
        p.reg.api_version = GGML_BACKEND_API_VERSION;
        p.reg.iface.get_name = reg_get_name;
        p.reg.iface.get_device_count = reg_get_device_count;
        p.reg.iface.get_device = reg_get_device;
        p.reg.iface.get_proc_address = reg_get_proc_address;
        p.reg.context = nullptr;
        memset(&p.dev.iface, 0, sizeof(p.dev.iface));
        p.dev.iface.get_name = dev_get_name;
        p.dev.iface.get_description = dev_get_description;
        p.dev.iface.get_memory = dev_get_memory;
        p.dev.iface.get_type = dev_get_type;
        p.dev.iface.get_props = dev_get_props;
        p.dev.iface.init_backend = dev_init_backend;
        p.dev.iface.get_buffer_type = dev_get_buffer_type;
        p.dev.iface.supports_op = dev_supports_op;
        p.dev.iface.supports_buft = dev_supports_buft;
        p.dev.iface.offload_op = dev_offload_op;
        p.dev.reg = &p.reg;
        p.dev.context = nullptr;
        memset(&p.buft.iface, 0, sizeof(p.buft.iface));
        p.buft.iface.get_name = buft_get_name;
        p.buft.iface.alloc_buffer = buft_alloc_buffer;
        p.buft.iface.get_alignment = buft_get_alignment;
        p.buft.iface.get_max_size = buft_get_max_size;
        p.buft.iface.get_alloc_size = buft_get_alloc_size;
        p.buft.iface.is_host = buft_is_host;
        p.buft.device = &p.dev;
        p.buft.context = nullptr;
    });
    return &p.reg;
}

}  // namespace

extern "C" {

// NULL tells the loader the backend cannot be used (it prints "failed to initialize backend from <path>").
GGML_BACKEND_API ggml_backend_reg_t ggml_backend_init(void) {
    if (ac_runtime_abi_version() != AC_ABI_VERSION) {
        fprintf(stderr, "ggml-ameva-b200: refusing to load: libac_runtime_b200.so has ABI %u, built for %u\n",
                ac_runtime_abi_version(), (unsigned)AC_ABI_VERSION);
        return nullptr;
    }
    return registry();
}

GGML_BACKEND_API int ggml_backend_score(void) { return 100; }

}  // extern "C"
