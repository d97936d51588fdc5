// ggml backend plugin over libac_runtime_b200.so: the quantized MUL_MAT of a ggml graph, and the f32 row ops between two
// of them, on B200.
//
// Exports ggml_backend_init() / ggml_backend_score() with C linkage, as the reference's plugin does
// (adapters/llama/ggml-ameva/ggml-ameva.cpp:5693-5707), the ggml_backend_ameva_* helper surface of its public header
// (ggml-ameva.h:19-98: lifecycle, counters, host-side failure injection) and fills the registry / device / buffer-type /
// buffer / backend tables of ggml's backend interface (ggml-backend-impl.h, API version 2). It is compiled against the
// ggml headers of the host application (llama.cpp b8471 / ggml 0.9.8 is what the reference builds with); none of ggml is
// part of this repository. Behaviour kept from the reference plugin:
//   - buffer type: alignment 64, not host memory (weights live in a device layout), alloc size = the device layout's
//     size for repacked weights, ggml_nbytes otherwise (ggml-ameva-buffer.cpp:662-696);
//   - set_tensor repacks Q4_0 / Q8_0 / Q4_K matrices into the device regions, get_tensor returns the uploaded ggml
//     bytes, partial ranges and row-range views included (tests/ameva_qmm_check.cpp:103-127, 184-196); ggml has no error
//     return there, so a failed transfer aborts (ggml-ameva-buffer.cpp:196-219);
//   - a MUL_MAT whose src0 is a range of rows of a repacked weight runs on that range (ggml-ameva.cpp:1332-1338);
//   - supports_buft = the own buffer type only, so the scheduler copies foreign inputs in (ggml-ameva-device.cpp:314-317);
//   - graph_compute checks every node first and returns GGML_STATUS_FAILED without recording anything when one cannot
//     run (ggml-ameva.cpp:5330-5341); the scratch for quantized activations is reserved as the largest need over all
//     nodes before anything is recorded (:5382-5422); consecutive MUL_MATs that share src1 quantize it once
//     (:2154-2158, 2738-2749), and for one activation row they become one launch; a one-row MUL_MAT followed by its ADD or
//     SWIGLU consumer, and RMS_NORM followed by its MUL, run as one kernel (ameva_find_fusion, :4345-4378); the whole
//     graph is one batch, and the call returns after completion (synchronize = NULL); calls are serialised by a mutex;
//   - props: async = false, host_buffer = false, events = false (ggml-ameva-device.cpp:271-281).
// The kernel choice per MUL_MAT is the library's (ac_b200_mul_mat_plan), not a second copy of it.
// Scope: MUL_MAT with a Q4_0 / Q8_0 / Q4_K src0 (2-D, contiguous, or a row range of one) and f32 src1 / dst; ADD and MUL
// of f32 rows (same shape, or src1 one row); GLU in its split SWIGLU form; RMS_NORM over f32 rows; the no-op view nodes.
// Other ops are reported unsupported, which is how the scheduler keeps them on another backend.
#include <algorithm>
#include <atomic>
#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstdlib>
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
#include "../../include/ggml_ameva_b200.h"

namespace {

constexpr size_t kAlign = 64;
char* const kBase = reinterpret_cast<char*>(0x1000);   // tensor->data = kBase + offset inside the device buffer

[[noreturn]] void die(const char* what, AcResult rc) {
    fprintf(stderr, "ggml-ameva-b200: %s failed (AcResult %d)\n", what, (int)rc);
    abort();
}

struct Counters {
    std::atomic<int64_t> supports_query{0}, supported_op{0}, gpu_op{0}, mul_mat{0}, ctx_create{0}, ctx_destroy{0},
        kernel_create{0}, kernel_destroy{0}, buffer_create{0}, buffer_destroy{0}, event_create{0}, event_destroy{0},
        repacked_tensors{0}, repacked_bytes{0}, qmv{0}, mmq{0}, mmqb{0}, fused_pairs{0};
};
Counters g_count;
std::atomic<int> g_fail{AMEVA_FAIL_NONE};

struct Plugin {                 // one per process
    std::mutex mutex;
    AcContext* ctx = nullptr;
    std::string name;
    ggml_backend_reg reg{};
    ggml_backend_device dev{};
    ggml_backend_buffer_type buft{};
    int live_backends = 0, live_buffers = 0;
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
        g_count.ctx_create++;
        char nm[128] = {0};
        ac_runtime_context_get_device_name(p.ctx, nm, sizeof(nm));
        p.name = nm;
    }
    return p.ctx;
}

// Q5_0 and IQ4_NL weights are d * int8: they live on the device as Q8_0 regions and run on the Q8_0 kernels
// (ac_b200_device_type); what is uploaded and read back keeps the tensor's own type.
enum ggml_type dev_type(enum ggml_type t) { return (t == GGML_TYPE_Q5_0 || t == GGML_TYPE_IQ4_NL) ? GGML_TYPE_Q8_0 : t; }
bool repacked_type(enum ggml_type t) {
    t = dev_type(t);
    return t == GGML_TYPE_Q4_0 || t == GGML_TYPE_Q8_0 || t == GGML_TYPE_Q4_K || t == GGML_TYPE_Q6_K || t == GGML_TYPE_Q5_K ||
           t == GGML_TYPE_IQ4_XS || t == GGML_TYPE_Q4_1 || t == GGML_TYPE_Q5_1 || t == GGML_TYPE_Q3_K || t == GGML_TYPE_Q2_K;
}
// activations quantized per 256 (Q8_K records) and the ameva_mmvqb kernel family
bool per_256(enum ggml_type t) {
    return t == GGML_TYPE_Q4_K || t == GGML_TYPE_Q6_K || t == GGML_TYPE_Q5_K || t == GGML_TYPE_IQ4_XS || t == GGML_TYPE_Q3_K ||
           t == GGML_TYPE_Q2_K;
}
// types with one GEMV kernel each (weights decoded to bytes at upload): no fused, grouped or tensor-core variants
bool byte_decoded(enum ggml_type t) {
    return t == GGML_TYPE_Q6_K || t == GGML_TYPE_Q5_K || t == GGML_TYPE_IQ4_XS || t == GGML_TYPE_Q4_1 || t == GGML_TYPE_Q5_1 ||
           t == GGML_TYPE_Q3_K || t == GGML_TYPE_Q2_K;
}
uint32_t block_elems(enum ggml_type t) { return per_256(t) ? 256u : 32u; }
uint32_t payload_bytes(enum ggml_type t) {   // of the device regions
    t = dev_type(t);
    if (t == GGML_TYPE_Q4_1 || t == GGML_TYPE_Q5_1) return 32u;
    return t == GGML_TYPE_Q4_0 ? 16u : (t == GGML_TYPE_Q8_0 ? 32u : (byte_decoded(t) ? 256u : 128u));
}
uint32_t scale_bytes(enum ggml_type t) {
    if (t == GGML_TYPE_Q4_1 || t == GGML_TYPE_Q5_1) return 4u;
    if (t == GGML_TYPE_Q3_K) return 14u;
    if (t == GGML_TYPE_Q2_K) return 20u;
    return (t == GGML_TYPE_Q4_K || t == GGML_TYPE_Q5_K) ? 16u : (t == GGML_TYPE_Q6_K ? 18u : (t == GGML_TYPE_IQ4_XS ? 8u : 2u));
}

// A tensor that can be kept in the device weight layout: a supported quantized type, plain 2-D, contiguous, not a view.
bool repackable(const ggml_tensor* t) {
    return t && repacked_type(t->type) && t->ne[2] == 1 && t->ne[3] == 1 && ggml_is_contiguous(t) && t->view_src == nullptr &&
           t->ne[0] % block_elems(t->type) == 0;
}
bool repack_all() {   // AMEVA_B200_REPACK_ALL=1: every such tensor, whatever its buffer's usage (hosts that set the usage late)
    static const bool on = [] {
        const char* e = getenv("AMEVA_B200_REPACK_ALL");
        return e && e[0] == '1';
    }();
    return on;
}
// A weight this backend keeps in its device layout: such a tensor in a buffer whose usage is WEIGHTS (the rule of the
// reference, ggml-ameva-buffer.cpp:392-394). A quantized tensor anywhere else (a q8_0 / q4_0 KV cache) keeps ggml's
// block layout.
bool is_repacked_weight(const ggml_tensor* t) {
    return repackable(t) && (repack_all() || (t->buffer && ggml_backend_buffer_get_usage(t->buffer) == GGML_BACKEND_BUFFER_USAGE_WEIGHTS));
}
// q8_0 / q4_0 data in ggml's block layout (a quantized KV cache, or a view of one)
bool is_kvq(const ggml_tensor* t) {
    if (!t || (t->type != GGML_TYPE_Q8_0 && t->type != GGML_TYPE_Q4_0)) return false;
    return !is_repacked_weight(t) && !(t->view_src && is_repacked_weight(t->view_src));
}
uint32_t kvq_block_bytes(enum ggml_type t) { return t == GGML_TYPE_Q8_0 ? 34u : 18u; }
bool kvq_rows(const ggml_tensor* t) {   // whole blocks along dimension 0, the other strides even and within 32 bits
    if (t->ne[0] % 32 || t->nb[0] != kvq_block_bytes(t->type)) return false;
    for (int i = 1; i < 4; ++i)
        if (t->nb[i] % 2 || t->nb[i] > 0xFFFFFFFFull) return false;
    return true;
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
    // per repacked weight (by its offset in the buffer): the tensor's magnitude as a power of two, from its block scales
    // at upload (ac_b200_weight_exponent); tensors fp16 does not hold comfortably stay off the tensor-core kernel
    std::map<size_t, int> w_exp;
};

size_t tensor_offset(const ggml_tensor* t) { return (size_t)((const char*)t->data - kBase); }

// The repacked weight a tensor is, or is a byte range of: the tensor itself, or its view_src when that is a repacked
// weight (ggml sets a view's data to the base's data + view_offs). extra = where the tensor starts inside the base, in
// bytes of the ggml layout.
const ggml_tensor* repacked_base(const ggml_tensor* t, size_t* extra) {
    if (is_repacked_weight(t)) {
        *extra = 0;
        return t;
    }
    if (t && t->view_src && is_repacked_weight(t->view_src)) {
        *extra = t->view_offs;
        return t->view_src;
    }
    return nullptr;
}

void buffer_free(ggml_backend_buffer_t buffer) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    if (b->buf && ac_runtime_buffer_destroy(b->buf) == AC_SUCCESS) g_count.buffer_destroy++;
    plugin().live_buffers--;
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
    size_t extra = 0;
    const ggml_tensor* base = repacked_base(tensor, &extra);
    if (!base) {
        const AcResult rc = ac_runtime_buffer_write(b->buf, tensor_offset(tensor) + offset, data, size);
        if (rc != AC_SUCCESS) die("buffer_write", rc);
        return;
    }
    offset += extra;   // a view of a repacked weight: a byte range of the base's ggml image
    const size_t nbytes = ggml_nbytes(base);
    if (offset > nbytes || size > nbytes - offset) die("set_tensor range", AC_ERR_INVALID_BUFFER_SIZE);
    const uint64_t rows = (uint64_t)base->ne[1], k = (uint64_t)base->ne[0];
    const uint64_t total = device_bytes(base, nullptr);
    std::vector<uint8_t> blocks;
    const void* src = data;
    const bool first_upload = b->w_exp.find(tensor_offset(base)) == b->w_exp.end();
    if (offset != 0 || size != nbytes) {   // a partial range: patch the ggml image of what is on the device
        std::vector<uint8_t> dev(total);
        blocks.resize(nbytes);
        AcResult rc = ac_runtime_buffer_read(b->buf, tensor_offset(base), dev.data(), total);
        if (rc == AC_SUCCESS) rc = ac_b200_repack_from_device((uint32_t)base->type, dev.data(), rows, k, blocks.data());
        if (rc != AC_SUCCESS) die("partial set_tensor read-back", rc);
        memcpy(blocks.data() + offset, data, size);
        src = blocks.data();
    }
    // the ggml -> regions permutation runs on the device, fed from the runtime's pinned staging chunks
    // (ggml-ameva-buffer.cpp:300-330 stages chunks and repacks on the CPU)
    AcResult rc = ac_b200_weight_upload(b->buf, tensor_offset(base), (uint32_t)base->type, src, rows, k);
    int32_t w_exp = 0;
    if (rc == AC_SUCCESS) rc = ac_b200_weight_exponent((uint32_t)base->type, src, rows, k, &w_exp);
    if (rc != AC_SUCCESS) die("set_tensor", rc);
    b->w_exp[tensor_offset(base)] = w_exp;
    if (first_upload) {
        g_count.repacked_tensors++;
        g_count.repacked_bytes += (int64_t)total;
    }
}

void buffer_get_tensor(ggml_backend_buffer_t buffer, const ggml_tensor* tensor, void* data, size_t offset, size_t size) {
    BufferCtx* b = (BufferCtx*)buffer->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    size_t extra = 0;
    const ggml_tensor* base = repacked_base(tensor, &extra);
    if (!base) {
        const AcResult rc = ac_runtime_buffer_read(b->buf, tensor_offset(tensor) + offset, data, size);
        if (rc != AC_SUCCESS) die("buffer_read", rc);
        return;
    }
    offset += extra;
    const size_t nbytes = ggml_nbytes(base);
    if (offset > nbytes || size > nbytes - offset) die("get_tensor range", AC_ERR_INVALID_BUFFER_SIZE);
    const uint64_t rows = (uint64_t)base->ne[1], k = (uint64_t)base->ne[0];
    const uint64_t total = device_bytes(base, nullptr);
    std::vector<uint8_t> dev(total), blocks(nbytes);
    AcResult rc = ac_runtime_buffer_read(b->buf, tensor_offset(base), dev.data(), total);
    if (rc == AC_SUCCESS) rc = ac_b200_repack_from_device((uint32_t)base->type, dev.data(), rows, k, blocks.data());
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
const char* buft_get_name(ggml_backend_buffer_type_t) { return GGML_AMEVA_B200_NAME; }

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
    g_count.buffer_create++;
    plugin().live_buffers++;
    return ggml_backend_buffer_init(buft, buffer_iface(), b, size);
}

size_t buft_get_alignment(ggml_backend_buffer_type_t) { return kAlign; }

size_t buft_get_max_size(ggml_backend_buffer_type_t) {
    std::lock_guard<std::mutex> lock(plugin().mutex);
    AcContext* ctx = context();
    AcDeviceLimits lim;
    memset(&lim, 0, sizeof(lim));
    lim.abi_version = AC_ABI_VERSION;
    lim.struct_size = (uint32_t)sizeof(lim);
    if (!ctx || ac_runtime_context_get_limits(ctx, &lim) != AC_SUCCESS) return SIZE_MAX;
    return (size_t)lim.max_memory_allocation_size;
}

size_t buft_get_alloc_size(ggml_backend_buffer_type_t, const ggml_tensor* tensor) {
    if (repackable(tensor)) {   // (asked before the tensor has a buffer: room for either layout)
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
    AcBuffer* kv_f16[2] = {nullptr, nullptr};   // a quantized K / V view dequantized to f16 for FLASH_ATTN_EXT
    size_t kv_f16_bytes[2] = {0, 0};
    AcBuffer* gh = nullptr;   // fp16 (scale, offset) per 16 weights: the scale table of ameva_mmtc_b8, rewritten per MUL_MAT
    size_t aq_bytes = 0, ad_bytes = 0, ah_bytes = 0, ae_bytes = 0, gh_bytes = 0;
    AcBuffer* op_status = nullptr;   // {count, lowest node} of refused GET_ROWS / SET_ROWS indices
    AcBuffer* fa_part = nullptr;     // partial results of the key splits of FLASH_ATTN_EXT
    size_t op_status_bytes = 0, fa_part_bytes = 0;
};

AcKernel* kernel(Backend* be, const char* name) {
    auto it = be->kernels.find(name);
    if (it != be->kernels.end()) return it->second;
    AcKernel* k = nullptr;
    if (ac_runtime_kernel_create_builtin(context(), name, &k) != AC_SUCCESS) return nullptr;
    g_count.kernel_create++;
    be->kernels[name] = k;
    return k;
}

// Called before a batch is begun (nothing retains the old buffer then), with the largest need over the graph's nodes.
bool grow(AcBuffer** buf, size_t* have, size_t need) {
    if (*have >= need) return true;
    if (*buf) {
        const AcResult rc = ac_runtime_buffer_destroy(*buf);
        if (rc != AC_SUCCESS) {
            fprintf(stderr, "ggml-ameva-b200: scratch buffer still in use (AcResult %d)\n", (int)rc);
            return false;
        }
        g_count.buffer_destroy++;
    }
    *buf = nullptr;
    *have = 0;
    AcBufferDesc d = {AC_ABI_VERSION, (uint32_t)sizeof(AcBufferDesc), need, AC_BUFFER_USAGE_STORAGE, 0};
    if (ac_runtime_buffer_create(context(), &d, buf) != AC_SUCCESS) return false;
    g_count.buffer_create++;
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
BufferCtx* buffer_of(const ggml_tensor* t) { return (BufferCtx*)(t->view_src ? t->view_src : t)->buffer->context; }

bool is_f32_rows(const ggml_tensor* t) {   // f32, rows contiguous and packed ([ne1 * ne2 * ne3][ne0])
    return t && t->type == GGML_TYPE_F32 && ggml_is_contiguous(t);
}
int64_t n_rows(const ggml_tensor* t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
int64_t n_elems(const ggml_tensor* t) { return t->ne[0] * n_rows(t); }

bool overlap(const ggml_tensor* a, const ggml_tensor* b) {
    if (!a || !b || !a->data || !b->data || buffer_of(a) != buffer_of(b)) return false;
    const char *a0 = (const char*)a->data, *b0 = (const char*)b->data;
    return a0 < b0 + ggml_nbytes(b) && b0 < a0 + ggml_nbytes(a);
}
bool same_elements(const ggml_tensor* a, const ggml_tensor* b) {   // an in-place result
    return a->data == b->data && buffer_of(a) == buffer_of(b) && ggml_nbytes(a) == ggml_nbytes(b);
}

// A MUL_MAT's weight operand resolved to device addresses: the whole repacked tensor or a range of its rows.
struct WeightRef {
    BufferCtx* buf;
    uint64_t q_off, q_range, s_off, s_range;   // byte ranges of the payload and scale regions inside the buffer
    uint32_t N, K;
    enum ggml_type type;
};

// Why a MUL_MAT node cannot run here; NULL when it can (the reference's mul_mat_qmm_reason, ggml-ameva.cpp:1326-1377,
// reduced to this backend's kernels). With `out`, also resolves the weight operand and the kernel family.
const char* mul_mat_reason(const ggml_tensor* node, WeightRef* out = nullptr, uint32_t* out_path = nullptr) {
    const ggml_tensor *w = node->src[0], *x = node->src[1];
    if (!w || !x) return "missing operand";
    size_t extra = 0;
    const ggml_tensor* base = repacked_base(w, &extra);
    if (!base) return "src0 is not a 2-D contiguous Q4_0 / Q8_0 / Q4_K matrix (or a row range of one)";
    uint64_t row0 = 0;
    if (w != base) {   // rows [row0, row0 + ne1) of the base: same K, same row pitch, whole rows
        if (w->type != base->type || w->ne[0] != base->ne[0] || w->ne[2] != 1 || w->ne[3] != 1 || w->nb[0] != base->nb[0] ||
            w->nb[1] != base->nb[1] || extra % base->nb[1])
            return "src0 views a repacked weight but is not a range of its rows";
        row0 = extra / base->nb[1];
        if (row0 + (uint64_t)w->ne[1] > (uint64_t)base->ne[1]) return "row range outside the weight";
    }
    if (!own_buffer(base) || !own_buffer(x) || !own_buffer(node)) return "an operand is not in an AMEVA_B200 buffer";
    if (x->type != GGML_TYPE_F32 || node->type != GGML_TYPE_F32) return "src1 / dst are not f32";
    if (!ggml_is_contiguous(x) || !ggml_is_contiguous(node)) return "src1 / dst are not contiguous";
    if (x->ne[2] != 1 || x->ne[3] != 1 || node->ne[2] != 1 || node->ne[3] != 1) return "batched (3-D / 4-D) operands";
    if (x->ne[0] != w->ne[0] || node->ne[0] != w->ne[1] || node->ne[1] != x->ne[1]) return "shape mismatch";
    const uint64_t K = (uint64_t)w->ne[0], N = (uint64_t)w->ne[1], M = (uint64_t)x->ne[1];
    const uint64_t nblk_row = K / block_elems(w->type);
    uint64_t s_off = 0;
    device_bytes(base, &s_off);
    const uint64_t q_off = tensor_offset(base) + row0 * nblk_row * payload_bytes(w->type);
    const uint64_t sc_off = tensor_offset(base) + s_off + row0 * nblk_row * scale_bytes(w->type);
    if (q_off % kAlign || sc_off % kAlign) return "the row range does not start on a 64-byte boundary of the device layout";
    if (tensor_offset(x) % kAlign || tensor_offset(node) % kAlign) return "unaligned tensor";
    BufferCtx* wb = buffer_of(base);
    auto it = wb->w_exp.find(tensor_offset(base));
    const int w_exp = it == wb->w_exp.end() ? 0 : it->second;
    uint32_t path = AC_B200_PATH_NONE;
    const uint32_t flags = AC_B200_PLAN_HOST_LAUNCH | (AC_B200_WEIGHT_RANGE_EXTREME(w_exp) ? AC_B200_PLAN_WEIGHT_RANGE : 0u);
    if (ac_b200_mul_mat_plan((uint32_t)w->type, M, N, K, flags, &path) != AC_SUCCESS) return "shape outside the kernels' contract";
    // more than 8 activation rows on the GEMV family run as chunks of 8 rows: the chunks' scratch and output offsets
    // (8 K, 8 scale rows, 32 N bytes) must keep the 64-byte binding alignment
    if (M > 8 && path == AC_B200_PATH_GEMV && (K % 64 || (32 * N) % 64)) return "chunked M > 8 needs K % 64 == 0, N % 2 == 0";
    if (out) {
        out->buf = wb;
        out->q_off = q_off;
        out->q_range = N * nblk_row * payload_bytes(w->type);
        out->s_off = sc_off;
        out->s_range = N * nblk_row * scale_bytes(w->type);
        out->N = (uint32_t)N;
        out->K = (uint32_t)K;
        out->type = dev_type(w->type);
    }
    if (out_path) *out_path = path;
    return nullptr;
}

bool binary_supported(const ggml_tensor* node) {   // ADD / MUL of f32 rows: same shape, or src1 one row of the same width
    const ggml_tensor *a = node->src[0], *b = node->src[1];
    if (!a || !b || !is_f32_rows(a) || !is_f32_rows(b) || !is_f32_rows(node)) return false;
    if (a->ne[0] != node->ne[0] || n_rows(a) != n_rows(node) || b->ne[0] != a->ne[0]) return false;
    const int64_t br = n_rows(b);
    return br >= 1 && (br == 1 || br == n_rows(a));
}
bool glu_supported(const ggml_tensor* node) {      // the split SWIGLU: silu(src0) * src1
    const ggml_tensor *a = node->src[0], *b = node->src[1];
    return a && b && node->op_params[0] == (int32_t)GGML_GLU_OP_SWIGLU && node->op_params[1] == 0 && is_f32_rows(a) &&
           is_f32_rows(b) && is_f32_rows(node) && n_elems(a) == n_elems(b) && n_elems(a) == n_elems(node);
}
bool rms_norm_supported(const ggml_tensor* node) {
    const ggml_tensor* a = node->src[0];
    return a && is_f32_rows(a) && is_f32_rows(node) && n_elems(a) == n_elems(node) && a->ne[0] == node->ne[0];
}

// ---- the ops around the mul_mats of a decoder layer: ROPE, GET_ROWS, SET_ROWS, SOFT_MAX, FLASH_ATTN_EXT -------------------
// They run under the reference's kernel contracts (ggml-ameva.cpp:3965-3995 enc_rope, :4037-4060 enc_set_rows,
// :4113-4135 enc_get_rows, enc_soft_max, enc_flash_attn): strides in elements of the tensor's type, a tensor that does
// not start on a 64-byte boundary of its buffer is bound from the boundary below with its element offset in the push
// constants.
size_t elem_size(enum ggml_type t) {
    switch (t) {
        case GGML_TYPE_F32: case GGML_TYPE_I32: return 4;
        case GGML_TYPE_F16: return 2;
        case GGML_TYPE_I64: return 8;
        default: return 0;
    }
}
bool elem_strides(const ggml_tensor* t, size_t es) {   // element 0 stride = one element, the others whole elements in 32 bits
    if (!t || !es || t->nb[0] != es) return false;
    for (int i = 1; i < 4; ++i)
        if (t->nb[i] % es || t->nb[i] / es > 0xFFFFFFFFull) return false;
    return true;
}
bool whole_elem_strides(const ggml_tensor* t, size_t es) {   // any layout whose strides are whole elements (a transposed view)
    if (!t || !es) return false;
    for (int i = 0; i < 4; ++i)
        if (t->nb[i] % es || t->nb[i] / es > 0xFFFFFFFFull) return false;
    return true;
}
uint32_t st(const ggml_tensor* t, int i, size_t es) { return (uint32_t)(t->nb[i] / es); }

// the op code of ameva_unary for a node (ameva_unary.comp:4-6), -1 when the kernel has none
int unary_code(const ggml_tensor* node) {
    switch (node->op) {
        case GGML_OP_SCALE: return 0;
        case GGML_OP_SQR: return 9;
        case GGML_OP_SQRT: return 10;
        case GGML_OP_SIN: return 13;
        case GGML_OP_COS: return 14;
        case GGML_OP_LEAKY_RELU: return 15;
        case GGML_OP_UNARY:
            switch ((enum ggml_unary_op)node->op_params[0]) {
                case GGML_UNARY_OP_TANH: return 1;
                case GGML_UNARY_OP_SILU: return 2;
                case GGML_UNARY_OP_GELU: return 3;
                case GGML_UNARY_OP_GELU_ERF: return 4;
                case GGML_UNARY_OP_GELU_QUICK: return 5;
                case GGML_UNARY_OP_RELU: return 6;
                case GGML_UNARY_OP_SIGMOID: return 7;
                case GGML_UNARY_OP_NEG: return 8;
                case GGML_UNARY_OP_EXP: return 11;
                case GGML_UNARY_OP_ABS: return 12;
                case GGML_UNARY_OP_SGN: return 16;
                case GGML_UNARY_OP_STEP: return 17;
                case GGML_UNARY_OP_FLOOR: return 18;
                default: return -1;
            }
        default: return -1;
    }
}
bool is_unary_like(enum ggml_op op) {
    return op == GGML_OP_SCALE || op == GGML_OP_UNARY || op == GGML_OP_SQR || op == GGML_OP_SQRT || op == GGML_OP_SIN ||
           op == GGML_OP_COS || op == GGML_OP_LEAKY_RELU;
}

bool is_layer_op(enum ggml_op op) {
    if (is_unary_like(op)) return true;
    return op == GGML_OP_ROPE || op == GGML_OP_GET_ROWS || op == GGML_OP_SET_ROWS || op == GGML_OP_SOFT_MAX ||
           op == GGML_OP_FLASH_ATTN_EXT || op == GGML_OP_CPY || op == GGML_OP_CONT || op == GGML_OP_DUP;
}
float param_f32(const ggml_tensor* t, int i) {
    float f;
    memcpy(&f, &t->op_params[i], 4);
    return f;
}

const char* layer_op_static_reason(const ggml_tensor* node) {
    const ggml_tensor *a = node->src[0], *b = node->src[1];
    if (is_unary_like(node->op)) {
        if (unary_code(node) < 0) return "unary op without a kernel";
        if (!a || a->type != GGML_TYPE_F32 || node->type != GGML_TYPE_F32 || !elem_strides(a, 4) || !elem_strides(node, 4)) return "unary: f32 rows only";
        for (int i = 0; i < 4; ++i)
            if (a->ne[i] != node->ne[i]) return "unary: shape";
        return nullptr;
    }
    switch (node->op) {
        case GGML_OP_ROPE: {
            if (!a || !b || (a->type != GGML_TYPE_F32 && a->type != GGML_TYPE_F16) || node->type != a->type) return "rope: f32 or f16 only";
            const size_t es = elem_size(a->type);
            if (!elem_strides(a, es) || !elem_strides(node, es)) return "rope: strides are not whole elements";
            if (b->type != GGML_TYPE_I32 || b->ne[0] < a->ne[2] || b->nb[0] != 4) return "rope: positions are not i32 [ne2]";
            const int n_dims = node->op_params[1], mode = node->op_params[2];
            if (mode != 0 && mode != 2) return "rope: only the NORMAL and NEOX modes";
            if (n_dims < 0 || n_dims > a->ne[0] || (n_dims & 1) || (a->ne[0] & 1)) return "rope: n_dims";
            if (node->src[2] && (node->src[2]->type != GGML_TYPE_F32 || node->src[2]->ne[0] < n_dims / 2)) return "rope: frequency factors";
            for (int i = 0; i < 4; ++i)
                if (a->ne[i] != node->ne[i]) return "rope: shape";
            return nullptr;
        }
        case GGML_OP_CPY:
        case GGML_OP_CONT:
        case GGML_OP_DUP: {
            if (a && is_kvq(node)) {   // f32 -> q8_0 / q4_0 of the same shape (the KV-cache shift writes the rotated K back)
                if (a->type != GGML_TYPE_F32 || !(a->ne[0] == node->ne[0] && a->ne[1] == node->ne[1] && a->ne[2] == node->ne[2] && a->ne[3] == node->ne[3])) return "cpy: to a quantized type from f32 of the same shape only";
                if (!elem_strides(a, 4) || !kvq_rows(node)) return "cpy: to a quantized type: rows are not whole blocks";
                return nullptr;
            }
            if (a && is_kvq(a)) {      // q8_0 / q4_0 -> f32 / f16 (the shift casts K to f32)
                if (node->type != GGML_TYPE_F32 && node->type != GGML_TYPE_F16) return "cpy: from a quantized type to f32 / f16 only";
                if (!kvq_rows(a) || !whole_elem_strides(node, elem_size(node->type))) return "cpy: from a quantized type: rows are not whole blocks";
                if (a->ne[0] * a->ne[1] * a->ne[2] * a->ne[3] != node->ne[0] * node->ne[1] * node->ne[2] * node->ne[3]) return "cpy: element counts differ";
                return nullptr;
            }
            if (!a || (a->type != GGML_TYPE_F32 && a->type != GGML_TYPE_F16) || (node->type != GGML_TYPE_F32 && node->type != GGML_TYPE_F16))
                return "cpy: between f32 and f16 only";
            if (!whole_elem_strides(a, elem_size(a->type)) || !whole_elem_strides(node, elem_size(node->type))) return "cpy: strides are not whole elements";
            if (a->ne[0] * a->ne[1] * a->ne[2] * a->ne[3] != node->ne[0] * node->ne[1] * node->ne[2] * node->ne[3]) return "cpy: element counts differ";
            return nullptr;
        }
        case GGML_OP_GET_ROWS: {
            if (a && b && is_repacked_weight(a)) {   // a quantized table kept in the device weight layout (token embeddings)
                if (node->type != GGML_TYPE_F32 || b->type != GGML_TYPE_I32 || !elem_strides(b, 4) || !elem_strides(node, 4))
                    return "get_rows: quantized table to f32 with i32 indices";
                if (b->ne[1] != 1 || b->ne[2] != 1 || node->ne[0] != a->ne[0] || node->ne[1] != b->ne[0] || node->ne[2] != 1 ||
                    node->ne[3] != 1)
                    return "get_rows: a quantized table is looked up with one row of indices";
                return nullptr;
            }
            if (!a || !b || (a->type != GGML_TYPE_F32 && a->type != GGML_TYPE_F16) || node->type != GGML_TYPE_F32) return "get_rows: f32 / f16 rows to f32";
            if (b->type != GGML_TYPE_I32 || !elem_strides(b, 4) || !elem_strides(a, elem_size(a->type)) || !elem_strides(node, 4))
                return "get_rows: indices are not i32 or strides are not whole elements";
            if (node->ne[0] != a->ne[0] || node->ne[1] != b->ne[0] || node->ne[2] != b->ne[1] || node->ne[3] != b->ne[2]) return "get_rows: shape";
            return nullptr;
        }
        case GGML_OP_SET_ROWS: {
            if (a && b && is_kvq(node)) {   // the write of a quantized KV cache
                if (a->type != GGML_TYPE_F32 || !elem_strides(a, 4) || !kvq_rows(node)) return "set_rows: f32 rows to whole q8_0 / q4_0 blocks";
                if ((b->type != GGML_TYPE_I64 && b->type != GGML_TYPE_I32) || b->nb[0] != elem_size(b->type) || b->nb[1] % 4 || b->nb[2] % 4)
                    return "set_rows: indices";
                if (a->ne[0] != node->ne[0] || a->ne[2] != node->ne[2] || a->ne[3] != node->ne[3] || b->ne[0] != a->ne[1] || !b->ne[1] || !b->ne[2])
                    return "set_rows: shape";
                return nullptr;
            }
            if (!a || !b || a->type != GGML_TYPE_F32 || (node->type != GGML_TYPE_F32 && node->type != GGML_TYPE_F16)) return "set_rows: f32 rows to f32 / f16";
            if ((b->type != GGML_TYPE_I64 && b->type != GGML_TYPE_I32) || b->nb[0] != elem_size(b->type) || b->nb[1] % 4 || b->nb[2] % 4)
                return "set_rows: indices";
            if (!elem_strides(a, 4) || !elem_strides(node, elem_size(node->type))) return "set_rows: strides are not whole elements";
            if (a->ne[0] != node->ne[0] || a->ne[2] != node->ne[2] || a->ne[3] != node->ne[3] || b->ne[0] != a->ne[1] || !b->ne[1] || !b->ne[2])
                return "set_rows: shape";
            return nullptr;
        }
        case GGML_OP_SOFT_MAX: {
            if (!a || a->type != GGML_TYPE_F32 || node->type != GGML_TYPE_F32 || !elem_strides(a, 4) || !elem_strides(node, 4)) return "soft_max: f32 only";
            if (node->src[2]) return "soft_max: attention sinks";
            if (param_f32(node, 1) != 0.0f) return "soft_max: ALiBi bias";
            if (b) {
                if ((b->type != GGML_TYPE_F32 && b->type != GGML_TYPE_F16) || !elem_strides(b, elem_size(b->type))) return "soft_max: mask type";
                if (b->ne[0] != a->ne[0] || b->ne[1] < a->ne[1] || !b->ne[2] || !b->ne[3] || a->ne[2] % b->ne[2] || a->ne[3] % b->ne[3])
                    return "soft_max: mask shape";
            }
            return nullptr;
        }
        case GGML_OP_FLASH_ATTN_EXT: {
            const ggml_tensor *k = node->src[1], *v = node->src[2], *m = node->src[3];
            const bool kq = k && is_kvq(k), vq = v && is_kvq(v);   // (dequantized to f16 scratch before the attention kernel)
            if (!a || !k || !v || a->type != GGML_TYPE_F32 || (k->type != GGML_TYPE_F16 && !kq) || (v->type != GGML_TYPE_F16 && !vq) ||
                node->type != GGML_TYPE_F32)
                return "flash_attn: f32 queries on an f16 / q8_0 / q4_0 cache only";
            if (node->src[4]) return "flash_attn: attention sinks";
            if (param_f32(node, 1) != 0.0f) return "flash_attn: ALiBi bias";
            const int64_t D = a->ne[0];
            if ((D != 64 && D != 128 && D != 256) || k->ne[0] != D || v->ne[0] != D) return "flash_attn: head size";
            if (a->ne[3] != 1 || k->ne[3] != 1 || v->ne[3] != 1 || k->ne[1] != v->ne[1] || k->ne[2] != v->ne[2] || !k->ne[2] ||
                a->ne[2] % k->ne[2] || a->ne[2] / k->ne[2] > 8)
                return "flash_attn: head grouping";
            if (!elem_strides(a, 4) || !(kq ? kvq_rows(k) : elem_strides(k, 2)) || !(vq ? kvq_rows(v) : elem_strides(v, 2)) ||
                !ggml_is_contiguous(node))
                return "flash_attn: strides";
            if ((!kq && (k->nb[1] | k->nb[2]) % 16) || (!vq && (v->nb[1] | v->nb[2]) % 16)) return "flash_attn: cache rows are not 16-byte aligned";
            if (node->ne[0] != D || node->ne[1] != a->ne[2] || node->ne[2] != a->ne[1]) return "flash_attn: result shape";
            if (m && (m->type != GGML_TYPE_F16 || !elem_strides(m, 2) || m->ne[0] < k->ne[1] || m->ne[1] < a->ne[1] || !m->ne[2] || m->ne[3] != 1))
                return "flash_attn: mask";
            return nullptr;
        }
        default: return "op has no encoder";
    }
}

AcBufferBinding bind(AcBuffer* b, uint64_t off, uint64_t range);

// a tensor bound from the 64-byte boundary below it; elem = where the tensor starts inside the binding, in elements
struct ElemBind {
    AcBufferBinding b;
    uint32_t elem;
};
bool bind_elems(const ggml_tensor* t, size_t es, ElemBind* out) {
    const size_t off = tensor_offset(t), base = off & ~(size_t)(kAlign - 1), rem = off - base;
    if (rem % es) return false;
    out->b = bind(buffer_of(t)->buf, base, rem + ggml_nbytes(t));
    out->elem = (uint32_t)(rem / es);
    return true;
}

const char* layer_op_reason(const ggml_tensor* node) {
    if (const char* why = layer_op_static_reason(node)) return why;
    for (int i = 0; i < GGML_MAX_SRC; ++i) {
        const ggml_tensor* t = node->src[i];
        if (!t) continue;
        if (!own_buffer(t)) return "an operand is not in an AMEVA_B200 buffer";
        if (node->op == GGML_OP_GET_ROWS && i == 0 && is_repacked_weight(t)) {
            if (tensor_offset(t) % kAlign) return "get_rows: the table does not start on a 64-byte boundary";
            continue;
        }
        if (is_kvq(t)) {
            if (tensor_offset(t) % 2) return "a quantized operand does not start on an even byte";
            continue;
        }
        if (!elem_size(t->type) || tensor_offset(t) % elem_size(t->type)) return "an operand does not start on an element boundary";
    }
    if (!own_buffer(node) || (is_kvq(node) ? tensor_offset(node) % 2 : (!elem_size(node->type) || tensor_offset(node) % elem_size(node->type))))
        return "dst is not in an AMEVA_B200 buffer";
    if (node->op == GGML_OP_FLASH_ATTN_EXT && ((!is_kvq(node->src[1]) && tensor_offset(node->src[1]) % 16) ||
                                               (!is_kvq(node->src[2]) && tensor_offset(node->src[2]) % 16) || tensor_offset(node) % 16))
        return "flash_attn: cache or result not 16-byte aligned";
    return nullptr;
}

uint32_t f32_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

// ggml_rope_yarn_corr_dims (ggml.c): the pair indices between which YaRN blends interpolation and extrapolation
void rope_corr_dims(int n_dims, int n_ctx_orig, float freq_base, float beta_fast, float beta_slow, float dims[2]) {
    auto corr_dim = [&](float n_rot) {
        return n_dims * logf(n_ctx_orig / (n_rot * 2.0f * 3.14159265358979323846f)) / (2.0f * logf(freq_base));
    };
    const float start = floorf(corr_dim(beta_fast)), end = ceilf(corr_dim(beta_slow));
    dims[0] = std::max(0.0f, start);
    dims[1] = std::min((float)(n_dims - 1), end);
}

// shapes and types only (at planning time tensors may not be allocated yet)
bool op_supported_static(const ggml_tensor* op) {
    if (is_view_op(op->op)) return true;
    switch (op->op) {
        case GGML_OP_MUL_MAT: {
            const ggml_tensor *w = op->src[0], *x = op->src[1];
            if (!w || !x || !repacked_type(w->type) || w->ne[2] != 1 || w->ne[3] != 1 || x->type != GGML_TYPE_F32 ||
                op->type != GGML_TYPE_F32 || x->ne[2] != 1 || x->ne[3] != 1 || !ggml_is_contiguous(x) ||
                w->ne[0] % block_elems(w->type))
                return false;
            uint32_t path = 0;
            return ac_b200_mul_mat_plan((uint32_t)w->type, (uint64_t)x->ne[1], (uint64_t)w->ne[1], (uint64_t)w->ne[0],
                                        AC_B200_PLAN_HOST_LAUNCH, &path) == AC_SUCCESS;
        }
        case GGML_OP_ADD:
        case GGML_OP_MUL: return binary_supported(op);
        case GGML_OP_GLU: return glu_supported(op);
        case GGML_OP_RMS_NORM: return rms_norm_supported(op);
        default: return is_layer_op(op->op) && !layer_op_static_reason(op);
    }
}

const char* node_reason(const ggml_tensor* node) {
    if (is_view_op(node->op)) return nullptr;
    if (node->op == GGML_OP_MUL_MAT) return mul_mat_reason(node);
    if (is_layer_op(node->op)) return layer_op_reason(node);
    if (!op_supported_static(node)) return "op, type or shape not built";
    for (int i = 0; i < GGML_MAX_SRC && node->src[i]; ++i)
        if (!own_buffer(node->src[i]) || tensor_offset(node->src[i]) % kAlign)
            return "an operand is not in an AMEVA_B200 buffer (or unaligned)";
    if (!own_buffer(node) || tensor_offset(node) % kAlign) return "dst is not in an AMEVA_B200 buffer (or unaligned)";
    return nullptr;
}

AcBufferBinding bind(AcBuffer* b, uint64_t off, uint64_t range) {
    AcBufferBinding r = {b, off, range};
    return r;
}
AcBufferBinding bind_tensor(const ggml_tensor* t) { return bind(buffer_of(t)->buf, tensor_offset(t), ggml_nbytes(t)); }

// What graph_compute remembers while it records one graph.
struct Recorder {
    Backend* be = nullptr;
    AcCommandBatch* batch = nullptr;
    // the activation rows last quantized into the scratch (reused by the next MUL_MAT with the same src1 and scheme)
    const void* q_data = nullptr;
    uint32_t q_M = 0, q_K = 0;
    int q_scheme = -1;   // 0 per-32, 1 per-256; +2 when the fp16 operand was written too
    int64_t gpu_ops = 0, mul_mats = 0, mmq = 0, mmqb = 0, fused = 0;
    bool rows_ops = false;   // a GET_ROWS / SET_ROWS was recorded: the index status is read after the batch
};

struct QuantizedRows {
    const void* data = nullptr;
    uint32_t M = 0, K = 0;
    int scheme = -1;
};

bool dispatch(Recorder& r, const char* name, const AcBufferBinding* b, uint32_t nb, const uint32_t* push, size_t push_bytes) {
    AcKernel* k = kernel(r.be, name);
    if (!k) return false;
    const AcDim3 grid = {1, 1, 1};   // the launchers size their own grids
    return ac_runtime_batch_dispatch_bindings(r.batch, k, b, nb, push, push_bytes, grid) == AC_SUCCESS;
}

const char* type_name(enum ggml_type t) {
    if (t == GGML_TYPE_Q4_1) return "q4_1";
    if (t == GGML_TYPE_Q5_1) return "q5_1";
    if (t == GGML_TYPE_Q3_K) return "q3_K";
    if (t == GGML_TYPE_Q2_K) return "q2_K";
    return t == GGML_TYPE_Q4_0 ? "q4_0" : (t == GGML_TYPE_Q8_0 ? "q8_0" : (t == GGML_TYPE_Q6_K ? "q6_K" : (t == GGML_TYPE_Q5_K ? "q5_K" : (t == GGML_TYPE_IQ4_XS ? "iq4_xs" : "q4_K"))));
}

// activation quantization into the scratch, unless the same rows are there already
bool record_quantize(Recorder& r, const ggml_tensor* x, enum ggml_type wtype, uint32_t M, uint32_t K, bool tc) {
    const bool q4k = per_256(wtype);
    const int scheme = (q4k ? 1 : 0) + (tc ? 2 : 0);
    if (r.q_data == x->data && r.q_M == M && r.q_K == K && (r.q_scheme == scheme || r.q_scheme == scheme + 2)) return true;
    const uint64_t ad_need = q4k ? (uint64_t)M * (K / 256) * 48u : (uint64_t)M * (K / 32) * 4u;
    std::string name = q4k ? "ameva_quant_a8b" : "ameva_quant_a8";
    if (tc) name += "_f16";
    AcBufferBinding b[5] = {bind(buffer_of(x)->buf, tensor_offset(x), (uint64_t)M * K * 4), bind(r.be->aq, 0, (uint64_t)M * K),
                            bind(r.be->ad, 0, ad_need), bind(r.be->ah, 0, (uint64_t)M * K * 2),
                            bind(r.be->ae, 0, (uint64_t)M * 4)};
    const uint32_t push[4] = {M, K, K, 0};   // ties-to-even per-32 / ggml's per-256 convention
    if (!dispatch(r, name.c_str(), b, tc ? 5 : 3, push, sizeof(push))) return false;
    ac_runtime_batch_barrier(r.batch);
    r.q_data = x->data;
    r.q_M = M;
    r.q_K = K;
    r.q_scheme = scheme;
    return true;
}

// Epilogue of a one-row MUL_MAT fused with the node that consumes it (AmevaEpilogue, ggml-ameva.cpp:2272-2279).
struct Epilogue {
    uint32_t mode = 0;   // 1 out = v + e, 2 out = silu(v) * e, 3 out = silu(e) * v
    const ggml_tensor* e = nullptr;
    const ggml_tensor* out = nullptr;
};

// Whether n1 consumes the one-row product n0 in a way the GEMV's epilogue computes (ameva_find_fusion, :4345-4378).
Epilogue find_epilogue(const ggml_tensor* n0, const ggml_tensor* n1) {
    Epilogue f;
    if (!n1 || n0->op != GGML_OP_MUL_MAT || n0->src[1]->ne[1] != 1) return f;
    if (byte_decoded(n0->src[0]->type)) return f;   // (their one kernel has no fused consumer)
    const int64_t N = n0->ne[0];
    if (n1->op != GGML_OP_ADD && n1->op != GGML_OP_GLU) return f;
    if (node_reason(n1)) return f;
    if (!is_f32_rows(n1) || n_elems(n1) != N) return f;
    const ggml_tensor* other = n1->src[0] == n0 ? n1->src[1] : (n1->src[1] == n0 ? n1->src[0] : nullptr);
    if (!other || other == n0 || n_elems(other) != N) return f;
    // the activation row is read by every CTA: the fused output must not overlap it at all; it may overlap the product
    // or the other operand only as the same elements (in place)
    if (overlap(n1, n0->src[1])) return f;
    if (overlap(n1, n0) && !same_elements(n1, n0)) return f;
    if (overlap(n1, other) && !same_elements(n1, other)) return f;
    if (n1->op == GGML_OP_ADD) f.mode = 1;
    else f.mode = n1->src[0] == n0 ? 2u : 3u;
    f.e = other;
    f.out = n1;
    return f;
}

// quantize + mul_mat of one node
bool record_mul_mat(Recorder& r, const ggml_tensor* node, const Epilogue& ep) {
    WeightRef w;
    uint32_t path = 0;
    if (mul_mat_reason(node, &w, &path)) return false;
    const ggml_tensor* x = node->src[1];
    const uint32_t K = w.K, N = w.N, M = (uint32_t)x->ne[1];
    const bool q4k = per_256(w.type);
    const char* tname = type_name(w.type);
    const uint64_t ad_need = q4k ? (uint64_t)M * (K / 256) * 48u : (uint64_t)M * (K / 32) * 4u;
    const AcBufferBinding Q = bind(w.buf->buf, w.q_off, w.q_range), S = bind(w.buf->buf, w.s_off, w.s_range);
    const AcBufferBinding X = bind_tensor(x), Y = bind_tensor(node);
    r.mul_mats++;
    if (ep.mode) path = AC_B200_PATH_GEMV;   // the fused consumers live on the register-staged one-row kernels
    // the row sits quantized in the scratch already (the fused RMS norm + quantize, or an earlier MUL_MAT on it)
    if (path == AC_B200_PATH_GEMV_FQ && r.q_data == x->data && r.q_M == M && r.q_K == K && (r.q_scheme & 1) == (q4k ? 1 : 0))
        path = AC_B200_PATH_GEMV;
    if (path != AC_B200_PATH_GEMM_TC) {
        r.mmq++;
        if (q4k) r.mmqb++;
    }
    switch (path) {
        case AC_B200_PATH_GEMV_FQ: {   // one launch that quantizes the row inside the GEMV
            AcBufferBinding b[4] = {Q, S, X, Y};
            const uint32_t push[3] = {N, K, 0};   // ties-to-even per-32 / ggml's per-256 convention
            return dispatch(r, (std::string(q4k ? "ameva_mmvqb_" : "ameva_mmvq_") + tname + "_fq").c_str(), b, 4, push,
                            sizeof(push));
        }
        case AC_B200_PATH_GEMM_TC: {
            if (!record_quantize(r, x, w.type, M, K, true)) return false;
            if (byte_decoded(w.type)) {
                // the types decoded to bytes share one kernel, which reads (scale, offset) per 16 weights from a table
                // that ameva_mmtc_scales writes from the weight's scale records (64 bytes per 256 weights)
                const AcBufferBinding H = bind(r.be->gh, 0, (uint64_t)N * (K / 16) * 4);
                AcBufferBinding sb[2] = {S, H};
                const uint32_t spush[3] = {(uint32_t)w.type, N, K};
                if (!dispatch(r, "ameva_mmtc_scales", sb, 2, spush, sizeof(spush))) return false;
                ac_runtime_batch_barrier(r.batch);
                const bool is_signed = w.type == GGML_TYPE_Q6_K || w.type == GGML_TYPE_IQ4_XS || w.type == GGML_TYPE_Q3_K;
                AcBufferBinding b8[5] = {Q, H, bind(r.be->ah, 0, (uint64_t)M * K * 2), Y, bind(r.be->ae, 0, (uint64_t)M * 4)};
                const uint32_t push8[6] = {M, N, K, N, 0, is_signed ? 1u : 0u};
                if (!dispatch(r, "ameva_mmtc_b8", b8, 5, push8, sizeof(push8))) return false;
                ac_runtime_batch_barrier(r.batch);   // the next product's table may overwrite this one
                return true;
            }
            AcBufferBinding b[5] = {Q, S, bind(r.be->ah, 0, (uint64_t)M * K * 2), Y, bind(r.be->ae, 0, (uint64_t)M * 4)};
            const uint32_t push[5] = {M, N, K, N, 0};
            return dispatch(r, (std::string("ameva_mmtc_") + tname).c_str(), b, 5, push, sizeof(push));
        }
        case AC_B200_PATH_GEMV_MMA: {
            if (!record_quantize(r, x, w.type, M, K, false)) return false;
            AcBufferBinding b[5] = {Q, S, bind(r.be->aq, 0, (uint64_t)M * K), bind(r.be->ad, 0, ad_need), Y};
            const uint32_t push[4] = {M, N, K, N};
            return dispatch(r, "ameva_mmvm_q4_K", b, 5, push, sizeof(push));
        }
        case AC_B200_PATH_GEMV_STREAMED: {
            if (!record_quantize(r, x, w.type, M, K, false)) return false;
            AcBufferBinding b[12] = {Q, S, bind(r.be->aq, 0, (uint64_t)M * K), bind(r.be->ad, 0, ad_need), Y, Y, Y, Y, Y, Y, Y, Y};
            const uint32_t push[6] = {M, N, K, N, 0, 0};
            return dispatch(r, (std::string("ameva_mmvs_") + tname).c_str(), b, 12, push, sizeof(push));
        }
        case AC_B200_PATH_GEMV: {
            if (!record_quantize(r, x, w.type, M, K, false)) return false;
            std::string name = std::string(q4k ? "ameva_mmvqb_" : "ameva_mmvq_") + tname;
            if (ep.mode) {
                AcBufferBinding b[7] = {Q, S, bind(r.be->aq, 0, (uint64_t)K), bind(r.be->ad, 0, ad_need), Y, bind_tensor(ep.e),
                                        bind_tensor(ep.out)};
                const uint32_t push[5] = {1, N, K, N, ep.mode};
                return dispatch(r, (name + "_ep").c_str(), b, 7, push, sizeof(push));
            }
            const uint64_t ad_row = q4k ? (uint64_t)(K / 256) * 48u : (uint64_t)(K / 32) * 4u;
            for (uint32_t m0 = 0; m0 < M; m0 += 8) {   // chunks of 8 rows
                const uint32_t mc = M - m0 < 8 ? M - m0 : 8;
                AcBufferBinding b[5] = {Q, S, bind(r.be->aq, (uint64_t)m0 * K, (uint64_t)mc * K),
                                        bind(r.be->ad, m0 * ad_row, mc * ad_row),
                                        bind(buffer_of(node)->buf, tensor_offset(node) + (uint64_t)m0 * N * 4, (uint64_t)mc * N * 4)};
                const uint32_t push[4] = {mc, N, K, N};
                if (!dispatch(r, name.c_str(), b, 5, push, sizeof(push))) return false;
            }
            return true;
        }
        default: return false;
    }
}

// Consecutive one-row MUL_MATs that share src1 (q / k / v; gate / up) as one launch. nodes[0..count) are the MUL_MATs.
bool record_group(Recorder& r, const ggml_tensor* const* nodes, uint32_t count) {
    WeightRef w[4];
    for (uint32_t j = 0; j < count; ++j)
        if (mul_mat_reason(nodes[j], &w[j])) return false;
    const bool q4k = per_256(w[0].type);
    AcBufferBinding b[13];
    uint32_t push[7] = {w[0].K, 0, count, 0, 0, 0, 0};
    for (uint32_t j = 0; j < 4; ++j) {
        const uint32_t jj = j < count ? j : 0;
        b[3 * j] = bind(w[jj].buf->buf, w[jj].q_off, w[jj].q_range);
        b[3 * j + 1] = bind(w[jj].buf->buf, w[jj].s_off, w[jj].s_range);
        b[3 * j + 2] = bind_tensor(nodes[jj]);
        if (j < count) push[3 + j] = w[j].N;
    }
    r.mul_mats += count;
    r.mmq += count;
    if (q4k) r.mmqb += count;
    r.fused += count - 1;
    const ggml_tensor* x = nodes[0]->src[1];
    const std::string name = std::string(q4k ? "ameva_mmvqgb_" : "ameva_mmvqg_") + type_name(w[0].type);
    // the row is in the scratch already (the fused RMS norm + quantize wrote it, or an earlier MUL_MAT): no quantize
    // inside the launch
    if (r.q_data == x->data && r.q_M == 1 && r.q_K == w[0].K && (r.q_scheme & 1) == (q4k ? 1 : 0)) {
        AcBufferBinding bb[14];
        for (int i = 0; i < 12; ++i) bb[i] = b[i];
        bb[12] = bind(r.be->aq, 0, w[0].K);
        bb[13] = bind(r.be->ad, 0, q4k ? (uint64_t)(w[0].K / 256) * 48u : (uint64_t)(w[0].K / 32) * 4u);
        return dispatch(r, name.c_str(), bb, 14, push, sizeof(push));
    }
    b[12] = bind_tensor(x);
    return dispatch(r, (name + "_fq").c_str(), b, 13, push, sizeof(push));
}

// Can node b join the group that starts with node a? (one activation row, the same src1, type and K, an even N, the
// one-launch path for the shape, outputs that do not overlap the shared activation row or each other)
bool groups_with(const ggml_tensor* a, const ggml_tensor* b) {
    if (b->op != GGML_OP_MUL_MAT) return false;
    WeightRef wa, wb;
    uint32_t pa = 0, pb = 0;
    if (mul_mat_reason(a, &wa, &pa) || mul_mat_reason(b, &wb, &pb)) return false;
    return pa == AC_B200_PATH_GEMV_FQ && pb == AC_B200_PATH_GEMV_FQ && a->src[1]->data == b->src[1]->data &&
           buffer_of(a->src[1]) == buffer_of(b->src[1]) && a->src[1]->ne[1] == 1 && b->src[1]->ne[1] == 1 && wa.type == wb.type &&
           wa.K == wb.K && wa.N % 2 == 0 && wb.N % 2 == 0 && !overlap(b, a->src[1]) && !overlap(a, a->src[1]) && !overlap(a, b);
}

bool record_elementwise(Recorder& r, const ggml_tensor* node, const ggml_tensor* fused_mul) {
    switch (node->op) {
        case GGML_OP_ADD:
        case GGML_OP_MUL: {
            AcBufferBinding b[3] = {bind_tensor(node->src[0]), bind_tensor(node->src[1]), bind_tensor(node)};
            const uint32_t push[3] = {(uint32_t)n_rows(node), (uint32_t)node->ne[0], (uint32_t)n_rows(node->src[1])};
            return dispatch(r, node->op == GGML_OP_ADD ? "ameva_add_f32" : "ameva_mul_f32", b, 3, push, sizeof(push));
        }
        case GGML_OP_GLU: {
            AcBufferBinding b[3] = {bind_tensor(node->src[0]), bind_tensor(node->src[1]), bind_tensor(node)};
            const uint32_t push[1] = {(uint32_t)n_elems(node)};
            return dispatch(r, "ameva_swiglu_f32", b, 3, push, sizeof(push));
        }
        case GGML_OP_RMS_NORM: {
            // alone, or with the MUL by a weight row that follows it (one kernel writes the MUL's output)
            const ggml_tensor* wt = nullptr;
            const ggml_tensor* out = node;
            if (fused_mul) {
                wt = fused_mul->src[0] == node ? fused_mul->src[1] : fused_mul->src[0];
                out = fused_mul;
            }
            AcBufferBinding b[3] = {bind_tensor(node->src[0]), wt ? bind_tensor(wt) : bind_tensor(node->src[0]), bind_tensor(out)};
            uint32_t push[4] = {(uint32_t)n_rows(node), (uint32_t)node->ne[0], 0, wt ? 1u : 0u};
            memcpy(&push[2], &node->op_params[0], 4);   // eps
            return dispatch(r, "ameva_rms_norm_f32", b, 3, push, sizeof(push));
        }
        default: return false;
    }
}

// ROPE, GET_ROWS, SET_ROWS, SOFT_MAX, FLASH_ATTN_EXT: push constants as the reference's encoders build them
// f32 rows -> q8_0 / q4_0 blocks with ameva_set_rows_q8_0 / _q4_0: SET_ROWS (idx given) or a same-shape CPY (idx == nullptr);
// the reference's enc_store_quantized (ggml-ameva.cpp:4008-4036)
bool record_store_quantized(Recorder& r, const ggml_tensor* node, const ggml_tensor* a, const ggml_tensor* idx,
                            const AcBufferBinding& status, int node_index) {
    ElemBind ba, bi, bd;
    if (!bind_elems(a, 4, &ba) || !bind_elems(node, 2, &bd) || (idx && !bind_elems(idx, 4, &bi))) return false;
    if (!idx) bi = ba;   // binding 1 is not read in identity mode
    const uint32_t mode = !idx ? 0u : (idx->type == GGML_TYPE_I64 ? 2u : 1u);
    const uint32_t pc[21] = {(uint32_t)(a->ne[0] / 32), (uint32_t)a->ne[1], (uint32_t)a->ne[2], (uint32_t)a->ne[3],
                             ba.elem, st(a, 1, 4), st(a, 2, 4), st(a, 3, 4),
                             idx ? bi.elem : 0u, idx ? (uint32_t)(idx->nb[0] / 4) : 0u, idx ? (uint32_t)(idx->nb[1] / 4) : 0u,
                             idx ? (uint32_t)(idx->nb[2] / 4) : 0u, idx ? (uint32_t)idx->ne[1] : 1u, idx ? (uint32_t)idx->ne[2] : 1u,
                             mode, (uint32_t)node->ne[1],
                             bd.elem * 2u, (uint32_t)node->nb[1], (uint32_t)node->nb[2], (uint32_t)node->nb[3], (uint32_t)node_index};
    const AcBufferBinding bb[4] = {ba.b, bi.b, status, bd.b};
    if (idx) r.rows_ops = true;
    return dispatch(r, node->type == GGML_TYPE_Q8_0 ? "ameva_set_rows_q8_0" : "ameva_set_rows_q4_0", bb, 4, pc, sizeof(pc));
}

bool record_layer_op(Recorder& r, const ggml_tensor* node, int node_index) {
    const ggml_tensor *a = node->src[0], *b = node->src[1];
    const AcBufferBinding status = bind(r.be->op_status, 0, 256);
    if (is_unary_like(node->op)) {
        ElemBind ba, bd;
        if (!bind_elems(a, 4, &ba) || !bind_elems(node, 4, &bd)) return false;
        uint32_t p0 = 0, p1 = 0;
        if (node->op == GGML_OP_SCALE) {
            p0 = f32_bits(param_f32(node, 0));
            p1 = f32_bits(param_f32(node, 1));
        } else if (node->op == GGML_OP_LEAKY_RELU) {
            p0 = f32_bits(param_f32(node, 0));
        }
        const uint32_t pc[15] = {(uint32_t)node->ne[0], (uint32_t)node->ne[1], (uint32_t)node->ne[2], (uint32_t)node->ne[3],
                                 ba.elem, st(a, 1, 4), st(a, 2, 4), st(a, 3, 4), bd.elem, st(node, 1, 4), st(node, 2, 4),
                                 st(node, 3, 4), (uint32_t)unary_code(node), p0, p1};
        const AcBufferBinding bb[2] = {ba.b, bd.b};
        return dispatch(r, "ameva_unary", bb, 2, pc, sizeof(pc));
    }
    switch (node->op) {
        case GGML_OP_ROPE: {
            const ggml_tensor* ff = node->src[2];
            const size_t es = elem_size(a->type);
            ElemBind ba, bp, bf, bd;
            if (!bind_elems(a, es, &ba) || !bind_elems(b, 4, &bp) || !bind_elems(ff ? ff : b, 4, &bf) || !bind_elems(node, es, &bd)) return false;
            const int n_dims = node->op_params[1], mode = node->op_params[2], n_ctx_orig = node->op_params[4];
            const float freq_base = param_f32(node, 5), freq_scale = param_f32(node, 6), ext_factor = param_f32(node, 7),
                        attn_factor = param_f32(node, 8), beta_fast = param_f32(node, 9), beta_slow = param_f32(node, 10);
            float corr[2];
            rope_corr_dims(n_dims, n_ctx_orig, freq_base, beta_fast, beta_slow, corr);
            const float theta_scale = n_dims > 0 ? powf(freq_base, -2.0f / n_dims) : 1.0f;
            const uint32_t pc[23] = {(uint32_t)node->ne[0], (uint32_t)node->ne[1], (uint32_t)node->ne[2], (uint32_t)node->ne[3],
                                     ba.elem, st(a, 1, es), st(a, 2, es), st(a, 3, es),
                                     bd.elem, st(node, 1, es), st(node, 2, es), st(node, 3, es),
                                     bp.elem, ff ? bf.elem : 0u, (uint32_t)n_dims, mode == 2 ? 1u : 0u,
                                     ff ? 1u : 0u, f32_bits(theta_scale), f32_bits(freq_scale), f32_bits(ext_factor),
                                     f32_bits(attn_factor), f32_bits(corr[0]), f32_bits(corr[1])};
            const AcBufferBinding bb[4] = {ba.b, bp.b, bf.b, bd.b};
            return dispatch(r, a->type == GGML_TYPE_F16 ? "ameva_rope_f16" : "ameva_rope", bb, 4, pc, sizeof(pc));
        }
        case GGML_OP_CPY:
        case GGML_OP_CONT:
        case GGML_OP_DUP: {
            if (is_kvq(node)) return record_store_quantized(r, node, a, nullptr, status, node_index);
            if (is_kvq(a)) {   // addressed in bytes: offset and strides in bytes, a_s0 = the block size
                const size_t ds = elem_size(node->type);
                ElemBind ba, bd;
                if (!bind_elems(a, 2, &ba) || !bind_elems(node, ds, &bd)) return false;
                const uint32_t pc[19] = {(uint32_t)a->ne[0], (uint32_t)a->ne[1], (uint32_t)a->ne[2], (uint32_t)a->ne[3],
                                         ba.elem * 2u, (uint32_t)a->nb[0], (uint32_t)a->nb[1], (uint32_t)a->nb[2],
                                         (uint32_t)a->nb[3], (uint32_t)node->ne[0], (uint32_t)node->ne[1], (uint32_t)node->ne[2],
                                         bd.elem, st(node, 0, ds), st(node, 1, ds), st(node, 2, ds),
                                         st(node, 3, ds), a->type == GGML_TYPE_Q8_0 ? 2u : 3u, node->type == GGML_TYPE_F16 ? 1u : 0u};
                const AcBufferBinding bb[2] = {ba.b, bd.b};
                return dispatch(r, "ameva_cpy", bb, 2, pc, sizeof(pc));
            }
            const size_t es = elem_size(a->type), ds = elem_size(node->type);
            ElemBind ba, bd;
            if (!bind_elems(a, es, &ba) || !bind_elems(node, ds, &bd)) return false;
            const uint32_t pc[19] = {(uint32_t)a->ne[0], (uint32_t)a->ne[1], (uint32_t)a->ne[2], (uint32_t)a->ne[3],
                                     ba.elem, st(a, 0, es), st(a, 1, es), st(a, 2, es),
                                     st(a, 3, es), (uint32_t)node->ne[0], (uint32_t)node->ne[1], (uint32_t)node->ne[2],
                                     bd.elem, st(node, 0, ds), st(node, 1, ds), st(node, 2, ds),
                                     st(node, 3, ds), a->type == GGML_TYPE_F16 ? 1u : 0u, node->type == GGML_TYPE_F16 ? 1u : 0u};
            const AcBufferBinding bb[2] = {ba.b, bd.b};
            return dispatch(r, "ameva_cpy", bb, 2, pc, sizeof(pc));
        }
        case GGML_OP_GET_ROWS: {
            if (is_repacked_weight(a)) {
                // ameva_get_rows_<type>_rp: the table in the device layout (payload region, scale region at s_off)
                ElemBind bi, bd;
                if (!bind_elems(b, 4, &bi) || !bind_elems(node, 4, &bd)) return false;
                uint64_t s_off = 0;
                const uint64_t total = device_bytes(a, &s_off);
                const uint64_t nblk_row = (uint64_t)a->ne[0] / block_elems(a->type);
                const uint64_t q_row = nblk_row * payload_bytes(a->type), s_row = nblk_row * scale_bytes(dev_type(a->type));
                if (s_off > 0xFFFFFFFFull || q_row > 0xFFFFFFFFull) return false;
                const uint32_t pc[25] = {(uint32_t)node->ne[0], (uint32_t)b->ne[0], 1u, 1u, 0u, 0u, 0u, 0u,
                                         bi.elem, st(b, 0, 4), 0u, 0u, bd.elem, st(node, 1, 4), st(node, 2, 4), st(node, 3, 4),
                                         (uint32_t)a->ne[1], (uint32_t)node_index, 0u, (uint32_t)a->ne[1],
                                         0u, (uint32_t)s_off, (uint32_t)q_row, 0u, (uint32_t)s_row};
                const AcBufferBinding bb[4] = {bind(buffer_of(a)->buf, tensor_offset(a), total), bi.b, status, bd.b};
                std::string name = std::string("ameva_get_rows_") + type_name(dev_type(a->type)) + "_rp";
                for (char& ch : name) ch = (char)tolower((unsigned char)ch);
                r.rows_ops = true;
                return dispatch(r, name.c_str(), bb, 4, pc, sizeof(pc));
            }
            const size_t es = elem_size(a->type);
            ElemBind ba, bi, bd;
            if (!bind_elems(a, es, &ba) || !bind_elems(b, 4, &bi) || !bind_elems(node, 4, &bd)) return false;
            const uint32_t pc[19] = {(uint32_t)node->ne[0], (uint32_t)b->ne[0], (uint32_t)b->ne[1], (uint32_t)b->ne[2],
                                     ba.elem, st(a, 1, es), st(a, 2, es), st(a, 3, es),
                                     bi.elem, st(b, 0, 4), st(b, 1, 4), st(b, 2, 4),
                                     bd.elem, st(node, 1, 4), st(node, 2, 4), st(node, 3, 4),
                                     a->type == GGML_TYPE_F16 ? 1u : 0u, (uint32_t)a->ne[1], (uint32_t)node_index};
            const AcBufferBinding bb[4] = {ba.b, bi.b, status, bd.b};
            r.rows_ops = true;
            return dispatch(r, "ameva_get_rows", bb, 4, pc, sizeof(pc));
        }
        case GGML_OP_SET_ROWS: {
            if (is_kvq(node)) return record_store_quantized(r, node, a, b, status, node_index);
            const size_t es = elem_size(node->type);
            ElemBind ba, bi, bd;
            if (!bind_elems(a, 4, &ba) || !bind_elems(b, 4, &bi) || !bind_elems(node, es, &bd)) return false;
            const uint32_t pc[22] = {(uint32_t)a->ne[0], (uint32_t)a->ne[1], (uint32_t)a->ne[2], (uint32_t)a->ne[3],
                                     ba.elem, st(a, 1, 4), st(a, 2, 4), st(a, 3, 4),
                                     bi.elem, (uint32_t)(b->nb[0] / 4), (uint32_t)(b->nb[1] / 4), (uint32_t)(b->nb[2] / 4),
                                     (uint32_t)b->ne[1], (uint32_t)b->ne[2], b->type == GGML_TYPE_I64 ? 1u : 0u, (uint32_t)node->ne[1],
                                     bd.elem, st(node, 1, es), st(node, 2, es), st(node, 3, es),
                                     node->type == GGML_TYPE_F16 ? 1u : 0u, (uint32_t)node_index};
            const AcBufferBinding bb[4] = {ba.b, bi.b, status, bd.b};
            r.rows_ops = true;
            return dispatch(r, "ameva_set_rows", bb, 4, pc, sizeof(pc));
        }
        case GGML_OP_SOFT_MAX: {
            const size_t ms = b ? elem_size(b->type) : 4;
            ElemBind ba, bd, bm;
            if (!bind_elems(a, 4, &ba) || !bind_elems(node, 4, &bd) || !bind_elems(b ? b : a, ms, &bm)) return false;
            const uint32_t nrows = (uint32_t)(node->ne[1] * node->ne[2] * node->ne[3]);
            const uint32_t pc[20] = {(uint32_t)node->ne[0], (uint32_t)node->ne[1], (uint32_t)node->ne[2], nrows,
                                     ba.elem, st(a, 1, 4), st(a, 2, 4), st(a, 3, 4),
                                     bd.elem, st(node, 1, 4), st(node, 2, 4), st(node, 3, 4),
                                     f32_bits(param_f32(node, 0)),
                                     b ? (b->type == GGML_TYPE_F16 ? 2u : 1u) : 0u, b ? bm.elem : 0u, b ? st(b, 1, ms) : 0u,
                                     b ? st(b, 2, ms) : 0u, b ? st(b, 3, ms) : 0u, b ? (uint32_t)b->ne[2] : 1u, b ? (uint32_t)b->ne[3] : 1u};
            const AcBufferBinding bb[3] = {ba.b, bd.b, bm.b};
            return dispatch(r, "ameva_soft_max", bb, 3, pc, sizeof(pc));
        }
        case GGML_OP_FLASH_ATTN_EXT: {
            const ggml_tensor *k = node->src[1], *v = node->src[2], *m = node->src[3];
            ElemBind bq, bk, bv, bm, bo;
            if (!bind_elems(a, 4, &bq) || !bind_elems(m ? m : a, m ? 2 : 4, &bm) || !bind_elems(node, 4, &bo)) return false;
            const uint32_t D = (uint32_t)a->ne[0];
            // a q8_0 / q4_0 cache is dequantized into f16 scratch [n_head_kv][n_kv][D] first (ameva_cpy from the quantized
            // view), and the attention kernel reads the scratch: one pass more over the cache than a kernel that decodes
            // the blocks itself would need
            uint32_t ks1 = 0, ks2 = 0, vs1 = 0, vs2 = 0;
            auto operand = [&](const ggml_tensor* t, AcBuffer* scratch, ElemBind* out, uint32_t* s1, uint32_t* s2) -> bool {
                if (!is_kvq(t)) {
                    if (!bind_elems(t, 2, out)) return false;
                    *s1 = st(t, 1, 2);
                    *s2 = st(t, 2, 2);
                    return true;
                }
                ElemBind src;
                if (!bind_elems(t, 2, &src)) return false;
                const uint64_t bytes = (uint64_t)t->ne[0] * t->ne[1] * t->ne[2] * 2u;
                const uint32_t cp[19] = {(uint32_t)t->ne[0], (uint32_t)t->ne[1], (uint32_t)t->ne[2], 1u,
                                         src.elem * 2u, (uint32_t)t->nb[0], (uint32_t)t->nb[1], (uint32_t)t->nb[2],
                                         (uint32_t)t->nb[3], (uint32_t)t->ne[0], (uint32_t)t->ne[1], (uint32_t)t->ne[2],
                                         0u, 1u, (uint32_t)t->ne[0], (uint32_t)(t->ne[0] * t->ne[1]),
                                         (uint32_t)(t->ne[0] * t->ne[1] * t->ne[2]), t->type == GGML_TYPE_Q8_0 ? 2u : 3u, 1u};
                const AcBufferBinding cb[2] = {src.b, bind(scratch, 0, bytes)};
                if (!dispatch(r, "ameva_cpy", cb, 2, cp, sizeof(cp))) return false;
                out->b = bind(scratch, 0, bytes);
                out->elem = 0;
                *s1 = (uint32_t)t->ne[0];
                *s2 = (uint32_t)(t->ne[0] * t->ne[1]);
                return true;
            };
            if (!operand(k, r.be->kv_f16[0], &bk, &ks1, &ks2) || !operand(v, r.be->kv_f16[1], &bv, &vs1, &vs2)) return false;
            if (is_kvq(k) || is_kvq(v)) ac_runtime_batch_barrier(r.batch);
            const uint32_t pc[31] = {D, D, (uint32_t)k->ne[1], (uint32_t)a->ne[1],
                                     (uint32_t)a->ne[2], (uint32_t)k->ne[2], 0x11u, m ? 1u : 0u,
                                     bq.elem, st(a, 1, 4), st(a, 2, 4), bk.elem,
                                     ks1, ks2, bv.elem, vs1,
                                     vs2, m ? bm.elem : 0u, m ? st(m, 1, 2) : 0u, m ? st(m, 2, 2) : 0u,
                                     m ? (uint32_t)m->ne[2] : 1u, bo.elem, f32_bits(param_f32(node, 0)), f32_bits(param_f32(node, 2)),
                                     0u, 0u, 0u, 0u, 0u, 0u, 0u};
            const AcBufferBinding bb[6] = {bq.b, bk.b, bv.b, bm.b, bo.b, bind(r.be->fa_part, 0, r.be->fa_part_bytes)};
            return dispatch(r, "ameva_flash_attn", bb, 6, pc, sizeof(pc));
        }
        default: return false;
    }
}

// RMS_NORM followed by MUL with a weight row of the same width (the RMS_NORM + MUL pair of ameva_find_fusion)
bool rms_mul_pair(const ggml_tensor* n0, const ggml_tensor* n1) {
    if (!n1 || n0->op != GGML_OP_RMS_NORM || n1->op != GGML_OP_MUL || node_reason(n1)) return false;
    const ggml_tensor* wt = n1->src[0] == n0 ? n1->src[1] : (n1->src[1] == n0 ? n1->src[0] : nullptr);
    if (!wt || wt == n0 || n_rows(wt) != 1 || wt->ne[0] != n0->ne[0] || n_elems(n1) != n_elems(n0)) return false;
    if (overlap(n1, wt)) return false;
    if (overlap(n1, n0->src[0]) && !same_elements(n1, n0->src[0])) return false;
    return true;
}

// RMS_NORM (+ the MUL by a weight row) whose result is the activation of the MUL_MAT `consumer`: one kernel writes the
// normalised rows and their quantized form into the scratch (ameva_rms_norm_quant_a8 / a8b), so the MUL_MAT (or the
// grouped launch it starts) finds its activations quantized. False when the pattern does not apply (nothing recorded).
bool record_norm_quantize(Recorder& r, const ggml_tensor* node, const ggml_tensor* fused_mul, const ggml_tensor* consumer,
                          QuantizedRows* fresh) {
    const ggml_tensor* out = fused_mul ? fused_mul : node;
    if (!consumer || consumer->op != GGML_OP_MUL_MAT || consumer->src[1] != out) return false;
    WeightRef w;
    uint32_t path = 0;
    if (mul_mat_reason(consumer, &w, &path)) return false;
    const uint32_t M = (uint32_t)n_rows(out), K = (uint32_t)out->ne[0];
    if (K != w.K || K > 32768u || (uint64_t)n_rows(out) != (uint64_t)out->ne[1] || !ggml_is_contiguous(node->src[0])) return false;
    const bool q4k = per_256(w.type), tc = path == AC_B200_PATH_GEMM_TC;
    if (path == AC_B200_PATH_GEMV && M > 8) return false;   // the exact chunked path quantizes per chunk layout as usual
    const ggml_tensor* wt = nullptr;
    if (fused_mul) wt = fused_mul->src[0] == node ? fused_mul->src[1] : fused_mul->src[0];
    const uint64_t ad_need = q4k ? (uint64_t)M * (K / 256) * 48u : (uint64_t)M * (K / 32) * 4u;
    AcBufferBinding b[7] = {bind_tensor(node->src[0]), wt ? bind_tensor(wt) : bind_tensor(node->src[0]), bind_tensor(out),
                            bind(r.be->aq, 0, (uint64_t)M * K), bind(r.be->ad, 0, ad_need),
                            tc ? bind(r.be->ah, 0, (uint64_t)M * K * 2) : bind(r.be->aq, 0, (uint64_t)M * K),
                            tc ? bind(r.be->ae, 0, (uint64_t)M * 4) : bind(r.be->aq, 0, (uint64_t)M * K)};
    uint32_t push[7] = {M, K, K, 0, 0, wt ? 1u : 0u, tc ? 1u : 0u};
    memcpy(&push[4], &node->op_params[0], 4);   // eps
    if (!dispatch(r, q4k ? "ameva_rms_norm_quant_a8b" : "ameva_rms_norm_quant_a8", b, 7, push, sizeof(push))) return false;
    fresh->data = out->data;
    fresh->M = M;
    fresh->K = K;
    fresh->scheme = (q4k ? 1 : 0) + (tc ? 2 : 0);
    return true;
}

const char* backend_get_name(ggml_backend_t) { return GGML_AMEVA_B200_NAME; }

void backend_free(ggml_backend_t backend) {
    Backend* be = (Backend*)backend->context;
    {
        std::lock_guard<std::mutex> lock(plugin().mutex);
        for (auto& kv : be->kernels)
            if (ac_runtime_kernel_destroy(kv.second) == AC_SUCCESS) g_count.kernel_destroy++;
        for (AcBuffer* b : {be->aq, be->ad, be->ah, be->ae, be->gh, be->op_status, be->fa_part, be->kv_f16[0], be->kv_f16[1]})
            if (b && ac_runtime_buffer_destroy(b) == AC_SUCCESS) g_count.buffer_destroy++;
        plugin().live_backends--;
    }
    delete be;
    delete backend;
}

int next_compute_node(ggml_cgraph* g, int i, int n) {   // the first node after i that computes something, or -1
    for (int j = i + 1; j < n; ++j) {
        const ggml_tensor* t = ggml_graph_node(g, j);
        if (!is_view_op(t->op) && !ggml_is_empty(t)) return j;
    }
    return -1;
}

enum ggml_status backend_graph_compute(ggml_backend_t backend, ggml_cgraph* cgraph) {
    Backend* be = (Backend*)backend->context;
    std::lock_guard<std::mutex> lock(plugin().mutex);
    const int fi = g_fail.load();
    const int n = ggml_graph_n_nodes(cgraph);
    int work = 0;
    for (int i = 0; i < n; ++i) {   // every node first: nothing is recorded if one cannot run
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (const char* why = node_reason(node)) {
            fprintf(stderr, "ggml-ameva-b200: node %d (%s, %s) cannot run here: %s\n", i, ggml_op_name(node->op), node->name, why);
            return GGML_STATUS_FAILED;
        }
        if (!is_view_op(node->op) && !ggml_is_empty(node)) ++work;
    }
    if (work == 0) return GGML_STATUS_SUCCESS;
    if (fi == AMEVA_FAIL_TENSOR_RANGE_OOB || fi == AMEVA_FAIL_MAP_SRC0 || fi == AMEVA_FAIL_MAP_SRC1 || fi == AMEVA_FAIL_MAP_DST ||
        fi == AMEVA_FAIL_OFFSET_OVERFLOW || fi == AMEVA_FAIL_FLUSH_SRC0 || fi == AMEVA_FAIL_FLUSH_SRC1) {
        fprintf(stderr, "ggml-ameva-b200 [FAILURE_INJECTION]: point %d triggered while binding\n", fi);
        return GGML_STATUS_FAILED;
    }
    // scratch for the quantized activations: the largest need over all nodes, reserved before anything is recorded
    size_t aq_need = 0, ad_need = 0, ah_need = 0, ae_need = 0, gh_need = 0;
    for (int i = 0; i < n; ++i) {
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (node->op != GGML_OP_MUL_MAT) continue;
        const ggml_tensor *w = node->src[0], *x = node->src[1];
        const size_t K = (size_t)w->ne[0], M = (size_t)x->ne[1];
        aq_need = std::max(aq_need, M * K);
        ad_need = std::max(ad_need, per_256(w->type) ? M * (K / 256) * 48u : M * (K / 32) * 4u);
        if (M > 8 && K % 256 == 0) {
            ah_need = std::max(ah_need, M * K * 2);
            ae_need = std::max(ae_need, M * 4);
            if (byte_decoded(w->type)) gh_need = std::max(gh_need, (size_t)w->ne[1] * (K / 16) * 4);
        }
    }
    if ((aq_need && !grow(&be->aq, &be->aq_bytes, aq_need)) || (ad_need && !grow(&be->ad, &be->ad_bytes, ad_need)) ||
        (ah_need && !grow(&be->ah, &be->ah_bytes, ah_need)) || (ae_need && !grow(&be->ae, &be->ae_bytes, ae_need)) ||
        (gh_need && !grow(&be->gh, &be->gh_bytes, gh_need)))
        return GGML_STATUS_ALLOC_FAILED;
    size_t kvf_need[2] = {0, 0};
    for (int i = 0; i < n; ++i) {
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (node->op != GGML_OP_FLASH_ATTN_EXT) continue;
        for (int j = 0; j < 2; ++j) {
            const ggml_tensor* t = node->src[1 + j];
            if (t && is_kvq(t)) kvf_need[j] = std::max(kvf_need[j], (size_t)(t->ne[0] * t->ne[1] * t->ne[2] * 2));
        }
    }
    for (int j = 0; j < 2; ++j)
        if (kvf_need[j] && !grow(&be->kv_f16[j], &be->kv_f16_bytes[j], kvf_need[j])) return GGML_STATUS_ALLOC_FAILED;
    bool layer_ops = false;
    for (int i = 0; i < n && !layer_ops; ++i) layer_ops = is_layer_op(ggml_graph_node(cgraph, i)->op);
    if (layer_ops) {
        if (!grow(&be->op_status, &be->op_status_bytes, 256) || !grow(&be->fa_part, &be->fa_part_bytes, 8u << 20)) return GGML_STATUS_ALLOC_FAILED;
        const uint32_t clear[2] = {0u, 0xFFFFFFFFu};
        if (ac_runtime_buffer_write(be->op_status, 0, clear, sizeof(clear)) != AC_SUCCESS) return GGML_STATUS_FAILED;
    }
    Recorder r;
    r.be = be;
    AcBatchDesc bd = {AC_ABI_VERSION, (uint32_t)sizeof(AcBatchDesc), 16384u, 0u};
    if (ac_runtime_batch_begin_ex(context(), &bd, &r.batch) != AC_SUCCESS) return GGML_STATUS_ALLOC_FAILED;
    bool ok = true;
    for (int i = 0; i < n && ok;) {
        const ggml_tensor* node = ggml_graph_node(cgraph, i);
        if (is_view_op(node->op) || ggml_is_empty(node)) {
            ++i;
            continue;
        }
        const int j = next_compute_node(cgraph, i, n);
        const ggml_tensor* next = j >= 0 ? ggml_graph_node(cgraph, j) : nullptr;
        int consumed_upto = i;   // index of the last node this step computes
        QuantizedRows fresh;     // rows this step itself quantized into the scratch while producing them
        if (node->op == GGML_OP_MUL_MAT) {
            // a run of one-row MUL_MATs sharing src1: one launch (up to four)
            const ggml_tensor* grp[4] = {node, nullptr, nullptr, nullptr};
            uint32_t count = 1;
            int last = i;
            for (int jj = j; jj >= 0 && count < 4 && groups_with(node, ggml_graph_node(cgraph, jj));
                 jj = next_compute_node(cgraph, jj, n)) {
                bool clash = false;   // no member may write what another member writes
                for (uint32_t q = 1; q < count && !clash; ++q) clash = overlap(ggml_graph_node(cgraph, jj), grp[q]);
                if (clash) break;
                grp[count++] = ggml_graph_node(cgraph, jj);
                last = jj;
            }
            if (count > 1) {
                ok = record_group(r, grp, count);   // (quantizes inside the kernel: the scratch holds nothing of this src1)
                r.gpu_ops += count;
                consumed_upto = last;
            } else {
                const Epilogue ep = find_epilogue(node, next);
                ok = record_mul_mat(r, node, ep);
                r.gpu_ops += 1;
                if (ep.mode) {
                    r.gpu_ops += 1;
                    r.fused += 1;
                    consumed_upto = j;
                }
            }
        } else if (node->op == GGML_OP_RMS_NORM) {
            const bool pair = rms_mul_pair(node, next);
            // the MUL_MAT that consumes the result (the next computing node): its quantize joins this launch
            const int jc = next_compute_node(cgraph, pair ? j : i, n);
            const ggml_tensor* consumer = jc >= 0 ? ggml_graph_node(cgraph, jc) : nullptr;
            if (!record_norm_quantize(r, node, pair ? next : nullptr, consumer, &fresh)) ok = record_elementwise(r, node, pair ? next : nullptr);
            r.gpu_ops += pair ? 2 : 1;
            if (pair) {
                r.fused += 1;
                consumed_upto = j;
            }
        } else if (is_layer_op(node->op)) {
            ok = record_layer_op(r, node, i);
            r.gpu_ops += 1;
        } else {
            ok = record_elementwise(r, node, nullptr);
            r.gpu_ops += 1;
        }
        // a node that wrote over the rows whose quantized form sits in the scratch invalidates it
        for (int q = i; q <= consumed_upto && r.q_data; ++q) {
            const ggml_tensor* t = ggml_graph_node(cgraph, q);
            if (is_view_op(t->op)) continue;
            const char* d0 = (const char*)t->data;
            const char* x0 = (const char*)r.q_data;
            if (d0 < x0 + (size_t)r.q_M * r.q_K * 4 && x0 < d0 + ggml_nbytes(t)) r.q_data = nullptr;
        }
        if (fresh.data) {
            r.q_data = fresh.data;
            r.q_M = fresh.M;
            r.q_K = fresh.K;
            r.q_scheme = fresh.scheme;
        }
        ac_runtime_batch_barrier(r.batch);
        i = consumed_upto + 1;
    }
    if (ok && fi == AMEVA_FAIL_DISPATCH) {
        fprintf(stderr, "ggml-ameva-b200 [FAILURE_INJECTION]: DISPATCH_FAIL triggered\n");
        ok = false;
    }
    if (!ok) {
        ac_runtime_batch_abort(r.batch);
        ac_runtime_batch_destroy(r.batch);
        return GGML_STATUS_FAILED;
    }
    AcEvent* ev = nullptr;
    AcResult rc = ac_runtime_batch_submit(r.batch, &ev);
    if (rc == AC_SUCCESS && ev) {
        g_count.event_create++;
        rc = ac_runtime_event_wait(ev, fi == AMEVA_FAIL_WAIT_TIMEOUT ? 1ull : 600ull * 1000000000ull);
        if (fi == AMEVA_FAIL_WAIT_TIMEOUT) {
            // the injected 1 ns limit has run out (or the work was already done): the graph is reported failed either way,
            // after the work has finished, so that nothing is still writing when the caller looks at its tensors
            fprintf(stderr, "ggml-ameva-b200 [FAILURE_INJECTION]: WAIT_TIMEOUT triggered\n");
            ac_runtime_event_wait(ev, 600ull * 1000000000ull);
            rc = AC_ERR_LAUNCH_TIMEOUT;
        }
        if (ac_runtime_event_destroy(ev) == AC_SUCCESS) g_count.event_destroy++;
    }
    ac_runtime_batch_destroy(r.batch);
    if (rc == AC_SUCCESS && r.rows_ops) {   // an index outside its table or cache fails the graph (ggml asserts on the CPU)
        uint32_t st2[2] = {0u, 0u};
        rc = ac_runtime_buffer_read(be->op_status, 0, st2, sizeof(st2));
        if (rc == AC_SUCCESS && st2[0]) {
            fprintf(stderr, "ggml-ameva-b200: %u row indices out of range, first at node %u\n", st2[0], st2[1]);
            rc = AC_ERR_KERNEL_ARG_INVALID;
        }
    }
    if (rc == AC_SUCCESS && fi == AMEVA_FAIL_INVALIDATE_DST) {
        fprintf(stderr, "ggml-ameva-b200 [FAILURE_INJECTION]: INVALIDATE_DST_FAIL triggered\n");
        rc = AC_ERR_BUFFER_NOT_MAPPED;
    }
    if (rc != AC_SUCCESS) return GGML_STATUS_FAILED;
    g_count.gpu_op += r.gpu_ops;
    g_count.mul_mat += r.mul_mats;
    g_count.qmv += r.mul_mats;
    g_count.mmq += r.mmq;
    g_count.mmqb += r.mmqb;
    g_count.fused_pairs += r.fused;
    return GGML_STATUS_SUCCESS;
}

ggml_guid_t backend_guid() {
    static ggml_guid guid = {0xa3, 0x1e, 0xb2, 0x00, 0x5c, 0x47, 0x4d, 0x0b, 0x91, 0x6a, 0xb2, 0x00, 0xac, 0xde, 0x10, 0x0a};
    return &guid;
}

// ---- device -----------------------------------------------------------------------------------------------------------
const char* dev_get_name(ggml_backend_dev_t) { return GGML_AMEVA_B200_DEVICE_NAME; }
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
        plugin().live_backends++;
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
    g_count.supports_query++;
    const bool yes = op_supported_static(op);
    if (yes) g_count.supported_op++;
    return yes;
}
bool dev_supports_buft(ggml_backend_dev_t, ggml_backend_buffer_type_t buft) { return buft == &plugin().buft; }
bool dev_offload_op(ggml_backend_dev_t, const ggml_tensor*) { return false; }

// ---- registry ---------------------------------------------------------------------------------------------------------
const char* reg_get_name(ggml_backend_reg_t) { return GGML_AMEVA_B200_NAME; }
size_t reg_get_device_count(ggml_backend_reg_t) { return 1; }
ggml_backend_dev_t reg_get_device(ggml_backend_reg_t, size_t index) { return index == 0 ? &plugin().dev : nullptr; }
void* reg_get_proc_address(ggml_backend_reg_t, const char* name);

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

// ggml's struct layouts and enum values, read through the loaded ggml's own accessors, against the headers this file was
// compiled with (the vtables of ggml-backend-impl.h are not versioned: ggml-ameva-device.cpp:408-414).
const char* ggml_backend_ameva_abi_check(void) {
    static std::once_flag once;
    static char msg[320];
    static const char* result = nullptr;
    std::call_once(once, [] {
        const char* what = nullptr;
        Plugin& p = plugin();
        registry();
        ggml_backend pb = {};
        pb.device = &p.dev;
        ggml_backend_buffer_type pbt = {};
        pbt.device = &p.dev;
        ggml_backend_buffer pbuf = {};
        pbuf.buft = &pbt;
        pbuf.size = 0x5A17;
        pbuf.usage = GGML_BACKEND_BUFFER_USAGE_WEIGHTS;
        ggml_backend_device pd = {};
        pd.reg = &p.reg;
        if (ggml_backend_get_device(&pb) != &p.dev) what = "struct ggml_backend (ggml_backend_i member count)";
        else if (ggml_backend_buffer_get_size(&pbuf) != 0x5A17 || ggml_backend_buffer_get_type(&pbuf) != &pbt ||
                 ggml_backend_buffer_get_usage(&pbuf) != GGML_BACKEND_BUFFER_USAGE_WEIGHTS)
            what = "struct ggml_backend_buffer (ggml_backend_buffer_i member count)";
        else if (ggml_backend_buft_get_device(&pbt) != &p.dev) what = "struct ggml_backend_buffer_type";
        else if (ggml_backend_dev_backend_reg(&pd) != &p.reg) what = "struct ggml_backend_device";
        static const struct {
            enum ggml_op op;
            const char* name;
        } kOps[] = {{GGML_OP_NONE, "NONE"},       {GGML_OP_ADD, "ADD"},         {GGML_OP_MUL, "MUL"},   {GGML_OP_RMS_NORM, "RMS_NORM"},
                    {GGML_OP_MUL_MAT, "MUL_MAT"}, {GGML_OP_RESHAPE, "RESHAPE"}, {GGML_OP_VIEW, "VIEW"}, {GGML_OP_PERMUTE, "PERMUTE"},
                    {GGML_OP_TRANSPOSE, "TRANSPOSE"}, {GGML_OP_GLU, "GLU"}, {GGML_OP_ROPE, "ROPE"}, {GGML_OP_GET_ROWS, "GET_ROWS"},
                    {GGML_OP_SET_ROWS, "SET_ROWS"}, {GGML_OP_SOFT_MAX, "SOFT_MAX"}, {GGML_OP_FLASH_ATTN_EXT, "FLASH_ATTN_EXT"},
                    {GGML_OP_CPY, "CPY"}, {GGML_OP_CONT, "CONT"}, {GGML_OP_DUP, "DUP"}, {GGML_OP_SCALE, "SCALE"},
                    {GGML_OP_UNARY, "UNARY"}, {GGML_OP_SQR, "SQR"}};
        static const struct {
            enum ggml_type type;
            const char* name;
        } kTypes[] = {{GGML_TYPE_F32, "f32"}, {GGML_TYPE_Q4_0, "q4_0"}, {GGML_TYPE_Q8_0, "q8_0"}, {GGML_TYPE_Q4_K, "q4_K"},
                      {GGML_TYPE_F16, "f16"}, {GGML_TYPE_I32, "i32"}, {GGML_TYPE_I64, "i64"}, {GGML_TYPE_Q6_K, "q6_K"}, {GGML_TYPE_Q5_K, "q5_K"}, {GGML_TYPE_IQ4_XS, "iq4_xs"}, {GGML_TYPE_Q4_1, "q4_1"}, {GGML_TYPE_Q5_1, "q5_1"}, {GGML_TYPE_Q3_K, "q3_K"}, {GGML_TYPE_Q2_K, "q2_K"}};
        for (const auto& o : kOps)
            if (!what && strcmp(ggml_op_name(o.op), o.name) != 0) what = "enum ggml_op";
        for (const auto& t : kTypes)
            if (!what && strcmp(ggml_type_name(t.type), t.name) != 0) what = "enum ggml_type";
        if (!what) {   // struct ggml_tensor: a MUL_MAT node built by the loaded ggml, read back with this file's layout
            ggml_init_params ip = {8 * ggml_tensor_overhead(), nullptr, true};
            ggml_context* tctx = ggml_init(ip);
            if (!tctx) {
                what = "ggml_init for the tensor layout probe";
            } else {
                ggml_tensor* a = ggml_new_tensor_2d(tctx, GGML_TYPE_F32, 8, 3);
                ggml_tensor* b = ggml_new_tensor_2d(tctx, GGML_TYPE_F32, 8, 2);
                ggml_tensor* c = ggml_mul_mat(tctx, a, b);
                if (!c || c->op != GGML_OP_MUL_MAT || c->src[0] != a || c->src[1] != b || c->type != GGML_TYPE_F32 || c->ne[0] != 3 ||
                    c->ne[1] != 2 || a->nb[1] != 32 || ggml_nbytes(c) != 24)
                    what = "struct ggml_tensor";
                char probe_name[512];
                memset(probe_name, 'n', sizeof(probe_name) - 1);
                probe_name[sizeof(probe_name) - 1] = 0;
                if (!what && strlen(ggml_get_name(ggml_set_name(c, probe_name))) != sizeof(c->name) - 1)
                    what = "struct ggml_tensor (GGML_MAX_NAME)";
                ggml_free(tctx);
            }
        }
        if (what) {
            snprintf(msg, sizeof(msg),
                     "ABI mismatch with the loaded ggml: %s differs from the ggml headers libggml-ameva-b200.so was compiled "
                     "with (offsetof(ggml_backend, device)=%zu). Rebuild it against the ggml of the program that loads it.",
                     what, offsetof(ggml_backend, device));
            result = msg;
        }
    });
    return result;
}

// NULL tells the loader the backend cannot be used (it prints "failed to initialize backend from <path>").
GGML_BACKEND_API ggml_backend_reg_t ggml_backend_init(void) {
    if (ac_runtime_abi_version() != AC_ABI_VERSION) {
        fprintf(stderr, "ggml-ameva-b200: refusing to load: libac_runtime_b200.so has ABI %u, built for %u\n",
                ac_runtime_abi_version(), (unsigned)AC_ABI_VERSION);
        return nullptr;
    }
    if (const char* why = ggml_backend_ameva_abi_check()) {
        fprintf(stderr, "ggml-ameva-b200: refusing to load: %s\n", why);
        return nullptr;
    }
    return registry();
}

GGML_BACKEND_API int ggml_backend_score(void) { return 100; }

ggml_backend_reg_t ggml_backend_ameva_reg(void) { return registry(); }

ggml_backend_t ggml_backend_ameva_init(size_t dev_num) {
    if (dev_num != 0 || ggml_backend_ameva_abi_check()) return nullptr;
    registry();
    return dev_init_backend(&plugin().dev, nullptr);
}

bool ggml_backend_is_ameva(ggml_backend_t backend) { return backend && ggml_guid_matches(backend->guid, backend_guid()); }

ggml_backend_buffer_type_t ggml_backend_ameva_buffer_type(size_t dev_num) {
    if (dev_num != 0) return nullptr;
    registry();
    return &plugin().buft;
}

void ggml_backend_ameva_register(void) {
    if (const char* why = ggml_backend_ameva_abi_check()) {
        fprintf(stderr, "ggml-ameva-b200: not registering the backend: %s\n", why);
        return;
    }
    ggml_backend_register(ggml_backend_ameva_reg());
}

void ggml_backend_ameva_teardown(void) {
    Plugin& p = plugin();
    std::lock_guard<std::mutex> lock(p.mutex);
    if (!p.ctx) return;
    if (p.live_backends || p.live_buffers) {
        fprintf(stderr, "ggml-ameva-b200: teardown with %d backend(s) and %d buffer(s) alive: context kept\n", p.live_backends,
                p.live_buffers);
        return;
    }
    const AcResult rc = ac_runtime_context_destroy(p.ctx);
    if (rc != AC_SUCCESS) {
        fprintf(stderr, "ggml-ameva-b200: context destroy failed (AcResult %d): something still owns runtime objects\n", (int)rc);
        return;
    }
    g_count.ctx_destroy++;
    p.ctx = nullptr;
}

int64_t ggml_backend_ameva_get_supports_query_count(void) { return g_count.supports_query.load(); }
int64_t ggml_backend_ameva_get_supported_op_count(void) { return g_count.supported_op.load(); }
int64_t ggml_backend_ameva_get_gpu_op_count(void) { return g_count.gpu_op.load(); }
int64_t ggml_backend_ameva_get_q5_0_cpu_dequant_count(void) { return 0; }
int64_t ggml_backend_ameva_get_f32_gpu_sgemm_dispatch_count(void) { return g_count.mul_mat.load(); }
int64_t ggml_backend_ameva_get_context_create_count(void) { return g_count.ctx_create.load(); }
int64_t ggml_backend_ameva_get_context_destroy_count(void) { return g_count.ctx_destroy.load(); }
int64_t ggml_backend_ameva_get_kernel_create_count(void) { return g_count.kernel_create.load(); }
int64_t ggml_backend_ameva_get_kernel_destroy_count(void) { return g_count.kernel_destroy.load(); }
int64_t ggml_backend_ameva_get_buffer_create_count(void) { return g_count.buffer_create.load(); }
int64_t ggml_backend_ameva_get_buffer_destroy_count(void) { return g_count.buffer_destroy.load(); }
int64_t ggml_backend_ameva_get_event_create_count(void) { return g_count.event_create.load(); }
int64_t ggml_backend_ameva_get_event_destroy_count(void) { return g_count.event_destroy.load(); }
int64_t ggml_backend_ameva_get_q5_0_staging_alloc_count(void) { return 0; }
int64_t ggml_backend_ameva_get_q5_0_staging_free_count(void) { return 0; }
int64_t ggml_backend_ameva_get_repacked_tensor_count(void) { return g_count.repacked_tensors.load(); }
int64_t ggml_backend_ameva_get_repacked_bytes(void) { return g_count.repacked_bytes.load(); }
int64_t ggml_backend_ameva_get_qmv_mul_mat_count(void) { return g_count.qmv.load(); }
int64_t ggml_backend_ameva_get_mmq_mul_mat_count(void) { return g_count.mmq.load(); }
int64_t ggml_backend_ameva_get_mmqb_mul_mat_count(void) { return g_count.mmqb.load(); }
int64_t ggml_backend_ameva_get_fused_pair_count(void) { return g_count.fused_pairs.load(); }
const char* ggml_backend_ameva_get_build_commit(void) {
#ifdef AMEVA_B200_BUILD_COMMIT
    return AMEVA_B200_BUILD_COMMIT;
#else
    return "unknown";
#endif
}
void ggml_backend_ameva_reset_counters(void) {
    // activity counters only; the repacked tensor and byte counts describe stored weights (ggml-ameva-device.cpp:129-145)
    g_count.supports_query = 0;
    g_count.supported_op = 0;
    g_count.gpu_op = 0;
    g_count.mul_mat = 0;
    g_count.buffer_create = 0;
    g_count.buffer_destroy = 0;
    g_count.event_create = 0;
    g_count.event_destroy = 0;
    g_count.qmv = 0;
    g_count.mmq = 0;
    g_count.mmqb = 0;
    g_count.fused_pairs = 0;
}

void ggml_backend_ameva_set_failure_injection(AmevaFailureInjectionPoint point) { g_fail.store((int)point); }
AmevaFailureInjectionPoint ggml_backend_ameva_get_failure_injection(void) { return (AmevaFailureInjectionPoint)g_fail.load(); }

}  // extern "C"

namespace {
struct ProcEntry {
    const char* name;
    void* fn;
};
void* reg_get_proc_address(ggml_backend_reg_t, const char* name) {
    static const ProcEntry table[] = {
        {"ggml_backend_ameva_get_gpu_op_count", (void*)ggml_backend_ameva_get_gpu_op_count},
        {"ggml_backend_ameva_get_fused_pair_count", (void*)ggml_backend_ameva_get_fused_pair_count},
        {"ggml_backend_ameva_get_qmv_mul_mat_count", (void*)ggml_backend_ameva_get_qmv_mul_mat_count},
        {"ggml_backend_ameva_get_mmq_mul_mat_count", (void*)ggml_backend_ameva_get_mmq_mul_mat_count},
        {"ggml_backend_ameva_get_mmqb_mul_mat_count", (void*)ggml_backend_ameva_get_mmqb_mul_mat_count},
        {"ggml_backend_ameva_get_repacked_tensor_count", (void*)ggml_backend_ameva_get_repacked_tensor_count},
        {"ggml_backend_ameva_get_repacked_bytes", (void*)ggml_backend_ameva_get_repacked_bytes},
        {"ggml_backend_ameva_reset_counters", (void*)ggml_backend_ameva_reset_counters},
        {"ggml_backend_ameva_set_failure_injection", (void*)ggml_backend_ameva_set_failure_injection},
        {"ggml_backend_ameva_get_failure_injection", (void*)ggml_backend_ameva_get_failure_injection},
        {"ggml_backend_ameva_teardown", (void*)ggml_backend_ameva_teardown},
        {"ggml_backend_ameva_abi_check", (void*)ggml_backend_ameva_abi_check},
    };
    if (!name) return nullptr;
    for (const ProcEntry& e : table)
        if (strcmp(e.name, name) == 0) return e.fn;
    return nullptr;
}
}  // namespace
