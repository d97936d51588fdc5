// GGUF files as the source of the mul_mat weights: header, metadata and tensor directory of a memory-mapped file, the
// byte size of every tensor, and the upload of a weight tensor into the device layout. Host code only.
//
// Behaviour follows the reference loader (src/amuda/amuda_gguf.c of uno-km/ameva-compute): limits (:11-16), value
// skipping with a recursion bound (:139-201), tensor sizing with overflow checks and the I2_S trailer (:203-330), the
// parse order and the error code of every failure (:334-647), lookup, scale and close (:649-700). The tensor bytes
// stay in the mapping; ac_b200_gguf_upload_tensor streams them through the device-side repack without a host copy of
// the tensor.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>

#include "../../include/amuda_gguf_b200.h"

namespace {

constexpr uint64_t kMaxPairs = 65536, kMaxTensors = 65536, kMaxString = 65536;
constexpr uint64_t kMaxMetadataBytes = 64ull << 20, kMaxDirectoryBytes = 32ull << 20;
constexpr uint32_t kMaxDepth = 16;

// Little-endian cursor over the mapping; every read checks what is left.
struct Cursor {
    const uint8_t* at;
    const uint8_t* end;
    size_t left() const { return (size_t)(end - at); }
    bool skip(uint64_t n) {
        if (n > left()) return false;
        at += n;
        return true;
    }
    template <typename T>
    bool get(T* v) {
        if (sizeof(T) > left()) return false;
        uint64_t x = 0;
        for (size_t i = 0; i < sizeof(T); ++i) x |= (uint64_t)at[i] << (8 * i);
        *v = (T)x;
        at += sizeof(T);
        return true;
    }
    bool get_f32(float* v) {
        uint32_t u;
        if (!get(&u)) return false;
        memcpy(v, &u, 4);
        return true;
    }
    // a length-prefixed string; what does not fit `cap - 1` bytes is cut, the cursor passes the whole string
    bool get_string(char* dst, size_t cap) {
        uint64_t n;
        if (!get(&n) || n > kMaxString || n > left()) return false;
        if (dst && cap) {
            const size_t c = n < cap - 1 ? (size_t)n : cap - 1;
            memcpy(dst, at, c);
            dst[c] = 0;
        }
        at += n;
        return true;
    }
};

size_t scalar_bytes(uint32_t vtype) {
    switch (vtype) {
        case GGUF_TYPE_UINT8: case GGUF_TYPE_INT8: case GGUF_TYPE_BOOL: return 1;
        case GGUF_TYPE_UINT16: case GGUF_TYPE_INT16: return 2;
        case GGUF_TYPE_UINT32: case GGUF_TYPE_INT32: case GGUF_TYPE_FLOAT32: return 4;
        case GGUF_TYPE_UINT64: case GGUF_TYPE_INT64: case GGUF_TYPE_FLOAT64: return 8;
        default: return 0;
    }
}

bool skip_value(Cursor& c, uint32_t vtype, uint32_t depth) {
    if (depth > kMaxDepth) return false;
    if (const size_t b = scalar_bytes(vtype)) return c.skip(b);
    if (vtype == GGUF_TYPE_STRING) return c.get_string(nullptr, 0);
    if (vtype != GGUF_TYPE_ARRAY) return false;
    uint32_t et;
    uint64_t n;
    if (!c.get(&et) || !c.get(&n)) return false;
    if (const size_t b = scalar_bytes(et)) return n <= SIZE_MAX / b && c.skip(n * b);
    for (uint64_t i = 0; i < n; ++i)
        if (!skip_value(c, et, depth + 1)) return false;
    return true;
}

// a u32 or u64 value into a u32 field; other value types are passed over
bool get_count(Cursor& c, uint32_t vtype, uint32_t* out) {
    if (vtype == GGUF_TYPE_UINT32) return c.get(out);
    if (vtype == GGUF_TYPE_UINT64) {
        uint64_t v;
        if (!c.get(&v)) return false;
        *out = (uint32_t)v;
        return true;
    }
    return skip_value(c, vtype, 0);
}
bool get_real(Cursor& c, uint32_t vtype, float* out) {
    return vtype == GGUF_TYPE_FLOAT32 ? c.get_f32(out) : skip_value(c, vtype, 0);
}

bool mul_ok(uint64_t a, uint64_t b, uint64_t* out) {
    if (a && b > UINT64_MAX / a) return false;
    *out = a * b;
    return true;
}

// elements per block and bytes per block of the ggml types the reference sizes (amuda_gguf.c:217-312)
struct BlockRule {
    uint32_t type, elems, bytes;
};
constexpr BlockRule kRules[] = {
    {0, 1, 4},      {1, 1, 2},      {2, 32, 18},    {3, 32, 20},    {6, 32, 22},     {7, 32, 24},    {8, 32, 34},
    {9, 32, 40},    {10, 256, 84},  {11, 256, 110}, {12, 256, 144}, {13, 256, 176},  {14, 256, 210}, {15, 256, 292},
};
constexpr uint32_t kTypeI2S = 36;

void release(GgufModel* m) {
    if (!m) return;
    free(m->tensors);
    if (m->mmap_addr && m->mmap_size) munmap(m->mmap_addr, m->mmap_size);
    if (m->fd >= 0) close(m->fd);
    free(m);
}

}  // namespace

extern "C" {

AcResult ac_b200_gguf_tensor_size(uint32_t type, const uint64_t* ne, uint32_t n_dims, size_t* out_size) {
    if (!ne || n_dims < 1 || n_dims > 4 || !out_size) return AC_ERR_INVALID_ARGUMENT;
    uint64_t n = 1;
    for (uint32_t i = 0; i < n_dims; ++i)
        if (ne[i] == 0 || !mul_ok(n, ne[i], &n)) return AC_ERR_BINARY_CORRUPTED;
    uint64_t bytes = 0;
    if (type == kTypeI2S) {
        bytes = n / 4 + (n % 4 ? 1 : 0);   // four ternary weights per byte, then the 32-byte trailer with the scale
        if (bytes > UINT64_MAX - 32) return AC_ERR_BINARY_CORRUPTED;
        bytes += 32;
    } else {
        const BlockRule* rule = nullptr;
        for (const BlockRule& r : kRules)
            if (r.type == type) rule = &r;
        if (!rule) return AC_ERR_DEVICE_NOT_SUPPORTED;
        const uint64_t blocks = n / rule->elems + (n % rule->elems ? 1 : 0);
        if (!mul_ok(blocks, rule->bytes, &bytes)) return AC_ERR_BINARY_CORRUPTED;
    }
    if (bytes > SIZE_MAX) return AC_ERR_BINARY_CORRUPTED;
    *out_size = (size_t)bytes;
    return AC_SUCCESS;
}

AcResult ac_gguf_open(const char* file_path, GgufModel** out_model) {
    if (!file_path || !out_model) return AC_ERR_NULL_POINTER;
    *out_model = nullptr;
    const int fd = open(file_path, O_RDONLY);
    if (fd < 0) return AC_ERR_BINARY_CORRUPTED;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return AC_ERR_BINARY_CORRUPTED;
    }
    const size_t file_size = (size_t)st.st_size;
    void* map = mmap(nullptr, file_size, PROT_READ, MAP_SHARED, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return AC_ERR_OUT_OF_HOST_MEMORY;
    }
    GgufModel* m = (GgufModel*)calloc(1, sizeof(GgufModel));
    if (!m) {
        munmap(map, file_size);
        close(fd);
        return AC_ERR_OUT_OF_HOST_MEMORY;
    }
    m->fd = fd;
    m->mmap_addr = map;
    m->mmap_size = file_size;
    const uint8_t* base = (const uint8_t*)map;
    Cursor c{base, base + file_size};
    auto bail = [&](AcResult rc) {
        release(m);
        return rc;
    };

    uint32_t magic = 0;
    if (!c.get(&magic) || magic != GGUF_MAGIC) return bail(AC_ERR_BINARY_CORRUPTED);
    if (!c.get(&m->version) || (m->version != 2 && m->version != 3)) return bail(AC_ERR_DEVICE_NOT_SUPPORTED);
    if (!c.get(&m->tensor_count) || m->tensor_count > kMaxTensors) return bail(AC_ERR_BINARY_CORRUPTED);
    if (!c.get(&m->metadata_kv_count) || m->metadata_kv_count > kMaxPairs) return bail(AC_ERR_BINARY_CORRUPTED);

    uint64_t alignment = 32;
    GgufModelConfig& cfg = m->config;
    for (uint64_t i = 0; i < m->metadata_kv_count; ++i) {
        if ((size_t)(c.at - base) > kMaxMetadataBytes) return bail(AC_ERR_BINARY_CORRUPTED);
        char key[128] = {0};
        uint32_t vtype = 0;
        if (!c.get_string(key, sizeof(key)) || !c.get(&vtype)) return bail(AC_ERR_BINARY_CORRUPTED);
        bool ok;
        const size_t alen = strlen(cfg.arch);
        const char* sub = (alen && strncmp(key, cfg.arch, alen) == 0 && key[alen] == '.') ? key + alen + 1 : nullptr;
        if (strcmp(key, "general.architecture") == 0 && vtype == GGUF_TYPE_STRING) {
            ok = c.get_string(cfg.arch, sizeof(cfg.arch));
        } else if (strcmp(key, "general.alignment") == 0) {
            if (vtype == GGUF_TYPE_UINT32) {
                uint32_t a = 0;
                ok = c.get(&a);
                alignment = a;
            } else if (vtype == GGUF_TYPE_UINT64) {
                ok = c.get(&alignment);
            } else {
                ok = skip_value(c, vtype, 0);
            }
            if (ok && (alignment == 0 || (alignment & (alignment - 1)) || alignment > (1ull << 30))) ok = false;
        } else if (!sub) {
            ok = skip_value(c, vtype, 0);
        } else if (strcmp(sub, "context_length") == 0) {
            ok = get_count(c, vtype, &cfg.context_length);
        } else if (strcmp(sub, "embedding_length") == 0) {
            ok = get_count(c, vtype, &cfg.embedding_length);
        } else if (strcmp(sub, "block_count") == 0) {
            ok = get_count(c, vtype, &cfg.block_count);
        } else if (strcmp(sub, "feed_forward_length") == 0) {
            ok = get_count(c, vtype, &cfg.feed_forward_length);
        } else if (strcmp(sub, "attention.head_count") == 0) {
            ok = get_count(c, vtype, &cfg.head_count);
        } else if (strcmp(sub, "attention.head_count_kv") == 0) {
            ok = get_count(c, vtype, &cfg.head_count_kv);
        } else if (strcmp(sub, "attention.layer_norm_rms_epsilon") == 0) {
            ok = get_real(c, vtype, &cfg.rms_norm_eps);
        } else if (strcmp(sub, "rope.freq_base") == 0) {
            ok = get_real(c, vtype, &cfg.rope_freq_base);
        } else if (strcmp(sub, "vocab_size") == 0) {
            ok = get_count(c, vtype, &cfg.vocab_size);
        } else {
            ok = skip_value(c, vtype, 0);
        }
        if (!ok) return bail(AC_ERR_BINARY_CORRUPTED);
    }

    if (m->tensor_count) {
        if (m->tensor_count * sizeof(GgufTensor) > kMaxDirectoryBytes) return bail(AC_ERR_BINARY_CORRUPTED);
        m->tensors = (GgufTensor*)calloc(m->tensor_count, sizeof(GgufTensor));
        if (!m->tensors) return bail(AC_ERR_OUT_OF_HOST_MEMORY);
    }
    for (uint64_t i = 0; i < m->tensor_count; ++i) {
        GgufTensor& t = m->tensors[i];
        if (!c.get_string(t.name, sizeof(t.name)) || !c.get(&t.n_dims) || t.n_dims < 1 || t.n_dims > 4)
            return bail(AC_ERR_BINARY_CORRUPTED);
        for (uint32_t d = 0; d < t.n_dims; ++d)
            if (!c.get(&t.ne[d]) || t.ne[d] == 0) return bail(AC_ERR_BINARY_CORRUPTED);
        if (!c.get(&t.type) || !c.get(&t.offset)) return bail(AC_ERR_BINARY_CORRUPTED);
        const AcResult rc = ac_b200_gguf_tensor_size(t.type, t.ne, t.n_dims, &t.size_bytes);
        if (rc != AC_SUCCESS) return bail(rc);
    }
    if (m->tensor_count) {
        // the tensor data starts at the next multiple of the alignment; every tensor must lie inside the file
        const uint64_t here = (uint64_t)(c.at - base), rem = here % alignment;
        const uint64_t data0 = rem ? here + (alignment - rem) : here;
        if (data0 > file_size) return bail(AC_ERR_BINARY_CORRUPTED);
        const uint64_t avail = file_size - data0;
        for (uint64_t i = 0; i < m->tensor_count; ++i) {
            GgufTensor& t = m->tensors[i];
            if (t.offset > avail || t.size_bytes > avail - t.offset) return bail(AC_ERR_BINARY_CORRUPTED);
            t.data_ptr = (void*)(base + data0 + t.offset);
        }
    }
    *out_model = m;
    return AC_SUCCESS;
}

GgufTensor* ac_gguf_get_tensor(GgufModel* model, const char* tensor_name) {
    if (!model || !tensor_name || !model->tensors) return nullptr;
    for (uint64_t i = 0; i < model->tensor_count; ++i)
        if (strcmp(model->tensors[i].name, tensor_name) == 0) return &model->tensors[i];
    return nullptr;
}

AcResult ac_gguf_get_tensor_scale(const GgufTensor* tensor, float* out_scale) {
    if (!tensor || !out_scale) return AC_ERR_NULL_POINTER;
    if (tensor->type == 0u || tensor->type == 1u) {
        *out_scale = 1.0f;
        return AC_SUCCESS;
    }
    if (tensor->type != kTypeI2S) return AC_ERR_DEVICE_NOT_SUPPORTED;
    if (!tensor->data_ptr) return AC_ERR_BINARY_CORRUPTED;
    uint64_t n = 0;
    if (!mul_ok(tensor->ne[0], tensor->n_dims > 1 ? tensor->ne[1] : 1, &n)) return AC_ERR_BINARY_CORRUPTED;
    const uint64_t packed = n / 4;   // the scale sits directly behind the payload of the first two dimensions
    if (packed > tensor->size_bytes || tensor->size_bytes - packed < sizeof(float)) return AC_ERR_BINARY_CORRUPTED;
    memcpy(out_scale, (const uint8_t*)tensor->data_ptr + packed, sizeof(float));
    return AC_SUCCESS;
}

void ac_gguf_close(GgufModel* model) { release(model); }

AcResult ac_b200_gguf_device_size(const GgufTensor* tensor, size_t* out_size) {
    if (!tensor || !out_size) return AC_ERR_NULL_POINTER;
    if (tensor->n_dims != 2) return AC_ERR_INVALID_SHAPE;
    uint64_t total = 0, s_off = 0;
    const AcResult rc = ac_b200_device_layout(tensor->type, tensor->ne[1], tensor->ne[0], &total, &s_off);
    if (rc != AC_SUCCESS) return rc;
    *out_size = (size_t)total;
    return AC_SUCCESS;
}

AcResult ac_b200_gguf_upload_tensor(AcContext* ctx, GgufTensor* tensor, AcBuffer** out_buf) {
    if (!out_buf) return AC_ERR_NULL_POINTER;
    *out_buf = nullptr;
    if (!tensor) return AC_ERR_NULL_POINTER;
    if (!tensor->data_ptr) return AC_ERR_BINARY_CORRUPTED;
    size_t total = 0;
    AcResult rc = ac_b200_gguf_device_size(tensor, &total);
    if (rc != AC_SUCCESS) return rc;
    AcBufferDesc desc;
    memset(&desc, 0, sizeof(desc));
    desc.abi_version = AC_ABI_VERSION;
    desc.struct_size = sizeof(desc);
    desc.size_bytes = total;
    desc.usage = AC_BUFFER_USAGE_STORAGE | AC_BUFFER_USAGE_TRANSFER_SRC | AC_BUFFER_USAGE_TRANSFER_DST;
    AcBuffer* buf = nullptr;
    rc = ac_runtime_buffer_create(ctx, &desc, &buf);
    if (rc != AC_SUCCESS) return rc;
    rc = ac_b200_weight_upload(buf, 0, tensor->type, tensor->data_ptr, tensor->ne[1], tensor->ne[0]);
    if (rc != AC_SUCCESS) {
        ac_runtime_buffer_destroy(buf);
        return rc;
    }
    tensor->ac_buf = buf;
    *out_buf = buf;
    return AC_SUCCESS;
}

}  // extern "C"
