/* GGUF model files as the source of the mul_mat weights: tensor directory, tensor sizing and upload.
 *
 * Mirrors the reference's loader interface (include/amuda_gguf.h:19-112 of uno-km/ameva-compute, implementation
 * src/amuda/amuda_gguf.c): the same four function names, the same struct layouts and the same error codes, so a host
 * written against the reference binds unchanged. Exported by libac_runtime_b200.so.
 *
 * Sizing rules kept from the reference (amuda_gguf.c:203-330): a tensor has 1..4 non-zero dimensions whose product must
 * not overflow 64 bits; block types take ceil(n / block) * block_bytes; I2_S (BitNet ternary, type 36) takes
 * ceil(n / 4) payload bytes plus a 32-byte trailer whose first four bytes are the tensor's fp32 scale; an unknown type
 * is AC_ERR_DEVICE_NOT_SUPPORTED, any overflow AC_ERR_BINARY_CORRUPTED. */
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "ac_runtime_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GGUF_MAGIC 0x46554747u /* "GGUF", little endian */

typedef enum {
    GGUF_TYPE_UINT8 = 0,
    GGUF_TYPE_INT8 = 1,
    GGUF_TYPE_UINT16 = 2,
    GGUF_TYPE_INT16 = 3,
    GGUF_TYPE_UINT32 = 4,
    GGUF_TYPE_INT32 = 5,
    GGUF_TYPE_FLOAT32 = 6,
    GGUF_TYPE_BOOL = 7,
    GGUF_TYPE_STRING = 8,
    GGUF_TYPE_ARRAY = 9,
    GGUF_TYPE_UINT64 = 10,
    GGUF_TYPE_INT64 = 11,
    GGUF_TYPE_FLOAT64 = 12,
} GgufType;

/* One entry of the tensor directory (amuda_gguf.h:58-67). data_ptr points into the mapping of the file. */
typedef struct {
    char name[64];
    uint32_t n_dims;
    uint64_t ne[4];
    uint32_t type; /* ggml type number */
    uint64_t offset;
    void* data_ptr;
    size_t size_bytes;
    struct AcBuffer* ac_buf; /* device copy made by ac_b200_gguf_upload_tensor, NULL before; owned by the caller */
} GgufTensor;

/* The metadata keys "<arch>.<key>" the reference reads (amuda_gguf.h:69-80). */
typedef struct {
    char arch[32];
    uint32_t context_length;
    uint32_t embedding_length;
    uint32_t block_count;
    uint32_t feed_forward_length;
    uint32_t head_count;
    uint32_t head_count_kv;
    float rms_norm_eps;
    float rope_freq_base;
    uint32_t vocab_size;
} GgufModelConfig;

typedef struct {
    void* mmap_addr;
    size_t mmap_size;
    int fd;
    uint32_t version;
    uint64_t tensor_count;
    uint64_t metadata_kv_count;
    GgufModelConfig config;
    GgufTensor* tensors;
} GgufModel;

/* Maps the file read-only and parses header, metadata and tensor directory (amuda_gguf.c:334-647). Versions 2 and 3;
 * at most 65536 tensors and 65536 metadata pairs; strings up to 65536 bytes; general.alignment a power of two up to
 * 2^30 (default 32); every tensor must lie inside the file. *out_model is NULL on failure. */
AcResult ac_gguf_open(const char* file_path, GgufModel** out_model);

/* Exact-name lookup, NULL when absent (amuda_gguf.c:649-657). */
GgufTensor* ac_gguf_get_tensor(GgufModel* model, const char* tensor_name);

/* I2_S: the fp32 scale stored behind the packed payload; F32 / F16: 1.0; other types AC_ERR_DEVICE_NOT_SUPPORTED
 * (amuda_gguf.c:659-681). */
AcResult ac_gguf_get_tensor_scale(const GgufTensor* tensor, float* out_scale);

void ac_gguf_close(GgufModel* model);

/* The sizing rule on its own (static in the reference, amuda_gguf.c:203-330). */
AcResult ac_b200_gguf_tensor_size(uint32_t type, const uint64_t* ne, uint32_t n_dims, size_t* out_size);

/* Bytes of the device ("regions") layout of a 2-D weight of a type the mul_mat kernels take (Q4_0, Q8_0, Q4_K, I2_S);
 * AC_ERR_DEVICE_NOT_SUPPORTED for other types, AC_ERR_INVALID_SHAPE when ne[0] is not a multiple of the type's block. */
AcResult ac_b200_gguf_device_size(const GgufTensor* tensor, size_t* out_size);

/* Creates a device buffer of that size in `ctx`, streams the tensor's blocks from the mapping through the device-side
 * repack (ac_b200_weight_upload) and stores the buffer in tensor->ac_buf and *out_buf. The scale of an I2_S tensor is
 * read with ac_gguf_get_tensor_scale by the caller. The buffer belongs to the caller (ac_runtime_buffer_destroy). */
AcResult ac_b200_gguf_upload_tensor(AcContext* ctx, GgufTensor* tensor, AcBuffer** out_buf);

#ifdef __cplusplus
}
#endif
