/* Public helper surface of the ggml backend plugin libggml-ameva-b200.so.
 *
 * Mirrors the reference plugin's header (adapters/llama/ggml-ameva/ggml-ameva.h:19-98 of uno-km/ameva-compute): the
 * same function names, so a host or test written against the reference finds them here, with the meanings below.
 * Include after ggml.h and ggml-backend.h of the application the plugin is loaded into. */
#pragma once

#include "ggml-backend.h"
#include "ggml.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GGML_AMEVA_B200_NAME "AMEVA_B200"
#define GGML_AMEVA_B200_DEVICE_NAME "AMEVA_B200_0"

/* Backend and device lifecycle (ggml-ameva.h:19-25). dev_num must be 0. */
GGML_API ggml_backend_t ggml_backend_ameva_init(size_t dev_num);
GGML_API bool ggml_backend_is_ameva(ggml_backend_t backend);
GGML_API ggml_backend_buffer_type_t ggml_backend_ameva_buffer_type(size_t dev_num);
GGML_API ggml_backend_reg_t ggml_backend_ameva_reg(void);
GGML_API void ggml_backend_ameva_register(void);   /* after the ABI self-check; prints why when it does not register */
GGML_API void ggml_backend_ameva_teardown(void);   /* destroys the runtime context once no backend or buffer is left */

/* Loader entry points (ggml-ameva.h:27-29). */
GGML_BACKEND_API ggml_backend_reg_t ggml_backend_init(void);
GGML_BACKEND_API int ggml_backend_score(void);

/* NULL when the ggml the process runs agrees with the headers the plugin was compiled against on every struct layout
 * and enum value the plugin relies on, else a message (ameva_abi_check, ggml-ameva-device.cpp:415-495). */
GGML_API const char* ggml_backend_ameva_abi_check(void);

/* Counters: the reference's tests use them as ground truth for what ran where (ggml-ameva.h:31-80). Monotonic;
 * reset_counters clears the activity counters and leaves the stored-state ones (repacked tensors / bytes).
 *   supports_query / supported_op   calls of supports_op and how many answered yes
 *   gpu_op                          graph nodes completed on the GPU (any op; views are not counted)
 *   f32_gpu_sgemm_dispatch          MUL_MAT nodes completed on the GPU, whatever the weight type (name kept)
 *   q5_0_cpu_dequant, q5_0_staging_alloc / free   stay 0: nothing is dequantized or staged on the CPU (names kept)
 *   qmv_mul_mat                     MUL_MAT nodes completed with weights in the device layout (all of them here)
 *   mmq_mul_mat                     of those, the ones on integer dot products over int8 activations (dp4a / mma.sync)
 *   mmqb_mul_mat                    of those, the ones with one activation scale per 256 (Q4_K x Q8_K)
 *   fused_pair                      nodes computed by the launch of an earlier node: the consumer of a fused MUL_MAT +
 *                                   ADD / SWIGLU or RMS_NORM + MUL pair counts 1, every projection after the first of
 *                                   a grouped q/k/v or gate/up launch counts 1
 *   context / kernel / buffer / event create and destroy   runtime objects made and released by the plugin */
GGML_API int64_t ggml_backend_ameva_get_supports_query_count(void);
GGML_API int64_t ggml_backend_ameva_get_supported_op_count(void);
GGML_API int64_t ggml_backend_ameva_get_gpu_op_count(void);
GGML_API int64_t ggml_backend_ameva_get_q5_0_cpu_dequant_count(void);
GGML_API int64_t ggml_backend_ameva_get_f32_gpu_sgemm_dispatch_count(void);
GGML_API int64_t ggml_backend_ameva_get_context_create_count(void);
GGML_API int64_t ggml_backend_ameva_get_context_destroy_count(void);
GGML_API int64_t ggml_backend_ameva_get_kernel_create_count(void);
GGML_API int64_t ggml_backend_ameva_get_kernel_destroy_count(void);
GGML_API int64_t ggml_backend_ameva_get_buffer_create_count(void);
GGML_API int64_t ggml_backend_ameva_get_buffer_destroy_count(void);
GGML_API int64_t ggml_backend_ameva_get_event_create_count(void);
GGML_API int64_t ggml_backend_ameva_get_event_destroy_count(void);
GGML_API int64_t ggml_backend_ameva_get_q5_0_staging_alloc_count(void);
GGML_API int64_t ggml_backend_ameva_get_q5_0_staging_free_count(void);
GGML_API int64_t ggml_backend_ameva_get_repacked_tensor_count(void);
GGML_API int64_t ggml_backend_ameva_get_repacked_bytes(void);
GGML_API int64_t ggml_backend_ameva_get_qmv_mul_mat_count(void);
GGML_API int64_t ggml_backend_ameva_get_mmq_mul_mat_count(void);
GGML_API int64_t ggml_backend_ameva_get_mmqb_mul_mat_count(void);
GGML_API int64_t ggml_backend_ameva_get_fused_pair_count(void);
GGML_API const char* ggml_backend_ameva_get_build_commit(void);
GGML_API void ggml_backend_ameva_reset_counters(void);

/* Failure injection on the HOST side of graph_compute (ggml-ameva.h:83-98): with a point set, the next graph_compute
 * calls return GGML_STATUS_FAILED at that point and gpu_op_count does not move. No GPU fault is involved: the binding
 * points fail before anything is recorded, DISPATCH discards the recorded batch, WAIT_TIMEOUT waits with a 1 ns limit
 * (then lets the work finish before returning), INVALIDATE_DST fails after completion. Stays set until set to NONE. */
typedef enum {
    AMEVA_FAIL_NONE = 0,
    AMEVA_FAIL_MAP_SRC0 = 1,
    AMEVA_FAIL_MAP_SRC1 = 2,
    AMEVA_FAIL_MAP_DST = 3,
    AMEVA_FAIL_FLUSH_SRC0 = 4,
    AMEVA_FAIL_FLUSH_SRC1 = 5,
    AMEVA_FAIL_DISPATCH = 6,
    AMEVA_FAIL_WAIT_TIMEOUT = 7,
    AMEVA_FAIL_INVALIDATE_DST = 8,
    AMEVA_FAIL_OFFSET_OVERFLOW = 9,
    AMEVA_FAIL_TENSOR_RANGE_OOB = 10,
} AmevaFailureInjectionPoint;

GGML_API void ggml_backend_ameva_set_failure_injection(AmevaFailureInjectionPoint point);
GGML_API AmevaFailureInjectionPoint ggml_backend_ameva_get_failure_injection(void);

#ifdef __cplusplus
}
#endif
