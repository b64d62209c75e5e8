/*
 * cann_ops_tensor_types.h - status codes, enumerations and opaque handle types of the ops-tensor host API.
 *
 * Every name and numeric value that exists in the reference header (include/cann_ops_tensor_types.h:24-132 of
 * Atlas-Ascend-Fork/ops-tensor) is kept, so code compiled against the reference links and runs unchanged.  The
 * additions (marked "B200 addition") are the data types, attributes and enumerations the quantized-contraction
 * path needs; they use values the reference does not assign.
 */
#ifndef CANN_OPS_TENSOR_TYPES_H
#define CANN_OPS_TENSOR_TYPES_H

#include <stdint.h>

/* Status codes (reference :24-36). */
typedef enum {
    ACLTENSOR_STATUS_SUCCESS = 0,
    ACLTENSOR_STATUS_NOT_INITIALIZED = 1,
    ACLTENSOR_STATUS_ALLOC_FAILED = 3,
    ACLTENSOR_STATUS_INVALID_VALUE = 7,
    ACLTENSOR_STATUS_ARCH_MISMATCH = 8,
    ACLTENSOR_STATUS_EXECUTION_FAILED = 13,
    ACLTENSOR_STATUS_INTERNAL_ERROR = 14,
    ACLTENSOR_STATUS_NOT_SUPPORTED = 15,
    ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE = 19,
    ACLTENSOR_STATUS_INSUFFICIENT_DRIVER = 20,
    ACLTENSOR_STATUS_IO_ERROR = 21,
} acltensorStatus_t;

/* Element types (reference :41-52). */
typedef enum {
    ACLTENSOR_R_16F = 0,
    ACLTENSOR_R_32F = 1,
    ACLTENSOR_R_64F = 2,
    ACLTENSOR_R_16BF = 3,
    ACLTENSOR_R_8I = 4,
    ACLTENSOR_R_8U = 5,
    ACLTENSOR_R_32I = 6,
    ACLTENSOR_R_32U = 7,
    ACLTENSOR_C_32F = 8,
    ACLTENSOR_C_64F = 9,
    /* B200 additions: narrow floating-point operand and scale types of the quantized matmul path.  The reference
     * uses the same formats on the device side only (fp8_e4m3fn_t, fp4x2_e2m1_t, fp8_e8m0_t:
     * include/tensor_api/impl/tensor_api/arch/utils/check_data_type.h:33-53). */
    ACLTENSOR_R_8F_E4M3 = 32,
    ACLTENSOR_R_8F_E5M2 = 33,
    ACLTENSOR_R_4F_E2M1 = 34,  /* two elements per byte, low nibble first; extents count elements */
    ACLTENSOR_R_8F_UE8M0 = 35, /* power-of-two scale, value 2^(byte-127) */
    ACLTENSOR_R_64I = 36,      /* group lists */
} acltensorDataType_t;

/* Compute precision (reference :57-65). */
typedef enum {
    ACLTENSOR_COMPUTE_DESC_32F = (1U << 2),
    ACLTENSOR_COMPUTE_DESC_NONE = 0,
    ACLTENSOR_COMPUTE_DESC_16F = (1U << 0),
    ACLTENSOR_COMPUTE_DESC_64F = (1U << 4),
    ACLTENSOR_COMPUTE_DESC_16BF = (1U << 10),
    ACLTENSOR_COMPUTE_DESC_C32F = (1U << 11),
    ACLTENSOR_COMPUTE_DESC_C64F = (1U << 12),
} acltensorComputeDescriptor_t;

/* Operators (reference :70-107). */
typedef enum {
    ACLTENSOR_OP_IDENTITY = 1,
    ACLTENSOR_OP_SQRT = 2,
    ACLTENSOR_OP_ADD = 3,
    ACLTENSOR_OP_MUL = 5,
    ACLTENSOR_OP_MAX = 6,
    ACLTENSOR_OP_MIN = 7,
    ACLTENSOR_OP_RELU = 8,
    ACLTENSOR_OP_CONJ = 9,
    ACLTENSOR_OP_RCP = 10,
    ACLTENSOR_OP_SIGMOID = 11,
    ACLTENSOR_OP_TANH = 12,
    ACLTENSOR_OP_EXP = 22,
    ACLTENSOR_OP_LOG = 23,
    ACLTENSOR_OP_ABS = 24,
    ACLTENSOR_OP_NEG = 25,
    ACLTENSOR_OP_SIN = 26,
    ACLTENSOR_OP_COS = 27,
    ACLTENSOR_OP_TAN = 28,
    ACLTENSOR_OP_SINH = 29,
    ACLTENSOR_OP_COSH = 30,
    ACLTENSOR_OP_ASIN = 31,
    ACLTENSOR_OP_ACOS = 32,
    ACLTENSOR_OP_ATAN = 33,
    ACLTENSOR_OP_CEIL = 37,
    ACLTENSOR_OP_FLOOR = 38,
    ACLTENSOR_OP_GELU = 39, /* in a contraction epilogue: the tanh form */
    ACLTENSOR_OP_SILU = 40,
    ACLTENSOR_OP_SUB = 50,
    ACLTENSOR_OP_DIV = 51,
    ACLTENSOR_OP_POW = 52,
    ACLTENSOR_OP_UNKNOWN = 126,
} acltensorOperator_t;

/* Algorithm selection (reference :111-114). */
typedef enum {
    ACLTENSOR_ALGO_DEFAULT = -1,
    ACLTENSOR_ALGO_DEFAULT_PATIENT = -6,
} acltensorAlgo_t;

/* Workspace preference (reference :119-123). */
typedef enum {
    ACLTENSOR_WORKSPACE_MIN = 1,
    ACLTENSOR_WORKSPACE_DEFAULT = 2,
    ACLTENSOR_WORKSPACE_MAX = 3,
} acltensorWorksizePreference_t;

/* B200 addition: how an operand of a contraction is scaled. */
typedef enum {
    ACLTENSOR_SCALE_NONE = 0,
    ACLTENSOR_SCALE_MX_E8M0_VEC32 = 1, /* one E8M0 byte per 32 K, rows of ceil(K/64)*2 bytes */
    ACLTENSOR_SCALE_FP32_1X128 = 2,    /* one float per 128 K of each row */
    ACLTENSOR_SCALE_FP32_128X128 = 3,  /* one float per 128(K) x 128(N) block, indexed [k_block][n_block] */
    ACLTENSOR_SCALE_PER_TENSOR = 4,    /* INT8: one float32 for the whole operand (QuantMode PERTENSOR,
                                          include/blaze/gemm/utils/common_utils.h:98-107) */
    ACLTENSOR_SCALE_PER_CHANNEL = 5,   /* INT8 B: one 64-bit word per output column, float32 bits in the low word
                                          (QuantMode PERCHANNEL; the scale array of kernel_qbmm_cube.h:190-192) */
} acltensorScaleMode_t;

/* B200 addition: tile scheduling hint of a contraction. */
typedef enum {
    ACLTENSOR_SPLIT_AUTO = 0,
    ACLTENSOR_SPLIT_DATA_PARALLEL = 1,
    ACLTENSOR_SPLIT_STREAM_K = 2,
} acltensorSplitPolicy_t;

/* B200 addition: attributes of an operation descriptor (acltensorOperationDescriptorSetAttribute).  The entry
 * points are reserved by the reference's roadmap (lib/core/operation_descriptor.cpp:183-189). */
typedef enum {
    ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_A = 1,     /* int32: acltensorScaleMode_t */
    ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_B = 2,     /* int32 */
    ACLTENSOR_OPERATION_DESCRIPTOR_EPILOGUE_ACT = 3,     /* int32: ACLTENSOR_OP_IDENTITY / RELU / GELU / SILU / SIGMOID / TANH */
    ACLTENSOR_OPERATION_DESCRIPTOR_BIAS_TYPE = 4,        /* int32: acltensorDataType_t of the bias (16BF) or -1 for none */
    ACLTENSOR_OPERATION_DESCRIPTOR_GROUP_COUNT = 5,      /* int32: number of groups (0 = dense) */
    ACLTENSOR_OPERATION_DESCRIPTOR_SPLIT_POLICY = 6,     /* int32: acltensorSplitPolicy_t */
    ACLTENSOR_OPERATION_DESCRIPTOR_TILE_N = 7,           /* int32: 0 = heuristic */
    ACLTENSOR_OPERATION_DESCRIPTOR_SM_LIMIT = 8,         /* int32: 0 = all SMs */
    ACLTENSOR_OPERATION_DESCRIPTOR_B_IS_STATIC = 9,      /* int32: 1 = B and its scales do not change between calls,
                                                            so weight pre-passes kept in the workspace are reused
                                                            while this plan was the last one to use that workspace
                                                            (another plan's call on the same buffer re-runs them) */
    ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_D = 12,    /* acltensorScaleMode_t of a quantised D (dtype R_8F_E4M3): must equal SCALE_MODE_A; scales go to aux->scaleD */
    ACLTENSOR_OPERATION_DESCRIPTOR_BIAS_PER_BATCH = 11,  /* int32: 1 = bias is [batches][N] (batched contraction) */
    ACLTENSOR_OPERATION_DESCRIPTOR_CTA_PAIR = 10,        /* int32: 0 = heuristic, 1 = single-CTA tiles, 2 = 2-CTA 256-row tiles */
} acltensorOperationDescriptorAttribute_t;

/* Opaque handles (reference :128-132). */
typedef struct acltensorHandle* acltensorHandle_t;
typedef struct acltensorTensorDescriptor* acltensorTensorDescriptor_t;
typedef struct acltensorOperationDescriptor* acltensorOperationDescriptor_t;
typedef struct acltensorPlanPreference* acltensorPlanPreference_t;
typedef struct acltensorPlan* acltensorPlan_t;

#endif /* CANN_OPS_TENSOR_TYPES_H */
