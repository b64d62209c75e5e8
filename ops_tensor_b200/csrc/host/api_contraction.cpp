// Quantized contraction: descriptor creation, attributes, workspace estimation, plan completion, execution, and
// the two registered solutions (MX block-scaled and FP8 with float32 group/block scales) that forward to the
// kernel C-ABI in launch.cu.
//
// The entry-point names are the ones the reference reserves (lib/core/operation_descriptor.cpp:183-189,
// lib/core/plan_preference.cpp:58, docs/implementation.md:57-74); argument checking follows the conventions of its
// implemented entry points: NULL required argument -> INVALID_VALUE, anything the build cannot do -> NOT_SUPPORTED.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "blaze_b200.h"
#include "cann_ops_tensor.h"
#include "objects.hpp"
#include "registry.hpp"

using namespace acltensor;

namespace {

int find_mode(const std::vector<int32_t>& modes, int32_t label) {
    for (size_t i = 0; i < modes.size(); ++i)
        if (modes[i] == label) return static_cast<int>(i);
    return -1;
}

int activation_of(int32_t op) {
    switch (op) {
        case ACLTENSOR_OP_IDENTITY: return BLAZE_ACT_IDENTITY;
        case ACLTENSOR_OP_RELU: return BLAZE_ACT_RELU;
        case ACLTENSOR_OP_GELU: return BLAZE_ACT_GELU_TANH;
        case ACLTENSOR_OP_SILU: return BLAZE_ACT_SILU;
        case ACLTENSOR_OP_SIGMOID: return BLAZE_ACT_SIGMOID;
        case ACLTENSOR_OP_TANH: return BLAZE_ACT_TANH;
        default: return -1;
    }
}

int out_type_of(acltensorDataType_t t) {
    switch (t) {
        case ACLTENSOR_R_16F: return BLAZE_OUT_F16;
        case ACLTENSOR_R_32F: return BLAZE_OUT_F32;
        case ACLTENSOR_R_8F_E4M3: return BLAZE_OUT_MX_E4M3;
        default: return BLAZE_OUT_BF16;
    }
}

int sched_of(int32_t policy) {
    switch (policy) {
        case ACLTENSOR_SPLIT_DATA_PARALLEL: return BLAZE_SCHED_DATA_PARALLEL;
        case ACLTENSOR_SPLIT_STREAM_K: return BLAZE_SCHED_STREAM_K;
        default: return BLAZE_SCHED_AUTO;
    }
}

bool fits_int32(int64_t v) { return v >= 0 && v <= 0x7fffffffLL; }

// ---- MX solution ---------------------------------------------------------------------------------------------

void fill_mx_args(const acltensorOperationDescriptor& op, blazeMxGemmArgs* a) {
    std::memset(a, 0, sizeof(*a));
    a->struct_size = sizeof(*a);
    a->M = static_cast<int32_t>(op.M);
    a->N = static_cast<int32_t>(op.N);
    a->K = static_cast<int32_t>(op.K);
    auto elem_of = [](acltensorDataType_t t) {
        return t == ACLTENSOR_R_4F_E2M1 ? BLAZE_ELEM_E2M1 : (t == ACLTENSOR_R_8F_E5M2 ? BLAZE_ELEM_E5M2 : BLAZE_ELEM_E4M3);
    };
    a->b_elem = elem_of(op.descB->dataType);
    a->a_elem = elem_of(op.descA->dataType);
    a->lda = a->a_elem == BLAZE_ELEM_E2M1 ? op.lda / 2 : op.lda;      // bytes
    a->ldb = a->b_elem == BLAZE_ELEM_E2M1 ? op.ldb / 2 : op.ldb;      // bytes
    a->ldr = op.ldc;
    a->ldd = op.ldd;
    a->activation = activation_of(op.epilogueAct);
    a->d_type = out_type_of(op.descD->dataType);
    a->b_layout = op.bNMajor ? BLAZE_B_N_MAJOR : BLAZE_B_K_MAJOR;
    a->tile_n = op.tileN;
    a->sm_limit = op.smLimit;
    a->cta_pair = op.ctaPair;
}

void fill_batch(const acltensorOperationDescriptor& op, blazeBatchDims* b) {
    std::memset(b, 0, sizeof(*b));
    for (int i = 0; i < 4; ++i) {
        b->c[i] = op.batchC[i];
        b->a[i] = op.batchA[i];
        b->b[i] = op.batchB[i];
    }
    b->bias_per_batch = op.biasPerBatch;
}

acltensorStatus_t MxWorkspace(const acltensorOperationDescriptor& op, int32_t splitPolicy, uint64_t* bytes) {
    blazeMxGemmArgs a;
    fill_mx_args(op, &a);
    a.sched = sched_of(splitPolicy);
    size_t n = 0;
    blazeBatchDims bd;
    fill_batch(op, &bd);
    const int st = op.batchModes > 0 ? blazeMxGemmBatchedWorkspaceSize(&a, &bd, &n) : blazeMxGemmWorkspaceSize(&a, &n);
    *bytes = n;
    return static_cast<acltensorStatus_t>(st);
}

acltensorStatus_t MxExecute(const ContractionArgs& c) {
    blazeMxGemmArgs a;
    fill_mx_args(*c.op, &a);
    a.sched = sched_of(c.splitPolicy);
    a.A = c.A;
    a.B = c.B;
    a.scaleA = c.scaleA;
    a.scaleB = c.scaleB;
    a.bias = c.bias;
    a.residual = c.C;
    a.D = c.D;
    a.scaleD = c.scaleD;
    a.reuse_b_prepass = c.reuseBPrepass ? 1 : 0;
    a.workspace = c.workspace;
    a.workspace_bytes = c.workspaceSize;
    if (c.op->batchModes > 0) {
        blazeBatchDims bd;
        fill_batch(*c.op, &bd);
        return static_cast<acltensorStatus_t>(blazeMxGemmBatched(&a, &bd, c.stream));
    }
    return static_cast<acltensorStatus_t>(blazeMxGemm(&a, c.stream));
}

// ---- FP8 solution --------------------------------------------------------------------------------------------

void fill_fp8_args(const acltensorOperationDescriptor& op, int32_t splitPolicy, blazeFp8GemmArgs* a) {
    std::memset(a, 0, sizeof(*a));
    a->struct_size = sizeof(*a);
    a->M = static_cast<int32_t>(op.M);
    a->N = static_cast<int32_t>(op.N);
    a->K = static_cast<int32_t>(op.K);
    a->groups = op.groupCount;
    a->lda = op.lda;
    a->ldb = op.ldb;
    a->ldr = op.ldc;
    a->ldd = op.ldd;
    a->activation = activation_of(op.epilogueAct);
    a->d_type = op.descD->dataType == ACLTENSOR_R_8F_E4M3 ? BLAZE_OUT_FP8_128 : out_type_of(op.descD->dataType);
    a->sched = sched_of(splitPolicy);
    a->sm_limit = op.smLimit;
    a->b_is_static = op.bIsStatic != 0 ? 1 : 0;
}

acltensorStatus_t Fp8Workspace(const acltensorOperationDescriptor& op, int32_t splitPolicy, uint64_t* bytes) {
    if (op.batchModes > 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;          // batch broadcast is an MX feature
    if (op.bNMajor) return ACLTENSOR_STATUS_NOT_SUPPORTED;                 // so is the N-major weight
    blazeFp8GemmArgs a;
    fill_fp8_args(op, splitPolicy, &a);
    size_t n = 0;
    const int st = blazeFp8GemmWorkspaceSize(&a, &n);
    *bytes = n;
    return static_cast<acltensorStatus_t>(st);
}

acltensorStatus_t Fp8Execute(const ContractionArgs& c) {
    blazeFp8GemmArgs a;
    fill_fp8_args(*c.op, c.splitPolicy, &a);
    a.group_rows = c.groupList;
    a.A = c.A;
    a.B = c.B;
    a.scaleA = c.scaleA;
    a.scaleB = c.scaleB;
    a.bias = c.bias;
    a.residual = c.C;
    a.D = c.D;
    a.scaleD = c.scaleD;
    a.workspace = c.workspace;
    a.workspace_bytes = c.workspaceSize;
    return static_cast<acltensorStatus_t>(blazeFp8Gemm(&a, c.stream));
}

// ---- unscaled solutions: INT8 A8W8 and fp16 / bf16 ----------------------------------------------------------

bool is_dense_type(acltensorDataType_t t) {
    return t == ACLTENSOR_R_8I || t == ACLTENSOR_R_16F || t == ACLTENSOR_R_16BF;
}

acltensorStatus_t DenseWorkspace(const acltensorOperationDescriptor& op, int32_t splitPolicy, uint64_t* bytes) {
    (void)splitPolicy;
    // whole 256 x 256 tiles per CTA pair: no batch modes, groups, N-major weights or quantised outputs here
    if (op.batchModes > 0 || op.groupCount > 0 || op.bNMajor) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (op.descD->dataType == ACLTENSOR_R_8F_E4M3) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (op.splitPolicy == ACLTENSOR_SPLIT_STREAM_K) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    *bytes = 0;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t DenseExecute(const ContractionArgs& c) {
    const acltensorOperationDescriptor& op = *c.op;
    blazeDenseGemmArgs a;
    std::memset(&a, 0, sizeof(a));
    a.struct_size = sizeof(a);
    a.M = static_cast<int32_t>(op.M);
    a.N = static_cast<int32_t>(op.N);
    a.K = static_cast<int32_t>(op.K);
    a.kind = op.descA->dataType == ACLTENSOR_R_8I ? BLAZE_DENSE_S8
                                                  : (op.descA->dataType == ACLTENSOR_R_16F ? BLAZE_DENSE_F16 : BLAZE_DENSE_BF16);
    a.A = c.A;
    a.lda = op.lda;
    a.B = c.B;
    a.ldb = op.ldb;
    if (op.scaleModeB == ACLTENSOR_SCALE_PER_CHANNEL) {
        a.scale_mode = BLAZE_DENSE_SCALE_PER_CHANNEL;
        a.scaleN = c.scaleB;
    } else if (op.scaleModeA == ACLTENSOR_SCALE_PER_TENSOR) {
        a.scale_mode = BLAZE_DENSE_SCALE_PER_TENSOR;
        a.scaleA = c.scaleA;
        a.scaleB = c.scaleB;
    }
    a.activation = activation_of(op.epilogueAct);
    a.bias = c.bias;
    a.residual = c.C;
    a.ldr = op.ldc;
    a.D = c.D;
    a.ldd = op.ldd;
    a.d_type = op.descD->dataType == ACLTENSOR_R_32I ? BLAZE_OUT_S32 : out_type_of(op.descD->dataType);
    a.sm_limit = op.smLimit;
    return static_cast<acltensorStatus_t>(blazeDenseGemm(&a, c.stream));
}

}  // namespace

REGISTER_CONTRACTION_SOLUTION(Int8PerTensor, R_8I, R_8I, PER_TENSOR, PER_TENSOR, 2, DenseWorkspace, DenseExecute);
REGISTER_CONTRACTION_SOLUTION(Int8PerChannel, R_8I, R_8I, NONE, PER_CHANNEL, 2, DenseWorkspace, DenseExecute);
REGISTER_CONTRACTION_SOLUTION(Int8Sums, R_8I, R_8I, NONE, NONE, 2, DenseWorkspace, DenseExecute);
REGISTER_CONTRACTION_SOLUTION(HalfMatmul, R_16F, R_16F, NONE, NONE, 2, DenseWorkspace, DenseExecute);
REGISTER_CONTRACTION_SOLUTION(Bf16Matmul, R_16BF, R_16BF, NONE, NONE, 2, DenseWorkspace, DenseExecute);
REGISTER_CONTRACTION_SOLUTION(MxFp8, R_8F_E4M3, R_8F_E4M3, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(MxW4A8, R_8F_E4M3, R_4F_E2M1, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(MxE5M2, R_8F_E5M2, R_8F_E5M2, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(MxE4M3E5M2, R_8F_E4M3, R_8F_E5M2, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(MxE5M2E4M3, R_8F_E5M2, R_8F_E4M3, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(MxW4E5M2, R_8F_E5M2, R_4F_E2M1, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(MxFp4, R_4F_E2M1, R_4F_E2M1, MX_E8M0_VEC32, MX_E8M0_VEC32, 2, MxWorkspace, MxExecute);
REGISTER_CONTRACTION_SOLUTION(Fp8Block, R_8F_E4M3, R_8F_E4M3, FP32_1X128, FP32_128X128, 0, Fp8Workspace, Fp8Execute);

// ------------------------------------------------------------------------------------------------ descriptor

acltensorStatus_t acltensorCreateContraction(const acltensorHandle_t handle, acltensorOperationDescriptor_t* desc,
                                             const acltensorTensorDescriptor_t descA, const int32_t modeA[],
                                             acltensorOperator_t opA, const acltensorTensorDescriptor_t descB,
                                             const int32_t modeB[], acltensorOperator_t opB,
                                             const acltensorTensorDescriptor_t descC, const int32_t modeC[],
                                             acltensorOperator_t opC, const acltensorTensorDescriptor_t descD,
                                             const int32_t modeD[], const acltensorComputeDescriptor_t descCompute) {
    (void)handle;
    if (desc == nullptr || descA == nullptr || descB == nullptr || descD == nullptr)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if (modeA == nullptr || modeB == nullptr || modeD == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (descC != nullptr && modeC == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (opA != ACLTENSOR_OP_IDENTITY || opB != ACLTENSOR_OP_IDENTITY || opC != ACLTENSOR_OP_IDENTITY)
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const acltensorStatus_t cst = CheckComputeDescriptor(descCompute);
    if (cst != ACLTENSOR_STATUS_SUCCESS) return cst;

    const bool dense = is_dense_type(descA->dataType);
    if (dense) {
        // INT8 x INT8 (A8W8) and fp16 / bf16: both operands of one type
        if (descB->dataType != descA->dataType) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    } else {
        if (descA->dataType != ACLTENSOR_R_8F_E4M3 && descA->dataType != ACLTENSOR_R_8F_E5M2 &&
            descA->dataType != ACLTENSOR_R_4F_E2M1)
            return ACLTENSOR_STATUS_NOT_SUPPORTED;
        // operand pairs of the reference (check_data_type.h:41-50: every pairing of the two 8-bit types, and FP4 x FP4)
        // plus the mixed W4A8 pairs: no FP4 A with an 8-bit B
        if (descA->dataType == ACLTENSOR_R_4F_E2M1 && descB->dataType != ACLTENSOR_R_4F_E2M1)
            return ACLTENSOR_STATUS_NOT_SUPPORTED;
        if (descB->dataType != ACLTENSOR_R_8F_E4M3 && descB->dataType != ACLTENSOR_R_8F_E5M2 &&
            descB->dataType != ACLTENSOR_R_4F_E2M1)
            return ACLTENSOR_STATUS_NOT_SUPPORTED;
    }
    // output: the three cast-on-store modes (bf16, half, float32), E4M3 codes for the quantising epilogue, or the raw
    // int32 sums of an INT8 product
    if (descD->dataType != ACLTENSOR_R_16BF && descD->dataType != ACLTENSOR_R_16F && descD->dataType != ACLTENSOR_R_32F &&
        descD->dataType != ACLTENSOR_R_8F_E4M3 && !(descD->dataType == ACLTENSOR_R_32I && descA->dataType == ACLTENSOR_R_8I))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (dense && descD->dataType == ACLTENSOR_R_8F_E4M3) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (descC != nullptr && descC->dataType != ACLTENSOR_R_16BF) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    // D = [batch..., m, n] with up to four batch modes; A = [its batch modes..., m, k]; B = [its batch modes..., n, k]
    // or, without batch modes in D, [group, n, k].  A batch mode missing from an operand is a broadcast.
    if (descD->numModes < 2 || descD->numModes > 6 || descA->numModes < 2 || descB->numModes < 2)
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const uint32_t nBatch = descD->numModes - 2;
    std::vector<int32_t> fullA(modeA, modeA + descA->numModes), fullB(modeB, modeB + descB->numModes),
        fullD(modeD, modeD + descD->numModes);
    const std::vector<int32_t> batchLabels(fullD.begin(), fullD.begin() + nBatch);
    const bool groupedB = nBatch == 0 && descB->numModes == 3;
    const uint32_t leadA = descA->numModes - 2, leadB = groupedB ? 0 : descB->numModes - 2;
    if (leadA > nBatch || leadB > nBatch) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (descC != nullptr && descC->numModes != descD->numModes) return ACLTENSOR_STATUS_NOT_SUPPORTED;

    // the two innermost modes of every tensor are the matrix modes
    std::vector<int32_t> mA(fullA.begin() + leadA, fullA.end()), mB(fullB.begin() + leadB, fullB.end()),
        mD(fullD.begin() + nBatch, fullD.end());
    const int64_t* lensA = descA->lens.data() + leadA;
    const int64_t* stridesA = descA->strides.data() + leadA;
    const int64_t* lensB = descB->lens.data() + leadB;
    const int64_t* stridesB = descB->strides.data() + leadB;
    const int64_t* lensD = descD->lens.data() + nBatch;
    const int64_t* stridesD = descD->strides.data() + nBatch;
    const int32_t mLabel = mD[0], nLabel = mD[1];
    if (mLabel == nLabel) return ACLTENSOR_STATUS_INVALID_VALUE;
    const int aM = find_mode(mA, mLabel);
    if (aM < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    const int aK = 1 - aM;
    const int32_t kLabel = mA[aK];
    if (kLabel == mLabel || kLabel == nLabel) return ACLTENSOR_STATUS_INVALID_VALUE;
    const int bN = find_mode(mB, nLabel), bK = find_mode(mB, kLabel);
    if (bN < 0 || bK < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    int bG = -1;
    if (groupedB) {
        bG = 3 - bN - bK;
        if (mB[bG] == mLabel || mB[bG] == nLabel || mB[bG] == kLabel) return ACLTENSOR_STATUS_INVALID_VALUE;
    }
    const int64_t M = lensD[0], N = lensD[1], K = lensA[aK];
    if (lensA[aM] != M || lensB[bN] != N || lensB[bK] != K) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (!fits_int32(M) || !fits_int32(N) || !fits_int32(K)) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    // K must be the contiguous mode of A, n the contiguous mode of the output; B is K-contiguous ("DN", what every
    // config uses) or, for a plain E4M3 matrix, N-contiguous ("ND": transposed once into the workspace)
    if (stridesA[aK] != 1 || stridesD[1] != 1) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const bool bNMajor = stridesB[bK] != 1 && stridesB[bN] == 1;
    if (stridesB[bK] != 1 && !bNMajor) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (bNMajor && (groupedB || nBatch > 0 ||
                    (descB->dataType != ACLTENSOR_R_8F_E4M3 && descB->dataType != ACLTENSOR_R_8F_E5M2)))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (descC != nullptr) {
        for (uint32_t i = 0; i < descD->numModes; ++i) {
            if (modeC[i] != fullD[i] || descC->lens[i] != descD->lens[i]) return ACLTENSOR_STATUS_INVALID_VALUE;
        }
        if (descC->strides[nBatch + 1] != 1) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    }
    int64_t groupStride = 0;
    int32_t groups = 0;
    if (bG >= 0) {
        if (bG != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;                 // group must be the outermost mode
        groups = static_cast<int32_t>(lensB[bG]);
        groupStride = stridesB[bG];
        if (groupStride != N * stridesB[bN]) return ACLTENSOR_STATUS_NOT_SUPPORTED;   // groups back to back
        if (descB->dataType != ACLTENSOR_R_8F_E4M3) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    }

    // batch extents, right-aligned in four slots; every tensor must be packed batch after batch
    int32_t batchC[4] = {1, 1, 1, 1}, batchA[4] = {1, 1, 1, 1}, batchB[4] = {1, 1, 1, 1};
    if (nBatch > 0) {
        if (aM != 0 || bN != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;      // [.., m, k] and [.., n, k] only
        auto walk = [&](const acltensorTensorDescriptor_t t, const std::vector<int32_t>& modes, uint32_t lead,
                        int32_t* out) -> acltensorStatus_t {
            int64_t expect = t->lens[lead] * t->strides[lead];              // rows x row pitch of one matrix
            uint32_t next = nBatch;                                         // batch labels must keep D's order
            for (int i = static_cast<int>(lead) - 1; i >= 0; --i) {
                int pos = -1;
                for (uint32_t j = 0; j < next; ++j)
                    if (batchLabels[j] == modes[i]) pos = static_cast<int>(j);
                if (pos < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
                if (t->lens[i] != descD->lens[pos]) return ACLTENSOR_STATUS_INVALID_VALUE;
                if (t->strides[i] != expect) return ACLTENSOR_STATUS_NOT_SUPPORTED;
                if (!fits_int32(t->lens[i])) return ACLTENSOR_STATUS_NOT_SUPPORTED;
                expect *= t->lens[i];
                out[4 - nBatch + pos] = static_cast<int32_t>(t->lens[i]);
                next = static_cast<uint32_t>(pos);
            }
            return ACLTENSOR_STATUS_SUCCESS;
        };
        acltensorStatus_t st = walk(descD, fullD, nBatch, batchC);
        if (st == ACLTENSOR_STATUS_SUCCESS) st = walk(descA, fullA, leadA, batchA);
        if (st == ACLTENSOR_STATUS_SUCCESS) st = walk(descB, fullB, leadB, batchB);
        if (st == ACLTENSOR_STATUS_SUCCESS && descC != nullptr) {
            int32_t batchR[4] = {1, 1, 1, 1};
            st = walk(descC, fullD, nBatch, batchR);
        }
        if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    }

    acltensorOperationDescriptor* d = new (std::nothrow) acltensorOperationDescriptor();
    if (d == nullptr) return ACLTENSOR_STATUS_ALLOC_FAILED;
    d->operationType = OperationType::CONTRACTION;
    d->descA = descA;
    d->descB = descB;
    d->descC = descC;
    d->descD = descD;
    d->modeA = fullA;
    d->modeB = fullB;
    d->modeD = fullD;
    if (descC != nullptr) d->modeC.assign(modeC, modeC + descC->numModes);
    d->batchModes = static_cast<int32_t>(nBatch);
    for (int i = 0; i < 4; ++i) {
        d->batchC[i] = batchC[i];
        d->batchA[i] = batchA[i];
        d->batchB[i] = batchB[i];
    }
    d->opA = opA;
    d->opB = opB;
    d->opC = opC;
    d->descCompute = descCompute;
    d->M = M;
    d->N = N;
    d->K = K;
    d->lda = stridesA[aM];
    d->ldb = bNMajor ? stridesB[bK] : stridesB[bN];
    d->bNMajor = bNMajor ? 1 : 0;
    d->ldc = descC ? descC->strides[nBatch] : 0;
    d->ldd = stridesD[0];
    d->groupStrideB = groupStride;
    d->groupCount = groups;
    *desc = d;
    return ACLTENSOR_STATUS_SUCCESS;
}

namespace {

int32_t* attribute_slot(acltensorOperationDescriptor* d, acltensorOperationDescriptorAttribute_t attr) {
    switch (attr) {
        case ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_A: return &d->scaleModeA;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_B: return &d->scaleModeB;
        case ACLTENSOR_OPERATION_DESCRIPTOR_EPILOGUE_ACT: return &d->epilogueAct;
        case ACLTENSOR_OPERATION_DESCRIPTOR_BIAS_TYPE: return &d->biasType;
        case ACLTENSOR_OPERATION_DESCRIPTOR_GROUP_COUNT: return &d->groupCount;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SPLIT_POLICY: return &d->splitPolicy;
        case ACLTENSOR_OPERATION_DESCRIPTOR_TILE_N: return &d->tileN;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SM_LIMIT: return &d->smLimit;
        case ACLTENSOR_OPERATION_DESCRIPTOR_B_IS_STATIC: return &d->bIsStatic;
        case ACLTENSOR_OPERATION_DESCRIPTOR_CTA_PAIR: return &d->ctaPair;
        case ACLTENSOR_OPERATION_DESCRIPTOR_BIAS_PER_BATCH: return &d->biasPerBatch;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_D: return &d->scaleModeD;
        default: return nullptr;
    }
}

}  // namespace

acltensorStatus_t acltensorOperationDescriptorSetAttribute(const acltensorHandle_t handle,
                                                           acltensorOperationDescriptor_t desc,
                                                           acltensorOperationDescriptorAttribute_t attr,
                                                           const void* buf, size_t sizeInBytes) {
    (void)handle;
    if (desc == nullptr || buf == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (sizeInBytes != sizeof(int32_t)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (desc->operationType != OperationType::CONTRACTION) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    int32_t* slot = attribute_slot(desc, attr);
    if (slot == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    int32_t v;
    std::memcpy(&v, buf, sizeof(v));
    switch (attr) {
        case ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_A:
        case ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_B:
            if (v < ACLTENSOR_SCALE_NONE || v > ACLTENSOR_SCALE_PER_CHANNEL) return ACLTENSOR_STATUS_INVALID_VALUE;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_EPILOGUE_ACT:
            if (activation_of(v) < 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_BIAS_TYPE:
            // bf16 everywhere, except the int32 bias an INT8 product adds to its sums
            if (v != -1 && v != ACLTENSOR_R_16BF &&
                !(v == ACLTENSOR_R_32I && desc->descA != nullptr && desc->descA->dataType == ACLTENSOR_R_8I))
                return ACLTENSOR_STATUS_NOT_SUPPORTED;
            if (v == ACLTENSOR_R_16BF && desc->descA != nullptr && desc->descA->dataType == ACLTENSOR_R_8I)
                return ACLTENSOR_STATUS_NOT_SUPPORTED;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_GROUP_COUNT:
            // the group count is fixed by the rank-3 B descriptor; setting it may only restate that value
            if (v != desc->groupCount) return ACLTENSOR_STATUS_INVALID_VALUE;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SPLIT_POLICY:
            if (v < ACLTENSOR_SPLIT_AUTO || v > ACLTENSOR_SPLIT_STREAM_K) return ACLTENSOR_STATUS_INVALID_VALUE;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_TILE_N:
            if (v != 0 && v != 128 && v != 224 && v != 256) return ACLTENSOR_STATUS_NOT_SUPPORTED;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SM_LIMIT:
            if (v < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_CTA_PAIR:
            if (v < 0 || v > 2) return ACLTENSOR_STATUS_INVALID_VALUE;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_BIAS_PER_BATCH:
            if (v < 0 || v > 1) return ACLTENSOR_STATUS_INVALID_VALUE;
            break;
        case ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_D:
            if (v != ACLTENSOR_SCALE_NONE && v != ACLTENSOR_SCALE_MX_E8M0_VEC32 && v != ACLTENSOR_SCALE_FP32_1X128)
                return ACLTENSOR_STATUS_NOT_SUPPORTED;
            break;
        default:
            break;
    }
    *slot = v;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorOperationDescriptorGetAttribute(const acltensorHandle_t handle,
                                                           const acltensorOperationDescriptor_t desc,
                                                           acltensorOperationDescriptorAttribute_t attr, void* buf,
                                                           size_t sizeInBytes) {
    (void)handle;
    if (desc == nullptr || buf == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (sizeInBytes != sizeof(int32_t)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (desc->operationType != OperationType::CONTRACTION) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const int32_t* slot = attribute_slot(desc, attr);
    if (slot == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    std::memcpy(buf, slot, sizeof(int32_t));
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ planning

namespace {

std::shared_ptr<ContractionSolution> solution_for(const acltensorOperationDescriptor& op) {
    // the registry keys on "B carries a group mode" (3) or not (2); batch modes do not change the solution
    ContractionUid uid{op.descA->dataType, op.descB->dataType, op.scaleModeA, op.scaleModeB,
                       op.groupCount > 0 ? 3u : 2u};
    return ContractionSolutionRegistry::instance().getSolution(uid);
}

}  // namespace

acltensorStatus_t acltensorEstimateWorkspaceSize(const acltensorHandle_t handle,
                                                 const acltensorOperationDescriptor_t desc,
                                                 const acltensorPlanPreference_t pref,
                                                 const acltensorWorksizePreference_t workspacePref,
                                                 uint64_t* workspaceSizeEstimate) {
    (void)handle;
    if (desc == nullptr || pref == nullptr || workspaceSizeEstimate == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (workspacePref < ACLTENSOR_WORKSPACE_MIN || workspacePref > ACLTENSOR_WORKSPACE_MAX)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if (desc->operationType == OperationType::ELEMENTWISE_BINARY) {
        *workspaceSizeEstimate = 0;
        return ACLTENSOR_STATUS_SUCCESS;
    }
    if (desc->operationType != OperationType::CONTRACTION) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    auto solution = solution_for(*desc);
    if (!solution) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    int32_t policy = desc->splitPolicy;
    if (workspacePref == ACLTENSOR_WORKSPACE_MIN) policy = ACLTENSOR_SPLIT_DATA_PARALLEL;
    if (workspacePref == ACLTENSOR_WORKSPACE_MAX && desc->groupCount == 0) policy = ACLTENSOR_SPLIT_STREAM_K;
    return solution->workspaceSize(*desc, policy, workspaceSizeEstimate);
}

namespace {

// Everything that decides which kernel configuration is best, as one token without blanks.
std::string contraction_key(const acltensorOperationDescriptor& op, const acltensorHandle* handle) {
    char buf[256];
    std::snprintf(buf, sizeof(buf), "c:%lld:%lld:%lld:a%d:b%d:d%d:c%d:sa%d:sb%d:sd%d:act%d:bias%d:g%d:bm%d:nm%d:st%d:sm%d",
                  (long long)op.M, (long long)op.N, (long long)op.K, (int)op.descA->dataType, (int)op.descB->dataType,
                  (int)op.descD->dataType, op.descC ? 1 : 0, op.scaleModeA, op.scaleModeB, op.scaleModeD, op.epilogueAct,
                  op.biasType, op.groupCount, op.batchModes, op.bNMajor, op.bIsStatic,
                  op.smLimit > 0 ? op.smLimit : (handle ? handle->smCount : 0));
    return buf;
}

std::unique_ptr<acltensorOperationDescriptor> with_choice(const acltensorOperationDescriptor& op, const PlanChoice& c) {
    std::unique_ptr<acltensorOperationDescriptor> t(new (std::nothrow) acltensorOperationDescriptor(op));
    if (t) {
        t->tileN = c.tileN;
        t->ctaPair = c.ctaPair;
        t->splitPolicy = c.splitPolicy;
    }
    return t;
}

// What a PATIENT plan times: the launch layer's own choice, then each tile shape and scheduler mode by itself.
const PlanChoice kCandidates[] = {
    {0, 0, ACLTENSOR_SPLIT_AUTO},          {256, 2, ACLTENSOR_SPLIT_AUTO},          {224, 2, ACLTENSOR_SPLIT_AUTO},
    {128, 1, ACLTENSOR_SPLIT_AUTO},        {224, 1, ACLTENSOR_SPLIT_AUTO},          {0, 0, ACLTENSOR_SPLIT_DATA_PARALLEL},
    {0, 0, ACLTENSOR_SPLIT_STREAM_K},
};

}  // namespace

namespace acltensor {

acltensorStatus_t FinishContractionPlan(acltensorPlan* plan, uint64_t workspaceSizeLimit, const acltensorHandle* handle) {
    const acltensorOperationDescriptor& caller_op = *plan->opDesc;
    if (caller_op.descA == nullptr || caller_op.descB == nullptr || caller_op.descD == nullptr)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    auto solution = solution_for(caller_op);
    if (!solution) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    plan->choice = PlanChoice{caller_op.tileN, caller_op.ctaPair, caller_op.splitPolicy};
    // a descriptor that leaves tile shape and scheduler open may take them from the handle's plan cache, or have them
    // timed at the first execution (PATIENT)
    const bool open_choice = handle != nullptr && caller_op.tileN == 0 && caller_op.ctaPair == 0 &&
                             caller_op.splitPolicy == ACLTENSOR_SPLIT_AUTO;
    if (open_choice) {
        plan->cache = handle->planCache;
        plan->cacheKey = contraction_key(caller_op, handle);
        PlanChoice cached;
        if (plan->cache->find(plan->cacheKey, &cached)) {
            auto tuned = with_choice(caller_op, cached);
            uint64_t bytes = 0;
            if (tuned && solution->workspaceSize(*tuned, cached.splitPolicy, &bytes) == ACLTENSOR_STATUS_SUCCESS &&
                bytes <= workspaceSizeLimit) {
                plan->tunedOp = std::move(tuned);
                plan->choice = cached;
            }
        } else if (plan->pref->algo == ACLTENSOR_ALGO_DEFAULT_PATIENT) {
            plan->needsTuning = true;
        }
    }
    const acltensorOperationDescriptor& op = plan->tunedOp ? *plan->tunedOp : caller_op;
    int32_t policy = op.splitPolicy;
    uint64_t need = 0;
    acltensorStatus_t st = solution->workspaceSize(op, policy, &need);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    if (need > workspaceSizeLimit && policy != ACLTENSOR_SPLIT_DATA_PARALLEL) {
        // stream-K needs a fix-up buffer; fall back to whole tiles per CTA when the caller cannot give one
        uint64_t fallback = 0;
        st = solution->workspaceSize(op, ACLTENSOR_SPLIT_DATA_PARALLEL, &fallback);
        if (st != ACLTENSOR_STATUS_SUCCESS) return st;
        if (fallback <= workspaceSizeLimit) {
            policy = ACLTENSOR_SPLIT_DATA_PARALLEL;
            need = fallback;
        }
    }
    if (need > workspaceSizeLimit) return ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE;
    if (plan->needsTuning) {
        // ask for enough workspace to try every candidate the limit allows
        for (const PlanChoice& c : kCandidates) {
            auto cand = with_choice(caller_op, c);
            uint64_t bytes = 0;
            if (cand && solution->workspaceSize(*cand, c.splitPolicy, &bytes) == ACLTENSOR_STATUS_SUCCESS &&
                bytes <= workspaceSizeLimit && bytes > need)
                need = bytes;
        }
    }
    plan->requiredWorkspace = need;
    plan->splitPolicy = policy;
    plan->choice.splitPolicy = policy;
    plan->solution = solution;
    plan->pref->solution = solution;
    return ACLTENSOR_STATUS_SUCCESS;
}

}  // namespace acltensor

// ------------------------------------------------------------------------------------------------ execution

namespace {

// Which plan wrote into a workspace buffer last.  A plan with B_IS_STATIC keeps its weight's pre-pass (re-tiled scales,
// expanded or transposed codes) in the workspace between calls; if another plan has used the same buffer in between
// (one workspace shared by several plans, as callers of BLAS-style libraries do), those bytes are gone and the
// pre-pass must run again.  Small table, most recently used last.
std::mutex g_workspace_mutex;
std::vector<std::pair<const void*, uint64_t>> g_workspace_user;
std::atomic<uint64_t> g_next_plan_stamp{1};

bool workspace_last_used_by(const void* workspace, uint64_t stamp) {
    std::lock_guard<std::mutex> lock(g_workspace_mutex);
    for (const auto& e : g_workspace_user)
        if (e.first == workspace) return e.second == stamp;
    return false;
}

void note_workspace_user(const void* workspace, uint64_t stamp) {
    if (workspace == nullptr) return;
    std::lock_guard<std::mutex> lock(g_workspace_mutex);
    for (size_t i = 0; i < g_workspace_user.size(); ++i) {
        if (g_workspace_user[i].first == workspace) {
            g_workspace_user.erase(g_workspace_user.begin() + static_cast<std::ptrdiff_t>(i));
            break;
        }
    }
    g_workspace_user.emplace_back(workspace, stamp);
    // a buffer that fell out of the table simply runs its pre-pass again
    if (g_workspace_user.size() > 256) g_workspace_user.erase(g_workspace_user.begin());
}

}  // namespace

acltensorStatus_t acltensorContract(const acltensorHandle_t handle, const acltensorPlan_t plan, const void* alpha,
                                    const void* A, const void* B, const void* beta, const void* C, void* D,
                                    const acltensorContractionAux_t* aux, void* workspace, uint64_t workspaceSize,
                                    aclrtStream stream) {
    if (plan == nullptr || A == nullptr || B == nullptr || D == nullptr || aux == nullptr)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if (handle != nullptr && handle->deviceId >= 0) {
        // a handle is bound to the device that was current when it was created; a call made with another device
        // current would launch there with this handle's SM count and plan cache
        int32_t device = -1;
        if (blazeCurrentDevice(&device) == ACLTENSOR_STATUS_SUCCESS && device != handle->deviceId)
            return ACLTENSOR_STATUS_INVALID_VALUE;
    }
    acltensorOperationDescriptor* op = plan->opDesc;
    if (op == nullptr || plan->pref == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (op->operationType != OperationType::CONTRACTION) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (!plan->solution) return ACLTENSOR_STATUS_INTERNAL_ERROR;
    if (alpha != nullptr && *static_cast<const float*>(alpha) != 1.0f) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    bool use_c = (op->descC != nullptr);
    if (beta != nullptr) {
        const float b = *static_cast<const float*>(beta);
        if (b == 0.0f) use_c = false;
        else if (b != 1.0f) return ACLTENSOR_STATUS_NOT_SUPPORTED;
        else if (op->descC == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    }
    if (use_c && C == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (op->scaleModeA != ACLTENSOR_SCALE_NONE && aux->scaleA == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (op->scaleModeB != ACLTENSOR_SCALE_NONE && aux->scaleB == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (op->biasType >= 0 && aux->bias == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (op->groupCount > 0 && aux->groupList == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    // a quantised D needs its scale mode declared and somewhere to put the scales, and nothing else may ask for them
    const bool quantD = op->descD->dataType == ACLTENSOR_R_8F_E4M3;
    // the output is quantised the way the A operand is: MX kernels emit MX scales, the FP8 kernel 1x128 scales
    const int32_t wantModeD = quantD ? op->scaleModeA : ACLTENSOR_SCALE_NONE;
    if (op->scaleModeD != wantModeD) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (quantD && aux->scaleD == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (workspaceSize < plan->requiredWorkspace) return ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE;
    if (plan->requiredWorkspace > 0 && workspace == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;

    ContractionArgs args;
    args.op = plan->tunedOp ? plan->tunedOp.get() : op;
    args.splitPolicy = plan->splitPolicy;
    args.A = A;
    args.B = B;
    args.C = use_c ? C : nullptr;
    args.D = D;
    args.scaleA = aux->scaleA;
    args.scaleB = aux->scaleB;
    args.bias = op->biasType >= 0 ? aux->bias : nullptr;
    args.groupList = op->groupCount > 0 ? aux->groupList : nullptr;
    args.scaleD = quantD ? aux->scaleD : nullptr;
    args.workspace = workspace;
    args.workspaceSize = workspaceSize;
    args.stream = stream;
    if (plan->stamp == 0) plan->stamp = g_next_plan_stamp.fetch_add(1);
    args.reuseBPrepass = op->bIsStatic != 0 && plan->preparedB == B && plan->preparedScaleB == aux->scaleB &&
                         plan->preparedWorkspace == workspace && workspace != nullptr &&
                         workspace_last_used_by(workspace, plan->stamp);
    note_workspace_user(workspace, plan->stamp);
    auto solution = std::static_pointer_cast<ContractionSolution>(plan->solution);
    if (plan->needsTuning) {
        // PATIENT: time every candidate that is valid for this problem and fits the workspace given, keep the fastest.
        // An in-place residual (C == D) would be added once per timed run, so such a call is left untuned.
        plan->needsTuning = false;
        void* timer = nullptr;
        if (!(use_c && C == D) && blazeTimerCreate(&timer) == ACLTENSOR_STATUS_SUCCESS) {
            float best_ms = 0.0f;
            int best = -1;
            std::unique_ptr<acltensorOperationDescriptor> best_op;
            for (int i = 0; i < (int)(sizeof(kCandidates) / sizeof(kCandidates[0])); ++i) {
                const PlanChoice& c = kCandidates[i];
                auto cand = with_choice(*op, c);
                uint64_t bytes = 0;
                if (!cand || solution->workspaceSize(*cand, c.splitPolicy, &bytes) != ACLTENSOR_STATUS_SUCCESS ||
                    bytes > workspaceSize)
                    continue;
                ContractionArgs trial = args;
                trial.op = cand.get();
                trial.splitPolicy = c.splitPolicy;
                trial.reuseBPrepass = false;
                if (solution->execute(trial) != ACLTENSOR_STATUS_SUCCESS) continue;      // warm-up, weight pre-pass
                trial.reuseBPrepass = op->bIsStatic != 0 && workspace != nullptr;
                float ms = 0.0f;
                bool ok = blazeTimerStart(timer, stream) == ACLTENSOR_STATUS_SUCCESS;
                for (int r = 0; r < 3 && ok; ++r) ok = solution->execute(trial) == ACLTENSOR_STATUS_SUCCESS;
                ok = ok && blazeTimerStop(timer, stream, &ms) == ACLTENSOR_STATUS_SUCCESS;
                if (ok && (best < 0 || ms < best_ms)) {
                    best = i;
                    best_ms = ms;
                    best_op = std::move(cand);
                }
            }
            blazeTimerDestroy(timer);
            if (best >= 0) {
                plan->choice = kCandidates[best];
                plan->splitPolicy = kCandidates[best].splitPolicy;
                plan->tunedOp = std::move(best_op);
                if (plan->cache && !plan->cacheKey.empty()) plan->cache->insert(plan->cacheKey, plan->choice);
                args.op = plan->tunedOp.get();
                args.splitPolicy = plan->splitPolicy;
            }
        }
        plan->preparedB = nullptr;                 // the workspace holds the last candidate's pre-pass, not ours
        args.reuseBPrepass = false;
    }
    const acltensorStatus_t st = solution->execute(args);
    if (st == ACLTENSOR_STATUS_SUCCESS) {
        plan->preparedB = B;
        plan->preparedScaleB = aux->scaleB;
        plan->preparedWorkspace = workspace;
    } else {
        plan->preparedB = nullptr;
    }
    return st;
}

acltensorStatus_t acltensorQuantize(const acltensorHandle_t handle, const void* src, int64_t ldSrc, int64_t rows,
                                    int64_t cols, acltensorScaleMode_t scaleMode, acltensorDataType_t dType,
                                    void* codes, int64_t ldCodesBytes, void* scales, aclrtStream stream) {
    (void)handle;
    if (!fits_int32(rows) || !fits_int32(cols)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (rows == 0 || cols == 0) return ACLTENSOR_STATUS_SUCCESS;            // nothing to quantise, pointers may be null
    if (src == nullptr || codes == nullptr || scales == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    const int32_t r = static_cast<int32_t>(rows), c = static_cast<int32_t>(cols);
    switch (scaleMode) {
        case ACLTENSOR_SCALE_MX_E8M0_VEC32:
            if (dType != ACLTENSOR_R_8F_E4M3 && dType != ACLTENSOR_R_8F_E5M2 && dType != ACLTENSOR_R_4F_E2M1)
                return ACLTENSOR_STATUS_NOT_SUPPORTED;
            return static_cast<acltensorStatus_t>(blazeQuantizeMx(
                src, ldSrc, r, c,
                dType == ACLTENSOR_R_4F_E2M1 ? BLAZE_ELEM_E2M1 : (dType == ACLTENSOR_R_8F_E5M2 ? BLAZE_ELEM_E5M2 : BLAZE_ELEM_E4M3),
                codes, ldCodesBytes, scales, stream));
        case ACLTENSOR_SCALE_FP32_1X128:
            if (dType != ACLTENSOR_R_8F_E4M3) return ACLTENSOR_STATUS_NOT_SUPPORTED;
            return static_cast<acltensorStatus_t>(
                blazeQuantizeFp8RowGroups(src, ldSrc, r, c, codes, ldCodesBytes, scales, stream));
        case ACLTENSOR_SCALE_FP32_128X128:
            if (dType != ACLTENSOR_R_8F_E4M3) return ACLTENSOR_STATUS_NOT_SUPPORTED;
            return static_cast<acltensorStatus_t>(
                blazeQuantizeFp8Blocks(src, ldSrc, r, c, codes, ldCodesBytes, scales, stream));
        default:
            return ACLTENSOR_STATUS_NOT_SUPPORTED;
    }
}
