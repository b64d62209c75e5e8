/*
 * blaze_b200.h - the thin C ABI that launches the sm_100a kernels of the Blaze quantized-matmul path.
 *
 * The acltensor* host API (cann_ops_tensor.h) is built on these entry points; they are exported as well so that a
 * foreign-function binding (ctypes, cgo, JNI ...) can reach the kernels with plain pointers and sizes.  All pointers
 * named "device" are CUDA device pointers, `stream` is a cudaStream_t passed as void*.  Every function returns an
 * acltensorStatus_t value as int (0 = success).  Calls are asynchronous on `stream` unless stated otherwise.
 *
 * Each entry point names the part of the reference (Atlas-Ascend-Fork/ops-tensor) it stands in for.
 */
#ifndef BLAZE_B200_H
#define BLAZE_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32) || defined(__CYGWIN__)
#define BLAZE_API __declspec(dllexport)
#else
#define BLAZE_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Element formats of quantized operands (A8/W8/W4). */
typedef enum {
    BLAZE_ELEM_E4M3 = 0, /* 8-bit, one byte per element */
    BLAZE_ELEM_E2M1 = 1, /* 4-bit, two per byte, low nibble = even K index
                            (include/blaze/gemm/tile/arch35/shift_w4_to_w8.h:88-99) */
    BLAZE_ELEM_E5M2 = 2  /* 8-bit, one byte per element: with E4M3 the 8-bit types of the reference's MX operand pairs
                            (include/tensor_api/impl/tensor_api/arch/utils/check_data_type.h:41-50) */
} blazeElem_t;

/* Element type of the output D: the cast-on-store modes of the reference's fix pipe
 * (include/tensor_api/impl/tensor_api/arch/cube/utils/l0c2out_utils.h:122-132). */
typedef enum {
    BLAZE_OUT_BF16 = 0,
    BLAZE_OUT_F16 = 1,
    BLAZE_OUT_F32 = 2,
    BLAZE_OUT_MX_E4M3 = 3, /* MX GEMM only: D leaves quantised - E4M3 codes [M][ldd bytes] plus E8M0 scales
                              scaleD [M][ceil(N/64)*2], one per 32 columns: the A operand of the next MX GEMM, bit-equal
                              to blazeQuantizeMx applied to the float32 result */
    BLAZE_OUT_FP8_128 = 4  /* FP8 GEMM only: E4M3 codes [M][ldd bytes] plus float32 scales scaleD [M][ceil(N/128)]
                              (amax / 448 per 128 columns): the A operand of the next FP8 GEMM, bit-equal to
                              blazeQuantizeFp8RowGroups applied to the float32 result */
} blazeOutType_t;

/* Storage order of B.  K-major: [N][ldb], K contiguous, scales [N][ceil(K/64)*2] (what every config uses).  N-major:
 * [K][ldb], N contiguous, with the scale layout the reference pairs with it: [ceil(K/64)][N][2]
 * (include/tensor_api/impl/tensor_api/tensor/layout_pattern.h:204-215); E4M3 only.  An N-major B is transposed once
 * into the workspace (reused across calls like the other weight pre-passes). */
typedef enum { BLAZE_B_K_MAJOR = 0, BLAZE_B_N_MAJOR = 1 } blazeBLayout_t;

/* Fused activation, applied after bias and before the residual add. */
typedef enum {
    BLAZE_ACT_IDENTITY = 0,
    BLAZE_ACT_RELU = 1,
    BLAZE_ACT_GELU_TANH = 2,
    BLAZE_ACT_SILU = 3,     /* x * sigmoid(x) */
    BLAZE_ACT_SIGMOID = 4,
    BLAZE_ACT_TANH = 5
} blazeActivation_t;

/* How the output tiles are scheduled over the SMs. */
typedef enum {
    BLAZE_SCHED_AUTO = 0,          /* heuristic */
    BLAZE_SCHED_DATA_PARALLEL = 1, /* one CTA per output tile, full K */
    BLAZE_SCHED_STREAM_K = 2       /* (tile, k-block) units split evenly, fp32 fix-up in workspace */
} blazeSched_t;

/* ------------------------------------------------------------------------------------------------------------
 * MX block-scaled GEMM:  D = act(A x B^T + bias) + residual, fp32 accumulation, bf16 / half / float32 output.
 *   A  [M][lda] codes, K-contiguous (E4M3 or packed E2M1)  scaleA [M][ceil(K/64)*2] E8M0 bytes, one per 32 K
 *   B  [N][ldb] codes, K-contiguous (E4M3 or packed E2M1)  scaleB [N][ceil(K/64)*2]
 * Stands in for GemmUniversal<KernelMmadWithScaleMx>::operator() and its Params
 * (include/blaze/gemm/kernel/kernel_qbmm_mx.h:80-115, :154-176) with the scale layouts of
 * include/tensor_api/impl/tensor_api/tensor/layout_pattern.h:180-226.
 * Constraints: K % 16 == 0, N % 8 == 0, lda/ldb multiples of 16 bytes, ldd/ldr multiples of 8 elements, all base
 * pointers 16-byte aligned.  A packed E2M1 B with K % 128 == 0, ldb % 32 == 0 and a 32-byte aligned base is read as it
 * is; any other packed B is first expanded to one-byte codes in the workspace (same results, N x K more bytes).
 * ------------------------------------------------------------------------------------------------------------ */
#define BLAZE_MAX_PEERS 7 /* further copies of D that a GEMM epilogue can write (peerD) */

typedef struct {
    size_t struct_size; /* sizeof(blazeMxGemmArgs), for forward compatibility */
    int32_t M, N, K;
    int32_t b_elem;          /* blazeElem_t of B */
    const void* A;           /* device */
    int64_t lda;             /* bytes between rows of A */
    const void* B;           /* device */
    int64_t ldb;             /* bytes between rows of B */
    const void* scaleA;      /* device, E8M0 */
    const void* scaleB;      /* device, E8M0 */
    const void* bias;        /* device bf16[N] or NULL */
    const void* residual;    /* device bf16 [M][ldr] or NULL */
    int64_t ldr;             /* elements */
    void* D;                 /* device [M][ldd], bf16 unless d_type says otherwise */
    int64_t ldd;             /* elements */
    int32_t activation;      /* blazeActivation_t */
    int32_t tile_n;          /* 0 = choose; else 128, 224 or 256 (256 only with 2-CTA tiles) */
    int32_t reuse_b_prepass; /* 1: workspace still holds B's re-tiled scales / expanded codes from the previous call */
    int32_t sm_limit;        /* 0 = all SMs; else cap on the persistent grid */
    int32_t cta_pair;        /* 0 = choose; 1 = 128-row tiles, one CTA each; 2 = 256-row tiles on 2-CTA clusters */
    int32_t a_elem;          /* blazeElem_t of A: 0 = E4M3; BLAZE_ELEM_E2M1 = packed 4-bit A (the FP4 x FP4 pair of
                                include/tensor_api/impl/tensor_api/arch/cube/mmad/check_data_type.h:41-50); needs
                                K % 128 == 0, lda % 32 == 0, a 32-byte aligned A, and an E2M1 B */
    void* workspace;         /* device, 256-byte aligned */
    size_t workspace_bytes;
    int32_t d_type;          /* blazeOutType_t of D (ldd counts elements of that type) */
    int32_t b_layout;        /* blazeBLayout_t */
    void* scaleD;            /* device, E8M0 scales of D when d_type is BLAZE_OUT_MX_E4M3, else NULL */
    int32_t sched;           /* blazeSched_t; stream-K applies to the single-CTA tiles (skinny M or N) */
    int32_t n_peers;         /* 0..BLAZE_MAX_PEERS: copies of D that the epilogue also writes (see peerD) */
    void* peerD[7];          /* device pointers this GPU can store to - typically the slot of this rank in the other
                                GPUs' gathered output (peer-mapped symmetric memory) - same shape, ldd and type as D.
                                Every output tile is stored to D and to each of them straight from the epilogue, so an
                                N-sharded GEMM ends with the whole matrix on every GPU without a separate all-gather.
                                Needs the 2-CTA tiles, a bf16 / f16 D and 1 KB more workspace. */
} blazeMxGemmArgs;

/* Device timer on a stream (a pair of CUDA events), for callers above this ABI that have no CUDA headers: Start
 * records, Stop records, waits for the stream to get there and returns the milliseconds in between. */
BLAZE_API int blazeTimerCreate(void** timer);
BLAZE_API int blazeTimerStart(void* timer, void* stream);
BLAZE_API int blazeTimerStop(void* timer, void* stream, float* milliseconds);
BLAZE_API int blazeTimerDestroy(void* timer);

BLAZE_API int blazeMxGemmWorkspaceSize(const blazeMxGemmArgs* args, size_t* bytes);
BLAZE_API int blazeMxGemm(const blazeMxGemmArgs* args, void* stream);

/*
 * The same MX GEMM for hosts that cannot give the library device memory: a serving process that has handed the whole
 * GPU to its own memory pool, or a latency-critical loop in which a device allocation (which synchronises the GPU)
 * is forbidden.  No counterpart in the reference.
 *
 * args->workspace and args->workspace_bytes are ignored: the re-tiled scale factors live in a fixed 8 MiB array that
 * is part of the library image (every GPU that loads the library holds those 8 MiB until the process exits).  The
 * call allocates nothing and frees nothing.  Limits and rules:
 *   - B must be BLAZE_ELEM_E4M3 (packed E2M1 would need an N x K expansion buffer) and K-major (an N-major B would
 *     need a transposed copy): NOT_SUPPORTED otherwise; stream-K and peer outputs are not offered either;
 *   - a problem whose re-tiled scales exceed 8 MiB - about 512*(ceil(M/128) + 2*ceil(N/224))*ceil(K/128) bytes, e.g.
 *     M = N = K = 8192 needs 4.4 MiB - is refused with ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE before anything runs
 *     (blazeMxGemm keeps four copies of B's scale blocks on 2-CTA tiles to save a tensor-pipe copy per K step; this
 *     call does the same while that fits the array and keeps a single copy otherwise);
 *   - the first call on a device looks up the array's device address (one-time set-up, with that device current);
 *     make that first call outside any stream capture;
 *   - all calls share the one array, which still holds the previous call's tiles; each call rewrites the part it
 *     uses, so calls must not overlap on the GPU (use one stream, or order them with events) - overlapping calls race;
 *   - reuse_b_prepass is ignored (the weight's scale tiles are rebuilt every call).
 * device_status is an optional device pointer to a zero-initialised int32 that receives the code of a kernel wait
 * that gave up (see blazeDeviceStatus); with NULL the code goes to a word inside the library, which blazeDeviceStatus /
 * acltensorGetDeviceStatus report (and reset) together with the status of the other entry points.
 */
BLAZE_API int blazeMxGemmNoAlloc(const blazeMxGemmArgs* args, int32_t* device_status, void* stream);

/*
 * Batched MX GEMM with broadcast: D[b] = act(A[ia(b)] x B[ib(b)]^T + bias) + residual[b] over up to four batch
 * dimensions, the loop nest of GemmUniversal<...>::ProcessWithBatch (include/blaze/gemm/kernel/kernel_qbmm_mx.h:282-338)
 * with the per-batch offsets of AddBatchOffset (:340-377).  c[] are the batch extents of D (outermost first, 1 for an
 * unused dimension); a[i] and b[i] are c[i], or 1 when that operand is broadcast along dimension i.  Every operand is
 * packed batch after batch: A[prod(a)][M][lda], scaleA[prod(a)][M][ceil(K/64)*2], B[prod(b)][N][ldb], scaleB likewise,
 * D and residual [prod(c)][M][ldd / ldr], bias [N] or, with bias_per_batch, [prod(c)][N].  `args` describes one
 * batch.  When B is the same for every batch and A is not broadcast, the batches are rows of one tall GEMM and run as
 * a single launch; otherwise one launch per batch on `stream`, sharing the workspace.
 */
typedef struct {
    int32_t c[4];
    int32_t a[4];
    int32_t b[4];
    int32_t bias_per_batch;
    int32_t reserved;
} blazeBatchDims;

BLAZE_API int blazeMxGemmBatchedWorkspaceSize(const blazeMxGemmArgs* args, const blazeBatchDims* batch, size_t* bytes);
BLAZE_API int blazeMxGemmBatched(const blazeMxGemmArgs* args, const blazeBatchDims* batch, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * FP8 GEMM with float32 scales (1x128 groups of A, 128x128 blocks of B), dense or grouped, data-parallel or
 * stream-K.  D = act(sum_kb sa*sb*(A_kb x B_kb^T) + bias) + residual, bf16 output.
 *   A  [M][lda] E4M3               scaleA [M][ceil(K/128)] fp32
 *   B  [G][N][ldb] E4M3            scaleB [G][ceil(K/128)][ceil(N/128)] fp32
 *   group_rows  device int64[G]: rows of A (and D) belonging to each group, in order; NULL / groups==0 = dense.
 * The reference only names these modes (QuantMode PERGROUP/PERBLOCK: include/blaze/gemm/utils/common_utils.h:98-107;
 * groupListGmAddr: include/blaze/gemm/block/block_mmad_matmul_basic.h:68); stream-K follows
 * GemmUniversal<KernelMultiBlockStreamK> (include/blaze/gemm/kernel/kernel_matmul_streamk.h:71-228) and
 * BlockEpilogueMatmulStreamK (include/blaze/epilogue/block/block_epilogue_matmul_streamk.h:99-265).
 * Constraints: K % 16 == 0, N % 8 == 0, groups <= 1024, grouped B is contiguous per group (ldb * N bytes apart).
 * ------------------------------------------------------------------------------------------------------------ */
typedef struct {
    size_t struct_size;
    int32_t M, N, K;
    int32_t groups;
    const void* group_rows; /* device int64[groups] */
    const void* A;
    int64_t lda;
    const void* B;
    int64_t ldb;
    const void* scaleA;
    const void* scaleB;
    const void* bias;
    const void* residual;
    int64_t ldr;
    void* D;
    int64_t ldd;
    int32_t activation;
    int32_t sched;    /* blazeSched_t */
    int32_t sm_limit; /* 0 = all SMs */
    int32_t d_type;   /* blazeOutType_t of D */
    void* workspace;
    size_t workspace_bytes;
    void* scaleD;     /* device float32 scales of D when d_type is BLAZE_OUT_FP8_128, else NULL */
    int32_t n_peers;  /* 0..BLAZE_MAX_PEERS further copies of D, as in blazeMxGemmArgs (bf16 / f16 D only) */
    int32_t b_is_static; /* 1: B and scaleB are not written by the kernel that precedes this call in the stream (weights):
                            a dense problem then requests its first weight tiles while that kernel is still running */
    void* peerD[7];
} blazeFp8GemmArgs;

BLAZE_API int blazeFp8GemmWorkspaceSize(const blazeFp8GemmArgs* args, size_t* bytes);
BLAZE_API int blazeFp8Gemm(const blazeFp8GemmArgs* args, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Unscaled GEMMs of the Blaze surface: INT8 x INT8 with int32 accumulation and de-quantisation on store (A8W8), and
 * fp16 / bf16 with float32 accumulation.  D = act(A x B^T + bias) + residual; A [M][lda], B [N][ldb], both K-contiguous.
 * INT8 stands in for GemmUniversal<..., KernelQbmmCube> + BlockMmad<...A8W8FixpipeQuant>
 * (include/blaze/gemm/kernel/kernel_qbmm_cube.h:43-140, include/blaze/gemm/block/block_mmad_a8w8_fixpipe_quant.h:42-527):
 * the int32 sum (plus an optional int32 bias per column, the reference's accumulator init) is converted to float32
 * and multiplied by a scale whose low 13 mantissa bits are cleared, as the reference prepares it for its fix pipe
 * (DEQ_SCALE_MUL, kernel_qbmm_cube.h:68, :190-220): per tensor scaleA[0] * scaleB[0], or per channel the low 32 bits of
 * scaleN[n]; BLAZE_DENSE_SCALE_NONE stores the plain conversion, or the raw sums when d_type is BLAZE_OUT_S32 (the
 * reference's int32 output mode, block_mmad_a8w8_fixpipe_quant.h:228).  The 16-bit kinds stand in for the basic
 * matmul kernel (include/blaze/gemm/kernel/kernel_matmul_basic.h:32-200).
 * Constraints: K bytes per row a multiple of 16, N % 8 == 0, lda / ldb (elements) give 16-byte multiples, base pointers
 * 16-byte aligned, ldd / ldr multiples of 8 elements.  No workspace.
 * ------------------------------------------------------------------------------------------------------------ */
typedef enum { BLAZE_DENSE_S8 = 0, BLAZE_DENSE_F16 = 1, BLAZE_DENSE_BF16 = 2 } blazeDenseKind_t;
typedef enum { BLAZE_DENSE_SCALE_NONE = 0, BLAZE_DENSE_SCALE_PER_TENSOR = 1, BLAZE_DENSE_SCALE_PER_CHANNEL = 2 } blazeDenseScale_t;
#define BLAZE_OUT_S32 5 /* continues blazeOutType_t: raw int32 sums of an INT8 product */

typedef struct {
    size_t struct_size;
    int32_t M, N, K;
    int32_t kind;           /* blazeDenseKind_t */
    const void* A;          /* device */
    int64_t lda;            /* elements between rows of A */
    const void* B;          /* device */
    int64_t ldb;            /* elements between rows of B */
    int32_t scale_mode;     /* blazeDenseScale_t (INT8 only) */
    int32_t activation;     /* blazeActivation_t */
    const void* scaleA;     /* device float32[1] (per tensor) */
    const void* scaleB;     /* device float32[1] (per tensor) */
    const void* scaleN;     /* device uint64[N] (per channel) */
    const void* bias;       /* device: int32[N] for INT8, bf16[N] for the 16-bit kinds, or NULL */
    const void* residual;   /* device bf16 [M][ldr] or NULL */
    int64_t ldr;
    void* D;                /* device [M][ldd] */
    int64_t ldd;
    int32_t d_type;         /* BLAZE_OUT_BF16 / F16 / F32, or BLAZE_OUT_S32 (INT8 without scale) */
    int32_t sm_limit;       /* 0 = all SMs */
} blazeDenseGemmArgs;

BLAZE_API int blazeDenseGemm(const blazeDenseGemmArgs* args, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Quantisers (fp32 source, round-to-nearest-even, saturating).  The reference has no quantiser; these produce the
 * operand and scale layouts its MX kernel consumes (include/blaze/gemm/kernel/kernel_qbmm_mx.h:383-404).
 * ------------------------------------------------------------------------------------------------------------ */
/* x [rows][ldx] fp32 -> codes [rows][ld_codes bytes], scales [rows][ceil(K/64)*2] E8M0.  K % 4 == 0. */
BLAZE_API int blazeQuantizeMx(const void* x, int64_t ldx, int32_t rows, int32_t K, int32_t elem, void* codes,
                              int64_t ld_codes, void* scales, void* stream);
/* x [rows][ldx] fp32 -> E4M3 codes [rows][ld_codes], scales [rows][ceil(K/128)] fp32 (amax/448). */
BLAZE_API int blazeQuantizeFp8RowGroups(const void* x, int64_t ldx, int32_t rows, int32_t K, void* codes,
                                        int64_t ld_codes, void* scales, void* stream);
/* w [N][ldw] fp32 (K-contiguous weight) -> E4M3 codes [N][ld_codes], scales [ceil(K/128)][ceil(N/128)] fp32. */
BLAZE_API int blazeQuantizeFp8Blocks(const void* w, int64_t ldw, int32_t N, int32_t K, void* codes, int64_t ld_codes,
                                     void* scales, void* stream);

/* D = A + C on n floats: the CUDA stand-in for the reference's only shipped operator
 * (src/add/add_kernel.cpp:173-189). */
BLAZE_API int blazeAddF32(const void* A, const void* C, void* D, int64_t n, void* stream);

/* Device status word of the current device: 0 while every kernel wait completed, else the code of the first
 * wait that gave up (see DeviceStatus in csrc/ptx.cuh), including waits inside blazeMxGemmNoAlloc calls that were given
 * no status pointer.  Synchronises the device.  reset != 0 clears it. */
BLAZE_API int blazeDeviceStatus(int32_t* value, int32_t reset);

/* Closing signal of a fused gather (the GEMM's epilogue stored its tiles into the peers' buffers, `peerD`): tells every
 * peer "all stores of my launches up to `value` have been issued and completed", and waits until every peer has said
 * the same.  One CTA, behind the GEMM on `stream`: it stores `value` (system scope, release) into slot `my_rank` of each
 * peer's flag array - peer STORES only, no load ever reads another GPU's memory - and then polls this GPU's own array
 * until the slots of all `peer_ranks` hold a value >= `value`.  The wait is bounded (`limit_cycles` SM cycles, <= 2^33;
 * 0 = ~1 s): when it expires the kernel records code 6 in the device status word and returns.  `value` must grow from
 * call to call (a step counter); the arrays (uint64 per rank, zero before the first call) live in memory every rank has
 * mapped, e.g. torch symmetric memory.  Replaces a one-element all-reduce (~14 us of collective launch and handshake).
 * No counterpart in the reference (its ranks exchange nothing on this path). */
typedef struct blazePeerSignalArgs {
    size_t struct_size;                        /* sizeof(blazePeerSignalArgs) */
    int32_t my_rank;
    int32_t n_peers;                           /* 1 .. BLAZE_MAX_PEERS */
    int32_t peer_ranks[BLAZE_MAX_PEERS];       /* rank of peer q (its slot in this GPU's array) */
    void* local_flags;                         /* this GPU's array, uint64 [ranks] */
    void* peer_flags[BLAZE_MAX_PEERS];         /* peer q's array as mapped into this process, uint64 [ranks] */
    uint64_t value;
    int64_t limit_cycles;
} blazePeerSignalArgs;
BLAZE_API int blazePeerSignal(const blazePeerSignalArgs* args, void* stream);

/* Diagnostic of the failure-reporting path (no counterpart in the reference): launches one CTA that waits, for at most
 * `limit_cycles` SM cycles (<= 2^31), on a barrier nothing signals.  The wait expires, the kernel returns normally, and
 * the next blazeDeviceStatus / acltensorGetDeviceStatus reports code 7.  Nothing hangs or faults. */
BLAZE_API int blazeSelfTestWaitTimeout(int64_t limit_cycles, void* stream);

/* SM count and compute capability of the current device (the handle's device query). */
BLAZE_API int blazeDeviceInfo(int32_t* sm_count, int32_t* cc_major, int32_t* cc_minor);

/* Ordinal of the CUDA device current in the calling thread: what a handle binds to at acltensorCreate (the role of
 * the reference's platform query in lib/core/handle.cpp:75-92). */
BLAZE_API int blazeCurrentDevice(int32_t* device);

#ifdef __cplusplus
}
#endif
#endif /* BLAZE_B200_H */
