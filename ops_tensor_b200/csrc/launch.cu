// C-ABI layer of the kernel library: argument checking, workspace carving, TMA descriptor encoding, tile/grid
// heuristics and the kernel launches themselves.  Nothing here allocates per call; the only allocation is the
// 4-byte per-device status word made on first use of a device.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>

#include "blaze_b200.h"
#include "cann_ops_tensor_types.h"
#include "gemm_dense_pair.cuh"
#include "gemm_fp8.cuh"
#include "gemm_mx.cuh"
#include "gemm_mx_pair.cuh"
#include "launch.h"

namespace blaze {

// ------------------------------------------------------------------------------------------------ device context

static std::mutex g_ctx_mutex;
static DeviceContext g_ctx[64];

DeviceContext* current_context() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    DeviceContext& c = g_ctx[dev];
    if (c.device == dev) return &c;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    int* word = nullptr;
    if (cudaMalloc(&word, 256) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    cudaMemset(word, 0, 256);
    c.sm_count = prop.multiProcessorCount;
    c.cc_major = prop.major;
    c.cc_minor = prop.minor;
    c.status_word = word;
    c.device = dev;
    return &c;
}

// ------------------------------------------------------------------------------------------------ tensor maps

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// Byte matrix [rows][row_bytes valid, pitch bytes apart], boxes of 128 bytes x box_rows, 128-byte swizzle, zero fill
// outside the matrix.
static bool make_tmap_bytes(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t pitch,
                            uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                          elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Packed 4-bit operand [rows][pitch bytes], K elements per row, two per byte: TMA unpacks every 16 codes (8 bytes) into
// a 16-byte slot of shared memory, the form the f8f6f4 tensor-core kinds read 4-bit operands in, so a row of 128
// codes fills the same 128 swizzled bytes as a row of 128 one-byte codes.  The driver wants the base 32-byte aligned,
// the pitch a multiple of 32 bytes and whole 128-code boxes along K; the caller checks those and falls back to the
// expansion pre-pass when the encoder refuses.
static bool make_tmap_packed4(CUtensorMap* map, const void* base, uint64_t k_elems, uint64_t rows, uint64_t pitch_bytes,
                              uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {k_elems, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box,
                          elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// bf16 output matrix [rows][cols valid, ld elements apart] written in 32 x 32 blocks staged with the 64-byte swizzle.
// (Half outputs use the same shape; float32 outputs leave as 32 x 16 blocks, again 64 bytes per row.)
static bool make_tmap_store(CUtensorMap* map, void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems,
                            int out_type) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const bool f32 = out_type == BLAZE_OUT_F32;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    if (out_type == BLAZE_OUT_MX_E4M3) {                    // one-byte codes: 32 x 32-byte blocks, no swizzle
        const cuuint64_t strides8[1] = {ld_elems};
        const cuuint32_t box8[2] = {32, 32};
        return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides8, box8, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    const cuuint64_t strides[1] = {ld_elems * (f32 ? 4 : 2)};
    const cuuint32_t box[2] = {f32 ? 16u : 32u, 32};
    const CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                       : (out_type == BLAZE_OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                    : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    const CUresult r = fn(map, dt, 2, base, dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static inline size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

static int status_of(cudaError_t e) {
    if (e == cudaSuccess) return ACLTENSOR_STATUS_SUCCESS;
    cudaGetLastError();
    return ACLTENSOR_STATUS_EXECUTION_FAILED;
}

// ------------------------------------------------------------------------------------------------ MX GEMM

struct MxPlan {
    bool pair;          // 256-row tiles on 2-CTA clusters
    int tile_n;
    int sfb_replicas;   // copies of every 512-byte scale block of B in the re-tiled array
    bool mxf4;          // FP4 x FP4 on kind::mxf4 (dense 4-bit tiles, K = 256 per stage)
    bool stream_k;      // single-CTA tiles: (tile, K step) units split evenly over the grid; 2-CTA tiles: the tiles of
                        // the last, partly filled round cut along K so that every pair gets the same share of them
    int grid;           // CTAs of the kernel (2-CTA tiles: only when stream_k is set)
    size_t flags_off, partials_off, flags_bytes, partials_bytes;
    int sf_k_steps;     // 128-K blocks of the re-tiled scale arrays
    int m_tiles, n_tiles, k_steps;
    size_t sfa_bytes, sfb_bytes, b_expand_bytes, b_scale_rows_bytes;
    size_t sfa_off, sfb_off, b_expand_off, b_scale_rows_off, total;
    size_t peer_maps_off;   // tensor maps of the peer outputs (1 KB), when the call names any
};

static int choose_tile_n(int M, int N, int sms, int requested) {
    if (requested == 128 || requested == 224) return requested;
    if (N <= 128) return 128;
    const long long mt = (M + 127) / 128;
    auto cost = [&](int bn) {
        const long long tiles = mt * ((N + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        return waves * (bn + 24);            // per-tile time ~ tile width plus a fixed ramp
    };
    return cost(224) <= cost(128) ? 224 : 128;
}

// Width of the 256-row paired tiles: the one whose last wave wastes less, 256 on a tie (a K step then carries more MMA
// work per scale copy and per operand byte).
static int choose_pair_tile_n(int M, int N, int sms) {
    const long long pairs = sms / 2 > 0 ? sms / 2 : 1;
    const long long m_tiles = (M + 255) / 256;
    long long best_cost = 0;
    int best = 256;
    for (int w : {256, 224}) {
        const long long tiles = m_tiles * ((N + w - 1) / w);
        const long long cost = ((tiles + pairs - 1) / pairs) * w;
        if (best_cost == 0 || cost < best_cost) {
            best_cost = cost;
            best = w;
        }
    }
    return best;
}

// `wide_scale_copy` = false keeps one copy of B's scale blocks (a quarter of the workspace, one more tensor-pipe copy
// per K step); the allocation-free entry uses it when the replicated form does not fit its fixed array.
// `allow_split` = false keeps whole tiles per CTA (no stream-K workspace), likewise for that entry.
static int plan_mx(const blazeMxGemmArgs* a, int sms, MxPlan* pl, bool wide_scale_copy = true, bool allow_split = true) {
    if (!a || a->struct_size != sizeof(blazeMxGemmArgs)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->M < 0 || a->N < 0 || a->K < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->b_elem < BLAZE_ELEM_E4M3 || a->b_elem > BLAZE_ELEM_E5M2) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->a_elem < BLAZE_ELEM_E4M3 || a->a_elem > BLAZE_ELEM_E5M2) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->d_type < BLAZE_OUT_BF16 || a->d_type > BLAZE_OUT_MX_E4M3) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->b_layout != BLAZE_B_K_MAJOR && a->b_layout != BLAZE_B_N_MAJOR) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->b_layout == BLAZE_B_N_MAJOR && a->b_elem == BLAZE_ELEM_E2M1) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    // legal operand pairs: FP8 x FP8, FP8 x FP4 (W4A8) and FP4 x FP4; a 4-bit A is only read natively
    if (a->a_elem == BLAZE_ELEM_E2M1 && (a->b_elem != BLAZE_ELEM_E2M1 || (a->K % 128) != 0))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->activation < BLAZE_ACT_IDENTITY || a->activation > BLAZE_ACT_TANH) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->tile_n != 0 && a->tile_n != 128 && a->tile_n != 224 && a->tile_n != 256) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if ((a->K % 16) != 0 || (a->N % 8) != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->cta_pair < 0 || a->cta_pair > 2) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->cta_pair == 2 && a->tile_n == 128) return ACLTENSOR_STATUS_NOT_SUPPORTED;    // paired tiles: 256 x 224 / 256
    if (a->cta_pair == 1 && a->tile_n == 256) return ACLTENSOR_STATUS_NOT_SUPPORTED;    // 256 wide only on pairs
    // 256-row tiles on CTA pairs once there are at least two 128-row blocks and more than one 128-column block
    // (an explicit tile_n of 128 or 224 without cta_pair = 2 keeps the single-CTA kernel of that width)
    pl->pair = a->cta_pair == 2 || a->tile_n == 256 ||
               (a->cta_pair == 0 && a->tile_n == 0 && a->M > 128 && a->N > 128 && sms >= 2);
    if (pl->pair) {
        pl->tile_n = a->tile_n ? a->tile_n : choose_pair_tile_n(a->M, a->N, sms);
    } else {
        pl->tile_n = choose_tile_n(a->M, a->N, sms, a->tile_n);
    }
    // FP4 x FP4 at the double rate needs the 2-CTA 256-wide tiles, whole 256-K stages and the replicated scale blocks
    pl->mxf4 = a->a_elem == BLAZE_ELEM_E2M1 && a->b_elem == BLAZE_ELEM_E2M1 && pl->pair && wide_scale_copy &&
               (a->tile_n == 0 || a->tile_n == 256) && (a->K % 256) == 0 && a->K > 0;
    if (pl->mxf4) pl->tile_n = 256;
    pl->m_tiles = pl->pair ? (a->M + 255) / 256 : (a->M + 127) / 128;
    pl->n_tiles = (a->N + pl->tile_n - 1) / pl->tile_n;
    pl->sf_k_steps = (a->K + 127) / 128;
    pl->k_steps = pl->mxf4 ? a->K / 256 : pl->sf_k_steps;
    pl->sfa_bytes = (size_t)sf_tiled_bytes(a->M, a->K, 128);
    pl->sfb_replicas = (pl->pair && wide_scale_copy) ? 4 : 1;        // the wide copy has no lane broadcast
    pl->sfb_bytes = (size_t)sf_tiled_bytes(a->N, a->K, pl->tile_n, pl->sfb_replicas);
    // room for a one-byte-per-code K-major copy of B: the expansion of a packed E2M1 B, or the transpose of an N-major B
    pl->b_expand_bytes = ((a->b_elem == BLAZE_ELEM_E2M1 && !pl->mxf4) || a->b_layout == BLAZE_B_N_MAJOR)
                             ? (size_t)a->N * (size_t)a->K : 0;
    pl->b_scale_rows_bytes = a->b_layout == BLAZE_B_N_MAJOR ? (size_t)a->N * (size_t)(((a->K + 63) / 64) * 2) : 0;
    pl->sfa_off = 0;
    pl->sfb_off = round256(pl->sfa_bytes);
    pl->b_expand_off = pl->sfb_off + round256(pl->sfb_bytes);
    pl->b_scale_rows_off = pl->b_expand_off + round256(pl->b_expand_bytes);
    // Skinny problems (few single-CTA tiles, long K) split along K as well: the cost model of the FP8 scheduler, in units
    // of one K step on one SM
    int eff_sms = sms;
    if (a->sm_limit > 0 && a->sm_limit < eff_sms) eff_sms = a->sm_limit;
    const long long tiles = (long long)pl->m_tiles * pl->n_tiles;
    pl->stream_k = false;
    pl->grid = (int)(tiles < eff_sms ? (tiles > 0 ? tiles : 1) : eff_sms);
    if (a->sched < BLAZE_SCHED_AUTO || a->sched > BLAZE_SCHED_STREAM_K) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (!pl->pair && allow_split && tiles > 0 && pl->k_steps >= 2 && a->sched != BLAZE_SCHED_DATA_PARALLEL) {
        // as in plan_fp8: all SMs, or every tile cut into s equal K ranges for the s whose modelled cost (K steps
        // + fixed cost + 4.7 steps per CTA the owner has to wait for and add) is least
        const long long units = tiles * pl->k_steps;
        long long used = units < eff_sms ? units : eff_sms;
        const double whole_tiles = (double)((tiles + eff_sms - 1) / eff_sms) * pl->k_steps;
        double split = (double)((units + used - 1) / used) + 17.0 + 4.7 * ((double)used / (double)tiles);
        for (long long s_cut = 2; s_cut * tiles <= eff_sms && s_cut <= pl->k_steps; ++s_cut) {
            const double c = (double)((pl->k_steps + s_cut - 1) / s_cut) + 12.0 + 4.7 * (double)(s_cut - 1);
            if (c < split) {
                split = c;
                used = s_cut * tiles;
            }
        }
        if (a->sched == BLAZE_SCHED_STREAM_K || split < whole_tiles) {
            pl->stream_k = true;
            pl->grid = (int)used;
        }
    }
    if (pl->pair && allow_split && tiles > 0 && pl->k_steps >= 2 && a->sched != BLAZE_SCHED_DATA_PARALLEL) {
        // 2-CTA tiles: whole rounds run as they are; the R tiles left for the last round may be cut along K so that
        // every pair gets an even share of their K steps.  Measured on B200 the fix-up (256 KB of partial sums per tile
        // through L2, read back chunk by chunk inside the owner's epilogue) costs about 14 us, some 30 K steps:
        // 8192 x 1024 x 8192 takes 81 us split against 75 us whole, so the split is only chosen by itself for very
        // long K; a caller can still force it
        const long long pairs = eff_sms / 2 > 0 ? eff_sms / 2 : 1;
        const long long rest = tiles % pairs;
        if (rest > 0) {
            const double whole = (double)pl->k_steps;
            const double even = (double)((rest * pl->k_steps + pairs - 1) / pairs) + 30.0 + (double)pairs / (double)rest;
            if (a->sched == BLAZE_SCHED_STREAM_K || even <= 0.9 * whole) {
                pl->stream_k = true;
                pl->grid = (int)(2 * pairs);
            }
        }
    }
    pl->flags_bytes = pl->stream_k ? round256((size_t)pl->grid * sizeof(int)) : 0;
    pl->partials_bytes = pl->stream_k ? (size_t)pl->grid * 128 * (size_t)pl->tile_n * sizeof(float) : 0;
    pl->flags_off = pl->b_scale_rows_off + round256(pl->b_scale_rows_bytes);
    pl->partials_off = pl->flags_off + pl->flags_bytes;
    pl->total = pl->partials_off + round256(pl->partials_bytes);
    pl->peer_maps_off = pl->total;
    if (a->n_peers < 0 || a->n_peers > BLAZE_MAX_PEERS) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->n_peers > 0) {
        // the epilogue of the 2-CTA kernel stores 16-bit tiles through the extra maps; nothing else does
        if (!pl->pair || (a->d_type != BLAZE_OUT_BF16 && a->d_type != BLAZE_OUT_F16)) return ACLTENSOR_STATUS_NOT_SUPPORTED;
        pl->total += 1024;
    }
    return ACLTENSOR_STATUS_SUCCESS;
}

// Launch of a GEMM kernel that follows its scale re-tile pre-pass in the stream: programmatic stream serialisation
// lets the GEMM's blocks set themselves up while the pre-pass is still running; the kernel's producer thread waits for
// the pre-pass (griddepcontrol.wait) before its first load.
template <class... KArgs, class... Args>
static cudaError_t launch_after_prepass(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                                        const Args&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int kBN, int kAct>
static cudaError_t launch_mx_instance(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                                      const MxGemmParams& p, int grid, cudaStream_t stream) {
    constexpr int kStages = kBN <= 128 ? 6 : 4;       // as many operand stages as fit beside the epilogue's staging blocks
    using L = MxGemmSmem<kBN, kStages>;
    static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory per CTA");
    auto kernel = mx_gemm_kernel<kBN, kStages, kAct>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev & 63] = true;
    }
    return launch_after_prepass(kernel, grid, 192, L::kDynamicBytes, stream, ta, tb, td, p);
}

template <int kBN>
static cudaError_t launch_mx_act(int act, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                                 const MxGemmParams& p, int grid, cudaStream_t stream) {
    switch (act) {
        case BLAZE_ACT_RELU: return launch_mx_instance<kBN, ACT_RELU>(ta, tb, td, p, grid, stream);
        case BLAZE_ACT_GELU_TANH: return launch_mx_instance<kBN, ACT_GELU_TANH>(ta, tb, td, p, grid, stream);
        case BLAZE_ACT_SILU: return launch_mx_instance<kBN, ACT_SILU>(ta, tb, td, p, grid, stream);
        case BLAZE_ACT_SIGMOID: return launch_mx_instance<kBN, ACT_SIGMOID>(ta, tb, td, p, grid, stream);
        case BLAZE_ACT_TANH: return launch_mx_instance<kBN, ACT_TANH>(ta, tb, td, p, grid, stream);
        default: return launch_mx_instance<kBN, ACT_IDENTITY>(ta, tb, td, p, grid, stream);
    }
}

// Row-major matrix of 512-byte scale-factor blocks, loaded `box_rows` blocks at a time, no swizzle.
static bool make_tmap_sf_blocks(CUtensorMap* map, const void* base, uint64_t blocks, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {128, blocks};                 // 128 x 4-byte words per block
    const cuuint64_t strides[1] = {512};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
                          elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int kBN, int kAct, bool kWide, bool kMxf4 = false>
static cudaError_t launch_mx_pair_instance(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa,
                                           const CUtensorMap& tsb, const CUtensorMap& td, const MxGemmParams& p,
                                           int pairs, cudaStream_t stream) {
    constexpr int kStages = kWide ? 5 : 6;           // the replicated scale block costs a stage of shared memory
    using L = MxPairSmem<kBN, kStages, kWide, kMxf4>;
    auto kernel = mx_gemm_pair_kernel<kBN, kStages, kAct, kWide, kMxf4>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev & 63] = true;
    }
    // cluster of 2 set on the kernel
    return launch_after_prepass(kernel, 2 * pairs, 192, L::kDynamicBytes, stream, ta, tb, tsa, tsb, td, p);
}

template <int kBN, bool kWide, bool kMxf4 = false>
static cudaError_t launch_mx_pair_act(int act, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa,
                                      const CUtensorMap& tsb, const CUtensorMap& td, const MxGemmParams& p, int pairs,
                                      cudaStream_t stream) {
    switch (act) {
        case BLAZE_ACT_RELU: return launch_mx_pair_instance<kBN, ACT_RELU, kWide, kMxf4>(ta, tb, tsa, tsb, td, p, pairs, stream);
        case BLAZE_ACT_GELU_TANH: return launch_mx_pair_instance<kBN, ACT_GELU_TANH, kWide, kMxf4>(ta, tb, tsa, tsb, td, p, pairs, stream);
        case BLAZE_ACT_SILU: return launch_mx_pair_instance<kBN, ACT_SILU, kWide, kMxf4>(ta, tb, tsa, tsb, td, p, pairs, stream);
        case BLAZE_ACT_SIGMOID: return launch_mx_pair_instance<kBN, ACT_SIGMOID, kWide, kMxf4>(ta, tb, tsa, tsb, td, p, pairs, stream);
        case BLAZE_ACT_TANH: return launch_mx_pair_instance<kBN, ACT_TANH, kWide, kMxf4>(ta, tb, tsa, tsb, td, p, pairs, stream);
        default: return launch_mx_pair_instance<kBN, ACT_IDENTITY, kWide, kMxf4>(ta, tb, tsa, tsb, td, p, pairs, stream);
    }
}

// Encodes the tensor maps and launches the GEMM kernel the plan chose.  `sfa_tiled` / `sfb_tiled` hold the re-tiled
// scales, `b_codes` the 8-bit B operand (the caller's, or the expansion of a packed E2M1 one).
// `b_packed4`: b_codes is the caller's packed E2M1 operand and `tb_packed` its tensor map (built by the caller, who
// had to know whether the encoder accepts it before choosing between this and the expansion pre-pass).
static int run_mx_kernel(const blazeMxGemmArgs* a, const MxPlan& pl, const uint8_t* sfa_tiled, const uint8_t* sfb_tiled,
                         const uint8_t* b_codes, int64_t b_pitch, int* status_word, int sm_count,
                         cudaStream_t stream, const CUtensorMap* tb_packed = nullptr,
                         const CUtensorMap* ta_packed = nullptr) {
    MxGemmParams p;
    p.M = a->M; p.N = a->N; p.K = a->K;
    p.m_tiles = pl.m_tiles; p.n_tiles = pl.n_tiles; p.k_steps = pl.k_steps;
    p.sf_k_steps = pl.sf_k_steps;
    p.window = pl.pair ? (pl.m_tiles < 8 ? pl.m_tiles : 8) : (pl.m_tiles < 16 ? pl.m_tiles : 16);
    p.sfa_tiled = sfa_tiled;
    p.sfb_tiled = sfb_tiled;
    p.bias = static_cast<const __nv_bfloat16*>(a->bias);
    p.residual = static_cast<const __nv_bfloat16*>(a->residual);
    p.ldr = a->ldr;
    p.D = static_cast<__nv_bfloat16*>(a->D);
    p.ldd = a->ldd;
    p.status = status_word;
    // one-byte codes are E4M3 or E5M2 as the caller says (an expanded E2M1 weight holds E4M3 codes)
    p.b_format = tb_packed ? FMT_E2M1 : (a->b_elem == BLAZE_ELEM_E5M2 ? FMT_E5M2 : FMT_E4M3);
    p.b_tx_shift = tb_packed ? 1 : 0;        // a 4-bit load reports the bytes it read, not the bytes it wrote
    p.stream_k = pl.stream_k ? 1 : 0;
    p.flags = pl.stream_k ? reinterpret_cast<int*>(static_cast<uint8_t*>(a->workspace) + pl.flags_off) : nullptr;
    p.partials = pl.stream_k ? reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + pl.partials_off) : nullptr;
    p.out_type = a->d_type;
    p.scale_d = static_cast<uint8_t*>(a->scaleD);
    p.scale_cols_d = ((a->N + 63) / 64) * 2;
    if (a->d_type == BLAZE_OUT_MX_E4M3 && (!a->scaleD || (a->ldd % 16) != 0)) return ACLTENSOR_STATUS_INVALID_VALUE;
    p.a_format = ta_packed ? FMT_E2M1 : (a->a_elem == BLAZE_ELEM_E5M2 ? FMT_E5M2 : FMT_E4M3);
    p.a_tx_shift = ta_packed ? 1 : 0;
    p.peer_maps = nullptr;
    p.n_peers = 0;
    if (a->n_peers > 0) {
        // one more map of D's shape per peer copy, handed to the kernel through the workspace
        CUtensorMap peer[BLAZE_MAX_PEERS];
        for (int i = 0; i < a->n_peers; ++i) {
            if (!a->peerD[i] || !aligned16(a->peerD[i])) return ACLTENSOR_STATUS_INVALID_VALUE;
            if (!make_tmap_store(&peer[i], a->peerD[i], (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->ldd, a->d_type))
                return ACLTENSOR_STATUS_INTERNAL_ERROR;
        }
        void* dst = static_cast<uint8_t*>(a->workspace) + pl.peer_maps_off;
        cudaError_t ce = cudaMemcpyAsync(dst, peer, sizeof(CUtensorMap) * a->n_peers, cudaMemcpyHostToDevice, stream);
        if (ce != cudaSuccess) return status_of(ce);
        p.peer_maps = static_cast<const CUtensorMap*>(dst);
        p.n_peers = a->n_peers;
    }

    const long long tiles = (long long)pl.m_tiles * pl.n_tiles;
    int sms = sm_count;
    if (a->sm_limit > 0 && a->sm_limit < sms) sms = a->sm_limit;
    CUtensorMap ta, tb, td;
    cudaError_t e;
    if (!make_tmap_store(&td, a->D, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->ldd, a->d_type))
        return ACLTENSOR_STATUS_INTERNAL_ERROR;
    if (pl.pair) {
        CUtensorMap tsa, tsb;
        const uint64_t sfa_blocks = (uint64_t)((a->M + 127) / 128) * pl.sf_k_steps;
        const uint64_t sfb_blocks = (uint64_t)pl.n_tiles * pl.sf_k_steps * 2 * pl.sfb_replicas;
        const uint64_t k_bytes = pl.mxf4 ? (uint64_t)a->K / 2 : (uint64_t)a->K;      // dense 4-bit rows for kind::mxf4
        const uint32_t sf_per_stage = pl.mxf4 ? 2 : 1;
        if (!(ta_packed || make_tmap_bytes(&ta, a->A, k_bytes, (uint64_t)a->M, (uint64_t)a->lda, 128)) ||
            !(tb_packed || make_tmap_bytes(&tb, b_codes, k_bytes, (uint64_t)a->N, (uint64_t)b_pitch, (uint32_t)pl.tile_n / 2)) ||
            !make_tmap_sf_blocks(&tsa, sfa_tiled, sfa_blocks, sf_per_stage) ||
            !make_tmap_sf_blocks(&tsb, sfb_tiled, sfb_blocks, 2 * pl.sfb_replicas * sf_per_stage))
            return ACLTENSOR_STATUS_INTERNAL_ERROR;
        if (tb_packed) tb = *tb_packed;
        if (ta_packed) ta = *ta_packed;
        int pairs = sms / 2;
        if (pairs < 1) pairs = 1;
        if (tiles < pairs && !pl.stream_k) pairs = (int)tiles;      // a split last round uses every pair
        const bool wide = pl.sfb_replicas == 4;
        if (pl.mxf4) {
            e = launch_mx_pair_act<256, true, true>(a->activation, ta, tb, tsa, tsb, td, p, pairs, stream);
        } else if (pl.tile_n == 256) {
            e = wide ? launch_mx_pair_act<256, true>(a->activation, ta, tb, tsa, tsb, td, p, pairs, stream)
                     : launch_mx_pair_act<256, false>(a->activation, ta, tb, tsa, tsb, td, p, pairs, stream);
        } else {
            e = wide ? launch_mx_pair_act<224, true>(a->activation, ta, tb, tsa, tsb, td, p, pairs, stream)
                     : launch_mx_pair_act<224, false>(a->activation, ta, tb, tsa, tsb, td, p, pairs, stream);
        }
        return status_of(e);
    }
    if (!(ta_packed || make_tmap_bytes(&ta, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->lda, 128)) ||
        !(tb_packed || make_tmap_bytes(&tb, b_codes, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)b_pitch, (uint32_t)pl.tile_n)))
        return ACLTENSOR_STATUS_INTERNAL_ERROR;
    if (tb_packed) tb = *tb_packed;
    if (ta_packed) ta = *ta_packed;
    const int grid = pl.grid;
    if (pl.tile_n == 224)
        e = launch_mx_act<224>(a->activation, ta, tb, td, p, grid, stream);
    else
        e = launch_mx_act<128>(a->activation, ta, tb, td, p, grid, stream);
    return status_of(e);
}

}  // namespace blaze

using namespace blaze;

extern "C" int blazeMxGemmWorkspaceSize(const blazeMxGemmArgs* args, size_t* bytes) {
    if (!bytes) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    const int sms = ctx ? ctx->sm_count : 148;
    MxPlan pl;
    const int st = plan_mx(args, sms, &pl);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    *bytes = pl.total;
    return ACLTENSOR_STATUS_SUCCESS;
}

extern "C" int blazeMxGemm(const blazeMxGemmArgs* a, void* stream_v) {
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    if (ctx->cc_major != 10) return ACLTENSOR_STATUS_ARCH_MISMATCH;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    MxPlan pl;
    int st = plan_mx(a, ctx->sm_count, &pl);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    if (a->M == 0 || a->N == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!a->A || !a->B || !a->scaleA || !a->scaleB || !a->D) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->K == 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const int64_t min_ldb = a->b_layout == BLAZE_B_N_MAJOR ? a->N : (a->b_elem == BLAZE_ELEM_E2M1 ? a->K / 2 : a->K);
    const int64_t min_lda = a->a_elem == BLAZE_ELEM_E2M1 ? a->K / 2 : a->K;
    if (a->lda < min_lda || a->ldb < min_ldb || a->ldd < a->N || (a->residual && a->ldr < a->N))
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if ((a->lda % 16) || (a->ldb % 16) || (a->ldd % 8) || (a->residual && (a->ldr % 8)))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (!aligned16(a->A) || !aligned16(a->B) || !aligned16(a->D) || !aligned16(a->bias) || !aligned16(a->residual))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->b_elem == BLAZE_ELEM_E2M1 && (a->ldb % 8)) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (pl.total > 0 && (!a->workspace || a->workspace_bytes < pl.total)) return ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return ACLTENSOR_STATUS_INVALID_VALUE;

    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    uint8_t* sfa_tiled = ws + pl.sfa_off;
    uint8_t* sfb_tiled = ws + pl.sfb_off;
    const uint8_t* b_codes = static_cast<const uint8_t*>(a->B);
    int64_t b_pitch = a->ldb;

    // the kernel that re-tiles A's scales runs on every call: it also clears the stream-K fix-up flags, which the GEMM
    // expects at zero and which still hold the previous call's marks (or whatever the workspace held before)
    cudaError_t e = launch_sf_retile(static_cast<const uint8_t*>(a->scaleA), a->M, a->K, 128, 1, sfa_tiled, ctx->sm_count,
                                     stream, pl.stream_k ? reinterpret_cast<int*>(ws + pl.flags_off) : nullptr,
                                     (int)(pl.flags_bytes / 4));
    if (e != cudaSuccess) return status_of(e);
    // A packed E2M1 weight is fed to the tensor core as it is when TMA can unpack it (whole 128-code boxes along K,
    // 32-byte aligned rows); otherwise it is expanded once to one-byte E4M3 codes of the same values.
    if (pl.mxf4) {
        // FP4 x FP4 at the double rate: both operands stay packed, plain byte loads, kind::mxf4
        if (!a->reuse_b_prepass) {
            e = launch_sf_retile(static_cast<const uint8_t*>(a->scaleB), a->N, a->K, pl.tile_n, pl.sfb_replicas, sfb_tiled,
                                 ctx->sm_count, stream);
            if (e != cudaSuccess) return status_of(e);
        }
        return run_mx_kernel(a, pl, sfa_tiled, sfb_tiled, b_codes, b_pitch, ctx->status_word, ctx->sm_count, stream);
    }
    CUtensorMap tb_packed;
    bool native4 = false;
    if (a->b_elem == BLAZE_ELEM_E2M1 && (a->K % 128) == 0 && (a->ldb % 32) == 0 &&
        (reinterpret_cast<uintptr_t>(a->B) & 31) == 0) {
        native4 = make_tmap_packed4(&tb_packed, a->B, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->ldb,
                                    (uint32_t)(pl.pair ? pl.tile_n / 2 : pl.tile_n));
    }
    CUtensorMap ta_packed;
    if (a->a_elem == BLAZE_ELEM_E2M1) {
        // FP4 x FP4: both operands must take the native route
        if (!native4 || (a->lda % 32) != 0 || (reinterpret_cast<uintptr_t>(a->A) & 31) != 0 ||
            !make_tmap_packed4(&ta_packed, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->lda, 128))
            return ACLTENSOR_STATUS_NOT_SUPPORTED;
    }
    if ((a->b_elem == BLAZE_ELEM_E2M1 && !native4) || a->b_layout == BLAZE_B_N_MAJOR) {
        b_codes = ws + pl.b_expand_off;
        b_pitch = a->K;
    }
    if (!a->reuse_b_prepass) {
        const uint8_t* scale_b_rows = static_cast<const uint8_t*>(a->scaleB);
        if (a->b_layout == BLAZE_B_N_MAJOR) {
            // B arrives [K][N]: keep a K-major copy and row-major scales in the workspace (once per weight)
            e = launch_transpose_bytes(static_cast<const uint8_t*>(a->B), a->ldb, a->K, a->N, ws + pl.b_expand_off, a->K,
                                       stream);
            if (e != cudaSuccess) return status_of(e);
            e = launch_scale_pairs_to_rows(scale_b_rows, a->N, a->K, ws + pl.b_scale_rows_off, ctx->sm_count, stream);
            if (e != cudaSuccess) return status_of(e);
            scale_b_rows = ws + pl.b_scale_rows_off;
        }
        e = launch_sf_retile(scale_b_rows, a->N, a->K, pl.tile_n, pl.sfb_replicas, sfb_tiled, ctx->sm_count,
                             stream);
        if (e != cudaSuccess) return status_of(e);
        if (a->b_elem == BLAZE_ELEM_E2M1 && !native4) {
            e = launch_e2m1_expand(static_cast<const uint8_t*>(a->B), a->ldb, a->N, a->K, ws + pl.b_expand_off, a->K,
                                   ctx->sm_count, stream);
            if (e != cudaSuccess) return status_of(e);
        }
    }

    return run_mx_kernel(a, pl, sfa_tiled, sfb_tiled, b_codes, b_pitch, ctx->status_word, ctx->sm_count, stream,
                         native4 ? &tb_packed : nullptr, a->a_elem == BLAZE_ELEM_E2M1 ? &ta_packed : nullptr);
}

// ------------------------------------------------------------------------------------------------ batched MX GEMM

namespace blaze {

struct BatchWalk {
    long long count_c, count_a, count_b;
    bool folds;          // all batches are rows of one GEMM
};

static int check_batch(const blazeMxGemmArgs* a, const blazeBatchDims* bd, BatchWalk* w) {
    if (!a || !bd || a->struct_size != sizeof(blazeMxGemmArgs)) return ACLTENSOR_STATUS_INVALID_VALUE;
    w->count_c = w->count_a = w->count_b = 1;
    bool a_full = true, b_one = true;
    for (int i = 0; i < 4; ++i) {
        if (bd->c[i] < 1 || bd->a[i] < 1 || bd->b[i] < 1) return ACLTENSOR_STATUS_INVALID_VALUE;
        if ((bd->a[i] != bd->c[i] && bd->a[i] != 1) || (bd->b[i] != bd->c[i] && bd->b[i] != 1))
            return ACLTENSOR_STATUS_INVALID_VALUE;
        w->count_c *= bd->c[i];
        w->count_a *= bd->a[i];
        w->count_b *= bd->b[i];
        a_full = a_full && bd->a[i] == bd->c[i];
        b_one = b_one && bd->b[i] == 1;
    }
    if (w->count_c > 0x7fffffffLL) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->b_layout != BLAZE_B_K_MAJOR && w->count_b > 1) return ACLTENSOR_STATUS_NOT_SUPPORTED;   // batches of B are K-major
    // one tall GEMM: same weight for every batch, one A per batch, one bias, rows of consecutive batches adjacent
    w->folds = a_full && b_one && !bd->bias_per_batch && w->count_c * (long long)a->M <= 0x7fffffffLL;
    return ACLTENSOR_STATUS_SUCCESS;
}

}  // namespace blaze

extern "C" int blazeMxGemmBatchedWorkspaceSize(const blazeMxGemmArgs* args, const blazeBatchDims* batch, size_t* bytes) {
    if (!bytes) return ACLTENSOR_STATUS_INVALID_VALUE;
    BatchWalk w;
    const int st = check_batch(args, batch, &w);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    blazeMxGemmArgs one = *args;
    if (w.folds) one.M = (int32_t)(w.count_c * args->M);
    return blazeMxGemmWorkspaceSize(&one, bytes);
}

extern "C" int blazeMxGemmBatched(const blazeMxGemmArgs* args, const blazeBatchDims* bd, void* stream) {
    BatchWalk w;
    int st = check_batch(args, bd, &w);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    if (args->n_peers != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;      // peer copies belong to the plain call
    blazeMxGemmArgs one = *args;
    if (w.folds) {
        one.M = (int32_t)(w.count_c * args->M);
        return blazeMxGemm(&one, stream);
    }
    const int64_t scale_cols = ((int64_t)(args->K + 63) / 64) * 2;
    const int64_t a_bytes = (int64_t)args->M * args->lda, sa_bytes = (int64_t)args->M * scale_cols;
    const int64_t b_bytes = (int64_t)args->N * args->ldb, sb_bytes = (int64_t)args->N * scale_cols;
    // D's element size follows its type; a quantised D also advances its scale rows batch by batch
    const int64_t d_elem = args->d_type == BLAZE_OUT_F32 ? 4 : (args->d_type == BLAZE_OUT_MX_E4M3 ? 1 : 2);
    const int64_t d_bytes = (int64_t)args->M * args->ldd * d_elem, r_bytes = (int64_t)args->M * args->ldr * 2;
    const int64_t sd_bytes = (int64_t)args->M * (((int64_t)args->N + 63) / 64) * 2;
    // strides of the operands' own batch spaces, innermost dimension last
    long long stride_a[4], stride_b[4];
    long long sa = 1, sb = 1;
    for (int i = 3; i >= 0; --i) {
        stride_a[i] = bd->a[i] == 1 ? 0 : sa;
        stride_b[i] = bd->b[i] == 1 ? 0 : sb;
        sa *= bd->a[i];
        sb *= bd->b[i];
    }
    long long last_ib = -1;
    long long ic = 0;
    for (int i0 = 0; i0 < bd->c[0]; ++i0)
        for (int i1 = 0; i1 < bd->c[1]; ++i1)
            for (int i2 = 0; i2 < bd->c[2]; ++i2)
                for (int i3 = 0; i3 < bd->c[3]; ++i3, ++ic) {
                    const long long ia = i0 * stride_a[0] + i1 * stride_a[1] + i2 * stride_a[2] + i3 * stride_a[3];
                    const long long ib = i0 * stride_b[0] + i1 * stride_b[1] + i2 * stride_b[2] + i3 * stride_b[3];
                    one.A = static_cast<const uint8_t*>(args->A) + ia * a_bytes;
                    one.scaleA = static_cast<const uint8_t*>(args->scaleA) + ia * sa_bytes;
                    one.B = static_cast<const uint8_t*>(args->B) + ib * b_bytes;
                    one.scaleB = static_cast<const uint8_t*>(args->scaleB) + ib * sb_bytes;
                    one.D = static_cast<uint8_t*>(args->D) + ic * d_bytes;
                    if (args->scaleD) one.scaleD = static_cast<uint8_t*>(args->scaleD) + ic * sd_bytes;
                    if (args->residual) one.residual = static_cast<const uint8_t*>(args->residual) + ic * r_bytes;
                    if (args->bias && bd->bias_per_batch)
                        one.bias = static_cast<const uint8_t*>(args->bias) + ic * (int64_t)args->N * 2;
                    // the workspace keeps the weight's pre-pass of the batch before: reuse it while B stays the same
                    one.reuse_b_prepass = (ib == last_ib || (ic == 0 && args->reuse_b_prepass)) ? 1 : 0;
                    st = blazeMxGemm(&one, stream);
                    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
                    last_ib = ib;
                }
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ FP8 GEMM

namespace blaze {

struct Fp8Plan {
    int m_tiles, n_tiles, k_blocks;
    int grid;
    int stream_k;
    size_t flags_bytes, partial_bytes, total;
};

static int plan_fp8(const blazeFp8GemmArgs* a, int sm_count, Fp8Plan* pl) {
    if (!a || a->struct_size != sizeof(blazeFp8GemmArgs)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->M < 0 || a->N < 0 || a->K < 0 || a->groups < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->groups > kFp8MaxGroups) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->activation < BLAZE_ACT_IDENTITY || a->activation > BLAZE_ACT_TANH) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->n_peers < 0 || a->n_peers > BLAZE_MAX_PEERS) return ACLTENSOR_STATUS_INVALID_VALUE;
    // only the 16-bit output rows leave as bulk copies that can be repeated towards the peers
    if (a->n_peers > 0 && a->d_type != BLAZE_OUT_BF16 && a->d_type != BLAZE_OUT_F16) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->sched < BLAZE_SCHED_AUTO || a->sched > BLAZE_SCHED_STREAM_K) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->d_type != BLAZE_OUT_FP8_128 && (a->d_type < BLAZE_OUT_BF16 || a->d_type > BLAZE_OUT_F32))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if ((a->K % 16) != 0 || (a->N % 8) != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    int sms = sm_count;
    if (a->sm_limit > 0 && a->sm_limit < sms) sms = a->sm_limit;
    pl->n_tiles = (a->N + 127) / 128;
    pl->k_blocks = (a->K + 127) / 128;
    pl->m_tiles = a->groups > 0 ? (a->M + 127) / 128 + a->groups : (a->M + 127) / 128;   // grouped: upper bound
    const long long tiles = (long long)pl->m_tiles * pl->n_tiles;
    int stream_k = 0;
    long long split_grid = 0;
    if (a->groups == 0 && tiles > 0 && pl->k_blocks >= 2) {
        // Cost of the schedules in units of one K block on one SM (about 0.34 us).  Whole tiles: rounds x K blocks.
        // Split along K: the evenly split units, plus a fixed cost (partial tiles through L2, the hand-over marks) and
        // 2.8 blocks (~0.9 us) for every other CTA of its tile whose 64 KB partial tile the owner reads and adds
        // (measured on 7 tiles of 144 blocks, M = 128: cut 2 / 4 / 8 / 16 / 21 ways 30.8 / 21.3 / 18.9 / 22.9 / 27.1 us;
        // the marks of all contributors are polled side by side, so the walk costs the reads only).  So the number
        // of CTAs is chosen too: every tile cut into s equal K ranges (s * tiles CTAs) for the s that costs least, or
        // all SMs.
        const long long units = tiles * pl->k_blocks;
        const double whole_tiles = (double)((tiles + sms - 1) / sms) * pl->k_blocks;
        long long best_grid = units < sms ? units : sms;
        double best = (double)((units + best_grid - 1) / best_grid) + 17.0 + 2.8 * ((double)best_grid / (double)tiles);
        for (long long s_cut = 2; s_cut * tiles <= sms && s_cut <= pl->k_blocks; ++s_cut) {
            const double c = (double)((pl->k_blocks + s_cut - 1) / s_cut) + 15.0 + 2.8 * (double)(s_cut - 1);
            if (c < best) {
                best = c;
                best_grid = s_cut * tiles;
            }
        }
        if (a->sched == BLAZE_SCHED_STREAM_K || (a->sched == BLAZE_SCHED_AUTO && best < whole_tiles)) {
            stream_k = 1;
            split_grid = best_grid;
        }
    }
    if (a->groups > 0 && tiles > 0 && pl->k_blocks >= 2 && a->sched != BLAZE_SCHED_DATA_PARALLEL) {
        // grouped: the tile count depends on the group list, which lives on the device; the kernel applies the same
        // cost model itself unless the caller forces the split
        stream_k = a->sched == BLAZE_SCHED_STREAM_K ? 1 : 2;
    }
    pl->stream_k = stream_k;
    long long grid = tiles < sms ? tiles : sms;
    if (stream_k) {
        const long long units = tiles * pl->k_blocks;
        grid = split_grid > 0 ? split_grid : (units < sms ? units : sms);
    }
    if (grid < 1) grid = 1;
    pl->grid = (int)grid;
    pl->flags_bytes = stream_k ? round256((size_t)grid * sizeof(unsigned long long)) : 0;
    pl->partial_bytes = stream_k ? (size_t)grid * 128 * 128 * sizeof(float) : 0;
    pl->total = pl->flags_bytes + pl->partial_bytes;
    return ACLTENSOR_STATUS_SUCCESS;
}

// A value for the stream-K hand-over marks that no earlier launch of this process has used: a per-process random
// high word (so bytes left in a workspace by anything else cannot match) over a launch counter that skips zero.
static unsigned long long next_stream_k_epoch() {
    static const unsigned long long nonce = []() {
        std::random_device rd;
        unsigned long long n = (static_cast<unsigned long long>(rd()) << 32) ^ static_cast<unsigned long long>(
                                   std::chrono::steady_clock::now().time_since_epoch().count());
        return (n | (1ull << 63)) & 0xFFFFFFFF00000000ull;
    }();
    static std::atomic<uint32_t> counter{0};
    uint32_t c = counter.fetch_add(1) + 1;
    if (c == 0) c = counter.fetch_add(1) + 1;
    return nonce | c;
}

template <int kAct, int kStages>
static cudaError_t launch_fp8_stages(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                                     const Fp8PeerMaps& pm, const Fp8GemmParams& p, int grid, cudaStream_t stream) {
#ifndef LAB_ISSUERS
#define LAB_ISSUERS 2
#endif
    constexpr int kIssuers = LAB_ISSUERS;
    using L = Fp8GemmSmem<kStages>;
    static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory per CTA");
    auto kernel = fp8_gemm_kernel<kStages, kAct, kIssuers>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev & 63] = true;
    }
    // behind whatever precedes it in the stream (the kernel that zeroes the fix-up flags, or the previous GEMM): set-up
    // overlaps that kernel's tail, every thread waits for it before the role loops start
    return launch_after_prepass(kernel, grid, 288 + 32 * kIssuers, L::kDynamicBytes, stream, ta, tb, td, pm, p);
}

template <int kAct>
static cudaError_t launch_fp8_instance(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                                       const Fp8PeerMaps& pm, const Fp8GemmParams& p, int grid, cudaStream_t stream) {
    // One tcgen05.commit per K block serves the accumulator ring (4 TMEM stages) and the operand ring.  Two MMA-issuing
    // threads take the K blocks in turn.  Operand stages: 5 when the weights are streamed once by a single row of
    // tiles (decode, C5: 36.7 -> 35.7 us), else 4 (grouped C4: 115 us with 4, 118 us with 5 - those shapes are bound
    // by the L2 -> shared-memory traffic of 128x128 tiles, 32 KB per K block, not by load latency).
    if (p.groups == 0 && p.m_tiles == 1) return launch_fp8_stages<kAct, 5>(ta, tb, td, pm, p, grid, stream);
    return launch_fp8_stages<kAct, 4>(ta, tb, td, pm, p, grid, stream);
}

}  // namespace blaze

extern "C" int blazeFp8GemmWorkspaceSize(const blazeFp8GemmArgs* args, size_t* bytes) {
    if (!bytes) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    Fp8Plan pl;
    const int st = plan_fp8(args, ctx ? ctx->sm_count : 148, &pl);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    *bytes = pl.total;
    return ACLTENSOR_STATUS_SUCCESS;
}

extern "C" int blazeFp8Gemm(const blazeFp8GemmArgs* a, void* stream_v) {
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    if (ctx->cc_major != 10) return ACLTENSOR_STATUS_ARCH_MISMATCH;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    Fp8Plan pl;
    int st = plan_fp8(a, ctx->sm_count, &pl);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    if (a->M == 0 || a->N == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!a->A || !a->B || !a->scaleA || !a->scaleB || !a->D) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->groups > 0 && !a->group_rows) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->K == 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->lda < a->K || a->ldb < a->K || a->ldd < a->N || (a->residual && a->ldr < a->N))
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if ((a->lda % 16) || (a->ldb % 16) || (a->ldd % 8) || (a->residual && (a->ldr % 8)))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (!aligned16(a->A) || !aligned16(a->B) || !aligned16(a->D) || !aligned16(a->bias) || !aligned16(a->residual))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (pl.total > 0 && (!a->workspace || a->workspace_bytes < pl.total)) return ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE;
    if (pl.total > 0 && (reinterpret_cast<uintptr_t>(a->workspace) & 255)) return ACLTENSOR_STATUS_INVALID_VALUE;

    const int groups = a->groups;
    const uint64_t b_rows = (uint64_t)(groups > 0 ? groups : 1) * (uint64_t)a->N;
    CUtensorMap ta, tb, td;
    // (the store map is used for 16-bit outputs only; the other output types get a valid map of their own shape)
    const int td_type = a->d_type == BLAZE_OUT_FP8_128 ? BLAZE_OUT_MX_E4M3 : a->d_type;
    if (!make_tmap_bytes(&ta, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->lda, 128) ||
        !make_tmap_bytes(&tb, a->B, (uint64_t)a->K, b_rows, (uint64_t)a->ldb, 128) ||
        !make_tmap_store(&td, a->D, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->ldd, td_type))
        return ACLTENSOR_STATUS_INTERNAL_ERROR;

    Fp8GemmParams p;
    p.M = a->M; p.N = a->N; p.K = a->K;
    p.n_tiles = pl.n_tiles; p.k_blocks = pl.k_blocks;
    p.m_tiles = (a->M + 127) / 128;
    p.window = p.m_tiles < 8 ? p.m_tiles : 8;
    if (p.window < 1) p.window = 1;
    p.groups = groups;
    p.group_rows = static_cast<const long long*>(a->group_rows);
    p.sa = static_cast<const float*>(a->scaleA);
    p.sb = static_cast<const float*>(a->scaleB);
    p.n_blocks = (a->N + 127) / 128;
    p.bias = static_cast<const __nv_bfloat16*>(a->bias);
    p.residual = static_cast<const __nv_bfloat16*>(a->residual);
    p.ldr = a->ldr;
    p.D = static_cast<__nv_bfloat16*>(a->D);
    p.ldd = a->ldd;
    p.out_type = a->d_type;
    p.scale_d = static_cast<float*>(a->scaleD);
    if (a->d_type == BLAZE_OUT_FP8_128 && (!a->scaleD || (a->ldd % 16) != 0)) return ACLTENSOR_STATUS_INVALID_VALUE;
    p.n_peers = a->n_peers;
    Fp8PeerMaps pm;
    std::memset(&pm, 0, sizeof(pm));
    for (int i = 0; i < BLAZE_MAX_PEERS; ++i) {
        p.peer_d[i] = i < a->n_peers ? static_cast<uint8_t*>(a->peerD[i]) : nullptr;
        if (i < a->n_peers && (!a->peerD[i] || !aligned16(a->peerD[i]))) return ACLTENSOR_STATUS_INVALID_VALUE;
        // the tiled output copies reach a peer through its own tensor map (same shape, pitch and type as D)
        if (i < a->n_peers &&
            !make_tmap_store(&pm.m[i], a->peerD[i], (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->ldd, a->d_type))
            return ACLTENSOR_STATUS_INTERNAL_ERROR;
    }
    p.stream_k = pl.stream_k;
    p.flags = nullptr;
    p.partials = nullptr;
    p.status = ctx->status_word;
    p.epoch = 0;
    p.b_static = a->b_is_static != 0 ? 1 : 0;
    if (pl.stream_k) {
        p.flags = static_cast<unsigned long long*>(a->workspace);
        p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + pl.flags_bytes);
        p.epoch = next_stream_k_epoch();
    }
    cudaError_t e;
    switch (a->activation) {
        case BLAZE_ACT_RELU: e = launch_fp8_instance<ACT_RELU>(ta, tb, td, pm, p, pl.grid, stream); break;
        case BLAZE_ACT_GELU_TANH: e = launch_fp8_instance<ACT_GELU_TANH>(ta, tb, td, pm, p, pl.grid, stream); break;
        case BLAZE_ACT_SILU: e = launch_fp8_instance<ACT_SILU>(ta, tb, td, pm, p, pl.grid, stream); break;
        case BLAZE_ACT_SIGMOID: e = launch_fp8_instance<ACT_SIGMOID>(ta, tb, td, pm, p, pl.grid, stream); break;
        case BLAZE_ACT_TANH: e = launch_fp8_instance<ACT_TANH>(ta, tb, td, pm, p, pl.grid, stream); break;
        default: e = launch_fp8_instance<ACT_IDENTITY>(ta, tb, td, pm, p, pl.grid, stream); break;
    }
    return status_of(e);
}

// ------------------------------------------------------------------------------------------------ unscaled GEMMs

namespace blaze {

template <int kKind, int kAct>
static cudaError_t launch_dense_instance(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                                         const DenseGemmParams& p, int pairs, cudaStream_t stream) {
    constexpr int kStages = 6;
    using L = DensePairSmem<kStages>;
    static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory per CTA");
    auto kernel = dense_gemm_pair_kernel<kKind, kStages, kAct>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev & 63] = true;
    }
    return launch_after_prepass(kernel, 2 * pairs, 192, L::kDynamicBytes, stream, ta, tb, td, p);
}

template <int kKind>
static cudaError_t launch_dense_act(int act, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                                    const DenseGemmParams& p, int pairs, cudaStream_t stream) {
    switch (act) {
        case BLAZE_ACT_RELU: return launch_dense_instance<kKind, ACT_RELU>(ta, tb, td, p, pairs, stream);
        case BLAZE_ACT_GELU_TANH: return launch_dense_instance<kKind, ACT_GELU_TANH>(ta, tb, td, p, pairs, stream);
        case BLAZE_ACT_SILU: return launch_dense_instance<kKind, ACT_SILU>(ta, tb, td, p, pairs, stream);
        case BLAZE_ACT_SIGMOID: return launch_dense_instance<kKind, ACT_SIGMOID>(ta, tb, td, p, pairs, stream);
        case BLAZE_ACT_TANH: return launch_dense_instance<kKind, ACT_TANH>(ta, tb, td, p, pairs, stream);
        default: return launch_dense_instance<kKind, ACT_IDENTITY>(ta, tb, td, p, pairs, stream);
    }
}

}  // namespace blaze

extern "C" int blazeDenseGemm(const blazeDenseGemmArgs* a, void* stream_v) {
    if (!a || a->struct_size != sizeof(blazeDenseGemmArgs)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->M < 0 || a->N < 0 || a->K < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->kind < BLAZE_DENSE_S8 || a->kind > BLAZE_DENSE_BF16) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->activation < BLAZE_ACT_IDENTITY || a->activation > BLAZE_ACT_TANH) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->scale_mode < BLAZE_DENSE_SCALE_NONE || a->scale_mode > BLAZE_DENSE_SCALE_PER_CHANNEL)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    const bool s8 = a->kind == BLAZE_DENSE_S8;
    if (!s8 && a->scale_mode != BLAZE_DENSE_SCALE_NONE) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const bool raw = a->d_type == BLAZE_OUT_S32;
    if (!raw && (a->d_type < BLAZE_OUT_BF16 || a->d_type > BLAZE_OUT_F32)) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    // raw int32 sums: INT8 only, nothing that would touch them as floats
    if (raw && (!s8 || a->scale_mode != BLAZE_DENSE_SCALE_NONE || a->activation != BLAZE_ACT_IDENTITY || a->residual))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const int64_t esize = s8 ? 1 : 2;
    if (((int64_t)a->K * esize) % 16 != 0 || (a->N % 8) != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    if (ctx->cc_major != 10) return ACLTENSOR_STATUS_ARCH_MISMATCH;
    if (a->M == 0 || a->N == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!a->A || !a->B || !a->D) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->K == 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->scale_mode == BLAZE_DENSE_SCALE_PER_TENSOR && (!a->scaleA || !a->scaleB)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->scale_mode == BLAZE_DENSE_SCALE_PER_CHANNEL && !a->scaleN) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->lda < a->K || a->ldb < a->K || a->ldd < a->N || (a->residual && a->ldr < a->N))
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if (((a->lda * esize) % 16) || ((a->ldb * esize) % 16) || (a->ldd % 8) || (a->residual && (a->ldr % 8)))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (!aligned16(a->A) || !aligned16(a->B) || !aligned16(a->D) || !aligned16(a->bias) || !aligned16(a->residual))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    DenseGemmParams p;
    p.M = a->M; p.N = a->N; p.K = a->K;
    p.m_tiles = (a->M + 255) / 256;
    p.n_tiles = (a->N + 255) / 256;
    p.k_steps = (int)(((int64_t)a->K * esize + 127) / 128);
    p.window = p.m_tiles < 8 ? p.m_tiles : 8;
    p.scale_mode = a->scale_mode;
    p.scale_a = static_cast<const float*>(a->scaleA);
    p.scale_b = static_cast<const float*>(a->scaleB);
    p.scale_n = static_cast<const unsigned long long*>(a->scaleN);
    p.bias_i32 = s8 ? static_cast<const int*>(a->bias) : nullptr;
    p.bias = s8 ? nullptr : static_cast<const __nv_bfloat16*>(a->bias);
    p.residual = static_cast<const __nv_bfloat16*>(a->residual);
    p.ldr = a->ldr;
    p.out_type = a->d_type;
    p.status = ctx->status_word;

    // operands as rows of bytes (a K block is 128 bytes for either element size); D by its own element type
    CUtensorMap ta, tb, td;
    if (!make_tmap_bytes(&ta, a->A, (uint64_t)a->K * esize, (uint64_t)a->M, (uint64_t)a->lda * esize, 128) ||
        !make_tmap_bytes(&tb, a->B, (uint64_t)a->K * esize, (uint64_t)a->N, (uint64_t)a->ldb * esize, 128) ||
        !make_tmap_store(&td, a->D, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->ldd, raw ? BLAZE_OUT_F32 : a->d_type))
        return ACLTENSOR_STATUS_INTERNAL_ERROR;
    int sms = ctx->sm_count;
    if (a->sm_limit > 0 && a->sm_limit < sms) sms = a->sm_limit;
    int pairs = sms / 2 > 0 ? sms / 2 : 1;
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles < pairs) pairs = (int)tiles;
    cudaError_t e;
    if (a->kind == BLAZE_DENSE_S8) e = launch_dense_act<DENSE_S8>(a->activation, ta, tb, td, p, pairs, stream);
    else if (a->kind == BLAZE_DENSE_F16) e = launch_dense_act<DENSE_F16>(a->activation, ta, tb, td, p, pairs, stream);
    else e = launch_dense_act<DENSE_BF16>(a->activation, ta, tb, td, p, pairs, stream);
    return status_of(e);
}

// ------------------------------------------------------------------------------------------------ quantisers & misc

namespace blaze {
struct EventTimer {
    cudaEvent_t begin, end;
};
}  // namespace blaze

extern "C" int blazeTimerCreate(void** timer) {
    if (!timer) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (!current_context()) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    EventTimer* t = new (std::nothrow) EventTimer();
    if (!t) return ACLTENSOR_STATUS_ALLOC_FAILED;
    if (cudaEventCreate(&t->begin) != cudaSuccess) { delete t; return ACLTENSOR_STATUS_INTERNAL_ERROR; }
    if (cudaEventCreate(&t->end) != cudaSuccess) { cudaEventDestroy(t->begin); delete t; return ACLTENSOR_STATUS_INTERNAL_ERROR; }
    *timer = t;
    return ACLTENSOR_STATUS_SUCCESS;
}

extern "C" int blazeTimerStart(void* timer, void* stream) {
    if (!timer) return ACLTENSOR_STATUS_INVALID_VALUE;
    return status_of(cudaEventRecord(static_cast<EventTimer*>(timer)->begin, static_cast<cudaStream_t>(stream)));
}

extern "C" int blazeTimerStop(void* timer, void* stream, float* milliseconds) {
    if (!timer || !milliseconds) return ACLTENSOR_STATUS_INVALID_VALUE;
    EventTimer* t = static_cast<EventTimer*>(timer);
    cudaError_t e = cudaEventRecord(t->end, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaEventSynchronize(t->end);
    if (e == cudaSuccess) e = cudaEventElapsedTime(milliseconds, t->begin, t->end);
    return status_of(e);
}

extern "C" int blazeTimerDestroy(void* timer) {
    if (!timer) return ACLTENSOR_STATUS_SUCCESS;
    EventTimer* t = static_cast<EventTimer*>(timer);
    cudaEventDestroy(t->begin);
    cudaEventDestroy(t->end);
    delete t;
    return ACLTENSOR_STATUS_SUCCESS;
}

extern "C" int blazeQuantizeMx(const void* x, int64_t ldx, int32_t rows, int32_t K, int32_t elem, void* codes,
                               int64_t ld_codes, void* scales, void* stream) {
    if (rows < 0 || K < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (rows == 0 || K == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!x || !codes || !scales) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (elem < BLAZE_ELEM_E4M3 || elem > BLAZE_ELEM_E5M2) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if ((K % 4) || (ldx % 4) || !aligned16(x)) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    const int64_t min_ld = elem == BLAZE_ELEM_E2M1 ? K / 2 : K;
    if (ldx < K || ld_codes < min_ld) return ACLTENSOR_STATUS_INVALID_VALUE;
    if ((ld_codes % (elem == BLAZE_ELEM_E2M1 ? 2 : 4)) || (reinterpret_cast<uintptr_t>(codes) & 3))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    return status_of(launch_quant_mx(static_cast<const float*>(x), ldx, rows, K, elem,
                                     static_cast<uint8_t*>(codes), ld_codes, static_cast<uint8_t*>(scales),
                                     ctx->sm_count, static_cast<cudaStream_t>(stream)));
}

extern "C" int blazeQuantizeFp8RowGroups(const void* x, int64_t ldx, int32_t rows, int32_t K, void* codes,
                                         int64_t ld_codes, void* scales, void* stream) {
    if (rows < 0 || K < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (rows == 0 || K == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!x || !codes || !scales) return ACLTENSOR_STATUS_INVALID_VALUE;
    if ((K % 4) || (ldx % 4) || (ld_codes % 4) || !aligned16(x) || (reinterpret_cast<uintptr_t>(codes) & 3))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (ldx < K || ld_codes < K) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    return status_of(launch_quant_fp8_1x128(static_cast<const float*>(x), ldx, rows, K, static_cast<uint8_t*>(codes),
                                            ld_codes, static_cast<float*>(scales), ctx->sm_count,
                                            static_cast<cudaStream_t>(stream)));
}

extern "C" int blazeQuantizeFp8Blocks(const void* w, int64_t ldw, int32_t N, int32_t K, void* codes, int64_t ld_codes,
                                      void* scales, void* stream) {
    if (N < 0 || K < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (N == 0 || K == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!w || !codes || !scales) return ACLTENSOR_STATUS_INVALID_VALUE;
    if ((K % 4) || (ldw % 4) || (ld_codes % 4) || !aligned16(w) || (reinterpret_cast<uintptr_t>(codes) & 3))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (ldw < K || ld_codes < K) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    return status_of(launch_quant_fp8_128x128(static_cast<const float*>(w), ldw, N, K, static_cast<uint8_t*>(codes),
                                              ld_codes, static_cast<float*>(scales), ctx->sm_count,
                                              static_cast<cudaStream_t>(stream)));
}

extern "C" int blazeAddF32(const void* A, const void* C, void* D, int64_t n, void* stream) {
    if (n < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (n == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!A || !C || !D) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    return status_of(launch_add_f32(static_cast<const float*>(A), static_cast<const float*>(C), static_cast<float*>(D),
                                    n, ctx->sm_count, static_cast<cudaStream_t>(stream)));
}

namespace blaze {
// Status word of the allocation-free entry point on device `dev` (it lives in the library image, not in the
// context's allocation): 0 if that entry has not run on the device.  Defined with the entry point below.
static int noalloc_status_fetch(int dev, bool reset);
}  // namespace blaze

extern "C" int blazeDeviceStatus(int32_t* value, int32_t reset) {
    if (!value) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    int v = 0;
    if (cudaMemcpy(&v, ctx->status_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return status_of(cudaErrorUnknown);
    if (reset && v != 0) cudaMemset(ctx->status_word, 0, sizeof(int));
    // calls of blazeMxGemmNoAlloc that were given no status pointer report here as well
    const int w = noalloc_status_fetch(ctx->device, reset != 0);
    *value = v != 0 ? v : w;
    return ACLTENSOR_STATUS_SUCCESS;
}

// Diagnostic: one CTA waits, with the given cycle budget, on a barrier that nothing ever signals.  The wait gives
// up, records DEV_TIMEOUT_SELFTEST in the status word and the kernel returns normally: the path a real
// synchronisation failure would take, exercised without hanging or faulting anything.
__global__ void wait_timeout_selftest_kernel(int* status, long long limit_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        blaze::mbar_init(&bar, 1);
        abort_flag = 0;
        blaze::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        blaze::mbar_wait(&bar, 0, &abort_flag, status, blaze::DEV_TIMEOUT_SELFTEST, limit_cycles);
    }
    __syncthreads();
}

extern "C" int blazeSelfTestWaitTimeout(int64_t limit_cycles, void* stream) {
    if (limit_cycles < 0 || limit_cycles > (1LL << 31)) return ACLTENSOR_STATUS_INVALID_VALUE;    // at most ~1 s
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx->status_word, limit_cycles);
    return status_of(cudaGetLastError());
}

// Closing signal of a fused gather: lane q stores `value` into slot `my_rank` of peer q's flag array (release, system
// scope: the GEMM before this kernel in the stream has completed, its stores into the peer's memory with it), then polls
// this GPU's own array for peer q's slot.  Peer stores and local loads only.  The wait is bounded.
struct PeerSignalParams {
    unsigned long long* local_flags;
    unsigned long long* peer_flags[BLAZE_MAX_PEERS];
    int peer_ranks[BLAZE_MAX_PEERS];
    int n_peers;
    int my_rank;
    unsigned long long value;
    long long limit_cycles;
    int* status;
};

__global__ void peer_signal_kernel(const PeerSignalParams p) {
    // launched with programmatic stream serialisation: the next kernel in the stream may set itself up while this one
    // waits for its peers, and this one is resident before the GEMM ahead of it has drained; it signals only after
    // that GEMM has completed
    blaze::grid_launch_dependents();
    blaze::grid_dependency_wait();
    const int q = (int)threadIdx.x;
    if (q >= p.n_peers) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.peer_flags[q] + p.my_rank), "l"(p.value) : "memory");
    const unsigned long long* mine = p.local_flags + p.peer_ranks[q];
    const long long t0 = clock64();
    for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(mine) : "memory");
        if (seen >= p.value) break;
        if (clock64() - t0 > p.limit_cycles) {
            atomicCAS(p.status, 0, blaze::DEV_TIMEOUT_PEER);
            break;
        }
        __nanosleep(100);
    }
}

extern "C" int blazePeerSignal(const blazePeerSignalArgs* a, void* stream) {
    if (!a || a->struct_size < sizeof(blazePeerSignalArgs)) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->n_peers < 1 || a->n_peers > BLAZE_MAX_PEERS || !a->local_flags || a->my_rank < 0)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->limit_cycles < 0 || a->limit_cycles > (1LL << 33)) return ACLTENSOR_STATUS_INVALID_VALUE;
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    PeerSignalParams p;
    p.local_flags = static_cast<unsigned long long*>(a->local_flags);
    for (int q = 0; q < a->n_peers; ++q) {
        if (!a->peer_flags[q] || a->peer_ranks[q] < 0 || a->peer_ranks[q] == a->my_rank) return ACLTENSOR_STATUS_INVALID_VALUE;
        p.peer_flags[q] = static_cast<unsigned long long*>(a->peer_flags[q]);
        p.peer_ranks[q] = a->peer_ranks[q];
    }
    p.n_peers = a->n_peers;
    p.my_rank = a->my_rank;
    p.value = a->value;
    p.limit_cycles = a->limit_cycles > 0 ? a->limit_cycles : (1LL << 31);
    p.status = ctx->status_word;
    return status_of(launch_after_prepass(peer_signal_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), p));
}

extern "C" int blazeDeviceInfo(int32_t* sm_count, int32_t* cc_major, int32_t* cc_minor) {
    DeviceContext* ctx = current_context();
    if (!ctx) return ACLTENSOR_STATUS_NOT_INITIALIZED;
    if (sm_count) *sm_count = ctx->sm_count;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    return ACLTENSOR_STATUS_SUCCESS;
}

extern "C" int blazeCurrentDevice(int32_t* device) {
    if (!device) return ACLTENSOR_STATUS_INVALID_VALUE;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return ACLTENSOR_STATUS_NOT_INITIALIZED;
    }
    *device = dev;
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ MX GEMM without allocation
//
// blazeMxGemm needs caller-provided device scratch for the re-tiled scale factors.  Hosts that hand a plugin no
// allocator - an inference server that has reserved the whole GPU for its own memory pool, a real-time loop in which
// a device allocation would synchronise the GPU - cannot size and allocate that buffer.  For them the same GEMM is
// offered with the scratch held in a fixed 8 MiB array that is part of the library image on every device that loads it.

namespace blaze {

constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_mx_noalloc_scratch[kNoAllocScratchBytes];
static __device__ __align__(256) int g_mx_noalloc_status[64];

struct NoAllocDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;     // device address of g_mx_noalloc_scratch on this device
    int* status = nullptr;                // device address of g_mx_noalloc_status on this device
    int sm_count = 0;
    int cc_major = 0;
};
static std::mutex g_noalloc_mutex;
static NoAllocDevice g_noalloc[64];

// Resolves, once per device and with that device current, the device addresses behind the two symbols.  In host
// code the symbol names are only handles; a kernel must be given the addresses returned here.
static int noalloc_setup(NoAllocDevice** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return ACLTENSOR_STATUS_NOT_INITIALIZED;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocDevice& d = g_noalloc[dev];
    if (!d.ready) {
        void* scratch = nullptr;
        void* status = nullptr;
        if (cudaGetSymbolAddress(&scratch, g_mx_noalloc_scratch) != cudaSuccess ||
            cudaGetSymbolAddress(&status, g_mx_noalloc_status) != cudaSuccess) {
            cudaGetLastError();
            return ACLTENSOR_STATUS_NOT_INITIALIZED;
        }
        int sms = 0, major = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
            cudaGetLastError();
            return ACLTENSOR_STATUS_NOT_INITIALIZED;
        }
        d.scratch = static_cast<unsigned char*>(scratch);
        d.status = static_cast<int*>(status);
        d.sm_count = sms;
        d.cc_major = major;
        d.ready = true;
    }
    *out = &d;
    return ACLTENSOR_STATUS_SUCCESS;
}

static int noalloc_status_fetch(int dev, bool reset) {
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (dev < 0 || dev >= 64 || !g_noalloc[dev].ready) return 0;
        word = g_noalloc[dev].status;
    }
    int v = 0;
    if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (reset && v != 0) cudaMemset(word, 0, sizeof(int));
    return v;
}

}  // namespace blaze

extern "C" int blazeMxGemmNoAlloc(const blazeMxGemmArgs* a, int32_t* device_status, void* stream_v) {
    NoAllocDevice* nd = nullptr;
    int st = noalloc_setup(&nd);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    if (nd->cc_major != 10) return ACLTENSOR_STATUS_ARCH_MISMATCH;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    MxPlan pl;
    st = plan_mx(a, nd->sm_count, &pl, true, false);        // no stream-K: its partial tiles would not fit the array
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    if (a->n_peers != 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (pl.total > kNoAllocScratchBytes) {
        // four copies of B's scale blocks do not fit the array: keep one copy (one more scale copy per K step)
        st = plan_mx(a, nd->sm_count, &pl, false, false);
        if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    }
    if (a->b_elem == BLAZE_ELEM_E2M1) return ACLTENSOR_STATUS_NOT_SUPPORTED;      // packed E2M1 needs an N x K expansion buffer
    if (a->b_layout != BLAZE_B_K_MAJOR) return ACLTENSOR_STATUS_NOT_SUPPORTED;    // so does the transpose of an N-major B
    if (pl.total > kNoAllocScratchBytes) return ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE;   // problem too large for the fixed array
    if (a->M == 0 || a->N == 0) return ACLTENSOR_STATUS_SUCCESS;
    if (!a->A || !a->B || !a->scaleA || !a->scaleB || !a->D) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (a->K == 0) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (a->lda < a->K || a->ldb < a->K || a->ldd < a->N || (a->residual && a->ldr < a->N))
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if ((a->lda % 16) || (a->ldb % 16) || (a->ldd % 8) || (a->residual && (a->ldr % 8)))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (!aligned16(a->A) || !aligned16(a->B) || !aligned16(a->D) || !aligned16(a->bias) || !aligned16(a->residual))
        return ACLTENSOR_STATUS_NOT_SUPPORTED;

    uint8_t* sfa_tiled = nd->scratch + pl.sfa_off;
    uint8_t* sfb_tiled = nd->scratch + pl.sfb_off;
    // the array still holds the previous call's tiles: both scale arrays are rebuilt in full on every call
    cudaError_t e = launch_sf_retile(static_cast<const uint8_t*>(a->scaleA), a->M, a->K, 128, 1, sfa_tiled, nd->sm_count,
                                     stream);
    if (e != cudaSuccess) return status_of(e);
    e = launch_sf_retile(static_cast<const uint8_t*>(a->scaleB), a->N, a->K, pl.tile_n, pl.sfb_replicas, sfb_tiled, nd->sm_count, stream);
    if (e != cudaSuccess) return status_of(e);

    return run_mx_kernel(a, pl, sfa_tiled, sfb_tiled, static_cast<const uint8_t*>(a->B), a->ldb,
                         device_status ? reinterpret_cast<int*>(device_status) : nd->status, nd->sm_count, stream);
}
