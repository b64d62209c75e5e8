// Unscaled GEMMs of the Blaze surface on the 2-CTA tile skeleton of gemm_mx_pair.cuh: INT8 x INT8 with int32
// accumulation and de-quantisation on store (A8W8), and fp16 / bf16 with float32 accumulation.
//
//   INT8:  D[m,n] = act( float(sum_k A[m,k] * B[n,k] + bias_i32[n]) * scale[n] ) + residual[m,n]
//   16-bit: D[m,n] = act( sum_k A[m,k] * B[n,k] + bias[n] ) + residual[m,n]
//
// They stand where the reference has GemmUniversal<..., KernelQbmmCube> with BlockMmad<...A8W8FixpipeQuant>
// (include/blaze/gemm/kernel/kernel_qbmm_cube.h:43-140, scale handling :190-220;
// include/blaze/gemm/block/block_mmad_a8w8_fixpipe_quant.h:42-527, scale applied on store :227-234, bias as
// accumulator init :309) and the basic matmul kernel (include/blaze/gemm/kernel/kernel_matmul_basic.h:32-200).
// The scale the reference hands its fix pipe is a float32 whose low 13 mantissa bits are cleared
// (DEQ_SCALE_MUL = 0xFFFFE000, kernel_qbmm_cube.h:68): per tensor the product scaleA[0] * scaleB[0], per channel the
// low word of a 64-bit entry per column.  The same masking is applied here, so results are bit-identical to
// float16(float32(int32 sum) * masked scale).
//
// 256 x 256 tiles on a cluster of two CTAs (tcgen05 cta_group::2, kind::i8 or kind::f16): each CTA stages its 128 rows
// of A and its 128 rows of B per 128-byte K block (128 INT8 or 64 16-bit elements), the even CTA issues four MMAs per
// block, two accumulators of 256 columns fill the 512 TMEM columns, the epilogue of tile i overlaps the mainloop of
// tile i+1.  Every load is an ordinary per-CTA TMA load; the odd CTA's loads credit the leader's barrier.
#pragma once

#include "gemm_mx_pair.cuh"

namespace blaze {

enum DenseKind : int { DENSE_S8 = 0, DENSE_F16 = 1, DENSE_BF16 = 2 };
enum DenseScale : int { DENSE_SCALE_NONE = 0, DENSE_SCALE_PER_TENSOR = 1, DENSE_SCALE_PER_CHANNEL = 2 };

struct DenseGemmParams {
    int M, N, K;
    int m_tiles, n_tiles, k_steps;      // 256-row tiles, 256-column tiles, 128-byte K blocks
    int window;
    int scale_mode;                     // DenseScale (INT8 only)
    const float* scale_a;               // per tensor: one float each
    const float* scale_b;
    const unsigned long long* scale_n;  // per channel: [N], float32 bits in the low word
    const int* bias_i32;                // INT8: [N] added to the int32 sum, or nullptr
    const __nv_bfloat16* bias;          // 16-bit kinds: [N] or nullptr
    const __nv_bfloat16* residual;
    long long ldr;
    int out_type;                       // OutType of D (OUT_S32: the raw int32 sums of an INT8 product)
    int* status;
};

constexpr int OUT_S32 = 5;              // continues OutType: raw int32 accumulators (INT8 product, no scale)

template <int kStages>
struct DensePairSmem {
    static constexpr int kBN = 256;
    static constexpr int kABytes = 128 * 128;
    static constexpr int kBHalfBytes = (kBN / 2) * 128;
    static constexpr int kStageBytes = kABytes + kBHalfBytes;
    static constexpr int kBarOffset = kStages * kStageBytes;
    static constexpr int kNumBars = 2 * kStages + 4;
    static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
    static constexpr int kEpiOffset = (kMiscOffset + 16 + 1023) / 1024 * 1024;
    static constexpr int kTotal = kEpiOffset + kEpiStageBytes;
    static constexpr int kDynamicBytes = kTotal + 1024;
    static constexpr uint32_t kTxBytesPerCta = kABytes + kBHalfBytes;
};

// Instruction descriptors: kind::i8 (signed 8-bit operands, int32 accumulate) and kind::f16 (fp16 or bf16 operands,
// float32 accumulate), both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_s8(uint32_t m, uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t umma_idesc_f16(bool bf16, uint32_t m, uint32_t n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

template <int kKind>
__device__ __forceinline__ void umma_dense_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    if constexpr (kKind == DENSE_S8) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

template <int kKind, int kStages, int kAct>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
dense_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_d, const DenseGemmParams p) {
    grid_launch_dependents();
    using L = DensePairSmem<kStages>;
    constexpr int kBN = L::kBN;
    constexpr int kAccStages = 2;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
    uint64_t* full_bar = bars;                       // used in the leader only
    uint64_t* empty_bar = bars + kStages;            // one per CTA, released by the leader's commits
    uint64_t* tmem_full_bar = bars + 2 * kStages;    // one per CTA
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;   // leader only: the 8 epilogue warps of the pair arrive
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full_bar[s], 1);
            mbar_init(&tmem_empty_bar[s], 8);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 5) tmem_alloc<2>(tmem_base_slot, kTmemCols);
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_d);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                  // both CTAs' barriers exist before anyone signals across
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int num_tiles = p.m_tiles * p.n_tiles;
    // the operand tensor maps describe rows of bytes, so a K block is 128 units along x for either element size
    constexpr int kElemsPerBlock = 128;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        // The whole warp walks the loop and an elected lane issues: with warp-uniform control flow the addresses and
        // descriptors live in uniform registers, where the copy-engine and tensor-core instructions take their operands.
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            grid_dependency_wait();
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int mt, nt;
                tile_coords(t, p.m_tiles, p.n_tiles, p.window, mt, nt);
                const int a_row = mt * 256 + (int)cta_rank * 128;
                const int b_row = nt * kBN + (int)cta_rank * (kBN / 2);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    uint8_t* a_dst = smem + stage * L::kStageBytes;
                    const uint32_t bar = map_to_cta(&full_bar[stage], 0);
                    if (elect_one()) {
                        if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * L::kTxBytesPerCta);
                        tma_load_2d_to_pair_bar(a_dst, &tmap_a, bar, ks * kElemsPerBlock, a_row, kEvictNormal);
                        tma_load_2d_to_pair_bar(a_dst + L::kABytes, &tmap_b, bar, ks * kElemsPerBlock, b_row, kEvictNormal);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only; whole warp,
        // elected lane issues)
        if (cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            constexpr uint32_t idesc = kKind == DENSE_S8 ? umma_idesc_s8(256, kBN) : umma_idesc_f16(kKind == DENSE_BF16, 256, kBN);
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, DEV_TIMEOUT_SMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + L::kABytes);
                    if (elect_one()) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {        // 32 bytes of K per instruction = 2 units of 16 bytes
                            umma_dense_pair<kKind>(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, (ks | j) != 0 ? 1u : 0u);
                        }
                        umma_commit_pair(&empty_bar[stage], 0x3);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) umma_commit_pair(&tmem_full_bar[acc], 0x3);
                __syncwarp();
                if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 0..3 (both CTAs)
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t chunk_counter = 0;
        bool ok = true;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        uint8_t* stage_buf = smem + L::kEpiOffset + warp * kEpiStageBytesPerWarp;
        // an INT8 product leaves as raw int32 sums through the float32 store path (same 4-byte elements)
        const int store_type = p.out_type == OUT_S32 ? OUT_F32 : p.out_type;
        const EpilogueArgs ea{p.M, p.N, kKind == DENSE_S8 ? nullptr : p.bias, p.residual, p.ldr, store_type, nullptr, 0};
        float tensor_scale = 1.0f;
        if (kKind == DENSE_S8 && p.scale_mode == DENSE_SCALE_PER_TENSOR) {
            grid_dependency_wait();
            tensor_scale = __uint_as_float(__float_as_uint(__ldg(p.scale_a) * __ldg(p.scale_b)) & 0xFFFFE000u);
        }
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            int mt, nt;
            tile_coords(t, p.m_tiles, p.n_tiles, p.window, mt, nt);
            ok = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            uint64_t* release_bar = &tmem_empty_bar[acc];          // owned by the leader CTA
            const int col0 = nt * kBN;
            epilogue_store_tile_from<kBN, kAct>(
                tmem_base + lane_base + acc * kBN, ea, &tmap_d, stage_buf, mt * 256 + (int)cta_rank * 128 + warp * 32, col0,
                lane, chunk_counter, 0, []() {},
                [&]() {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(release_bar, 0);
                },
                [&](int c, uint32_t (&v)[32]) {
                    if constexpr (kKind == DENSE_S8) {
                        // int32 sums (+ int32 bias) -> float32 -> x scale: what the reference's fix pipe does on store
                        if (p.out_type == OUT_S32 && !p.bias_i32) return;
                        const int n0 = col0 + c * 32;
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const int n = n0 + e;
                            int sum = (int)v[e];
                            if (p.bias_i32 && n < p.N) sum += __ldg(p.bias_i32 + n);
                            if (p.out_type == OUT_S32) { v[e] = (uint32_t)sum; continue; }
                            float s = tensor_scale;
                            if (p.scale_mode == DENSE_SCALE_PER_CHANNEL && n < p.N)
                                s = __uint_as_float((uint32_t)__ldg(p.scale_n + n) & 0xFFFFE000u);
                            v[e] = __float_as_uint(__fmul_rn(__int2float_rn(sum), s));
                        }
                    }
                });
            if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
        }
        if (lane == 0) epilogue_drain_stores();
    }

    // ---------------------------------------------------------------------- teardown
    __syncthreads();
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();          // neither CTA leaves while its partner may still signal its barriers or read its tiles
    if (warp == 5) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

}  // namespace blaze
