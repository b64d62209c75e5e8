// G1: persistent MX block-scaled GEMM for sm_100a.
//
//   D[M,N] (bf16) = act( sum_k (A[m,k] * 2^(sa[m,k/32]-127)) * (B[n,k] * 2^(sb[n,k/32]-127)) + bias[n] ) + residual[m,n]
//
// A is [M,K] and B is [N,K], both K-contiguous 8-bit codes (E4M3, or E2M1 values stored as E4M3 codes by the
// weight pre-pass).  It stands where the reference has GemmUniversal<KernelMmadWithScaleMx> +
// BlockMmad<MatmulWithScaleMx> + BlockSchedulerQuantBatchMatmulV3
// (include/blaze/gemm/kernel/kernel_qbmm_mx.h:39-454, include/blaze/gemm/block/block_mmad_qbmm_mx.h:398-514,
// include/blaze/gemm/block/block_scheduler_qbmm.h:271-317), re-thought for Blackwell:
//
//   * warp 4 streams 128-byte-swizzled operand tiles (TMA) and pre-tiled scale-factor blocks (bulk copy) into a
//     kStages-deep shared-memory ring,
//   * one elected thread of warp 5 copies the scale blocks into TMEM (tcgen05.cp) and issues
//     tcgen05.mma.kind::mxf8f6f4.block_scale, four K=32 instructions per 128-wide K step,
//   * warps 0-3 drain a finished fp32 accumulator from TMEM (tcgen05.ld), apply bias / activation / residual and
//     hand bf16 blocks to TMA stores (epilogue.cuh), while the tensor core already fills the second accumulator.
//
// Tiles are visited in the reference's windowed serpentine order; each CTA takes tile ids
// blockIdx.x, blockIdx.x + gridDim.x, ...
#pragma once

#include "epilogue.cuh"
#include "ptx.cuh"

namespace blaze {

struct MxGemmParams {
    int M, N, K;
    int m_tiles, n_tiles, k_steps;
    int sf_k_steps;                // 128-K blocks per tile row in the re-tiled scale arrays (= k_steps except for kind::mxf4)
    int window;                    // M-tile rows per serpentine band
    const uint8_t* sfa_tiled;      // [m_tiles][k_steps][512]
    const uint8_t* sfb_tiled;      // [n_tiles][k_steps][kSfbBytes]
    const __nv_bfloat16* bias;     // [N] or nullptr
    const __nv_bfloat16* residual; // [M][ldr] or nullptr
    long long ldr;
    __nv_bfloat16* D;              // [M][ldd]
    long long ldd;
    int* status;
    uint32_t b_format;             // UmmaFormat of B in shared memory: FMT_E4M3, or FMT_E2M1 when TMA unpacks 4-bit codes
    uint32_t b_tx_shift;           // 1 when the B loads credit the barrier with the packed (half) byte count, else 0
    uint32_t a_format, a_tx_shift; // the same two for A
    int out_type;                  // OutType of D
    uint8_t* scale_d;              // OUT_MX_E4M3: [M][scale_cols_d] E8M0 scales of D
    int scale_cols_d;
};

template <int kBN, int kStages>
struct MxGemmSmem {
    static constexpr int kBM = 128;
    static constexpr int kBK = 128;
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = kBN * kBK;
    static constexpr int kSfaBytes = 512;
    static constexpr int kSfbBytes = ((kBN + 127) / 128) * 512;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSfOffset = kStages * kStageBytes;
    static constexpr int kBarOffset = kSfOffset + kStages * (kSfaBytes + kSfbBytes);
    // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    static constexpr int kNumBars = 2 * kStages + 4;
    static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
    static constexpr int kEpiOffset = (kMiscOffset + 16 + 1023) / 1024 * 1024;     // bf16 staging blocks of the epilogue
    static constexpr int kTotal = kEpiOffset + kEpiStageBytes;
    static constexpr int kDynamicBytes = kTotal + 1024;      // slack for manual 1024-byte alignment
    static constexpr uint32_t kTxBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int window, int& mt, int& nt) {
    const int band_tiles = window * n_tiles;
    const int band = t / band_tiles;
    const int rows = min(window, m_tiles - band * window);
    const int r = t - band * band_tiles;
    const int n_idx = r / rows;
    mt = band * window + (r - n_idx * rows);
    nt = (band & 1) ? (n_tiles - 1 - n_idx) : n_idx;
}

template <int kBN, int kStages, int kAct>
__global__ void __launch_bounds__(192, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_d, const MxGemmParams p) {
    using L = MxGemmSmem<kBN, kStages>;
    static_assert(kBN % 32 == 0 && kBN >= 32 && kBN <= 256, "tile N");
    constexpr int kAccStages = 2;
    constexpr int kSfaCol = kAccStages * kBN;
    constexpr int kSfbCol = kSfaCol + 4;
    static_assert(kSfbCol + 4 * ((kBN + 127) / 128) <= 512, "TMEM budget");
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + kStages;
    uint64_t* tmem_full_bar = bars + 2 * kStages;
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full_bar[s], 1);
            mbar_init(&tmem_empty_bar[s], 4);        // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc<1>(tmem_base_slot, kTmemCols);
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_d);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    const int num_tiles = p.m_tiles * p.n_tiles;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            grid_dependency_wait();        // the re-tiled scales come from the kernel launched just before this one
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int mt, nt;
                tile_coords(t, p.m_tiles, p.n_tiles, p.window, mt, nt);
                const uint8_t* sfa_src = p.sfa_tiled + (size_t)mt * p.k_steps * L::kSfaBytes;
                const uint8_t* sfb_src = p.sfb_tiled + (size_t)nt * p.k_steps * L::kSfbBytes;
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY);
                    if (!ok) break;
                    uint8_t* a_dst = smem + stage * L::kStageBytes;
                    uint8_t* b_dst = a_dst + L::kABytes;
                    uint8_t* sfa_dst = smem + L::kSfOffset + stage * (L::kSfaBytes + L::kSfbBytes);
                    uint8_t* sfb_dst = sfa_dst + L::kSfaBytes;
                    mbar_arrive_expect_tx(&full_bar[stage], L::kTxBytes - L::kBBytes - L::kABytes + (L::kBBytes >> p.b_tx_shift) +
                                                                 (L::kABytes >> p.a_tx_shift));
                    tma_load_2d(a_dst, &tmap_a, &full_bar[stage], ks * L::kBK, mt * L::kBM, kEvictNormal);
                    tma_load_2d(b_dst, &tmap_b, &full_bar[stage], ks * L::kBK, nt * kBN, kEvictNormal);
                    bulk_load(sfa_dst, sfa_src + (size_t)ks * L::kSfaBytes, L::kSfaBytes, &full_bar[stage]);
                    bulk_load(sfb_dst, sfb_src + (size_t)ks * L::kSfbBytes, L::kSfbBytes, &full_bar[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, DEV_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
                    const uint32_t b_addr = a_addr + L::kABytes;
                    const uint32_t sfa_addr = smem_u32(smem + L::kSfOffset + stage * (L::kSfaBytes + L::kSfbBytes));
                    const uint32_t sfb_addr = sfa_addr + L::kSfaBytes;
                    utccp_sf<1>(tmem_base + kSfaCol, umma_desc_sf(sfa_addr));
#pragma unroll
                    for (int i = 0; i < L::kSfbBytes / 512; ++i) {
                        utccp_sf<1>(tmem_base + kSfbCol + 4 * i, umma_desc_sf(sfb_addr + 512 * i));
                    }
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(b_addr);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // 32 bytes further along K inside the swizzled row = 2 units of 16 bytes
                        umma_mx<1>(d_tmem, a_desc + 2 * j, b_desc + 2 * j,
                                   umma_idesc_mx(p.a_format, p.b_format, 128, kBN, j, j), (ks | j) != 0 ? 1u : 0u,
                                   tmem_base + kSfaCol, tmem_base + kSfbCol);
                    }
                    umma_commit(&empty_bar[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&tmem_full_bar[acc]);
                if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 0..3
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t chunk_counter = 0;
        bool ok = true;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        uint8_t* stage_buf = smem + L::kEpiOffset + warp * kEpiStageBytesPerWarp;
        const EpilogueArgs ea{p.M, p.N, p.bias, p.residual, p.ldr, p.out_type, p.scale_d, p.scale_cols_d};
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int mt, nt;
            tile_coords(t, p.m_tiles, p.n_tiles, p.window, mt, nt);
            ok = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            uint64_t* release_bar = &tmem_empty_bar[acc];
            epilogue_store_tile<kBN, kAct>(tmem_base + lane_base + acc * kBN, ea, &tmap_d, stage_buf,
                                           mt * L::kBM + warp * 32, nt * kBN, lane, chunk_counter, [&]() {
                                               tcgen05_fence_before();
                                               __syncwarp();
                                               if (lane == 0) mbar_arrive(release_bar);
                                           });
            if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
        }
        if (lane == 0) epilogue_drain_stores();
    }

    // ---------------------------------------------------------------------- teardown
    __syncthreads();
    if (*abort_flag != 0) {
        // give copies and MMAs that may still be in flight time to land before shared memory and TMEM are released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 5) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

}  // namespace blaze
