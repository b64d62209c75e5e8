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
    int stream_k;                  // single-CTA kernel: split the (tile, K step) units evenly over the grid
    int* flags;                    // [gridDim.x], zeroed before the launch (stream-K only)
    float* partials;               // [gridDim.x][kBN / 32 chunks][8][128 rows][4] float32 (stream-K only)
    int out_type;                  // OutType of D
    uint8_t* scale_d;              // OUT_MX_E4M3: [M][scale_cols_d] E8M0 scales of D
    int scale_cols_d;
    const CUtensorMap* peer_maps;  // global memory: maps of the n_peers further copies of D (2-CTA kernel only)
    int n_peers;
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
    static constexpr int kNumBars = 2 * kStages + 5;
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

// One unit of work of the single-CTA kernel: K steps [ks0, ks1) of one output tile.
struct MxSegment {
    int tile;
    int ks0, ks1;
};

// Walks this CTA's segments; every warp role makes one with the same arguments and sees the same sequence.  Whole
// tiles dealt round-robin, or (stream-K) an even share of all (tile, K step) units: a tail of one tile, whole tiles, and
// a head of another.  The CTA that holds K step 0 of a tile owns it: it adds the partial sums the other CTAs left in
// the workspace, in CTA order, and runs the epilogue (the scheme of the reference's stream-K scheduler and epilogue,
// include/blaze/gemm/block/block_scheduler_matmul_streamk.h:90-146,
// include/blaze/epilogue/block/block_epilogue_matmul_streamk.h:99-265).
struct MxWorkWalker {
    int k_steps, num_tiles, stream_k;
    int next_tile;
    long long unit, unit_end;

    __device__ MxWorkWalker(const MxGemmParams& p, int num_tiles_)
        : k_steps(p.k_steps), num_tiles(num_tiles_), stream_k(p.stream_k), next_tile(blockIdx.x) {
        const long long total = (long long)num_tiles * k_steps;
        unit = total * blockIdx.x / gridDim.x;
        unit_end = total * (blockIdx.x + 1) / gridDim.x;
    }
    __device__ bool next(MxSegment& s) {
        if (!stream_k) {
            if (next_tile >= num_tiles) return false;
            s.tile = next_tile;
            s.ks0 = 0;
            s.ks1 = k_steps;
            next_tile += gridDim.x;
            return true;
        }
        if (unit >= unit_end) return false;
        s.tile = (int)(unit / k_steps);
        s.ks0 = (int)(unit - (long long)s.tile * k_steps);
        const long long left = unit_end - unit;
        s.ks1 = (int)((long long)(k_steps - s.ks0) < left ? k_steps : s.ks0 + left);
        unit += s.ks1 - s.ks0;
        return true;
    }
};

template <int kBN, int kStages, int kAct>
__global__ void __launch_bounds__(192, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_d, const MxGemmParams p) {
    grid_launch_dependents();        // the next kernel in the stream may start setting up as this one's CTAs retire
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
    uint64_t* fix_bar = bars + 2 * kStages + 4;      // the 128 epilogue threads, once, when this CTA leaves a partial tile
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
        mbar_init(fix_bar, 128);
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
        // The whole warp walks the loop and an elected lane issues: with warp-uniform control flow the addresses and
        // descriptors live in uniform registers, where the copy-engine and tensor-core instructions take their operands.
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            grid_dependency_wait();        // the re-tiled scales come from the kernel launched just before this one
            MxWorkWalker walk(p, num_tiles);
            MxSegment seg;
            while (ok && walk.next(seg)) {
                int mt, nt;
                tile_coords(seg.tile, p.m_tiles, p.n_tiles, p.window, mt, nt);
                const uint8_t* sfa_src = p.sfa_tiled + (size_t)mt * p.k_steps * L::kSfaBytes;
                const uint8_t* sfb_src = p.sfb_tiled + (size_t)nt * p.k_steps * L::kSfbBytes;
                for (int ks = seg.ks0; ks < seg.ks1; ++ks) {
                    ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    uint8_t* a_dst = smem + stage * L::kStageBytes;
                    uint8_t* b_dst = a_dst + L::kABytes;
                    uint8_t* sfa_dst = smem + L::kSfOffset + stage * (L::kSfaBytes + L::kSfbBytes);
                    uint8_t* sfb_dst = sfa_dst + L::kSfaBytes;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&full_bar[stage], L::kTxBytes - L::kBBytes - L::kABytes + (L::kBBytes >> p.b_tx_shift) +
                                                                     (L::kABytes >> p.a_tx_shift));
                        tma_load_2d(a_dst, &tmap_a, &full_bar[stage], ks * L::kBK, mt * L::kBM, kEvictNormal);
                        tma_load_2d(b_dst, &tmap_b, &full_bar[stage], ks * L::kBK, nt * kBN, kEvictNormal);
                        bulk_load(sfa_dst, sfa_src + (size_t)ks * L::kSfaBytes, L::kSfaBytes, &full_bar[stage]);
                        bulk_load(sfb_dst, sfb_src + (size_t)ks * L::kSfbBytes, L::kSfbBytes, &full_bar[stage]);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, elected lane issues)
        {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            MxWorkWalker walk(p, num_tiles);
            MxSegment seg;
            while (ok && walk.next(seg)) {
                ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int ks = seg.ks0; ks < seg.ks1; ++ks) {
                    ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, DEV_TIMEOUT_SMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
                    const uint32_t b_addr = a_addr + L::kABytes;
                    const uint32_t sfa_addr = smem_u32(smem + L::kSfOffset + stage * (L::kSfaBytes + L::kSfbBytes));
                    const uint32_t sfb_addr = sfa_addr + L::kSfaBytes;
                    if (elect_one()) {
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
                                   umma_idesc_mx(p.a_format, p.b_format, 128, kBN, j, j),
                                   (ks != seg.ks0 || j != 0) ? 1u : 0u, tmem_base + kSfaCol, tmem_base + kSfbCol);
                    }
                    umma_commit(&empty_bar[stage]);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) umma_commit(&tmem_full_bar[acc]);
                __syncwarp();
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
        MxWorkWalker walk(p, num_tiles);
        MxSegment seg;
        const int r_in_tile = warp * 32 + lane;
        constexpr int kChunks = kBN / 32;
        while (ok && walk.next(seg)) {
            int mt, nt;
            tile_coords(seg.tile, p.m_tiles, p.n_tiles, p.window, mt, nt);
            ok = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            uint64_t* release_bar = &tmem_empty_bar[acc];
            const uint32_t tmem_tile = tmem_base + lane_base + acc * kBN;
            auto release = [&]() {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(release_bar);
            };
            if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }

            if (seg.ks0 > 0) {
                // -------- contributor: leave the partial tile in this CTA's slot, [chunk][8][row][4] so that a warp
                // writes 512 contiguous bytes per instruction, then raise the flag
                float4* slot4 = reinterpret_cast<float4*>(p.partials + (size_t)blockIdx.x * (128 * kBN)) + r_in_tile;
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_tile + c * 32, v);
                    tmem_ld_wait();
                    if (c == kChunks - 1) release();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        __stcg(slot4 + (c * 8 + q) * 128,
                               make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                           __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])));
                    }
                }
                __threadfence();
                mbar_arrive(fix_bar);
                if (threadIdx.x == 0) {
                    if (mbar_wait(fix_bar, 0, abort_flag, p.status, DEV_TIMEOUT_FIXUP_FLAG)) {
                        __threadfence();
                        st_release_gpu(p.flags + blockIdx.x, 1);
                    }
                }
                continue;
            }
            int j_first = 0, j_last = -1;                // CTAs whose partial sums belong to this tile
            if (seg.ks1 < p.k_steps) {
                // -------- owner of a split tile: wait for the CTAs that hold its later K ranges
                const long long total = (long long)num_tiles * p.k_steps;
                const long long tile_end = (long long)(seg.tile + 1) * p.k_steps;
                j_first = blockIdx.x + 1;
                for (int j = j_first; j < (int)gridDim.x; ++j) {
                    if (total * j / gridDim.x >= tile_end) break;
                    const long long t0 = clock64();
                    while (ld_acquire_gpu(p.flags + j) == 0) {
                        if (*abort_flag != 0) { ok = false; break; }
                        if (clock64() - t0 > BLAZE_WAIT_LIMIT_CYCLES) {
                            *abort_flag = 1;
                            atomicCAS(p.status, 0, DEV_TIMEOUT_FIXUP_FLAG);
                            ok = false;
                            break;
                        }
                        __nanosleep(64);
                    }
                    if (!ok) break;
                    j_last = j;
                }
                ok = __all_sync(0xffffffffu, ok);        // also re-converges the warp after the per-thread polling
                if (!ok) break;
            }
            epilogue_store_tile_from<kBN, kAct>(
                tmem_tile, ea, &tmap_d, stage_buf, mt * L::kBM + warp * 32, nt * kBN, lane, chunk_counter, 0, []() {},
                release, [&](int c, uint32_t (&v)[32]) {
                    for (int j = j_first; j <= j_last; ++j) {       // in CTA order: the sum is the same on every run
                        const float4* slot4 =
                            reinterpret_cast<const float4*>(p.partials + (size_t)j * (128 * kBN)) + r_in_tile;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 w = __ldcg(slot4 + (c * 8 + q) * 128);
                            v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + w.x);
                            v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + w.y);
                            v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + w.z);
                            v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + w.w);
                        }
                    }
                });
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
