// G1, paired form: the MX block-scaled GEMM of gemm_mx.cuh on 256 x kBN tiles computed by two CTAs on neighbouring
// SMs (a cluster of 2, tcgen05 cta_group::2).
//
// Each CTA of a pair stages its own 128 rows of A and its own kBN/2 rows of B; the tensor cores of both SMs read the
// two B halves from both shared memories, so every SM loads (128 + kBN/2) x 128 bytes per K step instead of
// (128 + kBN) x 128, which is what bounds the single-CTA kernel (traffic through L2 and time to refill a stage).
// Only the even ("leader") CTA issues tcgen05.cp / tcgen05.mma; its commits arrive on the barriers of both CTAs.
//
// kBN = 224: two disjoint accumulators (2 x 224 columns) + 12 scale columns fit the 512 TMEM columns.
// kBN = 256: the two accumulators cannot both fit beside the scale columns, so they overlap by 16 columns
// (accumulator 0 = columns [0, 256), accumulator 1 = [240, 496), scales at 496).  The epilogue of a tile reads the 32
// columns that contain the shared ones first and signals "overlap read"; the first MMA of the next tile (which uses
// the other accumulator) waits for that signal, a bubble of one barrier round trip per tile.  In exchange a K step
// carries 14 % more MMA work per scale copy and per operand byte loaded.
// Every load is an ordinary per-CTA TMA load (no cluster multicast); the odd CTA's loads credit their bytes to the
// leader's "full" barrier.  The role of the reference code it replaces is the same as in gemm_mx.cuh
// (include/blaze/gemm/kernel/kernel_qbmm_mx.h:379-454, include/blaze/gemm/block/block_mmad_qbmm_mx.h:398-480).
#pragma once

#include "gemm_mx.cuh"

namespace blaze {

template <int kBN, int kStages, bool kWide = true, bool kMxf4 = false>
struct MxPairSmem {
    static constexpr int kBM = 128;                       // rows of A per CTA (256 per pair)
    static constexpr int kBK = 128;
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBHalfBytes = (kBN / 2) * kBK;
    static constexpr int kStageBytes = kABytes + kBHalfBytes;
    // kMxf4: operands are dense 4-bit codes, a 128-byte row holds K = 256, i.e. two 128-K scale blocks per stage
    static constexpr int kSfKPerStage = kMxf4 ? 2 : 1;
    static constexpr int kSfaBytes = 512 * kSfKPerStage;
    static constexpr int kSfbAtoms = (kBN + 127) / 128;
    // kWide: both scale atoms of B go into TMEM with one 128x256b tcgen05.cp (a scale copy costs tensor-pipe time per
    // instruction, not per byte).  That shape has no lane broadcast, so the re-tiled scale array holds each
    // 512-byte atom four times, once per 32-lane quadrant: [atom][quadrant][32 lanes][16 B] per K step.
    static constexpr bool kWideSfb = kWide;
    static constexpr int kSfbBlocksPerK = kWideSfb ? kSfbAtoms * 4 : kSfbAtoms;   // 512-byte blocks per 128 K
    static constexpr int kSfbBlocks = kSfbBlocksPerK * kSfKPerStage;              // per stage
    static constexpr int kSfbBytes = kSfbBlocks * 512;
    static constexpr int kSfOffset = kStages * kStageBytes;
    static constexpr int kBarOffset = kSfOffset + kStages * (kSfaBytes + kSfbBytes);
    static constexpr int kNumBars = 2 * kStages + 6;
    static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
    static constexpr int kEpiOffset = (kMiscOffset + 16 + 1023) / 1024 * 1024;
    static constexpr int kTotal = kEpiOffset + kEpiStageBytes;
    static constexpr int kDynamicBytes = kTotal + 1024;
    static constexpr uint32_t kTxBytesPerCta = kABytes + kBHalfBytes + kSfaBytes + kSfbBytes;
    static_assert(kStageBytes % 1024 == 0, "operand tiles must stay 1024-byte aligned");
};

__device__ __forceinline__ uint32_t map_to_cta(const void* smem_ptr, uint32_t cta_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(smem_ptr)), "r"(cta_rank));
    return remote;
}

// TMA load issued by either CTA of the pair; `bar_cluster_addr` is the shared::cluster address of the barrier that
// receives the byte count (the leader's).
__device__ __forceinline__ void tma_load_2d_to_pair_bar(void* smem_dst, const CUtensorMap* tmap,
                                                        uint32_t bar_cluster_addr, int x, int y, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(hint)
        : "memory");
}

// Walks the segments of one CTA pair.  Whole tiles are dealt round-robin; with `stream_k` the tiles of the last, partly
// filled round are instead cut along K so that every pair gets the same number of K steps of them: a pair then ends
// with a tail of one tile, possibly whole tiles, and a head of another.  The pair that holds K step 0 of a tile owns
// it, as in MxWorkWalker; the reference balances the same last round by re-splitting its tiles along M and N
// (include/blaze/gemm/block/block_scheduler_qbmm.h:120-136, :193-248).
struct MxPairWalker {
    int k_steps, num_tiles, num_pairs, full_tiles;
    int next_tile;
    long long unit, unit_end;      // K steps of the tiles [full_tiles, num_tiles), this pair's share

    __device__ MxPairWalker(const MxGemmParams& p, int num_tiles_, int pair, int num_pairs_)
        : k_steps(p.k_steps), num_tiles(num_tiles_), num_pairs(num_pairs_), next_tile(pair) {
        full_tiles = p.stream_k ? (num_tiles / num_pairs) * num_pairs : num_tiles;
        const long long total = (long long)(num_tiles - full_tiles) * k_steps;
        unit = total * pair / num_pairs;
        unit_end = total * (pair + 1) / num_pairs;
    }
    // first K step (in the numbering of the split tiles) of pair `q`
    __device__ long long first_unit_of(int q) const {
        return (long long)(num_tiles - full_tiles) * k_steps * q / num_pairs;
    }
    __device__ bool next(MxSegment& s) {
        if (next_tile < full_tiles) {
            s.tile = next_tile;
            s.ks0 = 0;
            s.ks1 = k_steps;
            next_tile += num_pairs;
            return true;
        }
        if (unit >= unit_end) return false;
        const int t = (int)(unit / k_steps);
        s.tile = full_tiles + t;
        s.ks0 = (int)(unit - (long long)t * k_steps);
        const long long left = unit_end - unit;
        s.ks1 = (int)((long long)(k_steps - s.ks0) < left ? k_steps : s.ks0 + left);
        unit += s.ks1 - s.ks0;
        return true;
    }
};

template <int kBN, int kStages, int kAct, bool kWide = true, bool kMxf4 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                    const __grid_constant__ CUtensorMap tmap_d, const MxGemmParams p) {
    grid_launch_dependents();        // the next kernel in the stream may start setting up as this one's CTAs retire
    using L = MxPairSmem<kBN, kStages, kWide, kMxf4>;
    static_assert(!kMxf4 || kWide, "the FP4 form copies B's scales with the wide copy");
    static_assert(kBN % 32 == 0 && kBN >= 32 && kBN <= 256, "tile N");
    constexpr int kAccStages = 2;
    constexpr int kSfCols = (4 + 4 * L::kSfbAtoms) * L::kSfKPerStage;
    constexpr int kSfReserve = (kSfCols + 15) / 16 * 16;
    constexpr bool kOverlap = kAccStages * kBN + kSfCols > 512;         // accumulators share their edge columns
    constexpr int kSfaCol = kOverlap ? 512 - kSfReserve : kAccStages * kBN;
    constexpr int kSfbCol = kSfaCol + 4 * L::kSfKPerStage;
    constexpr int kAccStride = kOverlap ? kSfaCol - kBN : kBN;           // column of accumulator 1
    static_assert(kSfbCol + 4 * L::kSfbAtoms * L::kSfKPerStage <= 512, "TMEM budget");
    static_assert(!kOverlap || (kBN - kAccStride <= 32 && kAccStride % 16 == 0), "shared columns fit one chunk");
    constexpr int kChunks = kBN / 32;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
    uint64_t* full_bar = bars;                       // used in the leader only
    uint64_t* empty_bar = bars + kStages;            // one per CTA, released by the leader's commits
    uint64_t* tmem_full_bar = bars + 2 * kStages;    // one per CTA
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;   // used in the leader only: 8 epilogue warps arrive
    uint64_t* overlap_bar = bars + 2 * kStages + 4;      // leader only: the shared accumulator columns were read
    uint64_t* fix_bar = bars + 2 * kStages + 5;          // this CTA's 128 epilogue threads, once: its partial tile is written
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
        mbar_init(overlap_bar, 8);
        mbar_init(fix_bar, 128);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc<2>(tmem_base_slot, kTmemCols);
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_sfa);
        tma_prefetch_desc(&tmap_sfb);
        tma_prefetch_desc(&tmap_d);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                  // both CTAs' barriers exist before anyone signals across
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    const int num_tiles = p.m_tiles * p.n_tiles;     // m_tiles counts 256-row tiles here

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        // (the whole warp walks the loop, an elected lane issues: see the MMA issuer below)
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // the re-tiled scales come from the kernel launched just before this one; everything above (barriers,
            // TMEM, descriptor prefetch) may overlap its tail
            grid_dependency_wait();
            MxPairWalker walk(p, num_tiles, pair, num_pairs);
            MxSegment seg;
            while (ok && walk.next(seg)) {
                int mt, nt;
                tile_coords(seg.tile, p.m_tiles, p.n_tiles, p.window, mt, nt);
                const int a_row = mt * 256 + (int)cta_rank * 128;
                const int b_row = nt * kBN + (int)cta_rank * (kBN / 2);
                const int sfa_row = (mt * 2 + (int)cta_rank) * p.sf_k_steps;
                const int sfb_row = nt * p.sf_k_steps * L::kSfbBlocksPerK;
                for (int ks = seg.ks0; ks < seg.ks1; ++ks) {
                    ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    uint8_t* a_dst = smem + stage * L::kStageBytes;
                    uint8_t* b_dst = a_dst + L::kABytes;
                    uint8_t* sfa_dst = smem + L::kSfOffset + stage * (L::kSfaBytes + L::kSfbBytes);
                    uint8_t* sfb_dst = sfa_dst + L::kSfaBytes;
                    const uint32_t bar = map_to_cta(&full_bar[stage], 0);
                    if (elect_one()) {
                        if (cta_rank == 0) {
                            mbar_arrive_expect_tx(&full_bar[stage], 2 * (L::kTxBytesPerCta - L::kBHalfBytes - L::kABytes +
                                                                         (L::kBHalfBytes >> p.b_tx_shift) +
                                                                         (L::kABytes >> p.a_tx_shift)));
                        }
                        tma_load_2d_to_pair_bar(a_dst, &tmap_a, bar, ks * L::kBK, a_row, kEvictNormal);
                        tma_load_2d_to_pair_bar(b_dst, &tmap_b, bar, ks * L::kBK, b_row, kEvictNormal);
                        tma_load_2d_to_pair_bar(sfa_dst, &tmap_sfa, bar, 0, sfa_row + ks * L::kSfKPerStage, kEvictNormal);
                        tma_load_2d_to_pair_bar(sfb_dst, &tmap_sfb, bar, 0, sfb_row + ks * L::kSfbBlocks, kEvictNormal);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        // The whole warp walks the loop and one elected lane issues the tcgen05 instructions: with warp-uniform control
        // flow the descriptors and addresses live in uniform registers, where those instructions take their operands;
        // inside a single-lane branch every operand of every instruction was first moved there, and this thread's
        // instruction stream - not the tensor core - set the pace of a K step.
        if (cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            uint32_t tiles_done = 0;
            bool ok = true;
            // constant words of the shared-memory descriptors and the four instruction descriptors of a K step
            const uint32_t smem_base = smem_u32(smem);
            const uint64_t sw0 = umma_desc_sw128(0);
            const uint32_t sw_hi = (uint32_t)(sw0 >> 32);
            const uint32_t sw_lo0 = (uint32_t)sw0 + (smem_base >> 4);
            const uint32_t sf_hi = (uint32_t)(umma_desc_sf(0) >> 32);
            const uint32_t sf_lo0 = (smem_base + L::kSfOffset) >> 4;
            const uint32_t sf_wide_lead = (uint32_t)umma_desc_sf_wide(0, 4 * 512);      // leading-offset field, low word
            const uint32_t full0 = smem_u32(&full_bar[0]);
            const uint32_t empty0 = smem_u32(&empty_bar[0]);
            uint32_t idesc_j[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if constexpr (kMxf4) {
                    const uint32_t id = (uint32_t)(j & 1) * 2;
                    idesc_j[j] = umma_idesc_mx(FMT_MXF4_E2M1, FMT_MXF4_E2M1, 256, kBN, id, id);
                } else {
                    idesc_j[j] = umma_idesc_mx(p.a_format, p.b_format, 256, kBN, j, j);
                }
            }
            auto desc_of = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            MxPairWalker walk(p, num_tiles, pair, num_pairs);
            MxSegment seg;
            while (ok && walk.next(seg)) {
                ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (kOverlap && tiles_done != 0) {
                    // the previous tile's epilogue must have read the columns this accumulator shares with it
                    ok = mbar_wait(overlap_bar, (tiles_done - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                ++tiles_done;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccStride;
                for (int ks = seg.ks0; ks < seg.ks1; ++ks) {
                    const int first = ks == seg.ks0 ? 0 : 1;          // the segment's first MMA overwrites the accumulator
                    ok = mbar_wait_addr(full0 + stage * 8, phase, abort_flag, p.status, DEV_TIMEOUT_SMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                    // descriptors from precomputed words: this thread's instruction count, not the tensor core, set the
                    // pace of a K step when every descriptor was rebuilt from its address
                    const uint32_t a_lo = sw_lo0 + stage * (L::kStageBytes >> 4);
                    const uint32_t b_lo = a_lo + (L::kABytes >> 4);
                    const uint32_t sfa_lo = sf_lo0 + stage * ((L::kSfaBytes + L::kSfbBytes) >> 4);
                    const uint32_t sfb_lo = sfa_lo + (L::kSfaBytes >> 4);
                    if (elect_one()) {
                    if constexpr (kMxf4) {
                        // two 128-K scale blocks per stage: A's by the broadcasting copy, B's two atoms by one wide copy
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            utccp_sf<2>(tmem_base + kSfaCol + 4 * h, desc_of(sfa_lo + (512 >> 4) * h, sf_hi));
                            utccp_sf_wide<2>(tmem_base + kSfbCol + 8 * h,
                                             desc_of((sfb_lo + h * ((L::kSfbBytes / 2) >> 4)) | sf_wide_lead, sf_hi));
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            // K = 64 per instruction = 32 bytes of packed codes; scale bytes 2 (j % 2) and + 1 of
                            // block j / 2
                            umma_mxf4_pair(d_tmem, desc_of(a_lo + 2 * j, sw_hi), desc_of(b_lo + 2 * j, sw_hi), idesc_j[j],
                                           (first | j) != 0 ? 1u : 0u, tmem_base + kSfaCol + 4 * (j >> 1),
                                           tmem_base + kSfbCol + 8 * (j >> 1));
                        }
                    } else {
                        utccp_sf<2>(tmem_base + kSfaCol, desc_of(sfa_lo, sf_hi));
                        if constexpr (L::kWideSfb) {
                            utccp_sf_wide<2>(tmem_base + kSfbCol, desc_of(sfb_lo | sf_wide_lead, sf_hi));
                        } else {
#pragma unroll
                            for (int i = 0; i < L::kSfbAtoms; ++i) {
                                utccp_sf<2>(tmem_base + kSfbCol + 4 * i, desc_of(sfb_lo + (512 >> 4) * i, sf_hi));
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            umma_mx<2>(d_tmem, desc_of(a_lo + 2 * j, sw_hi), desc_of(b_lo + 2 * j, sw_hi), idesc_j[j],
                                       (first | j) != 0 ? 1u : 0u, tmem_base + kSfaCol, tmem_base + kSfbCol);
                        }
                    }
                    umma_commit_pair_addr(empty0 + stage * 8, 0x3);
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
        const EpilogueArgs ea{p.M, p.N, p.bias, p.residual, p.ldr, p.out_type, p.scale_d, p.scale_cols_d,
                              p.peer_maps, p.n_peers};
        MxPairWalker walk(p, num_tiles, pair, num_pairs);
        MxSegment seg;
        const int r_in_tile = warp * 32 + lane;
        while (ok && walk.next(seg)) {
            int mt, nt;
            tile_coords(seg.tile, p.m_tiles, p.n_tiles, p.window, mt, nt);
            ok = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            uint64_t* release_bar = &tmem_empty_bar[acc];          // owned by the leader CTA
            // accumulator 0 shares its last columns, accumulator 1 its first: start with the chunk that holds them
            const int first_chunk = (kOverlap && acc == 0) ? kChunks - 1 : 0;
            const uint32_t tmem_tile = tmem_base + lane_base + acc * kAccStride;
            auto early = [&]() {
                if (kOverlap) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(overlap_bar, 0);
                }
            };
            auto release = [&]() {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(release_bar, 0);
            };
            if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }

            if (seg.ks0 > 0) {
                // -------- contributor: this CTA's 128 rows of the partial tile go to its slot of the workspace,
                // [chunk][8][row][4] so that a warp writes 512 contiguous bytes per instruction, then the mark is raised
                float4* slot4 = reinterpret_cast<float4*>(p.partials + (size_t)blockIdx.x * (128 * kBN)) + r_in_tile;
#pragma unroll 1
                for (int i = 0; i < kChunks; ++i) {
                    int c = first_chunk + i;
                    if (c >= kChunks) c -= kChunks;
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_tile + c * 32, v);
                    tmem_ld_wait();
                    if (i == 0) early();
                    if (i == kChunks - 1) release();
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
            int q_first = 0, q_last = -1;                // pairs whose partial sums belong to this tile
            if (seg.ks1 < p.k_steps) {
                // -------- owner of a split tile: wait for the same-ranked CTAs of the pairs that hold its later K ranges
                const long long tile_end = (long long)(seg.tile - walk.full_tiles + 1) * p.k_steps;
                q_first = pair + 1;
                for (int q = q_first; q < num_pairs; ++q) {
                    if (walk.first_unit_of(q) >= tile_end) break;
                    const int* flag = p.flags + (2 * q + (int)cta_rank);
                    const long long t0 = clock64();
                    while (ld_acquire_gpu(flag) == 0) {
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
                    q_last = q;
                }
                ok = __all_sync(0xffffffffu, ok);        // also re-converges the warp after the per-thread polling
                if (!ok) break;
            }
            epilogue_store_tile_from<kBN, kAct>(
                tmem_tile, ea, &tmap_d, stage_buf, mt * 256 + (int)cta_rank * 128 + warp * 32, nt * kBN, lane,
                chunk_counter, first_chunk, early, release, [&](int c, uint32_t (&v)[32]) {
                    for (int q = q_first; q <= q_last; ++q) {       // in pair order: the sum is the same on every run
                        const float4* slot4 = reinterpret_cast<const float4*>(
                                                  p.partials + (size_t)(2 * q + (int)cta_rank) * (128 * kBN)) + r_in_tile;
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float4 w = __ldcg(slot4 + (c * 8 + u) * 128);
                            v[4 * u] = __float_as_uint(__uint_as_float(v[4 * u]) + w.x);
                            v[4 * u + 1] = __float_as_uint(__uint_as_float(v[4 * u + 1]) + w.y);
                            v[4 * u + 2] = __float_as_uint(__uint_as_float(v[4 * u + 2]) + w.z);
                            v[4 * u + 3] = __float_as_uint(__uint_as_float(v[4 * u + 3]) + w.w);
                        }
                    }
                });
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
