// G2 / G3 / G4: persistent FP8 (E4M3) GEMM with float32 scales, one per 1x128 K-group of A and one per 128x128 block
// of B, in three flavours chosen at launch: dense data-parallel, dense stream-K (split along K with a
// deterministic fix-up, for skinny or K-heavy shapes) and grouped (per-expert B, rows of A partitioned by a
// device-side group list).
//
//   D[m,n] (bf16) = act( sum_kb sa[m,kb] * sb[g,kb,n/128] * (sum_{k in kb} A[m,k] * B[g,n,k]) + bias[n] ) + residual[m,n]
//
// The reference names these modes (QuantMode PERGROUP/PERBLOCK, include/blaze/gemm/utils/common_utils.h:98-107;
// PER_BLOCK_SIZE = 128, :59; 128-aligned tail tiles in include/blaze/gemm/block/block_scheduler_qbmm.h:212-223;
// groupListGmAddr in include/blaze/gemm/block/block_mmad_matmul_basic.h:68) without implementing them; the split of
// work along K with an fp32 workspace and an ordered reduction follows its stream-K kernel
// (include/blaze/gemm/kernel/kernel_matmul_streamk.h:98-228,
//  include/blaze/epilogue/block/block_epilogue_matmul_streamk.h:123-184).
//
// float32 scales cannot ride on the hardware block-scale path, so every 128-deep K block is multiplied into a
// fresh TMEM accumulator (4 stages of 128 columns) and promoted into registers by eight epilogue warps (two per
// TMEM lane quadrant, 64 columns each): acc += (sa * sb) * block, while the tensor core works on the next blocks.
// Warps 0-7: promotion + epilogue, warp 8: TMA producer, warps 9 and 10: MMA issuers taking K blocks in turn.
// One tcgen05.commit per K block: "block g is done" is barrier g % 8; the promotion warps wait on it for the accumulator
// (TMEM stage g % 4), the TMA thread for the operand stage (g % kStages).
#pragma once

#include "ptx.cuh"

namespace blaze {

constexpr int kFp8MaxGroups = 1024;

struct Fp8GemmParams {
    int M, N, K;                    // M = total rows of A (all groups)
    int n_tiles, k_blocks;
    int m_tiles;                    // dense: ceil(M/128); grouped: unused
    int window;
    int groups;                     // 0 = dense
    const long long* group_rows;    // device int64[groups]
    const float* sa;                // [M][k_blocks]
    const float* sb;                // [groups or 1][k_blocks][n_blocks]
    int n_blocks;                   // ceil(N/128)
    const __nv_bfloat16* bias;      // [N] or nullptr
    const __nv_bfloat16* residual;  // [M][ldr] or nullptr
    long long ldr;
    __nv_bfloat16* D;
    long long ldd;
    int stream_k;                   // 0: whole tiles per CTA; 1: the (tile, k-block) units split evenly over the grid;
                                    // 2: the kernel chooses between the two once it knows the tile count (grouped)
    float* partials;                // [gridDim.x][32 column quads][128 rows][4] fp32 (stream-K only)
    int out_type;                   // OutType of D (ldd counts elements of that type)
    float* scale_d;                 // OUT_FP8_128: [M][n_blocks] float32 scales of D
    // Stream-K hand-over marks, [gridDim.x]: a contributor stores `epoch` (a value no earlier launch of this process
    // used, so whatever the workspace held before cannot be mistaken for it) behind its partial tile; the tile's owner
    // waits for exactly that value and clears the mark before the kernel ends, so that a replay of the same launch
    // from a CUDA graph - same epoch - starts from cleared marks as well.  No reset pass before the launch.
    unsigned long long* flags;
    unsigned long long epoch;
    int b_static;                   // B does not depend on the preceding kernel in the stream: its first tiles may be
                                    // requested while that kernel is still running (dense problems only)
    int* status;
    uint8_t* peer_d[7];             // further copies of D (same pitch and type) that 16-bit output rows are also sent to:
    int n_peers;                    // this GPU's slot in the other GPUs' gathered outputs
};

// Tensor maps of the further copies of D (`peer_d`), for the tiled output copies; entries beyond n_peers are unused.
struct Fp8PeerMaps {
    CUtensorMap m[7];
};

template <int kStages>
struct Fp8GemmSmem {
    static constexpr int kTile = 128;
    static constexpr int kABytes = kTile * kTile;
    static constexpr int kBBytes = kTile * kTile;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOffset = kStages * kStageBytes;
    static constexpr int kAccStages = 4;
    // "MMAs of K block g have finished" is signalled on barrier g % 8 (parity (g / 8) % 2).  The promotion warps wait on
    // it for the accumulator (TMEM stage g % 4) and the TMA thread for the operand stage (g % kStages), so one
    // tcgen05.commit per block serves both rings; eight barriers keep the parities unambiguous for any kStages <= 8.
    static constexpr int kDoneBars = 8;
    // full[kStages], done[8], tmem_empty[4], fixup, amax exchange
    static constexpr int kNumBars = kStages + kDoneBars + kAccStages + 2;
    static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
    static constexpr int kGroupOffset = kMiscOffset + 16;       // int row_start[G+1], int mtile_start[G+1]
    static constexpr int kAmaxOffset = kGroupOffset + 2 * (kFp8MaxGroups + 1) * 4;   // float amax[2 tiles][<= 4 column parts][128]
    // 16-bit outputs leave through shared memory.  A promotion warp whose 32 rows may all be written stages them as
    // two 32 x 32 blocks (64-byte rows, 64-byte swizzle) and one lane hands both to the copy engine as tiled stores.
    // (The same blocks go to every peer copy of D through the peers' tensor maps.)  A warp that must stop at a group's
    // last row stages plain rows (padded by 16 bytes against bank conflicts) and every thread issues a bulk copy of its
    // own row, to D and to each peer.
    static constexpr int kStoreRowPitch = 64 * 2 + 16;
    static constexpr int kStoreWarpBytes = 5 * 1024;                                     // >= 32 * kStoreRowPitch, >= 2 * 2048
    static constexpr int kStoreOffset = (kAmaxOffset + 2 * 4 * 128 * 4 + 1023) & ~1023;  // swizzled blocks: 1 KB aligned
    static_assert(kStoreRowPitch % 16 == 0 && 32 * kStoreRowPitch <= kStoreWarpBytes, "staged rows are read and written as uint4");
    static constexpr int kTotal = kStoreOffset + 8 * kStoreWarpBytes;
    static constexpr int kDynamicBytes = kTotal + 1024;
    static constexpr uint32_t kTxBytes = kABytes + kBBytes;
};

// One unit of work: K blocks [kb0, kb1) of one output tile.
struct Fp8Segment {
    int m0;          // first row of A / D
    int row_end;     // rows >= row_end are not stored
    int nt;          // N tile
    int group;       // expert (0 when dense)
    int kb0, kb1;
    int tile;        // linear tile id (stream-K bookkeeping)
};

// Walks the segments of this CTA.  Every warp role instantiates one with identical arguments, so all roles see
// the same sequence.
struct Fp8WorkWalker {
    const Fp8GemmParams& p;
    const int* row_start;     // shared memory, grouped only
    const int* mtile_start;   // shared memory, grouped only
    int total_m_tiles;
    int num_tiles;
    bool split;               // stream-K: units of (tile, k-block) instead of whole tiles
    // data-parallel state
    int next_tile;
    // stream-K state
    long long unit, unit_end;

    __device__ Fp8WorkWalker(const Fp8GemmParams& p_, const int* row_start_, const int* mtile_start_)
        : p(p_), row_start(row_start_), mtile_start(mtile_start_) {
        total_m_tiles = p.groups > 0 ? mtile_start[p.groups] : p.m_tiles;
        num_tiles = total_m_tiles * p.n_tiles;
        split = p.stream_k == 1;
        if (p.stream_k == 2 && num_tiles > 0) {
            // the host's cost model (plan_fp8), evaluated here because a grouped problem's tile count is only known on
            // the device: K blocks per SM for whole tiles against an even split plus its fix-up cost
            const int cta = (int)gridDim.x;
            const float whole = (float)((num_tiles + cta - 1) / cta) * (float)p.k_blocks;
            const long long units = (long long)num_tiles * p.k_blocks;
            const float even = (float)((units + cta - 1) / cta) + 17.0f + 2.8f * (float)cta / (float)num_tiles;
            split = p.k_blocks >= 2 && even < whole;
        }
        next_tile = blockIdx.x;
        const long long total = (long long)num_tiles * p.k_blocks;
        unit = total * blockIdx.x / gridDim.x;
        unit_end = total * (blockIdx.x + 1) / gridDim.x;
    }

    __device__ void locate(int t, Fp8Segment& s) const {
        s.tile = t;
        if (p.groups > 0) {
            const int gm = t / p.n_tiles;
            s.nt = t - gm * p.n_tiles;
            int lo = 0, hi = p.groups;            // largest g with mtile_start[g] <= gm
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (mtile_start[mid] <= gm) lo = mid; else hi = mid;
            }
            s.group = lo;
            s.m0 = row_start[lo] + (gm - mtile_start[lo]) * 128;
            s.row_end = row_start[lo + 1];
        } else {
            int mt;
            tile_coords_fp8(t, mt, s.nt);
            s.group = 0;
            s.m0 = mt * 128;
            s.row_end = p.M;
        }
    }

    __device__ void tile_coords_fp8(int t, int& mt, int& nt) const {
        const int band_tiles = p.window * p.n_tiles;
        const int band = t / band_tiles;
        const int rows = min(p.window, p.m_tiles - band * p.window);
        const int r = t - band * band_tiles;
        const int n_idx = r / rows;
        mt = band * p.window + (r - n_idx * rows);
        nt = (band & 1) ? (p.n_tiles - 1 - n_idx) : n_idx;
    }

    __device__ bool next(Fp8Segment& s) {
        if (split) {
            if (unit >= unit_end) return false;
            const int t = (int)(unit / p.k_blocks);
            const int kb = (int)(unit - (long long)t * p.k_blocks);
            const long long room = unit_end - unit;
            const int kb1 = (int)min((long long)p.k_blocks, kb + room);
            locate(t, s);
            s.kb0 = kb;
            s.kb1 = kb1;
            unit += kb1 - kb;
            return true;
        }
        if (next_tile >= num_tiles) return false;
        locate(next_tile, s);
        s.kb0 = 0;
        s.kb1 = p.k_blocks;
        next_tile += gridDim.x;
        return true;
    }
};

template <int kStages, int kAct, int kIssuers = 1, int kParts = 2>
__global__ void __launch_bounds__(128 * kParts + 32 + 32 * kIssuers, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ Fp8PeerMaps peer_maps,
                const Fp8GemmParams p) {
    grid_launch_dependents();        // the next kernel in the stream may start setting up as this one's CTAs retire
    using L = Fp8GemmSmem<kStages>;
    constexpr int kAccStages = L::kAccStages;
    // With as many operand stages as accumulator stages, block g uses stage g % 4 of both rings, and one barrier says
    // "go" for it: the 8 promotion warps' "accumulator stage free", the TMA thread's arrival and the tile bytes all
    // complete the same phase.  The MMA issuer then waits on one barrier per K block instead of two (each wait costs
    // the issuing thread ~100 cycles of a ~450-cycle iteration).
#ifndef LAB_MERGED
#define LAB_MERGED 1
#endif
    constexpr bool kMerged = LAB_MERGED && (kStages == kAccStages);
    static_assert(kStages <= L::kDoneBars && kAccStages <= kStages, "see Fp8GemmSmem::kDoneBars");
    static_assert(kParts == 2, "the output staging area holds eight warps' rows");
    constexpr uint32_t kTmemCols = 512;
    // warp roles: 4 * kParts promotion warps (TMEM lane quadrant = warp % 4, column part = warp / 4), one TMA warp, then
    // the MMA issuer warps
    constexpr int kPromoWarps = 4 * kParts;
    constexpr int kCols = 128 / kParts;              // accumulator columns per promotion thread
    constexpr int kTmaWarp = kPromoWarps;
    constexpr int kMmaWarp0 = kPromoWarps + 1;
    static_assert(kParts == 2 || kParts == 4, "64 or 32 columns per promotion thread");

    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
    uint64_t* full_bar = bars;
    uint64_t* tmem_full_bar = bars + kStages;                       // the eight "block done" barriers
    uint64_t* tmem_empty_bar = tmem_full_bar + L::kDoneBars;
    uint64_t* fix_bar = tmem_empty_bar + kAccStages;
    uint64_t* amax_bar = fix_bar + 1;              // the 256 promotion threads, once per quantised output tile
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);
    int* fix_range = reinterpret_cast<int*>(smem + L::kMiscOffset + 8);     // contributors of the split tile this CTA owns
    int* row_start = reinterpret_cast<int*>(smem + L::kGroupOffset);
    int* mtile_start = row_start + (kFp8MaxGroups + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], kMerged ? 1 + 4 * kParts : 1);
        }
        for (int s = 0; s < L::kDoneBars; ++s) mbar_init(&tmem_full_bar[s], 1);
        for (int s = 0; s < kAccStages; ++s) mbar_init(&tmem_empty_bar[s], kPromoWarps);
        mbar_init(fix_bar, 32 * kPromoWarps);
        mbar_init(amax_bar, 32 * kPromoWarps);
        *abort_flag = 0;
        fix_range[0] = 0;
        fix_range[1] = -1;
        fence_mbar_init();
    }
    if (warp == kMmaWarp0 && p.groups > 0) {
        // Prefix sums of rows and of 128-row tiles over the group list (which an earlier kernel may have produced),
        // 32 groups per step with warp scans: one thread walking the list paid an L2 round trip per group, 27 us
        // for 128 groups.  Counts are clamped so that the groups never step outside A.
        grid_dependency_wait();
        long long carry_rows = 0;
        int carry_tiles = 0;
#pragma unroll 4
        for (int base = 0; base < p.groups; base += 32) {
            const int g = base + lane;
            long long r = (g < p.groups) ? __ldg(p.group_rows + g) : 0;
            r = r < 0 ? 0 : (r > p.M ? (long long)p.M : r);
            long long incl = r;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const long long o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            const long long end = min(carry_rows + incl, (long long)p.M);
            const long long start = min(carry_rows + incl - r, (long long)p.M);
            const int t = (int)((end - start + 127) >> 7);
            int t_incl = t;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, t_incl, d);
                if (lane >= d) t_incl += o;
            }
            if (g < p.groups) {
                row_start[g] = (int)start;
                mtile_start[g] = carry_tiles + t_incl - t;
            }
            carry_rows = __shfl_sync(0xffffffffu, end, 31);
            carry_tiles += __shfl_sync(0xffffffffu, t_incl, 31);
        }
        if (lane == 0) {
            row_start[p.groups] = (int)carry_rows;
            mtile_start[p.groups] = carry_tiles;
        }
    }
    if (warp == kMmaWarp0) {
        tmem_alloc<1>(tmem_base_slot, kTmemCols);
    }
    if (warp == kTmaWarp && lane == 0) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_d);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // Launched with programmatic stream serialisation: everything above may overlap the tail of the previous kernel
    // in the stream; nothing below touches global memory before that kernel has finished - except the TMA thread's
    // first weight tiles when the caller has declared the weights independent of that kernel.
    if (warp != kTmaWarp) grid_dependency_wait();

    // The two single-thread loops below run once per 128-deep K block, i.e. every 256 tensor-core cycles: they are
    // written with precomputed shared-memory addresses and descriptor words so that their instruction count, not
    // the tensor core, does not set the pace.
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(&full_bar[0]);
    const uint32_t tfull0 = smem_u32(&tmem_full_bar[0]);
    const uint32_t tempty0 = smem_u32(&tmem_empty_bar[0]);

    if (warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer
        // The whole warp walks the loop and an elected lane issues: with warp-uniform control flow the addresses live in
        // uniform registers, where the copy-engine (and tensor-core) instructions take their operands; inside a
        // single-lane branch every operand of every such instruction is first moved there.
        {
            Fp8WorkWalker walk(p, row_start, mtile_start);
            Fp8Segment seg;
            uint32_t stage = 0;
            uint32_t g = 0;                  // K blocks issued by this CTA so far
            bool ok = true;
            // B is streamed once when there is a single row of tiles; keep A (re-read by every N tile) instead
            const uint64_t b_hint = (p.groups == 0 && p.m_tiles == 1) ? kEvictFirst : kEvictNormal;
            // Static weights of a dense problem: arm the first stages and request their B tiles now, while the previous
            // kernel in the stream may still be running; the A tiles follow once it has finished.
            uint32_t early = 0;
            if (p.b_static && p.groups == 0) {
                Fp8WorkWalker ahead(p, row_start, mtile_start);
                Fp8Segment sg;
                while (early < (uint32_t)kStages && ahead.next(sg)) {
                    for (int kb = sg.kb0; kb < sg.kb1 && early < (uint32_t)kStages; ++kb, ++early) {
                        const uint32_t bar = full0 + early * 8;
                        if (elect_one()) {
                            mbar_arrive_expect_tx_addr(bar, L::kTxBytes);
                            tma_load_2d_addr(smem_base + early * L::kStageBytes + L::kABytes, &tmap_b, bar, kb * 128,
                                             sg.nt * 128, b_hint);
                        }
                        __syncwarp();
                    }
                }
            }
            grid_dependency_wait();
            while (ok && walk.next(seg)) {
                const int b_row = seg.group * p.N + seg.nt * 128;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (g < early) {                 // stage armed and B requested above: only A is missing
                        if (elect_one()) {
                            tma_load_2d_addr(smem_base + stage * L::kStageBytes, &tmap_a, full0 + stage * 8, kb * 128, seg.m0,
                                             kEvictNormal);
                        }
                        __syncwarp();
                        if (++stage == kStages) stage = 0;
                        ++g;
                        continue;
                    }
                    // the stage is free once the MMAs of the block that used it last (g - kStages) have finished; the
                    // block's "done" barrier says so, and the stage needs no commit of its own (~86 tensor-pipe cycles)
                    if (g >= (uint32_t)kStages) {
                        const uint32_t d = g - kStages;
                        ok = mbar_wait_addr(tfull0 + (d & 7) * 8, (d >> 3) & 1, abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    }
                    const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                    const uint32_t bar = full0 + stage * 8;
                    if (elect_one()) {
                        mbar_arrive_expect_tx_addr(bar, L::kTxBytes);
                        tma_load_2d_addr(a_dst, &tmap_a, bar, kb * 128, seg.m0, kEvictNormal);
                        tma_load_2d_addr(a_dst + L::kABytes, &tmap_b, bar, kb * 128, b_row, b_hint);
                    }
                    __syncwarp();
                    if (++stage == kStages) stage = 0;
                    ++g;
                }
            }
        }
    } else if (warp >= kMmaWarp0) {
        // ------------------------------------------------------------------ MMA issuer(s)
        // A K block has its own accumulator stage, so blocks are independent and kIssuers threads (one per warp) take
        // them in turn: while one thread polls its barriers the other's MMAs keep the tensor core busy (the tensor
        // core's instruction queue is too short to cover one thread's waits).
        // (whole warp, elected lane issues: see the TMA producer)
        {
            Fp8WorkWalker walk(p, row_start, mtile_start);
            Fp8Segment seg;
            uint32_t stage = 0;
            uint32_t phase = 0;
            uint32_t g = 0;
            const uint32_t my_turn = (uint32_t)(warp - kMmaWarp0);
            bool ok = true;
            constexpr uint32_t idesc = umma_idesc_f8(FMT_E4M3, FMT_E4M3, 128, 128);
            const uint64_t desc0 = umma_desc_sw128(0);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
            const uint32_t desc_lo0 = (uint32_t)desc0 + (smem_base >> 4);          // start-address field of stage 0's A tile
            while (ok && walk.next(seg)) {
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (kIssuers == 1 || (g % kIssuers) == my_turn) {
                        const uint32_t acc = g & 3;
                        if (!kMerged) {
                            ok = mbar_wait_addr(tempty0 + acc * 8, ((g >> 2) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY);
                            ok = __all_sync(0xffffffffu, ok);
                            if (!ok) break;
                        }
                        ok = mbar_wait_addr(full0 + stage * 8, phase, abort_flag, p.status, DEV_TIMEOUT_SMEM_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t a_lo = desc_lo0 + stage * (L::kStageBytes >> 4);
                        if (elect_one()) {
                            umma_f8_kblock(tmem_base + acc * 128, a_lo, a_lo + (L::kABytes >> 4), desc_hi, idesc);
                            umma_commit_addr(tfull0 + (g & 7) * 8);
                        }
                        __syncwarp();
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                    ++g;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        Fp8WorkWalker walk(p, row_start, mtile_start);
        Fp8Segment seg;
        uint32_t g = 0;
        bool ok = true;
        float* amax_smem = reinterpret_cast<float*>(smem + L::kAmaxOffset);
        int tile_parity = 0;
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may read
        const int part = warp >> 2;                     // which kCols of the tile's 128 columns
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const int r_in_tile = quad * 32 + lane;
        const int c0 = part * kCols;
        // The two scale factors of a K block come from global memory (L2 latency); they are fetched kScaleAhead
        // blocks ahead into a register ring so that the promotion never waits for them.  The ring is idle during a
        // tile's epilogue, so the first scales of the next segment are requested before the epilogue starts.
        constexpr int kScaleAhead = 4;
        float sa_q[kScaleAhead], sb_q[kScaleAhead];
        const bool sa_vec_ok = (p.k_blocks & 3) == 0 && (reinterpret_cast<uintptr_t>(p.sa) & 15) == 0;
        // requests the scales of blocks kb_first .. kb_first + 3 of a segment: A's as one 16-byte load when the batch is
        // whole and aligned (the usual case), B's four by pointer steps
        auto fetch_scales = [&](const float* sa_r, const float* sb_c, int kb_first, int kb_end, bool rows_in) {
            if (sa_vec_ok && (kb_first & 3) == 0 && kb_first + kScaleAhead <= kb_end) {
                const float4 a4 = rows_in ? __ldg(reinterpret_cast<const float4*>(sa_r + kb_first))
                                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                sa_q[0] = a4.x; sa_q[1] = a4.y; sa_q[2] = a4.z; sa_q[3] = a4.w;
                const float* b = sb_c + (long long)kb_first * p.n_blocks;
#pragma unroll
                for (int u = 0; u < kScaleAhead; ++u) {
                    sb_q[u] = __ldg(b);
                    b += p.n_blocks;
                }
                return;
            }
#pragma unroll
            for (int u = 0; u < kScaleAhead; ++u) {
                const int kq = kb_first + u;
                const bool in = rows_in && kq < kb_end;
                sa_q[u] = in ? __ldg(sa_r + kq) : 0.0f;
                sb_q[u] = kq < kb_end ? __ldg(sb_c + (long long)kq * p.n_blocks) : 0.0f;
            }
        };
        auto fetch_first_scales = [&](const Fp8Segment& sg) {
            const int row_f = sg.m0 + r_in_tile;
            const bool in_rows = row_f < sg.row_end;
            fetch_scales(p.sa + (long long)(in_rows ? row_f : 0) * p.k_blocks,
                         p.sb + (long long)sg.group * p.k_blocks * p.n_blocks + sg.nt, sg.kb0, sg.kb1, in_rows);
        };
        Fp8Segment next_seg;
        if (kMerged && lane == 0) {                     // the first use of each stage finds its accumulator free
            for (int i = 0; i < kAccStages; ++i) mbar_arrive(&full_bar[i]);
        }
        bool have = walk.next(seg);
        if (have) fetch_first_scales(seg);
        for (; ok && have; seg = next_seg) {
            const int row = seg.m0 + r_in_tile;
            const bool row_ok = row < seg.row_end;
            const float* sa_row = p.sa + (long long)(row_ok ? row : 0) * p.k_blocks;
            const float* sb_col = p.sb + (long long)seg.group * p.k_blocks * p.n_blocks + seg.nt;
            float accum[kCols];
#pragma unroll
            for (int j = 0; j < kCols; ++j) accum[j] = 0.0f;
            for (int kb0 = seg.kb0; kb0 < seg.kb1 && ok; kb0 += kScaleAhead) {
                // The scales of this batch of blocks were requested a batch ago: their products are taken out of the
                // load registers BEFORE the next batch is requested, so that nothing inside the batch waits on a
                // scoreboard that a load still in flight shares.
                float s_cur[kScaleAhead];
#pragma unroll
                for (int u = 0; u < kScaleAhead; ++u) s_cur[u] = sa_q[u] * sb_q[u];
                fetch_scales(sa_row, sb_col, kb0 + kScaleAhead, seg.kb1, row_ok);
#pragma unroll
                for (int u = 0; u < kScaleAhead; ++u) {
                    const int kb = kb0 + u;
                    if (kb >= seg.kb1) break;                                   // uniform across the CTA
                    const float s = s_cur[u];
                    const int acc = (int)(g & 3);
                    // one probe and a vote in the usual case (the block is done); the bounded wait only behind a miss
                    if (!__all_sync(0xffffffffu, mbar_try_wait(&tmem_full_bar[g & 7], (g >> 3) & 1))) {
                        ok = mbar_wait(&tmem_full_bar[g & 7], (g >> 3) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    }
                    tcgen05_fence_after();
                    // (a warp whose rows all lie beyond the group's end promotes them anyway: they are never stored, and
                    // a branch here cost every warp ~40 cycles per block)
                    {
                        uint32_t v[kCols];
                        if constexpr (kCols == 64) tmem_ld_32x64(tmem_base + lane_base + acc * 128 + c0, v);
                        else tmem_ld_32x32(tmem_base + lane_base + acc * 128 + c0, v);
                        tmem_ld_wait();
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(kMerged ? &full_bar[acc] : &tmem_empty_bar[acc]);    // the block is in registers: free the stage
#pragma unroll
                        for (int e = 0; e < kCols; e += 2) fma_f32x2(accum[e], accum[e + 1], v[e], v[e + 1], s);
                    }
                    ++g;
                }
            }
            if (!ok) break;
            have = walk.next(next_seg);
            if (have) fetch_first_scales(next_seg);

            const bool full_tile = (seg.kb0 == 0 && seg.kb1 == p.k_blocks);
            if (!full_tile && seg.kb0 > 0) {
                // -------- contributor: publish the partial tile
                float* slot = p.partials + (size_t)blockIdx.x * (128 * 128);
                if (row_ok) {
                    // layout [column quad][row][4]: a warp writes 512 contiguous bytes per instruction
                    float4* slot4 = reinterpret_cast<float4*>(slot) + (size_t)(c0 >> 2) * 128 + r_in_tile;
#pragma unroll
                    for (int j = 0; j < kCols / 4; ++j) {
                        __stcg(slot4 + j * 128, make_float4(accum[4 * j], accum[4 * j + 1], accum[4 * j + 2], accum[4 * j + 3]));
                    }
                }
                __threadfence();
                mbar_arrive(fix_bar);
                if (threadIdx.x == 0) {
                    if (mbar_wait(fix_bar, 0, abort_flag, p.status, DEV_TIMEOUT_FIXUP_FLAG)) {
                        __threadfence();
                        st_release_gpu_u64(p.flags + blockIdx.x, p.epoch);
                    }
                }
                continue;
            }
            if (!full_tile) {
                // -------- owner of a split tile: add the later K ranges in CTA order
                const long long total = (long long)walk.num_tiles * p.k_blocks;
                const long long tile_end = (long long)(seg.tile + 1) * p.k_blocks;
                int j_last = (int)blockIdx.x;                      // last CTA that holds a K range of this tile
                for (int j = blockIdx.x + 1; j < (int)gridDim.x; ++j) {
                    if (total * j / gridDim.x >= tile_end) break;
                    j_last = j;
                }
                if (threadIdx.x == 0 && j_last > (int)blockIdx.x) {     // marks to clear when the kernel ends
                    fix_range[0] = blockIdx.x + 1;
                    fix_range[1] = j_last;
                }
                // All contributors finish at about the same time, so their marks are polled side by side - one lane
                // per contributor, every warp for itself - instead of one L2 round trip after the other between the
                // partial tiles.
                for (int base = blockIdx.x + 1; base <= j_last && ok; base += 32) {
                    const int j = base + lane;
                    if (j <= j_last) {
                        const long long t0 = clock64();
                        while (ld_acquire_gpu_u64(p.flags + j) != p.epoch) {
                            if (*abort_flag != 0) { ok = false; break; }
                            if (clock64() - t0 > BLAZE_WAIT_LIMIT_CYCLES) {
                                *abort_flag = 1;
                                atomicCAS(p.status, 0, DEV_TIMEOUT_FIXUP_FLAG);
                                ok = false;
                                break;
                            }
                            __nanosleep(64);
                        }
                    }
                    ok = __all_sync(0xffffffffu, ok);      // re-converges the warp; orders the lanes' later loads
                }
                if (!ok) break;
                for (int j = blockIdx.x + 1; j <= j_last; ++j) {
                    const float* slot = p.partials + (size_t)j * (128 * 128);
                    if (row_ok) {
                        const float4* slot4 = reinterpret_cast<const float4*>(slot) + (size_t)(c0 >> 2) * 128 + r_in_tile;
#pragma unroll
                        for (int c = 0; c < kCols / 4; ++c) {
                            const float4 v4 = __ldcg(slot4 + c * 128);
                            accum[4 * c] += v4.x;
                            accum[4 * c + 1] += v4.y;
                            accum[4 * c + 2] += v4.z;
                            accum[4 * c + 3] += v4.w;
                        }
                    }
                }
                ok = __all_sync(0xffffffffu, ok);      // also re-converges the warp after the per-thread polling
                if (!ok) break;
            }

            // -------- fused epilogue: bias, activation, residual, cast; kCols consecutive outputs per thread
            const __nv_bfloat16* r_row = (p.residual && row_ok) ? p.residual + (long long)row * p.ldr : nullptr;
            float row_amax = 0.0f;
            const bool quantised_out = p.out_type == OUT_FP8_128;
            // a plain cast (grouped and dense GEMMs without epilogue operands) skips the pass over the accumulators
            const bool has_epilogue_math = kAct != ACT_IDENTITY || p.bias || p.residual || quantised_out;
#pragma unroll
            for (int q = 0; q < kCols / 8; ++q) {
                if (!has_epilogue_math) break;
                const int n = seg.nt * 128 + c0 + q * 8;
                if (row_ok && n < p.N) {
                    float x[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[e] = accum[q * 8 + e];
                    if (p.bias) {
                        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + n));
                        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            x[2 * e] += __uint_as_float(bw[e] << 16);
                            x[2 * e + 1] += __uint_as_float(bw[e] & 0xFFFF0000u);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[e] = apply_act<kAct>(x[e]);
                    if (r_row) {
                        const uint4 rv = *reinterpret_cast<const uint4*>(r_row + n);
                        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            x[2 * e] += __uint_as_float(rw[e] << 16);
                            x[2 * e + 1] += __uint_as_float(rw[e] & 0xFFFF0000u);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        accum[q * 8 + e] = x[e];
                        row_amax = fmaxf(row_amax, fabsf(x[e]));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) accum[q * 8 + e] = 0.0f;
                }
            }
            if (p.out_type == OUT_FP8_128) {
                // Quantising output: one float32 scale per row per 128 columns (this tile's width), amax / 448, and
                // E4M3 codes of x / scale - the A operand of the next FP8 GEMM, by the rules of quant_fp8_1x128_kernel.
                // The two warps that share a row (column halves) exchange their maxima through shared memory.
                float* amax_buf = amax_smem + (tile_parity * kParts) * 128;
                amax_buf[part * 128 + r_in_tile] = row_amax;
                mbar_arrive(amax_bar);                                     // all promotion warps
                ok = mbar_wait(amax_bar, (uint32_t)tile_parity, abort_flag, p.status, DEV_TIMEOUT_FIXUP_FLAG);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                float amax = row_amax;
#pragma unroll
                for (int o = 1; o < kParts; ++o) amax = fmaxf(amax, amax_buf[((part + o) % kParts) * 128 + r_in_tile]);
                tile_parity ^= 1;
                const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 448.0f);
                if (row_ok) {
                    uint8_t* d_row = reinterpret_cast<uint8_t*>(p.D) + (long long)row * p.ldd;
#pragma unroll
                    for (int q = 0; q < kCols / 16; ++q) {
                        const int n = seg.nt * 128 + c0 + q * 16;
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            w[e] = cvt_e4m3x4_sat(__fdiv_rn(accum[q * 16 + 4 * e], scale),
                                                  __fdiv_rn(accum[q * 16 + 4 * e + 1], scale),
                                                  __fdiv_rn(accum[q * 16 + 4 * e + 2], scale),
                                                  __fdiv_rn(accum[q * 16 + 4 * e + 3], scale));
                        }
                        if (n + 8 < p.N) {
                            *reinterpret_cast<uint4*>(d_row + n) = make_uint4(w[0], w[1], w[2], w[3]);
                        } else if (n < p.N) {
                            *reinterpret_cast<uint2*>(d_row + n) = make_uint2(w[0], w[1]);
                        }
                    }
                    if (part == 0 && seg.nt * 128 < p.N) p.scale_d[(long long)row * p.n_blocks + seg.nt] = scale;
                }
            } else if (p.out_type != OUT_F32) {
                // bf16 / f16: a thread holds kCols consecutive outputs of one row, so storing from registers would touch
                // 32 different lines per instruction (2.2 us per 128x128 tile).  The rows go through shared memory to
                // the copy engine instead.
                uint8_t* warp_stage = smem + L::kStoreOffset + warp * L::kStoreWarpBytes;
                const int n0 = seg.nt * 128 + c0;
                const int warp_row0 = seg.m0 + quad * 32;
                tma_store_wait_read<0>();                        // the previous tile's copies have read the staging area
                __syncwarp();
                // tiled stores clip at the matrix edges only: usable when no row of this warp lies beyond the group's
                // end (the next group's rows start there); 256 row copies per tile (times the number of copies of D)
                // kept the copy engine busy for ~4000 cycles in which the promotion warps could not start the next tile
                const bool tiled = p.groups == 0 || warp_row0 + 32 <= seg.row_end;
                if (tiled) {
                    const int sw = (lane >> 1) & 3;              // 64-byte swizzle: 16-byte slot ^= (row / 2) % 4
#pragma unroll
                    for (int h = 0; h < kCols / 32; ++h) {
                        uint8_t* my_row = warp_stage + h * 2048 + lane * 64;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float* x = accum + h * 32 + q * 8;
                            uint4 o;
                            if (p.out_type == OUT_F16) {
                                o = make_uint4(pack_f16(x[0], x[1]), pack_f16(x[2], x[3]), pack_f16(x[4], x[5]), pack_f16(x[6], x[7]));
                            } else {
                                o = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
                            }
                            *reinterpret_cast<uint4*>(my_row + ((q ^ sw) << 4)) = o;
                        }
                    }
                    fence_proxy_async();                         // the copy engine reads what this warp just wrote
                    __syncwarp();
                    if (lane == 0 && warp_row0 < seg.row_end) {
#pragma unroll
                        for (int h = 0; h < kCols / 32; ++h) {
                            if (n0 + 32 * h < p.N) {
                                tma_store_2d(&tmap_d, warp_stage + h * 2048, n0 + 32 * h, warp_row0);
                                for (int q = 0; q < p.n_peers; ++q) {
                                    tma_store_2d(&peer_maps.m[q], warp_stage + h * 2048, n0 + 32 * h, warp_row0);
                                }
                            }
                        }
                    }
                } else {
                    uint8_t* my_row = warp_stage + lane * L::kStoreRowPitch;
#pragma unroll
                    for (int q = 0; q < kCols / 8; ++q) {
                        const float* x = accum + q * 8;
                        uint4 o;
                        if (p.out_type == OUT_F16) {
                            o = make_uint4(pack_f16(x[0], x[1]), pack_f16(x[2], x[3]), pack_f16(x[4], x[5]), pack_f16(x[6], x[7]));
                        } else {
                            o = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
                        }
                        *reinterpret_cast<uint4*>(my_row + q * 16) = o;
                    }
                    fence_proxy_async();                         // the copy engine reads what this thread just wrote
                    if (row_ok && n0 < p.N) {
                        const uint32_t bytes = (uint32_t)min(kCols, p.N - n0) * 2u;      // N is a multiple of 8
                        const long long at = ((long long)row * p.ldd + n0) * 2;
                        bulk_store(reinterpret_cast<uint8_t*>(p.D) + at, my_row, bytes);
                        for (int q = 0; q < p.n_peers; ++q) bulk_store(p.peer_d[q] + at, my_row, bytes);
                    }
                }
                tma_store_commit();
            } else if (row_ok) {
                float* d_row = reinterpret_cast<float*>(p.D) + (long long)row * p.ldd;
#pragma unroll
                for (int q = 0; q < kCols / 4; ++q) {
                    const int n = seg.nt * 128 + c0 + q * 4;
                    if (n < p.N) {
                        *reinterpret_cast<float4*>(d_row + n) =
                            make_float4(accum[q * 4], accum[q * 4 + 1], accum[q * 4 + 2], accum[q * 4 + 3]);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (warp < kPromoWarps) tma_store_wait_read<0>();     // output rows the copy engine has not read yet
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag == 0) {
        // every thread of this CTA has seen these marks: clear them for the next launch that carries the same epoch
        for (int j = fix_range[0]; j <= fix_range[1]; ++j) p.flags[j] = 0ull;
    }
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == kMmaWarp0) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

}  // namespace blaze
