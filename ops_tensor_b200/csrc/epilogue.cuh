// Fused epilogue of the MX GEMM kernels: TMEM -> registers -> (bias, activation, residual, cast to bf16 / half /
// float32) -> shared memory -> TMA store.
//
// One warp owns 32 accumulator rows (its TMEM lane quadrant); each thread holds one row.  The tile is drained in
// chunks of 32 columns: tcgen05.ld brings 32 fp32 values per thread, the fused ops run in registers, the bf16
// results go to a 32 x 32 staging block in shared memory (64-byte rows, 64-byte swizzle, so the 16-byte writes of a
// warp are bank-conflict free) and one lane hands the block to TMA, which writes full 32-byte sectors and clips at
// the matrix edge.  Two staging blocks per warp alternate, so the store of chunk c overlaps the math of chunk c+1.
// This takes the place of the reference's fix-pipe store with cast (include/blaze/gemm/block/block_mmad_qbmm_mx.h:466-479,
// cast modes in include/tensor_api/impl/tensor_api/arch/cube/utils/l0c2out_utils.h:122-132), its bias-as-accumulator
// init (block_mmad_qbmm_mx.h:500-506) and the fusion hook (include/blaze/epilogue/fusion/default_fusion_op.h:28-56).
#pragma once

#include "ptx.cuh"

namespace blaze {

constexpr int kEpiStageBytesPerWarp = 2 * 32 * 64;      // two 32 x 32 bf16 blocks
constexpr int kEpiStageBytes = 4 * kEpiStageBytesPerWarp;

struct EpilogueArgs {
    int M, N;
    const __nv_bfloat16* bias;
    const __nv_bfloat16* residual;
    long long ldr;
    int out_type;       // OutType of D; the tensor map handed to the store has the matching element size and box
    uint8_t* scale_d;   // OUT_MX_E4M3: E8M0 scales of D, [M][scale_cols_d]
    int scale_cols_d;   // ceil(N / 64) * 2
    const CUtensorMap* peer_maps = nullptr;   // global memory: n_peers more maps of D's shape (16-bit outputs only);
    int n_peers = 0;                          // every staged block is stored through each of them as well
};

// Drains one accumulator tile.  `tmem_tile` = TMEM address of column 0 of the accumulator, lane field already set to
// this warp's quadrant.  `row0` = global row of lane 0, `col0` = global column of accumulator column 0.  `stage` =
// this warp's staging area (kEpiStageBytesPerWarp bytes, 512-byte aligned).  `chunk_counter` persists across tiles.
// The 32-column chunks are visited in the order first_chunk, first_chunk + 1, ... (wrapping).  `early()` is called
// once the TMEM read of the first visited chunk has completed, `release()` once the last TMEM read of the tile has
// completed; both run before the remaining math and stores.
// `post_load(c, v)` runs on the 32 raw accumulator values of chunk c before the fused ops (stream-K owners add the
// other CTAs' partial sums there).
template <int kBN, int kAct, class Early, class Release, class PostLoad>
__device__ __forceinline__ void epilogue_store_tile_from(uint32_t tmem_tile, const EpilogueArgs& ea,
                                                         const CUtensorMap* tmap_d, uint8_t* stage, int row0, int col0,
                                                         int lane, uint32_t& chunk_counter, int first_chunk,
                                                         Early early, Release release, PostLoad post_load) {
    const int row = row0 + lane;
    const bool row_ok = row < ea.M;
    const __nv_bfloat16* r_row = (ea.residual && row_ok) ? ea.residual + (long long)row * ea.ldr : nullptr;
    constexpr int kChunks = kBN / 32;
#pragma unroll 1
    for (int i = 0; i < kChunks; ++i) {
        int c = first_chunk + i;
        if (c >= kChunks) c -= kChunks;
        const int n0 = col0 + c * 32;
        if (n0 >= ea.N) {                       // whole chunk beyond the matrix: nothing to store
            if (i == 0) early();
            if (i == kChunks - 1) release();
            continue;
        }
        uint32_t v[32];
        tmem_ld_32x32(tmem_tile + c * 32, v);
        tmem_ld_wait();
        if (i == 0) early();
        if (i == kChunks - 1) release();
        post_load(c, v);

        // fused ops in place: v[] holds the finished float32 values afterwards
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int n = n0 + q * 8;
            float x[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(v[q * 8 + e]);
            const bool col_ok = n < ea.N;              // N is a multiple of 8
            if (ea.bias && col_ok) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(ea.bias + n));
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    x[2 * e] += __uint_as_float(bw[e] << 16);
                    x[2 * e + 1] += __uint_as_float(bw[e] & 0xFFFF0000u);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = apply_act<kAct>(x[e]);
            if (r_row && col_ok) {
                const uint4 rv = *reinterpret_cast<const uint4*>(r_row + n);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    x[2 * e] += __uint_as_float(rw[e] << 16);
                    x[2 * e + 1] += __uint_as_float(rw[e] & 0xFFFF0000u);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) v[q * 8 + e] = __float_as_uint(x[e]);
        }

        const int sw = (lane >> 1) & 3;                // 64-byte swizzle: 16-byte slot ^= (row / 2) % 4
        if (ea.out_type == OUT_F32) {
            // 4-byte outputs: the chunk leaves as two 32 x 16 blocks (64-byte rows, like the 16-bit case)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (n0 + 16 * h >= ea.N) break;
                uint8_t* block = stage + (chunk_counter & 1) * (32 * 64);
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                uint8_t* my_row = block + lane * 64;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    *reinterpret_cast<uint4*>(my_row + ((q ^ sw) << 4)) =
                        make_uint4(v[h * 16 + q * 4], v[h * 16 + q * 4 + 1], v[h * 16 + q * 4 + 2], v[h * 16 + q * 4 + 3]);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(tmap_d, block, n0 + 16 * h, row0);
                    tma_store_commit();
                }
                ++chunk_counter;
            }
            continue;
        }

        if (ea.out_type == OUT_MX_E4M3) {
            // this thread's 32 columns are one MX group of its row: scale from the largest magnitude, then the codes,
            // by the rules of the stand-alone quantiser (quant_mx_kernel)
            uint32_t m = 0;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                if (n0 + (e & ~7) >= ea.N) v[e] = 0;                  // columns beyond the matrix do not exist
                m = max(m, v[e] & 0x7FFFFFFFu);
            }
            const bool has_nan = m > 0x7F800000u;
            float amax = __uint_as_float(m);
            if (has_nan) {
                amax = 0.0f;
#pragma unroll
                for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(__uint_as_float(v[e])));
            }
            const int field = (__float_as_uint(amax) >> 23) & 0xFF;
            int byte = min(max(field - 8, 0), 254);
            if (amax == 0.0f) byte = 127;
            const int eff = byte;
            if (has_nan) byte = 255;
            const float inv =
                (eff == 254) ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(254 - eff) << 23);
            uint32_t codes[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                codes[e] = cvt_e4m3x4_sat(__uint_as_float(v[4 * e]) * inv, __uint_as_float(v[4 * e + 1]) * inv,
                                          __uint_as_float(v[4 * e + 2]) * inv, __uint_as_float(v[4 * e + 3]) * inv);
            }
            if (row_ok) {
                const int g = n0 >> 5;
                uint8_t* srow = ea.scale_d + (long long)row * ea.scale_cols_d;
                srow[g] = (uint8_t)byte;
                if (n0 + 32 >= ea.N && g + 1 < ea.scale_cols_d) srow[g + 1] = 127;      // pad column of an odd count
            }
            uint8_t* block = stage + (chunk_counter & 1) * (32 * 64);
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
            uint8_t* my_row = block + lane * 32;                      // 32 rows x 32 bytes, no swizzle
            *reinterpret_cast<uint4*>(my_row) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
            *reinterpret_cast<uint4*>(my_row + 16) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(tmap_d, block, n0, row0);
                tma_store_commit();
            }
            ++chunk_counter;
            continue;
        }

        uint32_t packed[16];
        if (ea.out_type == OUT_F16) {
#pragma unroll
            for (int e = 0; e < 16; ++e) packed[e] = pack_f16(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) packed[e] = pack_bf16(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
        }

        // staging block: make sure TMA has finished reading it (at most one younger store may still be in flight)
        uint8_t* block = stage + (chunk_counter & 1) * (32 * 64);
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* my_row = block + lane * 64;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            *reinterpret_cast<uint4*>(my_row + ((q ^ sw) << 4)) =
                make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(tmap_d, block, n0, row0);
            for (int q = 0; q < ea.n_peers; ++q) tma_store_2d(ea.peer_maps + q, block, n0, row0);
            tma_store_commit();
        }
        ++chunk_counter;
    }
}

// The common case: chunks in ascending order, one release at the end.
template <int kBN, int kAct, class Release>
__device__ __forceinline__ void epilogue_store_tile(uint32_t tmem_tile, const EpilogueArgs& ea,
                                                    const CUtensorMap* tmap_d, uint8_t* stage, int row0, int col0,
                                                    int lane, uint32_t& chunk_counter, Release release) {
    epilogue_store_tile_from<kBN, kAct>(tmem_tile, ea, tmap_d, stage, row0, col0, lane, chunk_counter, 0, []() {},
                                        release, [](int, uint32_t (&)[32]) {});
}

template <int kBN, int kAct, class Early, class Release>
__device__ __forceinline__ void epilogue_store_tile_from(uint32_t tmem_tile, const EpilogueArgs& ea,
                                                         const CUtensorMap* tmap_d, uint8_t* stage, int row0, int col0,
                                                         int lane, uint32_t& chunk_counter, int first_chunk,
                                                         Early early, Release release) {
    epilogue_store_tile_from<kBN, kAct>(tmem_tile, ea, tmap_d, stage, row0, col0, lane, chunk_counter, first_chunk, early,
                                        release, [](int, uint32_t (&)[32]) {});
}

// To be called by lane 0 of every epilogue warp before the kernel ends.
__device__ __forceinline__ void epilogue_drain_stores() { tma_store_wait<0>(); }

}  // namespace blaze
