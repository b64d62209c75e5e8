// Q1-Q3 and the small data-layout kernels around the GEMMs.  All of them are HBM-bound streaming kernels: loads and
// stores are 16-byte (or the widest the element allows) and fully coalesced per warp, grids are sized in multiples
// of the SM count.
//
//   quant_mx          fp32 -> E4M3 or packed E2M1 codes + one E8M0 byte per 32 K        (MX formats)
//   quant_fp8_1x128   fp32 -> E4M3 codes + one fp32 scale per 128 K of each row          (activations)
//   quant_fp8_128x128 fp32 -> E4M3 codes + one fp32 scale per 128x128 block              (weights)
//   sf_retile         row-major E8M0 scale rows -> the 32x16-byte blocks the tensor core's scale copy reads
//   e2m1_expand       packed E2M1 -> E4M3 codes holding the same values                  (W4 weight pre-pass)
//   add_f32           D = A + C                                                          (the one elementwise op)
//
// Rounding is IEEE round-to-nearest-even with saturation; divisions are IEEE (__fdiv_rn), so results are bit-equal
// to the numpy oracle.  Scale layouts are the reference's: `[rows][ceil(K/64)*2]` bytes for MX
// (include/blaze/gemm/kernel/kernel_qbmm_mx.h:383-385), low nibble = even K index for packed E2M1
// (include/blaze/gemm/tile/arch35/shift_w4_to_w8.h:88-99).
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "launch.h"

namespace blaze {

// Four floats -> four E4M3 bytes (x in the low byte), two conversions of a pair each.
__device__ __forceinline__ uint32_t cvt_e4m3x4(float x, float y, float z, float w) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x, y), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(z, w), __NV_SATFINITE, __NV_E4M3);
    return (lo & 0xFFFFu) | (hi << 16);
}

// Four floats -> four E5M2 bytes.
__device__ __forceinline__ uint32_t cvt_e5m2x4(float x, float y, float z, float w) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x, y), __NV_SATFINITE, __NV_E5M2);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(z, w), __NV_SATFINITE, __NV_E5M2);
    return (lo & 0xFFFFu) | (hi << 16);
}

// Four floats -> four E2M1 nibbles (x in the lowest).
__device__ __forceinline__ uint16_t cvt_e2m1x4(float x, float y, float z, float w) {
    const uint32_t lo = __nv_cvt_float2_to_fp4x2(make_float2(x, y), __NV_E2M1, cudaRoundNearest);
    const uint32_t hi = __nv_cvt_float2_to_fp4x2(make_float2(z, w), __NV_E2M1, cudaRoundNearest);
    return (uint16_t)((lo & 0xFFu) | ((hi & 0xFFu) << 8));
}

// w = q * d + r.  Work-item counts almost always fit 32 bits, where the division is a handful of instructions
// instead of the 64-bit software routine.
__device__ __forceinline__ void split_index(long long w, int d, int& q, int& r) {
    if ((unsigned long long)w <= 0xFFFFFFFFull) {
        const uint32_t w32 = (uint32_t)w;
        q = (int)(w32 / (uint32_t)d);
        r = (int)(w32 - (uint32_t)q * (uint32_t)d);
    } else {
        q = (int)(w / d);
        r = (int)(w - (long long)q * d);
    }
}

// ---------------------------------------------------------------------------------------------------- MX

// A warp's work item is kQuantUnroll consecutive 128-wide chunks of one row (2 KB of fp32): all of its 16-byte loads
// are issued before the first conversion, which keeps enough bytes in flight per SM to cover HBM latency, and the
// row/column split of the item index is paid once per item.
constexpr int kQuantUnroll = 4;

// Within a chunk 8 lanes share a group of 32, 4 floats per lane.
// kElem: 0 = E4M3, 1 = packed E2M1, 2 = E5M2 (the values of blazeElem_t).
template <int kElem>
__global__ void __launch_bounds__(256) quant_mx_kernel(const float* __restrict__ x, long long ldx, int rows, int K,
                                                       uint8_t* __restrict__ codes, long long ldc_bytes,
                                                       uint8_t* __restrict__ scales, int scale_cols) {
    const int chunks_per_row = (K + 127) >> 7;
    const int items_per_row = (chunks_per_row + kQuantUnroll - 1) / kQuantUnroll;
    const long long total = (long long)rows * items_per_row;
    const int lane = threadIdx.x & 31;
    constexpr bool kE2M1 = kElem == 1;
    const int emax = kE2M1 ? 2 : (kElem == 2 ? 15 : 8);
    const int n_groups = (K + 31) >> 5;
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += stride) {
        int row, item;
        split_index(w, items_per_row, row, item);
        const int k0 = item * (128 * kQuantUnroll) + lane * 4;
        const float* src = x + (long long)row * ldx + k0;
        float4 vals[kQuantUnroll];
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u) {
            vals[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + u * 128 < K) vals[u] = __ldcs(reinterpret_cast<const float4*>(src + u * 128));   // K % 4 == 0
        }
        uint8_t* code_row = codes + (long long)row * ldc_bytes;
        uint8_t* scale_row = scales + (long long)row * scale_cols;
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u) {
            const int chunk = item * kQuantUnroll + u;
            if (chunk >= chunks_per_row) break;                            // uniform over the warp
            const int k = k0 + u * 128;
            const float4 v = vals[u];
            // |x| as integers order like the floats, with every NaN above infinity: one max finds both the largest
            // magnitude and whether the group holds a NaN
            uint32_t m = max(max(__float_as_uint(v.x) & 0x7FFFFFFFu, __float_as_uint(v.y) & 0x7FFFFFFFu),
                             max(__float_as_uint(v.z) & 0x7FFFFFFFu, __float_as_uint(v.w) & 0x7FFFFFFFu));
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
            const bool has_nan = m > 0x7F800000u;
            float amax = __uint_as_float(m);
            if (__any_sync(0xffffffffu, has_nan)) {
                // rare: the scale of a group with NaNs comes from its largest finite magnitude (fmaxf drops NaNs)
                amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            }
            const int field = (__float_as_uint(amax) >> 23) & 0xFF;
            int byte = min(max(field - emax, 0), 254);
            if (amax == 0.0f) byte = 127;
            const int eff = byte;
            if (has_nan) byte = 255;
            const float inv =
                (eff == 254) ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(254 - eff) << 23);
            const float q0 = v.x * inv, q1 = v.y * inv, q2 = v.z * inv, q3 = v.w * inv;
            if (k < K) {
                if (kE2M1) {
                    *reinterpret_cast<uint16_t*>(code_row + (k >> 1)) = cvt_e2m1x4(q0, q1, q2, q3);
                } else if (kElem == 2) {
                    *reinterpret_cast<uint32_t*>(code_row + k) = cvt_e5m2x4(q0, q1, q2, q3);
                } else {
                    *reinterpret_cast<uint32_t*>(code_row + k) = cvt_e4m3x4(q0, q1, q2, q3);
                }
            }
            const int g = chunk * 4 + (lane >> 3);
            if ((lane & 7) == 0 && g < scale_cols) scale_row[g] = (g < n_groups) ? (uint8_t)byte : (uint8_t)127;
        }
    }
}

// ---------------------------------------------------------------------------------------------------- FP8, fp32 scales

// One warp per (row, 128-wide K group), kQuantUnroll consecutive groups per work item.
__global__ void __launch_bounds__(256) quant_fp8_1x128_kernel(const float* __restrict__ x, long long ldx, int rows, int K,
                                                              uint8_t* __restrict__ codes, long long ldc,
                                                              float* __restrict__ scales, int k_blocks) {
    const int items_per_row = (k_blocks + kQuantUnroll - 1) / kQuantUnroll;
    const long long total = (long long)rows * items_per_row;
    const int lane = threadIdx.x & 31;
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += stride) {
        int row, item;
        split_index(w, items_per_row, row, item);
        const int k0 = item * (128 * kQuantUnroll) + lane * 4;
        const float* src = x + (long long)row * ldx + k0;
        float4 vals[kQuantUnroll];
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u) {
            vals[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + u * 128 < K) vals[u] = __ldcs(reinterpret_cast<const float4*>(src + u * 128));
        }
        uint8_t* code_row = codes + (long long)row * ldc;
        float* scale_row = scales + (long long)row * k_blocks;
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u) {
            const int kb = item * kQuantUnroll + u;
            if (kb >= k_blocks) break;                                     // uniform over the warp
            const int k = k0 + u * 128;
            const float4 v = vals[u];
            float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 448.0f);
            if (k < K) {
                *reinterpret_cast<uint32_t*>(code_row + k) =
                    cvt_e4m3x4(__fdiv_rn(v.x, scale), __fdiv_rn(v.y, scale), __fdiv_rn(v.z, scale),
                               __fdiv_rn(v.w, scale));
            }
            if (lane == 0) scale_row[kb] = scale;
        }
    }
}

// One CTA (256 threads) per 128x128 block of a K-contiguous weight [N][K]; the block is read twice, the second
// time out of L1/L2.
__global__ void __launch_bounds__(256) quant_fp8_128x128_kernel(const float* __restrict__ w, long long ldw, int N, int K,
                                                                uint8_t* __restrict__ codes, long long ldc,
                                                                float* __restrict__ scales, int n_blocks, int k_blocks) {
    __shared__ float warp_max[8];
    __shared__ float block_scale;
    const long long total = (long long)n_blocks * k_blocks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long b = blockIdx.x; b < total; b += gridDim.x) {
        const int nb = (int)(b / k_blocks);
        const int kb = (int)(b - (long long)nb * k_blocks);
        const int k = kb * 128 + lane * 4;
        float amax = 0.0f;
        for (int r = warp; r < 128; r += 8) {
            const int n = nb * 128 + r;
            if (n < N && k < K) {
                const float4 v = *reinterpret_cast<const float4*>(w + (long long)n * ldw + k);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) warp_max[warp] = amax;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = warp_max[0];
            for (int i = 1; i < 8; ++i) m = fmaxf(m, warp_max[i]);
            block_scale = (m == 0.0f) ? 1.0f : __fdiv_rn(m, 448.0f);
            scales[(long long)kb * n_blocks + nb] = block_scale;
        }
        __syncthreads();
        const float scale = block_scale;
        for (int r = warp; r < 128; r += 8) {
            const int n = nb * 128 + r;
            if (n < N && k < K) {
                const float4 v = *reinterpret_cast<const float4*>(w + (long long)n * ldw + k);
                *reinterpret_cast<uint32_t*>(codes + (long long)n * ldc + k) =
                    cvt_e4m3x4(__fdiv_rn(v.x, scale), __fdiv_rn(v.y, scale), __fdiv_rn(v.z, scale),
                               __fdiv_rn(v.w, scale));
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------------- layout helpers

// out[tile][k_step][atom][replica][lane 0..31][quarter 0..3][kk 0..3] = scale[row][k_step*4 + kk],
// row = tile*tile_rows + atom*128 + quarter*32 + lane; anything outside the matrix is 127 (2^0).  `replicas` is 1,
// or 4 where the kernel copies the block into TMEM without the lane broadcast (one copy per 32-lane quadrant).
__global__ void __launch_bounds__(256) sf_retile_kernel(const uint8_t* __restrict__ in, int rows, int scale_cols,
                                                        int valid_groups, int tile_rows, int k_steps, int replicas,
                                                        uint32_t* __restrict__ out, long long out_words,
                                                        int* __restrict__ zero_ptr, int zero_words) {
    const int atoms = (tile_rows + 127) >> 7;
    // the GEMM that follows may set itself up (barriers, TMEM, descriptors) while this kernel runs; it waits for this
    // grid to finish before it loads the first scale block
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // launched with programmatic stream serialisation itself: the previous kernel in the stream (a GEMM that reads
    // these tiles, or the producer of the scales) must have finished before anything is read or written
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // side job for the GEMM behind this kernel: its stream-K fix-up flags start at zero
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < zero_words; i += gridDim.x * blockDim.x) zero_ptr[i] = 0;
    if ((scale_cols & 15) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
        // 16 scale bytes (four K steps) of one row per thread: one 16-byte load instead of sixteen byte loads from
        // rows that are scale_cols bytes apart; the four words go to the four K steps' blocks, 32 consecutive words
        // per warp and store.
        const int ks_groups = (k_steps + 3) >> 2;
        const long long items = out_words / replicas / k_steps * ks_groups;      // (tile, ks group, atom, lane, quarter)
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < items;
             i += (long long)gridDim.x * blockDim.x) {
            long long r = i;
            const int quarter = (int)(r & 3); r >>= 2;
            const int lane = (int)(r & 31); r >>= 5;
            const int atom = (int)(r % atoms); r /= atoms;
            const int ksg = (int)(r % ks_groups);
            const int tile = (int)(r / ks_groups);
            const int in_tile = atom * 128 + quarter * 32 + lane;
            const int row = tile * tile_rows + in_tile;
            uint32_t w[4] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu};
            if (in_tile < tile_rows && row < rows) {
                const int g0 = ksg * 16;
                if (g0 + 16 <= scale_cols && g0 + 16 <= valid_groups) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(in + (long long)row * scale_cols + g0));
                    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t word = 0;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int g = g0 + u * 4 + kk;
                            const uint32_t b = (g < valid_groups && g < scale_cols) ? in[(long long)row * scale_cols + g] : 127u;
                            word |= b << (8 * kk);
                        }
                        w[u] = word;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int ks = ksg * 4 + u;
                if (ks >= k_steps) break;
                const long long block = (((long long)tile * k_steps + ks) * atoms + atom) * replicas;
                for (int rep = 0; rep < replicas; ++rep) out[((block + rep) * 32 + lane) * 4 + quarter] = w[u];
            }
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < out_words;
         i += (long long)gridDim.x * blockDim.x) {
        long long r = i;
        const int quarter = (int)(r & 3); r >>= 2;
        const int lane = (int)(r & 31); r >>= 5;
        r /= replicas;
        const int atom = (int)(r % atoms); r /= atoms;
        const int ks = (int)(r % k_steps);
        const int tile = (int)(r / k_steps);
        const int in_tile = atom * 128 + quarter * 32 + lane;
        const int row = tile * tile_rows + in_tile;
        uint32_t word = 0x7F7F7F7Fu;
        if (in_tile < tile_rows && row < rows) {
            word = 0;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const int g = ks * 4 + kk;
                const uint32_t b = (g < valid_groups && g < scale_cols) ? in[(long long)row * scale_cols + g] : 127u;
                word |= b << (8 * kk);
            }
        }
        out[i] = word;
    }
}

// Each thread turns 8 packed bytes (16 E2M1 values) into 16 E4M3 bytes.
__global__ void __launch_bounds__(256) e2m1_expand_kernel(const uint8_t* __restrict__ in, long long ld_in, int rows,
                                                          int K, uint8_t* __restrict__ out, long long ld_out) {
    const int vec_per_row = K >> 4;           // K is a multiple of 16
    const long long total = (long long)rows * vec_per_row;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // see sf_retile_kernel
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / vec_per_row);
        const int v = (int)(i - (long long)row * vec_per_row);
        const uint2 src = *reinterpret_cast<const uint2*>(in + (long long)row * ld_in + (long long)v * 8);
        const uint32_t words[2] = {src.x, src.y};
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t acc = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t nib = (words[h] >> (16 * q + 4 * e)) & 0xF;
                    const uint32_t mag = nib & 7;
                    // 0, .5, 1, 1.5, 2, 3, 4, 6 as E4M3 codes, one byte per magnitude
                    const uint32_t code = (uint32_t)((0x4C4844403C383000ull >> (8 * mag)) & 0xFF) | ((nib & 8) << 4);
                    acc |= code << (8 * e);
                }
                o[h * 2 + q] = acc;
            }
        }
        *reinterpret_cast<uint4*>(out + (long long)row * ld_out + (long long)v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(256) add_f32_kernel(const float* __restrict__ a, const float* __restrict__ c,
                                                      float* __restrict__ d, long long n) {
    const long long n4 = n >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d)) & 15) == 0;
    if (aligned) {
        for (long long i = tid; i < n4; i += stride) {
            const float4 x = reinterpret_cast<const float4*>(a)[i];
            const float4 y = reinterpret_cast<const float4*>(c)[i];
            reinterpret_cast<float4*>(d)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
        }
        for (long long i = n4 * 4 + tid; i < n; i += stride) d[i] = a[i] + c[i];
    } else {
        for (long long i = tid; i < n; i += stride) d[i] = a[i] + c[i];
    }
}

// in [K][ld_in] bytes (N contiguous) -> out [N][ld_out] bytes (K contiguous), 64 x 64 tiles through shared memory.
__global__ void __launch_bounds__(256) transpose_bytes_kernel(const uint8_t* __restrict__ in, long long ld_in, int K, int N,
                                                              uint8_t* __restrict__ out, long long ld_out) {
    __shared__ uint8_t tile[64][64 + 4];
    const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int kk = i >> 6, nn = i & 63;
        tile[kk][nn] = (k0 + kk < K && n0 + nn < N) ? in[(long long)(k0 + kk) * ld_in + n0 + nn] : (uint8_t)0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int nn = i >> 6, kk = i & 63;
        if (n0 + nn < N && k0 + kk < K) out[(long long)(n0 + nn) * ld_out + k0 + kk] = tile[kk][nn];
    }
}

// MX scales of an N-major B, stored [scale_cols / 2][N][2] (the two K groups of a pair side by side for every n:
// include/tensor_api/impl/tensor_api/tensor/layout_pattern.h:204-215) -> row-major [N][scale_cols].
__global__ void __launch_bounds__(256) scale_pairs_to_rows_kernel(const uint8_t* __restrict__ in, int N, int scale_cols,
                                                                 uint8_t* __restrict__ out) {
    const long long total = (long long)N * (scale_cols >> 1);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int pair = (int)(i / N);
        const int n = (int)(i - (long long)pair * N);
        const uint16_t v = *reinterpret_cast<const uint16_t*>(in + 2 * i);          // in[pair][n][0..1]
        *reinterpret_cast<uint16_t*>(out + (long long)n * scale_cols + 2 * pair) = v;
    }
}

// ---------------------------------------------------------------------------------------------------- launchers

// Launch with programmatic stream serialisation: the kernel may be scheduled while its predecessor in the stream is
// still running, and waits for it (griddepcontrol.wait) before it touches memory.
template <class... KArgs, class... Args>
static cudaError_t launch_programmatic(void (*kernel)(KArgs...), int grid, int block, cudaStream_t stream,
                                       const Args&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

cudaError_t launch_transpose_bytes(const uint8_t* in, long long ld_in, int K, int N, uint8_t* out, long long ld_out,
                                   cudaStream_t stream) {
    if (K <= 0 || N <= 0) return cudaSuccess;
    transpose_bytes_kernel<<<dim3((N + 63) / 64, (K + 63) / 64), 256, 0, stream>>>(in, ld_in, K, N, out, ld_out);
    return cudaGetLastError();
}

cudaError_t launch_scale_pairs_to_rows(const uint8_t* in, int N, int K, uint8_t* out, int sm_count, cudaStream_t stream) {
    const int scale_cols = ((K + 63) / 64) * 2;
    if (N <= 0 || scale_cols <= 0) return cudaSuccess;
    long long blocks = ((long long)N * (scale_cols / 2) + 255) / 256;
    if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
    const int grid = (int)blocks;
    scale_pairs_to_rows_kernel<<<grid, 256, 0, stream>>>(in, N, scale_cols, out);
    return cudaGetLastError();
}

static int grid_for(long long work_items, int per_block, int sm_count) {
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = (long long)sm_count * 8;          // a multiple of the SM count
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

cudaError_t launch_quant_mx(const float* x, long long ldx, int rows, int K, int elem, uint8_t* codes,
                            long long ldc_bytes, uint8_t* scales, int sm_count, cudaStream_t stream) {
    if (rows <= 0 || K <= 0) return cudaSuccess;
    const long long warps = (long long)rows * (((K + 127) / 128 + kQuantUnroll - 1) / kQuantUnroll);
    const int grid = grid_for(warps, 8, sm_count);
    const int scale_cols = ((K + 63) / 64) * 2;
    if (elem == 1)
        quant_mx_kernel<1><<<grid, 256, 0, stream>>>(x, ldx, rows, K, codes, ldc_bytes, scales, scale_cols);
    else if (elem == 2)
        quant_mx_kernel<2><<<grid, 256, 0, stream>>>(x, ldx, rows, K, codes, ldc_bytes, scales, scale_cols);
    else
        quant_mx_kernel<0><<<grid, 256, 0, stream>>>(x, ldx, rows, K, codes, ldc_bytes, scales, scale_cols);
    return cudaGetLastError();
}

cudaError_t launch_quant_fp8_1x128(const float* x, long long ldx, int rows, int K, uint8_t* codes, long long ldc,
                                   float* scales, int sm_count, cudaStream_t stream) {
    if (rows <= 0 || K <= 0) return cudaSuccess;
    const int k_blocks = (K + 127) / 128;
    const int grid = grid_for((long long)rows * ((k_blocks + kQuantUnroll - 1) / kQuantUnroll), 8, sm_count);
    quant_fp8_1x128_kernel<<<grid, 256, 0, stream>>>(x, ldx, rows, K, codes, ldc, scales, k_blocks);
    return cudaGetLastError();
}

cudaError_t launch_quant_fp8_128x128(const float* w, long long ldw, int N, int K, uint8_t* codes, long long ldc,
                                     float* scales, int sm_count, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return cudaSuccess;
    const int n_blocks = (N + 127) / 128, k_blocks = (K + 127) / 128;
    const int grid = grid_for((long long)n_blocks * k_blocks, 1, sm_count);
    quant_fp8_128x128_kernel<<<grid, 256, 0, stream>>>(w, ldw, N, K, codes, ldc, scales, n_blocks, k_blocks);
    return cudaGetLastError();
}

cudaError_t launch_sf_retile(const uint8_t* in, int rows, int K, int tile_rows, int replicas, uint8_t* out,
                             int sm_count, cudaStream_t stream, int* zero_ptr, int zero_words) {
    const int scale_cols = ((K + 63) / 64) * 2;
    const int valid_groups = (K + 31) / 32;
    const int k_steps = (K + 127) / 128;
    const long long words = sf_tiled_bytes(rows, K, tile_rows, replicas) / 4;
    if (words <= 0) return cudaSuccess;
    const int grid = grid_for(words, 256, sm_count);
    return launch_programmatic(sf_retile_kernel, grid, 256, stream, in, rows, scale_cols, valid_groups, tile_rows, k_steps,
                               replicas, reinterpret_cast<uint32_t*>(out), words, zero_ptr, zero_ptr ? zero_words : 0);
}

cudaError_t launch_e2m1_expand(const uint8_t* in, long long ld_in, int rows, int K, uint8_t* out, long long ld_out,
                               int sm_count, cudaStream_t stream) {
    if (rows <= 0 || K <= 0) return cudaSuccess;
    const int grid = grid_for((long long)rows * (K / 16), 256, sm_count);
    e2m1_expand_kernel<<<grid, 256, 0, stream>>>(in, ld_in, rows, K, out, ld_out);
    return cudaGetLastError();
}

cudaError_t launch_add_f32(const float* a, const float* c, float* d, long long n, int sm_count, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    const int grid = grid_for((n + 3) / 4, 256, sm_count);
    add_f32_kernel<<<grid, 256, 0, stream>>>(a, c, d, n);
    return cudaGetLastError();
}

}  // namespace blaze
