// Internal C++ declarations shared by the kernel translation units and the C-ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace blaze {

struct DeviceContext {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    int* status_word = nullptr;     // device int, zero while no kernel wait has given up
};

// Per-device context of the current device (created on first use; thread-safe).  nullptr if no usable device.
DeviceContext* current_context();

// Bytes of the re-tiled scale-factor array for `rows` x K with tiles of `tile_rows` rows, every 512-byte block
// stored `replicas` times in a row.
inline long long sf_tiled_bytes(int rows, int K, int tile_rows, int replicas = 1) {
    const long long tiles = (rows + tile_rows - 1) / tile_rows;
    const long long k_steps = (K + 127) / 128;
    const long long atoms = (tile_rows + 127) / 128;
    return tiles * k_steps * atoms * replicas * 512;
}

// `elem`: 0 = E4M3, 1 = packed E2M1, 2 = E5M2.
cudaError_t launch_quant_mx(const float* x, long long ldx, int rows, int K, int elem, uint8_t* codes,
                            long long ldc_bytes, uint8_t* scales, int sm_count, cudaStream_t stream);
cudaError_t launch_quant_fp8_1x128(const float* x, long long ldx, int rows, int K, uint8_t* codes, long long ldc,
                                   float* scales, int sm_count, cudaStream_t stream);
cudaError_t launch_quant_fp8_128x128(const float* w, long long ldw, int N, int K, uint8_t* codes, long long ldc,
                                     float* scales, int sm_count, cudaStream_t stream);
// `zero_ptr` / `zero_words`: 32-bit words the same kernel also clears (the stream-K flags of the GEMM that follows).
cudaError_t launch_sf_retile(const uint8_t* in, int rows, int K, int tile_rows, int replicas, uint8_t* out,
                             int sm_count, cudaStream_t stream, int* zero_ptr = nullptr, int zero_words = 0);
cudaError_t launch_e2m1_expand(const uint8_t* in, long long ld_in, int rows, int K, uint8_t* out, long long ld_out,
                               int sm_count, cudaStream_t stream);
// Pre-pass for a B stored [K][N] (N contiguous): its transpose [N][K] and its scales as rows [N][ceil(K/64)*2].
cudaError_t launch_transpose_bytes(const uint8_t* in, long long ld_in, int K, int N, uint8_t* out, long long ld_out,
                                   cudaStream_t stream);
cudaError_t launch_scale_pairs_to_rows(const uint8_t* in, int N, int K, uint8_t* out, int sm_count, cudaStream_t stream);
cudaError_t launch_add_f32(const float* a, const float* c, float* d, long long n, int sm_count, cudaStream_t stream);

}  // namespace blaze
