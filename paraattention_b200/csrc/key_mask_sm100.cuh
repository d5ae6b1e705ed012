// Key-padding mask for the attention kernel: a boolean mask over key rows, one byte per key as
// PyTorch stores torch.bool, packed into 64-bit words per (batch, chunk) so that a softmax
// thread fetches the 64 keys of its half tile with one load.
#pragma once
#include <cstdint>

namespace pa {

// One warp per output word. mask is [batch][n_chunks * rows] bytes (batch stride given);
// out is [batch][n_chunks][words] with words = ceil(rows / 64); bits past `rows` are zero.
__global__ void pack_key_mask_kernel(const uint8_t* __restrict__ mask, long long batch_stride, int batch,
                                     int n_chunks, int rows, unsigned long long* __restrict__ out) {
    const int words = (rows + 63) / 64;
    const long long total = static_cast<long long>(batch) * n_chunks * words;
    const int lane = threadIdx.x & 31;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long w = warp0; w < total; w += n_warps) {
        const int word = static_cast<int>(w % words);
        const long long t = w / words;
        const int chunk = static_cast<int>(t % n_chunks);
        const int b = static_cast<int>(t / n_chunks);
        const uint8_t* src = mask + b * batch_stride + static_cast<long long>(chunk) * rows;
        const int r0 = word * 64 + lane;
        const int r1 = r0 + 32;
        const bool lo = r0 < rows && src[r0] != 0;
        const bool hi = r1 < rows && src[r1] != 0;
        const unsigned long long blo = __ballot_sync(0xffffffffu, lo);
        const unsigned long long bhi = __ballot_sync(0xffffffffu, hi);
        if (lane == 0) out[w] = blo | (bhi << 32);
    }
}

}  // namespace pa
