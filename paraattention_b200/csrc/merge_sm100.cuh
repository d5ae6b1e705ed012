// Standalone merge of two partial attention results, the arithmetic of torch's _SDPAMerger
// (out -= sigmoid(lse_b - lse) * (out - out_b); lse -= logsigmoid(lse - lse_b)) as one HBM-bound
// pass. The chunked attention kernel never needs it (its running state stays on chip); it
// exists for callers that hold partial (out, lse) pairs computed separately.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace pa {

template <int kDtype>  // 0 bf16, 1 f16, 2 f32 block_out
__device__ __forceinline__ float load_block(const void* p, long long i) {
    if constexpr (kDtype == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    if constexpr (kDtype == 1) return __half2float(static_cast<const __half*>(p)[i]);
    return static_cast<const float*>(p)[i];
}

// acc_out: fp32 [rows, d]; acc_lse: fp32 [rows]; one warp per row, grid-stride over rows.
template <int kDtype>
__global__ void merge_out_lse_kernel(float* __restrict__ acc_out, float* __restrict__ acc_lse,
                                     const void* __restrict__ blk_out, const float* __restrict__ blk_lse,
                                     long long rows, int d) {
    const int lane = threadIdx.x & 31;
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const float la = acc_lse[r], lb = blk_lse[r];
        const float x = lb - la;
        const float sig = 1.0f / (1.0f + __expf(-x));
        // logsigmoid(la - lb) = -softplus(lb - la)
        const float softplus = fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x)));
        for (int c = lane; c < d; c += 32) {
            const long long i = r * d + c;
            const float a = acc_out[i];
            acc_out[i] = a - sig * (a - load_block<kDtype>(blk_out, i));
        }
        __syncwarp();
        if (lane == 0) acc_lse[r] = la + softplus;
    }
}

}  // namespace pa
