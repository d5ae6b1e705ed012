// First-Block-Cache kernels (HBM-bound, 16-byte vector accesses, deterministic reductions).
//
// fbc_residual_diff_kernel fuses what the reference does in ~8 elementwise/reduction passes:
//   cur  = bf16(h1 - h0)                       first-block residual
//   sums = ( sum |bf16(prev - cur)| , sum |prev| )   accumulated in fp32
// and optionally stores cur as the next step's prev. Per-CTA partial sums go to caller
// scratch; the last CTA to finish (ticket counter) adds them in a fixed order, so the result
// does not depend on scheduling, and also emits the bf16-rounded means and their bf16 ratio.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace pa {

constexpr int kFbcThreads = 256;
constexpr int kFbcMaxBlocks = 148 * 8;

__device__ __forceinline__ float bf16_round_f(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float f16_round_f(float x) { return __half2float(__float2half_rn(x)); }

template <bool kBF16>
__device__ __forceinline__ float lo16(uint32_t w) {
    if constexpr (kBF16) return __uint_as_float(w << 16);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
}
template <bool kBF16>
__device__ __forceinline__ float hi16(uint32_t w) {
    if constexpr (kBF16) return __uint_as_float(w & 0xffff0000u);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}
template <bool kBF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if constexpr (kBF16) {
        const uint32_t a = __bfloat16_as_ushort(__float2bfloat16_rn(lo));
        const uint32_t b = __bfloat16_as_ushort(__float2bfloat16_rn(hi));
        return a | (b << 16);
    } else {
        const uint32_t a = __half_as_ushort(__float2half_rn(lo));
        const uint32_t b = __half_as_ushort(__float2half_rn(hi));
        return a | (b << 16);
    }
}
template <bool kBF16>
__device__ __forceinline__ float round16(float x) {
    if constexpr (kBF16) return bf16_round_f(x);
    return f16_round_f(x);
}

// result[0] = sum|prev-cur|, [1] = sum|prev|, [2] = rounded mean diff, [3] = rounded mean prev,
// [4] = rounded ratio [2]/[3]. scratch: 2*gridDim.x floats of partials followed by one uint32
// ticket that must be zero before the launch (the kernel leaves it zero again).
template <bool kBF16>
__device__ __forceinline__ void fbc_finish(float acc_d, float acc_p, float* scratch, float* result,
                                           long long count) {
    __shared__ float sh[2][kFbcThreads / 32];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        acc_d += __shfl_xor_sync(0xffffffffu, acc_d, o);
        acc_p += __shfl_xor_sync(0xffffffffu, acc_p, o);
    }
    if (lane == 0) {
        sh[0][warp] = acc_d;
        sh[1][warp] = acc_p;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float d = 0.f, p = 0.f;
        for (int w = 0; w < kFbcThreads / 32; ++w) {
            d += sh[0][w];
            p += sh[1][w];
        }
        scratch[2 * blockIdx.x] = d;
        scratch[2 * blockIdx.x + 1] = p;
        __threadfence();
        unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch + 2 * gridDim.x);
        const unsigned int t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
        if (is_last) {
            __threadfence();
            double dd = 0.0, pp = 0.0;
            const volatile float* vs = scratch;
            for (unsigned int b = 0; b < gridDim.x; ++b) {
                dd += vs[2 * b];
                pp += vs[2 * b + 1];
            }
            const float sd = static_cast<float>(dd), sp = static_cast<float>(pp);
            result[0] = sd;
            result[1] = sp;
            const float md = round16<kBF16>(sd / static_cast<float>(count));
            const float mp = round16<kBF16>(sp / static_cast<float>(count));
            result[2] = md;
            result[3] = mp;
            result[4] = round16<kBF16>(md / mp);
            *ticket = 0u;
        }
    }
}

// Dense case (downsample factor 1): n8 = numel / 8 vectors of 8 elements.
template <bool kBF16>
__global__ void __launch_bounds__(kFbcThreads)
fbc_residual_diff_kernel(const uint4* __restrict__ h1, const uint4* __restrict__ h0,
                         const uint4* __restrict__ prev, uint4* __restrict__ new_resid, long long n8,
                         float* scratch, float* result) {
    float acc_d = 0.f, acc_p = 0.f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
        // (h0 == nullptr: the residual is h1 itself, i.e. the caller compares two given tensors)
        const uint4 a = __ldg(h1 + i), b = h0 != nullptr ? __ldg(h0 + i) : make_uint4(0, 0, 0, 0);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t cw[4];
        float cur[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            cur[2 * k] = round16<kBF16>(lo16<kBF16>(aw[k]) - lo16<kBF16>(bw[k]));
            cur[2 * k + 1] = round16<kBF16>(hi16<kBF16>(aw[k]) - hi16<kBF16>(bw[k]));
            cw[k] = pack16<kBF16>(cur[2 * k], cur[2 * k + 1]);
        }
        if (prev != nullptr) {
            const uint4 p = __ldg(prev + i);
            const uint32_t pw[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float p0 = lo16<kBF16>(pw[k]), p1 = hi16<kBF16>(pw[k]);
                acc_d += fabsf(round16<kBF16>(p0 - cur[2 * k])) + fabsf(round16<kBF16>(p1 - cur[2 * k + 1]));
                acc_p += fabsf(p0) + fabsf(p1);
            }
        }
        if (new_resid != nullptr) __stcs(new_resid + i, make_uint4(cw[0], cw[1], cw[2], cw[3]));
    }
    fbc_finish<kBF16>(acc_d, acc_p, scratch, result, n8 * 8);
}

// Strided case: only every `ds`-th element of the last dimension (length cols) takes part and
// prev / new_resid are compact [rows, cols_ds]. One element per thread iteration.
template <bool kBF16>
__global__ void __launch_bounds__(kFbcThreads)
fbc_residual_diff_strided_kernel(const uint16_t* __restrict__ h1, const uint16_t* __restrict__ h0,
                                 const uint16_t* __restrict__ prev, uint16_t* __restrict__ new_resid,
                                 long long rows, int cols, int ds, float* scratch, float* result) {
    const int cols_ds = (cols + ds - 1) / ds;
    const long long n = rows * cols_ds;
    float acc_d = 0.f, acc_p = 0.f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long r = i / cols_ds;
        const int c = static_cast<int>(i % cols_ds) * ds;
        const long long src = r * cols + c;
        const float cur = round16<kBF16>(lo16<kBF16>(h1[src]) - (h0 != nullptr ? lo16<kBF16>(h0[src]) : 0.f));
        if (prev != nullptr) {
            const float p = lo16<kBF16>(prev[i]);
            acc_d += fabsf(round16<kBF16>(p - cur));
            acc_p += fabsf(p);
        }
        if (new_resid != nullptr) new_resid[i] = static_cast<uint16_t>(pack16<kBF16>(cur, 0.f) & 0xffffu);
    }
    fbc_finish<kBF16>(acc_d, acc_p, scratch, result, n);
}

// out = round16(a + b): residual form (h - h0 with negate) and residual apply (h + resid).
template <bool kBF16, bool kSub>
__global__ void __launch_bounds__(kFbcThreads)
fbc_axpy_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out, long long n8) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 x = __ldcs(a + i), y = __ldcs(b + i);
        const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float l = kSub ? lo16<kBF16>(xw[k]) - lo16<kBF16>(yw[k]) : lo16<kBF16>(xw[k]) + lo16<kBF16>(yw[k]);
            const float h = kSub ? hi16<kBF16>(xw[k]) - hi16<kBF16>(yw[k]) : hi16<kBF16>(xw[k]) + hi16<kBF16>(yw[k]);
            ow[k] = pack16<kBF16>(l, h);
        }
        __stcs(out + i, make_uint4(ow[0], ow[1], ow[2], ow[3]));
    }
}

// The same for sizes or addresses the 16-byte form cannot take: one element per thread iteration.
template <bool kBF16, bool kSub>
__global__ void __launch_bounds__(kFbcThreads)
fbc_axpy_scalar_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b, uint16_t* __restrict__ out,
                       long long n) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float x = lo16<kBF16>(a[i]), y = lo16<kBF16>(b[i]);
        out[i] = static_cast<uint16_t>(pack16<kBF16>(kSub ? x - y : x + y, 0.f) & 0xffffu);
    }
}

}  // namespace pa
