// TaylorSeer for the First Block Cache (HBM-bound, 16-byte vector accesses).
//
// The cached residual Y of the skipped blocks is extrapolated instead of being reused as is:
// on a computed step finite differences give derivative estimates
//     d_0 = Y,   d_{i+1} = (d_i - prev_i) / window
// and on a skipped step the residual is the Taylor sum
//     sum_i  d_i * elapsed^i / i!
// Each kernel is one pass over the tensors; the intermediate roundings to the tensors' 16-bit
// type are the ones a chain of separate tensor operations would make, so results are the
// same bit for bit.
#pragma once
#include <cstdint>

#include "fbc_sm100.cuh"

namespace pa {

constexpr int kTaylorMaxOrder = 5;  // d_0 .. d_4

// a / w rounded to nearest (the value of an IEEE division) without the general division
// sequence: w is a small positive integer whose reciprocal rw is correctly rounded, so two
// residual corrections of a * rw land on the correctly rounded quotient; operands outside a
// comfortable range take the IEEE path.
__device__ __forceinline__ float div_rn_by_small(float a, float w, float rw) {
    const float mag = fabsf(a);
    if (a != 0.0f && !(mag > 1e-30f && mag < 1e30f)) return __fdiv_rn(a, w);
    float q = a * rw;
    float r = __fmaf_rn(-q, w, a);
    q = __fmaf_rn(r, rw, q);
    r = __fmaf_rn(-q, w, a);
    return __fmaf_rn(r, rw, q);
}

struct TaylorUpdateParams {
    const uint4* y;                          // d_0 of this step
    const uint4* prev[kTaylorMaxOrder - 1];  // d_0 .. d_{depth-1} of the previous computed step
    uint4* cur[kTaylorMaxOrder - 1];         // receives d_1 .. d_depth of this step
    int depth;
    float window;
    long long n8;                            // number of 8-element vectors
};

template <bool kBF16>
__global__ void __launch_bounds__(kFbcThreads)
taylor_update_kernel(const __grid_constant__ TaylorUpdateParams p) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const float rw = __frcp_rn(p.window);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n8; i += stride) {
        // all loads first: the stores below must not hold back the later loads
        uint4 d = __ldg(p.y + i);
        uint4 pv[kTaylorMaxOrder - 1];
#pragma unroll
        for (int k = 0; k < kTaylorMaxOrder - 1; ++k)
            if (k < p.depth) pv[k] = __ldg(p.prev[k] + i);
        uint32_t* dw = reinterpret_cast<uint32_t*>(&d);
#pragma unroll
        for (int k = 0; k < kTaylorMaxOrder - 1; ++k) {
            if (k < p.depth) {
                const uint32_t* pw = reinterpret_cast<const uint32_t*>(&pv[k]);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    // (d - prev) is a tensor of the 16-bit type, so is the quotient
                    const float lo = round16<kBF16>(lo16<kBF16>(dw[w]) - lo16<kBF16>(pw[w]));
                    const float hi = round16<kBF16>(hi16<kBF16>(dw[w]) - hi16<kBF16>(pw[w]));
                    dw[w] = pack16<kBF16>(div_rn_by_small(lo, p.window, rw), div_rn_by_small(hi, p.window, rw));
                }
                __stcs(p.cur[k] + i, d);  // streaming store: not read again by this kernel
            }
        }
    }
}

struct TaylorApproxParams {
    const uint4* d[kTaylorMaxOrder];  // d_0 .. d_{terms-1}
    float coef[kTaylorMaxOrder];      // 1 / i!
    float power[kTaylorMaxOrder];     // elapsed^i
    int terms;
    const uint4* add;                 // optional: the tensor the extrapolated residual is added to
    uint4* out;
    long long n8;
};

template <bool kBF16>
__global__ void __launch_bounds__(kFbcThreads)
taylor_approx_kernel(const __grid_constant__ TaylorApproxParams p) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n8; i += stride) {
        const uint4 d0 = __ldg(p.d[0] + i);
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&d0);
        float acc[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            acc[2 * w] = lo16<kBF16>(w0[w]);   // the i = 0 term is d_0 itself
            acc[2 * w + 1] = hi16<kBF16>(w0[w]);
        }
#pragma unroll
        for (int k = 1; k < kTaylorMaxOrder; ++k) {
            if (k < p.terms) {
                const uint4 dk = __ldg(p.d[k] + i);
                const uint32_t* wk = reinterpret_cast<const uint32_t*>(&dk);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    // ((1/k!) * d_k) * elapsed^k, each product a tensor of the 16-bit type, then the sum
                    const float lo = round16<kBF16>(round16<kBF16>(p.coef[k] * lo16<kBF16>(wk[w])) * p.power[k]);
                    const float hi = round16<kBF16>(round16<kBF16>(p.coef[k] * hi16<kBF16>(wk[w])) * p.power[k]);
                    acc[2 * w] = round16<kBF16>(acc[2 * w] + lo);
                    acc[2 * w + 1] = round16<kBF16>(acc[2 * w + 1] + hi);
                }
            }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
        if (p.add != nullptr) {
            const uint4 a = __ldg(p.add + i);
            const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
#pragma unroll
            for (int w = 0; w < 4; ++w)
                ow[w] = pack16<kBF16>(acc[2 * w] + lo16<kBF16>(aw[w]), acc[2 * w + 1] + hi16<kBF16>(aw[w]));
        } else {
#pragma unroll
            for (int w = 0; w < 4; ++w) ow[w] = pack16<kBF16>(acc[2 * w], acc[2 * w + 1]);
        }
        __stcs(p.out + i, o);  // streaming store: not read again by this kernel
    }
}

}  // namespace pa
