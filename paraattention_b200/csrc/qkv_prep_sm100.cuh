// The neighbours of attention in a diffusion-transformer block, fused into one HBM-bound pass:
// per-head RMSNorm of q and k (with a learned per-channel weight), rotary position embedding
// of both, and the placement of q, k and v into the [batch, rows, heads, head_dim] buffers the
// attention call reads (a dual-stream block writes its text and image streams into one joint
// buffer this way, so the torch.cat of the eager sequence disappears as well).
//
// One warp per (batch, row, head): head_dim 128 = 4 consecutive elements per lane, 64 = 2, so
// the rotary pairs (2i, 2i+1) never straddle lanes. Rounding points follow the eager sequence
//   n = round(x * rsqrt(mean(x^2) + eps));  w = round(n * weight);
//   out = round(w * cos + rot(w) * sin)      (two fp32 products and one fp32 sum, no fma)
// so that results agree with it to the last bit except where the mean's summation order shows.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "fbc_sm100.cuh"  // lo16 / hi16 / pack16 / round16

namespace pa {

struct QkvPrepParams {
    const uint16_t* src[3];   // q, k, v projections (v may be NULL)
    uint16_t* dst[3];
    long long s_sb[3], s_ss[3], s_sh[3];  // element strides (batch, row, head) of the sources
    long long d_sb[3], d_ss[3], d_sh[3];  // ... of the destinations
    const uint16_t* w[2];     // RMSNorm weights of q and k, [head_dim] in the tensors' dtype, or NULL
    const float* cos;         // [table rows, head_dim] fp32, or NULL (no rotary embedding)
    const float* sin;
    long long table_row0;     // row of the tables that belongs to row 0 of this call
    int batch, rows, heads;
    float eps;
};

constexpr int kPrepThreads = 256;

template <bool kBF16, int kD>
__global__ void __launch_bounds__(kPrepThreads)
qkv_prep_kernel(const __grid_constant__ QkvPrepParams p) {
    constexpr int kPer = kD / 32;  // elements per lane: 4 or 2
    const int lane = threadIdx.x & 31;
    const long long warps = static_cast<long long>(gridDim.x) * (kPrepThreads / 32);
    const long long total = static_cast<long long>(p.batch) * p.rows * p.heads;
    for (long long idx = static_cast<long long>(blockIdx.x) * (kPrepThreads / 32) + (threadIdx.x >> 5); idx < total;
         idx += warps) {
        const int h = static_cast<int>(idx % p.heads);
        const long long t = idx / p.heads;
        const int row = static_cast<int>(t % p.rows);
        const int b = static_cast<int>(t / p.rows);
        float cs[kPer], sn[kPer];
        if (p.cos != nullptr) {
            const long long off = (p.table_row0 + row) * kD + lane * kPer;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                cs[i] = __ldg(p.cos + off + i);
                sn[i] = __ldg(p.sin + off + i);
            }
        }
#pragma unroll
        for (int which = 0; which < 3; ++which) {
            if (p.src[which] == nullptr) continue;
            const uint16_t* s = p.src[which] + b * p.s_sb[which] + row * p.s_ss[which] + h * p.s_sh[which] + lane * kPer;
            uint16_t* d = p.dst[which] + b * p.d_sb[which] + row * p.d_ss[which] + h * p.d_sh[which] + lane * kPer;
            uint32_t raw[kPer / 2];
            if (kPer == 4) {
                const uint2 v = *reinterpret_cast<const uint2*>(s);
                raw[0] = v.x;
                raw[kPer / 2 - 1] = v.y;
            } else {
                raw[0] = *reinterpret_cast<const uint32_t*>(s);
            }
            if (which < 2) {
                float x[kPer];
#pragma unroll
                for (int i = 0; i < kPer / 2; ++i) {
                    x[2 * i] = lo16<kBF16>(raw[i]);
                    x[2 * i + 1] = hi16<kBF16>(raw[i]);
                }
                if (p.w[which] != nullptr) {
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < kPer; ++i) ss += x[i] * x[i];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    const float rs = rsqrtf(ss / static_cast<float>(kD) + p.eps);
#pragma unroll
                    for (int i = 0; i < kPer; ++i) {
                        const float wgt = lo16<kBF16>(p.w[which][lane * kPer + i]);
                        x[i] = round16<kBF16>(__fmul_rn(round16<kBF16>(__fmul_rn(x[i], rs)), wgt));
                    }
                }
                if (p.cos != nullptr) {
#pragma unroll
                    for (int i = 0; i < kPer; i += 2) {
                        const float a = x[i], c = x[i + 1];
                        x[i] = round16<kBF16>(__fadd_rn(__fmul_rn(a, cs[i]), __fmul_rn(-c, sn[i])));
                        x[i + 1] = round16<kBF16>(__fadd_rn(__fmul_rn(c, cs[i + 1]), __fmul_rn(a, sn[i + 1])));
                    }
                }
#pragma unroll
                for (int i = 0; i < kPer / 2; ++i) raw[i] = pack16<kBF16>(x[2 * i], x[2 * i + 1]);
            }
            if (kPer == 4) {
                *reinterpret_cast<uint2*>(d) = make_uint2(raw[0], raw[kPer / 2 - 1]);
            } else {
                *reinterpret_cast<uint32_t*>(d) = raw[0];
            }
        }
    }
}

}  // namespace pa
