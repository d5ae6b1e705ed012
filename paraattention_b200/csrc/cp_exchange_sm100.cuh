// Context-parallel exchange: every rank pushes head-slices of its local shards straight into
// the staging buffers of the ranks that will consume them (plain 16-byte peer stores over
// NVLink; no multicast), then bumps an arrival counter on the destination with a
// system-scope release. Consumers wait (bounded) on that counter, either inside the
// attention kernel's TMA producer or with flag_wait_kernel below.
#pragma once
#include <cstdint>

#include "../../include/pa_b200.h"
#include "pa_ptx.cuh"

namespace pa {

struct PushParams {
    pa_push_job jobs[PA_MAX_PUSH_JOBS];
    int n_jobs;
    uint32_t* flag[PA_MAX_CHUNKS];  // per destination, in that destination's memory
    int n_dest;
    int first_dest;   // destinations are served in the order first_dest, first_dest-1, ... (mod n_dest)
    int n_push_ctas;  // fused form only: how many leading CTAs of the attention grid push
};

constexpr int kPushThreads = 256;  // stand-alone kernel: small enough to share an SM
constexpr int kPushUnroll = 4;     // independent 16-byte loads in flight per thread

__device__ __forceinline__ void push_row_ptrs(const pa_push_job& job, long long r, const uint4*& s, uint4*& d) {
    const int row = static_cast<int>(r % job.rows);
    const long long t = r / job.rows;
    const int h = static_cast<int>(t % job.heads);
    const int b = static_cast<int>(t / job.heads);
    s = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(job.src) + b * job.src_stride[0] +
                                       (job.head0 + h) * job.src_stride[1] + row * job.src_stride[2]);
    d = reinterpret_cast<uint4*>(static_cast<uint16_t*>(job.dst) + b * job.dst_stride[0] + h * job.dst_stride[1] +
                                 row * job.dst_stride[2]);
}

// All threads of the calling CTA copy this CTA's share (CTA `cta` of `n_ctas`) of every job
// bound for `dest`, then one thread publishes the arrival with a system-scope release.
// A row of head_dim 128 is 256 B = 16 lanes x 16 B, one of head_dim 64 is 8 lanes. Must be
// called by the whole CTA.
__device__ __forceinline__ void push_to_dest(const PushParams& p, int dest, int cta, int n_ctas) {
    for (int j = 0; j < p.n_jobs; ++j) {
        const pa_push_job& job = p.jobs[j];
        if (job.dest != dest) continue;
        const int lane_bits = (job.head_dim == 64) ? 3 : 4;
        const int lane16 = threadIdx.x & ((1 << lane_bits) - 1);
        const int sub = threadIdx.x >> lane_bits;
        const int rows_per_cta = blockDim.x >> lane_bits;
        const long long step = static_cast<long long>(n_ctas) * rows_per_cta;
        const long long total = static_cast<long long>(job.batch) * job.heads * job.rows;
        for (long long r0 = static_cast<long long>(cta) * rows_per_cta + sub; r0 < total; r0 += step * kPushUnroll) {
            uint4 val[kPushUnroll];
            uint4* dptr[kPushUnroll];
#pragma unroll
            for (int u = 0; u < kPushUnroll; ++u) {
                const long long r = r0 + u * step;
                dptr[u] = nullptr;
                if (r < total) {
                    const uint4* s;
                    push_row_ptrs(job, r, s, dptr[u]);
                    val[u] = __ldg(s + lane16);
                }
            }
#pragma unroll
            for (int u = 0; u < kPushUnroll; ++u)
                if (dptr[u] != nullptr) dptr[u][lane16] = val[u];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && p.flag[dest] != nullptr) {
        __threadfence_system();
        red_release_sys_add(p.flag[dest], 1u);
    }
}

// Stand-alone form: grid = (ctas_per_dest, n_dest).
__global__ void __launch_bounds__(kPushThreads, 6)
cp_push_kernel(const __grid_constant__ PushParams p) {
    push_to_dest(p, blockIdx.y, blockIdx.x, gridDim.x);
}

struct FlagWaitParams {
    const uint32_t* flag[PA_MAX_CHUNKS];
    int n;
    uint32_t expect;
    int* status;
    unsigned long long wait_ns;
    int code;
};

// One thread per counter; returns when all counters reached `expect` or the limit ran out
// (then the status word receives `code`). Kernels launched after it on the same stream see
// everything the counters' writers published before their release.
__global__ void flag_wait_kernel(const __grid_constant__ FlagWaitParams p) {
    if (threadIdx.x < p.n && p.flag[threadIdx.x] != nullptr) {
        flag_wait_ge(p.flag[threadIdx.x], p.expect, nullptr, p.status, p.wait_ns, p.code);
    }
    __threadfence_system();
}

}  // namespace pa
