// C ABI of libpa_b200: argument validation, tensor-map encoding and kernel launches.
// No entry point here allocates device memory or synchronises the device.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/pa_b200.h"
#include "attn_fwd_sm100.cuh"
#include "fbc_sm100.cuh"
#include "key_mask_sm100.cuh"
#include "merge_sm100.cuh"
#include "qkv_prep_sm100.cuh"
#include "taylor_sm100.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// Streaming multiprocessors of the current device (cached per device): grid caps of the
// grid-stride kernels are multiples of it.
int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

// 5-D map over [chunk][batch][head][row][head_dim] with element strides (head_dim stride 1); the box is
// 64 elements x 128 rows with the 128-byte swizzle the MMA descriptors expect.
int make_map(CUtensorMap* map, const void* base, int dtype, int head_dim, int rows, int heads, int batch, int chunks,
             int64_t s_row, int64_t s_head, int64_t s_batch, int64_t s_chunk, const char* what) {
    EncodeTiledFn enc = get_encode_fn();
    if (enc == nullptr) return fail(PA_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return fail(PA_EINVAL, "%s: base pointer must be 16-byte aligned", what);
    cuuint64_t dims[5] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads),
                          static_cast<cuuint64_t>(batch), static_cast<cuuint64_t>(chunks)};
    int64_t es[4] = {s_row, s_head, s_batch, s_chunk};
    cuuint64_t strides[4];
    for (int i = 0; i < 4; ++i) {
        int64_t s = es[i];
        if (dims[i + 1] == 1 && (s <= 0 || (s * 2) % 16 != 0)) s = 128;  // never dereferenced
        if (s <= 0) return fail(PA_EINVAL, "%s: stride %d must be positive", what, i);
        if ((s * 2) % 16 != 0) return fail(PA_EINVAL, "%s: byte stride %d must be a multiple of 16", what, i);
        if (static_cast<uint64_t>(s) * 2 >= (1ull << 40)) return fail(PA_EINVAL, "%s: stride %d too large", what, i);
        strides[i] = static_cast<cuuint64_t>(s) * 2;
    }
    cuuint32_t box[5] = {64, 128, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUtensorMapDataType dt = dtype == PA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = enc(map, dt, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PA_ECUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, int(r));
    return PA_OK;
}

template <bool kBF16, bool kCausal, int kD, bool kSplit = false>
int launch_attn_inst(const CUtensorMap* maps, const pa::AttnParams& p, const pa::PushParams& push, int grid,
                cudaStream_t stream) {
    auto kern = pa::attn_fwd_kernel<kBF16, kCausal, kD, kSplit>;
    static bool configured[64] = {};  // per instantiation and device
    static std::mutex mu;
    {
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> g(mu);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pa::kAttnSmemBytes);
            if (e != cudaSuccess) return fail(PA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    kern<<<grid, pa::kAttnThreads, pa::kAttnSmemBytes, stream>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p, push);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "attention launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

// One launch over all work units, or - when the last wave is split - one over the whole waves
// and a second one in which every remaining unit belongs to split_k CTAs.
template <bool kBF16>
int launch_attn(const CUtensorMap* maps, const pa::AttnParams& p, const pa::PushParams& push, int grid,
                cudaStream_t stream, int head_dim) {
    if (p.split_k > 1) {
        int rc = PA_OK;
        if (p.split_from > 0) {
            pa::AttnParams whole = p;
            whole.split_k = 1;
            rc = launch_attn<kBF16>(maps, whole, push, p.split_from, stream, head_dim);
            if (rc != PA_OK) return rc;
        }
        pa::PushParams tail_push;  // (a launch with pushers is never split)
        memset(&tail_push, 0, sizeof(tail_push));
        const int tail_grid = (grid - p.split_from) * p.split_k;
        pa::AttnParams tail = p;
        tail.unit_base = p.split_from;
        return head_dim == 64 ? launch_attn_inst<kBF16, false, 64, true>(maps, tail, tail_push, tail_grid, stream)
                              : launch_attn_inst<kBF16, false, 128, true>(maps, tail, tail_push, tail_grid, stream);
    }
    if (head_dim == 64) {
        return p.causal ? launch_attn_inst<kBF16, true, 64>(maps, p, push, grid, stream)
                        : launch_attn_inst<kBF16, false, 64>(maps, p, push, grid, stream);
    }
    return p.causal ? launch_attn_inst<kBF16, true, 128>(maps, p, push, grid, stream)
                    : launch_attn_inst<kBF16, false, 128>(maps, p, push, grid, stream);
}

// Split of the last wave. A grid of `units` equally long CTAs on `sms` SMs takes
// ceil(units / sms) rounds although the last round may be nearly empty (384 units on 148 SMs:
// 2.59 rounds of work in the time of 3). With a workspace the units of the last round are each
// given to k CTAs that take 1/k of the key/value tiles and combine their results in the
// kernel's epilogue, so that the last round costs ceil(tail * k / sms) short rounds instead of a
// whole one. Times are modelled from measurements on B200 (both head dims): 1.8 us per
// key/value tile of a CTA plus 16 us per CTA for everything around the tile loop, 26 us for a
// CTA that also exchanges partial results. k is the value in [2, 8] with the lowest modelled
// time that leaves at least 8 tiles per CTA and fits the workspace; nothing is split unless the
// model promises 3 % of the call. Causal runs (units of unequal length, long ones first) are
// left alone, and so are launches led by pushing CTAs (`pushers`): CTAs that push first, or
// wait for a peer's chunk, finish tens of microseconds apart, and the launch of the shares
// starts only when the last of them has finished. Measured with real peers, the split lost:
// 8 GPUs at 256 tiles per unit 1.604 ms against 1.495 ms whole, at 36 tiles 260 us against
// 222 us; 2 GPUs at 36 tiles 257 us against 218 us.
struct TailSplit {
    int from = 0, k = 1;
    long long grid = 0;
    size_t cnt_bytes = 0, ml_bytes = 0, o_bytes = 0;
};

TailSplit plan_tail_split(long long units, int sms, long long kv_tiles, int head_dim, bool causal, bool pushers,
                          int64_t ws_bytes) {
    TailSplit r;
    r.from = int(units);
    r.grid = units;
    if (causal || ws_bytes <= 0 || sms <= 0 || units <= 0) return r;
    const long long tail = units % sms;
    if (tail == 0) return r;
    if (pushers) return r;
    const double t_tile = 1.8, t_cta = 16.0, t_share = 26.0;  // microseconds
    const double t_unit = double(kv_tiles) * t_tile + t_cta;
    const double t_now = double(units / sms + 1) * t_unit;
    double best = t_unit;
    int best_k = 1;
    for (int k = 2; k <= 8; ++k) {
        if (kv_tiles / k < 8) break;
        const size_t need = 256 + size_t(tail) * 9 * 4 + size_t(tail) * k * 256 * (8 + size_t(head_dim) * 4) + 512;
        if (need > size_t(ws_bytes)) break;
        const long long rounds = (tail * k + sms - 1) / sms;
        const double t = double(rounds) * (double((kv_tiles + k - 1) / k) * t_tile + t_share);
        if (t < best - 1e-9) {
            best = t;
            best_k = k;
        }
    }
    if (best_k == 1 || (t_unit - best) / t_now < 0.03) return r;
    r.k = best_k;
    r.from = int(units - tail);
    r.grid = (units - tail) + tail * best_k;
    r.cnt_bytes = (size_t(tail) * 9 * 4 + 255) & ~size_t(255);
    r.ml_bytes = (size_t(tail) * best_k * 256 * 8 + 255) & ~size_t(255);
    r.o_bytes = size_t(tail) * best_k * 256 * size_t(head_dim) * 4;
    return r;
}

// Fills the split fields of `p` and zeroes the counters on the stream; returns the grid size.
int apply_tail_split(pa::AttnParams* p, long long units, long long kv_tiles, int head_dim, bool pushers, void* ws,
                     int64_t ws_bytes, cudaStream_t s, long long* grid) {
    p->split_from = int(units);
    p->split_k = 1;
    *grid = units;
    if (ws == nullptr) return PA_OK;
    if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return fail(PA_EINVAL, "workspace must be 256-byte aligned");
    const TailSplit t = plan_tail_split(units, sm_count(), kv_tiles, head_dim, p->causal != 0, pushers, ws_bytes);
    if (t.k == 1) return PA_OK;
    if ((units - t.from) * t.k > 0x7fffffffLL) return PA_OK;
    uint8_t* base = static_cast<uint8_t*>(ws);
    p->part_cnt = reinterpret_cast<unsigned int*>(base);
    p->part_ml = reinterpret_cast<float2*>(base + t.cnt_bytes);
    p->part_o = reinterpret_cast<float*>(base + t.cnt_bytes + t.ml_bytes);
    p->split_from = t.from;
    p->split_k = t.k;
    cudaError_t e = cudaMemsetAsync(p->part_cnt, 0, t.cnt_bytes, s);
    if (e != cudaSuccess) return fail(PA_ECUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return PA_OK;
}

int check_common(int head_dim, int dtype, float scale) {
    if (head_dim != 128 && head_dim != 64) return fail(PA_ENOTSUP, "head_dim %d: only 64 and 128 are built", head_dim);
    if (dtype != PA_BF16 && dtype != PA_F16) return fail(PA_EINVAL, "dtype %d: expected PA_BF16 or PA_F16", dtype);
    if (!(scale > 0.f) || !std::isfinite(scale)) return fail(PA_EINVAL, "scale must be positive and finite");
    return PA_OK;
}

int out_checks(const void* out, const int64_t* o_stride) {
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return fail(PA_EINVAL, "out: base pointer must be 16-byte aligned");
    for (int i = 0; i < 3; ++i)
        if ((o_stride[i] * 2) % 16 != 0) return fail(PA_EINVAL, "out: byte stride %d must be a multiple of 16", i);
    return PA_OK;
}

int attn_fwd_impl(const pa_attn_args* a, void* stream, long long* dbg_t = nullptr, int dbg_steps = 0) {
    if (a == nullptr) return fail(PA_EINVAL, "args is NULL");
    if (!a->q || !a->k || !a->v || !a->out) return fail(PA_EINVAL, "q, k, v and out must be non-NULL");
    if (a->batch <= 0 || a->heads <= 0 || a->seq_q <= 0 || a->seq_kv <= 0)
        return fail(PA_EINVAL, "batch, heads, seq_q and seq_kv must be positive");
    int rc = check_common(a->head_dim, a->dtype, a->scale);
    if (rc != PA_OK) return rc;
    rc = out_checks(a->out, a->o_stride);
    if (rc != PA_OK) return rc;

    CUtensorMap maps[6];
    CUtensorMap &mq = maps[0], &mk = maps[1], &mv = maps[2];
    rc = make_map(&mq, a->q, a->dtype, a->head_dim, a->seq_q, a->heads, a->batch, 1, a->q_stride[2], a->q_stride[1], a->q_stride[0], 0, "q");
    if (rc != PA_OK) return rc;
    rc = make_map(&mk, a->k, a->dtype, a->head_dim, a->seq_kv, a->heads, a->batch, 1, a->k_stride[2], a->k_stride[1], a->k_stride[0], 0, "k");
    if (rc != PA_OK) return rc;
    rc = make_map(&mv, a->v, a->dtype, a->head_dim, a->seq_kv, a->heads, a->batch, 1, a->v_stride[2], a->v_stride[1], a->v_stride[0], 0, "v");
    if (rc != PA_OK) return rc;

    maps[3] = mq;
    maps[4] = mk;
    maps[5] = mv;
    pa::AttnParams p;
    memset(&p, 0, sizeof(p));
    p.q_local_chunk = -1;
    p.kv_local_chunk = -1;
    p.batch = a->batch;
    p.heads = a->heads;
    p.n_q_chunks = 1;
    p.q_rows = a->seq_q;
    p.n_kv_chunks = 1;
    p.kv_rows = a->seq_kv;
    p.causal = a->is_causal ? 1 : 0;  // both sequences start at position 0: key j visible to query i iff j <= i
    p.scale = a->scale;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.out[0] = a->out;
    p.lse[0] = a->lse;
    p.o_sb = a->o_stride[0];
    p.o_sh = a->o_stride[1];
    p.o_ss = a->o_stride[2];
    p.l_sb = static_cast<long long>(a->heads) * a->seq_q;
    p.l_sh = a->seq_q;
    p.status = a->status;
    p.wait_ns = a->wait_limit_ns ? a->wait_limit_ns : 2000000000ull;
    p.key_bits = reinterpret_cast<const unsigned long long*>(a->key_bits);
    p.kb_sb = (a->seq_kv + 63) / 64;
    p.kb_sc = 0;
#if PA_TIMELINE
    p.dbg_t = dbg_t;
    p.dbg_steps = dbg_steps;
#else
    (void)dbg_t;
    (void)dbg_steps;
#endif

    const long long pairs = (a->seq_q + 255) / 256;
    const long long units = pairs * a->heads * a->batch;
    if (units > 0x7fffffffLL) return fail(PA_EINVAL, "problem too large for one launch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long grid = units;
    rc = apply_tail_split(&p, units, (a->seq_kv + 127) / 128, a->head_dim, false, a->workspace, a->workspace_bytes, s,
                          &grid);
    if (rc != PA_OK) return rc;
    pa::PushParams push;
    memset(&push, 0, sizeof(push));
    return a->dtype == PA_BF16 ? launch_attn<true>(maps, p, push, int(grid), s, a->head_dim)
                               : launch_attn<false>(maps, p, push, int(grid), s, a->head_dim);
}

int fill_push(const pa_cp_push_args* a, pa::PushParams* p) {
    if (a->n_jobs < 0 || a->n_jobs > PA_MAX_PUSH_JOBS) return fail(PA_EINVAL, "n_jobs must be in [0, %d]", PA_MAX_PUSH_JOBS);
    if (a->n_dest < 1 || a->n_dest > PA_MAX_CHUNKS) return fail(PA_EINVAL, "n_dest must be in [1, %d]", PA_MAX_CHUNKS);
    if (a->ctas_per_dest < 1 || a->ctas_per_dest > 1024) return fail(PA_EINVAL, "ctas_per_dest must be in [1, 1024]");
    if (a->first_dest < 0 || a->first_dest >= a->n_dest) return fail(PA_EINVAL, "first_dest out of range");
    memset(p, 0, sizeof(*p));
    for (int j = 0; j < a->n_jobs; ++j) {
        const pa_push_job& job = a->jobs[j];
        if (!job.src || !job.dst) return fail(PA_EINVAL, "job %d: src and dst must be non-NULL", j);
        if (job.dest < 0 || job.dest >= a->n_dest) return fail(PA_EINVAL, "job %d: dest out of range", j);
        if (job.batch <= 0 || job.heads <= 0 || job.rows <= 0 || job.head0 < 0)
            return fail(PA_EINVAL, "job %d: batch, heads, rows must be positive", j);
        if (job.head_dim != 0 && job.head_dim != 64 && job.head_dim != 128)
            return fail(PA_EINVAL, "job %d: head_dim must be 64 or 128 (0 = 128)", j);
        if ((reinterpret_cast<uintptr_t>(job.src) & 15u) || (reinterpret_cast<uintptr_t>(job.dst) & 15u))
            return fail(PA_EINVAL, "job %d: src and dst must be 16-byte aligned", j);
        for (int i = 0; i < 3; ++i)
            if ((job.src_stride[i] * 2) % 16 != 0 || (job.dst_stride[i] * 2) % 16 != 0)
                return fail(PA_EINVAL, "job %d: byte strides must be multiples of 16", j);
        p->jobs[j] = job;
    }
    p->n_jobs = a->n_jobs;
    p->n_dest = a->n_dest;
    p->first_dest = a->first_dest;
    for (int d = 0; d < PA_MAX_CHUNKS; ++d) p->flag[d] = a->flag[d];
    return PA_OK;
}

}  // namespace

extern "C" {

const char* pa_last_error(void) { return g_err; }
int pa_version(void) { return 1; }

int64_t pa_attn_workspace_bytes(void) { return int64_t(64) << 20; }

int pa_attn_split_plan(int64_t units, int32_t sm_count_, int64_t kv_tiles, int32_t head_dim, int32_t is_causal,
                       int32_t fused_push, int64_t workspace_bytes, int32_t* split_from, int32_t* split_k) {
    if (units <= 0 || sm_count_ <= 0 || kv_tiles <= 0 || (head_dim != 64 && head_dim != 128))
        return fail(PA_EINVAL, "units, sm_count and kv_tiles must be positive, head_dim 64 or 128");
    const TailSplit t = plan_tail_split(units, sm_count_, kv_tiles, head_dim, is_causal != 0, fused_push != 0,
                                        workspace_bytes);
    if (split_from != nullptr) *split_from = t.from;
    if (split_k != nullptr) *split_k = t.k;
    return PA_OK;
}

int pa_attn_fwd(const pa_attn_args* args, void* stream) { return attn_fwd_impl(args, stream); }

#if PA_TIMELINE
// Profiling builds only (-DPA_TIMELINE=1; not declared in the public header, not in the shipped
// library): pa_attn_fwd whose first CTA records clock64() stamps of its pipeline phases for the
// first `steps` key/value tiles into stamps[5][steps][8] (softmax of query tile 0, of query
// tile 1, MMA issuer, TMA producer, MMA operand waits).
int pa_timeline_attn_fwd(const pa_attn_args* args, long long* stamps, int steps, void* stream) {
    return attn_fwd_impl(args, stream, stamps, steps);
}
#endif

int pa_cp_attn_fwd(const pa_cp_attn_args* a, void* stream) {
    if (a == nullptr) return fail(PA_EINVAL, "args is NULL");
    if (!a->q_stage || !a->k_stage || !a->v_stage) return fail(PA_EINVAL, "staging pointers must be non-NULL");
    if (a->batch <= 0 || a->heads <= 0 || a->q_rows <= 0 || a->kv_rows <= 0)
        return fail(PA_EINVAL, "batch, heads, q_rows and kv_rows must be positive");
    if (a->n_q_chunks < 1 || a->n_q_chunks > PA_MAX_CHUNKS || a->n_kv_chunks < 1 || a->n_kv_chunks > PA_MAX_CHUNKS)
        return fail(PA_EINVAL, "chunk counts must be in [1, %d]", PA_MAX_CHUNKS);
    if (a->q_first < 0 || a->q_first >= a->n_q_chunks || a->kv_first < 0 || a->kv_first >= a->n_kv_chunks)
        return fail(PA_EINVAL, "q_first / kv_first out of range");
    int rc = check_common(a->head_dim, a->dtype, a->scale);
    if (rc != PA_OK) return rc;
    for (int c = 0; c < a->n_q_chunks; ++c) {
        if (a->out[c] == nullptr) return fail(PA_EINVAL, "out[%d] is NULL", c);
        rc = out_checks(a->out[c], a->o_stride);
        if (rc != PA_OK) return rc;
    }
    CUtensorMap maps[6];
    CUtensorMap &mq = maps[0], &mk = maps[1], &mv = maps[2];
    const int64_t D = a->head_dim;
    const int64_t qs_h = int64_t(a->q_rows) * D, qs_b = qs_h * a->heads, qs_c = qs_b * a->batch;
    const int64_t ks_h = int64_t(a->kv_rows) * D, ks_b = ks_h * a->heads, ks_c = ks_b * a->batch;
    rc = make_map(&mq, a->q_stage, a->dtype, a->head_dim, a->q_rows, a->heads, a->batch, a->n_q_chunks, D, qs_h, qs_b, qs_c, "q_stage");
    if (rc != PA_OK) return rc;
    rc = make_map(&mk, a->k_stage, a->dtype, a->head_dim, a->kv_rows, a->heads, a->batch, a->n_kv_chunks, D, ks_h, ks_b, ks_c, "k_stage");
    if (rc != PA_OK) return rc;
    rc = make_map(&mv, a->v_stage, a->dtype, a->head_dim, a->kv_rows, a->heads, a->batch, a->n_kv_chunks, D, ks_h, ks_b, ks_c, "v_stage");
    if (rc != PA_OK) return rc;

    maps[3] = mq;
    maps[4] = mk;
    maps[5] = mv;
    pa::AttnParams p;
    memset(&p, 0, sizeof(p));
    p.q_local_chunk = -1;
    p.kv_local_chunk = -1;
    if (a->q_local != nullptr || a->k_local != nullptr || a->v_local != nullptr) {
        if (a->local_head_offset < 0 || a->local_total_heads < a->local_head_offset + a->heads)
            return fail(PA_EINVAL, "local_head_offset + heads exceeds local_total_heads");
        p.local_head0 = a->local_head_offset;
    }
    if (a->q_local != nullptr) {
        rc = make_map(&maps[3], a->q_local, a->dtype, a->head_dim, a->q_rows, a->local_total_heads, a->batch, 1, a->q_local_stride[2],
                      a->q_local_stride[1], a->q_local_stride[0], 0, "q_local");
        if (rc != PA_OK) return rc;
        p.q_local_chunk = a->q_first;
    }
    if (a->k_local != nullptr || a->v_local != nullptr) {
        if (a->k_local == nullptr || a->v_local == nullptr) return fail(PA_EINVAL, "k_local and v_local go together");
        rc = make_map(&maps[4], a->k_local, a->dtype, a->head_dim, a->kv_rows, a->local_total_heads, a->batch, 1, a->k_local_stride[2],
                      a->k_local_stride[1], a->k_local_stride[0], 0, "k_local");
        if (rc != PA_OK) return rc;
        rc = make_map(&maps[5], a->v_local, a->dtype, a->head_dim, a->kv_rows, a->local_total_heads, a->batch, 1, a->v_local_stride[2],
                      a->v_local_stride[1], a->v_local_stride[0], 0, "v_local");
        if (rc != PA_OK) return rc;
        p.kv_local_chunk = a->kv_first;
    }
    p.batch = a->batch;
    p.heads = a->heads;
    p.n_q_chunks = a->n_q_chunks;
    p.q_rows = a->q_rows;
    p.q_first = a->q_first;
    p.n_kv_chunks = a->n_kv_chunks;
    p.kv_rows = a->kv_rows;
    p.kv_first = a->kv_first;
    p.causal = a->is_causal ? 1 : 0;
    if (p.causal) {
        for (int c = 0; c < a->n_q_chunks; ++c) {
            if (a->q_pos[c] < 0) return fail(PA_EINVAL, "q_pos[%d] is negative", c);
            p.q_pos[c] = a->q_pos[c];
        }
        for (int c = 0; c < a->n_kv_chunks; ++c) {
            if (a->kv_pos[c] < 0) return fail(PA_EINVAL, "kv_pos[%d] is negative", c);
            p.kv_pos[c] = a->kv_pos[c];
        }
    }
    p.scale = a->scale;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    for (int c = 0; c < PA_MAX_CHUNKS; ++c) {
        // fold the head offset into the base pointers
        p.out[c] = a->out[c] ? static_cast<void*>(static_cast<uint16_t*>(a->out[c]) + int64_t(a->out_head_offset) * a->o_stride[1]) : nullptr;
        p.lse[c] = a->lse[c] ? a->lse[c] + int64_t(a->out_head_offset) * a->lse_stride[1] : nullptr;
        p.q_flag[c] = a->q_flag[c];
        p.kv_flag[c] = a->kv_flag[c];
        p.done_flag[c] = a->done_flag[c];
    }
    p.o_sb = a->o_stride[0];
    p.o_sh = a->o_stride[1];
    p.o_ss = a->o_stride[2];
    p.l_sb = a->lse_stride[0];
    p.l_sh = a->lse_stride[1];
    p.flag_expect = a->flag_expect;
    p.key_bits = reinterpret_cast<const unsigned long long*>(a->key_bits);
    p.kb_sc = (a->kv_rows + 63) / 64;
    p.kb_sb = p.kb_sc * a->n_kv_chunks;
    p.status = a->status;
    p.wait_ns = a->wait_limit_ns ? a->wait_limit_ns : 2000000000ull;

    const long long pairs = (a->q_rows + 255) / 256;
    const long long units = pairs * a->heads * a->batch * a->n_q_chunks;
    if (units > 0x7fffffffLL) return fail(PA_EINVAL, "problem too large for one launch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long grid = units;
    rc = apply_tail_split(&p, units, static_cast<long long>((a->kv_rows + 127) / 128) * a->n_kv_chunks, a->head_dim,
                          a->fused_push != nullptr, a->workspace, a->workspace_bytes, s, &grid);
    if (rc != PA_OK) return rc;
    pa::PushParams push;
    memset(&push, 0, sizeof(push));
    if (a->fused_push != nullptr) {
        rc = fill_push(a->fused_push, &push);
        if (rc != PA_OK) return rc;
        // pushers must all be resident at once: never more than the work units (whatever the
        // split of the last wave makes of them: the peers count on this number) or one wave of SMs
        int n = a->fused_push->ctas_per_dest;
        if (n > units) n = int(units);
        if (n > sm_count()) n = sm_count();
        push.n_push_ctas = n;
    }
    return a->dtype == PA_BF16 ? launch_attn<true>(maps, p, push, int(grid), s, a->head_dim)
                               : launch_attn<false>(maps, p, push, int(grid), s, a->head_dim);
}

int pa_pack_key_mask(const uint8_t* mask, int64_t batch_stride, int32_t batch, int32_t n_chunks, int32_t rows,
                     uint64_t* out, void* stream) {
    if (mask == nullptr || out == nullptr) return fail(PA_EINVAL, "pack_key_mask: NULL pointer");
    if (batch <= 0 || n_chunks <= 0 || rows <= 0) return fail(PA_EINVAL, "pack_key_mask: batch, n_chunks, rows must be positive");
    if (batch_stride < int64_t(n_chunks) * rows) return fail(PA_EINVAL, "pack_key_mask: batch stride shorter than a row of keys");
    const long long total = static_cast<long long>(batch) * n_chunks * ((rows + 63) / 64);
    long long blocks = (total + 7) / 8;  // 8 warps per block
    if (blocks > static_cast<long long>(sm_count()) * 8) blocks = static_cast<long long>(sm_count()) * 8;
    pa::pack_key_mask_kernel<<<int(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        mask, batch_stride, batch, n_chunks, rows, reinterpret_cast<unsigned long long*>(out));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "pack_key_mask launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int pa_cp_push(const pa_cp_push_args* a, void* stream) {
    if (a == nullptr) return fail(PA_EINVAL, "args is NULL");
    pa::PushParams p;
    int rc = fill_push(a, &p);
    if (rc != PA_OK) return rc;
    dim3 grid(a->ctas_per_dest, a->n_dest);
    pa::cp_push_kernel<<<grid, pa::kPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "push launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int pa_flag_wait(const uint32_t* const* flag, int32_t n, uint32_t expect, int32_t* status, uint64_t wait_limit_ns,
                 int32_t code, void* stream) {
    if (flag == nullptr || n < 1 || n > PA_MAX_CHUNKS) return fail(PA_EINVAL, "flag list must hold 1..%d pointers", PA_MAX_CHUNKS);
    pa::FlagWaitParams p;
    memset(&p, 0, sizeof(p));
    for (int i = 0; i < n; ++i) p.flag[i] = flag[i];
    p.n = n;
    p.expect = expect;
    p.status = status;
    p.wait_ns = wait_limit_ns ? wait_limit_ns : 2000000000ull;
    p.code = code;
    pa::flag_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "flag wait launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int pa_merge_out_lse(float* acc_out, float* acc_lse, const void* blk_out, const float* blk_lse, int64_t rows,
                     int32_t d, int32_t blk_dtype, void* stream) {
    if (!acc_out || !acc_lse || !blk_out || !blk_lse) return fail(PA_EINVAL, "merge: NULL pointer");
    if (rows <= 0 || d <= 0) return fail(PA_EINVAL, "merge: rows and d must be positive");
    const int threads = 256;
    long long blocks = (rows + 7) / 8;
    if (blocks > static_cast<long long>(sm_count()) * 16) blocks = static_cast<long long>(sm_count()) * 16;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (blk_dtype) {
        case 0: pa::merge_out_lse_kernel<0><<<int(blocks), threads, 0, s>>>(acc_out, acc_lse, blk_out, blk_lse, rows, d); break;
        case 1: pa::merge_out_lse_kernel<1><<<int(blocks), threads, 0, s>>>(acc_out, acc_lse, blk_out, blk_lse, rows, d); break;
        case 2: pa::merge_out_lse_kernel<2><<<int(blocks), threads, 0, s>>>(acc_out, acc_lse, blk_out, blk_lse, rows, d); break;
        default: return fail(PA_EINVAL, "merge: blk_dtype must be 0 (bf16), 1 (f16) or 2 (f32)");
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "merge launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int64_t pa_fbc_scratch_bytes(void) { return int64_t(2 * pa::kFbcMaxBlocks) * 4 + 4; }

int pa_fbc_residual_diff(const void* h1, const void* h0, const void* prev, void* new_resid, int64_t rows,
                         int32_t cols, int32_t downsample, int32_t dtype, float* result, void* scratch,
                         void* stream) {
    if (!h1 || !result || !scratch) return fail(PA_EINVAL, "fbc: h1, result and scratch must be non-NULL");
    if (rows <= 0 || cols <= 0 || downsample < 1) return fail(PA_EINVAL, "fbc: rows, cols must be positive and downsample >= 1");
    if (dtype != PA_BF16 && dtype != PA_F16) return fail(PA_EINVAL, "fbc: dtype must be PA_BF16 or PA_F16");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* sc = static_cast<float*>(scratch);
    const long long numel = static_cast<long long>(rows) * cols;
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (downsample == 1 && numel % 8 == 0 && aligned16(h1) && aligned16(h0) && aligned16(prev) && aligned16(new_resid)) {
        const long long n8 = numel / 8;
        long long blocks = (n8 + pa::kFbcThreads - 1) / pa::kFbcThreads;
        if (blocks > pa::kFbcMaxBlocks) blocks = pa::kFbcMaxBlocks;
        // the ticket sits right behind the partials of this launch's grid
        if (dtype == PA_BF16)
            pa::fbc_residual_diff_kernel<true><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint4*>(h1), static_cast<const uint4*>(h0), static_cast<const uint4*>(prev),
                static_cast<uint4*>(new_resid), n8, sc + 2 * (pa::kFbcMaxBlocks - blocks), result);
        else
            pa::fbc_residual_diff_kernel<false><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint4*>(h1), static_cast<const uint4*>(h0), static_cast<const uint4*>(prev),
                static_cast<uint4*>(new_resid), n8, sc + 2 * (pa::kFbcMaxBlocks - blocks), result);
    } else {
        const int cols_ds = (cols + downsample - 1) / downsample;
        const long long n = static_cast<long long>(rows) * cols_ds;
        long long blocks = (n + pa::kFbcThreads - 1) / pa::kFbcThreads;
        if (blocks > pa::kFbcMaxBlocks) blocks = pa::kFbcMaxBlocks;
        if (dtype == PA_BF16)
            pa::fbc_residual_diff_strided_kernel<true><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint16_t*>(h1), static_cast<const uint16_t*>(h0), static_cast<const uint16_t*>(prev),
                static_cast<uint16_t*>(new_resid), rows, cols, downsample, sc + 2 * (pa::kFbcMaxBlocks - blocks), result);
        else
            pa::fbc_residual_diff_strided_kernel<false><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint16_t*>(h1), static_cast<const uint16_t*>(h0), static_cast<const uint16_t*>(prev),
                static_cast<uint16_t*>(new_resid), rows, cols, downsample, sc + 2 * (pa::kFbcMaxBlocks - blocks), result);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "fbc launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

// ---- pa_fbc_residual_diff with built-in scratch ------------------------------------------------
// Some hosts can hand this library input and output buffers but have nothing to give it as
// scratch: a serving process whose device memory was carved up once at start-up and then frozen,
// or a thin binding from another runtime that only forwards pointers it was handed and owns no
// device allocator. For them the partial-sum scratch of the cache-decision kernel lives in the
// library image itself. The array below is file-scope device memory: every GPU that loads the
// library carries one copy (4864 bytes) until the process exits.
//
// On the host, `g_fbc_static_scratch` is only a handle for the symbol, never a device address.
// The address a kernel may use is looked up per device with cudaGetSymbolAddress (below) while
// that device is current.
constexpr int kFbcStaticMaxBlocks = 148 * 4;
constexpr size_t kFbcStaticBytes = ((2 * kFbcStaticMaxBlocks + 1) * sizeof(float) + 255) / 256 * 256;
static __device__ __align__(256) unsigned char g_fbc_static_scratch[kFbcStaticBytes];
static void* g_fbc_static_ptr[64] = {};
static std::mutex g_fbc_static_mu;

int pa_fbc_residual_diff_static(const void* h1, const void* h0, const void* prev, void* new_resid, int64_t rows,
                                int32_t cols, int32_t downsample, int32_t dtype, float* result, void* stream) {
    if (!h1 || !result) return fail(PA_EINVAL, "fbc static: h1 and result must be non-NULL");
    if (rows <= 0 || cols <= 0 || downsample < 1)
        return fail(PA_EINVAL, "fbc static: rows, cols must be positive and downsample >= 1");
    if (dtype != PA_BF16 && dtype != PA_F16) return fail(PA_EINVAL, "fbc static: dtype must be PA_BF16 or PA_F16");
    const long long numel = static_cast<long long>(rows) * cols;
    if (numel > PA_FBC_STATIC_MAX_NUMEL)
        return fail(PA_EINVAL, "fbc static: %lld elements exceed the limit of %lld of the built-in scratch variant; "
                    "use pa_fbc_residual_diff with caller scratch", numel, static_cast<long long>(PA_FBC_STATIC_MAX_NUMEL));
    // set-up, once per device, with that device current
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(PA_ECUDA, "fbc static: cudaGetDevice: %s", cudaGetErrorString(e));
    void* sptr = nullptr;
    {
        std::lock_guard<std::mutex> g(g_fbc_static_mu);
        if (g_fbc_static_ptr[dev] == nullptr) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_fbc_static_scratch);
            if (e != cudaSuccess || p == nullptr)
                return fail(PA_ECUDA, "fbc static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_fbc_static_ptr[dev] = p;
        }
        sptr = g_fbc_static_ptr[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* sc = static_cast<float*>(sptr);
    // The array keeps whatever the last call left: the ticket word must start at zero.
    e = cudaMemsetAsync(sc + 2 * kFbcStaticMaxBlocks, 0, sizeof(float), s);
    if (e != cudaSuccess) return fail(PA_ECUDA, "fbc static: cudaMemsetAsync: %s", cudaGetErrorString(e));
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (downsample == 1 && numel % 8 == 0 && aligned16(h1) && aligned16(h0) && aligned16(prev) && aligned16(new_resid)) {
        const long long n8 = numel / 8;
        long long blocks = (n8 + pa::kFbcThreads - 1) / pa::kFbcThreads;
        if (blocks > kFbcStaticMaxBlocks) blocks = kFbcStaticMaxBlocks;
        float* base = sc + 2 * (kFbcStaticMaxBlocks - blocks);  // the ticket sits right behind this grid's partials
        if (dtype == PA_BF16)
            pa::fbc_residual_diff_kernel<true><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint4*>(h1), static_cast<const uint4*>(h0), static_cast<const uint4*>(prev),
                static_cast<uint4*>(new_resid), n8, base, result);
        else
            pa::fbc_residual_diff_kernel<false><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint4*>(h1), static_cast<const uint4*>(h0), static_cast<const uint4*>(prev),
                static_cast<uint4*>(new_resid), n8, base, result);
    } else {
        const int cols_ds = (cols + downsample - 1) / downsample;
        const long long n = static_cast<long long>(rows) * cols_ds;
        long long blocks = (n + pa::kFbcThreads - 1) / pa::kFbcThreads;
        if (blocks > kFbcStaticMaxBlocks) blocks = kFbcStaticMaxBlocks;
        float* base = sc + 2 * (kFbcStaticMaxBlocks - blocks);
        if (dtype == PA_BF16)
            pa::fbc_residual_diff_strided_kernel<true><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint16_t*>(h1), static_cast<const uint16_t*>(h0), static_cast<const uint16_t*>(prev),
                static_cast<uint16_t*>(new_resid), rows, cols, downsample, base, result);
        else
            pa::fbc_residual_diff_strided_kernel<false><<<int(blocks), pa::kFbcThreads, 0, s>>>(
                static_cast<const uint16_t*>(h1), static_cast<const uint16_t*>(h0), static_cast<const uint16_t*>(prev),
                static_cast<uint16_t*>(new_resid), rows, cols, downsample, base, result);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "fbc static launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int pa_fbc_axpy(const void* a, const void* b, void* out, int64_t numel, int32_t sub, int32_t dtype, void* stream) {
    if (!a || !b || !out) return fail(PA_EINVAL, "axpy: NULL pointer");
    if (numel <= 0) return fail(PA_EINVAL, "axpy: numel must be positive");
    if (dtype != PA_BF16 && dtype != PA_F16) return fail(PA_EINVAL, "axpy: dtype must be PA_BF16 or PA_F16");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = numel % 8 == 0 &&
                     ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (!vec) {
        // odd sizes or addresses: one 16-bit element per thread iteration
        if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 1u)
            return fail(PA_EINVAL, "axpy: pointers must be 2-byte aligned");
        long long blocks = (numel + pa::kFbcThreads - 1) / pa::kFbcThreads;
        const long long cap = static_cast<long long>(sm_count()) * 16;
        if (blocks > cap) blocks = cap;
        const uint16_t *sa = static_cast<const uint16_t*>(a), *sb = static_cast<const uint16_t*>(b);
        uint16_t* so = static_cast<uint16_t*>(out);
        if (dtype == PA_BF16) {
            if (sub) pa::fbc_axpy_scalar_kernel<true, true><<<int(blocks), pa::kFbcThreads, 0, s>>>(sa, sb, so, numel);
            else pa::fbc_axpy_scalar_kernel<true, false><<<int(blocks), pa::kFbcThreads, 0, s>>>(sa, sb, so, numel);
        } else {
            if (sub) pa::fbc_axpy_scalar_kernel<false, true><<<int(blocks), pa::kFbcThreads, 0, s>>>(sa, sb, so, numel);
            else pa::fbc_axpy_scalar_kernel<false, false><<<int(blocks), pa::kFbcThreads, 0, s>>>(sa, sb, so, numel);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(PA_ECUDA, "axpy launch: %s", cudaGetErrorString(e));
        return PA_OK;
    }
    const long long n8 = numel / 8;
    long long blocks = (n8 + pa::kFbcThreads - 1) / pa::kFbcThreads;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    const uint4 *pa_ = static_cast<const uint4*>(a), *pb_ = static_cast<const uint4*>(b);
    uint4* po = static_cast<uint4*>(out);
    if (dtype == PA_BF16) {
        if (sub) pa::fbc_axpy_kernel<true, true><<<int(blocks), pa::kFbcThreads, 0, s>>>(pa_, pb_, po, n8);
        else pa::fbc_axpy_kernel<true, false><<<int(blocks), pa::kFbcThreads, 0, s>>>(pa_, pb_, po, n8);
    } else {
        if (sub) pa::fbc_axpy_kernel<false, true><<<int(blocks), pa::kFbcThreads, 0, s>>>(pa_, pb_, po, n8);
        else pa::fbc_axpy_kernel<false, false><<<int(blocks), pa::kFbcThreads, 0, s>>>(pa_, pb_, po, n8);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "axpy launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int pa_qkv_prep(const pa_qkv_prep_args* a, void* stream) {
    if (a == nullptr) return fail(PA_EINVAL, "qkv_prep: args is NULL");
    if (a->batch <= 0 || a->rows <= 0 || a->heads <= 0) return fail(PA_EINVAL, "qkv_prep: batch, rows, heads must be positive");
    if (a->head_dim != 64 && a->head_dim != 128) return fail(PA_ENOTSUP, "qkv_prep: head_dim %d: only 64 and 128 are built", a->head_dim);
    if (a->dtype != PA_BF16 && a->dtype != PA_F16) return fail(PA_EINVAL, "qkv_prep: dtype must be PA_BF16 or PA_F16");
    if ((a->cos == nullptr) != (a->sin == nullptr)) return fail(PA_EINVAL, "qkv_prep: cos and sin go together");
    if (!(a->eps >= 0.f)) return fail(PA_EINVAL, "qkv_prep: eps must not be negative");
    pa::QkvPrepParams p;
    memset(&p, 0, sizeof(p));
    const unsigned align = a->head_dim == 128 ? 7u : 3u;  // one lane moves 8 or 4 bytes
    const void* src[3] = {a->q, a->k, a->v};
    void* dst[3] = {a->q_out, a->k_out, a->v_out};
    const int64_t* ss[3] = {a->q_stride, a->k_stride, a->v_stride};
    const int64_t* ds[3] = {a->q_out_stride, a->k_out_stride, a->v_out_stride};
    for (int i = 0; i < 3; ++i) {
        if (src[i] == nullptr) {
            if (i < 2) return fail(PA_EINVAL, "qkv_prep: q and k must be non-NULL");
            continue;
        }
        if (dst[i] == nullptr) return fail(PA_EINVAL, "qkv_prep: output %d is NULL", i);
        if ((reinterpret_cast<uintptr_t>(src[i]) & align) || (reinterpret_cast<uintptr_t>(dst[i]) & align))
            return fail(PA_EINVAL, "qkv_prep: tensor %d: base pointers must be %u-byte aligned", i, align + 1);
        for (int d = 0; d < 3; ++d)
            if (((ss[i][d] * 2) & align) || ((ds[i][d] * 2) & align))
                return fail(PA_EINVAL, "qkv_prep: tensor %d: byte strides must be multiples of %u", i, align + 1);
        p.src[i] = static_cast<const uint16_t*>(src[i]);
        p.dst[i] = static_cast<uint16_t*>(dst[i]);
        p.s_sb[i] = ss[i][0]; p.s_ss[i] = ss[i][1]; p.s_sh[i] = ss[i][2];
        p.d_sb[i] = ds[i][0]; p.d_ss[i] = ds[i][1]; p.d_sh[i] = ds[i][2];
    }
    p.w[0] = static_cast<const uint16_t*>(a->q_weight);
    p.w[1] = static_cast<const uint16_t*>(a->k_weight);
    p.cos = a->cos;
    p.sin = a->sin;
    p.table_row0 = a->table_row0;
    p.batch = a->batch; p.rows = a->rows; p.heads = a->heads;
    p.eps = a->eps;
    const long long total = static_cast<long long>(a->batch) * a->rows * a->heads;
    long long blocks = (total + pa::kPrepThreads / 32 - 1) / (pa::kPrepThreads / 32);
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a->dtype == PA_BF16) {
        if (a->head_dim == 128) pa::qkv_prep_kernel<true, 128><<<int(blocks), pa::kPrepThreads, 0, s>>>(p);
        else pa::qkv_prep_kernel<true, 64><<<int(blocks), pa::kPrepThreads, 0, s>>>(p);
    } else {
        if (a->head_dim == 128) pa::qkv_prep_kernel<false, 128><<<int(blocks), pa::kPrepThreads, 0, s>>>(p);
        else pa::qkv_prep_kernel<false, 64><<<int(blocks), pa::kPrepThreads, 0, s>>>(p);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "qkv_prep launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

namespace {
int taylor_checks(const char* what, int64_t numel, int32_t dtype) {
    if (numel <= 0 || numel % 8 != 0) return fail(PA_EINVAL, "%s: numel must be a positive multiple of 8", what);
    if (dtype != PA_BF16 && dtype != PA_F16) return fail(PA_EINVAL, "%s: dtype must be PA_BF16 or PA_F16", what);
    return PA_OK;
}
bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }
int taylor_blocks(long long n8) {
    long long blocks = (n8 + pa::kFbcThreads - 1) / pa::kFbcThreads;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    return int(blocks > cap ? cap : blocks);
}
}  // namespace

int pa_taylor_update(const void* y, const void* const* prev, void* const* cur, int32_t depth, int32_t window,
                     int64_t numel, int32_t dtype, void* stream) {
    if (depth == 0) return PA_OK;  // nothing to derive yet
    if (!y || !prev || !cur) return fail(PA_EINVAL, "taylor_update: NULL pointer");
    if (depth < 0 || depth > pa::kTaylorMaxOrder - 1)
        return fail(PA_EINVAL, "taylor_update: depth must be in [0, %d]", pa::kTaylorMaxOrder - 1);
    if (window <= 0) return fail(PA_EINVAL, "taylor_update: window must be positive");
    int rc = taylor_checks("taylor_update", numel, dtype);
    if (rc != PA_OK) return rc;
    pa::TaylorUpdateParams p;
    memset(&p, 0, sizeof(p));
    if (misaligned(y)) return fail(PA_EINVAL, "taylor_update: pointers must be 16-byte aligned");
    p.y = static_cast<const uint4*>(y);
    for (int i = 0; i < depth; ++i) {
        if (!prev[i] || !cur[i]) return fail(PA_EINVAL, "taylor_update: prev[%d] / cur[%d] is NULL", i, i);
        if (misaligned(prev[i]) || misaligned(cur[i])) return fail(PA_EINVAL, "taylor_update: pointers must be 16-byte aligned");
        p.prev[i] = static_cast<const uint4*>(prev[i]);
        p.cur[i] = static_cast<uint4*>(cur[i]);
    }
    p.depth = depth;
    p.window = static_cast<float>(window);
    p.n8 = numel / 8;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == PA_BF16) pa::taylor_update_kernel<true><<<taylor_blocks(p.n8), pa::kFbcThreads, 0, s>>>(p);
    else pa::taylor_update_kernel<false><<<taylor_blocks(p.n8), pa::kFbcThreads, 0, s>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "taylor_update launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

int pa_taylor_approx(const void* const* d, int32_t terms, int32_t elapsed, const void* add, void* out, int64_t numel,
                     int32_t dtype, void* stream) {
    if (!d || !out) return fail(PA_EINVAL, "taylor_approx: NULL pointer");
    if (terms < 1 || terms > pa::kTaylorMaxOrder) return fail(PA_EINVAL, "taylor_approx: terms must be in [1, %d]", pa::kTaylorMaxOrder);
    if (elapsed < 0) return fail(PA_EINVAL, "taylor_approx: elapsed must not be negative");
    int rc = taylor_checks("taylor_approx", numel, dtype);
    if (rc != PA_OK) return rc;
    pa::TaylorApproxParams p;
    memset(&p, 0, sizeof(p));
    double fact = 1.0, pw = 1.0;
    for (int i = 0; i < terms; ++i) {
        if (!d[i]) return fail(PA_EINVAL, "taylor_approx: d[%d] is NULL", i);
        if (misaligned(d[i])) return fail(PA_EINVAL, "taylor_approx: pointers must be 16-byte aligned");
        p.d[i] = static_cast<const uint4*>(d[i]);
        if (i > 0) {
            fact *= i;
            pw *= elapsed;
        }
        p.coef[i] = static_cast<float>(1.0 / fact);  // the scalar a tensor operation would see
        p.power[i] = static_cast<float>(pw);
    }
    if (misaligned(out) || (add && misaligned(add))) return fail(PA_EINVAL, "taylor_approx: pointers must be 16-byte aligned");
    p.terms = terms;
    p.add = static_cast<const uint4*>(add);
    p.out = static_cast<uint4*>(out);
    p.n8 = numel / 8;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == PA_BF16) pa::taylor_approx_kernel<true><<<taylor_blocks(p.n8), pa::kFbcThreads, 0, s>>>(p);
    else pa::taylor_approx_kernel<false><<<taylor_blocks(p.n8), pa::kFbcThreads, 0, s>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PA_ECUDA, "taylor_approx launch: %s", cudaGetErrorString(e));
    return PA_OK;
}

}  // extern "C"
