// Flash-attention forward for B200 (sm_100a): tcgen05 MMA with TMEM accumulators, TMA loads.
//
// One CTA owns two query tiles of 128 rows (same batch/head/chunk) and walks every key/value
// tile of 128 rows. Warp roles (20 warps):
//   warps 0-15  softmax. Warp w serves TMEM lane quarter w%4 (32 query rows) of query tile
//               (w/4)%2 and key-column half w/8: two threads share a query row, each owns
//               64 of the tile's 128 key columns (and, in the epilogue, half of O's columns).
//   warp  16    MMA issuer (one thread): S_t = Q_t K_j^T into TMEM, O_t += P_t V_j from TMEM
//   warp  17    TMA producer (one thread): Q once, then K_j / V_j through a 2-stage ring
//   warps 18-19 idle; they complete the control warpgroup that gives registers away
// TMEM columns (512 allocated): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512) for
// head_dim 128 (O0 [256,320) O1 [320,384) for head_dim 64);
// P_t (bf16/f16) overwrites S_t in place - each thread packs its 64 probabilities into the
// first 32 of its own 64 logit columns - and is the TMEM A operand of P V.
// While the softmax warps of one tile work, the tensor core runs the other tile's GEMMs; the
// two column halves of P are handed over separately, so P V starts on the first half while the
// second is still being exponentiated.
//
// In context-parallel runs the same launch also performs the exchange (see the fused push
// below): one kernel per attention call and rank, no collective library call on the path.
//
// Template parameters select bf16 / f16, head_dim 64 / 128 and causal masking; a key-padding
// mask is a run-time option (one 64-bit word of key flags per half tile).
//
// Key/value rows come as a list of equally sized chunks (one per source rank in context
// parallel runs, one in total otherwise); running max / sum / O stay on chip across
// chunks, so no out/LSE merge pass exists. A chunk whose ready counter is given is waited
// for (bounded) by the producer just before its first tile is loaded.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "../../include/pa_b200.h"
#include "pa_ptx.cuh"
#include "cp_exchange_sm100.cuh"

namespace pa {

// head_dim is a template parameter of the kernel (kD = 64 or 128). Shared-memory slots keep
// the 128-wide size for both: a 64-wide tile is one swizzle atom and fills the first half.
constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kHalfBytes = 128 * 128;       // 128 rows x 64 elements x 2 B (one swizzle atom wide)
constexpr int kTileBytes = 2 * kHalfBytes;  // 128 x 128 x 2 B
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 16;
constexpr int kMmaWarp = 16;
constexpr int kTmaWarp = 17;
constexpr int kAttnThreads = 640;  // 4 softmax warpgroups + 1 control warpgroup
#ifndef PA_REGS_SOFTMAX
#define PA_REGS_SOFTMAX 104
#endif
#ifndef PA_REGS_CONTROL
#define PA_REGS_CONTROL 64
#endif
constexpr int kRegsLaunch = 96;  // 65536 / 640 rounded down to a multiple of 8
constexpr int kRegsSoftmax = PA_REGS_SOFTMAX;
constexpr int kRegsControl = PA_REGS_CONTROL;
// Each scheduler partition holds one warp of each of the five warpgroups, so what its four
// softmax warps gain must be covered by what its control warp gives up - otherwise
// setmaxnreg.inc would wait forever.
static_assert(4 * kRegsSoftmax + kRegsControl <= 5 * kRegsLaunch, "setmaxnreg budget exceeds the launch allocation");
static_assert(kRegsSoftmax % 8 == 0 && kRegsControl % 8 == 0, "setmaxnreg counts are multiples of 8");
constexpr int kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColO0 = 256;
// log2-domain growth of the running row maximum that is tolerated before O is rescaled
constexpr float kRescaleThreshold = 8.0f;
// of every 8 pairs of probabilities, how many are exponentiated with the FMA-pipe polynomial
#ifndef PA_POLY_PAIRS_OF_8
#define PA_POLY_PAIRS_OF_8 0
#endif
constexpr int kPolyPairsOf8 = PA_POLY_PAIRS_OF_8;
#ifndef PA_POLY_HALF1
#define PA_POLY_HALF1 0
#endif
constexpr bool kPolyHalf1 = PA_POLY_HALF1 != 0;

struct AttnParams {
    int batch, heads;
    int n_q_chunks, q_rows, q_first;
    int n_kv_chunks, kv_rows, kv_first;
    float scale, scale_log2;
    void* out[PA_MAX_CHUNKS];
    float* lse[PA_MAX_CHUNKS];
    long long o_sb, o_sh, o_ss;
    long long l_sb, l_sh;
    const uint32_t* q_flag[PA_MAX_CHUNKS];
    const uint32_t* kv_flag[PA_MAX_CHUNKS];
    uint32_t flag_expect;
    uint32_t* done_flag[PA_MAX_CHUNKS];
    int* status;
    unsigned long long wait_ns;
    // chunks read in place from this rank's own tensors instead of the staging buffers (-1: none)
    int q_local_chunk, kv_local_chunk, local_head0;
    // causal masking (kernels instantiated with kCausal read these; `causal` selects them): a key at global position kv_pos[chunk] + col is visible to the query at
    // global position q_pos[chunk] + row iff it is not later (top-left aligned, as torch SDPA)
    int causal;
    long long q_pos[PA_MAX_CHUNKS];
    long long kv_pos[PA_MAX_CHUNKS];
    // key mask (NULL: every key is valid): bit i of word [batch][chunk][i / 64] tells whether key
    // row i of that chunk may be attended to; strides in 64-bit words
    const unsigned long long* key_bits;
    long long kb_sb, kb_sc;
    // debug instantiation only
    float* dbg_s;      // raw S of CTA 0: [tile][kv tile][row][col]
    int v_lbo, v_sbo;  // B descriptor of V (bytes)
    int pv_split;      // 1: issue P V as two N=64 MMAs
    long long* dbg_t;  // clock64 stamps of CTA 0: [role 0..2][step][8]; roles: softmax 0, softmax 1, MMA issuer
    int dbg_steps;
};

#ifndef PA_TIMELINE
#define PA_TIMELINE 0  // 1: the stamps are also compiled into the production instantiation (profiling builds)
#endif
template <bool kDebug>
__device__ __forceinline__ void dbg_stamp(const AttnParams& p, int role, int step, int slot, bool who) {
    if (kDebug || PA_TIMELINE) {
        if (p.dbg_t != nullptr && blockIdx.x == 0 && who && step < p.dbg_steps)
            p.dbg_t[(static_cast<size_t>(role) * p.dbg_steps + step) * 8 + slot] = clock64();
    }
}

struct AttnSmemCtl {
    uint64_t q_full;
    uint64_t k_full[kStages], k_empty[kStages];
    uint64_t v_full[kStages], v_empty[kStages];
    uint64_t s_full[2], p_full[2][2], o_done[2];
    uint64_t teardown;
    uint32_t tmem_base;
    int abort;
    float xch[2][2][2][kTileM];  // [step parity][query tile][column half][row]: row max / row sum exchange
};

constexpr int kAttnCtlBytes = 4608;
constexpr int kAttnSmemBytes = 1024 /*align slack*/ + 2 * kTileBytes /*Q*/ +
                               kStages * kTileBytes /*K*/ + kStages * kTileBytes /*V*/ + kAttnCtlBytes;
static_assert(sizeof(AttnSmemCtl) <= kAttnCtlBytes, "control block too large");

// Barrier among the 64 threads (two warps) that share 32 query rows.
__device__ __forceinline__ void pair_sync(int id) {
    asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

template <bool kBF16, bool kDebug, bool kCausal, int kD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_ql,
                const __grid_constant__ CUtensorMap tm_kl, const __grid_constant__ CUtensorMap tm_vl,
                const __grid_constant__ AttnParams p, const __grid_constant__ PushParams push) {
    static_assert(kD == 64 || kD == 128, "head_dim 64 or 128");
    static_assert(!kDebug || kD == 128, "the debug hooks exist for head_dim 128 only");
    constexpr int kAtoms = kD / 64;                    // 64-element swizzle atoms per row
    constexpr int kOperandBytes = kAtoms * kHalfBytes; // bytes one Q / K / V tile occupies
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    const uint32_t sQ = smem_u32(smem);
    const uint32_t sK = sQ + 2 * kTileBytes;
    const uint32_t sV = sK + kStages * kTileBytes;
    AttnSmemCtl* ctl = reinterpret_cast<AttnSmemCtl*>(smem + 2 * kTileBytes + 2 * kStages * kTileBytes);
    volatile int* s_abort = &ctl->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // A grid in which some CTA already gave up drains without touching TMEM or TMA.
    if (threadIdx.x == 0) {
        int st = 0;
        if (p.status != nullptr) st = *reinterpret_cast<volatile int*>(p.status);
        ctl->abort = st;
    }
    __syncthreads();
    if (ctl->abort != 0) return;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&ctl->q_full), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&ctl->k_full[s]), 1);
            mbar_init(smem_u32(&ctl->k_empty[s]), 1);
            mbar_init(smem_u32(&ctl->v_full[s]), 1);
            mbar_init(smem_u32(&ctl->v_empty[s]), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(smem_u32(&ctl->s_full[t]), 1);
            mbar_init(smem_u32(&ctl->p_full[t][0]), 128);
            mbar_init(smem_u32(&ctl->p_full[t][1]), 128);
            mbar_init(smem_u32(&ctl->o_done[t]), 1);
        }
        mbar_init(smem_u32(&ctl->teardown), 1);
        mbar_init_fence();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    if (warp == kTmaWarp && lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        if (p.q_local_chunk >= 0) tma_prefetch_desc(&tm_ql);
        if (p.kv_local_chunk >= 0) {
            tma_prefetch_desc(&tm_kl);
            tma_prefetch_desc(&tm_vl);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    // ---- which work unit: (batch, head, query chunk, pair of query tiles) -------------------
    // The CTAs that push first (the leading ones of the grid) take the LAST work units: those
    // belong to the query chunk that arrives last (and, in a causal run, to the short early
    // tiles), so the units that can start at once go to CTAs that start at once.
    const int pairs_per_chunk = (p.q_rows + 2 * kTileM - 1) / (2 * kTileM);
    int unit = blockIdx.x;
    if (push.n_push_ctas > 0) {
        unit -= push.n_push_ctas;
        if (unit < 0) unit += gridDim.x;
    }
    int pair = unit % pairs_per_chunk;
    unit /= pairs_per_chunk;
    // the late query tiles of a causal run see the most keys: schedule them first
    if (kCausal) pair = pairs_per_chunk - 1 - pair;
    const int head = unit % p.heads;
    unit /= p.heads;
    const int bidx = unit % p.batch;
    unit /= p.batch;
    const int qc = (p.q_first + unit) % p.n_q_chunks;
    const int row0 = pair * 2 * kTileM;

    const int tiles_per_chunk = (p.kv_rows + kTileN - 1) / kTileN;
    // Causal runs skip the key/value tiles that lie wholly after this CTA's last query row. All
    // roles derive the same tile list from tiles_in_chunk().
    const long long q_last = kCausal ? p.q_pos[qc] + min(row0 + 2 * kTileM, p.q_rows) - 1 : 0;
    auto tiles_in_chunk = [&](int c) -> int {
        if (!kCausal) return tiles_per_chunk;
        const long long visible = q_last - p.kv_pos[c] + 1;  // key rows of this chunk some query may see
        if (visible <= 0) return 0;
        const long long t = (visible + kTileN - 1) / kTileN;
        return t < tiles_per_chunk ? static_cast<int>(t) : tiles_per_chunk;
    };
    int n_tiles = 0;
    for (int c = 0; c < p.n_kv_chunks; ++c) n_tiles += tiles_in_chunk(c);
    const uint64_t pipe_limit = p.wait_ns + 1000000000ull;

    // Fused exchange: the leading CTAs of the grid (always resident in the first wave, and
    // waiting for nobody) first store this rank's Q/K/V head-slices into the staging buffers
    // of the ranks that consume them - own buffer first, then the ranks below in descending
    // order (a consumer walks its chunks upwards from its own rank, so the first chunk it
    // needs from a peer is the one that peer sends first) - and only then take up their
    // attention tiles. Every other CTA starts computing at once and
    // meets a chunk only when it needs it.
    if (push.n_push_ctas > 0 && static_cast<int>(blockIdx.x) < push.n_push_ctas) {
        for (int di = 0; di < push.n_dest; ++di) {
            int dest = push.first_dest - di;
            if (dest < 0) dest += push.n_dest;
            push_to_dest(push, dest, blockIdx.x, push.n_push_ctas);
        }
    }

    // Registers move from the control warpgroup to the softmax warpgroups. Each role's code is
    // dominated by its own setmaxnreg so that the register allocator budgets the regions
    // separately.
    if (warp >= kSoftmaxWarps) setmaxnreg_dec<kRegsControl>();
    if (warp == kTmaWarp) {
        // =============================== TMA producer ======================================
        if (lane == 0 && n_tiles > 0) {
            int issued = 0;
            bool ok = true;
            const bool q_in_place = (qc == p.q_local_chunk);
            if (!q_in_place && p.q_flag[qc] != nullptr) {
                ok = flag_wait_ge(p.q_flag[qc], p.flag_expect, s_abort, p.status, p.wait_ns,
                                  PA_DEV_TIMEOUT_Q);
                fence_proxy_async_global();
            }
            if (ok) {
                const uint32_t bq = smem_u32(&ctl->q_full);
                const CUtensorMap* mq = q_in_place ? &tm_ql : &tm_q;
                const int hq = q_in_place ? head + p.local_head0 : head;
                const int cq = q_in_place ? 0 : qc;
                mbar_expect_tx(bq, 2 * kOperandBytes);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int h = 0; h < kAtoms; ++h)
                        tma_load_5d(sQ + t * kTileBytes + h * kHalfBytes, mq, bq, h * 64,
                                    row0 + t * kTileM, hq, bidx, cq);
            }
            int j = 0;
            for (int ci = 0; ci < p.n_kv_chunks && ok; ++ci) {
                int c = p.kv_first + ci;
                if (c >= p.n_kv_chunks) c -= p.n_kv_chunks;
                const int tiles_c = tiles_in_chunk(c);
                if (tiles_c == 0) continue;
                const bool kv_in_place = (c == p.kv_local_chunk);
                if (!kv_in_place && p.kv_flag[c] != nullptr) {
                    ok = flag_wait_ge(p.kv_flag[c], p.flag_expect, s_abort, p.status, p.wait_ns,
                                      PA_DEV_TIMEOUT_KV);
                    fence_proxy_async_global();
                    if (!ok) break;
                }
                const CUtensorMap* mk = kv_in_place ? &tm_kl : &tm_k;
                const CUtensorMap* mv = kv_in_place ? &tm_vl : &tm_v;
                const int hk = kv_in_place ? head + p.local_head0 : head;
                const int ck = kv_in_place ? 0 : c;
                for (int t = 0; t < tiles_c; ++t, ++j) {
                    const int st = j & 1;
                    const uint32_t ph = (j >> 1) & 1;
                    const uint32_t bk = smem_u32(&ctl->k_full[st]);
                    const uint32_t bv = smem_u32(&ctl->v_full[st]);
                    if (j >= kStages) {
                        ok = mbar_wait(smem_u32(&ctl->k_empty[st]), ph ^ 1, s_abort, p.status,
                                       pipe_limit, PA_DEV_TIMEOUT_PIPE);
                        if (!ok) break;
                    }
                    mbar_expect_tx(bk, kOperandBytes);
                    tma_load_5d(sK + st * kTileBytes, mk, bk, 0, t * kTileN, hk, bidx, ck);
                    if (kAtoms == 2)
                        tma_load_5d(sK + st * kTileBytes + kHalfBytes, mk, bk, 64, t * kTileN, hk, bidx, ck);
                    if (j >= kStages) {
                        ok = mbar_wait(smem_u32(&ctl->v_empty[st]), ph ^ 1, s_abort, p.status,
                                       pipe_limit, PA_DEV_TIMEOUT_PIPE);
                        if (!ok) {
                            issued = j + 1;  // K of tile j is in flight, V is not
                            break;
                        }
                    }
                    mbar_expect_tx(bv, kOperandBytes);
                    tma_load_5d(sV + st * kTileBytes, mv, bv, 0, t * kTileN, hk, bidx, ck);
                    if (kAtoms == 2)
                        tma_load_5d(sV + st * kTileBytes + kHalfBytes, mv, bv, 64, t * kTileN, hk, bidx, ck);
                    issued = j + 1;
                }
            }
            if (*s_abort != 0) {
                // Leave only once the copies already issued have landed (bounded by time).
                int none = 0;
                volatile int* no_abort = &none;
                mbar_wait(smem_u32(&ctl->q_full), 0, no_abort, nullptr, 100000000ull, 0);
                for (int jj = (issued > 2 ? issued - 2 : 0); jj < issued; ++jj) {
                    const int st = jj & 1;
                    const uint32_t ph = (jj >> 1) & 1;
                    mbar_wait(smem_u32(&ctl->k_full[st]), ph, no_abort, nullptr, 100000000ull, 0);
                    mbar_wait(smem_u32(&ctl->v_full[st]), ph, no_abort, nullptr, 100000000ull, 0);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // =============================== MMA issuer ========================================
        // The issuer must keep ahead of the tensor core (64 cycles per 128x128x16 MMA): the
        // k-step loops are unrolled and every descriptor is a base plus a constant.
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t idesc_qk = make_idesc_f16(kBF16, false, kTileM, kTileN);
            constexpr uint32_t idesc_pv = make_idesc_f16(kBF16, true, kTileM, kD);
            constexpr uint32_t idesc_pv64 = make_idesc_f16(kBF16, true, kTileM, 64);
            const uint32_t v_lbo = kDebug ? static_cast<uint32_t>(p.v_lbo) : kHalfBytes;
            const uint32_t v_sbo = kDebug ? static_cast<uint32_t>(p.v_sbo) : 1024u;
            const bool pv_split = kDebug ? (p.pv_split != 0) : false;

            // Descriptors differ from a per-operand base only in the start-address field (units
            // of 16 bytes).
            const uint64_t dq0 = smem_desc_sw128(sQ, 16, 1024);
            const uint64_t dk0 = smem_desc_sw128(sK, 16, 1024);
            const uint64_t dv0 = smem_desc_sw128(sV, v_lbo, v_sbo);
            auto issue_qk = [&](int t, int st) {
                const uint64_t a0 = dq0 + static_cast<uint64_t>((t * kTileBytes) >> 4);
                const uint64_t b0 = dk0 + static_cast<uint64_t>((st * kTileBytes) >> 4);
                const uint32_t d = tmem + kColS0 + t * kTileN;
#pragma unroll
                for (int ks = 0; ks < kD / 16; ++ks) {
                    const uint64_t off = static_cast<uint64_t>(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
                    tc_mma_ss(d, a0 + off, b0 + off, idesc_qk, ks > 0 ? 1u : 0u);
                }
            };
            // P V for key rows [64*half, 64*half+64) of the tile: four k-steps
            auto issue_pv_half = [&](int t, int st, int half, bool acc) {
                const uint64_t b0 = dv0 + static_cast<uint64_t>((st * kTileBytes) >> 4);
                const uint32_t a0 = tmem + kColS0 + t * kTileN;
                const uint32_t d = tmem + kColO0 + t * kD;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    const int ks = half * 4 + k4;
                    const uint64_t b = b0 + static_cast<uint64_t>((ks * 16 * 128) >> 4);
                    const uint32_t accum = (acc || ks > 0) ? 1u : 0u;
                    // P of column half h lives at S columns [64h, 64h+32): 8 columns per k-step
                    const uint32_t a = a0 + half * 64 + k4 * 8;
                    if (!pv_split) {
                        tc_mma_ts(d, a, b, idesc_pv, accum);
                    } else {
                        tc_mma_ts(d, a, b, idesc_pv64, accum);
                        tc_mma_ts(d + 64, a, b + static_cast<uint64_t>(kHalfBytes >> 4), idesc_pv64, accum);
                    }
                }
            };

            bool ok = mbar_wait(smem_u32(&ctl->q_full), 0, s_abort, p.status, pipe_limit,
                                PA_DEV_TIMEOUT_PIPE);
            ok = ok && mbar_wait(smem_u32(&ctl->k_full[0]), 0, s_abort, p.status, pipe_limit,
                                 PA_DEV_TIMEOUT_PIPE);
            if (ok) {
                tc_fence_after();
                issue_qk(0, 0);
                tc_commit(smem_u32(&ctl->s_full[0]));
                issue_qk(1, 0);
                tc_commit(smem_u32(&ctl->s_full[1]));
                tc_commit(smem_u32(&ctl->k_empty[0]));
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int stn = (j + 1) & 1;
                const uint32_t phn = ((j + 1) >> 1) & 1;
                const bool more = (j + 1 < n_tiles);
                ok = mbar_wait(smem_u32(&ctl->v_full[st]), ph, s_abort, p.status, pipe_limit,
                               PA_DEV_TIMEOUT_PIPE);
                if (ok && more)
                    ok = mbar_wait(smem_u32(&ctl->k_full[stn]), phn, s_abort, p.status, pipe_limit,
                                   PA_DEV_TIMEOUT_PIPE);
                if (!ok) break;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    dbg_stamp<kDebug>(p, 2, j, t * 4 + 0, true);
                    ok = mbar_wait(smem_u32(&ctl->p_full[t][0]), j & 1, s_abort, p.status, pipe_limit,
                                   PA_DEV_TIMEOUT_PIPE);
                    if (!ok) break;
                    dbg_stamp<kDebug>(p, 2, j, t * 4 + 1, true);
                    tc_fence_after();
                    issue_pv_half(t, st, 0, j > 0);
                    ok = mbar_wait(smem_u32(&ctl->p_full[t][1]), j & 1, s_abort, p.status, pipe_limit,
                                   PA_DEV_TIMEOUT_PIPE);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv_half(t, st, 1, j > 0);
                    tc_commit(smem_u32(&ctl->o_done[t]));
                    if (t == 1) tc_commit(smem_u32(&ctl->v_empty[st]));
                    dbg_stamp<kDebug>(p, 2, j, t * 4 + 2, true);
                    if (more) {
                        issue_qk(t, stn);
                        tc_commit(smem_u32(&ctl->s_full[t]));
                        if (t == 1) tc_commit(smem_u32(&ctl->k_empty[stn]));
                    }
                    dbg_stamp<kDebug>(p, 2, j, t * 4 + 3, true);
                }
            }
            if (!ok) {
                // Nothing may still be running on the tensor core when TMEM is released.
                int none = 0;
                volatile int* no_abort = &none;
                tc_commit(smem_u32(&ctl->teardown));
                mbar_wait(smem_u32(&ctl->teardown), 0, no_abort, nullptr, 100000000ull, 0);
            }
        }
    } else if (warp < kSoftmaxWarps) {
        // =============================== softmax + epilogue ================================
        setmaxnreg_inc<kRegsSoftmax>();
        const int quarter = warp & 3;
        const int t = (warp >> 2) & 1;
        const int half = warp >> 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t tS = tmem + lane_base + kColS0 + t * kTileN + half * 64;  // my 64 logit columns
        const uint32_t tO = tmem + lane_base + kColO0 + t * kD + half * (kD / 2);  // my half of the output columns
        const uint32_t bs = smem_u32(&ctl->s_full[t]);
        const uint32_t bp = smem_u32(&ctl->p_full[t][half]);
        const uint32_t bo = smem_u32(&ctl->o_done[t]);
        const int pair_bar = 1 + t * 4 + quarter;
        const float sl = p.scale_log2;
        const bool stamper = (quarter == 0 && lane == 0 && half == 0);

        float m_ref = -INFINITY;
        float l_sum = 0.f;  // over my columns only
        bool ok = true;
        int j = 0;
        const long long q_here = kCausal ? p.q_pos[qc] + row0 + t * kTileM + row_in_tile : 0;  // my row's global position
        for (int ci = 0; ci < p.n_kv_chunks; ++ci) {
            int c_kv = p.kv_first + ci;
            if (c_kv >= p.n_kv_chunks) c_kv -= p.n_kv_chunks;
            const int tiles_c = tiles_in_chunk(c_kv);
            for (int tk = 0; tk < tiles_c; ++tk, ++j) {
                int valid = min(kTileN, p.kv_rows - tk * kTileN) - half * 64;  // of my 64 columns
                if (kCausal) {
                    const long long lim = q_here - (p.kv_pos[c_kv] + tk * kTileN + half * 64) + 1;
                    valid = static_cast<int>(lim < valid ? (lim < 0 ? 0 : lim) : valid);
                }
                // which of my 64 columns count: the key mask word (same for the whole warp), cut
                // at the ragged end of the chunk and at the causal diagonal
                unsigned long long live = ~0ull;
                if (p.key_bits != nullptr && valid > 0)  // (a half tile past the chunk's end has no word)
                    live = __ldg(p.key_bits + bidx * p.kb_sb + c_kv * p.kb_sc + tk * 2 + half);
                if (valid < 64) live &= (valid <= 0) ? 0ull : ((1ull << valid) - 1ull);
                dbg_stamp<kDebug>(p, t, j, 0, stamper);
                // A wait that gives up does not leave the loop: the two partner warps must meet at
                // every pair barrier below, and once the abort word is set no wait blocks any more.
                ok = mbar_wait(bs, j & 1, s_abort, p.status, pipe_limit, PA_DEV_TIMEOUT_PIPE) && ok;
                dbg_stamp<kDebug>(p, t, j, 1, stamper);
                tc_fence_after();
                // Pass 1: row maximum of my 64 logits. The logits are not kept: pass 2 reads them
                // again from TMEM 32 columns at a time, which keeps the thread within its register
                // budget (TMEM bandwidth is plentiful, registers are not).
                float mx[2];
                {
                    uint32_t s[2][32];
                    tmem_ld32(tS, s[0]);
                    tmem_ld32(tS + 32, s[1]);
                    tc_wait_ld();
                    tmem_ld_fence(s[0]);
                    tmem_ld_fence(s[1]);
                    dbg_stamp<kDebug>(p, t, j, 2, stamper);
                    if (kDebug && p.dbg_s != nullptr && blockIdx.x == 0) {
                        float* d = p.dbg_s + ((static_cast<size_t>(t) * n_tiles + j) * 128 + row_in_tile) * 128 + half * 64;
#pragma unroll
                        for (int c = 0; c < 2; ++c)
#pragma unroll
                            for (int i = 0; i < 32; ++i) d[c * 32 + i] = __uint_as_float(s[c][i]);
                    }
                    if (live != ~0ull) {
#pragma unroll
                        for (int c = 0; c < 2; ++c)
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (((live >> (c * 32 + i)) & 1ull) == 0) s[c][i] = 0xff800000u;  // -inf
                    }
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        mx[c] = fmaxf(__uint_as_float(s[c][0]), __uint_as_float(s[c][1]));
#pragma unroll
                        for (int i = 2; i < 32; i += 2)
                            mx[c] = fmax3(mx[c], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
                    }
                }
                // row maximum over both column halves: swap partial maxima with the partner thread
                const float mine = fmaxf(mx[0], mx[1]);
                ctl->xch[j & 1][t][half][row_in_tile] = mine;
                pair_sync(pair_bar);
                const float m_new = fmax3(mine, ctl->xch[j & 1][t][half ^ 1][row_in_tile], m_ref);
                const bool grow = (m_new - m_ref) * sl > kRescaleThreshold;
                if (__any_sync(0xffffffffu, grow)) {  // same decision in both partner warps
                    // (a row that has seen no visible key yet keeps m = -inf: scale by 1, not by NaN)
                    const float alpha = (m_new == -INFINITY) ? 1.0f : ex2_approx((m_ref - m_new) * sl);
                    l_sum *= alpha;
                    m_ref = m_new;
                    if (j > 0) {
                        ok = mbar_wait(bo, (j - 1) & 1, s_abort, p.status, pipe_limit,
                                       PA_DEV_TIMEOUT_PIPE) && ok;
                        tc_fence_after();
#pragma unroll
                        for (int c = 0; c < kAtoms; ++c) {
                            uint32_t o[32];
                            tmem_ld32(tO + c * 32, o);
                            tc_wait_ld();
                            tmem_ld_fence(o);
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(tO + c * 32, o);
                        }
                        // P V of this step adds to all 128 output columns as soon as the first
                        // half of P is handed over: both halves of O must be rescaled by then.
                        tc_wait_st();
                        tc_fence_before();
                        pair_sync(pair_bar);
                        tc_fence_after();
                    }
                }
                const float neg = (m_ref == -INFINITY) ? 0.0f : -m_ref * sl;
                dbg_stamp<kDebug>(p, t, j, 3, stamper);
                // p = 2^(s*sl - m*sl) in packed fp32x2 arithmetic. The exponentials are split between
                // the special-function unit and an FMA-pipe polynomial so that neither pipe alone
                // bounds the softmax: either the warps of column half 1 take the polynomial for all
                // their elements (kPolyHalf1) or kPolyPairsOf8 of every 8 element pairs do.
                const float2 sl2 = make_float2(sl, sl);
                const float2 neg2 = make_float2(neg, neg);
                // Pass 2, per 32-column chunk: reload, exponentiate, pack, and store the 16 packed
                // words over logit columns of my own that are already consumed (chunk c goes to my
                // columns [16c, 16c+16)), so partner threads never touch each other's columns.
                float2 ls[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t sc[32];
                    tmem_ld32(tS + c * 32, sc);
                    tc_wait_ld();
                    tmem_ld_fence(sc);
                    if (live != ~0ull) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (((live >> (c * 32 + i)) & 1ull) == 0) sc[i] = 0xff800000u;  // -inf
                    }
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 x = __ffma2_rn(
                            make_float2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), sl2, neg2);
                        float2 e;
                        if (kPolyHalf1 ? (half == 1) : (((i >> 1) & 7) < kPolyPairsOf8)) {
                            e = exp2_poly2(x);
                        } else {
                            e.x = ex2_approx(x.x);
                            e.y = ex2_approx(x.y);
                        }
                        ls[c] = __fadd2_rn(ls[c], e);
                        pk[i >> 1] = kBF16 ? pack_bf16x2(e.x, e.y) : pack_f16x2(e.x, e.y);
                    }
                    tmem_st16(tS + c * 16, pk);
                }
                {
                    const float2 a = __fadd2_rn(ls[0], ls[1]);
                    l_sum += a.x + a.y;
                }
                dbg_stamp<kDebug>(p, t, j, 4, stamper);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(bp);
                dbg_stamp<kDebug>(p, t, j, 5, stamper);
            }
        }
        // (a CTA whose queries see no key at all writes zeros and an LSE of -inf)
        const bool empty = (n_tiles == 0);
        if (!empty)
            ok = mbar_wait(bo, (n_tiles - 1) & 1, s_abort, p.status, pipe_limit, PA_DEV_TIMEOUT_PIPE) && ok;
        // row sum over both halves
        ctl->xch[n_tiles & 1][t][half][row_in_tile] = l_sum;
        pair_sync(pair_bar);
        const float l_row = l_sum + ctl->xch[n_tiles & 1][t][half ^ 1][row_in_tile];
        if (ok) {
            tc_fence_after();
            const int row = row0 + t * kTileM + row_in_tile;
            const bool in_range = row < p.q_rows;
            // a row that saw no key (all masked) comes out as zeros with an LSE of -inf
            const float inv = (empty || !(l_row > 0.0f)) ? 0.0f : 1.0f / l_row;
            uint16_t* orow = reinterpret_cast<uint16_t*>(p.out[qc]) +
                             (static_cast<long long>(bidx) * p.o_sb + static_cast<long long>(head) * p.o_sh +
                              static_cast<long long>(row) * p.o_ss) + half * (kD / 2);
#pragma unroll
            for (int c = 0; c < kAtoms; ++c) {
                uint32_t o[32];
                tmem_ld32(tO + c * 32, o);
                tc_wait_ld();
                tmem_ld_fence(o);
                if (empty) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;
                }
                if (in_range) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint4 w;
                        uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float a = __uint_as_float(o[v4 * 8 + 2 * i]) * inv;
                            const float b = __uint_as_float(o[v4 * 8 + 2 * i + 1]) * inv;
                            wp[i] = kBF16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
                        }
                        *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = w;
                    }
                }
            }
            if (half == 0 && in_range && p.lse[qc] != nullptr) {
                p.lse[qc][static_cast<long long>(bidx) * p.l_sb + static_cast<long long>(head) * p.l_sh + row] =
                    m_ref * p.scale + __logf(l_row);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (p.done_flag[qc] != nullptr && *s_abort == 0) {
        // every output store of this CTA is ordered before the counter update
        if (threadIdx.x == 0) {
            __threadfence_system();
            red_release_sys_add(p.done_flag[qc], 1u);
        }
    }
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace pa
