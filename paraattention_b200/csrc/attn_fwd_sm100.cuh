// Flash-attention forward for B200 (sm_100a): tcgen05 MMA with TMEM accumulators, TMA loads.
//
// One CTA owns two query tiles of 128 rows (same batch/head/chunk) and walks every key/value
// tile of 128 rows. Warp roles (10 warps):
//   warps 0-7   softmax: one thread per query row. Warp w serves TMEM lane quarter w%4 (32 query
//               rows) of query tile w/4 - all 128 key columns of a tile and, in the epilogue,
//               the whole output row.
//   warp  8     MMA issuer (the warp in lockstep, one elected lane issues): S_t = Q_t K_j^T into
//               TMEM, O_t += P_t V_j from TMEM
//   warp  9     TMA producer (one thread): Q once, then K_j / V_j through a 2-stage ring
// TMEM columns (512 allocated): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512) for
// head_dim 128 (O0 [256,320) O1 [320,384) for head_dim 64);
// P_t (bf16/f16) overwrites S_t in place: the probabilities of key columns [32c, 32c+32) are
// packed into consumed S columns of the same half of the tile ([64*(c/2) + 16*(c%2), +16)),
// and P is the TMEM A operand of P V.
//
// Every query tile is run as two half-tiles in the key dimension (key columns 0-63 and 64-127
// of each key/value tile), each with its own chain  Q K^T (N = 64) -> softmax -> P V -> next
// Q K^T. A softmax thread alternates between the halves; while it works on one, the tensor core
// runs the other half's P V and next Q K^T (and the other tile's), so MMA latency and the
// hand-overs in both directions are hidden instead of waited for. The price is the N = 64
// Q K^T, which runs at 48 instead of 32 cycles per MMA (shared-memory operand fetch).
//
// What bounds this kernel is each tile's chain softmax -> P V -> next Q K^T -> softmax, so the
// softmax is arranged to keep that chain short:
//  * ONE pass over the logits, 32 columns at a time (the next 32 in flight): a chunk is
//    exponentiated against the row reference - a maximum seen earlier - while its own maximum
//    is found on the side. If no row of the warp outgrew its reference by more than 2^8 (the
//    headroom that a lazily rescaled O allows anyway), the chunk's probabilities are stored
//    and handed to the tensor core at once, so P V of the first key columns runs while the
//    later ones are still being exponentiated. If some row did (the first chunk of a row
//    always does), the warp waits for the P V issued so far, moves the reference up, rescales
//    its rows of O and redoes that chunk from the logits it still holds in registers.
//  * no exchange between threads: a row's maximum, sum and O belong to one thread.
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

#ifndef PA_TIMELINE
#define PA_TIMELINE 0
#endif

namespace pa {

// head_dim is a template parameter of the kernel (kD = 64 or 128). Shared-memory slots keep
// the 128-wide size for both: a 64-wide tile is one swizzle atom and fills the first half.
constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kHalfBytes = 128 * 128;       // 128 rows x 64 elements x 2 B (one swizzle atom wide)
constexpr int kTileBytes = 2 * kHalfBytes;  // 128 x 128 x 2 B
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 8;
constexpr int kMmaWarp = 8;
constexpr int kTmaWarp = 9;
constexpr int kAttnThreads = 384;  // 2 softmax warpgroups + 1 control warpgroup
constexpr int kRegsLaunch = 168;   // 65536 / 384, rounded down to a multiple of 8
#ifndef PA_REGS_SOFTMAX
#define PA_REGS_SOFTMAX 168
#endif
#ifndef PA_REGS_CONTROL
#define PA_REGS_CONTROL 168
#endif
constexpr int kRegsSoftmax = PA_REGS_SOFTMAX;
constexpr int kRegsControl = PA_REGS_CONTROL;
static_assert(2 * kRegsSoftmax + kRegsControl <= 3 * kRegsLaunch, "setmaxnreg budget exceeds the launch allocation");
static_assert(kRegsSoftmax % 8 == 0 && kRegsControl % 8 == 0, "setmaxnreg counts are multiples of 8");
constexpr int kPieces = 4;         // P is handed to the tensor core in pieces of 32 key columns
constexpr int kPieceCols = kTileN / kPieces;
static_assert(kPieceCols == 32, "the softmax loads and hands over 32 columns at a time");
constexpr int kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColO0 = 256;
// log2-domain growth of the running row maximum that is tolerated before O is rescaled
constexpr float kRescaleThreshold = 8.0f;
// of every 8 pairs of probabilities, how many are exponentiated with the FMA-pipe polynomial
#ifndef PA_POLY_PAIRS_OF_8
#define PA_POLY_PAIRS_OF_8 0
#endif
constexpr int kPolyPairsOf8 = PA_POLY_PAIRS_OF_8;

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
    // Split of the last, under-filled wave, a launch of its own (the kSplit instantiation): work
    // units from `split_from` on are each computed by `split_k` consecutive CTAs, every one over
    // its own share of the key/value tiles. part_o [unit][share][head_dim / 4][256 rows][4] and
    // part_ml [unit][share][256 rows] (reference, row sum) hold the shares' results, part_cnt
    // [unit][9] counts finished warps (8) and finished CTAs (zeroed by the host before the launch).
    int split_from, split_k;
    int unit_base;  // kSplit launches: work unit of the first CTA
    float* part_o;
    float2* part_ml;
    unsigned int* part_cnt;
#if PA_TIMELINE
    long long* dbg_t;  // clock64 stamps of CTA 0: [role 0..4][step][8]; roles: softmax 0, softmax 1, MMA issuer, TMA producer, MMA operand waits
    int dbg_steps;
#endif
};

// Profiling builds (-DPA_TIMELINE=1, never the shipped library) let the first CTA record
// clock64() stamps of its pipeline phases; in every other build the calls compile to nothing.
__device__ __forceinline__ void dbg_stamp(const AttnParams& p, int role, int step, int slot, bool who) {
#if PA_TIMELINE
    if (p.dbg_t != nullptr && blockIdx.x == 0 && who && step < p.dbg_steps)
        p.dbg_t[(static_cast<size_t>(role) * p.dbg_steps + step) * 8 + slot] = clock64();
#endif
}

struct AttnSmemCtl {
    uint64_t q_full;
    uint64_t k_full[kStages], k_empty[kStages];
    uint64_t v_full[kStages], v_empty[kStages];
    uint64_t s_full[2][2];        // Q K^T of a query tile is in TMEM, per half of the key columns
    uint64_t p_full[2][kPieces];  // a piece of P of a query tile is in TMEM (128 arrivals)
    uint64_t o_done[2][kPieces];  // P V of a piece (and every MMA issued before it) is done
    uint64_t teardown;
    uint32_t tmem_base;
    int abort;
    // kSplit launches: which unit of the split wave, which share of its tiles, first tile. Kept
    // here (every thread writes the same values and reads them back where it needs them) rather
    // than in registers across the main loop.
    int split_unit, share, j_begin;
};

constexpr int kAttnCtlBytes = 512;
constexpr int kAttnSmemBytes = 1024 /*align slack*/ + 2 * kTileBytes /*Q*/ +
                               kStages * kTileBytes /*K*/ + kStages * kTileBytes /*V*/ + kAttnCtlBytes;
static_assert(sizeof(AttnSmemCtl) <= kAttnCtlBytes, "control block too large");

// Softmax of one thread over 32 logits held in registers: p = 2^(s * sl + neg) packed to 16-bit
// pairs (pk[i] = columns 2i, 2i+1), their fp32 sum, and the largest raw logit. With kMasked, columns whose bit in
// `live` is clear count as -inf (the unmasked instantiation carries no per-element mask code at
// all: it is the one that runs on every full tile). kPolyPairsOf8 of every 8 pairs take an
// FMA-pipe polynomial instead of the special-function unit (off by default).
template <bool kBF16, bool kMasked>
__device__ __forceinline__ void softmax_chunk(const uint32_t (&sc)[32], uint32_t live, float sl, float neg,
                                              uint32_t (&pk)[16], float& sum, float& mx) {
    const float2 sl2 = make_float2(sl, sl);
    const float2 neg2 = make_float2(neg, neg);
    float2 ls[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    float m[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float s0 = __uint_as_float(sc[i]), s1 = __uint_as_float(sc[i + 1]);
        if (kMasked) {
            if (((live >> i) & 1u) == 0) s0 = -INFINITY;
            if (((live >> (i + 1)) & 1u) == 0) s1 = -INFINITY;
        }
        m[(i >> 1) & 1] = fmax3(m[(i >> 1) & 1], s0, s1);
        const float2 x = __ffma2_rn(make_float2(s0, s1), sl2, neg2);
        float2 e;
        if (((i >> 1) & 7) < kPolyPairsOf8) {
            e = exp2_poly2(x);
        } else {
            e.x = ex2_approx(x.x);
            e.y = ex2_approx(x.y);
        }
        ls[(i >> 1) & 1] = __fadd2_rn(ls[(i >> 1) & 1], e);
        pk[i >> 1] = kBF16 ? pack_bf16x2(e.x, e.y) : pack_f16x2(e.x, e.y);
    }
    const float2 t = __fadd2_rn(ls[0], ls[1]);
    sum = t.x + t.y;
    mx = fmaxf(m[0], m[1]);
}

// The rare path of a softmax piece, kept out of line so that the loop every tile runs stays
// small: some row of the calling warp (all 32 lanes call) outgrew its reference `m_ref` with
// this piece's maximum `mx`. Every row moves its reference up to what it has seen; once the
// P V handed over so far has completed (`wait_o`: barrier `bo`, phase parity `par`) the warp's
// rows of O at `tO` are rescaled; the piece is reloaded from `tS_piece`, exponentiated against
// the new reference and stored to `tP`. Returns the new reference and the new row sum.
template <bool kBF16, int kD>
__device__ __noinline__ float2 softmax_piece_regrow(uint32_t tS_piece, uint32_t tP, uint32_t tO, uint32_t live, float sl,
                                                    float mx, float m_ref, float l_sum, bool wait_o, uint32_t bo,
                                                    uint32_t par, volatile int* s_abort, int* status,
                                                    unsigned long long limit_ns) {
    const float m_new = fmaxf(m_ref, mx);
    // (a row that has seen no visible key yet keeps m = -inf: scale by 1, not by NaN)
    const float alpha = (m_new == -INFINITY) ? 1.0f : ex2_approx((m_ref - m_new) * sl);
    if (wait_o) {
        mbar_wait(bo, par, s_abort, status, limit_ns, PA_DEV_TIMEOUT_PIPE);
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < kD / 32; ++b) {
            uint32_t o[32];
            tmem_ld32(tO + b * 32, o);
            tc_wait_ld();
            tmem_ld_fence(o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + b * 32, o);
        }
        // (ordered before the next P V by the caller's wait::st / fence / arrive for this piece)
    }
    uint32_t sc[32];
    tmem_ld32(tS_piece, sc);
    tc_wait_ld();
    tmem_ld_fence(sc);
    uint32_t pk[16];
    float ls, unused;
    softmax_chunk<kBF16, true>(sc, live, sl, (m_new == -INFINITY) ? 0.0f : -m_new * sl, pk, ls, unused);
    tmem_st16(tP, pk);
    return make_float2(m_new, l_sum * alpha + ls);
}

// Epilogue of a CTA that computed one share of a split work unit (all 32 lanes of a softmax warp
// call; one thread per query row). The warp stores its rows' unnormalised output, reference and
// row sum as this share's result and counts itself on the unit's counter for this warp slot;
// the warp that finds all the other shares already counted combines them with its own -
// out = sum_i 2^((m_i - m) * sl) O_i / sum_i 2^((m_i - m) * sl) l_i - and writes the final rows
// and their LSE. Nobody waits: the last warp to arrive does the work, whichever share it is.
// Returns nothing; rows beyond the query chunk (`in_range` false) are not written.
template <bool kBF16, int kD>
__device__ __noinline__ void split_epilogue(uint32_t tO, float m_ref, float l_sum, float sl, float scale, int lane,
                                            int slot_row, int share, int split_k, float* part_o, float2* part_ml,
                                            unsigned int* cnt, uint16_t* orow, float* lse_row, bool in_range) {
    // slot_row: this row's index within the unit's 256 rows. A share's output is stored as
    // [head_dim / 4][256 rows] groups of four columns, so that the 32 rows of a warp store and
    // load 512 contiguous bytes at a time.
    constexpr int kGroups = kD / 4;
    uint4* mine_o = reinterpret_cast<uint4*>(part_o) + static_cast<size_t>(share) * kGroups * (2 * kTileM) + slot_row;
#pragma unroll
    for (int b = 0; b < kD / 32; ++b) {
        uint32_t o[32];
        tmem_ld32(tO + b * 32, o);
        tc_wait_ld();
        tmem_ld_fence(o);
#pragma unroll
        for (int v4 = 0; v4 < 8; ++v4)
            __stcg(mine_o + static_cast<size_t>(b * 8 + v4) * (2 * kTileM),
                   make_uint4(o[4 * v4], o[4 * v4 + 1], o[4 * v4 + 2], o[4 * v4 + 3]));
    }
    __stcg(part_ml + static_cast<size_t>(share) * (2 * kTileM) + slot_row, make_float2(m_ref, l_sum));
    __threadfence();
    __syncwarp();
    unsigned int before = 0;
    if (lane == 0) before = atomicAdd(cnt, 1u);
    before = __shfl_sync(0xffffffffu, before, 0);
    if (before + 1u != static_cast<unsigned int>(split_k)) return;
    __threadfence();

    float m_tot = m_ref;
    for (int i = 0; i < split_k; ++i) {
        if (i == share) continue;
        m_tot = fmaxf(m_tot, __ldcg(part_ml + static_cast<size_t>(i) * (2 * kTileM) + slot_row).x);
    }
    // (a share whose rows saw no key has m = -inf and weighs nothing)
    auto weight = [&](float m) -> float { return (m == -INFINITY) ? 0.0f : ex2_approx((m - m_tot) * sl); };
    float l_tot = 0.0f;
    for (int i = 0; i < split_k; ++i) {
        const float2 ml = (i == share) ? make_float2(m_ref, l_sum)
                                       : __ldcg(part_ml + static_cast<size_t>(i) * (2 * kTileM) + slot_row);
        l_tot += ml.y * weight(ml.x);
    }
    const float inv = (l_tot > 0.0f) ? 1.0f / l_tot : 0.0f;
    // (the shares are added in index order, this warp's own at its place, whichever share it
    // is: the result does not depend on who arrives last)
#pragma unroll 1
    for (int b = 0; b < kD / 32; ++b) {
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
        for (int i = 0; i < split_k; ++i) {
            if (i == share) {
                const float w = weight(m_ref) * inv;
                uint32_t o[32];
                tmem_ld32(tO + b * 32, o);
                tc_wait_ld();
                tmem_ld_fence(o);
#pragma unroll
                for (int c = 0; c < 32; ++c) acc[c] = fmaf(__uint_as_float(o[c]), w, acc[c]);
                continue;
            }
            const float w = weight(__ldcg(part_ml + static_cast<size_t>(i) * (2 * kTileM) + slot_row).x) * inv;
            const uint4* src = reinterpret_cast<const uint4*>(part_o) +
                               (static_cast<size_t>(i) * kGroups + b * 8) * (2 * kTileM) + slot_row;
#pragma unroll
            for (int v4 = 0; v4 < 8; ++v4) {
                const uint4 x = __ldcg(src + static_cast<size_t>(v4) * (2 * kTileM));
                acc[4 * v4 + 0] = fmaf(__uint_as_float(x.x), w, acc[4 * v4 + 0]);
                acc[4 * v4 + 1] = fmaf(__uint_as_float(x.y), w, acc[4 * v4 + 1]);
                acc[4 * v4 + 2] = fmaf(__uint_as_float(x.z), w, acc[4 * v4 + 2]);
                acc[4 * v4 + 3] = fmaf(__uint_as_float(x.w), w, acc[4 * v4 + 3]);
            }
        }
        if (in_range) {
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
                uint4 w4;
                uint32_t* wp = reinterpret_cast<uint32_t*>(&w4);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    wp[i] = kBF16 ? pack_bf16x2(acc[v4 * 8 + 2 * i], acc[v4 * 8 + 2 * i + 1])
                                  : pack_f16x2(acc[v4 * 8 + 2 * i], acc[v4 * 8 + 2 * i + 1]);
                *reinterpret_cast<uint4*>(orow + b * 32 + v4 * 8) = w4;
            }
        }
    }
    if (in_range && lse_row != nullptr) *lse_row = (l_tot > 0.0f) ? m_tot * scale + __logf(l_tot) : -INFINITY;
}

// kSplit: the launch that computes the work units of a split last wave (see AttnParams); the
// instantiation without it carries none of that code.
template <bool kBF16, bool kCausal, int kD, bool kSplit = false>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_ql,
                const __grid_constant__ CUtensorMap tm_kl, const __grid_constant__ CUtensorMap tm_vl,
                const __grid_constant__ AttnParams p, const __grid_constant__ PushParams push) {
    static_assert(kD == 64 || kD == 128, "head_dim 64 or 128");
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
            mbar_init(smem_u32(&ctl->s_full[t][0]), 1);
            mbar_init(smem_u32(&ctl->s_full[t][1]), 1);
            for (int c = 0; c < kPieces; ++c) {
                mbar_init(smem_u32(&ctl->p_full[t][c]), kTileM);
                mbar_init(smem_u32(&ctl->o_done[t][c]), 1);
            }
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
    const int pairs_per_chunk = (p.q_rows + 2 * kTileM - 1) / (2 * kTileM);
    int unit = blockIdx.x;
    if (push.n_push_ctas > 0) {
        // CTAs that push before they compute take the LAST work units (the query chunk that
        // arrives last), so the units that can start at once go to CTAs that start at once
        unit -= push.n_push_ctas;
        if (unit < 0) unit += gridDim.x;
    }
    // (a unit of the split last wave belongs to split_k consecutive CTAs)
    volatile int* s_split = &ctl->split_unit;  // [0] unit of the split wave, [1] share, [2] first tile
    if (kSplit) {
        int split_unit = -1, share = 0;  // (units before split_from are computed whole)
        unit += p.unit_base;
        if (unit >= p.split_from) {
            split_unit = (unit - p.split_from) / p.split_k;
            share = (unit - p.split_from) - split_unit * p.split_k;
            unit = p.split_from + split_unit;
        }
        s_split[0] = split_unit;
        s_split[1] = share;
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
    // This CTA's part of the unit's tile list (all of it unless the unit is split): tiles
    // [j_begin, j_begin + n_tiles) in the order the chunks are walked.
    if (kSplit) {
        const int share = s_split[1];
        const int k = (s_split[0] >= 0) ? p.split_k : 1;
        const int j_begin = static_cast<int>(static_cast<long long>(n_tiles) * share / k);
        n_tiles = static_cast<int>(static_cast<long long>(n_tiles) * (share + 1) / k) - j_begin;
        s_split[2] = j_begin;
    }
    const uint64_t pipe_limit = p.wait_ns + 1000000000ull;

    // Fused exchange: the leading CTAs of the grid (always resident in the first wave, and
    // waiting for nobody) first store this rank's Q/K/V head-slices into the staging buffers
    // of the ranks that consume them - the ranks below first, in descending order (a consumer
    // walks its chunks upwards from its own rank, so the first chunk it needs from a peer is the
    // one that peer sends first) - and only then take up their attention tiles. Every other CTA
    // starts computing at once and meets a chunk only when it needs it. (Letting two spare warps
    // of every first-wave CTA copy in the background instead was measured slower on 2 and on 8
    // GPUs: the copy then takes most of the kernel's duration and the first remote chunk is late.)
    if (push.n_push_ctas > 0 && static_cast<int>(blockIdx.x) < push.n_push_ctas) {
        for (int di = 0; di < push.n_dest; ++di) {
            int dest = push.first_dest - di;
            if (dest < 0) dest += push.n_dest;
            push_to_dest(push, dest, blockIdx.x, push.n_push_ctas);
        }
    }

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
            int walked = 0;  // tiles of the chunks before this one
            for (int ci = 0; ci < p.n_kv_chunks && ok; ++ci) {
                int c = p.kv_first + ci;
                if (c >= p.n_kv_chunks) c -= p.n_kv_chunks;
                const int tiles_c = tiles_in_chunk(c);
                const int t_lo = kSplit ? max(0, s_split[2] - walked) : 0;
                const int t_hi = kSplit ? min(tiles_c, s_split[2] + n_tiles - walked) : tiles_c;
                if (kSplit) walked += tiles_c;
                if (t_lo >= t_hi) continue;  // (a chunk none of whose tiles are mine is not waited for)
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
                for (int t = t_lo; t < t_hi; ++t, ++j) {
                    const int st = j & 1;
                    const uint32_t ph = (j >> 1) & 1;
                    const uint32_t bk = smem_u32(&ctl->k_full[st]);
                    const uint32_t bv = smem_u32(&ctl->v_full[st]);
                    dbg_stamp(p, 3, j, 0, true);
                    if (j >= kStages) {
                        ok = mbar_wait(smem_u32(&ctl->k_empty[st]), ph ^ 1, s_abort, p.status,
                                       pipe_limit, PA_DEV_TIMEOUT_PIPE);
                        if (!ok) break;
                    }
                    dbg_stamp(p, 3, j, 1, true);
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
                    dbg_stamp(p, 3, j, 2, true);
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
        // The issuer must keep ahead of the tensor core (64 cycles per 128x128x16 MMA). All 32
        // lanes of the warp run this code in lockstep and every tcgen05.mma / tcgen05.commit is
        // predicated on one elected lane: control flow and descriptor arithmetic stay
        // warp-uniform, which costs about 24 cycles per issued MMA where a single lane running
        // the loop alone (a divergent region) needs 55 to 75 and falls behind the tensor core.
        // The k-step loops are unrolled and every descriptor is a base plus a constant.
        if (n_tiles > 0) {
            constexpr uint32_t idesc_qk = make_idesc_f16(kBF16, false, kTileM, kTileN / 2);
            constexpr uint32_t idesc_pv = make_idesc_f16(kBF16, true, kTileM, kD);
            const uint32_t leader = elect_one() ? 1u : 0u;
            const bool stamper = (lane == 0);

            // Descriptors differ from a per-operand base only in the start-address field (units
            // of 16 bytes, bits 0-13 of the low word; shared memory ends below 2^18, so adding
            // never carries out of the field): one high word per operand kind, 32-bit arithmetic
            // on the low words.
            const uint64_t dq0 = smem_desc_sw128(sQ, 16, 1024);
            const uint64_t dv0 = smem_desc_sw128(sV, kHalfBytes, 1024);
            const uint32_t hi_qk = static_cast<uint32_t>(dq0 >> 32);
            const uint32_t hi_v = static_cast<uint32_t>(dv0 >> 32);
            const uint32_t lo_q = static_cast<uint32_t>(dq0);
            const uint32_t lo_k = static_cast<uint32_t>(smem_desc_sw128(sK, 16, 1024));
            const uint32_t lo_v = static_cast<uint32_t>(dv0);
            // Q K^T of one half of a key/value tile's rows (N = 64): key rows [64*half, 64*half+64)
            // sit 8 KB into the tile's shared-memory slot; S columns [64*half, 64*half+64).
            auto issue_qk_half = [&](int t, int st, int half) {
                const uint32_t a0 = lo_q + ((t * kTileBytes) >> 4);
                const uint32_t b0 = lo_k + ((st * kTileBytes + half * 64 * 128) >> 4);
                const uint32_t d = tmem + kColS0 + t * kTileN + half * (kTileN / 2);
#pragma unroll
                for (int ks = 0; ks < kD / 16; ++ks) {
                    const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
                    tc_mma_ss_elect(d, a0 + off, hi_qk, b0 + off, hi_qk, idesc_qk, ks > 0 ? 1u : 0u, leader);
                }
            };
            // P V for key rows [32*piece, 32*piece+32) of the tile: two k-steps of 16 keys. The
            // piece's probabilities sit in its half of the S columns, at [64*(piece/2) +
            // 16*(piece%2), +16), 8 columns per k-step.
            auto issue_pv_piece = [&](int t, int st, int piece, bool acc) {
                const uint32_t b0 = lo_v + ((st * kTileBytes) >> 4);
                const uint32_t a0 = tmem + kColS0 + t * kTileN;
                const uint32_t d = tmem + kColO0 + t * kD;
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                    const int ks = piece * 2 + k2;
                    const uint32_t b = b0 + ((ks * 16 * 128) >> 4);
                    const uint32_t accum = (acc || ks > 0) ? 1u : 0u;
                    tc_mma_ts_elect(d, a0 + (piece >> 1) * (kTileN / 2) + (ks & 3) * 8, b, hi_v, idesc_pv, accum, leader);
                }
            };

            bool ok = mbar_wait(smem_u32(&ctl->q_full), 0, s_abort, p.status, pipe_limit,
                                PA_DEV_TIMEOUT_PIPE);
            ok = ok && mbar_wait(smem_u32(&ctl->k_full[0]), 0, s_abort, p.status, pipe_limit,
                                 PA_DEV_TIMEOUT_PIPE);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        issue_qk_half(t, 0, half);
                        tc_commit_elect(smem_u32(&ctl->s_full[t][half]), leader);
                    }
                tc_commit_elect(smem_u32(&ctl->k_empty[0]), leader);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int stn = (j + 1) & 1;
                const uint32_t phn = ((j + 1) >> 1) & 1;
                const bool more = (j + 1 < n_tiles);
                dbg_stamp(p, 4, j, 0, stamper);
                ok = mbar_wait(smem_u32(&ctl->v_full[st]), ph, s_abort, p.status, pipe_limit,
                               PA_DEV_TIMEOUT_PIPE);
                dbg_stamp(p, 4, j, 1, stamper);
                if (ok && more)
                    ok = mbar_wait(smem_u32(&ctl->k_full[stn]), phn, s_abort, p.status, pipe_limit,
                                   PA_DEV_TIMEOUT_PIPE);
                dbg_stamp(p, 4, j, 2, stamper);
                // (every lane polls the same barriers; the vote keeps the warp in one piece when a
                // wait gives up in some lanes only)
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // Each query tile is two independent half-tiles in the key dimension, each with its
                // own chain softmax -> P V -> next Q K^T: while the softmax works on one half, the
                // tensor core does the other half's P V and next Q K^T, so neither the MMA latency
                // nor the hand-overs are ever waited for. (The N = 64 Q K^T runs at 48 instead of
                // 32 cycles per MMA - shared-memory operand fetch - which this overlap pays for.)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        dbg_stamp(p, 2, j, (half * 2 + t) * 2 + 0, stamper);
#pragma unroll
                        for (int c = 2 * half; c < 2 * half + 2; ++c) {
                            ok = mbar_wait(smem_u32(&ctl->p_full[t][c]), j & 1, s_abort, p.status, pipe_limit,
                                           PA_DEV_TIMEOUT_PIPE);
                            ok = __all_sync(0xffffffffu, ok);
                            if (!ok) break;
                            tc_fence_after();
                            issue_pv_piece(t, st, c, j > 0);
                            // one barrier per piece (one phase per tile each): a softmax warp that has to
                            // rescale O in the middle of a tile waits for the last piece issued so far
                            tc_commit_elect(smem_u32(&ctl->o_done[t][c]), leader);
                        }
                        if (!ok) break;
                        if (half == 1 && t == 1) tc_commit_elect(smem_u32(&ctl->v_empty[st]), leader);
                        if (more) {
                            issue_qk_half(t, stn, half);
                            tc_commit_elect(smem_u32(&ctl->s_full[t][half]), leader);
                            if (half == 1 && t == 1) tc_commit_elect(smem_u32(&ctl->k_empty[stn]), leader);
                        }
                        dbg_stamp(p, 2, j, (half * 2 + t) * 2 + 1, stamper);
                    }
                    if (!ok) break;
                }
            }
            if (!ok) {
                // Nothing may still be running on the tensor core when TMEM is released.
                int none = 0;
                volatile int* no_abort = &none;
                tc_commit_elect(smem_u32(&ctl->teardown), leader);
                mbar_wait(smem_u32(&ctl->teardown), 0, no_abort, nullptr, 100000000ull, 0);
            }
        }
    } else if (warp < kSoftmaxWarps) {
        // =============================== softmax + epilogue ================================
        setmaxnreg_inc<kRegsSoftmax>();
        const int quarter = warp & 3;
        const int t = warp >> 2;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t tS = tmem + lane_base + kColS0 + t * kTileN;  // my row's 128 logits
        const uint32_t tO = tmem + lane_base + kColO0 + t * kD;      // my row of the output
        const float sl = p.scale_log2;
        const bool stamper = (quarter == 0 && lane == 0);

        float m_ref = -INFINITY;  // the reference my row's probabilities and O are scaled by
        float l_sum = 0.f;
        bool ok = true;
        int j = 0;
        uint32_t buf[2][32];  // the logits of the piece at hand and of the next one
        bool pre = false;     // the load of the next piece has been issued
        int pending = -1;     // piece whose probabilities are stored but not handed over yet
        const long long q_here = kCausal ? p.q_pos[qc] + row0 + t * kTileM + row_in_tile : 0;  // my row's global position
        int walked = 0;
        for (int ci = 0; ci < p.n_kv_chunks; ++ci) {
            int c_kv = p.kv_first + ci;
            if (c_kv >= p.n_kv_chunks) c_kv -= p.n_kv_chunks;
            const int tiles_c = tiles_in_chunk(c_kv);
            const int t_lo = kSplit ? max(0, s_split[2] - walked) : 0;
            const int t_hi = kSplit ? min(tiles_c, s_split[2] + n_tiles - walked) : tiles_c;
            if (kSplit) walked += tiles_c;
            for (int tk = t_lo; tk < t_hi; ++tk, ++j) {
                // which of the tile's 128 key columns count for my row: the key mask words (the
                // same for the whole warp), cut at the ragged end of the chunk and at the causal
                // diagonal
                const int exist = min(kTileN, p.kv_rows - tk * kTileN);
                int valid = exist;
                if (kCausal) {
                    const long long lim = q_here - (p.kv_pos[c_kv] + tk * kTileN) + 1;
                    valid = static_cast<int>(lim < valid ? (lim < 0 ? 0 : lim) : valid);
                }
                unsigned long long kw[2] = {~0ull, ~0ull};
                if (p.key_bits != nullptr) {  // (a half tile past the chunk's end has no word)
                    const unsigned long long* w = p.key_bits + bidx * p.kb_sb + c_kv * p.kb_sc + tk * 2;
                    kw[0] = __ldg(w);
                    if (exist > 64) kw[1] = __ldg(w + 1);
                }
                const bool plain = (valid == kTileN) && (p.key_bits == nullptr);
                const bool plain_warp = __all_sync(0xffffffffu, plain);
                // The tile is worked on as two halves of its key columns (pieces 0,1 and 2,3), each as
                // soon as its Q K^T has landed; while this thread is busy with one half the tensor
                // core runs the other half's P V and next Q K^T. The pieces form one rolling
                // pipeline across halves and tiles: while piece c is exponentiated the load of
                // the next piece is in flight - if that piece opens a new half, only when its
                // Q K^T is already there (one non-blocking look at the barrier), which it is
                // whenever the tensor core is ahead - and the hand-over of a half's first piece is
                // issued behind the second piece's exponentials, when its TMEM store has long landed.
#pragma unroll
                for (int c = 0; c < kPieces; ++c) {
                    const int half = c >> 1, i = c & 1;
                    uint32_t(&sc)[32] = buf[i];
                    if (!pre) {
                        if (pending >= 0) {  // never block with a hand-over outstanding
                            tc_wait_st();
                            tc_fence_before();
                            mbar_arrive(smem_u32(&ctl->p_full[t][pending]));
                            pending = -1;
                        }
                        if (i == 0) {
                            dbg_stamp(p, t, j, half * 4 + 0, stamper);
                            // A wait that gives up does not leave the loop: once the abort word is set
                            // no wait blocks any more, and the arrivals keep the other roles moving.
                            ok = mbar_wait(smem_u32(&ctl->s_full[t][half]), j & 1, s_abort, p.status, pipe_limit,
                                           PA_DEV_TIMEOUT_PIPE) && ok;
                            tc_fence_after();
                            dbg_stamp(p, t, j, half * 4 + 1, stamper);
                        }
                        tmem_ld32(tS + c * kPieceCols, sc);
                    }
                    tc_wait_ld();
                    tmem_ld_fence(sc);
                    // the next piece: same half - its logits are there; first piece of the other half or
                    // of the next tile - only if its Q K^T has already been committed
                    pre = false;
                    if (i == 0) {
                        pre = true;
                    } else if (c == 1) {
                        pre = __all_sync(0xffffffffu, mbar_try_wait(smem_u32(&ctl->s_full[t][1]), j & 1));
                    } else if (j + 1 < n_tiles) {
                        pre = __all_sync(0xffffffffu, mbar_try_wait(smem_u32(&ctl->s_full[t][0]), (j + 1) & 1));
                    }
                    if (pre) {
                        if (i == 1) tc_fence_after();
                        tmem_ld32(tS + ((c + 1) & 3) * kPieceCols, buf[i ^ 1]);
                    }
                    uint32_t live = 0xffffffffu;
                    uint32_t pk[16];
                    float ls, mx;
                    const float neg = (m_ref == -INFINITY) ? 0.0f : -m_ref * sl;
                    if (plain_warp) {
                        softmax_chunk<kBF16, false>(sc, live, sl, neg, pk, ls, mx);
                    } else {
                        const int v = valid - c * kPieceCols;
                        live = (v >= 32) ? 0xffffffffu : (v <= 0 ? 0u : ((1u << v) - 1u));
                        live &= static_cast<uint32_t>(kw[half] >> (i * 32));
                        softmax_chunk<kBF16, true>(sc, live, sl, neg, pk, ls, mx);
                    }
                    if (pending >= 0) {  // the previous piece, behind this piece's exponentials
                        tc_wait_st();
                        tc_fence_before();
                        mbar_arrive(smem_u32(&ctl->p_full[t][pending]));
                        pending = -1;
                    }
                    // (m_ref = mx = -inf: NaN > threshold is false, the row stays empty)
                    const bool grow = (mx - m_ref) * sl > kRescaleThreshold;
                    // P of key columns [32c, 32c+32) goes over consumed S columns of its half
                    const uint32_t tP = tS + half * (kTileN / 2) + i * (kPieceCols / 2);
                    if (__any_sync(0xffffffffu, grow)) {
                        if (pre) {  // no load may be in flight across the call
                            tc_wait_ld();
                            tmem_ld_fence(buf[i ^ 1]);
                        }
                        // every P V handed over so far must have been added to O before O is
                        // rescaled: the last one is waited for (MMAs complete in order)
                        const uint32_t bo = (c > 0) ? smem_u32(&ctl->o_done[t][c - 1])
                                                    : smem_u32(&ctl->o_done[t][kPieces - 1]);
                        const uint32_t par = (c > 0) ? (j & 1) : ((j - 1) & 1);
                        const float2 r = softmax_piece_regrow<kBF16, kD>(
                            tS + c * kPieceCols, tP, tO, live, sl, mx, m_ref, l_sum, j > 0 || c > 0, bo, par, s_abort,
                            p.status, pipe_limit);
                        m_ref = r.x;
                        l_sum = r.y;
                    } else {
                        l_sum += ls;
                        tmem_st16(tP, pk);
                    }
                    // (a half's last piece is handed over at once: its P V and the half's next Q K^T
                    // have only the time this thread spends on the other half)
                    if (i == 0) {
                        pending = c;
                    } else {
                        tc_wait_st();
                        tc_fence_before();
                        mbar_arrive(smem_u32(&ctl->p_full[t][c]));
                    }
                    if (i == 1) dbg_stamp(p, t, j, half * 4 + 3, stamper);
                }
            }
        }
        if (pending >= 0) {
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&ctl->p_full[t][pending]));
        }
        // (a CTA whose queries see no key at all writes zeros and an LSE of -inf)
        const bool empty = (n_tiles == 0);
        if (!empty)
            ok = mbar_wait(smem_u32(&ctl->o_done[t][kPieces - 1]), (n_tiles - 1) & 1, s_abort, p.status, pipe_limit,
                           PA_DEV_TIMEOUT_PIPE) && ok;
        if (ok) {
            tc_fence_after();
            const int row = row0 + t * kTileM + row_in_tile;
            const bool in_range = row < p.q_rows;
            // a row that saw no key (all masked) comes out as zeros with an LSE of -inf
            const float inv = (empty || !(l_sum > 0.0f)) ? 0.0f : 1.0f / l_sum;
            uint16_t* orow = reinterpret_cast<uint16_t*>(p.out[qc]) +
                             (static_cast<long long>(bidx) * p.o_sb + static_cast<long long>(head) * p.o_sh +
                              static_cast<long long>(row) * p.o_ss);
            if (kSplit && s_split[0] >= 0) {
                const int split_unit = s_split[0], share = s_split[1];
                const size_t base = static_cast<size_t>(split_unit) * p.split_k * (2 * kTileM);
                float* lse_row = (p.lse[qc] == nullptr) ? nullptr
                                                        : p.lse[qc] + static_cast<long long>(bidx) * p.l_sb +
                                                              static_cast<long long>(head) * p.l_sh + row;
                split_epilogue<kBF16, kD>(tO, empty ? -INFINITY : m_ref, empty ? 0.0f : l_sum, sl, p.scale, lane,
                                          t * kTileM + row_in_tile, share, p.split_k, p.part_o + base * kD,
                                          p.part_ml + base, p.part_cnt + split_unit * 9 + warp, orow, lse_row,
                                          in_range);
            } else {
#pragma unroll
            for (int b = 0; b < kD / 32; ++b) {
                uint32_t o[32];
                tmem_ld32(tO + b * 32, o);
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
                            const float b2 = __uint_as_float(o[v4 * 8 + 2 * i + 1]) * inv;
                            wp[i] = kBF16 ? pack_bf16x2(a, b2) : pack_f16x2(a, b2);
                        }
                        *reinterpret_cast<uint4*>(orow + b * 32 + v4 * 8) = w;
                    }
                }
            }
            if (in_range && p.lse[qc] != nullptr) {
                p.lse[qc][static_cast<long long>(bidx) * p.l_sb + static_cast<long long>(head) * p.l_sh + row] =
                    m_ref * p.scale + __logf(l_sum);
            }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (p.done_flag[qc] != nullptr && *s_abort == 0) {
        // every output store of this CTA is ordered before the counter update
        // (of a split unit's CTAs the one that finishes last reports the unit: by then every
        // share's warps have written whatever rows fell to them)
        if (threadIdx.x == 0) {
            __threadfence_system();
            bool report = true;
            if (kSplit && s_split[0] >= 0) {
                report = (atomicAdd(p.part_cnt + s_split[0] * 9 + 8, 1u) + 1u == static_cast<unsigned int>(p.split_k));
                if (report) __threadfence_system();
            }
            if (report) red_release_sys_add(p.done_flag[qc], 1u);
        }
    }
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace pa
