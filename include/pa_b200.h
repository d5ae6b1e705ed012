/*
 * pa_b200 — C ABI of the B200 (sm_100a) context-parallel attention library.
 *
 * Every entry point takes raw device pointers, explicit element strides and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), returns an int status (PA_OK or a negative code),
 * never throws, never synchronises the device, and — unless its comment says otherwise —
 * never allocates device memory: scratch is provided by the caller. pa_last_error()
 * returns a human-readable message for the last failing call on the calling thread.
 *
 * The Python package `paraattention_b200` binds these with ctypes; the functions they
 * stand in for are cited as `file:line` of the ParaAttention source tree (or of PyTorch's
 * torch/distributed/tensor/experimental/_context_parallel/_attention.py, marked torch:).
 */
#ifndef PA_B200_H_
#define PA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_MAX_CHUNKS 8

enum pa_status {
    PA_OK = 0,
    PA_EINVAL = -1,    /* bad argument (shape, stride, alignment, null pointer) */
    PA_ENOTSUP = -2,   /* valid request this build has no kernel for */
    PA_ECUDA = -3,     /* a CUDA runtime / driver call failed */
    PA_ETIMEDOUT = -4  /* reported through a device status word, see pa_attn_args.status */
};

enum pa_dtype { PA_BF16 = 0, PA_F16 = 1 };

/* Codes a kernel writes into its device status word when a bounded wait runs out. */
enum pa_device_status {
    PA_DEV_OK = 0,
    PA_DEV_TIMEOUT_PIPE = 1,  /* an in-kernel pipeline barrier */
    PA_DEV_TIMEOUT_Q = 2,     /* a query chunk's ready flag */
    PA_DEV_TIMEOUT_KV = 3,    /* a key/value chunk's ready flag */
    PA_DEV_TIMEOUT_OUT = 4    /* the output-arrival counter */
};

const char* pa_last_error(void);
int pa_version(void);

/* ------------------------------------------------------------------------------------------
 * Attention forward: out = softmax(scale * q k^T) v, lse = logsumexp_k(scale * q k^T)
 * (natural log, fp32). Replaces the SDPA-with-LSE backends behind
 * torch.ops.para_attn.attention_forward_with_lse / attention_forward
 * (src/para_attn/ops/__init__.py:48-245).
 *
 * Tensors are [batch, heads, seq, head_dim] with arbitrary element strides for the first
 * three dims and stride 1 for head_dim (BSHD memory viewed as BHSD is fine). Base pointers
 * and byte strides of q, k, v must be multiples of 16 bytes; out needs 16-byte alignment of
 * base and strides too. head_dim must be 64 or 128; dtype bf16 or f16; accumulation is fp32.
 * lse may be NULL. status may be NULL; if given it must point to a zero-initialised device
 * int that receives a pa_device_status code when a wait inside the kernel gives up.
 * ---------------------------------------------------------------------------------------- */
typedef struct pa_attn_args {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;              /* [batch, heads, seq_q] contiguous, or NULL */
    int32_t batch, heads, seq_q, seq_kv, head_dim;
    int32_t dtype;           /* pa_dtype */
    int32_t is_causal;       /* top-left aligned causal mask, as torch SDPA */
    float scale;             /* softmax scale, e.g. 1/sqrt(head_dim) */
    int64_t q_stride[3];     /* element strides of (batch, head, seq) */
    int64_t k_stride[3];
    int64_t v_stride[3];
    int64_t o_stride[3];
    int32_t* status;         /* device int or NULL */
    uint64_t wait_limit_ns;  /* 0 = default (2 s) */
    /* Key-padding mask, or NULL when every key is valid: words written by pa_pack_key_mask with
     * n_chunks = 1 and rows = seq_kv, [batch][ceil(seq_kv / 64)]. Masked keys take no part in the
     * softmax: the same result as dropping them from k and v, which is what
     * _attention_forward_sparse_kv does with index_select (src/para_attn/ops/__init__.py:248-299).
     * A query row without any visible key comes out as zeros with an LSE of -inf. */
    const uint64_t* key_bits;
    /* Optional scratch (NULL: none), 256-byte aligned device memory of workspace_bytes bytes that
     * calls running at the same time must not share. With it, a non-causal launch whose last wave
     * of CTAs would leave most SMs idle gives each work unit of that wave to several CTAs that
     * split the keys among them and combine their partial results before the output is written
     * (same result up to fp32 summation order). pa_attn_workspace_bytes() is a size that covers
     * every shape; with less, fewer CTAs share a unit, or none. */
    void* workspace;
    int64_t workspace_bytes;
} pa_attn_args;

int64_t pa_attn_workspace_bytes(void);

/* What a launch with `units` work units (pairs of 128-row query tiles x heads x batch x query
 * chunks) and kv_tiles key/value tiles of 128 rows per unit does with a workspace of that size on
 * a device with sm_count SMs (fused_push != 0: a pa_cp_attn_fwd call whose leading CTAs push):
 * units [0, *split_from) are computed by one CTA each, every later
 * unit by *split_k CTAs in a second launch (*split_k = 1, *split_from = units: one launch,
 * nothing split). Needs no device. */
int pa_attn_split_plan(int64_t units, int32_t sm_count, int64_t kv_tiles, int32_t head_dim, int32_t is_causal,
                       int32_t fused_push, int64_t workspace_bytes, int32_t* split_from, int32_t* split_k);

int pa_attn_fwd(const pa_attn_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Chunked attention forward for context parallelism. Queries and keys/values live in
 * staging buffers laid out [chunk, batch, heads, rows, head_dim] (contiguous), one chunk per
 * source rank. Key/value chunks are consumed starting at kv_first and wrapping; each chunk
 * is used as soon as its ready counter (written by the owning rank's pa_cp_push) reaches
 * flag_expect, so transfers overlap the tiles already being computed, and the running
 * output / log-sum-exp never leave the SM between chunks. This folds the K/V rotation and
 * the out/LSE merge of torch:_templated_ring_attention (torch:...:309-478, 138-223) and the
 * head<->sequence all-to-alls of src/para_attn/para_attn_interface.py:52-119 into one launch.
 *
 * Output rows of query chunk c are written to out[c] (which may be a peer GPU's mapped
 * memory) at [batch, out_head_offset + head, row, :] with the given element strides, and
 * lse likewise if lse[c] != NULL. After a CTA has stored a tile for chunk c it adds 1 to
 * done_flag[c] (system-scope release) when that pointer is non-NULL.
 * ---------------------------------------------------------------------------------------- */
struct pa_cp_push_args;

typedef struct pa_cp_attn_args {
    const void* q_stage;     /* [n_q_chunks, batch, heads, q_rows, head_dim] */
    const void* k_stage;     /* [n_kv_chunks, batch, heads, kv_rows, head_dim] */
    const void* v_stage;
    int32_t batch, heads, head_dim, dtype;
    int32_t n_q_chunks, q_rows, q_first;
    int32_t n_kv_chunks, kv_rows, kv_first;
    float scale;
    void* out[PA_MAX_CHUNKS];
    float* lse[PA_MAX_CHUNKS];
    int64_t o_stride[3];     /* element strides (batch, head, row) inside out[c] */
    int64_t lse_stride[2];   /* element strides (batch, head) inside lse[c]; row stride 1 */
    int32_t out_head_offset;
    const uint32_t* q_flag[PA_MAX_CHUNKS];   /* NULL = chunk is already there */
    const uint32_t* kv_flag[PA_MAX_CHUNKS];
    uint32_t flag_expect;
    uint32_t* done_flag[PA_MAX_CHUNKS];
    int32_t* status;
    uint64_t wait_limit_ns;
    /* Fused exchange (may be NULL): the first fused_push->ctas_per_dest CTAs of this launch
     * (capped by the grid size and the number of SMs, so that all of them are resident at once)
     * perform the pushes described by *fused_push before they take up attention tiles, and add
     * 1 each to every destination's counter. The consumers' flag_expect must therefore grow by
     * that CTA count per call. The host struct is read during the call only. */
    const struct pa_cp_push_args* fused_push;
    /* Zero-copy own shard (each may be NULL): when given, query chunk q_first (key/value chunk
     * kv_first) is not read from the staging buffer but straight from this rank's own tensor,
     * [batch, all heads, rows, head_dim] with the given element strides, heads
     * [local_head_offset, local_head_offset + heads); its ready flag is ignored. */
    const void* q_local;
    const void* k_local;
    const void* v_local;
    int64_t q_local_stride[3];
    int64_t k_local_stride[3];
    int64_t v_local_stride[3];
    int32_t local_head_offset;
    int32_t local_total_heads;
    /* Causal masking over the whole (sharded) sequence: when is_causal != 0, row i of query
     * chunk c sits at global position q_pos[c] + i and row j of key/value chunk c at
     * kv_pos[c] + j; a key is visible to a query iff its position is not later. Key/value tiles
     * no query of a CTA can see are skipped (neither waited for nor read). This replaces the
     * per-step is_causal / skip logic of torch:_templated_ring_attention (torch:...:394-437)
     * and covers the Ulysses case, where every rank sees whole sequences. Query rows that see
     * no key at all come out as zeros with an LSE of -inf. */
    int32_t is_causal;
    int32_t pad_;
    int64_t q_pos[PA_MAX_CHUNKS];
    int64_t kv_pos[PA_MAX_CHUNKS];
    /* Key-padding mask over all chunks, or NULL: [batch][n_kv_chunks][ceil(kv_rows / 64)] words
     * from pa_pack_key_mask. Lifts the reference's "no mask with ring attention" limit
     * (src/para_attn/para_attn_interface.py:228). */
    const uint64_t* key_bits;
    /* Optional scratch, as in pa_attn_args (local device memory, never a peer's). Ignored when
     * fused_push is given: behind pushing CTAs the split was measured slower. */
    void* workspace;
    int64_t workspace_bytes;
} pa_cp_attn_args;

int pa_cp_attn_fwd(const pa_cp_attn_args* args, void* stream);

/* Packs a boolean key mask (one byte per key, non-zero = valid; [batch][n_chunks * rows] with the
 * given batch stride in bytes) into the words the attention entry points read:
 * out[batch][n_chunks][ceil(rows / 64)], bit i of a chunk's word i / 64 = key row i of that chunk.
 * Replaces the index construction of _attention_forward_sparse_kv
 * (src/para_attn/ops/__init__.py:271-283). */
int pa_pack_key_mask(const uint8_t* mask, int64_t batch_stride, int32_t batch, int32_t n_chunks, int32_t rows,
                     uint64_t* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * The neighbours of attention in a transformer block, one HBM-bound pass instead of a dozen
 * tensor operations: per-head RMSNorm of q and k with a per-channel weight, rotary embedding of
 * both, and placement of q, k, v into the buffers attention reads. No single counterpart in
 * the reference: it is what the models' attention processors do between the q/k/v projections
 * and the scaled_dot_product_attention call that the modes of
 * src/para_attn/para_attn_interface.py:279-495 intercept.
 *
 * q, k, v: [batch, rows, heads, head_dim] with element strides (batch, row, head), head_dim
 * contiguous (64 or 128). v and v_out may be NULL (then v is not touched). q_weight / k_weight:
 * [head_dim] in the tensors' dtype, or NULL (no normalisation). cos / sin: fp32 tables
 * [>= table_row0 + rows, head_dim] whose row table_row0 + r belongs to row r, or both NULL.
 * Rotation pairs are the adjacent elements (2i, 2i+1): out[2i] = x[2i] cos[2i] - x[2i+1] sin[2i],
 * out[2i+1] = x[2i+1] cos[2i+1] + x[2i] sin[2i+1]. Outputs may alias nothing but themselves.
 * ---------------------------------------------------------------------------------------- */
typedef struct pa_qkv_prep_args {
    const void* q;
    const void* k;
    const void* v;
    void* q_out;
    void* k_out;
    void* v_out;
    int64_t q_stride[3], k_stride[3], v_stride[3];              /* element strides (batch, row, head) */
    int64_t q_out_stride[3], k_out_stride[3], v_out_stride[3];
    const void* q_weight;
    const void* k_weight;
    const float* cos;
    const float* sin;
    int64_t table_row0;
    int32_t batch, rows, heads, head_dim;
    int32_t dtype;           /* pa_dtype */
    float eps;
} pa_qkv_prep_args;

int pa_qkv_prep(const pa_qkv_prep_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Exchange. Replaces the NCCL all_to_all_single calls of _sdpa_input_all_to_all /
 * _sdpa_output_all_to_all (src/para_attn/para_attn_interface.py:52-87, through
 * src/para_attn/primitives.py:72-78) and the K/V rotation of torch:_AllToAllRotater
 * (torch:247-263): each job copies rows [batch, head0..head0+heads, rows, head_dim] of a local
 * tensor to dst (normally a peer GPU's mapped staging buffer) with the given element
 * strides; when all jobs of a destination are stored, flag[dest] on that destination is
 * increased by ctas_per_dest in total (each CTA adds 1 with a system-scope release).
 * pa_cp_push is the stand-alone launch (grid ctas_per_dest x n_dest); the same description
 * can ride inside pa_cp_attn_fwd (pa_cp_attn_args.fused_push), which is what multi-GPU runs
 * use: a separate push kernel is not guaranteed to get SMs while attention CTAs that wait
 * for it fill the device.
 * ---------------------------------------------------------------------------------------- */
#define PA_MAX_PUSH_JOBS 24

typedef struct pa_push_job {
    const void* src;
    void* dst;
    int64_t src_stride[3];   /* element strides (batch, head, row); head_dim contiguous 16-bit elements per row */
    int64_t dst_stride[3];
    int32_t head0, heads, batch, rows;
    int32_t dest;            /* index into pa_cp_push_args.flag */
    int32_t head_dim;        /* 64 or 128; 0 means 128 */
} pa_push_job;

typedef struct pa_cp_push_args {
    pa_push_job jobs[PA_MAX_PUSH_JOBS];
    int32_t n_jobs;
    int32_t n_dest;
    uint32_t* flag[PA_MAX_CHUNKS];
    int32_t ctas_per_dest;
    int32_t first_dest;      /* fused form: destinations are served in the order first_dest,
                              * first_dest - 1, ... (mod n_dest), the order in which consumers
                              * that walk their chunks upwards from their own rank need them */
} pa_cp_push_args;

int pa_cp_push(const pa_cp_push_args* args, void* stream);

/* Stream-ordered bounded wait until every flag[i] >= expect (i < n). On timeout the device
 * status word receives `code` (a pa_device_status value). Stands where the reference calls
 * .wait() on a functional collective (src/para_attn/primitives.py:36-43). */
int pa_flag_wait(const uint32_t* const* flag, int32_t n, uint32_t expect, int32_t* status, uint64_t wait_limit_ns,
                 int32_t code, void* stream);

/* ------------------------------------------------------------------------------------------
 * Merge of two partial attention results, torch:_SDPAMerger._merge_one (torch:182-183):
 * acc_out (fp32 [rows, d]) and acc_lse (fp32 [rows]) are updated in place from a block's
 * out (blk_dtype: PA_BF16, PA_F16 or 2 = fp32) and lse (fp32).
 * ---------------------------------------------------------------------------------------- */
int pa_merge_out_lse(float* acc_out, float* acc_lse, const void* blk_out, const float* blk_lse, int64_t rows,
                     int32_t d, int32_t blk_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * First Block Cache. pa_fbc_residual_diff fuses the residual formation of
 * CachedTransformerBlocks.forward (src/para_attn/first_block_cache/utils.py:359) with the two
 * reductions of are_two_tensors_similar (utils.py:228-229) and the store of
 * set_first_hidden_states_residual (utils.py:289-295):
 *   cur = round(h1 - h0); result[0] = sum |round(prev - cur)|; result[1] = sum |prev|;
 *   result[2], result[3] = the two means rounded to dtype; result[4] = round(result[2]/result[3]).
 * h1, h0: [rows, cols] contiguous. With downsample > 1 only every downsample-th column takes
 * part and prev / new_resid are compact [rows, ceil(cols/downsample)]. prev and new_resid may
 * be NULL (no comparison / no store). result: 5 floats. scratch: pa_fbc_scratch_bytes() bytes
 * whose last 4 bytes (the ticket) must be zero before the first call; the kernel leaves them
 * zero. Calls sharing a scratch buffer must not overlap on the GPU.
 * ---------------------------------------------------------------------------------------- */
int64_t pa_fbc_scratch_bytes(void);
int pa_fbc_residual_diff(const void* h1, const void* h0, const void* prev, void* new_resid, int64_t rows,
                         int32_t cols, int32_t downsample, int32_t dtype, float* result, void* scratch,
                         void* stream);

/* pa_fbc_residual_diff for hosts that cannot supply scratch memory. It has no counterpart in
 * the reference. Meant for callers that own no device allocator at the point of the call - a
 * serving process whose GPU memory is partitioned once at start-up and frozen afterwards, or a
 * foreign-language binding that merely passes on buffers it was handed. The partial sums live
 * in a 4864-byte array built into the library image (one copy on every GPU that loads the
 * library, kept until the process ends); the call itself allocates and frees nothing.
 *
 * Same arguments and results as pa_fbc_residual_diff, without `scratch`. Limits and rules:
 *  - rows * cols must not exceed PA_FBC_STATIC_MAX_NUMEL (the grid is capped at 592 CTAs, and
 *    beyond that size the per-thread fp32 partial sums would lose accuracy); larger inputs are
 *    refused with PA_EINVAL;
 *  - the first call on each device looks up the array's device address (that device must be
 *    current); make that first call before any stream capture begins;
 *  - all calls on a device share the one array: the ticket word in it is cleared in stream
 *    order before each launch, and two calls that overlap on the GPU (different streams) race. */
#define PA_FBC_STATIC_MAX_NUMEL (1LL << 30)
int pa_fbc_residual_diff_static(const void* h1, const void* h0, const void* prev, void* new_resid, int64_t rows,
                                int32_t cols, int32_t downsample, int32_t dtype, float* result, void* stream);

/* out = round(a + b) (sub = 0) or round(a - b) (sub = 1), elementwise over numel 16-bit
 * elements (numel % 8 == 0, 16-byte aligned pointers): apply_prev_hidden_states_residual
 * (utils.py:237-259) and the residual formation at utils.py:443-444. */
int pa_fbc_axpy(const void* a, const void* b, void* out, int64_t numel, int32_t sub, int32_t dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * TaylorSeer (src/para_attn/first_block_cache/taylorseer.py), the extrapolating variant of the
 * cached residual. All tensors hold numel 16-bit elements (numel % 8 == 0, 16-byte aligned).
 *
 * pa_taylor_update: TaylorSeer.approximate_derivative (taylorseer.py:29-38) in one pass. y is
 * d_0 of the step just computed, prev[i] the d_i of the previous computed step (i < depth), and
 * cur[i] receives d_{i+1} = round(round(d_i - prev[i]) / window), chained in registers.
 * depth <= 4; depth 0 does nothing.
 *
 * pa_taylor_approx: TaylorSeer.approximate_value (taylorseer.py:40-48): out = d[0] +
 * sum_{i=1}^{terms-1} round(round(d[i] / i!) * elapsed^i) with the sum rounded after every
 * term, as the chain of tensor operations rounds; terms <= 5. With add != NULL the kernel also
 * performs the addition of apply_prev_hidden_states_residual (utils.py:238-243):
 * out = round(that + add).
 * ---------------------------------------------------------------------------------------- */
int pa_taylor_update(const void* y, const void* const* prev, void* const* cur, int32_t depth, int32_t window,
                     int64_t numel, int32_t dtype, void* stream);
int pa_taylor_approx(const void* const* d, int32_t terms, int32_t elapsed, const void* add, void* out, int64_t numel,
                     int32_t dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PA_B200_H_ */
