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
 * base and strides too. head_dim must be 128; dtype bf16 or f16; accumulation is fp32.
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
} pa_attn_args;

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
typedef struct pa_cp_attn_args {
    const void* q_stage;     /* [n_q_chunks, batch, heads, q_rows, 128] */
    const void* k_stage;     /* [n_kv_chunks, batch, heads, kv_rows, 128] */
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
} pa_cp_attn_args;

int pa_cp_attn_fwd(const pa_cp_attn_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PA_B200_H_ */
