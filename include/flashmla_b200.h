/*
 * flashmla_b200 -- C ABI of the B200 (sm_100a) MLA decode / sparse-prefill path.
 *
 * Every entry point takes plain device pointers, sizes and strides; nothing in a
 * signature depends on PyTorch.  All pointers are DEVICE pointers unless stated
 * otherwise; strides are in ELEMENTS of the pointed-to type unless the field name
 * ends in `_bytes`; `stream` is a cudaStream_t passed as void*.  Kernels are
 * enqueued on `stream` and the call returns without synchronising.
 *
 * Return value: 0 on success, otherwise one of the MLA_ERR_* codes;
 * mla_last_error() then returns a human-readable message (thread-local).
 *
 * The functions replace the five pybind11 functions of the reference's
 * `flash_mla.cuda` module (csrc/api/api.cpp:8-15) for the MLA path; each
 * declaration cites the reference interface it stands in for (paths relative to
 * the deepseek-ai/FlashMLA project root).
 */
#ifndef FLASHMLA_B200_H_
#define FLASHMLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLA_OK                 0
#define MLA_ERR_INVALID_ARG    1   /* shape / stride / alignment / null-pointer problem            */
#define MLA_ERR_UNSUPPORTED    2   /* a combination this library has no kernel for                 */
#define MLA_ERR_CUDA           3   /* a CUDA runtime / driver call failed                          */
#define MLA_ERR_DEVICE_STATUS  4   /* a kernel reported a bounded wait that ran out (see status)   */

/* One row of tile-scheduler metadata.  Same 32-byte layout as the reference's
 * DecodingSchedMeta (csrc/params.h:10-17). */
typedef struct {
    int32_t begin_req_idx;          /* first request of this SM partition                     */
    int32_t end_req_idx;            /* last request (inclusive)                               */
    int32_t begin_block_idx;        /* first 64-token block of the first request              */
    int32_t end_block_idx;          /* one past the last block of the last request            */
    int32_t begin_split_idx;        /* split number of the first request within that request  */
    int32_t is_first_req_splitted;
    int32_t is_last_req_splitted;
    int32_t _pad;                   /* never written                                          */
} mla_sched_meta_t;

/* Element type of q, the KV cache and out (dense decode; everything else is bf16).  Accumulation is fp32 either way. */
#define MLA_DTYPE_BF16  0
#define MLA_DTYPE_FP16  1

/* Which decode kernel family the partition count is asked for. */
#define MLA_MODE_DENSE_DECODE   0
#define MLA_MODE_SPARSE_DECODE  1

/* Message of the last failing call on this thread ("" if none). */
const char* mla_last_error(void);

/* Library ABI version (bumped when a struct below changes). */
int mla_abi_version(void);

/* Number of SM partitions the decode kernels of `mode` use on `device` for a
 * launch with these head counts / query length.  Stands in for the expression in
 * csrc/api/dense_decode.h:78 and DecodeImplBase::get_meta
 * (csrc/api/sparse_decode.h:92-99,126-133).  Returns <= 0 on error. */
int mla_num_sm_parts(int device, int mode, int h_q, int h_kv, int s_q);

/* Same, for a batch of `b` requests that all cost `blocks_per_request` KV blocks of 64 tokens (sparse decode with a
 * fixed top-k and no per-request lengths; the reference derives its partition count from the SM count alone at
 * csrc/api/sparse_decode.h:92-99).  May return fewer partitions than mla_num_sm_parts so that no partition
 * straddles two requests.  Deterministic in its arguments: callers that cache metadata get the same count back. */
int mla_num_sm_parts_uniform(int device, int mode, int h_q, int h_kv, int s_q, int b, int blocks_per_request);

/* Tile-scheduler metadata.  Replaces run_get_decoding_sched_meta_kernel
 * (csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu:109-114);
 * arguments mirror GetDecodeSchedMetaParams (csrc/params.h:127-143). */
typedef struct {
    int32_t b;                        /* batch size                                            */
    int32_t s_q;
    int32_t block_size_n;             /* tokens per scheduling block (64)                      */
    int32_t fixed_overhead_num_blocks;
    int32_t topk;                     /* -1 for dense attention                                */
    int32_t extra_topk;               /* 0 when there is no extra KV cache                     */
    const int32_t* topk_length;       /* [b] or NULL                                           */
    const int32_t* extra_topk_length; /* [b] or NULL                                           */
    const int32_t* seqlens_k;         /* [b], dense attention only                             */
    mla_sched_meta_t* meta;           /* out: [num_sm_parts]                                   */
    int32_t* num_splits;              /* out: [b + 1]                                          */
    int32_t num_sm_parts;
    void* stream;
} mla_sched_meta_args_t;
int mla_get_sched_meta(const mla_sched_meta_args_t* args);

/* Dense BF16 paged MLA decode (split-KV part; the caller runs mla_combine after
 * it).  Replaces sm90::run_flash_splitkv_mla_kernel as driven by
 * dense_attn_decode_interface (csrc/api/dense_decode.h:13-225); arguments mirror
 * DenseAttnDecodeParams (csrc/params.h:19-61).  Unlike the reference no
 * head/row regrouping copy of q is needed: the kernel addresses q and out
 * through the strides below. */
typedef struct {
    int32_t b, s_q, h_q, h_kv;
    int32_t d_qk, d_v;                /* 576, 512                                              */
    int32_t num_blocks;               /* pages in k_cache                                      */
    int32_t page_block_size;          /* 64                                                    */
    int32_t is_causal;
    float softmax_scale;

    const void* q;                    /* bf16 or fp16 (see dtype) [b, s_q, h_q, d_qk]          */
    int64_t q_stride_b, q_stride_s, q_stride_h;
    const void* k_cache;              /* same type [num_blocks, page_block_size, h_kv, d_qk]   */
    int64_t k_stride_block, k_stride_row, k_stride_head;
    const int32_t* block_table;       /* [b, max_blocks_per_seq]                               */
    int64_t block_table_stride_b;
    int32_t max_blocks_per_seq;
    const int32_t* seqlens_k;         /* [b]                                                   */

    void* out;                        /* same type as q [b, s_q, h_q, d_v]                     */
    int64_t o_stride_b, o_stride_s, o_stride_h;
    float* lse;                       /* fp32, element (b, s, h) at b*lse_stride_b + s*lse_stride_s + h*lse_stride_h */
    int64_t lse_stride_b, lse_stride_s, lse_stride_h;

    const mla_sched_meta_t* meta;     /* [num_sm_parts]                                        */
    const int32_t* num_splits;        /* [b + 1]                                               */
    int32_t num_sm_parts;

    float* lse_accum;                 /* scratch fp32 [b + num_sm_parts, s_q, h_q]   (base-2 LSE of each split) */
    float* o_accum;                   /* scratch fp32 [b + num_sm_parts, s_q, h_q, d_v]        */

    int32_t* status;                  /* optional device int32[4]; nonzero [0] after the launch means a bounded wait ran out */
    int32_t impl;                     /* 0 = pick the fastest kernel that supports the shape; 1 = portable kernel; 2 = tcgen05 kernel */
    int32_t dtype;                    /* MLA_DTYPE_BF16 or MLA_DTYPE_FP16 (the reference accepts both: csrc/api/dense_decode.h:33) */
    void* stream;
} mla_dense_decode_args_t;
int mla_dense_decode_fwd(const mla_dense_decode_args_t* args);

/* Sparse FP8 MLA decode (top-k gather of FP8 token records).  Two record forms, chosen by d_qk as the reference does
 * (csrc/api/sparse_decode.h:290-296,318-323):
 *   d_qk 576: 656 bytes per token = 512 e4m3 | 4 fp32 scales (one per 128 values) | 64 bf16 RoPE; V = the first 512 dims.
 *   d_qk 512 ("MODEL1"): a block holds page_block_size x [448 e4m3 | 64 bf16 RoPE] (576 bytes per token) followed by
 *            page_block_size x [7 e8m0 scales (one per 64 values) | 1 pad byte]; the tensor is the
 *            [num_blocks, page_block_size, 1, 584] view of it and V = all 512 dims.  Served by the all-shape kernel.
 * Replaces
 * DecodeImplBase::run as driven by sparse_attn_decode_interface
 * (csrc/api/sparse_decode.h:183-495); arguments mirror SparseAttnDecodeParams
 * (csrc/params.h:63-103).  The caller runs mla_combine (with attn_sink) after it. */
typedef struct {
    int32_t b, s_q, h_q;
    int32_t d_qk, d_v;                /* 576 or 512, 512                                       */
    float sm_scale;

    const void* q;                    /* bf16 [b, s_q, h_q, d_qk]                              */
    int64_t q_stride_b, q_stride_s, q_stride_h;

    const void* kv;                   /* bytes [num_blocks, page_block_size, 1, 656 or 584]    */
    int64_t kv_stride_block_bytes;    /* the layout inside a block is fixed (see above)        */
    int32_t num_blocks, page_block_size;
    const int32_t* indices;           /* [b, s_q, topk], page*page_block_size + offset, -1 = invalid */
    int64_t indices_stride_b, indices_stride_s;
    int32_t topk;
    const int32_t* topk_length;       /* [b] or NULL                                           */

    const void* extra_kv;             /* optional second cache, same record format, or NULL    */
    int64_t extra_kv_stride_block_bytes;
    int32_t extra_num_blocks, extra_page_block_size;
    const int32_t* extra_indices;     /* [b, s_q, extra_topk]                                  */
    int64_t extra_indices_stride_b, extra_indices_stride_s;
    int32_t extra_topk;               /* 0 when extra_kv is NULL                               */
    const int32_t* extra_topk_length; /* [b] or NULL                                           */

    const float* attn_sink;           /* [h_q] or NULL                                         */

    void* out;                        /* bf16 [b, s_q, h_q, d_v]                               */
    int64_t o_stride_b, o_stride_s, o_stride_h;
    float* lse;                       /* fp32 (b, s, h) strided as below                       */
    int64_t lse_stride_b, lse_stride_s, lse_stride_h;

    const mla_sched_meta_t* meta;
    const int32_t* num_splits;
    int32_t num_sm_parts;
    float* lse_accum;                 /* scratch fp32 [b + num_sm_parts, s_q, h_q]             */
    float* o_accum;                   /* scratch fp32 [b + num_sm_parts, s_q, h_q, d_v]        */

    int32_t* status;
    int32_t impl;
    void* stream;
} mla_sparse_decode_args_t;
int mla_sparse_decode_fwd(const mla_sparse_decode_args_t* args);

/* Split-KV combine: merges the per-split partial outputs of every request that
 * was split.  Replaces run_flash_mla_combine_kernel
 * (csrc/smxx/decode/combine/combine.cu:188-213); arguments mirror CombineParams
 * (csrc/params.h:105-125).  Requests with a single split are left untouched
 * (the decode kernel already wrote their final result). */
typedef struct {
    int32_t b, s_q, h_q, d_v;
    float* lse;
    int64_t lse_stride_b, lse_stride_s, lse_stride_h;
    void* out;                        /* bf16 or fp16 (see dtype)                              */
    int64_t o_stride_b, o_stride_s, o_stride_h;
    const float* lse_accum;           /* [splits, s_q, h_q] contiguous                         */
    const float* o_accum;             /* [splits, s_q, h_q, d_v] contiguous                    */
    const int32_t* num_splits;        /* [b + 1]                                               */
    const float* attn_sink;           /* [h_q] or NULL                                         */
    int32_t dtype;                    /* type of out: MLA_DTYPE_BF16 or MLA_DTYPE_FP16         */
    int32_t _pad;
    void* stream;
} mla_combine_args_t;
int mla_combine(const mla_combine_args_t* args);

/* Size of the split-KV scratch of one decode launch, for callers that allocate it themselves: the two decode entry
 * points above take o_accum [b + num_sm_parts, s_q, h_q, d_v] and lse_accum [b + num_sm_parts, s_q, h_q], both fp32,
 * the buffers the reference allocates inside its host glue (csrc/api/dense_decode.h:165-166,
 * csrc/api/sparse_decode.h:315-316).  Returns the bytes of ONE allocation that holds o_accum at offset 0 and lse_accum
 * at *lse_accum_offset_bytes (a multiple of 256, so both meet the kernels' alignment rules when the allocation is
 * 256-byte aligned); returns 0 and sets the error message on bad arguments.  Host-only: touches no device. */
size_t mla_workspace_bytes(int b, int s_q, int h_q, int d_v, int num_sm_parts, size_t* lse_accum_offset_bytes);

/* Token-sparse MLA prefill forward.  Replaces run_fwd_phase1_kernel as driven by
 * sparse_attn_prefill_interface (csrc/api/sparse_fwd.h:101-243); arguments mirror
 * SparseAttnFwdParams (csrc/params.h:145-168). */
typedef struct {
    int32_t s_q, s_kv, h_q, h_kv;     /* h_kv must be 1                                        */
    int32_t d_qk, d_v, topk;          /* d_qk 576 or 512, d_v 512                              */
    float sm_scale;
    const void* q;                    /* bf16 [s_q, h_q, d_qk]                                 */
    int64_t q_stride_s, q_stride_h;
    const void* kv;                   /* bf16 [s_kv, h_kv, d_qk]                               */
    int64_t kv_stride_s, kv_stride_h;
    const int32_t* indices;           /* [s_q, h_kv, topk]; invalid iff < 0 or >= s_kv         */
    int64_t indices_stride_s, indices_stride_h;
    const float* attn_sink;           /* [h_q] or NULL                                         */
    const int32_t* topk_length;       /* [s_q] or NULL                                         */
    void* out;                        /* bf16 [s_q, h_q, d_v] contiguous                       */
    float* max_logits;                /* fp32 [s_q, h_q] contiguous                            */
    float* lse;                       /* fp32 [s_q, h_q] contiguous                            */
    int32_t* status;
    int32_t impl;
    void* stream;
} mla_sparse_prefill_args_t;
int mla_sparse_prefill_fwd(const mla_sparse_prefill_args_t* args);

/* Dense decode INCLUDING the combine step, for callers that cannot allocate device memory (engines whose
 * decode loop runs on a memory plan fixed at start-up, where a cudaMalloc would stall the device or fail;
 * host runtimes that bind this ABI without a device allocator).  Same arguments as mla_dense_decode_fwd, but
 * args->lse_accum and args->o_accum are ignored: the split-KV scratch is a fixed array inside the library,
 * about 64 MiB per GPU that loads it, held until the process exits (enough for batch 128 with 128 heads on a 148-SM part:
 * (128 + 74) * 128 = 25856 rows).  Limit: (b + num_sm_parts) * s_q * h_q
 * must not exceed MLA_NOALLOC_MAX_ROWS, otherwise MLA_ERR_INVALID_ARG is returned.  The first call on each
 * device looks up the array's device address (make that call with the device current and before any stream
 * capture).  All calls on a GPU share the array: calls that may overlap on the GPU race and must be
 * serialised by the caller.  Nothing in the array needs clearing between calls.  Calls no allocation routine.
 * This entry point has no counterpart in the reference. */
#define MLA_NOALLOC_MAX_ROWS 32768
int mla_dense_decode_noalloc(const mla_dense_decode_args_t* args);

/* FP8 KV-cache writer (the step before sparse decode): bf16 token rows -> 656-byte records.  Replaces the torch
 * quantiser the reference ships with its tests (tests/quant.py:20-53, quantize_k_cache, V32 layout; record layout
 * flash_mla/flash_mla_interface.py:92-98): scale = amax/448 per group of 128 values (clamped to 1e-30), or with
 * pow2_scale != 0 the smallest power of two >= max(amax/448, 1e-4); q = e4m3(x / scale).
 * x: [num_blocks, block_size, 576] bf16 (strides in elements); out: [num_blocks, block_size, 656] bytes with a free
 * block stride (>= block_size * 656, multiple of 16).
 * layout 1 writes the 512-wide "MODEL1" form instead (tests/quant.py:55-75): x [num_blocks, block_size, 512]; per block
 * block_size x (448 e4m3 | 64 bf16) followed by block_size x (7 e8m0 scales | 1 zero byte); one power-of-two scale per 64
 * values (pow2_scale is ignored); block stride >= block_size * 584 (the reference pads it to a multiple of 576). */
typedef struct {
    const void* x;
    int64_t x_stride_block, x_stride_row;
    int32_t num_blocks, block_size;
    void* out;
    int64_t out_stride_block_bytes;
    int32_t pow2_scale;
    int32_t layout;                   /* 0: 656-byte records (d 576); 1: MODEL1 (d 512)        */
    void* stream;
} mla_quantize_args_t;
int mla_quantize_fp8_kvcache(const mla_quantize_args_t* args);

/* Self-test of the kernels' bounded barrier wait: launches one small CTA that waits, with the same helper the
 * attention kernels use, on a barrier nobody arrives on, with nothing else in flight.  After `limit_cycles` SM
 * cycles (at most 2e9) every one of its 64 threads gives up, the kernel returns normally and status[0] == code,
 * status[1] == 64 (status: device int32[4], zeroed by the caller); flag_out (device int32[2], optional) receives
 * {1, 0}: the CTA's abort flag, and the result of the wait.  This is how an expired wait looks to a caller of the
 * entry points above, which all take the same `status` words.  The default limit of the attention kernels is 2e9
 * cycles; the environment variable MLA_WAIT_LIMIT_CYCLES, read once, overrides it.
 * No counterpart in the reference (its kernels wait without a limit). */
int mla_selftest_bounded_wait(long long limit_cycles, int code, int32_t* status, int32_t* flag_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* FLASHMLA_B200_H_ */
