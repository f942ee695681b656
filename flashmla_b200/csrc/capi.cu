// extern "C" entry points of libflashmla_b200: argument validation and kernel selection.
// Declarations and the reference interfaces they replace: include/flashmla_b200.h.
#include "common.cuh"

#include <mutex>
#include <string.h>

namespace mla {

char* last_error_buffer() {
    static thread_local char buf[1024] = {0};
    return buf;
}

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 1024, fmt, ap);
    va_end(ap);
    return code;
}

int device_num_sms(int device) {
    static int cache[64];
    static std::mutex mu;
    if (device < 0 || device >= 64) return -1;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
        cache[device] = n;
    }
    return cache[device];
}

int current_device_num_sms() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    return device_num_sms(dev);
}

// allow_512: the sparse FP8 path also takes the 512-wide ("MODEL1") query / record form
static int check_decode_common(const char* who, bool allow_512, int b, int s_q, int h_q, int d_qk, int d_v, const void* q,
                               int64_t q_sb, int64_t q_ss, int64_t q_sh, const void* out, int64_t o_sb,
                               int64_t o_ss, int64_t o_sh, const void* lse, const void* meta,
                               const void* num_splits, int num_sm_parts, const void* lse_accum, const void* o_accum) {
    MLA_CHECK_ARG(b > 0 && s_q > 0 && h_q > 0, "%s: b, s_q and h_q must be positive (got %d, %d, %d)", who, b, s_q, h_q);
    MLA_CHECK_ARG(d_qk == 576 || (allow_512 && d_qk == 512), "%s: only head_dim %s supported (got %d)", who,
                  allow_512 ? "576 or 512 is" : "576 is", d_qk);
    MLA_CHECK_ARG(d_v == 512, "%s: only head_dim_v 512 is supported (got %d)", who, d_v);
    MLA_CHECK_ARG(q && out && lse, "%s: q, out and lse must not be null", who);
    MLA_CHECK_ARG(meta && num_splits && num_sm_parts > 0, "%s: tile-scheduler metadata is required", who);
    MLA_CHECK_ARG(lse_accum && o_accum, "%s: split-KV scratch buffers are required", who);
    MLA_CHECK_ARG(is_aligned16(q) && q_sb % 8 == 0 && q_ss % 8 == 0 && q_sh % 8 == 0,
                  "%s: q must be 16-byte aligned with strides that are multiples of 8 elements", who);
    MLA_CHECK_ARG(is_aligned16(out) && o_sb % 8 == 0 && o_ss % 8 == 0 && o_sh % 8 == 0,
                  "%s: out must be 16-byte aligned with strides that are multiples of 8 elements", who);
    MLA_CHECK_ARG(is_aligned16(o_accum), "%s: o_accum must be 16-byte aligned", who);
    return MLA_OK;
}

}  // namespace mla

using namespace mla;

extern "C" {

const char* mla_last_error(void) { return last_error_buffer(); }

int mla_abi_version(void) { return 2; }

int mla_num_sm_parts(int device, int mode, int h_q, int h_kv, int s_q) {
    const int sms = device_num_sms(device);
    if (sms <= 0) { set_error(MLA_ERR_CUDA, "mla_num_sm_parts: cannot query device %d", device); return -1; }
    if (h_q <= 0 || h_kv <= 0 || s_q <= 0 || h_q % h_kv != 0) {
        set_error(MLA_ERR_INVALID_ARG, "mla_num_sm_parts: bad head counts / s_q");
        return -1;
    }
    if (mode == MLA_MODE_DENSE_DECODE) {
        // A partition is walked, for every block of 128 query rows of every kv head, by a pair of CTAs on two
        // SMs (the tcgen05 kernel's score / value CTAs, or two 64-row CTAs of the portable kernel).
        const int rows = s_q * (h_q / h_kv);
        const int row_blocks = (rows + 127) / 128;
        int p = sms / 2 / h_kv / row_blocks;
        return p > 0 ? p : 1;
    } else if (mode == MLA_MODE_SPARSE_DECODE) {
        // up to 128 heads: one CTA pair of the tcgen05 kernel per partition and query token; more heads run on the
        // portable kernel, one CTA per 64 heads
        int p = h_q <= 128 ? sms / 2 / s_q : sms / s_q / ((h_q + 63) / 64);
        return p > 0 ? p : 1;
    }
    set_error(MLA_ERR_INVALID_ARG, "mla_num_sm_parts: unknown mode %d", mode);
    return -1;
}

int mla_num_sm_parts_uniform(int device, int mode, int h_q, int h_kv, int s_q, int b, int blocks_per_request) {
    const int p = mla_num_sm_parts(device, mode, h_q, h_kv, s_q);
    if (p <= 0) return p;
    if (b <= 0 || blocks_per_request <= 0) {
        set_error(MLA_ERR_INVALID_ARG, "mla_num_sm_parts_uniform: batch size and blocks per request must be positive");
        return -1;
    }
    if (b > p) return p;
    // Every request costs the same, so with exactly b partitions the greedy scheduler cuts at every request boundary
    // (budget = blocks + 2 * overhead per partition, a request costs blocks + overhead: one fits, two do not): no
    // partition walks two requests (one Q load and one epilogue each instead of two), no request is split and nothing
    // is left to combine.  That leaves p - b CTA pairs idle; take it when the extra blocks per partition cost less
    // than the boundary they save (about 8 blocks of 64 tokens, measured).  (For a multiple k > 1 of b the cuts
    // drift off the request boundaries - the scheduler's budget rounds up - so only k = 1 is offered.)
    const double blocks_greedy = (double)blocks_per_request * b / p;
    return ((double)blocks_per_request - blocks_greedy) < 8.0 ? b : p;
}

int mla_get_sched_meta(const mla_sched_meta_args_t* a) {
    MLA_CHECK_ARG(a != nullptr, "mla_get_sched_meta: null argument struct");
    return launch_sched_meta(*a);
}

int mla_combine(const mla_combine_args_t* a) {
    MLA_CHECK_ARG(a != nullptr, "mla_combine: null argument struct");
    return launch_combine(*a);
}

int mla_dense_decode_fwd(const mla_dense_decode_args_t* a) {
    MLA_CHECK_ARG(a != nullptr, "mla_dense_decode_fwd: null argument struct");
    int rc = check_decode_common("mla_dense_decode_fwd", false, a->b, a->s_q, a->h_q, a->d_qk, a->d_v, a->q, a->q_stride_b,
                                 a->q_stride_s, a->q_stride_h, a->out, a->o_stride_b, a->o_stride_s, a->o_stride_h,
                                 a->lse, a->meta, a->num_splits, a->num_sm_parts, a->lse_accum, a->o_accum);
    if (rc) return rc;
    MLA_CHECK_ARG(a->h_kv > 0 && a->h_q % a->h_kv == 0, "mla_dense_decode_fwd: h_kv (%d) must divide h_q (%d)", a->h_kv, a->h_q);
    MLA_CHECK_ARG(a->page_block_size == 64, "mla_dense_decode_fwd: page_block_size must be 64 (got %d)", a->page_block_size);
    MLA_CHECK_ARG(a->dtype == MLA_DTYPE_BF16 || a->dtype == MLA_DTYPE_FP16, "mla_dense_decode_fwd: dtype must be MLA_DTYPE_BF16 or MLA_DTYPE_FP16 (got %d)", a->dtype);
    MLA_CHECK_ARG(a->max_blocks_per_seq > 0, "mla_dense_decode_fwd: max_blocks_per_seq must be positive (got %d)", a->max_blocks_per_seq);
    MLA_CHECK_ARG(a->k_cache && a->block_table && a->seqlens_k, "mla_dense_decode_fwd: k_cache, block_table and seqlens_k must not be null");
    MLA_CHECK_ARG(a->num_blocks > 0, "mla_dense_decode_fwd: num_blocks must be positive");
    MLA_CHECK_ARG(is_aligned16(a->k_cache) && a->k_stride_block % 8 == 0 && a->k_stride_row % 8 == 0 && a->k_stride_head % 8 == 0,
                  "mla_dense_decode_fwd: k_cache must be 16-byte aligned with strides that are multiples of 8 elements");
    if (a->impl == 2) {
        if (!dense_decode_sm100_supports(*a))
            return set_error(MLA_ERR_UNSUPPORTED, "mla_dense_decode_fwd: the tcgen05 kernel does not support this shape");
        return launch_dense_decode_sm100(*a);
    }
    if (a->impl == 0 && dense_decode_sm100_supports(*a)) return launch_dense_decode_sm100(*a);
    if (a->dtype != MLA_DTYPE_BF16)
        return set_error(MLA_ERR_UNSUPPORTED, "mla_dense_decode_fwd: fp16 is served by the tcgen05 kernel only, which does not support this shape");
    return launch_dense_decode_portable(*a);
}

int mla_sparse_decode_fwd(const mla_sparse_decode_args_t* a) {
    MLA_CHECK_ARG(a != nullptr, "mla_sparse_decode_fwd: null argument struct");
    int rc = check_decode_common("mla_sparse_decode_fwd", true, a->b, a->s_q, a->h_q, a->d_qk, a->d_v, a->q, a->q_stride_b,
                                 a->q_stride_s, a->q_stride_h, a->out, a->o_stride_b, a->o_stride_s, a->o_stride_h,
                                 a->lse, a->meta, a->num_splits, a->num_sm_parts, a->lse_accum, a->o_accum);
    if (rc) return rc;
    MLA_CHECK_ARG(a->kv && a->indices && a->topk > 0, "mla_sparse_decode_fwd: kv, indices and topk are required");
    MLA_CHECK_ARG(a->page_block_size > 0 && a->num_blocks > 0, "mla_sparse_decode_fwd: bad page_block_size / num_blocks");
    MLA_CHECK_ARG(is_aligned16(a->kv) && a->kv_stride_block_bytes % 16 == 0,
                  "mla_sparse_decode_fwd: kv must be 16-byte aligned and its block stride a multiple of 16 bytes");
    // 576: 656-byte records; 512: 576 value bytes per token, then 8 scale bytes per token behind the block's tokens
    const int64_t rec_bytes = a->d_qk == 512 ? 584 : 656;
    MLA_CHECK_ARG(a->kv_stride_block_bytes >= (int64_t)a->page_block_size * rec_bytes,
                  "mla_sparse_decode_fwd: a kv block must hold page_block_size records of %d bytes", (int)rec_bytes);
    if (a->extra_kv) {
        MLA_CHECK_ARG(a->extra_indices && a->extra_topk > 0, "mla_sparse_decode_fwd: extra_indices must be provided with extra_kv");
        MLA_CHECK_ARG(a->extra_page_block_size > 0 && a->extra_num_blocks > 0, "mla_sparse_decode_fwd: bad extra page_block_size / num_blocks");
        MLA_CHECK_ARG(is_aligned16(a->extra_kv) && a->extra_kv_stride_block_bytes % 16 == 0,
                      "mla_sparse_decode_fwd: extra_kv must be 16-byte aligned and its block stride a multiple of 16 bytes");
        MLA_CHECK_ARG(a->extra_kv_stride_block_bytes >= (int64_t)a->extra_page_block_size * rec_bytes,
                      "mla_sparse_decode_fwd: an extra kv block must hold extra_page_block_size records of %d bytes", (int)rec_bytes);
    } else {
        MLA_CHECK_ARG(!a->extra_indices && !a->extra_topk_length, "mla_sparse_decode_fwd: extra_indices / extra_topk_length need extra_kv");
    }
    if (a->impl == 2) {
        if (!sparse_decode_sm100_supports(*a))
            return set_error(MLA_ERR_UNSUPPORTED, "mla_sparse_decode_fwd: the tcgen05 kernel does not support this shape");
        return launch_sparse_decode_sm100(*a);
    }
    // (also with few heads: the work is dominated by gathering and de-quantising the records, which the tcgen05
    // kernel does 2x faster than the portable one even when most of its 128 rows are padding)
    if (a->impl == 0 && sparse_decode_sm100_supports(*a)) return launch_sparse_decode_sm100(*a);
    return launch_sparse_decode_portable(*a);
}

int mla_sparse_prefill_fwd(const mla_sparse_prefill_args_t* a) {
    MLA_CHECK_ARG(a != nullptr, "mla_sparse_prefill_fwd: null argument struct");
    MLA_CHECK_ARG(a->s_q > 0 && a->s_kv > 0 && a->h_q > 0 && a->topk > 0, "mla_sparse_prefill_fwd: s_q, s_kv, h_q, topk must be positive");
    MLA_CHECK_ARG(a->h_kv == 1, "mla_sparse_prefill_fwd: h_kv must be 1 (got %d)", a->h_kv);
    MLA_CHECK_ARG((a->d_qk == 576 || a->d_qk == 512) && a->d_v == 512, "mla_sparse_prefill_fwd: only d_qk 576 or 512 with d_v 512 is supported");
    MLA_CHECK_ARG(a->q && a->kv && a->indices && a->out && a->max_logits && a->lse, "mla_sparse_prefill_fwd: null pointer");
    MLA_CHECK_ARG(is_aligned16(a->q) && a->q_stride_s % 8 == 0 && a->q_stride_h % 8 == 0,
                  "mla_sparse_prefill_fwd: q must be 16-byte aligned with strides that are multiples of 8 elements");
    MLA_CHECK_ARG(is_aligned16(a->kv) && a->kv_stride_s % 8 == 0,
                  "mla_sparse_prefill_fwd: kv must be 16-byte aligned with a row stride that is a multiple of 8 elements");
    MLA_CHECK_ARG(is_aligned16(a->out), "mla_sparse_prefill_fwd: out must be 16-byte aligned");
    if (a->impl == 2) {
        if (!sparse_prefill_sm100_supports(*a))
            return set_error(MLA_ERR_UNSUPPORTED, "mla_sparse_prefill_fwd: the tcgen05 kernel does not support this shape");
        return launch_sparse_prefill_sm100(*a);
    }
    if (a->impl == 0 && sparse_prefill_sm100_supports(*a)) return launch_sparse_prefill_sm100(*a);
    return launch_sparse_prefill_portable(*a);
}

size_t mla_workspace_bytes(int b, int s_q, int h_q, int d_v, int num_sm_parts, size_t* lse_accum_offset_bytes) {
    if (b <= 0 || s_q <= 0 || h_q <= 0 || d_v <= 0 || num_sm_parts <= 0) {
        set_error(MLA_ERR_INVALID_ARG, "mla_workspace_bytes: b, s_q, h_q, d_v and num_sm_parts must be positive");
        return 0;
    }
    const size_t rows = (size_t)(b + num_sm_parts) * (size_t)s_q * (size_t)h_q;
    const size_t o_bytes = (rows * (size_t)d_v * sizeof(float) + 255) / 256 * 256;
    if (lse_accum_offset_bytes) *lse_accum_offset_bytes = o_bytes;
    return o_bytes + rows * sizeof(float);
}

int mla_selftest_bounded_wait(long long limit_cycles, int code, int32_t* status, int32_t* flag_out, void* stream) {
    return launch_bounded_wait_selftest(limit_cycles, code, status, flag_out, stream);
}

int mla_quantize_fp8_kvcache(const mla_quantize_args_t* a) {
    MLA_CHECK_ARG(a != nullptr, "mla_quantize_fp8_kvcache: null argument struct");
    return launch_quantize_fp8(*a);
}

}  // extern "C"
