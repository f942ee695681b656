// C entry point around the reference's own tile-scheduler metadata kernel, for the parity tests only.
//
// TEST INFRASTRUCTURE ONLY: built by oracle/build_ref.py into oracle/_ref/libref_sched_meta.so together with the
// reference's UNMODIFIED csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu, compiled where it lies in a
// FlashMLA checkout (no reference source is copied).  Nothing under flashmla_b200/ may load it.
//
// Arguments are the fields of GetDecodeSchedMetaParams (csrc/params.h:127-143) as plain values and device pointers;
// `meta` receives num_sm_parts records of 8 int32 (DecodingSchedMeta, csrc/params.h:10-17), `num_splits` b + 1 int32.
#include <cuda_runtime_api.h>

#include "params.h"
#include "smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.h"

extern "C" int ref_get_decoding_sched_meta(int b, int s_q, int block_size_n, int fixed_overhead_num_blocks, int topk, int extra_topk,
                                           int* topk_length, int* extra_topk_length, int* seqlens_k, void* meta, int* num_splits,
                                           int num_sm_parts, void* stream) {
    GetDecodeSchedMetaParams p = {};
    p.b = b;
    p.s_q = s_q;
    p.block_size_n = block_size_n;
    p.fixed_overhead_num_blocks = fixed_overhead_num_blocks;
    p.topk = topk;
    p.extra_topk = extra_topk;
    p.topk_length = topk_length;
    p.extra_topk_length = extra_topk_length;
    p.seqlens_k_ptr = seqlens_k;
    p.tile_scheduler_metadata_ptr = reinterpret_cast<DecodingSchedMeta*>(meta);
    p.num_splits_ptr = num_splits;
    p.num_sm_parts = num_sm_parts;
    p.stream = reinterpret_cast<cudaStream_t>(stream);
    smxx::decode::run_get_decoding_sched_meta_kernel(p);
    return (int)cudaGetLastError();
}

// ---- the reference's own split-KV combine kernel (csrc/smxx/decode/combine/combine.cu, unmodified) ----------------------
// Arguments are the fields of CombineParams (csrc/params.h:105-125): lse is [b, s_q, h_q] fp32 (head stride 1), out is
// [b, s_q, h_q, 512] bf16, lse_accum [splits, s_q, h_q] and o_accum [splits, s_q, h_q, 512] fp32 contiguous.
#include "smxx/decode/combine/combine.h"
#include <cutlass/numeric_types.h>

extern "C" int ref_combine_bf16(int b, int s_q, int h_q, int d_v, float* lse, void* out, float* lse_accum, float* o_accum,
                                void* meta, int* num_splits, int num_sm_parts, float* attn_sink, void* stream) {
    CombineParams p = {};
    p.b = b; p.s_q = s_q; p.h_q = h_q; p.d_v = d_v;
    p.lse = lse; p.out = out;
    p.stride_lse_b = s_q * h_q; p.stride_lse_s_q = h_q;
    p.stride_o_b = s_q * h_q * d_v; p.stride_o_s_q = h_q * d_v; p.stride_o_h_q = d_v;
    p.lse_accum = lse_accum; p.o_accum = o_accum;
    p.stride_lse_accum_split = s_q * h_q; p.stride_lse_accum_s_q = h_q;
    p.stride_o_accum_split = s_q * h_q * d_v; p.stride_o_accum_s_q = h_q * d_v; p.stride_o_accum_h_q = d_v;
    p.tile_scheduler_metadata_ptr = reinterpret_cast<DecodingSchedMeta*>(meta);
    p.num_splits_ptr = num_splits;
    p.num_sm_parts = num_sm_parts;
    p.attn_sink = attn_sink;
    p.stream = reinterpret_cast<cudaStream_t>(stream);
    smxx::decode::run_flash_mla_combine_kernel<cutlass::bfloat16_t>(p);
    return (int)cudaGetLastError();
}
