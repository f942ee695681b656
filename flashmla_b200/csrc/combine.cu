// Split-KV combine: for every request whose KV range was split over several SM partitions, merge
// the per-split fp32 partial outputs O_s (each already normalised by its own row sum) and base-2
// log-sum-exps lse2_s into the final bf16 output and natural-log LSE:
//     g = log2 sum_s 2^{lse2_s},  out = sum_s 2^{lse2_s - g'} O_s,  lse = g * ln 2
// where g' additionally absorbs the attention sink: g' = g + log2(1 + 2^{sink*log2e - g}).
// Semantics follow csrc/smxx/decode/combine/combine.cu:72-160 of the reference.
//
// HBM-bound: per (request, query token, head) it reads n_splits * 2 KiB and writes 1 KiB.
// One warp per row; every lane keeps 16 output columns in registers (4 x float4 loads per split,
// fully coalesced 512 B per warp instruction), split weights are computed once per 32 splits and
// broadcast by shuffle, so there is no limit on the number of splits.
#include "common.cuh"
#include <cuda_fp16.h>

namespace mla {

constexpr int COMBINE_WARPS = 8;

__global__ void __launch_bounds__(COMBINE_WARPS * 32)
combine_kernel(const mla_combine_args_t a) {
    // launched with programmatic stream serialization: the decode kernel before it may still be running
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bs_idx = blockIdx.x;                       // request * s_q + query token
    const int req = bs_idx / a.s_q, t = bs_idx - req * a.s_q;
    const int head = blockIdx.y * COMBINE_WARPS + warp;
    if (head >= a.h_q) return;
    const int s0 = a.num_splits[req], s1 = a.num_splits[req + 1];
    const int n = s1 - s0;
    if (n <= 1) return;                                  // the decode kernel wrote the final result

    const int64_t row_stride = (int64_t)a.s_q * a.h_q;   // rows per split slot
    const float* lse_acc = a.lse_accum + (int64_t)s0 * row_stride + (int64_t)t * a.h_q + head;
    const float* o_acc = a.o_accum + ((int64_t)s0 * row_stride + (int64_t)t * a.h_q + head) * a.d_v;

    // pass 1: global log-sum-exp over the splits
    float mx = -INFINITY;
    for (int s = lane; s < n; s += 32) mx = fmaxf(mx, lse_acc[(int64_t)s * row_stride]);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (mx == -INFINITY) mx = 0.f;
    float sum = 0.f;
    for (int s = lane; s < n; s += 32) sum += exp2f(lse_acc[(int64_t)s * row_stride] - mx);
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float g = (sum == 0.f || sum != sum) ? INFINITY : log2f(sum) + mx;
    if (lane == 0)
        a.lse[req * a.lse_stride_b + t * a.lse_stride_s + head * a.lse_stride_h] = g * kLn2;
    if (a.attn_sink) {
        const float sink = a.attn_sink[head];
        if (g != INFINITY) g += log2f(1.f + exp2f(sink * kLog2e - g));
        else g = sink == -INFINITY ? INFINITY : sink * kLog2e;
    }

    // pass 2: weighted sum.  d_v = 512 = 32 lanes x 4 float4.
    float4 acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sb = 0; sb < n; sb += 32) {
        const int s_mine = sb + lane;
        const float w_mine = s_mine < n ? exp2f(lse_acc[(int64_t)s_mine * row_stride] - g) : 0.f;
        const int cnt = min(32, n - sb);
        for (int j = 0; j < cnt; ++j) {
            const float w = __shfl_sync(0xffffffffu, w_mine, j);
            const float4* src = reinterpret_cast<const float4*>(o_acc + (int64_t)(sb + j) * row_stride * a.d_v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = src[lane + i * 32];
                acc[i].x += w * v.x; acc[i].y += w * v.y; acc[i].z += w * v.z; acc[i].w += w * v.w;
            }
        }
    }
    // out is bf16 or fp16: both are 2 bytes wide
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + req * a.o_stride_b + t * a.o_stride_s + head * a.o_stride_h;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint2 packed;
        if (a.dtype == MLA_DTYPE_FP16) {
            __half2 lo = __floats2half2_rn(acc[i].x, acc[i].y);
            __half2 hi = __floats2half2_rn(acc[i].z, acc[i].w);
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
        }
        *reinterpret_cast<uint2*>(o + (lane + i * 32) * 4) = packed;
    }
}

int launch_combine(const mla_combine_args_t& a) {
    MLA_CHECK_ARG(a.b > 0 && a.s_q > 0 && a.h_q > 0, "combine: b, s_q, h_q must be positive");
    MLA_CHECK_ARG(a.d_v == 512, "combine: only d_v == 512 is supported (got %d)", a.d_v);
    MLA_CHECK_ARG(a.dtype == MLA_DTYPE_BF16 || a.dtype == MLA_DTYPE_FP16, "combine: dtype must be MLA_DTYPE_BF16 or MLA_DTYPE_FP16 (got %d)", a.dtype);
    MLA_CHECK_ARG(a.lse && a.out && a.lse_accum && a.o_accum && a.num_splits, "combine: null pointer");
    MLA_CHECK_ARG(is_aligned16(a.o_accum), "combine: o_accum must be 16-byte aligned");
    MLA_CHECK_ARG(((uintptr_t)a.out & 7u) == 0 && a.o_stride_b % 4 == 0 && a.o_stride_s % 4 == 0 && a.o_stride_h % 4 == 0,
                  "combine: out must be 8-byte aligned with strides that are multiples of 4 elements");
    dim3 grid(a.b * a.s_q, (a.h_q + COMBINE_WARPS - 1) / COMBINE_WARPS);
    MLA_CHECK_CUDA(launch_dependent(combine_kernel, grid, dim3(COMBINE_WARPS * 32), 0, (cudaStream_t)a.stream, a));
    return MLA_OK;
}

}  // namespace mla
