// FP8 KV-cache writer: bf16 token rows [576] -> 656-byte records (512 e4m3 | 4 fp32 scales | 64 bf16 RoPE), the
// format the sparse decode kernels read.  Follows the reference's test quantiser value for value
// (tests/quant.py:20-53 of the reference: scale = amax / 448 per group of 128, optionally rounded up to a power of
// two; q = e4m3(x / scale), round to nearest even).
//
// One warp per token: lane l holds values 16l .. 16l+15 (8 lanes per scale group), so the record's e4m3 part is
// one coalesced 512-byte store.  HBM-bound: 1152 bytes read + 656 bytes written per token.
//
// Layout 1 is the 512-wide "MODEL1" form (tests/quant.py:55-75 of the reference): 448 values in groups of 64 with
// power-of-two scales stored as e8m0 bytes, 64 bf16 RoPE values; a block is block_size x 576 value bytes followed by
// block_size x 8 scale bytes (7 scales + 1 pad).  Lanes 0-27 hold the quantised values (4 lanes per group), lanes 28-31
// the RoPE part.
#include "common.cuh"

#include <cuda_fp8.h>

namespace mla {

__device__ __forceinline__ float pow2_ceil(float s) {
    // smallest power of two >= s (s > 0, normal)
    const uint32_t bits = __float_as_uint(s);
    const uint32_t mant = bits & 0x007fffffu;
    return __uint_as_float((bits & 0x7f800000u) + (mant ? 0x00800000u : 0u));
}

__global__ void __launch_bounds__(256)
quantize_fp8_kernel(const mla_quantize_args_t a) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t ntok = (int64_t)a.num_blocks * a.block_size;
    for (int64_t tok = warp; tok < ntok; tok += nwarps) {
        const int64_t blk = tok / a.block_size, row = tok - blk * a.block_size;
        const __nv_bfloat16* x = (const __nv_bfloat16*)a.x + blk * a.x_stride_block + row * a.x_stride_row;
        uint8_t* out = (uint8_t*)a.out + blk * a.out_stride_block_bytes + row * 656;
        const uint4 v0 = __ldg(reinterpret_cast<const uint4*>(x + lane * 16));
        const uint4 v1 = __ldg(reinterpret_cast<const uint4*>(x + lane * 16 + 8));
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float f[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        float s = __fdiv_rn(amax, 448.f);
        s = a.pow2_scale ? pow2_ceil(fmaxf(s, 1e-4f)) : fmaxf(s, 1e-30f);
        uint32_t q[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b)
                word |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(f[4 * i + b], s), __NV_SATFINITE, __NV_E4M3) << (8 * b);
            q[i] = word;
        }
        *reinterpret_cast<uint4*>(out + lane * 16) = make_uint4(q[0], q[1], q[2], q[3]);
        const float sg = __shfl_sync(0xffffffffu, s, (lane & 3) * 8);          // lanes 0-3: scale of group `lane`
        if (lane < 4) reinterpret_cast<float*>(out + 512)[lane] = sg;
        if (lane < 8) *reinterpret_cast<uint4*>(out + 528 + lane * 16) = __ldg(reinterpret_cast<const uint4*>(x + 512 + lane * 8));
    }
}

__global__ void __launch_bounds__(256)
quantize_fp8_model1_kernel(const mla_quantize_args_t a) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t ntok = (int64_t)a.num_blocks * a.block_size;
    for (int64_t tok = warp; tok < ntok; tok += nwarps) {
        const int64_t blk = tok / a.block_size, row = tok - blk * a.block_size;
        const __nv_bfloat16* x = (const __nv_bfloat16*)a.x + blk * a.x_stride_block + row * a.x_stride_row;
        uint8_t* block = (uint8_t*)a.out + blk * a.out_stride_block_bytes;
        uint8_t* out = block + row * 576;
        const uint4 v0 = __ldg(reinterpret_cast<const uint4*>(x + lane * 16));
        const uint4 v1 = __ldg(reinterpret_cast<const uint4*>(x + lane * 16 + 8));
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float f[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float s = pow2_ceil(fmaxf(__fdiv_rn(amax, 448.f), 1e-4f));
        if (lane < 28) {
            uint32_t q[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t word = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    word |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(f[4 * i + b], s), __NV_SATFINITE, __NV_E4M3) << (8 * b);
                q[i] = word;
            }
            *reinterpret_cast<uint4*>(out + lane * 16) = make_uint4(q[0], q[1], q[2], q[3]);
        } else {
            *reinterpret_cast<uint4*>(out + 448 + (lane - 28) * 32) = v0;
            *reinterpret_cast<uint4*>(out + 448 + (lane - 28) * 32 + 16) = v1;
        }
        // lane g < 7 writes the scale of group g (held by lanes 4g .. 4g+3) as its exponent byte; lane 7 the pad byte
        const float sg = __shfl_sync(0xffffffffu, s, (lane & 7) * 4);
        if (lane < 8) block[(int64_t)a.block_size * 576 + row * 8 + lane] = lane < 7 ? (uint8_t)(__float_as_uint(sg) >> 23) : 0;
    }
}

int launch_quantize_fp8(const mla_quantize_args_t& a) {
    MLA_CHECK_ARG(a.x && a.out, "mla_quantize_fp8_kvcache: x and out must not be null");
    MLA_CHECK_ARG(a.num_blocks > 0 && a.block_size > 0, "mla_quantize_fp8_kvcache: num_blocks and block_size must be positive");
    MLA_CHECK_ARG(a.layout == 0 || a.layout == 1, "mla_quantize_fp8_kvcache: layout must be 0 (656-byte records) or 1 (MODEL1)");
    const int d = a.layout ? 512 : 576, rec = a.layout ? 584 : 656;
    MLA_CHECK_ARG(is_aligned16(a.x) && a.x_stride_block % 8 == 0 && a.x_stride_row % 8 == 0 && a.x_stride_row >= d,
                  "mla_quantize_fp8_kvcache: x must be 16-byte aligned with strides that are multiples of 8 elements");
    MLA_CHECK_ARG(is_aligned16(a.out) && a.out_stride_block_bytes % 16 == 0 && a.out_stride_block_bytes >= (int64_t)a.block_size * rec,
                  "mla_quantize_fp8_kvcache: out must be 16-byte aligned, block stride a multiple of 16 bytes and >= block_size * %d", rec);
    const int64_t ntok = (int64_t)a.num_blocks * a.block_size;
    const int sms = current_device_num_sms();
    int64_t blocks = (ntok + 7) / 8;
    const int64_t cap = (int64_t)(sms > 0 ? sms : 148) * 32;
    if (blocks > cap) blocks = cap;
    if (a.layout) quantize_fp8_model1_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)a.stream>>>(a);
    else quantize_fp8_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)a.stream>>>(a);
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

}  // namespace mla
