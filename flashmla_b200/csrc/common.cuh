// Shared host/device helpers of the flashmla_b200 CUDA sources.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/flashmla_b200.h"

namespace mla {

// ---- host-side error plumbing ------------------------------------------------------------
// The message of the last failure on this thread; read through mla_last_error().
char* last_error_buffer();
int set_error(int code, const char* fmt, ...);

#define MLA_CHECK_ARG(cond, ...)                                              \
    do {                                                                      \
        if (!(cond)) return ::mla::set_error(MLA_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

#define MLA_CHECK_CUDA(expr)                                                  \
    do {                                                                      \
        cudaError_t err__ = (expr);                                           \
        if (err__ != cudaSuccess)                                             \
            return ::mla::set_error(MLA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, \
                                    cudaGetErrorString(err__), __FILE__, __LINE__); \
    } while (0)

static inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Cached per-device properties (SM count, opt-in shared memory).
int device_num_sms(int device);
int current_device_num_sms();

// ---- kernel launchers (one per .cu file) -----------------------------------------------------
int launch_sched_meta(const mla_sched_meta_args_t& a);
int launch_combine(const mla_combine_args_t& a);
int launch_dense_decode_portable(const mla_dense_decode_args_t& a);
int launch_sparse_decode_portable(const mla_sparse_decode_args_t& a);
int launch_sparse_prefill_portable(const mla_sparse_prefill_args_t& a);
bool dense_decode_sm100_supports(const mla_dense_decode_args_t& a);
int launch_dense_decode_sm100(const mla_dense_decode_args_t& a);
bool sparse_prefill_sm100_supports(const mla_sparse_prefill_args_t& a);
int launch_sparse_prefill_sm100(const mla_sparse_prefill_args_t& a);
bool sparse_decode_sm100_supports(const mla_sparse_decode_args_t& a);
int launch_sparse_decode_sm100(const mla_sparse_decode_args_t& a);
int launch_quantize_fp8(const mla_quantize_args_t& a);
int launch_bounded_wait_selftest(long long limit_cycles, int code, int* status, int* flag_out, void* stream);

// Launch with programmatic stream serialization: the kernel may begin (prologue only - it must call
// griddepcontrol.wait before it touches memory the previous kernel of the stream writes) while that kernel drains.
// The reference chains its decode and combine kernels the same way (csrc/smxx/decode/combine/combine.cu:198-210).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace mla
