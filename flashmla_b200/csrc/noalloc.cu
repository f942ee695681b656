// Dense decode + combine for callers that must not allocate device memory.
//
// Who needs this: serving loops that plan all of their device memory once at start-up and then forbid
// allocation on the decode path (a cudaMalloc synchronises the whole device, can fail under fragmentation,
// and is not allowed while a stream is being captured), and host runtimes that bind this C ABI without
// owning a device allocator at all.  For them the split-KV scratch that mla_dense_decode_fwd expects from
// the caller lives here, in a fixed array inside the library image.
//
// Cost and limits: every GPU that loads the library keeps MLA_NOALLOC_MAX_ROWS * 513 floats (about 64 MiB)
// resident until the process exits.  The array is shared by all calls on a device and keeps the previous
// call's contents; no part of it has to start at zero (each split slot a request uses is written in full
// before the combine step reads it), so nothing is cleared.  Two calls whose kernels can overlap on the
// same GPU (different streams, no dependency between them) race on the array: serialise them.
//
// This entry point has no counterpart in the reference.
#include "common.cuh"

#include <mutex>

namespace mla {

// rows = (b + num_sm_parts) * s_q * h_q; per row 512 fp32 partial outputs + 1 fp32 base-2 LSE
static __device__ __align__(256) float g_noalloc_scratch[(size_t)MLA_NOALLOC_MAX_ROWS * 513];

// In host code the array's name is only a handle: the device address has to be asked for, per device, with
// that device current.  Done on the first call on each device and cached (under a lock: two host threads may
// make their first call at the same time).  The cache is keyed by device ordinal and is not refreshed after a
// cudaDeviceReset.
static float* g_scratch_ptr[64] = {};
static std::mutex g_scratch_mu;

static int scratch_for_current_device(float** out) {
    int dev = 0;
    MLA_CHECK_CUDA(cudaGetDevice(&dev));
    MLA_CHECK_ARG(dev >= 0 && dev < 64, "mla_dense_decode_noalloc: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        MLA_CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_ptr[dev];
    return MLA_OK;
}

}  // namespace mla

extern "C" int mla_dense_decode_noalloc(const mla_dense_decode_args_t* args) {
    using namespace mla;
    MLA_CHECK_ARG(args != nullptr, "mla_dense_decode_noalloc: null argument struct");
    MLA_CHECK_ARG(args->b > 0 && args->s_q > 0 && args->h_q > 0 && args->num_sm_parts > 0,
                  "mla_dense_decode_noalloc: b, s_q, h_q and num_sm_parts must be positive");
    const long long rows = (long long)(args->b + args->num_sm_parts) * args->s_q * args->h_q;
    if (rows > MLA_NOALLOC_MAX_ROWS)
        return set_error(MLA_ERR_INVALID_ARG,
                         "mla_dense_decode_noalloc: (b + num_sm_parts) * s_q * h_q = %lld rows of split scratch exceed the "
                         "built-in maximum of %d; use mla_dense_decode_fwd with caller-provided scratch",
                         rows, MLA_NOALLOC_MAX_ROWS);
    float* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;

    mla_dense_decode_args_t a = *args;
    a.o_accum = scratch;
    a.lse_accum = scratch + (size_t)MLA_NOALLOC_MAX_ROWS * 512;
    rc = mla_dense_decode_fwd(&a);
    if (rc) return rc;

    mla_combine_args_t c = {};
    c.b = a.b; c.s_q = a.s_q; c.h_q = a.h_q; c.d_v = a.d_v;
    c.lse = a.lse; c.lse_stride_b = a.lse_stride_b; c.lse_stride_s = a.lse_stride_s; c.lse_stride_h = a.lse_stride_h;
    c.out = a.out; c.o_stride_b = a.o_stride_b; c.o_stride_s = a.o_stride_s; c.o_stride_h = a.o_stride_h;
    c.lse_accum = a.lse_accum; c.o_accum = a.o_accum; c.num_splits = a.num_splits; c.attn_sink = nullptr;
    c.dtype = a.dtype;
    c.stream = a.stream;
    return mla_combine(&c);
}
