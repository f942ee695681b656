// Tile-scheduler metadata kernel: splits the 64-token KV blocks of a decode batch over the SM
// partitions of the decode kernels and records, per request, how many partial results (splits)
// the combine kernel has to merge.
//
// The greedy rule and every output value follow the reference kernel
// csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu:28-106 bit for bit for equal
// (num_sm_parts, block_size_n, fixed_overhead): each partition gets a budget of
// ceil(total/num_sm_parts) + fixed_overhead blocks, where every request costs its blocks plus
// fixed_overhead; whole requests are taken while they fit, otherwise the remaining budget minus the
// overhead is taken from the next request and the partition ends.
//
// Layout: one CTA; the per-request lengths are staged in shared memory by all threads, then one
// thread runs the O(b + num_sm_parts) serial walk over precomputed block counts (no division in the loop; the result is cached by the
// caller for the whole decode step).
#include "common.cuh"

namespace mla {

__global__ void __launch_bounds__(128, 1)
sched_meta_kernel(const mla_sched_meta_args_t a) {
    // the decode kernel that follows is launched with programmatic stream serialization: let its prologue (barrier and
    // tensor-memory set-up) start now; it waits for this kernel's completion before it reads the metadata
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ int smem_i[];
    int* nblk_s = smem_i;                // [b]  KV blocks of every request; -1 marks a zero-length request (1 block)
    int* nsplit_s = smem_i + a.b;        // [b + 1]
    __shared__ int total_s;
    const int b = a.b, bs = a.block_size_n, F = a.fixed_overhead_num_blocks;
    if (threadIdx.x == 0) total_s = 0;
    __syncthreads();

    int local_total = 0;
    for (int i = threadIdx.x; i < b; i += blockDim.x) {
        int s;
        if (a.topk == -1) {
            s = a.seqlens_k[i];
        } else {
            s = a.topk_length ? a.topk_length[i] : a.topk;
            if (s == 0) s = 1;
            if (a.extra_topk) {
                s = (s + bs - 1) / bs * bs;
                s += a.extra_topk_length ? a.extra_topk_length[i] : a.extra_topk;
            }
        }
        const int nblk = max(s - 1, 0) / bs + 1;       // a zero-length request still costs one block
        nblk_s[i] = s == 0 ? -1 : nblk;
        local_total += nblk + F;
    }
    atomicAdd(&total_s, local_total);
    __syncthreads();

    if (threadIdx.x == 0) {
        const int P = a.num_sm_parts;
        const int payload = (total_s + P - 1) / P + F;
        int now_req = 0, now_block = 0, now_split = 0, cum = 0;
        nsplit_s[0] = 0;
        const int last_block_req0 = abs(nblk_s[0]) - 1;
        for (int p = 0; p < P; ++p) {
            mla_sched_meta_t m;
            m.begin_req_idx = now_req;
            // A partition that starts after the last request reports the last block index of request 0
            // here: the reference reads one element past its first-block array, which is the first
            // element of its last-block array.  Consumers skip such partitions (begin_req_idx >= b).
            m.begin_block_idx = now_req < b ? now_block : last_block_req0;
            m.begin_split_idx = now_split;
            m.is_first_req_splitted = now_block != 0;
            int remain = payload;
            while (now_req < b) {
                const int rest = abs(nblk_s[now_req]) - now_block;
                if (remain >= rest + F) {
                    cum += now_split + 1;
                    nsplit_s[now_req + 1] = cum;
                    remain -= rest + F;
                    ++now_req;
                    now_block = 0;
                    now_split = 0;
                } else {
                    if (remain - F > 0) {
                        now_block += remain - F;
                        ++now_split;
                        remain = 0;
                    }
                    break;
                }
            }
            if (now_block > 0) {
                m.end_req_idx = now_req;
                m.end_block_idx = now_block;
            } else {
                m.end_req_idx = now_req - 1;
                m.end_block_idx = max(nblk_s[now_req - 1], 0);
            }
            const int n_end = nblk_s[m.end_req_idx];
            m.is_last_req_splitted = n_end > 0 && m.end_block_idx != n_end;
            if (m.begin_req_idx == m.end_req_idx) {
                m.is_first_req_splitted = m.is_last_req_splitted = (m.is_first_req_splitted || m.is_last_req_splitted);
            }
            m._pad = 0;
            a.meta[p] = m;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= b; i += blockDim.x) a.num_splits[i] = nsplit_s[i];
}

int launch_sched_meta(const mla_sched_meta_args_t& a) {
    MLA_CHECK_ARG(a.b > 0, "sched_meta: batch size must be positive (got %d)", a.b);
    MLA_CHECK_ARG(a.num_sm_parts > 0, "sched_meta: num_sm_parts must be positive (got %d)", a.num_sm_parts);
    MLA_CHECK_ARG(a.block_size_n > 0 && a.fixed_overhead_num_blocks >= 0, "sched_meta: bad block size / overhead");
    MLA_CHECK_ARG(a.meta && a.num_splits, "sched_meta: output pointers must not be null");
    MLA_CHECK_ARG(a.topk != -1 || a.seqlens_k, "sched_meta: seqlens_k is required for dense attention");
    const size_t smem = sizeof(int) * (2 * (size_t)a.b + 1);
    MLA_CHECK_ARG(smem <= 200 * 1024, "sched_meta: batch size %d too large (max 25000)", a.b);
    if (smem > 48 * 1024)
        MLA_CHECK_CUDA(cudaFuncSetAttribute(sched_meta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    sched_meta_kernel<<<1, 128, smem, (cudaStream_t)a.stream>>>(a);
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

}  // namespace mla
