// Portable MLA attention kernel (legacy mma.sync tensor path).
//
// One kernel template serves the three KV sources of the library:
//   DENSE          paged bf16 cache walked through the block table          (dense decode)
//   SPARSE_FP8     top-k gather of FP8 token records, de-quantised            (sparse decode)
//   SPARSE_BF16    top-k gather of bf16 rows from a flat [s_kv, d] tensor   (sparse prefill)
// The two sparse modes exist for both query/key widths of the reference: 576 (656-byte records with four fp32 scales)
// and 512 (the "MODEL1" form: 448 e4m3 + 64 bf16 RoPE per token, seven e8m0 scales per token stored behind the block's
// tokens; the RoPE part belongs to V as well).
// It accepts every head count, h_kv, s_q, page size and index pattern the host API admits and is
// the kernel used for shapes the tcgen05 kernels do not cover.  It is a correct, reasonably tiled
// flash-decoding kernel, not the speed-of-light path.
//
// Tiling: a CTA (8 warps) owns 64 query rows (rows = (query token, head) pairs that share one KV
// stream) and walks its KV range in sub-tiles of 32 tokens, double-buffered in shared memory:
//   phase 1  S = Q K^T        (64 x 32, k = 576)  warp (m-tile 0..3, token half 0..1)
//   phase 2  online softmax   4 threads per row, base-2 exponent with the scale folded in
//   phase 3  O += P V         every warp owns 64 of the 512 value columns for all 64 rows
// O lives in registers (128 fp32 per thread), Q / K / P in padded shared memory read by ldmatrix.
//
// Semantics (masking, empty rows, split vs. direct epilogue, attention sink) follow the reference
// kernels: csrc/sm90/decode/dense/splitkv_mla.cuh:959-1272, csrc/sm100/decode/head64/kernel.cuh:19-849,
// csrc/sm100/prefill/sparse/fwd/head128/phase1.cuh:65-614.
#include "common.cuh"

namespace mla {
namespace portable {

constexpr int BM = 64;            // query rows per CTA
constexpr int BN = 32;            // tokens per sub-tile
constexpr int BLK = 64;           // tokens per scheduling block (two sub-tiles)
constexpr int D_V = 512;
constexpr int LDK = 584;          // padded row length (elements) of Q / K tiles (either width): 1168 B = 4 words mod 32 banks
constexpr int LDP = 40;           // padded row length of the P tile
constexpr int LDS = 36;           // padded row length (floats) of the S tile
constexpr int NTHREADS = 256;
constexpr int FP8_ROW_BYTES = 656;
constexpr int M1_ROW_BYTES = 576;      // d_qk 512: 448 e4m3 + 64 bf16 per token; 8 scale bytes per token follow the block's tokens

enum Mode { DENSE = 0, SPARSE_FP8 = 1, SPARSE_BF16 = 2 };

struct Params {
    int b, s_q, h_q, h_kv, g;     // g = h_q / h_kv
    int rows;                     // valid rows of one row group: dense s_q*g, sparse h_q
    float scale_log2;
    const __nv_bfloat16* q; int64_t q_sb, q_ss, q_sh;
    __nv_bfloat16* out; int64_t o_sb, o_ss, o_sh;
    float* lse; int64_t l_sb, l_ss, l_sh;
    float* max_logits;
    const float* attn_sink;
    // dense
    const __nv_bfloat16* kc; int64_t k_sblock, k_srow, k_shead;
    const int* block_table; int64_t bt_sb; const int* seqlens; int causal;
    int max_blocks;               // width of the block table: blocks at or beyond it read no table entry and count as invalid
    // sparse fp8 (two scopes: main, extra)
    const uint8_t* kvb[2]; int64_t kvb_sblock[2]; int pbs[2]; int nblocks[2];
    const int* idx[2]; int64_t idx_sb[2], idx_ss[2]; int topk[2]; const int* topk_len[2];
    // sparse bf16 (prefill)
    const __nv_bfloat16* kvf; int64_t kvf_ss; int s_kv;
    // split-KV
    const mla_sched_meta_t* meta; const int* num_splits;
    float* lse_accum; float* o_accum;
};

struct Smem {
    __nv_bfloat16 q[BM * LDK];
    __nv_bfloat16 k[2][BN * LDK];
    float s[BM * LDS];
    __nv_bfloat16 p[BM * LDP];
    float m[BM], l[BM], f[BM];
    int valid[2][BN];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 e4m3 values (one uint4) times an fp32 scale -> 16 bf16 (two uint4), rounding once.
__device__ __forceinline__ void dequant16(const uint4& raw, float scale, uint4& lo, uint4& hi) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2_raw h0 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xffffu), __NV_E4M3);
        __half2_raw h1 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
        float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&h0));
        float2 f1 = __half22float2(*reinterpret_cast<__half2*>(&h1));
        __nv_bfloat162 b0 = __floats2bfloat162_rn(f0.x * scale, f0.y * scale);
        __nv_bfloat162 b1 = __floats2bfloat162_rn(f1.x * scale, f1.y * scale);
        o[2 * i] = *reinterpret_cast<uint32_t*>(&b0);
        o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b1);
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// Description of the KV stream one CTA walks for one request.
struct Stream {
    int req;            // request (decode) or query token (prefill)
    int t_fixed;        // query token for the sparse modes
    int hk;             // kv head (dense)
    int seqlen;         // dense: tokens of the request
    int len[2];         // sparse: number of positions that may be valid in scope 0 / 1
    int nblk0;          // sparse decode: blocks that belong to scope 0
    const int* idxp[2]; // sparse: index row of this (request, query token) in scope 0 / 1
};

// Loads sub-tile `st` (tokens [st*32, st*32+32) of the stream) into buffer `buf`.
// e8m0 scale byte -> fp32: 2^(e - 127); 0 is the subnormal 2^-127, 255 is NaN (as the format defines it)
__device__ __forceinline__ float e8m0_to_float(uint32_t e) {
    return __uint_as_float(e == 0 ? 0x00400000u : e == 255 ? 0x7fc00000u : e << 23);
}

template <int MODE, int DQK>
__device__ __forceinline__ void load_subtile(const Params& p, Smem& sm, const Stream& s, int st, int buf) {
    const int tid = threadIdx.x;
    __nv_bfloat16* dst = sm.k[buf];
    if (MODE == DENSE) {
        const int blk = st >> 1;
        const int page = blk < p.max_blocks ? p.block_table[(int64_t)s.req * p.bt_sb + blk] : -1;
        const bool page_ok = page >= 0 && page < p.nblocks[0];
        const __nv_bfloat16* base = p.kc + (int64_t)page * p.k_sblock + (int64_t)s.hk * p.k_shead;
        constexpr int NCH = DQK / 8;
        for (int c = tid; c < BN * NCH; c += NTHREADS) {
            const int tok = c / NCH, ch = c - tok * NCH;
            const int pos = st * BN + tok;
            const bool ok = page_ok && pos < s.seqlen;
            if (ch == 0) sm.valid[buf][tok] = ok;
            __nv_bfloat16* d = dst + tok * LDK + ch * 8;
            if (ok) cp_async16(d, base + (int64_t)(pos & (BLK - 1)) * p.k_srow + ch * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);      // unused cache may hold NaN
        }
    } else if (MODE == SPARSE_BF16) {
        constexpr int NCH = DQK / 8;
        for (int c = tid; c < BN * NCH; c += NTHREADS) {
            const int tok = c / NCH, ch = c - tok * NCH;
            const int pos = st * BN + tok;
            int id = -1;
            if (pos < s.len[0]) id = s.idxp[0][pos];
            const bool ok = id >= 0 && id < p.s_kv;
            if (ch == 0) sm.valid[buf][tok] = ok;
            __nv_bfloat16* d = dst + tok * LDK + ch * 8;
            if (ok) cp_async16(d, p.kvf + (int64_t)id * p.kvf_ss + ch * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
    } else {
        // FP8 records: NQ chunks of 16 e4m3 (-> 32 B of bf16) + 8 chunks of 16 B RoPE per token.
        constexpr bool M1 = DQK == 512;
        constexpr int NQ = M1 ? 28 : 32, NCH = NQ + 8, D_NOPE = NQ * 16;
        const int blk = st >> 1;
        const int scope = blk >= s.nblk0 ? 1 : 0;
        const int pos0 = (scope ? (blk - s.nblk0) : blk) * BLK + (st & 1) * BN;
        const int* idxp = s.idxp[scope];
        const uint8_t* kvb = p.kvb[scope];
        const int pbs = p.pbs[scope];
        const int64_t limit = (int64_t)p.nblocks[scope] * pbs;
        for (int c = tid; c < BN * NCH; c += NTHREADS) {
            const int tok = c / NCH, ch = c - tok * NCH;
            const int pos = pos0 + tok;
            int id = -1;
            if (pos < s.len[scope]) id = idxp[pos];
            const bool ok = id >= 0 && id < limit;
            if (ch == 0) sm.valid[buf][tok] = ok;
            __nv_bfloat16* drow = dst + tok * LDK;
            if (!ok) {
                if (ch < NQ) {
                    *reinterpret_cast<uint4*>(drow + ch * 16) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(drow + ch * 16 + 8) = make_uint4(0, 0, 0, 0);
                } else {
                    *reinterpret_cast<uint4*>(drow + D_NOPE + (ch - NQ) * 8) = make_uint4(0, 0, 0, 0);
                }
                continue;
            }
            const uint8_t* blk_base = kvb + (int64_t)(id / pbs) * p.kvb_sblock[scope];
            const int off = id % pbs;
            const uint8_t* rec = blk_base + (int64_t)off * (M1 ? M1_ROW_BYTES : FP8_ROW_BYTES);
            if (ch < NQ) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(rec + ch * 16));
                // 576: one fp32 scale per 128 values inside the record; 512: one e8m0 scale per 64 values behind the block's tokens
                const float scale = M1 ? e8m0_to_float(__ldg(blk_base + (int64_t)pbs * M1_ROW_BYTES + off * 8 + (ch >> 2)))
                                       : __ldg(reinterpret_cast<const float*>(rec + 512) + (ch >> 3));
                uint4 lo, hi;
                dequant16(raw, scale, lo, hi);
                *reinterpret_cast<uint4*>(drow + ch * 16) = lo;
                *reinterpret_cast<uint4*>(drow + ch * 16 + 8) = hi;
            } else {
                *reinterpret_cast<uint4*>(drow + D_NOPE + (ch - NQ) * 8) =
                    __ldg(reinterpret_cast<const uint4*>(rec + (M1 ? D_NOPE : 528) + (ch - NQ) * 16));
            }
        }
    }
}

template <int MODE, int DQK>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_portable_kernel(const Params p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_blk = MODE == SPARSE_BF16 ? blockIdx.y : blockIdx.x;

    // ---- which requests / block ranges does this CTA walk --------------------------------------
    int req_begin, req_end, sched_begin_block = 0, sched_end_block = 0, begin_split = 0;
    bool first_split = false, last_split = false;
    if (MODE == SPARSE_BF16) {
        req_begin = req_end = blockIdx.x;                   // one query token per CTA column
    } else {
        const mla_sched_meta_t m = p.meta[blockIdx.z];
        if (m.begin_req_idx >= p.b) return;
        req_begin = m.begin_req_idx; req_end = m.end_req_idx;
        sched_begin_block = m.begin_block_idx; sched_end_block = m.end_block_idx;
        begin_split = m.begin_split_idx;
        first_split = m.is_first_req_splitted; last_split = m.is_last_req_splitted;
    }

    const int mt = warp & 3, nh = warp >> 2;      // phase 1 role
    const int gid = lane >> 2, tig = lane & 3;

    for (int req = req_begin; req <= req_end; ++req) {
        Stream s;
        s.req = req; s.t_fixed = 0; s.hk = 0; s.seqlen = 0; s.len[0] = s.len[1] = 0; s.nblk0 = 0;
        s.idxp[0] = s.idxp[1] = nullptr;
        int blk_begin, blk_end;
        if (MODE == DENSE) {
            s.hk = blockIdx.y;
            s.seqlen = p.seqlens[req];
            blk_begin = req == req_begin ? sched_begin_block : 0;
            blk_end = req == req_end ? sched_end_block : (s.seqlen + BLK - 1) / BLK;
        } else if (MODE == SPARSE_FP8) {
            s.t_fixed = blockIdx.y;
            const int l0 = p.topk_len[0] ? p.topk_len[0][req] : p.topk[0];
            const int l1 = p.topk[1] ? (p.topk_len[1] ? p.topk_len[1][req] : p.topk[1]) : 0;
            s.len[0] = min(l0, p.topk[0]); s.len[1] = min(l1, p.topk[1]);
            s.nblk0 = max((l0 + BLK - 1) / BLK, 1);
            const int total = s.nblk0 + (l1 + BLK - 1) / BLK;
            blk_begin = req == req_begin ? sched_begin_block : 0;
            blk_end = req == req_end ? sched_end_block : total;
            s.idxp[0] = p.idx[0] + req * p.idx_sb[0] + s.t_fixed * p.idx_ss[0];
            if (p.topk[1]) s.idxp[1] = p.idx[1] + req * p.idx_sb[1] + s.t_fixed * p.idx_ss[1];
        } else {
            s.t_fixed = req;
            const int l0 = p.topk_len[0] ? p.topk_len[0][req] : p.topk[0];
            s.len[0] = min(l0, p.topk[0]);
            blk_begin = 0;
            blk_end = (s.len[0] + BLK - 1) / BLK;
            s.idxp[0] = p.idx[0] + req * p.idx_ss[0];
        }

        // ---- Q tile -> shared memory (rows beyond the valid ones are zero) -----------------------
        constexpr int QCH = DQK / 8;
        for (int c = tid; c < BM * QCH; c += NTHREADS) {
            const int r = c / QCH, ch = c - r * QCH;
            const int row = row_blk * BM + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < p.rows) {
                int t, hd;
                if (MODE == DENSE) { t = row / p.g; hd = s.hk * p.g + (row - t * p.g); }
                else { t = s.t_fixed; hd = row; }
                const __nv_bfloat16* src = (MODE == SPARSE_BF16)
                    ? p.q + (int64_t)t * p.q_ss + (int64_t)hd * p.q_sh
                    : p.q + (int64_t)req * p.q_sb + (int64_t)t * p.q_ss + (int64_t)hd * p.q_sh;
                v = *reinterpret_cast<const uint4*>(src + ch * 8);
            }
            *reinterpret_cast<uint4*>(sm.q + r * LDK + ch * 8) = v;
        }
        if (tid < BM) { sm.m[tid] = -INFINITY; sm.l[tid] = 0.f; }

        float acc[4][8][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;

        const int st_begin = blk_begin * 2, st_end = blk_end * 2;
        if (st_begin < st_end) { load_subtile<MODE, DQK>(p, sm, s, st_begin, 0); }
        cp_async_commit();

        for (int st = st_begin; st < st_end; ++st) {
            const int buf = (st - st_begin) & 1;
            if (st + 1 < st_end) load_subtile<MODE, DQK>(p, sm, s, st + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();

            // ---- phase 1: S = Q K^T ------------------------------------------------------------
            {
                float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
                const uint32_t a_base = smem_u32(sm.q + (mt * 16 + (lane & 15)) * LDK + (lane >> 4) * 8);
                const int mid = lane >> 3;
                const uint32_t b_base = smem_u32(sm.k[buf] + (nh * 16 + (mid >> 1) * 8 + (lane & 7)) * LDK + (mid & 1) * 8);
#pragma unroll 4
                for (int kk = 0; kk < DQK / 16; ++kk) {
                    uint32_t a[4], bfrag[4];
                    ldmatrix_x4(a, a_base + kk * 32);
                    ldmatrix_x4(bfrag, b_base + kk * 32);
                    mma_bf16(c0, a, bfrag[0], bfrag[1]);
                    mma_bf16(c1, a, bfrag[2], bfrag[3]);
                }
                float* srow0 = sm.s + (mt * 16 + gid) * LDS + nh * 16 + tig * 2;
                float* srow1 = srow0 + 8 * LDS;
                *reinterpret_cast<float2*>(srow0) = make_float2(c0[0], c0[1]);
                *reinterpret_cast<float2*>(srow1) = make_float2(c0[2], c0[3]);
                *reinterpret_cast<float2*>(srow0 + 8) = make_float2(c1[0], c1[1]);
                *reinterpret_cast<float2*>(srow1 + 8) = make_float2(c1[2], c1[3]);
            }
            __syncthreads();

            // ---- phase 2: online softmax (4 threads per row, 8 tokens each) -----------------------
            {
                const int r = tid >> 2, part = tid & 3;
                int limit = 0x7fffffff;               // dense causal: first masked token position of this row
                if (MODE == DENSE && p.causal) {
                    const int row = row_blk * BM + r;
                    const int t = min(row / p.g, p.s_q - 1);
                    limit = s.seqlen - (p.s_q - 1 - t);
                }
                float v[8];
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int tok = part * 8 + j;
                    const bool ok = sm.valid[buf][tok] && (st * BN + tok < limit);
                    v[j] = ok ? sm.s[r * LDS + tok] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, v[j]);
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_old = sm.m[r];
                const float m_new = fmaxf(m_old, mx);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                float sum = 0.f;
                __nv_bfloat16* prow = sm.p + r * LDP + part * 8;
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float e0 = exp2f(v[j] - m_use), e1 = exp2f(v[j + 1] - m_use);
                    __nv_bfloat162 pb = __floats2bfloat162_rn(e0, e1);
                    sum += e0 + e1;
                    packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
                }
                *reinterpret_cast<uint4*>(prow) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                __syncwarp();
                if (part == 0) {
                    const float f = exp2f(m_old - m_use);      // m_old = -inf -> 0
                    sm.f[r] = f;
                    sm.l[r] = sm.l[r] * f + sum;
                    sm.m[r] = m_new;
                }
            }
            __syncthreads();

            // ---- phase 3: O = O * f + P V --------------------------------------------------------
            {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float f0 = sm.f[i * 16 + gid], f1 = sm.f[i * 16 + gid + 8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc[i][j][0] *= f0; acc[i][j][1] *= f0;
                        acc[i][j][2] *= f1; acc[i][j][3] *= f1;
                    }
                }
                const int mid = lane >> 3;
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    uint32_t a[4][4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        ldmatrix_x4(a[i], smem_u32(sm.p + (i * 16 + (lane & 15)) * LDP + ks * 16 + (lane >> 4) * 8));
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) {
                        uint32_t bfrag[4];
                        ldmatrix_x4_trans(bfrag, smem_u32(sm.k[buf] + (ks * 16 + (mid & 1) * 8 + (lane & 7)) * LDK
                                                          + warp * 64 + jp * 16 + (mid >> 1) * 8));
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            mma_bf16(acc[i][jp * 2], a[i], bfrag[0], bfrag[1]);
                            mma_bf16(acc[i][jp * 2 + 1], a[i], bfrag[2], bfrag[3]);
                        }
                    }
                }
            }
            __syncthreads();
        }
        cp_async_wait<0>();
        __syncthreads();

        // ---- epilogue ----------------------------------------------------------------------------
        bool is_split = false;
        int slot = 0;
        if (MODE != SPARSE_BF16) {
            is_split = req == req_begin ? first_split : (req == req_end ? last_split : false);
            slot = p.num_splits[req] + (req == req_begin ? begin_split : 0);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = i * 16 + gid + half * 8;
                const int row = row_blk * BM + r;
                if (row >= p.rows) continue;
                int t, hd;
                if (MODE == DENSE) { t = row / p.g; hd = s.hk * p.g + (row - t * p.g); }
                else { t = s.t_fixed; hd = row; }
                const float L = sm.l[r], M = sm.m[r];
                const bool empty = !(L > 0.f);             // also catches NaN
                if (!is_split) {
                    float scale = empty ? 0.f : 1.f / L;
                    if (p.attn_sink && !empty) scale = 1.f / (L + exp2f(p.attn_sink[hd] * kLog2e - M));
                    __nv_bfloat16* o = (MODE == SPARSE_BF16)
                        ? p.out + (int64_t)t * p.o_ss + (int64_t)hd * p.o_sh
                        : p.out + (int64_t)req * p.o_sb + (int64_t)t * p.o_ss + (int64_t)hd * p.o_sh;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __nv_bfloat162 v = __floats2bfloat162_rn(acc[i][j][half * 2] * scale, acc[i][j][half * 2 + 1] * scale);
                        *reinterpret_cast<__nv_bfloat162*>(o + warp * 64 + j * 8 + tig * 2) = v;
                    }
                    if (warp == 0 && tig == 0) {
                        const float lse_nat = empty ? INFINITY : (log2f(L) + M) * kLn2;
                        if (MODE == SPARSE_BF16) {
                            p.lse[(int64_t)t * p.h_q + hd] = lse_nat;
                            p.max_logits[(int64_t)t * p.h_q + hd] = empty ? -INFINITY : M * kLn2;
                        } else {
                            p.lse[req * p.l_sb + t * p.l_ss + hd * p.l_sh] = lse_nat;
                        }
                    }
                } else {
                    const float scale = empty ? 0.f : 1.f / L;
                    const int64_t arow = ((int64_t)slot * p.s_q + t) * p.h_q + hd;
                    float* o = p.o_accum + arow * D_V;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float2*>(o + warp * 64 + j * 8 + tig * 2) =
                            make_float2(acc[i][j][half * 2] * scale, acc[i][j][half * 2 + 1] * scale);
                    if (warp == 0 && tig == 0) p.lse_accum[arow] = empty ? -INFINITY : log2f(L) + M;
                }
            }
        }
        __syncthreads();     // sm.l / sm.m / sm.q are rewritten for the next request
    }
}

template <int MODE, int DQK = 576>
static int launch(const Params& p, dim3 grid, cudaStream_t stream) {
    static bool configured[8] = {};
    int dev = 0;
    MLA_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 8 && !configured[dev]) {
        MLA_CHECK_CUDA(cudaFuncSetAttribute(attn_portable_kernel<MODE, DQK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
        configured[dev] = true;
    } else if (dev >= 8) {
        MLA_CHECK_CUDA(cudaFuncSetAttribute(attn_portable_kernel<MODE, DQK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
    }
    attn_portable_kernel<MODE, DQK><<<grid, NTHREADS, sizeof(Smem), stream>>>(p);
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

}  // namespace portable

int launch_dense_decode_portable(const mla_dense_decode_args_t& a) {
    portable::Params p = {};
    p.b = a.b; p.s_q = a.s_q; p.h_q = a.h_q; p.h_kv = a.h_kv; p.g = a.h_q / a.h_kv;
    p.rows = a.s_q * p.g;
    p.scale_log2 = a.softmax_scale * kLog2e;
    p.q = (const __nv_bfloat16*)a.q; p.q_sb = a.q_stride_b; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.o_sb = a.o_stride_b; p.o_ss = a.o_stride_s; p.o_sh = a.o_stride_h;
    p.lse = a.lse; p.l_sb = a.lse_stride_b; p.l_ss = a.lse_stride_s; p.l_sh = a.lse_stride_h;
    p.kc = (const __nv_bfloat16*)a.k_cache; p.k_sblock = a.k_stride_block; p.k_srow = a.k_stride_row; p.k_shead = a.k_stride_head;
    p.block_table = a.block_table; p.bt_sb = a.block_table_stride_b; p.seqlens = a.seqlens_k; p.nblocks[0] = a.num_blocks;
    p.max_blocks = a.max_blocks_per_seq;
    p.causal = a.is_causal && a.s_q > 1;
    p.meta = a.meta; p.num_splits = a.num_splits; p.lse_accum = a.lse_accum; p.o_accum = a.o_accum;
    dim3 grid((p.rows + portable::BM - 1) / portable::BM, a.h_kv, a.num_sm_parts);
    return portable::launch<portable::DENSE>(p, grid, (cudaStream_t)a.stream);
}

int launch_sparse_decode_portable(const mla_sparse_decode_args_t& a) {
    portable::Params p = {};
    p.b = a.b; p.s_q = a.s_q; p.h_q = a.h_q; p.h_kv = 1; p.g = a.h_q;
    p.rows = a.h_q;
    p.scale_log2 = a.sm_scale * kLog2e;
    p.q = (const __nv_bfloat16*)a.q; p.q_sb = a.q_stride_b; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.o_sb = a.o_stride_b; p.o_ss = a.o_stride_s; p.o_sh = a.o_stride_h;
    p.lse = a.lse; p.l_sb = a.lse_stride_b; p.l_ss = a.lse_stride_s; p.l_sh = a.lse_stride_h;
    p.attn_sink = a.attn_sink;
    p.kvb[0] = (const uint8_t*)a.kv; p.kvb_sblock[0] = a.kv_stride_block_bytes; p.pbs[0] = a.page_block_size; p.nblocks[0] = a.num_blocks;
    p.idx[0] = a.indices; p.idx_sb[0] = a.indices_stride_b; p.idx_ss[0] = a.indices_stride_s; p.topk[0] = a.topk; p.topk_len[0] = a.topk_length;
    p.kvb[1] = (const uint8_t*)a.extra_kv; p.kvb_sblock[1] = a.extra_kv_stride_block_bytes; p.pbs[1] = a.extra_page_block_size > 0 ? a.extra_page_block_size : 1;
    p.nblocks[1] = a.extra_num_blocks;
    p.idx[1] = a.extra_indices; p.idx_sb[1] = a.extra_indices_stride_b; p.idx_ss[1] = a.extra_indices_stride_s;
    p.topk[1] = a.extra_kv ? a.extra_topk : 0; p.topk_len[1] = a.extra_topk_length;
    p.meta = a.meta; p.num_splits = a.num_splits; p.lse_accum = a.lse_accum; p.o_accum = a.o_accum;
    dim3 grid((a.h_q + portable::BM - 1) / portable::BM, a.s_q, a.num_sm_parts);
    if (a.d_qk == 512) return portable::launch<portable::SPARSE_FP8, 512>(p, grid, (cudaStream_t)a.stream);
    return portable::launch<portable::SPARSE_FP8>(p, grid, (cudaStream_t)a.stream);
}

int launch_sparse_prefill_portable(const mla_sparse_prefill_args_t& a) {
    portable::Params p = {};
    p.b = a.s_q; p.s_q = 1; p.h_q = a.h_q; p.h_kv = 1; p.g = a.h_q;
    p.rows = a.h_q;
    p.scale_log2 = a.sm_scale * kLog2e;
    p.q = (const __nv_bfloat16*)a.q; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.o_ss = (int64_t)a.h_q * a.d_v; p.o_sh = a.d_v;
    p.lse = a.lse; p.max_logits = a.max_logits;
    p.attn_sink = a.attn_sink;
    p.kvf = (const __nv_bfloat16*)a.kv; p.kvf_ss = a.kv_stride_s; p.s_kv = a.s_kv;
    p.idx[0] = a.indices; p.idx_ss[0] = a.indices_stride_s; p.topk[0] = a.topk; p.topk_len[0] = a.topk_length;
    dim3 grid(a.s_q, (a.h_q + portable::BM - 1) / portable::BM, 1);   // query tokens on x: no 65535 limit
    if (a.d_qk == 512) return portable::launch<portable::SPARSE_BF16, 512>(p, grid, (cudaStream_t)a.stream);
    return portable::launch<portable::SPARSE_BF16>(p, grid, (cudaStream_t)a.stream);
}

}  // namespace mla
