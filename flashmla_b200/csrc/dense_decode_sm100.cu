// Dense BF16 paged MLA decode for sm_100a: tcgen05 MMAs with TMEM accumulators, fed by TMA loads of
// 64-token KV pages through the block table.
//
// Problem shape per (request, kv head): 128 query rows (query token x head, padded with zero rows)
// against a paged stream of 576-wide K rows whose first 512 columns are also V.  The fp32 output
// accumulator O[128 x 512] fills all 512 columns of one SM's tensor memory, so the work of one row
// block is split over a CLUSTER OF TWO CTAs on two SMs that walk the same KV range:
//
//   CTA 0 ("score" CTA)   TMEM: Q as the A operand (288 columns of packed bf16) + two S buffers.
//                         S = Q K^T per 64-token page (36 MMAs 128x64x16, A from tensor memory, B = the
//                         K page in shared memory, K-major, 128-byte swizzle, 3-stage TMA ring),
//                         online softmax by 128 threads (one row each, no shuffles), P (bf16) written
//                         straight into CTA 1's shared memory over DSMEM in the MMA operand layout.
//   CTA 1 ("value" CTA)   TMEM: O (512 columns).  O += P V per page (8 MMAs 128x256x16, A = P from shared
//                         memory, B = the first 512 columns of the same page viewed MN-major, 3-stage
//                         TMA ring), rare O rescale, epilogue (normalise, bf16 / fp32 split output).
//
// The tensor work divides 576 : 512 between the two SMs; each KV page is fetched from HBM by whichever
// CTA asks first and from L2 by the other.  No TMA multicast is used.
//
// Softmax uses the running maximum lazily: O is rescaled only when a row's maximum grew by more than 2^6
// since the value in use; P, the row sum and O always refer to the same maximum, so results are exact
// up to rounding.
//
// Every mbarrier wait is bounded (about a second); on expiry the thread records a code in the status
// words, stops waiting and the CTA pair winds down normally (tensor memory is released, both CTAs
// leave together).
//
// Behavioural reference: csrc/sm90/decode/dense/splitkv_mla.cuh:959-1272 (masking, split / direct
// epilogue, empty rows) of deepseek-ai/FlashMLA; the reference has no sm_100 dense decode kernel.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace mla {
namespace sm100 {

using namespace ptx;

constexpr int ROWS = 128;
constexpr int TOK = 64;               // tokens per page / tile
constexpr int D_QK = 576, D_V = 512;
constexpr int BOX_BYTES = 8192;       // one TMA box: 64 tokens x 64 bf16, 128-byte swizzled rows
constexpr int K_STAGE_BYTES = 9 * BOX_BYTES;
constexpr int V_STAGE_BYTES = 8 * BOX_BYTES;
constexpr int NSTAGE = 3;
constexpr int P_BYTES = ROWS * TOK * 2;
constexpr int NTHREADS = 256;
constexpr long long WAIT_LIMIT = 2000000000LL;    // SM cycles (about one second)
constexpr float RESCALE_THRESHOLD = 6.0f;         // log2 units

// tensor-memory columns of the score CTA
constexpr uint32_t TM_S0 = 0, TM_S1 = 64, TM_Q = 128;

struct Smem {
    // score CTA: 3 K stages (73,728 B each).  value CTA: 3 V stages (65,536 B each) + 2 P tiles.
    uint8_t data[NSTAGE * V_STAGE_BYTES + 2 * P_BYTES];
    float factor[2][ROWS];        // value CTA: per-row rescale factor that goes with P tile 0 / 1
    uint32_t resc_flag[2][4];     // value CTA: "some row of this warp's 32 rows needs a rescale"
    float fin_l[ROWS], fin_m[ROWS];   // value CTA: final row sum / running maximum of the request
    uint64_t kv_full[NSTAGE], kv_empty[NSTAGE];
    uint64_t s_full[2], s_empty[2], q_ready;
    uint64_t p_empty[2], fin_empty;                       // live in the score CTA, arrived by the value CTA
    uint64_t p_full[2], pv_done[2], corr_done[2], fin_full;   // live in the value CTA
    uint32_t tmem_base;
    uint32_t aborted;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");
static_assert(NSTAGE * K_STAGE_BYTES <= NSTAGE * V_STAGE_BYTES + 2 * P_BYTES, "K ring must fit");

struct Params {
    int b, s_q, h_q, h_kv, g, rows, causal;
    float scale_log2;
    const __nv_bfloat16* q; int64_t q_sb, q_ss, q_sh;
    __nv_bfloat16* out; int64_t o_sb, o_ss, o_sh;
    float* lse; int64_t l_sb, l_ss, l_sh;
    const int* block_table; int64_t bt_sb; const int* seqlens;
    const mla_sched_meta_t* meta; const int* num_splits;
    float* lse_accum; float* o_accum;
    int* status;
    int row_blocks;
};

// One unit of work of a partition: a request and the range of its 64-token blocks walked here.
struct Work {
    int req, blk_begin, blk_end, seqlen, is_split, slot;
};

struct Walker {
    mla_sched_meta_t m;
    const Params& p;
    int req;
    __device__ Walker(const Params& p_, int part) : p(p_) { m = p_.meta[part]; req = m.begin_req_idx; }
    __device__ bool valid() const { return m.begin_req_idx < p.b && req <= m.end_req_idx; }
    __device__ Work get() const {
        Work w;
        w.req = req;
        w.seqlen = p.seqlens[req];
        w.blk_begin = req == m.begin_req_idx ? m.begin_block_idx : 0;
        w.blk_end = req == m.end_req_idx ? m.end_block_idx : (w.seqlen + TOK - 1) / TOK;
        if (w.blk_end < w.blk_begin) w.blk_end = w.blk_begin;
        w.is_split = req == m.begin_req_idx ? m.is_first_req_splitted : (req == m.end_req_idx ? m.is_last_req_splitted : 0);
        w.slot = p.num_splits[req] + (req == m.begin_req_idx ? m.begin_split_idx : 0);
        return w;
    }
    __device__ void next() { ++req; }
};

// Bounded wait helper: after the first expiry the thread stops waiting altogether.
struct Waiter {
    bool aborted = false;
    int* status;
    uint32_t* smem_flag;
    __device__ Waiter(int* st, uint32_t* flag) : status(st), smem_flag(flag) {}
    template <bool CLUSTER>
    __device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity, int code) {
        if (aborted) return;
        if (!mbar_wait_bounded<CLUSTER>(smem_addr(bar), parity, WAIT_LIMIT)) {
            aborted = true;
            *smem_flag = 1;
            if (status) { atomicCAS(status, 0, code); atomicAdd(status + 1, 1); }
        }
    }
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
dense_decode_sm100_kernel(const __grid_constant__ CUtensorMap kmap, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    const uint32_t cta_rank = cluster_ctarank();          // 0 = score CTA, 1 = value CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_blk = blockIdx.y % p.row_blocks;
    const int hk = blockIdx.y / p.row_blocks;
    const int part = blockIdx.z;

    if ((smem_addr(smem_raw) & 1023u) != 0) {              // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, 900);
        return;                                            // both CTAs of the pair take this branch
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGE; ++i) { mbar_init(smem_addr(&sm.kv_full[i]), 1); mbar_init(smem_addr(&sm.kv_empty[i]), 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_addr(&sm.s_full[i]), 1);
            mbar_init(smem_addr(&sm.s_empty[i]), 128);
            mbar_init(smem_addr(&sm.p_empty[i]), 1);
            mbar_init(smem_addr(&sm.p_full[i]), 128);
            mbar_init(smem_addr(&sm.pv_done[i]), 1);
            mbar_init(smem_addr(&sm.corr_done[i]), 128);
        }
        mbar_init(smem_addr(&sm.q_ready), 128);
        mbar_init(smem_addr(&sm.fin_empty), 128);
        mbar_init(smem_addr(&sm.fin_full), 128);
        sm.aborted = 0;
        fence_mbar_init();
        prefetch_tensormap(&kmap);
    }
    if (warp == 1) { tmem_alloc(smem_addr(&sm.tmem_base), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    cluster_sync();                                        // the peer's barriers exist before anyone arrives remotely
    const uint32_t tmem = sm.tmem_base;
    Waiter wt(p.status, &sm.aborted);

    // =====================================================================================================
    if (warp == 0) {
        // ---------------- TMA producer (both CTAs): K pages (9 boxes) or V pages (8 boxes) --------------
        if (lane == 0) {
            const int nbox = cta_rank == 0 ? 9 : 8;
            const int stage_bytes = cta_rank == 0 ? K_STAGE_BYTES : V_STAGE_BYTES;
            uint32_t g = 0;
            for (Walker wk(p, part); wk.valid(); wk.next()) {
                const Work w = wk.get();
                const int* bt = p.block_table + (int64_t)w.req * p.bt_sb;
                int page_next = w.blk_begin < w.blk_end ? __ldg(bt + w.blk_begin) : 0;
                for (int blk = w.blk_begin; blk < w.blk_end; ++blk, ++g) {
                    const int page = page_next;
                    if (blk + 1 < w.blk_end) page_next = __ldg(bt + blk + 1);
                    const uint32_t stage = g % NSTAGE, ph = (g / NSTAGE) & 1;
                    wt.wait<false>(&sm.kv_empty[stage], ph ^ 1, 1 + cta_rank * 100);
                    const uint32_t bar = smem_addr(&sm.kv_full[stage]);
                    mbar_arrive_expect_tx(bar, stage_bytes);
                    const uint32_t dst = smem_addr(sm.data + stage * stage_bytes);
                    for (int j = 0; j < nbox; ++j) tma_load_4d(dst + j * BOX_BYTES, &kmap, bar, j * 64, hk, 0, page);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer -----------------------------------------------------------------------
        if (lane == 0) {
            uint32_t g = 0, nreq = 0;
            if (cta_rank == 0) {
                constexpr uint32_t idesc = make_idesc_bf16(ROWS, TOK, false);
                for (Walker wk(p, part); wk.valid(); wk.next(), ++nreq) {
                    const Work w = wk.get();
                    wt.wait<false>(&sm.q_ready, nreq & 1, 2);
                    for (int blk = w.blk_begin; blk < w.blk_end; ++blk, ++g) {
                        const uint32_t stage = g % NSTAGE, sb = g & 1;
                        wt.wait<false>(&sm.kv_full[stage], (g / NSTAGE) & 1, 3);
                        wt.wait<false>(&sm.s_empty[sb], ((g >> 1) & 1) ^ 1, 4);
                        tc_fence_after();
                        const uint32_t kbase = smem_addr(sm.data + stage * K_STAGE_BYTES);
                        const uint32_t d_tmem = tmem + (sb ? TM_S1 : TM_S0);
#pragma unroll 4
                        for (int kk = 0; kk < D_QK / 16; ++kk) {
                            const uint64_t bdesc = make_sw128_desc(kbase + (kk >> 2) * BOX_BYTES + (kk & 3) * 32, 16, 1024);
                            mma_ts(d_tmem, tmem + TM_Q + kk * 8, bdesc, idesc, kk > 0);
                        }
                        tc_commit(smem_addr(&sm.kv_empty[stage]));
                        tc_commit(smem_addr(&sm.s_full[sb]));
                    }
                }
            } else {
                constexpr uint32_t idesc = make_idesc_bf16(ROWS, 256, true);
                for (Walker wk(p, part); wk.valid(); wk.next(), ++nreq) {
                    const Work w = wk.get();
                    for (int blk = w.blk_begin; blk < w.blk_end; ++blk, ++g) {
                        const uint32_t stage = g % NSTAGE, pb = g & 1, pph = (g >> 1) & 1;
                        wt.wait<false>(&sm.kv_full[stage], (g / NSTAGE) & 1, 103);
                        wt.wait<true>(&sm.p_full[pb], pph, 104);
                        wt.wait<false>(&sm.corr_done[pb], pph, 105);
                        fence_proxy_async();
                        tc_fence_after();
                        const uint32_t vbase = smem_addr(sm.data + stage * V_STAGE_BYTES);
                        const uint32_t pbase = smem_addr(sm.data + NSTAGE * V_STAGE_BYTES + pb * P_BYTES);
#pragma unroll
                        for (int kt = 0; kt < TOK / 16; ++kt) {
                            const uint64_t adesc = make_sw128_desc(pbase + kt * 32, 16, 1024);
#pragma unroll
                            for (int nh = 0; nh < 2; ++nh) {
                                const uint64_t bdesc = make_sw128_desc(vbase + nh * 4 * BOX_BYTES + kt * 2048, BOX_BYTES, 1024);
                                mma_ss(tmem + nh * 256, adesc, bdesc, idesc, (blk > w.blk_begin || kt > 0) ? 1u : 0u);
                            }
                        }
                        tc_commit(smem_addr(&sm.kv_empty[stage]));
                        tc_commit(smem_addr(&sm.pv_done[pb]));
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ---------------- value CTA: tell the score CTA when a P tile has been consumed -------------------
        if (cta_rank == 1 && lane == 0) {
            uint32_t g = 0;
            const uint32_t remote_p_empty0 = map_to_cta(smem_addr(&sm.p_empty[0]), 0);
            const uint32_t remote_p_empty1 = map_to_cta(smem_addr(&sm.p_empty[1]), 0);
            for (Walker wk(p, part); wk.valid(); wk.next()) {
                const Work w = wk.get();
                for (int blk = w.blk_begin; blk < w.blk_end; ++blk, ++g) {
                    const uint32_t pb = g & 1;
                    wt.wait<false>(&sm.pv_done[pb], (g >> 1) & 1, 106);
                    mbar_arrive_remote(pb ? remote_p_empty1 : remote_p_empty0);
                }
            }
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;                     // row inside the block = TMEM lane
        const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int row = row_blk * ROWS + r;                       // row inside the (request, kv head) group
        const bool row_ok = row < p.rows;
        const int t = row_ok ? row / p.g : 0;
        const int hd = hk * p.g + (row_ok ? row - t * p.g : 0);
        uint32_t g = 0, nreq = 0;

        if (cta_rank == 0) {
            // ---------------- softmax warpgroup of the score CTA ---------------------------------------------
            const uint32_t remote_p = map_to_cta(smem_addr(sm.data + NSTAGE * V_STAGE_BYTES), 1);
            const uint32_t remote_factor = map_to_cta(smem_addr(&sm.factor[0][0]), 1);
            const uint32_t remote_flag = map_to_cta(smem_addr(&sm.resc_flag[0][0]), 1);
            const uint32_t remote_p_full0 = map_to_cta(smem_addr(&sm.p_full[0]), 1);
            const uint32_t remote_p_full1 = map_to_cta(smem_addr(&sm.p_full[1]), 1);
            const uint32_t remote_fin_l = map_to_cta(smem_addr(&sm.fin_l[r]), 1);
            const uint32_t remote_fin_m = map_to_cta(smem_addr(&sm.fin_m[r]), 1);
            const uint32_t remote_fin_full = map_to_cta(smem_addr(&sm.fin_full), 1);
            for (Walker wk(p, part); wk.valid(); wk.next(), ++nreq) {
                const Work w = wk.get();
                // Q row -> tensor memory (A operand: 2 bf16 per 32-bit column).  Every MMA that read the previous
                // request's Q has completed: this thread saw s_full of that request's last tile.
                {
                    const __nv_bfloat16* qrow = p.q + (int64_t)w.req * p.q_sb + (int64_t)t * p.q_ss + (int64_t)hd * p.q_sh;
#pragma unroll 1
                    for (int c = 0; c < D_QK / 64; ++c) {
                        uint32_t v[32];
                        if (row_ok) {
                            const uint4* src = reinterpret_cast<const uint4*>(qrow + c * 64);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const uint4 x = __ldg(src + i);
                                v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = 0u;
                        }
                        tmem_st32(tlane + TM_Q + c * 32, v);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(smem_addr(&sm.q_ready));
                }
                // first key position this row must NOT see
                const int limit = p.causal ? w.seqlen - (p.s_q - 1 - t) : w.seqlen;
                float m_run = -INFINITY, l_run = 0.f;
                for (int blk = w.blk_begin; blk < w.blk_end; ++blk, ++g) {
                    const uint32_t sb = g & 1, ph = (g >> 1) & 1;
                    wt.wait<false>(&sm.s_full[sb], ph, 5);
                    tc_fence_after();
                    uint32_t s[64];
                    {
                        uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[0]);
                        uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[32]);
                        tmem_ld32(tlane + (sb ? TM_S1 : TM_S0), lo);
                        tmem_ld32(tlane + (sb ? TM_S1 : TM_S0) + 32, hi);
                    }
                    tmem_wait_ld();
                    tc_fence_before();
                    mbar_arrive(smem_addr(&sm.s_empty[sb]));          // the MMA warp may overwrite this S buffer

                    const int nvalid = limit - blk * TOK;             // columns [0, nvalid) are visible
                    float mx = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const float v = i < nvalid ? __uint_as_float(s[i]) : -INFINITY;
                        s[i] = __float_as_uint(v);
                        mx = fmaxf(mx, v);
                    }
                    mx *= p.scale_log2;                                // scale > 0: max commutes with scaling
                    float factor = 1.f;
                    bool resc = false;
                    if (blk == w.blk_begin) {
                        m_run = mx;
                    } else if (mx > m_run + RESCALE_THRESHOLD) {
                        factor = ex2(m_run - mx);                      // m_run = -inf -> 0
                        l_run *= factor;
                        m_run = mx;
                        resc = true;
                    }
                    const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
                    uint32_t pk[32];
                    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const float e0 = ex2(fmaf(__uint_as_float(s[i]), p.scale_log2, neg_m));
                        const float e1 = ex2(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, neg_m));
                        sum0 += e0; sum1 += e1;
                        pk[i >> 1] = pack_bf16(e0, e1);
                    }
                    l_run += sum0 + sum1;
                    const bool any_resc = __any_sync(0xffffffffu, resc);

                    wt.wait<true>(&sm.p_empty[sb], ph ^ 1, 6);        // P tile `sb` of the value CTA is free
                    const uint32_t prow = remote_p + sb * P_BYTES + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch)
                        st_cluster_v4(prow + ((ch ^ (r & 7)) << 4), pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                    st_cluster_f32(remote_factor + (sb * ROWS + r) * 4, factor);
                    if (lane == 0) st_cluster_u32(remote_flag + (sb * 4 + (warp & 3)) * 4, any_resc ? 1u : 0u);
                    fence_proxy_async();
                    mbar_arrive_remote(sb ? remote_p_full1 : remote_p_full0);
                }
                // final statistics of this request for the epilogue in the value CTA
                wt.wait<true>(&sm.fin_empty, (nreq & 1) ^ 1, 7);
                st_cluster_f32(remote_fin_l, l_run);
                st_cluster_f32(remote_fin_m, m_run);
                mbar_arrive_remote(remote_fin_full);
            }
        } else {
            // ---------------- correction / epilogue warpgroup of the value CTA ---------------------------------
            const uint32_t remote_fin_empty = map_to_cta(smem_addr(&sm.fin_empty), 0);
            for (Walker wk(p, part); wk.valid(); wk.next(), ++nreq) {
                const Work w = wk.get();
                for (int blk = w.blk_begin; blk < w.blk_end; ++blk, ++g) {
                    const uint32_t pb = g & 1, ph = (g >> 1) & 1;
                    wt.wait<true>(&sm.p_full[pb], ph, 107);
                    const bool need = blk > w.blk_begin && sm.resc_flag[pb][warp & 3] != 0;    // warp-uniform
                    if (need) {
                        // every earlier PV MMA has finished before O is touched
                        wt.wait<false>(&sm.pv_done[pb ^ 1], ((g - 1) >> 1) & 1, 108);
                        tc_fence_after();
                        const float f = sm.factor[pb][r];
#pragma unroll 1
                        for (int c = 0; c < D_V / 32; ++c) {
                            uint32_t v[32];
                            tmem_ld32(tlane + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
                            tmem_st32(tlane + c * 32, v);
                        }
                        tmem_wait_st();
                    }
                    // Tokens at or beyond the sequence length may hold anything (NaN included) in the cache:
                    // their probabilities are zero, so their V rows are zeroed to keep 0 * NaN out of O.
                    const int nvalid = w.seqlen - blk * TOK;
                    if (nvalid < TOK) {
                        const uint32_t stage = g % NSTAGE;
                        wt.wait<false>(&sm.kv_full[stage], (g / NSTAGE) & 1, 109);
                        uint8_t* vst = sm.data + stage * V_STAGE_BYTES;
                        const int nz = (TOK - max(nvalid, 0)) * 8 * 8;      // rows x boxes x 16-byte chunks
                        const int tid = threadIdx.x - 128;
                        for (int i = tid; i < nz; i += 128) {
                            const int chunk = i & 7, box = (i >> 3) & 7, rr = max(nvalid, 0) + (i >> 6);
                            *reinterpret_cast<uint4*>(vst + box * BOX_BYTES + rr * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                        }
                        fence_proxy_async();
                    }
                    tc_fence_before();
                    mbar_arrive(smem_addr(&sm.corr_done[pb]));
                }
                // ---- epilogue -----------------------------------------------------------------------------------
                const bool has_tiles = w.blk_end > w.blk_begin;
                if (has_tiles) wt.wait<false>(&sm.pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, 110);
                wt.wait<true>(&sm.fin_full, nreq & 1, 111);
                tc_fence_after();
                const float L = sm.fin_l[r], M = sm.fin_m[r];
                const bool empty = !(L > 0.f) || !has_tiles;          // also catches NaN
                const float scale = empty ? 0.f : 1.f / L;
                if (!w.is_split) {
                    __nv_bfloat16* orow = p.out + (int64_t)w.req * p.o_sb + (int64_t)t * p.o_ss + (int64_t)hd * p.o_sh;
#pragma unroll 1
                    for (int c = 0; c < D_V / 32; ++c) {
                        uint32_t v[32];
                        if (has_tiles) { tmem_ld32(tlane + c * 32, v); tmem_wait_ld(); }
                        if (row_ok) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 o;
                                o.x = empty ? 0u : pack_bf16(__uint_as_float(v[8 * i]) * scale, __uint_as_float(v[8 * i + 1]) * scale);
                                o.y = empty ? 0u : pack_bf16(__uint_as_float(v[8 * i + 2]) * scale, __uint_as_float(v[8 * i + 3]) * scale);
                                o.z = empty ? 0u : pack_bf16(__uint_as_float(v[8 * i + 4]) * scale, __uint_as_float(v[8 * i + 5]) * scale);
                                o.w = empty ? 0u : pack_bf16(__uint_as_float(v[8 * i + 6]) * scale, __uint_as_float(v[8 * i + 7]) * scale);
                                *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = o;
                            }
                        }
                    }
                    if (row_ok) p.lse[w.req * p.l_sb + t * p.l_ss + hd * p.l_sh] = empty ? INFINITY : (log2f(L) + M) * kLn2;
                } else {
                    const int64_t arow = ((int64_t)w.slot * p.s_q + t) * p.h_q + hd;
                    float* orow = p.o_accum + arow * D_V;
#pragma unroll 1
                    for (int c = 0; c < D_V / 32; ++c) {
                        uint32_t v[32];
                        if (has_tiles) { tmem_ld32(tlane + c * 32, v); tmem_wait_ld(); }
                        if (row_ok) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                float4 o;
                                o.x = empty ? 0.f : __uint_as_float(v[4 * i]) * scale;
                                o.y = empty ? 0.f : __uint_as_float(v[4 * i + 1]) * scale;
                                o.z = empty ? 0.f : __uint_as_float(v[4 * i + 2]) * scale;
                                o.w = empty ? 0.f : __uint_as_float(v[4 * i + 3]) * scale;
                                *reinterpret_cast<float4*>(orow + c * 32 + i * 4) = o;
                            }
                        }
                    }
                    if (row_ok) p.lse_accum[arow] = empty ? -INFINITY : log2f(L) + M;
                }
                tc_fence_before();
                mbar_arrive_remote(remote_fin_empty);        // fin_l / fin_m may be rewritten
            }
        }
    }

    // ---- wind down: both CTAs leave together, tensor memory is released -----------------------------------
    tc_fence_before();
    __syncthreads();
    if (sm.aborted) {
        // a bounded wait ran out somewhere: give copies that may still be in flight time to land
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    cluster_sync();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
    }
    return fn;
}

}  // namespace sm100

bool dense_decode_sm100_supports(const mla_dense_decode_args_t& a) {
    if (a.d_qk != 576 || a.d_v != 512 || a.page_block_size != 64) return false;
    if (a.h_kv <= 0 || a.h_q % a.h_kv != 0) return false;
    // TMA: strides in bytes must be multiples of 16 and below 2^40
    const int64_t lim = (int64_t)1 << 39;
    if (a.k_stride_block <= 0 || a.k_stride_row <= 0 || a.k_stride_head <= 0) return false;
    if (a.k_stride_block >= lim || a.k_stride_row >= lim || a.k_stride_head >= lim) return false;
    if (a.k_stride_block % 8 || a.k_stride_row % 8 || a.k_stride_head % 8) return false;
    const int rows = a.s_q * (a.h_q / a.h_kv);
    const int64_t row_blocks = (rows + 127) / 128;
    if (row_blocks * a.h_kv > 65535 || a.num_sm_parts > 65535) return false;
    return true;
}

int launch_dense_decode_sm100(const mla_dense_decode_args_t& a) {
    using namespace sm100;
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return set_error(MLA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");

    CUtensorMap kmap;
    cuuint64_t dims[4] = {(cuuint64_t)D_QK, (cuuint64_t)a.h_kv, (cuuint64_t)a.page_block_size, (cuuint64_t)a.num_blocks};
    cuuint64_t strides[3] = {(cuuint64_t)a.k_stride_head * 2, (cuuint64_t)a.k_stride_row * 2, (cuuint64_t)a.k_stride_block * 2};
    cuuint32_t box[4] = {64, 1, 64, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode(&kmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(a.k_cache), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(MLA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);

    Params p = {};
    p.b = a.b; p.s_q = a.s_q; p.h_q = a.h_q; p.h_kv = a.h_kv; p.g = a.h_q / a.h_kv;
    p.rows = a.s_q * p.g;
    p.causal = (a.is_causal && a.s_q > 1) ? 1 : 0;
    p.scale_log2 = a.softmax_scale * kLog2e;
    p.q = (const __nv_bfloat16*)a.q; p.q_sb = a.q_stride_b; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.o_sb = a.o_stride_b; p.o_ss = a.o_stride_s; p.o_sh = a.o_stride_h;
    p.lse = a.lse; p.l_sb = a.lse_stride_b; p.l_ss = a.lse_stride_s; p.l_sh = a.lse_stride_h;
    p.block_table = a.block_table; p.bt_sb = a.block_table_stride_b; p.seqlens = a.seqlens_k;
    p.meta = a.meta; p.num_splits = a.num_splits; p.lse_accum = a.lse_accum; p.o_accum = a.o_accum;
    p.status = a.status;
    p.row_blocks = (p.rows + ROWS - 1) / ROWS;

    static bool configured[64] = {};
    int dev = 0;
    MLA_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        MLA_CHECK_CUDA(cudaFuncSetAttribute(dense_decode_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
        if (dev < 64) configured[dev] = true;
    }
    dim3 grid(2, p.row_blocks * a.h_kv, a.num_sm_parts);
    dense_decode_sm100_kernel<<<grid, NTHREADS, sizeof(Smem), (cudaStream_t)a.stream>>>(kmap, p);
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

}  // namespace mla
