// MLA attention for sm_100a: tcgen05 MMAs with TMEM accumulators.  One kernel template serves
//   MODE_DENSE          dense BF16 / FP16 paged decode, fed by TMA loads of 64-token KV pages through the block table
//   MODE_PREFILL        token-sparse prefill, KV rows gathered by index with cp.async
//   MODE_SPARSE_DECODE  sparse FP8 decode, 656-byte records gathered by index and de-quantised in shared memory
//
// Problem shape per (request, kv head): 128 query rows (query token x head, padded with zero rows)
// against a stream of 576-wide K rows whose first 512 columns are also V.  The fp32 output
// accumulator O[128 x 512] fills all 512 columns of one SM's tensor memory, so the work of one row
// block is split over a CLUSTER OF TWO CTAs on two SMs that walk the same KV range in tiles of 128
// tokens (two pages):
//
//   CTA 0 ("score" CTA)  S = Q K^T: 36 MMAs 128x128x16 per tile (N = 128 runs the tensor pipe at full
//       rate, N = 64 does not).  Q is the A operand and lives in tensor memory (packed bf16).  K arrives
//       through a ring of 48 KB groups; a group is three 64-dim chunks of a tile (each [128 tokens][64 dims],
//       K-major, 128-byte swizzle) and is refilled as soon as its twelve MMAs have retired.
//         dense mode:   all 576 dims of Q in tensor memory (288 columns) next to ONE S accumulator (128 columns);
//                       the shared memory this frees makes the ring FOUR groups deep (192 KB): the time a tile
//                       takes is the refill latency of a ring slot divided by the slots that can be in flight.
//         gather modes: dims 0..447 of Q in tensor memory, dims 448..575 in shared memory, two S accumulators,
//                       a ring of three groups.
//       Two softmax warpgroups (one per page of the tile, one thread per row and page) exchange row
//       maxima through shared memory, write P (bf16) in MMA operand layout to a staging buffer and
//       push it to CTA 1 with bulk shared-to-shared copies that complete on CTA 1's barriers.
//   CTA 1 ("value" CTA)  O += P V: per page 2 x 4 MMAs 128x256x16 (A = P from shared memory, B = the
//       first 512 dims of the page viewed MN-major; 5-slot ring of [64 tokens][256 dims]),
//       the rare O rescale, and the epilogue (normalise; bf16 output or fp32 split partials).
//
// The tensor work divides 576 : 512 between the two SMs; each KV page is fetched from HBM by whichever
// CTA asks first and from L2 by the other.  No TMA multicast is used.  (MMAs that span the CTA pair,
// cta_group::2, were considered and not used: with 64 of the 128 rows per CTA each CTA still has to stage its
// half of the tokens for Q K^T and ALL tokens of its half of the columns for P V - 136 KB per tile and CTA
// against 144 + 128 KB here - so neither the bytes that enter the SMs nor the ring depth improve.)
//
// Softmax uses the running maximum lazily: O is rescaled only when a row's maximum grew by more than 2^6
// since the value in use; P, the row sum and O always refer to the same maximum, so results are exact
// up to rounding.
//
// Every mbarrier wait is bounded (Params::wait_limit SM cycles, about a second by default).  A thread whose
// wait ran out records a code in the status words, raises the `aborted` flag of both CTAs and LEAVES its role:
// it issues no further arrival, MMA or copy.  Single-thread roles leave at once; warps leave together (a vote
// after every wait, because tcgen05.ld/st are warp-collective); the two softmax warpgroups, which meet at a
// named barrier every tile, carry the flag through that barrier (bar.red.or) and leave together behind it.
// Threads that depend on the one that left run into their own limit.  The wind-down then waits - again
// bounded - for this CTA's own MMAs and TMA loads, meets the peer CTA, gives copies between the two CTAs time
// to land, and only then frees tensor memory; both CTAs leave together.
//
// Behavioural reference: csrc/sm90/decode/dense/splitkv_mla.cuh:959-1272 (masking, split / direct
// epilogue, empty rows), csrc/sm100/decode/head64/kernel.cuh:19-849 (FP8 records, validity, attn_sink) and
// csrc/sm100/prefill/sparse/fwd/head128/phase1.cuh:65-614 (prefill outputs) of deepseek-ai/FlashMLA.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include <cuda_fp16.h>
#include <string.h>
#include <stdlib.h>
#include <mutex>

namespace mla {
namespace sm100 {

using namespace ptx;

constexpr int ROWS = 128;
constexpr int PAGE = 64;              // tokens per page
constexpr int D_V = 512;             // value columns = the first 512 of the 576 key columns
constexpr int BOX_BYTES = 8192;       // 64 tokens x 64 bf16, 128-byte swizzled rows
constexpr int K_CHUNK_BYTES = 2 * BOX_BYTES;  // one 64-dim chunk of a tile: [128 tokens][64 dims]
constexpr int K_GROUP_BYTES = 3 * K_CHUNK_BYTES;   // the K ring moves in groups of 3 chunks (one barrier pair per group)
constexpr int V_SLOT_BYTES = 4 * BOX_BYTES;   // half a page of V: [64 tokens][256 dims] as 4 boxes
constexpr int NVS = 5;                        // V ring slots
constexpr int P_SUB_BYTES = ROWS * PAGE * 2;  // P of one page: [128 rows][64 tokens] bf16
constexpr int NPB = 4;                        // P buffers in the value CTA: (tile parity, page of the tile)
constexpr int NRING = 5;                      // ring barriers: K groups (score CTA, 3 or 4) / V slots (value CTA, 5)
constexpr int SIDE_BYTES = 144;               // per warp and tile: 32 rescale factors + flag (+ pad)
constexpr int NTHREADS = 384;                 // dense mode: control warpgroup + two softmax / correction warpgroups
constexpr int NTHREADS_GATHER = 512;          // sparse modes: one more warpgroup that gathers KV rows by index
constexpr long long WAIT_LIMIT_DEFAULT = 2000000000LL;    // SM cycles (about one second)
constexpr long long DRAIN_LIMIT = 4000000LL;              // wind-down after an expired wait: per tracked operation
constexpr long long SETTLE_CYCLES = 400000LL;             // ... and for copies between the two CTAs
#ifndef MLA_TAIL_BULK
#define MLA_TAIL_BULK 1
#endif
#ifndef MLA_SLEEP_NS
#define MLA_SLEEP_NS 200u
#endif
constexpr float RESCALE_THRESHOLD = 6.0f;         // log2 units

enum { MODE_DENSE = 0, MODE_PREFILL = 1, MODE_SPARSE_DECODE = 2 };

// Shared-memory and tensor-memory plan of the score CTA, per mode (byte offsets inside Smem::data).
template <int MODE>
struct Lay {
    static constexpr bool DENSE = MODE == MODE_DENSE;
    // WIDE plan (dense decode): all 576 dims of Q in tensor memory (288 columns) next to ONE S accumulator, which frees
    // the shared memory for a K ring of FOUR groups.  The gather modes keep the narrow plan (dims 0..447 of Q in tensor
    // memory, 448..575 in shared memory, two S accumulators, three groups): prefill is paced by the copy instructions of
    // its gather warps, not by the ring (measured with the wide plan: 3.49 against 3.41 ms), and FP8 decode needs 4 KB for
    // the tokens' scales.
    static constexpr bool WIDE = MODE == MODE_DENSE;
    static constexpr int NKS = WIDE ? 4 : 3;              // K ring slots; group j of tile g is fill 3 g + j and uses slot (3 g + j) mod NKS
    static constexpr int S_BUFS = WIDE ? 1 : 2;           // S accumulators in tensor memory
    static constexpr int Q_TMEM_CHUNKS = WIDE ? 9 : 7;    // 64-dim chunks of Q kept in tensor memory (the rest in SC_Q78)
    static constexpr int Q_SPLIT = WIDE ? 5 : 4;          // chunks [0, Q_SPLIT) are moved there by softmax warpgroup 0, the others by 1
    static constexpr uint32_t TM_S = 0, TM_Q = 128 * S_BUFS;
    static constexpr int SC_Q78 = 0;                                    // narrow plan: Q dims 448..575, 2 x [128][64]
    static constexpr int SC_KRING = WIDE ? 0 : 2 * 16384;
    static constexpr int SC_STAGE = SC_KRING + NKS * K_GROUP_BYTES;     // 8 warps x 4 KB P staging
    static constexpr int SC_SIDE = SC_STAGE + 8 * 4096;                 // 4 warps x 144 B factor/flag staging
    static constexpr int SC_XMAX = SC_SIDE + 4 * SIDE_BYTES;            // [2][2][128] floats
    static constexpr int SC_END = SC_XMAX + 2 * 2 * ROWS * 4;
    // gather modes only
    static constexpr int SC_MASK = SC_END;                // validity bits of the last 4 tiles, [4][4] words
    static constexpr int SC_LSUM = SC_MASK + 64;          // narrow plan: row sums of softmax warpgroup 1, handed to warpgroup 0 at the end of a request
    static constexpr int SC_SCALES = SC_LSUM + ROWS * 4;  // FP8 decode: the 4 scales of every token of the last two tiles, [2][128] float4
    static constexpr int SC_TOTAL = DENSE ? SC_END : (WIDE ? SC_MASK + 64 : SC_SCALES + 2 * ROWS * 16);
    static_assert(TM_Q + Q_TMEM_CHUNKS * 32 <= 512, "tensor-memory columns of the score CTA");
};
// value CTA (all modes)
constexpr int VA_VRING = 0;
constexpr int VA_P = VA_VRING + NVS * V_SLOT_BYTES;
constexpr int VA_SIDE = VA_P + NPB * P_SUB_BYTES;         // factors + flag received with the first page of tile parity 0 / 1: [2][4][SIDE_BYTES]
constexpr int VA_FIN = VA_SIDE + 2 * 4 * SIDE_BYTES;      // final row sum / running maximum / true maximum of the request: 3 x [128] floats
constexpr int VA_END = VA_FIN + 3 * ROWS * 4;
constexpr int cmax(int a, int b) { return a > b ? a : b; }
constexpr int DATA_BYTES = cmax(cmax(VA_END, Lay<MODE_DENSE>::SC_TOTAL), cmax(Lay<MODE_PREFILL>::SC_TOTAL, Lay<MODE_SPARSE_DECODE>::SC_TOTAL));

struct Smem {
    uint8_t data[DATA_BYTES];
    uint64_t kv_full[NRING], kv_empty[NRING];     // K groups (score CTA) / V slots (value CTA)
    uint64_t s_full[2], s_empty[2], q_ready, stage_full[2];
    uint64_t p_empty[NPB], stage_free[2], fin_empty;              // live in the score CTA, arrived by the value CTA
    uint64_t p_full[NPB], pv_done[NPB], corr_done[NPB], fin_full; // live in the value CTA
    uint64_t q_landed, ring_released;    // score CTA: a request's Q boxes have landed / have been copied out of the K ring
    uint64_t raw_full[NRING];            // FP8 decode: the raw records of a K group (score CTA) / V slot (value CTA) have landed
    uint64_t drain;                      // wind-down after an expired wait: this CTA's MMAs have retired
    uint32_t tmem_base;
    uint32_t aborted;                    // a bounded wait ran out in this CTA or in its peer
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");

struct Params {
    int b, s_q, h_q, h_kv, g, rows, causal, num_blocks;
    int head_chunks;                       // dense mode: 64-column chunks between two kv heads of a cache row
    int max_blocks;                        // dense mode: width of the block table
    float scale_log2;
    long long wait_limit;                  // SM cycles after which a barrier wait gives up
    const __nv_bfloat16* q; int64_t q_sb, q_ss, q_sh;
    int q_tma, q_box_bytes;                // a request's Q comes as 9 TMA boxes of q_box_bytes through the empty K ring
    __nv_bfloat16* out; int64_t o_sb, o_ss, o_sh;
    float* lse; int64_t l_sb, l_ss, l_sh;
    const int* block_table; int64_t bt_sb; const int* seqlens;
    const mla_sched_meta_t* meta; const int* num_splits;
    float* lse_accum; float* o_accum;
    int* status;
    int row_blocks;
    // token-sparse prefill: one "request" is one query token, its keys are gathered by index
    const int* indices; int64_t idx_ss; int topk; const int* topk_len; int s_kv;
    const __nv_bfloat16* kv; int64_t kv_ss;
    // sparse FP8 decode: two index scopes (main cache, optional extra cache) of 656-byte token records
    const uint8_t* kvb[2]; int64_t kvb_sblock[2]; int pbs[2]; int nblocks[2];
    const int* sidx[2]; int64_t sidx_sb[2], sidx_ss[2]; int stopk[2]; const int* stopk_len[2];
    const float* attn_sink; float* max_logits;
};

// One unit of work of a partition: a request and the range of its 64-token blocks walked here.
struct Work {
    int req, blk_begin, blk_end, ntiles, seqlen, is_split, slot;
    int last;                   // dense decode: the partition's last request (nothing is loaded into the V ring after it)
    int len0, len1, nblk0;      // sparse decode: valid positions of the two index scopes, blocks of the first scope
};

template <int MODE>
struct Walker;

// dense decode: the requests and block range of one SM partition, from the tile-scheduler metadata
template <>
struct Walker<MODE_DENSE> {
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
        w.blk_end = req == m.end_req_idx ? m.end_block_idx : (w.seqlen + PAGE - 1) / PAGE;
        if (w.blk_end < w.blk_begin) w.blk_end = w.blk_begin;
        w.ntiles = (w.blk_end - w.blk_begin + 1) / 2;
        w.is_split = req == m.begin_req_idx ? m.is_first_req_splitted : (req == m.end_req_idx ? m.is_last_req_splitted : 0);
        w.slot = p.num_splits[req] + (req == m.begin_req_idx ? m.begin_split_idx : 0);
        w.last = req == m.end_req_idx;
        return w;
    }
    __device__ void next() { ++req; }
};

// sparse FP8 decode: like dense decode, but a request's "sequence" is its top-k list: blocks [0, nblk0) index the
// main cache, the following blocks the optional extra cache (block counts as in the tile scheduler)
template <>
struct Walker<MODE_SPARSE_DECODE> {
    mla_sched_meta_t m;
    const Params& p;
    int req;
    __device__ Walker(const Params& p_, int part) : p(p_) { m = p_.meta[part]; req = m.begin_req_idx; }
    __device__ bool valid() const { return m.begin_req_idx < p.b && req <= m.end_req_idx; }
    __device__ Work get() const {
        Work w;
        w.req = req;
        const int l0 = p.stopk_len[0] ? p.stopk_len[0][req] : p.stopk[0];
        const int l1 = p.stopk[1] ? (p.stopk_len[1] ? p.stopk_len[1][req] : p.stopk[1]) : 0;
        w.len0 = min(max(l0, 0), p.stopk[0]);
        w.len1 = min(max(l1, 0), p.stopk[1]);
        w.nblk0 = max((l0 + PAGE - 1) / PAGE, 1);
        const int total = w.nblk0 + (l1 + PAGE - 1) / PAGE;
        w.seqlen = total * PAGE;
        w.blk_begin = req == m.begin_req_idx ? m.begin_block_idx : 0;
        w.blk_end = req == m.end_req_idx ? m.end_block_idx : total;
        if (w.blk_end < w.blk_begin) w.blk_end = w.blk_begin;
        w.ntiles = (w.blk_end - w.blk_begin + 1) / 2;
        w.is_split = req == m.begin_req_idx ? m.is_first_req_splitted : (req == m.end_req_idx ? m.is_last_req_splitted : 0);
        w.slot = p.num_splits[req] + (req == m.begin_req_idx ? m.begin_split_idx : 0);
        return w;
    }
    __device__ void next() { ++req; }
};

// sparse prefill: CTA pair `part` takes query tokens part, part + gridDim.z, ... ; "seqlen" is the number of
// top-k positions that may be valid
template <>
struct Walker<MODE_PREFILL> {
    const Params& p;
    int req;
    __device__ Walker(const Params& p_, int part) : p(p_), req(part) {}
    __device__ bool valid() const { return req < p.b; }
    __device__ Work get() const {
        Work w;
        w.req = req;
        w.seqlen = p.topk_len ? min(max(p.topk_len[req], 0), p.topk) : p.topk;
        w.blk_begin = 0;
        w.blk_end = (w.seqlen + PAGE - 1) / PAGE;
        w.ntiles = (w.blk_end + 1) / 2;
        w.is_split = 0;
        w.slot = 0;
        return w;
    }
    __device__ void next() { req += gridDim.z; }
};

#ifndef MLA_PRESPIN_DENSE
#define MLA_PRESPIN_DENSE 0
#endif
#ifndef MLA_PRESPIN_GATHER
#define MLA_PRESPIN_GATHER 64
#endif

// What a thread does when one of its bounded waits runs out: first code and a count in the global status words,
// the `aborted` flag of this CTA and of its peer.  Shared with the self-test kernel at the end of this file.
// (Out of line on purpose: inlined at every wait site it cost the dense kernel 10 % - 0.176 against 0.160 ms - although
// it never runs: the hot loops of all roles have to share the instruction cache.)
__device__ __noinline__ void report_expired_wait(int* status, uint32_t* flag, uint32_t peer_flag, int code) {
    *reinterpret_cast<volatile uint32_t*>(flag) = 1;
    if (peer_flag) st_cluster_u32(peer_flag, 1u);
    if (status) { atomicCAS(status, 0, code); atomicAdd(status + 1, 1); }
}

// Bounded wait helper.  wait() returns false when the wait ran out now or earlier: the caller leaves its role.
// LEAN: no unrolled probes before the timed loop (dense mode).
template <bool LEAN>
struct Waiter {
    bool aborted = false;
    bool parked;                         // park the thread between probes instead of spinning
    uint32_t sleep_ns;                   // ... and sleep this long between probes
    long long limit;
    int* status;
    uint32_t* flag;
    uint32_t peer_flag;
    __device__ Waiter(int* st, uint32_t* flag_, uint32_t peer_flag_, long long limit_, bool park = false, uint32_t sleep = 0)
        : parked(park), sleep_ns(sleep), limit(limit_), status(st), flag(flag_), peer_flag(peer_flag_) {}
    template <bool CLUSTER>
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, int code) {
        if (aborted) return false;
        const bool ok = parked ? mbar_wait_bounded_parked<CLUSTER>(smem_addr(bar), parity, limit, sleep_ns)
                               : mbar_wait_bounded<CLUSTER, LEAN ? MLA_PRESPIN_DENSE : MLA_PRESPIN_GATHER>(smem_addr(bar), parity, limit);
        if (!ok) {
            aborted = true;
            report_expired_wait(status, flag, peer_flag, code);
        }
        return ok;
    }
};

// single-thread roles: leave at once
#define WAIT_OR_LEAVE(W, CL, bar, par, code) do { if (!(W).template wait<CL>(bar, par, code)) goto wind_down; } while (0)
// whole warps (all 32 lanes execute this): leave together, tcgen05.ld/st and shuffles are warp-collective
#define WAIT_WARP_OR_LEAVE(W, CL, bar, par, code) \
    do { (W).template wait<CL>(bar, par, code); if (__any_sync(0xffffffffu, (W).aborted)) goto wind_down; } while (0)
// the two softmax warpgroups of the score CTA: their named barrier carries the flag
#define BAR_OR_LEAVE(flag) do { if (named_bar_red_or(1, 256, flag)) goto wind_down; } while (0)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two fp32 -> one 32-bit word of the 16-bit input type (bf16 or fp16), `lo` in the low half
template <bool FP16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    uint32_t r;
    if (FP16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return pack16<false>(lo, hi); }

// e8m0 scale byte -> fp32: 2^(e - 127); 0 is the subnormal 2^-127, 255 is NaN (as the format defines it)
__device__ __forceinline__ float e8m0_to_float(uint32_t e) {
    return __uint_as_float(e == 0 ? 0x00400000u : e == 255 ? 0x7fc00000u : e << 23);
}

// 16 e4m3 values (one uint4) times an fp32 scale -> 16 bf16 (two uint4), one rounding: bf16(fp32(e4m3) * scale).
// (A conversion-free variant that places the e4m3 magnitude bits into an fp32 word and multiplies by scale * 2^120 is
// bit-identical but needs more instructions per value and measured slower.)
__device__ __forceinline__ void dequant16(const uint4& raw, float scale, uint4& lo, uint4& hi) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2_raw h0 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xffffu), __NV_E4M3);
        __half2_raw h1 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
        const float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&h0));
        const float2 f1 = __half22float2(*reinterpret_cast<__half2*>(&h1));
        o[2 * i] = pack_bf16(f0.x * scale, f0.y * scale);
        o[2 * i + 1] = pack_bf16(f1.x * scale, f1.y * scale);
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}
__device__ __forceinline__ const uint8_t* shfl_ptr(const uint8_t* ptr, int src_lane) {
    const unsigned long long v = reinterpret_cast<unsigned long long>(ptr);
    const uint32_t lo = __shfl_sync(0xffffffffu, (uint32_t)v, src_lane);
    const uint32_t hi = __shfl_sync(0xffffffffu, (uint32_t)(v >> 32), src_lane);
    return reinterpret_cast<const uint8_t*>(((unsigned long long)hi << 32) | lo);
}

// Rare paths of the value CTA's correction warpgroup, kept out of line so that the loop around them stays small.
// O rows times their rescale factor (each thread its own row = tensor-memory lane).
__device__ __noinline__ void rescale_o_rows(uint32_t tlane, float f) {
#pragma unroll 1
    for (int c = 0; c < D_V / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tlane + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * f);
        tmem_st32(tlane + c * 32, v);
    }
    tmem_wait_st();
}
// Rows [first, 64) of a dense V slot ([8-token group][chunk][8 rows x 128 B]) set to zero by threads 128..255.
__device__ __noinline__ void zero_v_rows(uint8_t* vst, int first) {
    const int nz = (PAGE - first) * 4 * 8;              // rows x boxes x 16-byte chunks
    for (int k = threadIdx.x - 128; k < nz; k += 128) {
        const int chunk = k & 7, box = (k >> 3) & 3, rr = first + (k >> 5);
        *reinterpret_cast<uint4*>(vst + (rr >> 3) * 4096 + box * 1024 + (rr & 7) * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
    }
}

// A request's Q row moved by the softmax threads themselves, one thread per row: the path for Q tensors whose base or
// strides do not fit a TMA box (several times slower than the boxes; kept out of line, it is rarely taken).
// Warpgroup `half` takes its share of the chunks: to tensor memory, in the gather modes chunks 7 / 8 to shared memory.
template <int MODE>
__device__ __noinline__ void load_q_by_threads(Smem& sm, const __nv_bfloat16* qrow, bool row_ok, int half, int r, uint32_t tlane, bool no_chunk8) {
    using L = Lay<MODE>;
    const int c_begin = half ? L::Q_SPLIT : 0, c_end = half ? L::Q_TMEM_CHUNKS : L::Q_SPLIT, c_smem = half ? 8 : 7;
#pragma unroll 1
    for (int c = c_begin; c < c_end + (L::WIDE ? 0 : 1); ++c) {
        const int chunk = c < c_end ? c : c_smem;
        uint32_t v[32];
        if (row_ok && !(no_chunk8 && chunk == 8)) {
            const uint4* src = reinterpret_cast<const uint4*>(qrow + chunk * 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 x = __ldg(src + i);
                v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (c < c_end) {
            tmem_st32(tlane + L::TM_Q + chunk * 32, v);
        } else {
            uint8_t* qdst = sm.data + L::SC_Q78 + (chunk - L::Q_TMEM_CHUNKS) * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *reinterpret_cast<uint4*>(qdst + ((ch ^ (r & 7)) << 4)) = make_uint4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
        }
    }
}

// ALT selects the second data format of a mode.  Dense mode: q, the cache and out are fp16 instead of bf16 (accumulation
// is fp32 either way).  Sparse FP8 decode: the 512-wide record form (448 e4m3 + 64 bf16 RoPE per token, seven e8m0 scales
// per token stored behind the block's tokens, V = all 512 dims): chunk 7 of a tile is the RoPE part, chunk 8 is zeros.
// Sparse prefill: 512-wide rows; the ninth 64-column chunk of Q and K is zeros.  (A compile-time switch in every mode: the
// same choice read from the parameters inside the gather loop cost the 576-wide prefill 8 %.)
template <int MODE, bool ALT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MODE == MODE_DENSE ? NTHREADS : NTHREADS_GATHER, 1)
attn_sm100_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const __grid_constant__ CUtensorMap qmap, const Params p) {
    using WalkerT = Walker<MODE>;
    using L = Lay<MODE>;
    constexpr int NKS = L::NKS;
    constexpr bool DENSE = MODE == MODE_DENSE;
    constexpr bool FP16 = ALT && MODE == MODE_DENSE;
    constexpr bool M1 = ALT && MODE == MODE_SPARSE_DECODE;
    constexpr bool NO_CHUNK8 = ALT && MODE != MODE_DENSE;  // 512-wide rows
    constexpr int REC_BYTES = M1 ? 576 : 656;              // bytes between two tokens' values inside a block
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    const uint32_t cta_rank = cluster_ctarank();          // 0 = score CTA, 1 = value CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_blk = MODE == MODE_SPARSE_DECODE ? 0 : blockIdx.y % p.row_blocks;
    const int hk = MODE == MODE_SPARSE_DECODE ? 0 : blockIdx.y / p.row_blocks;
    const int part = blockIdx.z;

    if ((smem_addr(smem_raw) & 1023u) != 0) {              // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, 900);
        return;                                            // both CTAs of the pair take this branch
    }

    if (threadIdx.x == 0) {
        // a ring slot is filled by TMA (one arrive.expect_tx + bytes) in dense mode, by the 128 gather threads otherwise
        // ... except the K groups of FP8 decode, which the 256 softmax threads of the score CTA hand over after de-quantising them
        const uint32_t full_count = DENSE ? 1 : (MODE == MODE_SPARSE_DECODE && cta_rank == 0) ? 256 : 128;
        for (int i = 0; i < NRING; ++i) { mbar_init(smem_addr(&sm.kv_full[i]), full_count); mbar_init(smem_addr(&sm.kv_empty[i]), 1); }
        for (int i = 0; i < NRING; ++i) mbar_init(smem_addr(&sm.raw_full[i]), 128);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_addr(&sm.s_full[i]), 1);
            mbar_init(smem_addr(&sm.s_empty[i]), 256);
            mbar_init(smem_addr(&sm.stage_free[i]), 1);
            mbar_init(smem_addr(&sm.stage_full[i]), 128);
        }
        for (int i = 0; i < NPB; ++i) {
            mbar_init(smem_addr(&sm.p_empty[i]), 1);
            mbar_init(smem_addr(&sm.p_full[i]), 1);        // one arrive.expect_tx by the sending thread
            mbar_init(smem_addr(&sm.pv_done[i]), 1);
            mbar_init(smem_addr(&sm.corr_done[i]), 128);
        }
        mbar_init(smem_addr(&sm.q_ready), 256);
        mbar_init(smem_addr(&sm.q_landed), 1);
        mbar_init(smem_addr(&sm.ring_released), 256);
        mbar_init(smem_addr(&sm.fin_empty), 128);
        mbar_init(smem_addr(&sm.fin_full), 128);
        mbar_init(smem_addr(&sm.drain), 1);
        sm.aborted = 0;
        // first use of every P buffer: its arrival and expected byte count are armed here (matters in the value CTA)
        for (int i = 0; i < NPB; ++i)
            mbar_arrive_expect_tx(smem_addr(&sm.p_full[i]), P_SUB_BYTES + ((i & 1) == 0 ? 4 * SIDE_BYTES : 0));
        fence_mbar_init();
        if (DENSE) prefetch_tensormap(cta_rank == 0 ? &kmap : &vmap);
        if (p.q_tma && cta_rank == 0) prefetch_tensormap(&qmap);
    }
    if (warp == 1) { tmem_alloc(smem_addr(&sm.tmem_base), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    cluster_sync();                                        // the peer's barriers exist before anyone arrives remotely
    // Programmatic dependent launch: everything above ran while the previous kernel of the stream (the tile scheduler,
    // or whatever produced q) was still draining; from here on its results are read.  The kernel after this one (the
    // split-KV combine) may be scheduled as SMs become free: it waits for this grid's completion itself.
    griddep_wait();
    griddep_launch_dependents();
    const uint32_t tmem = sm.tmem_base;
    // gather modes: the gather warps need the issue slots that waiting warps would otherwise spin on
    // (FP8 decode, where a tile takes several microseconds, also sleeps between probes)
    using WaiterT = Waiter<DENSE>;
    const uint32_t peer_flag = map_to_cta(smem_addr(&sm.aborted), cta_rank ^ 1u);
#ifndef MLA_DENSE_PARK_WARPS
#define MLA_DENSE_PARK_WARPS 99          // dense mode: warps from this index on park between barrier probes
#endif
#ifndef MLA_DENSE_PARK_SLEEP
#define MLA_DENSE_PARK_SLEEP 0u
#endif
    WaiterT wt(p.status, &sm.aborted, peer_flag, p.wait_limit, DENSE ? warp >= MLA_DENSE_PARK_WARPS : warp < 12,
               MODE == MODE_SPARSE_DECODE ? MLA_SLEEP_NS : (DENSE ? MLA_DENSE_PARK_SLEEP : 0u));
    const int oob_page = p.num_blocks;                     // a page coordinate outside the cache: TMA fills zeros
    // what the wind-down has to wait for after an expired wait (thread 0: ring fills and Q boxes it armed)
    uint32_t fills_armed = 0, q_armed = 0;

    // A request's Q (score CTA): nine [rows][64 columns] boxes into the K ring once the previous request's tiles
    // have left it (the softmax warpgroups move them on to tensor memory and release the ring); in the gather modes
    // chunks 7 and 8 go to their final place in shared memory instead.  Large boxes stream several times faster into
    // one SM than per-thread loads, and the request boundary - where the MMA warp idles - is what this shortens.
    auto issue_q = [&](const Work& w) {
        const uint32_t bar = smem_addr(&sm.q_landed);
        mbar_arrive_expect_tx(bar, 9u * (uint32_t)p.q_box_bytes);
        ++q_armed;
        // coordinates: (column, head, query token, request); prefill: a "request" is a query token of the only batch
        const int c1 = MODE == MODE_SPARSE_DECODE ? 0 : MODE == MODE_PREFILL ? row_blk * ROWS : hk * p.g;
        const int c2 = MODE == MODE_SPARSE_DECODE ? (int)blockIdx.y : MODE == MODE_PREFILL ? w.req : row_blk * (ROWS / p.g);
        const int c3 = MODE == MODE_PREFILL ? 0 : w.req;
#pragma unroll 1
        for (int c = 0; c < 9; ++c) {
            const uint32_t dst = c < L::Q_TMEM_CHUNKS ? smem_addr(sm.data + L::SC_KRING + c * 16384)
                                                      : smem_addr(sm.data + L::SC_Q78 + (c - L::Q_TMEM_CHUNKS) * 16384);
            tma_load_4d(dst, &qmap, bar, c * 64, c1, c2, c3);
        }
    };

    // =====================================================================================================
    // In the sparse modes the CTA has 512 threads that start with 128 registers each; every warpgroup re-sizes its
    // share as the first thing in its own branch (the compiler budgets registers per branch from this).
    if (warp < 4) {
    if (!DENSE) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ---------------------------------------------------------
        if (!DENSE) {
            // sparse modes: the gather warpgroup fills the rings
            if (p.q_tma && cta_rank == 0 && lane == 0) {
                uint32_t ks = 0, nreq = 0;
                for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq) {
                    const Work w = wk.get();
                    issue_q(w);
                    WAIT_OR_LEAVE(wt, false, &sm.ring_released, nreq & 1, 11);     // (a request without tiles must not be overtaken)
                    // The next request's boxes may go out once every MMA of this one has finished with the ring and with
                    // Q.  A parity wait only means what it says to a thread that has seen every earlier phase of the
                    // barrier, so this thread follows the ring fill by fill.
                    for (int i = 0; i < 3 * w.ntiles; ++i, ++ks)
                        WAIT_OR_LEAVE(wt, false, &sm.kv_empty[ks % NKS], (ks / NKS) & 1, 13);
                }
            }
        } else if (lane == 0) {
            uint32_t ks = 0;                               // ring fill counter (K groups or V half-pages)
            uint32_t nreq = 0;
            const int chunk0 = hk * p.head_chunks;         // the kv head's first 64-column chunk in the tensor maps
            for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq) {
                const Work w = wk.get();
                const int* bt = p.block_table + (int64_t)w.req * p.bt_sb;
                // a block index beyond the table's width reads no table entry: its keys are zeros
                auto page_of = [&](int blk) -> int { return (blk < w.blk_end && blk < p.max_blocks) ? __ldg(bt + blk) : oob_page; };
                // page ids are fetched one tile ahead so the block-table latency stays off the TMA issue path
                int nxt0 = oob_page, nxt1 = oob_page;
                if (w.ntiles > 0) { nxt0 = page_of(w.blk_begin); nxt1 = page_of(w.blk_begin + 1); }
                if (p.q_tma && cta_rank == 0) {
                    // the K ring stages this request's Q first: wait until the previous request's groups (and every MMA
                    // that read its Q) are done - slot s is free for its next fill -, send the boxes, and take the ring
                    // back once they have been copied out
                    for (uint32_t s = 0; s < (uint32_t)NKS; ++s) {
                        const uint32_t nf = ks + (uint32_t)(((int)s - (int)(ks % NKS) + NKS) % NKS);      // the next fill that uses slot s
                        WAIT_OR_LEAVE(wt, false, &sm.kv_empty[s], ((nf / NKS) & 1) ^ 1, 13);
                    }
                    issue_q(w);
                    WAIT_OR_LEAVE(wt, false, &sm.ring_released, nreq & 1, 11);
                }
                for (int i = 0; i < w.ntiles; ++i) {
                    const int page0 = nxt0, page1 = nxt1;
                    if (i + 1 < w.ntiles) {
                        const int nb = w.blk_begin + 2 * (i + 1);
                        nxt0 = page_of(nb);
                        nxt1 = page_of(nb + 1);
                    }
                    if (cta_rank == 0) {
                        for (int grp = 0; grp < 3; ++grp, ++ks) {
                            const uint32_t slot = ks % NKS;
                            WAIT_OR_LEAVE(wt, false, &sm.kv_empty[slot], ((ks / NKS) & 1) ^ 1, 1);
                            const uint32_t bar = smem_addr(&sm.kv_full[slot]);
                            mbar_arrive_expect_tx(bar, K_GROUP_BYTES);
                            fills_armed = ks + 1;
                            const uint32_t dst = smem_addr(sm.data + L::SC_KRING + slot * K_GROUP_BYTES);
                            // one box per page: 3 chunks x 64 tokens land as [8-token group][chunk][8 x 128 B]
                            tma_load_5d(dst, &kmap, bar, 0, 0, chunk0 + grp * 3, 0, page0);
                            tma_load_5d(dst + K_GROUP_BYTES / 2, &kmap, bar, 0, 0, chunk0 + grp * 3, 0, page1);
                        }
                    } else {
                        for (int h = 0; h < 2; ++h) {
                            const int page = h ? page1 : page0;
                            for (int nh = 0; nh < 2; ++nh, ++ks) {
                                const uint32_t slot = ks % NVS;
                                WAIT_OR_LEAVE(wt, false, &sm.kv_empty[slot], ((ks / NVS) & 1) ^ 1, 101);
                                const uint32_t bar = smem_addr(&sm.kv_full[slot]);
                                mbar_arrive_expect_tx(bar, V_SLOT_BYTES);
                                fills_armed = ks + 1;
                                const uint32_t dst = smem_addr(sm.data + VA_VRING + slot * V_SLOT_BYTES);
                                // one box: 4 chunks x 64 tokens as [8-token group][chunk][8 x 128 B]
                                tma_load_5d(dst, &vmap, bar, 0, 0, chunk0 + nh * 4, 0, page);
                            }
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer -----------------------------------------------------------------------
        if (lane == 0) {
            uint32_t g = 0, ks = 0, nreq = 0;
            if (cta_rank == 0) {
                constexpr uint32_t idesc = make_idesc_16(ROWS, 128, false, FP16);
                const uint32_t q78_lo = sw128_desc_lo(smem_addr(sm.data + L::SC_Q78), 16);
                const uint32_t kring_lo = sw128_desc_lo(smem_addr(sm.data + L::SC_KRING), 16);
                const uint32_t kv_empty0 = smem_addr(&sm.kv_empty[0]);
                const uint32_t kv_full0 = smem_addr(&sm.kv_full[0]);
                uint32_t slot = 0, par = 0;                 // ring position of the next group: slot = ks mod NKS, par = (ks / NKS) & 1
                for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq) {
                    const Work w = wk.get();
                    WAIT_OR_LEAVE(wt, false, &sm.q_ready, nreq & 1, 2);
                    for (int i = 0; i < w.ntiles; ++i, ++g) {
                        const uint32_t sb = L::S_BUFS == 2 ? (g & 1) : 0;
                        const uint32_t s_par = L::S_BUFS == 2 ? ((g >> 1) & 1) : (g & 1);
                        WAIT_OR_LEAVE(wt, false, &sm.s_empty[sb], s_par ^ 1, 4);
                        tc_fence_after();
                        const uint32_t d_tmem = tmem + L::TM_S + sb * 128;
                        // Descriptors advance by 32-bit adds only and the loop is fully unrolled: one thread issues
                        // everything, so its instruction latency is the issue rate.
                        constexpr uint32_t hi = sw128_desc_hi(1024);
                        // K operand: the gather modes store a tile as 9 chunks of [128 tokens][128 B]; the dense mode's
                        // TMA boxes interleave the 3 chunks of a ring group inside every 8-token group.
                        constexpr uint32_t hi_k = sw128_desc_hi(DENSE ? 3 * 1024 : 1024);
                        // The probe of the next group's barrier is issued before this group's MMAs so that its
                        // latency hides behind them (the MMA queue is shallow: time the issuing thread spends
                        // waiting is time the tensor pipe idles).
                        // (narrow plan: three slots, so group j of every tile sits in slot j with the tile's parity and
                        // every address below is a compile-time offset)
                        if (!L::WIDE) { slot = 0; par = g & 1; }
                        bool ready = mbar_try_wait(kv_full0 + slot * 8, par);
#pragma unroll
                        for (int grp = 0; grp < 3; ++grp) {
                            const uint32_t cur = L::WIDE ? slot : (uint32_t)grp;
                            if (!ready) WAIT_OR_LEAVE(wt, false, &sm.kv_full[cur], par, 3);
                            tc_fence_after();
                            if (L::WIDE) { if (++slot == (uint32_t)NKS) { slot = 0; par ^= 1; } }
                            if (grp < 2) ready = mbar_try_wait(kv_full0 + (L::WIDE ? slot : (uint32_t)(grp + 1)) * 8, par);
                            const uint32_t grp_lo = kring_lo + cur * (K_GROUP_BYTES >> 4);
#pragma unroll
                            for (int c = 0; c < 3; ++c) {
                                const int j = grp * 3 + c;
                                const uint32_t b_lo = DENSE ? grp_lo + c * (1024 >> 4) : grp_lo + c * (K_CHUNK_BYTES >> 4);
#pragma unroll
                                for (int k4 = 0; k4 < 4; ++k4) {
                                    const uint32_t acc = (j > 0 || k4 > 0) ? 1u : 0u;
                                    if (j < L::Q_TMEM_CHUNKS) mma_ts_lohi(d_tmem, tmem + L::TM_Q + j * 32 + k4 * 8, b_lo + k4 * 2, hi_k, idesc, acc);
                                    else mma_ss_lohi(d_tmem, q78_lo + (j - L::Q_TMEM_CHUNKS) * (16384 >> 4) + k4 * 2, hi, b_lo + k4 * 2, hi_k, idesc, acc);
                                }
                            }
                            tc_commit(kv_empty0 + cur * 8);
                        }
                        tc_commit(smem_addr(&sm.s_full[sb]));
                    }
                }
            } else {
                constexpr uint32_t idesc = make_idesc_16(ROWS, 256, true, FP16);
                // V operand (MN-major): LBO = stride between 64-dim chunks, SBO = stride between 8-token groups.  Gather
                // modes: 4 chunks of [64 tokens][128 B]; dense mode: chunks interleaved inside every 8-token group.
                constexpr uint32_t hi_a = sw128_desc_hi(1024), hi_b = sw128_desc_hi(DENSE ? 4 * 1024 : 1024);
                constexpr uint32_t v_kstep = (DENSE ? 2 * 4096 : 2 * 1024) >> 4;      // 16 tokens
                const uint32_t p_lo = sw128_desc_lo(smem_addr(sm.data + VA_P), 16);
                const uint32_t vring_lo = sw128_desc_lo(smem_addr(sm.data + VA_VRING), DENSE ? 1024 : BOX_BYTES);
                for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq) {
                    const Work w = wk.get();
                    for (int i = 0; i < w.ntiles; ++i, ++g) {
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t pb = (g & 1) * 2 + h, pph = (g >> 1) & 1;
                            WAIT_OR_LEAVE(wt, true, &sm.p_full[pb], pph, 104);
                            WAIT_OR_LEAVE(wt, false, &sm.corr_done[pb], pph, 105);
                            const uint32_t a_lo = p_lo + pb * (P_SUB_BYTES >> 4);
#pragma unroll
                            for (int nh = 0; nh < 2; ++nh, ++ks) {
                                const uint32_t slot = ks % NVS;
                                WAIT_OR_LEAVE(wt, false, &sm.kv_full[slot], (ks / NVS) & 1, 103);
                                if (nh == 0) fence_proxy_async_smem();
                                tc_fence_after();
                                const uint32_t b_lo = vring_lo + slot * (V_SLOT_BYTES >> 4);
#pragma unroll
                                for (int kt = 0; kt < PAGE / 16; ++kt)
                                    mma_ss_lohi(tmem + nh * 256, a_lo + kt * 2, hi_a, b_lo + kt * v_kstep, hi_b, idesc,
                                                (i > 0 || h > 0 || kt > 0) ? 1u : 0u);
                                tc_commit(smem_addr(&sm.kv_empty[slot]));
                            }
                            tc_commit(smem_addr(&sm.pv_done[pb]));
                        }
                    }
                }
            }
        }
    } else if (warp == 2 || warp == 3) {
        // ---------------- score CTA: push finished P pages (and, with page 0, the rescale factors) to the value CTA
        if (cta_rank == 0 && lane == 0) {
            const int half = warp - 2;
            uint32_t g = 0;
            const uint32_t src_p = smem_addr(sm.data + L::SC_STAGE + half * 4 * 4096);
            const uint32_t src_side = smem_addr(sm.data + L::SC_SIDE);
            const uint32_t remote_p = map_to_cta(smem_addr(sm.data + VA_P), 1);
            const uint32_t remote_side = map_to_cta(smem_addr(sm.data + VA_SIDE), 1);
            uint32_t remote_p_full[NPB];
            for (int i = 0; i < NPB; ++i) remote_p_full[i] = map_to_cta(smem_addr(&sm.p_full[i]), 1);
            for (WalkerT wk(p, part); wk.valid(); wk.next()) {
                const Work w = wk.get();
                for (int i = 0; i < w.ntiles; ++i, ++g) {
                    const uint32_t pb = (g & 1) * 2 + half;
                    WAIT_OR_LEAVE(wt, false, &sm.stage_full[half], g & 1, 9);
                    WAIT_OR_LEAVE(wt, true, &sm.p_empty[pb], ((g >> 1) & 1) ^ 1, 6);   // that P buffer of the value CTA has been consumed
                    // p_full[pb] is armed (arrival + expected bytes) by the value CTA itself: a remote arrive with
                    // release semantics costs over a microsecond, the copies below only count bytes.
                    bulk_copy_to_cluster(remote_p + pb * P_SUB_BYTES, src_p, P_SUB_BYTES, remote_p_full[pb]);
                    if (half == 0)
                        bulk_copy_to_cluster(remote_side + (g & 1) * 4 * SIDE_BYTES, src_side, 4 * SIDE_BYTES, remote_p_full[pb]);
                }
            }
        }
        // ---------------- value CTA: tell the score CTA when a P buffer has been consumed ------------------
        if (cta_rank == 1 && warp == 2 && lane == 0) {
            uint32_t g = 0;
            uint32_t remote_p_empty[NPB];
            for (int i = 0; i < NPB; ++i) remote_p_empty[i] = map_to_cta(smem_addr(&sm.p_empty[i]), 0);
            for (WalkerT wk(p, part); wk.valid(); wk.next()) {
                const Work w = wk.get();
                for (int i = 0; i < w.ntiles; ++i, ++g) {
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t pb = (g & 1) * 2 + h;
                        WAIT_OR_LEAVE(wt, false, &sm.pv_done[pb], (g >> 1) & 1, 106);
                        // arm the buffer's barrier for its next use, then let the score CTA refill it
                        mbar_arrive_expect_tx(smem_addr(&sm.p_full[pb]), P_SUB_BYTES + (h == 0 ? 4 * SIDE_BYTES : 0));
                        mbar_arrive_remote_relaxed(remote_p_empty[pb]);
                    }
                }
            }
        }
    }
    } else if (!DENSE && warp >= 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        // ---------------- gather warpgroup (sparse modes): fills the K ring (score CTA) / V ring (value CTA) by index ----
        // Every warp owns a block of tokens; one cp.async instruction of the warp copies consecutive 16-byte pieces of
        // ONE token row (coalesced 128-byte lines, no registers held, as many copies in flight as the ring has room
        // for) into the 128-byte-swizzled operand layout; invalid tokens get zeros (zero-size source).  The ring
        // barrier counts one arrival per thread, made by the copy engine when that thread's copies have landed.
        const int gw = warp - 12;                                 // warp inside the gather warpgroup
        uint32_t ks = 0, g = 0, nreq_p = 0;
        uint32_t* kmask = reinterpret_cast<uint32_t*>(sm.data + L::SC_MASK);
        if (MODE == MODE_SPARSE_DECODE) {
            // FP8 records: index -> (page, offset) -> 656-byte record = 512 e4m3 | 4 fp32 scales | 64 bf16 RoPE.
            // A "piece" is 16 e4m3 values (16 bytes) that de-quantise (one rounding: bf16(fp32(e4m3) * scale)) into two
            // 16-byte slots of a 128-byte operand row.  Two decoupled steps per ring element (a K group of 3 chunks in
            // the score CTA, a V slot of 4 chunks in the value CTA):
            //   copy:    this warpgroup brings every raw piece with cp.async straight into the UPPER of its own two
            //            destination slots (lanes = pieces of two token rows: coalesced, no registers held), RoPE pieces
            //            into their final place, and counts the landing on the element's raw_full barrier;
            //   convert: warps that are idle most of a tile's time in this mode - the softmax warpgroups of the score
            //            CTA, warps 8-11 of the value CTA - expand the pieces of their token row in place (a thread reads
            //            a slot only it will overwrite; 16-byte accesses, conflict-free thanks to the swizzle) and hand
            //            the element to the MMA warp.
            // Copying and converting run side by side on different warps; record pointers (and, in the score CTA, the
            // scales the converting threads read from shared memory) are fetched one tile ahead.  The conversion loops
            // are deliberately left rolled: with every instance unrolled the conversion code was several times the
            // instruction cache and the warps waited for instructions more than they computed.
            const int tq = blockIdx.y;
            bool ring_lent = false;                                       // the K ring first stages every request's Q
            uint32_t nreq_g = 0;
            float4 sc_cur = make_float4(0.f, 0.f, 0.f, 0.f);
            const uint32_t kring = smem_addr(sm.data + L::SC_KRING);
            const uint32_t vring = smem_addr(sm.data + VA_VRING);
            for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq_g) {
                const Work w = wk.get();
                ring_lent = p.q_tma && cta_rank == 0;
                if (ring_lent && w.ntiles == 0) WAIT_WARP_OR_LEAVE(wt, false, &sm.ring_released, nreq_g & 1, 211);   // follow every phase
                const int* idx0 = p.sidx[0] + (int64_t)w.req * p.sidx_sb[0] + (int64_t)tq * p.sidx_ss[0];
                const int* idx1 = p.stopk[1] ? p.sidx[1] + (int64_t)w.req * p.sidx_sb[1] + (int64_t)tq * p.sidx_ss[1] : nullptr;
                // index -> record address in two steps, so that the index of a tile can be loaded two tiles ahead and
                // turned into an address (and a scale load) one tile ahead without waiting on memory
                auto load_id = [&](int blk, int off) -> int {
                    if (blk >= w.blk_end) return -1;
                    const int scope = blk >= w.nblk0 ? 1 : 0;
                    const int pos = (scope ? blk - w.nblk0 : blk) * PAGE + off;
                    if (pos >= (scope ? w.len1 : w.len0)) return -1;
                    return __ldg((scope ? idx1 : idx0) + pos);
                };
                auto rec_of = [&](int blk, int id) -> const uint8_t* {
                    const int scope = blk >= w.nblk0 ? 1 : 0;
                    const int pbs = p.pbs[scope];
                    if (id < 0 || (int64_t)id >= (int64_t)p.nblocks[scope] * pbs) return nullptr;
                    return p.kvb[scope] + (int64_t)(id / pbs) * p.kvb_sblock[scope] + (int64_t)(id % pbs) * REC_BYTES;
                };
                // the token's scales as they are stored: four fp32 inside the record, or (512-wide form) eight bytes -
                // seven e8m0 exponents and a pad - behind the block's tokens, carried in the first two words
                auto scales_of = [&](int blk, int id, const uint8_t* rec) {
                    if (!rec) return make_float4(0.f, 0.f, 0.f, 0.f);
                    if (!M1) return __ldg(reinterpret_cast<const float4*>(rec + 512));
                    const int scope = blk >= w.nblk0 ? 1 : 0;
                    const int pbs = p.pbs[scope];
                    const uint2 e = __ldg(reinterpret_cast<const uint2*>(p.kvb[scope] + (int64_t)(id / pbs) * p.kvb_sblock[scope] +
                                                                         (int64_t)pbs * 576 + (int64_t)(id % pbs) * 8));
                    return make_float4(__uint_as_float(e.x), __uint_as_float(e.y), 0.f, 0.f);
                };
                if (cta_rank == 0) {
                    // warp gw owns tokens 32*gw .. 32*gw+31 of the tile; lane l looks up token 32*gw + l
                    const int tok = gw * 32 + lane;
                    const int myblk = w.blk_begin + (tok >> 6);              // this lane's block of tile 0
                    const int id_first = load_id(myblk, tok & 63);
                    const uint8_t* rec_next = rec_of(myblk, id_first);
                    float4 sc_next = scales_of(myblk, id_first, rec_next);
                    int id_next = load_id(myblk + 2, tok & 63);              // tile 1
                    for (int i = 0; i < w.ntiles; ++i, ++g) {
                        const uint8_t* rec = rec_next;
                        sc_cur = sc_next;
                        // validity bits and scales of this tile's tokens for the threads that convert / mask it (the fence
                        // comes before the prefetch loads are issued: it would wait for them)
                        const uint32_t bal = __ballot_sync(0xffffffffu, rec != nullptr);
                        if (lane == 0) kmask[(g & 3) * 4 + gw] = bal;
                        reinterpret_cast<float4*>(sm.data + L::SC_SCALES)[(g & 1) * ROWS + tok] = sc_cur;
                        __threadfence_block();
                        rec_next = rec_of(myblk + 2 * (i + 1), id_next);
                        sc_next = scales_of(myblk + 2 * (i + 1), id_next, rec_next);
                        id_next = load_id(myblk + 2 * (i + 2), tok & 63);
                        if (ring_lent) { WAIT_WARP_OR_LEAVE(wt, false, &sm.ring_released, nreq_g & 1, 211); ring_lent = false; }
#pragma unroll 1
                        for (int grp = 0; grp < 3; ++grp, ++ks) {
                            WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_empty[grp], ((ks / NKS) & 1) ^ 1, 201);
                            // copy: groups 0, 1: 12 raw pieces per row; group 2: 8 raw pieces + 8 RoPE pieces per row.  A copy
                            // instruction costs the warp the same whatever its active lanes: each one serves two rows.
                            // (512-wide form: every group has 12 pieces per row; group 2 is chunk 6 - 4 raw pieces - and the 8 RoPE
                            // pieces, which are chunk 7; chunk 8 is zeroed by the converting threads)
                            const int per_row = (grp < 2 || M1) ? 12 : 16;
                            const int sub = (grp < 2 || M1) ? (lane >= 12) + (lane >= 24) : lane >> 4, ql = lane - sub * per_row;
                            const bool active = sub < 2;
                            constexpr int N_RAW2 = M1 ? 4 : 8;               // raw pieces of group 2
                            const bool is_rope = grp == 2 && ql >= N_RAW2;
                            const int q = grp * 12 + ql;                      // raw piece index in the row
                            const int srcoff = is_rope ? (M1 ? 448 : 528) + (ql - N_RAW2) * 16 : q * 16;
                            const int dslot = is_rope ? ql - N_RAW2 : 2 * (q & 3) + 1;
                            const uint32_t dst0 = kring + (is_rope ? (M1 ? 7 : 8) : (q >> 2)) * K_CHUNK_BYTES + gw * 32 * 128;
#pragma unroll 8
                            for (int u = 0; u < 16; ++u) {
                                const int rr = 2 * u + (active ? sub : 0);
                                const uint8_t* r = shfl_ptr(rec, rr);
                                if (active)
                                    cp_async16_zfill(dst0 + rr * 128 + ((dslot ^ (rr & 7)) << 4), (r ? r : p.kvb[0]) + srcoff, r ? 16u : 0u);
                            }
                            // the softmax warpgroups expand the pieces in place once they have landed
                            cp_async_arrive_noinc(smem_addr(&sm.raw_full[grp]));
                        }
                    }
                } else {
                    // value CTA: warp gw owns tokens 16*gw .. 16*gw+15 of each page; lanes l and l + 16 look up the same token
                    const int tok = gw * 16 + (lane & 15);
                    const uint8_t* rec_next = rec_of(w.blk_begin, load_id(w.blk_begin, tok));
                    int id_next = load_id(w.blk_begin + 1, tok);
                    for (int i = 0; i < w.ntiles; ++i, ++g) {
#pragma unroll 1
                        for (int h = 0; h < 2; ++h) {
                            const uint8_t* rec = rec_next;
                            const int nblk = w.blk_begin + 2 * i + h + 1;
                            rec_next = rec_of(nblk, id_next);
                            id_next = load_id(nblk + 1, tok);
#pragma unroll 1
                            for (int nh = 0; nh < 2; ++nh, ++ks) {
                                const uint32_t slot = ks % NVS;
                                WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_empty[slot], ((ks / NVS) & 1) ^ 1, 202);
                                // copy: 16 raw pieces per row (dims nh*256 .. nh*256+255); one instruction serves two rows
                                const int ql = lane & 15, sub = lane >> 4;
                                const int q = nh * 16 + ql;
                                const uint32_t dst0 = vring + slot * V_SLOT_BYTES + (ql >> 2) * BOX_BYTES + gw * 16 * 128;
                                const int dslot = 2 * (ql & 3) + 1;
                                // (512-wide form, second half: 12 raw pieces - chunks 4, 5, 6 - and, below, the RoPE part as chunk 7)
                                const bool piece_ok = !M1 || nh == 0 || ql < 12;
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    const int rr = 2 * u + sub;
                                    const uint8_t* r = shfl_ptr(rec, rr);
                                    if (piece_ok)
                                        cp_async16_zfill(dst0 + rr * 128 + ((dslot ^ (rr & 7)) << 4), (r ? r : p.kvb[0]) + q * 16, r ? 16u : 0u);
                                }
                                if (M1 && nh == 1) {
                                    const int piece = lane & 7;
                                    const uint32_t dst7 = vring + slot * V_SLOT_BYTES + 3 * BOX_BYTES + gw * 16 * 128;
#pragma unroll
                                    for (int u = 0; u < 4; ++u) {
                                        const int rr = 4 * u + (lane >> 3);
                                        const uint8_t* r = shfl_ptr(rec, rr);
                                        cp_async16_zfill(dst7 + rr * 128 + ((piece ^ (rr & 7)) << 4), (r ? r : p.kvb[0]) + 448 + piece * 16, r ? 16u : 0u);
                                    }
                                }
                                cp_async_arrive_noinc(smem_addr(&sm.raw_full[slot]));      // warps 8-11 expand the pieces
                            }
                        }
                    }
                }
            }
        } else
        for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq_p) {
            const Work w = wk.get();
            bool ring_lent = p.q_tma && cta_rank == 0;          // the K ring first stages this query token's Q
            if (ring_lent && w.ntiles == 0) WAIT_WARP_OR_LEAVE(wt, false, &sm.ring_released, nreq_p & 1, 211);        // follow every phase
            const int* idx = p.indices + (int64_t)w.req * p.idx_ss;
            // the index of a tile's token is loaded one tile ahead (a load that is used at once costs its latency)
            int id_next = -1;
            if (cta_rank == 0) { const int pos0 = gw * 32 + lane; id_next = pos0 < w.seqlen ? __ldg(idx + pos0) : -1; }
            int vid_next = -1;                       // value CTA: index of this lane's token of the next page
            if (cta_rank == 1) { const int pos0 = gw * 16 + (lane & 15); vid_next = pos0 < w.seqlen ? __ldg(idx + pos0) : -1; }
            for (int i = 0; i < w.ntiles; ++i, ++g) {
                if (cta_rank == 0) {
                    // warp gw owns tokens 32*gw .. 32*gw+31 of the tile; lane l looks up token 32*gw + l
                    const int id = id_next;
                    const bool ok = id >= 0 && id < p.s_kv;
                    const uint32_t bal = __ballot_sync(0xffffffffu, ok);
                    if (lane == 0) { kmask[(g & 3) * 4 + gw] = bal; __threadfence_block(); }   // token 32w + l of the tile is bit l of word w
                    // (issued after the fence, which would otherwise wait for it)
                    { const int posn = (i + 1) * 128 + gw * 32 + lane; id_next = posn < w.seqlen ? __ldg(idx + posn) : -1; }
                    const int row_id = ok ? id : -1;
                    // A copy instruction costs the warp the same whatever its active lanes, so a token row (72 pieces of
                    // 16 bytes) is copied by two full-warp instructions (chunks 0-3, chunks 4-7) and the RoPE chunk of
                    // four rows by a third: 72 instructions per 32 rows.  The ring barriers still count per group of 3
                    // chunks: every group's arrival is issued once all copies that touch it have been issued.
                    // the tile's three groups are fills ks, ks + 1, ks + 2 of the ring; chunk c of the tile lives in the slot of
                    // group c / 3, at chunk position c % 3
                    const uint32_t ring0 = smem_addr(sm.data + L::SC_KRING) + gw * 32 * 128;
                    // (three slots: group j sits in slot j and every address below is a compile-time offset)
                    const uint32_t slot0 = L::WIDE ? ks % NKS : 0u, slot1 = L::WIDE ? (ks + 1) % NKS : 1u, slot2 = L::WIDE ? (ks + 2) % NKS : 2u;
                    const int c = lane & 7;
                    if (ring_lent) { WAIT_WARP_OR_LEAVE(wt, false, &sm.ring_released, nreq_p & 1, 211); ring_lent = false; }
                    WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_empty[slot0], ((ks / NKS) & 1) ^ 1, 201);
                    WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_empty[slot1], (((ks + 1) / NKS) & 1) ^ 1, 201);
                    {
                        const int ch = lane >> 3;                     // chunks 0-3: 0, 1, 2 in group 0, chunk 3 in group 1
                        const uint32_t dst0 = ring0 + (ch < 3 ? slot0 * K_GROUP_BYTES + ch * K_CHUNK_BYTES : slot1 * K_GROUP_BYTES);
#pragma unroll 8
                        for (int rr = 0; rr < 32; ++rr) {
                            const int rid = __shfl_sync(0xffffffffu, row_id, rr);
                            const __nv_bfloat16* src = p.kv + (int64_t)(rid < 0 ? 0 : rid) * p.kv_ss + lane * 8;
                            cp_async16_zfill(dst0 + rr * 128 + ((c ^ (rr & 7)) << 4), src, rid < 0 ? 0u : 16u);
                        }
                    }
                    cp_async_arrive_noinc(smem_addr(&sm.kv_full[slot0]));
                    WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_empty[slot2], (((ks + 2) / NKS) & 1) ^ 1, 201);
                    {
                        const int ch = 4 + (lane >> 3);               // chunks 4-7: 4, 5 in group 1, chunks 6, 7 in group 2
                        const uint32_t dst0 = ring0 + (ch < 6 ? slot1 * K_GROUP_BYTES + (ch - 3) * K_CHUNK_BYTES
                                                              : slot2 * K_GROUP_BYTES + (ch - 6) * K_CHUNK_BYTES);
#pragma unroll 8
                        for (int rr = 0; rr < 32; ++rr) {
                            const int rid = __shfl_sync(0xffffffffu, row_id, rr);
                            const __nv_bfloat16* src = p.kv + (int64_t)(rid < 0 ? 0 : rid) * p.kv_ss + (32 + lane) * 8;
                            cp_async16_zfill(dst0 + rr * 128 + ((c ^ (rr & 7)) << 4), src, rid < 0 ? 0u : 16u);
                        }
                    }
                    cp_async_arrive_noinc(smem_addr(&sm.kv_full[slot1]));
                    {
                        const uint32_t dst0 = ring0 + slot2 * K_GROUP_BYTES + 2 * K_CHUNK_BYTES;      // chunk 8
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            const int rr = 4 * q4 + (lane >> 3);
                            const int rid = __shfl_sync(0xffffffffu, row_id, rr);
                            // (rows of 512 columns have no ninth chunk: zeros, as for an invalid token)
                            const __nv_bfloat16* src = p.kv + (int64_t)(rid < 0 ? 0 : rid) * p.kv_ss + (NO_CHUNK8 ? 0 : (64 + c) * 8);
                            cp_async16_zfill(dst0 + rr * 128 + ((c ^ (rr & 7)) << 4), src, (rid < 0 || NO_CHUNK8) ? 0u : 16u);
                        }
                    }
                    cp_async_arrive_noinc(smem_addr(&sm.kv_full[slot2]));
                    ks += 3;
                } else {
                    // warp gw owns tokens 16*gw .. 16*gw+15 of each page; one instruction copies 512 bytes of one row
                    for (int h = 0; h < 2; ++h) {
                        const int id = vid_next;
                        { const int posn = i * 128 + (h + 1) * 64 + gw * 16 + (lane & 15); vid_next = posn < w.seqlen ? __ldg(idx + posn) : -1; }
                        const int row_id = (id >= 0 && id < p.s_kv) ? id : -1;
                        for (int nh = 0; nh < 2; ++nh, ++ks) {
                            const uint32_t slot = ks % NVS;
                            WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_empty[slot], ((ks / NVS) & 1) ^ 1, 202);
                            const int box = lane >> 3, c = lane & 7;
                            const uint32_t dst0 = smem_addr(sm.data + VA_VRING + slot * V_SLOT_BYTES) + box * BOX_BYTES + gw * 16 * 128;
#pragma unroll 8
                            for (int rr = 0; rr < 16; ++rr) {
                                const int rid = __shfl_sync(0xffffffffu, row_id, rr);
                                const __nv_bfloat16* src = p.kv + (int64_t)(rid < 0 ? 0 : rid) * p.kv_ss + (nh * 32 + lane) * 8;
                                cp_async16_zfill(dst0 + rr * 128 + ((c ^ (rr & 7)) << 4), src, rid < 0 ? 0u : 16u);
                            }
                            cp_async_arrive_noinc(smem_addr(&sm.kv_full[slot]));
                        }
                    }
                }
            }
        }
    } else {
        if (!DENSE) asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
        const int wq = warp & 3;                                  // TMEM lane quarter of this warp
        const int half = (warp - 4) >> 2;                         // score CTA: page of the tile this warpgroup owns
        const int r = wq * 32 + lane;                             // row inside the block = TMEM lane
        const uint32_t tlane = tmem + ((uint32_t)(wq * 32) << 16);
        const int row = row_blk * ROWS + r;                       // row inside the (request, kv head) group
        const bool row_ok = row < p.rows;
        // dense: rows are (query token, head of the kv group); sparse decode: the CTA pair serves one query token
        const int t = MODE == MODE_SPARSE_DECODE ? (int)blockIdx.y : (row_ok ? row / p.g : 0);
        const int hd = MODE == MODE_SPARSE_DECODE ? (row_ok ? row : 0) : hk * p.g + (row_ok ? row - t * p.g : 0);
        uint32_t g = 0, nreq = 0;

        if (cta_rank == 0) {
            // ---------------- softmax warpgroups of the score CTA --------------------------------------------
            // These 256 threads meet at a named barrier every tile, so none of them may leave alone: a thread whose
            // wait ran out keeps walking (its later waits return at once, it arrives nowhere and stores nothing
            // outside its own staging) until the next such barrier, which carries the flag to everyone (bar.red.or);
            // behind it all 256 leave together.
            uint8_t* stage = sm.data + L::SC_STAGE + (half * 4 + wq) * 4096;
            float* side_src = reinterpret_cast<float*>(sm.data + L::SC_SIDE + wq * SIDE_BYTES);
            float* xmax = reinterpret_cast<float*>(sm.data + L::SC_XMAX);
            const uint32_t remote_fin = map_to_cta(smem_addr(sm.data + VA_FIN), 1) + (uint32_t)r * 4u;
            const uint32_t remote_fin_full = map_to_cta(smem_addr(&sm.fin_full), 1);
            // FP8 decode: these 256 threads also de-quantise the K tiles in place (two threads per token row, every other
            // 16-value piece each), one tile ahead of the softmax they compute: tile g + 1 is converted before the scores
            // of tile g are awaited, so the MMA warp has the next tile while this warpgroup is busy with the softmax.
            uint32_t conv_tile = 0;
            WaiterT wt_fast(p.status, &sm.aborted, peer_flag, p.wait_limit);     // conversion sits on the MMA warp's critical path: no sleeping
            auto convert_tile = [&](const uint32_t tile) {
                const int sw = r & 7;
                float4 sc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int grp = 0; grp < 3; ++grp) {
                    if (!wt_fast.template wait<false>(&sm.raw_full[grp], tile & 1, 205)) { wt.aborted = true; return; }
                    // the tile's scales were stored (and fenced) by the gather warps before they issued its first copies
                    if (grp == 0) sc = reinterpret_cast<const float4*>(sm.data + L::SC_SCALES)[(tile & 1) * ROWS + r];
                    // group 2: chunks 6, 7 and the RoPE chunk (copied as it is); 512-wide form: chunk 6, the RoPE chunk and zeros
                    const int nconv = grp < 2 ? 3 : (M1 ? 1 : 2);
#pragma unroll 1
                    for (int cj = 0; cj < nconv; ++cj) {
                        const int j = grp * 3 + cj, sg = j >> 1;
                        uint8_t* rowp = sm.data + L::SC_KRING + j * K_CHUNK_BYTES + r * 128;
                        // one fp32 scale per two chunks, or one e8m0 exponent byte per chunk (byte j of the first two words)
                        const float scale = M1 ? e8m0_to_float((__float_as_uint(j < 4 ? sc.x : sc.y) >> (8 * (j & 3))) & 0xffu)
                                               : (sg == 0 ? sc.x : sg == 1 ? sc.y : sg == 2 ? sc.z : sc.w);
                        uint4 raw[2];
#pragma unroll
                        for (int k2 = 0; k2 < 2; ++k2) raw[k2] = *reinterpret_cast<const uint4*>(rowp + (((2 * (half + 2 * k2) + 1) ^ sw) << 4));
#pragma unroll
                        for (int k2 = 0; k2 < 2; ++k2) {
                            const int k = half + 2 * k2;
                            uint4 lo, hi;
                            dequant16(raw[k2], scale, lo, hi);
                            *reinterpret_cast<uint4*>(rowp + (((2 * k) ^ sw) << 4)) = lo;
                            *reinterpret_cast<uint4*>(rowp + (((2 * k + 1) ^ sw) << 4)) = hi;
                        }
                    }
                    if (M1 && grp == 2) {
                        // the ninth chunk of a 512-wide row does not exist: zeros (this thread's half of the token's row)
                        uint8_t* row8 = sm.data + L::SC_KRING + 8 * K_CHUNK_BYTES + r * 128;
#pragma unroll
                        for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(row8 + (((half * 4 + k) ^ sw) << 4)) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core's reads
                    mbar_arrive(smem_addr(&sm.kv_full[grp]));
                }
            };
            for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq) {
                const Work w = wk.get();
                // ---- Q row -> A operand: chunks [0, Q_TMEM_CHUNKS) to tensor memory (2 x 16 bit per 32-bit column), in the
                // gather modes chunks 7, 8 to shared memory (K-major, 128-byte swizzle).  Warpgroup 0 takes chunks
                // [0, Q_SPLIT) (and 7), warpgroup 1 the others (and 8).
                // Every MMA that read the previous request's Q has completed: this thread saw s_full of its last tile.
                {
                    const __nv_bfloat16* qrow = MODE == MODE_PREFILL
                        ? p.q + (int64_t)w.req * p.q_ss + (int64_t)hd * p.q_sh
                        : p.q + (int64_t)w.req * p.q_sb + (int64_t)t * p.q_ss + (int64_t)hd * p.q_sh;
                    const int c_begin = half ? L::Q_SPLIT : 0, c_end = half ? L::Q_TMEM_CHUNKS : L::Q_SPLIT;
                    if (p.q_tma) {
                        // Q arrived as TMA boxes: in the gather modes chunks 7 and 8 are in place; the others wait in the K
                        // ring as [row][128 B] with the 128-byte swizzle
                        wt.template wait<false>(&sm.q_landed, nreq & 1, 12);
#pragma unroll 1
                        for (int c = c_begin; c < c_end; ++c) {
                            const uint8_t* qsrc = sm.data + L::SC_KRING + c * 16384 + r * 128;
                            uint32_t v[32];
#pragma unroll
                            for (int ch = 0; ch < 8; ++ch) {
                                const uint4 x = *reinterpret_cast<const uint4*>(qsrc + ((ch ^ (r & 7)) << 4));
                                v[4 * ch] = x.x; v[4 * ch + 1] = x.y; v[4 * ch + 2] = x.z; v[4 * ch + 3] = x.w;
                            }
                            tmem_st32(tlane + L::TM_Q + c * 32, v);
                        }
                        tmem_wait_st();
                        if (!wt.aborted) mbar_arrive(smem_addr(&sm.ring_released));        // the producers may fill the ring with K now
                    } else {
                        load_q_by_threads<MODE>(sm, qrow, row_ok, half, r, tlane, NO_CHUNK8);
                    }
                    tmem_wait_st();
                    fence_proxy_async_smem();
                    tc_fence_before();
                    if (!wt.aborted) mbar_arrive(smem_addr(&sm.q_ready));
                }
                // first key position this row must NOT see (causal limit, and the end of this partition's range)
                const int limit = min(p.causal ? w.seqlen - (p.s_q - 1 - t) : w.seqlen, w.blk_end * PAGE);
                float m_run = -INFINITY, l_run = 0.f, m_true = -INFINITY;
                for (int i = 0; i < w.ntiles; ++i, ++g) {
                    const uint32_t sb = L::S_BUFS == 2 ? (g & 1) : 0;
                    const uint32_t ph = L::S_BUFS == 2 ? ((g >> 1) & 1) : (g & 1);
                    if (MODE == MODE_SPARSE_DECODE)
                        // one tile ahead, but never into the next request: its first tile can only be gathered after
                        // these threads have moved that request's Q out of the K ring
                        while (!wt.aborted && conv_tile <= g + 1 && conv_tile < g + (uint32_t)(w.ntiles - i)) convert_tile(conv_tile++);
                    wt.template wait<false>(&sm.s_full[sb], ph, 5);
                    tc_fence_after();
                    uint32_t s[64];
                    {
                        uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[0]);
                        uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[32]);
                        tmem_ld32(tlane + L::TM_S + sb * 128 + half * 64, lo);
                        tmem_ld32(tlane + L::TM_S + sb * 128 + half * 64 + 32, hi);
                    }
                    tmem_wait_ld();
                    tc_fence_before();
                    if (!wt.aborted) mbar_arrive(smem_addr(&sm.s_empty[sb]));          // the MMA warp may overwrite this S accumulator

                    if (!DENSE) {
                        // validity bits of the gathered tokens: token 32w + l of the tile is bit l of word w
                        const uint32_t* km = reinterpret_cast<const uint32_t*>(sm.data + L::SC_MASK) + (g & 3) * 4 + half * 2;
                        const uint32_t m0 = km[0], m1 = km[1];
                        if ((m0 & m1) != 0xffffffffu) {
#pragma unroll
                            for (int c = 0; c < 64; ++c)
                                if (!(((c < 32 ? m0 : m1) >> (c & 31)) & 1u)) s[c] = 0xff800000u;      // -inf
                        }
                    } else {
                        const int nvalid = limit - (w.blk_begin + 2 * i + half) * PAGE;   // columns [0, nvalid) are visible
                        if (nvalid < PAGE) {
#pragma unroll
                            for (int c = 0; c < 64; ++c)
                                if (c >= nvalid) s[c] = 0xff800000u;          // -inf
                        }
                    }
                    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 64; c += 2) {
                        mx0 = fmaxf(mx0, __uint_as_float(s[c]));
                        mx1 = fmaxf(mx1, __uint_as_float(s[c + 1]));
                    }
                    float mx = fmaxf(mx0, mx1);
                    // the row maximum over both pages of the tile; the barrier also carries the abort flag
                    xmax[((g & 1) * 2 + half) * ROWS + r] = mx;
                    BAR_OR_LEAVE(wt.aborted);
                    mx = fmaxf(mx, xmax[((g & 1) * 2 + (half ^ 1)) * ROWS + r]);
                    mx *= p.scale_log2;                                // scale > 0: max commutes with scaling
                    m_true = fmaxf(m_true, mx);
                    float factor = 1.f;
                    bool resc = false;
                    if (i == 0) {
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
                    for (int c = 0; c < 64; c += 2) {
                        const float e0 = ex2(fmaf(__uint_as_float(s[c]), p.scale_log2, neg_m));
                        const float e1 = ex2(fmaf(__uint_as_float(s[c + 1]), p.scale_log2, neg_m));
                        sum0 += e0; sum1 += e1;
                        pk[c >> 1] = pack16<FP16>(e0, e1);
                    }
                    l_run += sum0 + sum1;
                    const bool any_resc = __any_sync(0xffffffffu, resc);

                    // staging of this warp is free once the previous tile's copy has landed in the value CTA
                    wt.template wait<true>(&sm.stage_free[half], (g & 1) ^ 1, 8);
                    if (!wt.aborted) {
                        uint8_t* prow = stage + (lane >> 3) * 1024 + (lane & 7) * 128;
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch)
                            *reinterpret_cast<uint4*>(prow + ((ch ^ (lane & 7)) << 4)) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                        if (half == 0) {
                            side_src[lane] = factor;
                            if (lane == 0) reinterpret_cast<uint32_t*>(side_src)[32] = any_resc ? 1u : 0u;
                        }
                        fence_proxy_async_smem();                          // staging is read by the bulk-copy engine
                        mbar_arrive(smem_addr(&sm.stage_full[half]));      // the sender warp pushes it to the value CTA
                    }
                }
                // final statistics of this request for the epilogue in the value CTA: warpgroup 1 hands its row sums to
                // warpgroup 0, which sends sum, running maximum and true maximum.  (The wide plan has no spare shared memory:
                // the hand-over uses the row-maximum slots of the tile parity that is not in use.)
                {
                    float* lsum = L::WIDE ? xmax + ((g & 1) * 2) * ROWS : reinterpret_cast<float*>(sm.data + L::SC_LSUM);
                    if (half == 1) lsum[r] = l_run;
                    BAR_OR_LEAVE(wt.aborted);
                    if (half == 0) l_run += lsum[r];
                    BAR_OR_LEAVE(wt.aborted);
                }
                if (half == 0) {
                    wt.template wait<true>(&sm.fin_empty, (nreq & 1) ^ 1, 7);
                    if (!wt.aborted) {
                        st_cluster_f32(remote_fin, l_run);
                        st_cluster_f32(remote_fin + ROWS * 4, m_run);
                        st_cluster_f32(remote_fin + 2 * ROWS * 4, m_true);
                        mbar_arrive_remote(remote_fin_full);
                    }
                }
            }
        } else if (warp < 8) {
            // ---------------- correction / epilogue warpgroup of the value CTA ---------------------------------
            const uint32_t remote_fin_empty = map_to_cta(smem_addr(&sm.fin_empty), 0);
            const uint32_t remote_stage_free0 = map_to_cta(smem_addr(&sm.stage_free[0]), 0);
            const uint32_t remote_stage_free1 = map_to_cta(smem_addr(&sm.stage_free[1]), 0);
            const float* fin = reinterpret_cast<const float*>(sm.data + VA_FIN);
            uint32_t vs = 0;                                          // V ring slot counter
            // 16-bit output rows start on 32-byte boundaries: 256-bit stores may be used (decode modes; measured in one run
            // against 16-byte stores: dense 0.2134 -> 0.2088 ms, FP8 decode 0.1107 -> 0.1090 ms, prefill 3.348 -> 3.379 ms,
            // so prefill keeps the 16-byte stores)
            const bool wide_out = MODE != MODE_PREFILL && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0 &&
                                  ((p.o_sb | p.o_ss | p.o_sh) & 15) == 0;
            for (WalkerT wk(p, part); wk.valid(); wk.next(), ++nreq) {
                const Work w = wk.get();
                for (int i = 0; i < w.ntiles; ++i, ++g) {
                    for (int h = 0; h < 2; ++h, vs += 2) {
                        const uint32_t pb = (g & 1) * 2 + h, ph = (g >> 1) & 1;
                        WAIT_WARP_OR_LEAVE(wt, true, &sm.p_full[pb], ph, 107);
                        if (threadIdx.x == 128) {
                            mbar_arrive_remote_relaxed(h ? remote_stage_free1 : remote_stage_free0);   // the copy has landed
                        }
                        if (h == 0 && i > 0) {
                            const float* side = reinterpret_cast<const float*>(sm.data + VA_SIDE + ((g & 1) * 4 + wq) * SIDE_BYTES);
                            const bool need = reinterpret_cast<const uint32_t*>(side)[32] != 0;    // warp-uniform
                            if (need) {
                                // every earlier PV MMA has finished before O is touched
                                WAIT_WARP_OR_LEAVE(wt, false, &sm.pv_done[((g - 1) & 1) * 2 + 1], ((g - 1) >> 1) & 1, 108);
                                tc_fence_after();
                                rescale_o_rows(tlane, side[lane]);
                            }
                        }
                        // Tokens at or beyond the sequence length may hold anything (NaN included) in a real page:
                        // their probabilities are zero, so their V rows are zeroed to keep 0 * NaN out of O.
                        const int blk = w.blk_begin + 2 * i + h;
                        const int nvalid = w.seqlen - blk * PAGE;
                        if (DENSE && blk < w.blk_end && nvalid < PAGE) {
                            const int first = max(nvalid, 0);
                            for (int nh = 0; nh < 2; ++nh) {
                                const uint32_t slot = (vs + nh) % NVS;
                                WAIT_WARP_OR_LEAVE(wt, false, &sm.kv_full[slot], ((vs + nh) / NVS) & 1, 109);
                                zero_v_rows(sm.data + VA_VRING + slot * V_SLOT_BYTES, first);
                            }
                            fence_proxy_async_smem();
                        }
                        tc_fence_before();
                        mbar_arrive(smem_addr(&sm.corr_done[pb]));
                    }
                }
                // ---- epilogue -----------------------------------------------------------------------------------
                const bool has_tiles = w.ntiles > 0;
                if (has_tiles) WAIT_WARP_OR_LEAVE(wt, false, &sm.pv_done[((g - 1) & 1) * 2 + 1], ((g - 1) >> 1) & 1, 110);
                WAIT_WARP_OR_LEAVE(wt, true, &sm.fin_full, nreq & 1, 111);
                tc_fence_after();
                const float Lsum = fin[r], M = fin[ROWS + r];
                const bool empty = !(Lsum > 0.f) || !has_tiles;          // also catches NaN
                float scale = empty ? 0.f : 1.f / Lsum;
                if (!DENSE && !w.is_split && p.attn_sink && !empty && row_ok)
                    scale = 1.f / (Lsum + exp2f(p.attn_sink[hd] * kLog2e - M));
                if (!w.is_split) {
                    __nv_bfloat16* orow = MODE == MODE_PREFILL
                        ? p.out + ((int64_t)w.req * p.h_q + hd) * D_V
                        : p.out + (int64_t)w.req * p.o_sb + (int64_t)t * p.o_ss + (int64_t)hd * p.o_sh;
#pragma unroll 1
                    for (int c = 0; c < D_V / 32; ++c) {
                        uint32_t v[32];
                        if (has_tiles) { tmem_ld32(tlane + c * 32, v); tmem_wait_ld(); }
                        if (row_ok) {
                            uint32_t o[16];
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                o[e] = empty ? 0u : pack16<FP16>(__uint_as_float(v[2 * e]) * scale, __uint_as_float(v[2 * e + 1]) * scale);
                            if (wide_out) {                   // whole 32-byte sectors per store
                                st_global_v8(orow + c * 32, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
                                st_global_v8(orow + c * 32 + 16, o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]);
                            } else {
#pragma unroll
                                for (int k = 0; k < 4; ++k)
                                    *reinterpret_cast<uint4*>(orow + c * 32 + k * 8) = make_uint4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
                            }
                        }
                    }
                    if (row_ok) {
                        const float lse_nat = empty ? INFINITY : (log2f(Lsum) + M) * kLn2;
                        if (MODE == MODE_PREFILL) {
                            p.lse[(int64_t)w.req * p.h_q + hd] = lse_nat;
                            p.max_logits[(int64_t)w.req * p.h_q + hd] = empty ? -INFINITY : fin[2 * ROWS + r] * kLn2;
                        } else {
                            p.lse[w.req * p.l_sb + t * p.l_ss + hd * p.l_sh] = lse_nat;
                        }
                    }
                } else if (DENSE && MLA_TAIL_BULK && w.last && has_tiles) {
                    // The partition's last partial: the V ring is idle by now, so every thread stages its row there, half a
                    // row (1 KiB) at a time, and hands it to the bulk-copy engine as one piece.  Stores by the thread itself
                    // (one lane per row, 32 bytes per instruction) keep the load/store unit busy for 8 us per 256 KiB.
                    const int64_t arow = ((int64_t)w.slot * p.s_q + t) * p.h_q + hd;
                    float* orow = p.o_accum + arow * D_V;
                    uint8_t* rowbuf = sm.data + VA_VRING + r * 1040;          // 1040: rows 16 bytes apart in the banks
#pragma unroll 1
                    for (int hf = 0; hf < 2; ++hf) {
                        if (hf) bulk_wait_group_read0();
#pragma unroll 1
                        for (int c = 0; c < 8; ++c) {
                            uint32_t v[32];
                            tmem_ld32(tlane + hf * 256 + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                *reinterpret_cast<uint4*>(rowbuf + c * 128 + k * 16) =
                                    make_uint4(empty ? 0u : __float_as_uint(__uint_as_float(v[4 * k]) * scale),
                                               empty ? 0u : __float_as_uint(__uint_as_float(v[4 * k + 1]) * scale),
                                               empty ? 0u : __float_as_uint(__uint_as_float(v[4 * k + 2]) * scale),
                                               empty ? 0u : __float_as_uint(__uint_as_float(v[4 * k + 3]) * scale));
                        }
                        fence_proxy_async_smem();
                        if (row_ok) bulk_store_to_global(orow + hf * 256, smem_addr(rowbuf), 1024);
                        bulk_commit_group();
                    }
                    if (row_ok) p.lse_accum[arow] = empty ? -INFINITY : log2f(Lsum) + M;
                    bulk_wait_group0();
                } else {
                    const int64_t arow = ((int64_t)w.slot * p.s_q + t) * p.h_q + hd;
                    float* orow = p.o_accum + arow * D_V;
#pragma unroll 1
                    for (int c = 0; c < D_V / 32; ++c) {
                        uint32_t v[32];
                        if (has_tiles) { tmem_ld32(tlane + c * 32, v); tmem_wait_ld(); }
                        if (row_ok) {
                            // whole 32-byte sectors per store: each thread writes its own row, so a 16-byte store would
                            // send half-filled sectors and twice the instructions through the load/store unit
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                uint32_t o[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) o[e] = empty ? 0u : __float_as_uint(__uint_as_float(v[8 * k + e]) * scale);
                                st_global_v8(orow + c * 32 + k * 8, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
                            }
                        }
                    }
                    if (row_ok) p.lse_accum[arow] = empty ? -INFINITY : log2f(Lsum) + M;
                }
                tc_fence_before();
                mbar_arrive_remote(remote_fin_empty);        // the final statistics may be rewritten
            }
        } else if (MODE == MODE_SPARSE_DECODE) {
            // ---------------- value CTA, FP8 decode: warps 8-11 de-quantise the V slots in place ------------------
            // Thread = (token row of the page, half of the slot's four chunks).  It looks up its token's record by
            // itself, one page ahead, for the two scales it needs; the raw pieces were copied by the gather warpgroup.
            const int trow = r & 63, hb = r >> 6, sw = trow & 7;
            const int tq = blockIdx.y;
            uint32_t ks = 0;
            WaiterT wt_fast(p.status, &sm.aborted, peer_flag, p.wait_limit);   // this sits on the MMA warp's critical path: no sleeping
            for (WalkerT wk(p, part); wk.valid(); wk.next()) {
                const Work w = wk.get();
                const int* idx0 = p.sidx[0] + (int64_t)w.req * p.sidx_sb[0] + (int64_t)tq * p.sidx_ss[0];
                const int* idx1 = p.stopk[1] ? p.sidx[1] + (int64_t)w.req * p.sidx_sb[1] + (int64_t)tq * p.sidx_ss[1] : nullptr;
                auto load_id = [&](int blk) -> int {
                    if (blk >= w.blk_end) return -1;
                    const int scope = blk >= w.nblk0 ? 1 : 0;
                    const int pos = (scope ? blk - w.nblk0 : blk) * PAGE + trow;
                    if (pos >= (scope ? w.len1 : w.len0)) return -1;
                    return __ldg((scope ? idx1 : idx0) + pos);
                };
                auto scales_of_id = [&](int blk, int id) -> float4 {
                    const int scope = blk >= w.nblk0 ? 1 : 0;
                    const int pbs = p.pbs[scope];
                    if (id < 0 || (int64_t)id >= (int64_t)p.nblocks[scope] * pbs) return make_float4(0.f, 0.f, 0.f, 0.f);
                    if (M1) {
                        const uint2 e = __ldg(reinterpret_cast<const uint2*>(p.kvb[scope] + (int64_t)(id / pbs) * p.kvb_sblock[scope] +
                                                                             (int64_t)pbs * 576 + (int64_t)(id % pbs) * 8));
                        return make_float4(__uint_as_float(e.x), __uint_as_float(e.y), 0.f, 0.f);
                    }
                    return __ldg(reinterpret_cast<const float4*>(p.kvb[scope] + (int64_t)(id / pbs) * p.kvb_sblock[scope] +
                                                                 (int64_t)(id % pbs) * 656 + 512));
                };
                float4 sc_next = scales_of_id(w.blk_begin, load_id(w.blk_begin));
                int id_next = load_id(w.blk_begin + 1);
                for (int i = 0; i < w.ntiles; ++i) {
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        const float4 sc = sc_next;
                        const int nblk = w.blk_begin + 2 * i + h + 1;
                        sc_next = scales_of_id(nblk, id_next);
                        id_next = load_id(nblk + 1);
#pragma unroll 1
                        for (int nh = 0; nh < 2; ++nh, ++ks) {
                            const uint32_t slot = ks % NVS;
                            WAIT_WARP_OR_LEAVE(wt_fast, false, &sm.raw_full[slot], (ks / NVS) & 1, 206);
                            float scale = hb ? (nh ? sc.w : sc.y) : (nh ? sc.z : sc.x);
                            // (512-wide form: one exponent byte per chunk; chunk 7 is the RoPE part, copied as it is)
                            const int nconv = (M1 && nh == 1 && hb == 1) ? 1 : 2;
#pragma unroll 1
                            for (int cj = 0; cj < nconv; ++cj) {
                                if (M1) {
                                    const int c = nh * 4 + hb * 2 + cj;
                                    scale = e8m0_to_float((__float_as_uint(c < 4 ? sc.x : sc.y) >> (8 * (c & 3))) & 0xffu);
                                }
                                uint8_t* rowp = sm.data + VA_VRING + slot * V_SLOT_BYTES + (hb * 2 + cj) * BOX_BYTES + trow * 128;
                                uint4 raw[4];
#pragma unroll
                                for (int k = 0; k < 4; ++k) raw[k] = *reinterpret_cast<const uint4*>(rowp + (((2 * k + 1) ^ sw) << 4));
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    uint4 lo, hi;
                                    dequant16(raw[k], scale, lo, hi);
                                    *reinterpret_cast<uint4*>(rowp + (((2 * k) ^ sw) << 4)) = lo;
                                    *reinterpret_cast<uint4*>(rowp + (((2 * k + 1) ^ sw) << 4)) = hi;
                                }
                            }
                            fence_proxy_async_smem();              // generic-proxy stores -> visible to the tensor core's reads
                            mbar_arrive(smem_addr(&sm.kv_full[slot]));
                        }
                    }
                }
            }
        }
    }

wind_down:
    // ---- wind down: both CTAs leave together, tensor memory is released -----------------------------------
    if (!DENSE && warp >= 12) cp_async_wait_all();          // this thread's own row copies have landed
    tc_fence_before();
    if (__syncthreads_or((int)*reinterpret_cast<volatile uint32_t*>(&sm.aborted))) {
        // A bounded wait ran out in this CTA or in its peer; every thread of this CTA has left its role and issues
        // nothing more.  Wait - bounded again - for what this CTA still has in flight: its MMAs (they read shared memory
        // and write tensor memory) and the TMA loads into its rings.
        if (warp == 1 && lane == 0) {
            tc_commit(smem_addr(&sm.drain));
            mbar_wait_bounded<false, 0>(smem_addr(&sm.drain), 0, DRAIN_LIMIT);
        }
        if (threadIdx.x == 0) {
            if (DENSE) {
                const uint32_t nslots = cta_rank == 0 ? (uint32_t)NKS : (uint32_t)NVS;
                for (uint32_t back = 1; back <= nslots && back <= fills_armed; ++back) {
                    const uint32_t f = fills_armed - back;     // one of the last fills this thread armed: its slot has seen no later phase
                    mbar_wait_bounded<false, 0>(smem_addr(&sm.kv_full[f % nslots]), (f / nslots) & 1, DRAIN_LIMIT);
                }
            }
            if (q_armed) mbar_wait_bounded<false, 0>(smem_addr(&sm.q_landed), (q_armed - 1) & 1, DRAIN_LIMIT);
        }
    }
    cluster_sync();                                            // from here on neither CTA starts anything
    if (__syncthreads_or((int)*reinterpret_cast<volatile uint32_t*>(&sm.aborted))) {
        // copies from the peer's shared memory into this one (P pages, final statistics) that were still under way
        const long long t0 = clock64();
        while (clock64() - t0 < SETTLE_CYCLES) { }
    }
    cluster_sync();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---- self-test of the bounded wait: one CTA, one barrier nobody arrives on ---------------------------------
// Uses the same Waiter and the same reporting as the attention kernels, with nothing in flight (no TMA, no MMA, no
// cluster): the wait runs into `limit_cycles`, the status words are written, the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles, int code, int* flag_out) {
    __shared__ uint64_t bar;
    __shared__ uint32_t flag;
    if (threadIdx.x == 0) { mbar_init(smem_addr(&bar), 1); flag = 0; fence_mbar_init(); }
    __syncthreads();
    Waiter<true> lean(status, &flag, 0u, limit_cycles);
    Waiter<false> spin(status, &flag, 0u, limit_cycles);
    bool ok = true;
    if (threadIdx.x < 32) ok = lean.wait<false>(&bar, 0, code);
    else ok = spin.wait<false>(&bar, 0, code);
    // a second wait by the same thread returns at once
    if (threadIdx.x < 32) ok = lean.wait<false>(&bar, 0, code + 1) || ok;
    __syncthreads();
    if (threadIdx.x == 0 && flag_out) { flag_out[0] = (int)flag; flag_out[1] = ok ? 1 : 0; }
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

// Barrier-wait limit in SM cycles: the default, or MLA_WAIT_LIMIT_CYCLES from the environment (read once).
static long long wait_limit_cycles() {
    static const long long v = [] {
        const char* e = getenv("MLA_WAIT_LIMIT_CYCLES");
        const long long x = e ? atoll(e) : 0;
        return x > 0 ? x : WAIT_LIMIT_DEFAULT;
    }();
    return v;
}

// cudaFuncSetAttribute(max dynamic shared memory) once per kernel instance and device
template <typename K>
static int configure_once(K kernel, bool (&done)[64]) {
    static std::mutex mu;
    int dev = 0;
    MLA_CHECK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !done[dev]) {
        MLA_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
        if (dev >= 0 && dev < 64) done[dev] = true;
    }
    return MLA_OK;
}

}  // namespace sm100

int launch_bounded_wait_selftest(long long limit_cycles, int code, int* status, int* flag_out, void* stream) {
    MLA_CHECK_ARG(limit_cycles > 0 && limit_cycles <= 2000000000LL, "mla_selftest_bounded_wait: limit_cycles must be in (0, 2e9]");
    MLA_CHECK_ARG(status != nullptr, "mla_selftest_bounded_wait: status must not be null");
    sm100::bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, limit_cycles, code, flag_out);
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

bool dense_decode_sm100_supports(const mla_dense_decode_args_t& a) {
    if (a.d_qk != 576 || a.d_v != 512 || a.page_block_size != 64) return false;
    if (a.h_kv <= 0 || a.h_q % a.h_kv != 0) return false;
    // TMA: strides in bytes must be multiples of 16 and below 2^40
    const int64_t lim = (int64_t)1 << 39;
    if (a.k_stride_block <= 0 || a.k_stride_row <= 0 || a.k_stride_head <= 0) return false;
    if (a.k_stride_block >= lim || a.k_stride_row >= lim || a.k_stride_head >= lim) return false;
    if (a.k_stride_block % 8 || a.k_stride_row % 8 || a.k_stride_head % 8) return false;
    // the kv heads of a row are addressed as 64-column chunks of one tensor-map dimension
    if (a.h_kv > 1 && a.k_stride_head % 64) return false;
    const int rows = a.s_q * (a.h_q / a.h_kv);
    const int64_t row_blocks = (rows + 127) / 128;
    if (row_blocks * a.h_kv > 65535 || a.num_sm_parts > 65535) return false;
    if (!(a.softmax_scale > 0.f)) return false;       // the row maximum is taken before scaling
    if (reinterpret_cast<uintptr_t>(a.o_accum) & 31) return false;      // split partials leave with 256-bit stores
    return true;
}

// Tensor map over Q as (576 columns, heads, query tokens, requests) with boxes of 64 columns x box_h heads x box_t
// tokens.  Returns false (the kernels then load every Q with their own threads) when Q's base or strides do not meet
// TMA's 16-byte rules or the driver rejects the map.
static bool encode_q_map(CUtensorMap* qmap, const void* q, int b, int s_q, int h_q, int64_t sb, int64_t ss, int64_t sh,
                         int box_h, int box_t, int* box_bytes, bool fp16 = false, int d_qk = 576) {
    using namespace sm100;
    static const bool enabled = [] { const char* e = getenv("MLA_Q_TMA"); return !(e && e[0] == '0'); }();
    EncodeTiledFn encode = get_encode_fn();
    if (!enabled || !encode || !q) return false;
    if (h_q <= 1) sh = 576;                         // a dimension of extent 1 never strides: give it a legal value
    if (s_q <= 1) ss = sh * h_q;
    if (b <= 1) sb = ss * s_q;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || sb <= 0 || ss <= 0 || sh <= 0 || (sb % 8) || (ss % 8) || (sh % 8)) return false;
    if (sb * 2 >= (1ll << 40) || ss * 2 >= (1ll << 40) || sh * 2 >= (1ll << 40)) return false;
    if (box_h < 1 || box_h > 256 || box_t < 1 || box_t > 256 || box_h * box_t > ROWS) return false;
    // (512-wide rows: the ninth box of a request lies wholly outside the tensor and arrives as zeros)
    cuuint64_t dims[4] = {(cuuint64_t)d_qk, (cuuint64_t)h_q, (cuuint64_t)s_q, (cuuint64_t)b};
    cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_h, (cuuint32_t)box_t, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = encode(qmap, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(q),
                              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    *box_bytes = 128 * box_h * box_t;
    return true;
}

// The two cache tensor maps of a dense launch depend only on the cache tensor (pointer, strides, pages, heads, type):
// a decode loop calls with the same cache every step, so the last encoding is kept per host thread.
struct CacheMaps {
    const void* k_cache = nullptr;
    int64_t sb = 0, sr = 0, sh = 0;
    int num_blocks = 0, h_kv = 0, fp16 = 0;
    CUtensorMap kmap, vmap;
};

int launch_dense_decode_sm100(const mla_dense_decode_args_t& a) {
    using namespace sm100;
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return set_error(MLA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const bool fp16 = a.dtype == MLA_DTYPE_FP16;

    // The cache as a 5-D tensor (64 columns of a chunk, 8 tokens, chunks, 8 token groups, pages): one box brings
    // all 64 tokens of a page for 3 (K) or 4 (V) chunks in a single instruction, and lands as
    // [token group][chunk][8 rows x 128 B] - 1 KiB swizzle atoms that the MMA descriptors walk with a stride of
    // 3 or 4 KiB between token groups.  (The per-instruction cost of TMA is what limits one SM's fill rate: 8 KiB
    // boxes stream at 35-45 GB/s per SM, 24 KiB boxes at about 90.)
    const int head_chunks = a.h_kv > 1 ? (int)(a.k_stride_head / 64) : 9;
    static thread_local CacheMaps cm;
    if (cm.k_cache != a.k_cache || cm.sb != a.k_stride_block || cm.sr != a.k_stride_row || cm.sh != a.k_stride_head ||
        cm.num_blocks != a.num_blocks || cm.h_kv != a.h_kv || cm.fp16 != (int)fp16) {
        cm.k_cache = nullptr;
        const CUtensorMapDataType dt = fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        cuuint64_t dims[5] = {64, 8, (cuuint64_t)((a.h_kv - 1) * head_chunks + 9), 8, (cuuint64_t)a.num_blocks};
        cuuint64_t strides[4] = {(cuuint64_t)a.k_stride_row * 2, 128, (cuuint64_t)a.k_stride_row * 16, (cuuint64_t)a.k_stride_block * 2};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        cuuint32_t kbox[5] = {64, 8, 3, 8, 1};
        cuuint32_t vbox[5] = {64, 8, 4, 8, 1};
        CUresult r = encode(&cm.kmap, dt, 5, const_cast<void*>(a.k_cache), dims, strides, kbox, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS)
            r = encode(&cm.vmap, dt, 5, const_cast<void*>(a.k_cache), dims, strides, vbox, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(MLA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
        cm.k_cache = a.k_cache; cm.sb = a.k_stride_block; cm.sr = a.k_stride_row; cm.sh = a.k_stride_head;
        cm.num_blocks = a.num_blocks; cm.h_kv = a.h_kv; cm.fp16 = (int)fp16;
    }

    Params p = {};
    p.b = a.b; p.s_q = a.s_q; p.h_q = a.h_q; p.h_kv = a.h_kv; p.g = a.h_q / a.h_kv;
    p.rows = a.s_q * p.g;
    p.causal = (a.is_causal && a.s_q > 1) ? 1 : 0;
    p.scale_log2 = a.softmax_scale * kLog2e;
    p.wait_limit = wait_limit_cycles();
    p.q = (const __nv_bfloat16*)a.q; p.q_sb = a.q_stride_b; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.o_sb = a.o_stride_b; p.o_ss = a.o_stride_s; p.o_sh = a.o_stride_h;
    p.lse = a.lse; p.l_sb = a.lse_stride_b; p.l_ss = a.lse_stride_s; p.l_sh = a.lse_stride_h;
    p.block_table = a.block_table; p.bt_sb = a.block_table_stride_b; p.seqlens = a.seqlens_k;
    p.max_blocks = a.max_blocks_per_seq;
    p.meta = a.meta; p.num_splits = a.num_splits; p.lse_accum = a.lse_accum; p.o_accum = a.o_accum;
    p.status = a.status;
    p.row_blocks = (p.rows + ROWS - 1) / ROWS;
    p.num_blocks = a.num_blocks;
    p.head_chunks = head_chunks;
    CUtensorMap qmap;
    memset(&qmap, 0, sizeof(qmap));
    if (p.row_blocks == 1 || ROWS % p.g == 0)
        p.q_tma = encode_q_map(&qmap, a.q, a.b, a.s_q, a.h_q, a.q_stride_b, a.q_stride_s, a.q_stride_h, p.g,
                               p.row_blocks == 1 ? a.s_q : ROWS / p.g, &p.q_box_bytes, fp16) ? 1 : 0;

    dim3 grid(2, p.row_blocks * a.h_kv, a.num_sm_parts);
    if (fp16) {
        static bool configured[64] = {};
        if (int rc = configure_once(attn_sm100_kernel<MODE_DENSE, true>, configured)) return rc;
        MLA_CHECK_CUDA(launch_dependent(attn_sm100_kernel<MODE_DENSE, true>, grid, dim3(NTHREADS), sizeof(Smem), (cudaStream_t)a.stream, cm.kmap, cm.vmap, qmap, p));
    } else {
        static bool configured[64] = {};
        if (int rc = configure_once(attn_sm100_kernel<MODE_DENSE, false>, configured)) return rc;
        MLA_CHECK_CUDA(launch_dependent(attn_sm100_kernel<MODE_DENSE, false>, grid, dim3(NTHREADS), sizeof(Smem), (cudaStream_t)a.stream, cm.kmap, cm.vmap, qmap, p));
    }
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

bool sparse_prefill_sm100_supports(const mla_sparse_prefill_args_t& a) {
    if ((a.d_qk != 576 && a.d_qk != 512) || a.d_v != 512 || a.h_kv != 1) return false;
    if (a.kv_stride_s <= 0 || a.kv_stride_s % 8 || a.kv_stride_s >= ((int64_t)1 << 39)) return false;
    if (!(a.sm_scale > 0.f)) return false;
    if (a.h_q > 128 * 65535) return false;
    return true;
}

int launch_sparse_prefill_sm100(const mla_sparse_prefill_args_t& a) {
    using namespace sm100;
    CUtensorMap kmap;
    memset(&kmap, 0, sizeof(kmap));     // rows are gathered with cp.async by the kernel's own threads, no TMA descriptor

    Params p = {};
    p.b = a.s_q; p.s_q = 1; p.h_q = a.h_q; p.h_kv = 1; p.g = a.h_q; p.rows = a.h_q;
    p.causal = 0;
    p.scale_log2 = a.sm_scale * kLog2e;
    p.wait_limit = wait_limit_cycles();
    p.q = (const __nv_bfloat16*)a.q; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.lse = a.lse; p.max_logits = a.max_logits;
    p.attn_sink = a.attn_sink;
    p.indices = a.indices; p.idx_ss = a.indices_stride_s; p.topk = a.topk; p.topk_len = a.topk_length; p.s_kv = a.s_kv;
    p.kv = (const __nv_bfloat16*)a.kv; p.kv_ss = a.kv_stride_s;
    p.status = a.status;
    p.row_blocks = (p.rows + ROWS - 1) / ROWS;

    const bool d512 = a.d_qk == 512;
    static bool configured[64] = {}, configured_512[64] = {};
    if (int rc = d512 ? configure_once(attn_sm100_kernel<MODE_PREFILL, true>, configured_512)
                      : configure_once(attn_sm100_kernel<MODE_PREFILL, false>, configured)) return rc;
    const int sms = current_device_num_sms();
    int pairs = sms / 2 / p.row_blocks;
    if (pairs < 1) pairs = 1;
    if (pairs > a.s_q) pairs = a.s_q;
    dim3 grid(2, p.row_blocks, pairs);
    CUtensorMap qmap;
    memset(&qmap, 0, sizeof(qmap));
    p.q_tma = encode_q_map(&qmap, a.q, 1, a.s_q, a.h_q, 0, a.q_stride_s, a.q_stride_h, a.h_q < ROWS ? a.h_q : ROWS, 1,
                           &p.q_box_bytes, false, a.d_qk) ? 1 : 0;
    if (d512)
        MLA_CHECK_CUDA(launch_dependent(attn_sm100_kernel<MODE_PREFILL, true>, grid, dim3(NTHREADS_GATHER), sizeof(Smem), (cudaStream_t)a.stream, kmap, kmap, qmap, p));
    else
        MLA_CHECK_CUDA(launch_dependent(attn_sm100_kernel<MODE_PREFILL, false>, grid, dim3(NTHREADS_GATHER), sizeof(Smem), (cudaStream_t)a.stream, kmap, kmap, qmap, p));
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

bool sparse_decode_sm100_supports(const mla_sparse_decode_args_t& a) {
    if ((a.d_qk != 576 && a.d_qk != 512) || a.d_v != 512) return false;
    if (a.h_q > 128 || a.s_q > 65535 || a.num_sm_parts > 65535) return false;
    if (!(a.sm_scale > 0.f)) return false;
    if (reinterpret_cast<uintptr_t>(a.o_accum) & 31) return false;      // split partials leave with 256-bit stores
    return true;
}

int launch_sparse_decode_sm100(const mla_sparse_decode_args_t& a) {
    using namespace sm100;
    Params p = {};
    p.b = a.b; p.s_q = a.s_q; p.h_q = a.h_q; p.h_kv = 1; p.g = a.h_q; p.rows = a.h_q;
    p.causal = 0;
    p.scale_log2 = a.sm_scale * kLog2e;
    p.wait_limit = wait_limit_cycles();
    p.q = (const __nv_bfloat16*)a.q; p.q_sb = a.q_stride_b; p.q_ss = a.q_stride_s; p.q_sh = a.q_stride_h;
    p.out = (__nv_bfloat16*)a.out; p.o_sb = a.o_stride_b; p.o_ss = a.o_stride_s; p.o_sh = a.o_stride_h;
    p.lse = a.lse; p.l_sb = a.lse_stride_b; p.l_ss = a.lse_stride_s; p.l_sh = a.lse_stride_h;
    p.attn_sink = a.attn_sink;
    p.meta = a.meta; p.num_splits = a.num_splits; p.lse_accum = a.lse_accum; p.o_accum = a.o_accum;
    p.status = a.status;
    p.row_blocks = 1;
    p.kvb[0] = (const uint8_t*)a.kv; p.kvb_sblock[0] = a.kv_stride_block_bytes; p.pbs[0] = a.page_block_size; p.nblocks[0] = a.num_blocks;
    p.sidx[0] = a.indices; p.sidx_sb[0] = a.indices_stride_b; p.sidx_ss[0] = a.indices_stride_s; p.stopk[0] = a.topk;
    p.stopk_len[0] = a.topk_length;
    p.kvb[1] = (const uint8_t*)a.extra_kv; p.kvb_sblock[1] = a.extra_kv_stride_block_bytes;
    p.pbs[1] = a.extra_page_block_size > 0 ? a.extra_page_block_size : 1; p.nblocks[1] = a.extra_num_blocks;
    p.sidx[1] = a.extra_indices; p.sidx_sb[1] = a.extra_indices_stride_b; p.sidx_ss[1] = a.extra_indices_stride_s;
    p.stopk[1] = a.extra_kv ? a.extra_topk : 0; p.stopk_len[1] = a.extra_topk_length;

    const bool m1 = a.d_qk == 512;                  // the 512-wide record form: the ninth chunk of Q and K is zeros
    static bool configured[64] = {}, configured_m1[64] = {};
    if (int rc = m1 ? configure_once(attn_sm100_kernel<MODE_SPARSE_DECODE, true>, configured_m1)
                    : configure_once(attn_sm100_kernel<MODE_SPARSE_DECODE, false>, configured)) return rc;
    CUtensorMap unused_map, qmap;
    memset(&unused_map, 0, sizeof(unused_map));     // this mode gathers K and V with its own threads
    memset(&qmap, 0, sizeof(qmap));
    p.q_tma = encode_q_map(&qmap, a.q, a.b, a.s_q, a.h_q, a.q_stride_b, a.q_stride_s, a.q_stride_h,
                           a.h_q < ROWS ? a.h_q : ROWS, 1, &p.q_box_bytes, false, a.d_qk) ? 1 : 0;
    dim3 grid(2, a.s_q, a.num_sm_parts);
    if (m1)
        MLA_CHECK_CUDA(launch_dependent(attn_sm100_kernel<MODE_SPARSE_DECODE, true>, grid, dim3(NTHREADS_GATHER), sizeof(Smem), (cudaStream_t)a.stream, unused_map, unused_map, qmap, p));
    else
        MLA_CHECK_CUDA(launch_dependent(attn_sm100_kernel<MODE_SPARSE_DECODE, false>, grid, dim3(NTHREADS_GATHER), sizeof(Smem), (cudaStream_t)a.stream, unused_map, unused_map, qmap, p));
    MLA_CHECK_CUDA(cudaGetLastError());
    return MLA_OK;
}

}  // namespace mla
