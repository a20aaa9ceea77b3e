// The written-out backward at head dimension 256 on the 5th-generation tensor cores (bf16 / f16).
//
// At D = 256 a tile of 128 rows is 64 KiB and an f32 accumulator of 128 rows is 256 columns of tensor
// memory, so neither the four tiles a step of the D = 128 kernels keeps in shared memory nor their
// two accumulators beside two score tiles fit (bwd_sm100.cu).  Here every pass keeps ONE accumulator
// of 256 columns beside the score tiles, keeps its block's own rows resident (64 KiB a tensor) and
// streams the other side through a ring of HALF tiles - 128 rows x 128 of the 256 features, 32 KiB -
// which is all a k-step ever needs at once: a score product sums over the features, eight k-steps
// from the low half and eight from the high one, and a gradient product writes the low and the high
// 128 columns of the accumulator from the low and the high half.  A half that serves twice in a step
// (the score product and the gradient product) is fetched twice, from L2.  Every MMA is 128 x 128 x 16.
//
// One kernel body, three passes (deterministic: no atomics, fixed order of summation):
//   DQ   block = (128 queries, query head), Q and dO resident, K and V streamed in steps of 128 keys:
//        S = Q K^T, dP = dO V^T, dS = P (dP - delta) written over dP in the input dtype, dQ += dS K.
//   DK   block = (128 keys, key-value head), K and V resident, Q and dO streamed over the group's heads
//        and the queries that may see the block: S^T = K Q^T, dP^T = V dO^T, dS^T likewise, dK += dS^T Q.
//   DV   the same block and sweep, K resident only: S^T = K Q^T, P^T over S^T, dV += P^T dO; with the
//        columns dP^T does not use the score tile is double.
// DK is DQ with the roles of the two sides exchanged (the per-query log-sum-exp and delta then belong
// to the columns of a step instead of the rows); DK and DV run as one launch.  Eight products per pair
// of tiles where five are counted.  Warp roles as in bwd_sm100.cu: warp 0 issues the TMA loads in the
// order warp 1 - which owns tensor memory and issues the MMAs - consumes them, 16 elementwise warps
// (a row and 32 of a step's columns per thread), one warp that gathers a step's per-column vectors a
// step ahead.  Every mbarrier wait is bounded (sm100_ptx.cuh).
#include <cuda.h>

#include "bwd_common.cuh"
#include "common.cuh"
#include "sm100.h"
#include "sm100_kernels.h"
#include "sm100_ptx.cuh"

namespace dash {

using namespace ptx;

__device__ unsigned int g_sm100_bwd256_status = 0;  // sticky: non-zero once a bounded wait has run out

namespace {

constexpr int HD = 256;
constexpr int ROWS = 128;                    // rows of a tile, resident or streamed (and TMEM lanes)
constexpr int BOX = ROWS * 128;              // a TMA box: 128 rows of 64 features (128 bytes)
constexpr int HALF_TILE = 2 * BOX;           // 128 rows x 128 features: what the ring holds, 32 KiB
constexpr int FULL_TILE = 4 * BOX;           // 128 rows x 256 features: a resident tile, 64 KiB
constexpr int CG = 4;                        // elementwise warps per TMEM lane quadrant
constexpr int CW = ROWS / CG;                // columns of a step per elementwise thread
constexpr int EW_WARPS = 4 * CG;
constexpr int AUX_WARP = 2 + EW_WARPS;
constexpr int THREADS = 32 * (3 + EW_WARPS);
constexpr int MAX_SLOTS = 4;
constexpr float LOG2E = 1.4426950408889634f;
static_assert(CW == 32, "one 32-column TMEM load per thread and phase");

enum Pass { PASS_DQ = 0, PASS_DK = 1, PASS_DV = 2 };

// Resident tiles and ring slots of a pass: DQ and DK keep two tensors and re-fetch one streamed
// half per step, DV keeps one and fetches every half once.
__host__ __device__ constexpr int resident_tiles(int pass) { return pass == PASS_DV ? 1 : 2; }
__host__ __device__ constexpr int ring_slots(int pass) { return pass == PASS_DV ? 4 : 3; }

struct Barriers {
    uint64_t res_full;
    uint64_t full[MAX_SLOTS], empty[MAX_SLOTS];   // the ring of half tiles
    uint64_t s_full[2], s_free, dp_full, a_full[2];  // scores ready; scores taken; dP ready; the A operand (dS or P) written
    uint64_t aux_full[2], aux_free[2];
    uint64_t acc_ready;
};

struct alignas(16) ColumnAux {   // per column of a step (DK, DV: the step's queries)
    float lse2[ROWS];            // log-sum-exp in base 2, +inf for a query that saw no key or is out of range
    float delta[ROWS];
};

struct Tail {
    Barriers bar;
    ColumnAux aux[2];
    uint32_t tmem_base;
    unsigned int abort;
    int red_lo[4], red_hi[4];
};
constexpr size_t TAIL_BYTES = 3072;
static_assert(sizeof(Tail) <= TAIL_BYTES, "the tail of the kernel's shared memory");

// resident tiles | ring | tail; no slack: the window must start on a 1 KiB boundary (checked).
__host__ __device__ constexpr size_t smem_bytes(int pass) {
    return (size_t)resident_tiles(pass) * FULL_TILE + (size_t)ring_slots(pass) * HALF_TILE + TAIL_BYTES;
}

}  // namespace

namespace {

// One block's pass.  `r1` / `r2` are the tensor maps of the resident tensors (r2 unused by DV),
// `s1` / `s2` those of the streamed ones: DQ (Q, dO | K, V), DK and DV (K, V | Q, dO).
template <typename T, int PASS>
__device__ __forceinline__ void bwd256_pass(const CUtensorMap *r1, const CUtensorMap *r2, const CUtensorMap *s1,
                                            const CUtensorMap *s2, const Sm100BwdArgs &a, uint8_t *smem, int b, int row0,
                                            int res_head) {
    constexpr int NRES = resident_tiles(PASS), NS = ring_slots(PASS);
    constexpr bool ROWS_ARE_QUERIES = PASS == PASS_DQ;
    uint8_t *r1_s = smem, *r2_s = smem + FULL_TILE;          // r2_s only with two resident tiles
    uint8_t *ring = smem + NRES * FULL_TILE;                 // [NS][HALF_TILE]
    Tail &sh = *reinterpret_cast<Tail *>(ring + NS * HALF_TILE);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = a.hq / a.hkv;
    auto BAR = [&](uint64_t &x) { return smem_u32(&x); };

    if (threadIdx.x == 0) {
        sh.abort = *reinterpret_cast<volatile unsigned int *>(&g_sm100_bwd256_status);
        if ((smem_u32(smem) & 1023u) != 0) sh.abort = 1u;   // the swizzled tiles need a 1 KiB boundary
        mbar_init(BAR(sh.bar.res_full), 1);
        for (int i = 0; i < MAX_SLOTS; ++i) {
            mbar_init(BAR(sh.bar.full[i]), 1);
            mbar_init(BAR(sh.bar.empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(sh.bar.s_full[i]), 1);
            mbar_init(BAR(sh.bar.a_full[i]), EW_WARPS);   // one arrival per elementwise warp
            mbar_init(BAR(sh.bar.aux_full[i]), 1);
            mbar_init(BAR(sh.bar.aux_free[i]), EW_WARPS);
        }
        mbar_init(BAR(sh.bar.s_free), EW_WARPS);
        mbar_init(BAR(sh.bar.dp_full), 1);
        mbar_init(BAR(sh.bar.acc_ready), 1);
        fence_mbar_init();
        prefetch_tensormap(r1);
        if (NRES > 1) prefetch_tensormap(r2);
        prefetch_tensormap(s1);
        prefetch_tensormap(s2);
        // The resident tiles are on their way before the block knows what it sweeps: their flight covers
        // the rest of the set-up.  (A block with nothing to do waits for them at the end: shared memory
        // must not be written behind a block that has left.)
        const uint32_t full = BAR(sh.bar.res_full);
        mbar_expect_tx(full, NRES * FULL_TILE);
#pragma unroll
        for (int box = 0; box < 4; ++box) {
            tma_load_4d(smem_u32(r1_s + box * BOX), r1, full, 64 * box, res_head, row0, b);
            if (NRES > 1) tma_load_4d(smem_u32(r2_s + box * BOX), r2, full, 64 * box, res_head, row0, b);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
    }

    // This thread's row and the columns it may see: DQ a query and its interval of keys, DK / DV a
    // key and the interval of queries that see it (empty for a padded key).
    const int lane_base = 32 * (warp & 3), r = lane_base + lane, row = row0 + r;
    int lo = 0, hi = 0;
    if (warp >= 2 && warp < AUX_WARP) {
        if (ROWS_ARE_QUERIES) {
            row_bounds(a.mask, row, a.tq, a.tk, lo, hi);
            if (hi <= lo) { lo = a.tk; hi = 0; }
            if (warp < 6) {   // the first four warps cover every row
                const int wlo = warp_min_i(lo), whi = warp_max_i(hi);
                if (lane == 0) { sh.red_lo[warp - 2] = wlo; sh.red_hi[warp - 2] = whi; }
            }
        } else if (row < a.tk && !key_padded(a.mask, b, row)) {
            queries_of_key(a.mask, row, a.tq, a.tk, lo, hi);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    const bool aborted = sh.abort != 0;
    // The sweep: DQ the key tiles of the union of the rows' intervals, for the rows' own key-value
    // head; DK / DV the query tiles that may see the block, for each query head of the group.
    int col_first = 0, tiles = 0, head0 = 0;
    if (ROWS_ARE_QUERIES) {
        int cmin = a.tk, cmax = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) { cmin = min(cmin, sh.red_lo[i]); cmax = max(cmax, sh.red_hi[i]); }
        col_first = cmin;
        tiles = cmax > cmin ? (cmax - cmin + ROWS - 1) / ROWS : 0;
        head0 = res_head / group;
    } else {
        int qfirst, qend;
        query_range(a.mask, row0, min(row0 + ROWS, a.tk), a.tq, a.tk, qfirst, qend);
        col_first = qfirst;
        tiles = qend > qfirst ? (qend - qfirst + ROWS - 1) / ROWS : 0;
        head0 = res_head * group;
    }
    const int steps = aborted ? 0 : (ROWS_ARE_QUERIES ? tiles : tiles * group);
    auto step_head = [&](int t) { return ROWS_ARE_QUERIES ? head0 : head0 + t / tiles; };
    auto step_col0 = [&](int t) { return col_first + (ROWS_ARE_QUERIES ? t : t % tiles) * ROWS; };
    bool failed = aborted;
    constexpr uint32_t COL_S = 0, COL_DP = 128, COL_ACC = 256;

    if (warp == 0) {
        // ---------------- producer: the half tiles in the order the MMA warp takes them ----------------
        if (lane == 0 && steps > 0) {
            int n = 0;   // halves loaded so far: slot n % NS, phase (n / NS) & 1
            auto load = [&](const CUtensorMap *map, int t, int half) -> bool {
                const int slot = n % NS, ph = (n / NS) & 1;
                if (!mbar_wait(BAR(sh.bar.empty[slot]), ph ^ 1)) return false;
                const uint32_t full = BAR(sh.bar.full[slot]), dst = smem_u32(ring + slot * HALF_TILE);
                mbar_expect_tx(full, HALF_TILE);
                tma_load_4d(dst, map, full, 128 * half, step_head(t), step_col0(t), b);
                tma_load_4d(dst + BOX, map, full, 128 * half + 64, step_head(t), step_col0(t), b);
                ++n;
                return true;
            };
            auto both = [&](const CUtensorMap *map, int t) { return load(map, t, 0) && load(map, t, 1); };
            bool ok = both(s1, 0) && (PASS == PASS_DV || both(s2, 0));
            for (int t = 0; t < steps && ok; ++t) {
                if (t + 1 < steps) ok = both(s1, t + 1);                               // the next scores
                if (ok) ok = both(PASS == PASS_DV ? s2 : s1, t);                       // this step's gradient product
                if (ok && PASS != PASS_DV && t + 1 < steps) ok = both(s2, t + 1);      // the next dP
            }
            if (!ok) failed = true;
        }
    } else if (warp == AUX_WARP) {
        // ---------------- DK / DV: the per-query vectors of each step, gathered a step ahead ----------------
        if (!ROWS_ARE_QUERIES) {
            constexpr int RPL = ROWS / 32;   // columns per lane
            float lse_n[RPL], dl_n[RPL];
            auto gather = [&](int t) {
                const int h = step_head(t), q0 = step_col0(t);
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    const int q = min(q0 + lane + 32 * i, a.tq - 1);
                    const int64_t at = ((int64_t)b * a.tq + q) * a.hq + h;
                    lse_n[i] = a.lse[at];
                    dl_n[i] = a.delta[at];
                }
            };
            if (steps > 0) gather(0);
            for (int t = 0; t < steps; ++t) {
                const int st = t & 1, ph = (t >> 1) & 1, q0 = step_col0(t);
                float l2v[RPL], dlv[RPL];
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    const bool in = q0 + lane + 32 * i < a.tq;
                    l2v[i] = (!in || lse_n[i] == -INFINITY) ? INFINITY : lse_n[i] * LOG2E;
                    dlv[i] = in ? dl_n[i] : 0.f;
                }
                if (t + 1 < steps) gather(t + 1);
                // aux[st] is free once the elementwise warps are done with step t - 2.
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.aux_free[st]), ph ^ 1))) { failed = true; break; }
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    sh.aux[st].lse2[lane + 32 * i] = l2v[i];
                    sh.aux[st].delta[lane + 32 * i] = dlv[i];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(sh.bar.aux_full[st]));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        if (steps > 0) {
            constexpr uint32_t IDESC_SC = idesc_f16(ROWS, ROWS, Pack<T>::FMT, 0, 0);    // [128 resident rows x 128 streamed rows]
            constexpr uint32_t IDESC_ACC = idesc_f16(ROWS, 128, Pack<T>::FMT, 0, 1);    // [128 rows x 128 features], B MN-major
            const uint64_t r1_desc = smem_desc_sw128(smem_u32(r1_s), 16, 1024), r2_desc = smem_desc_sw128(smem_u32(r2_s), 16, 1024);
            auto a_cols = [](int ks) { return static_cast<uint32_t>(32 * (ks >> 1) + 8 * (ks & 1)); };
            int n = 0;   // halves taken so far
            // A score product into `cols`: sixteen k-steps over the features, eight from each half.
            auto scores = [&](uint64_t res_desc, uint32_t cols, uint32_t done_bar) -> bool {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int slot = n % NS, ph = (n / NS) & 1;
                    if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.full[slot]), ph))) return false;
                    tc_fence_after_sync();
                    const uint64_t sd = smem_desc_sw128(smem_u32(ring + slot * HALF_TILE), 16, 1024);
                    const uint32_t e = BAR(sh.bar.empty[slot]);
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            umma_f16(tmem + cols, desc_at(res_desc, (2 * half + (ks >> 2)) * BOX + (ks & 3) * 32),
                                     desc_at(sd, (ks >> 2) * BOX + (ks & 3) * 32), IDESC_SC, (half | ks) > 0 ? 1u : 0u);
                        umma_commit(e);
                        if (half == 1) umma_commit(done_bar);
                    }
                    __syncwarp();
                    ++n;
                }
                return true;
            };
            // The gradient product of step t: the accumulator's low and high 128 columns from the low and
            // the high half of the streamed tile, the A operand (dS, or P) from tensor memory at `a_at`.
            auto gradient = [&](int t, uint32_t a_at) -> bool {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int slot = n % NS, ph = (n / NS) & 1;
                    if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.full[slot]), ph))) return false;
                    tc_fence_after_sync();
                    const uint64_t sd = smem_desc_sw128(smem_u32(ring + slot * HALF_TILE), BOX, 1024);
                    const uint32_t e = BAR(sh.bar.empty[slot]);
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < ROWS / 16; ++ks)
                            umma_f16_ts(tmem + COL_ACC + half * 128, tmem + a_at + a_cols(ks), desc_at(sd, ks * 2048), IDESC_ACC,
                                        (t > 0 || ks > 0) ? 1u : 0u);
                        umma_commit(e);
                    }
                    __syncwarp();
                    ++n;
                }
                return true;
            };
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.res_full), 0))) failed = true;
            if (PASS == PASS_DV) {
                // The score tile is double (columns 0 and 128): S^T(t + 1) is issued ahead of dV(t).
                if (!failed && !scores(r1_desc, COL_S, BAR(sh.bar.s_full[0]))) failed = true;
                for (int t = 0; t < steps && !failed; ++t) {
                    if (t + 1 < steps && !scores(r1_desc, ((t + 1) & 1) * 128, BAR(sh.bar.s_full[(t + 1) & 1]))) { failed = true; break; }
                    if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.a_full[t & 1]), (t >> 1) & 1))) { failed = true; break; }
                    tc_fence_after_sync();
                    if (!gradient(t, (t & 1) * 128)) { failed = true; break; }
                }
            } else {
                if (!failed && !(scores(r1_desc, COL_S, BAR(sh.bar.s_full[0])) && scores(r2_desc, COL_DP, BAR(sh.bar.dp_full)))) failed = true;
                for (int t = 0; t < steps && !failed; ++t) {
                    if (t + 1 < steps) {   // the next scores, once the elementwise threads have taken these
                        if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.s_free), t & 1))) { failed = true; break; }
                        tc_fence_after_sync();
                        if (!scores(r1_desc, COL_S, BAR(sh.bar.s_full[0]))) { failed = true; break; }
                    }
                    if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.a_full[t & 1]), (t >> 1) & 1))) { failed = true; break; }
                    tc_fence_after_sync();
                    if (!gradient(t, COL_DP)) { failed = true; break; }
                    // The next dP goes over dS of this step, behind the product that reads it (MMAs execute in issue order).
                    if (t + 1 < steps && !scores(r2_desc, COL_DP, BAR(sh.bar.dp_full))) { failed = true; break; }
                }
            }
            if (!failed && elect_one()) umma_commit(BAR(sh.bar.acc_ready));
        }
    } else {
        // ---------------- elementwise: a resident row and 32 of the step's columns per thread ----------------
        const int cg = (warp - 2) >> 2, col0 = cg * CW;
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(lane_base) << 16);
        const bool padded = ROWS_ARE_QUERIES && a.mask.kind == 1;
        float l2 = INFINITY, dl = 0.f;   // DQ: this query's log-sum-exp (base 2) and delta
        if (ROWS_ARE_QUERIES && row < a.tq) {
            const int64_t at = ((int64_t)b * a.tq + row) * a.hq + res_head;
            const float x = a.lse[at];
            l2 = x == -INFINITY ? INFINITY : x * LOG2E;
            dl = a.delta[at];
        }
        for (int t = 0; t < steps && !failed; ++t) {
            const int st = t & 1, ph2 = (t >> 1) & 1;
            const int c0 = step_col0(t) + col0;   // the first of this thread's columns (a key of DQ, a query of DK / DV)
            uint32_t pb = 0;
            if (padded) {
                const int key = c0 + lane;
                pb = __ballot_sync(0xffffffffu, key >= a.tk || key_padded(a.mask, b, key));
            }
            if (!ROWS_ARE_QUERIES && !__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.aux_full[st]), ph2))) { failed = true; break; }
            const uint32_t s_at = PASS == PASS_DV ? st * 128 : COL_S;
            const bool s_ok = PASS == PASS_DV ? mbar_wait(BAR(sh.bar.s_full[st]), ph2) : mbar_wait(BAR(sh.bar.s_full[0]), t & 1);
            if (!__all_sync(0xffffffffu, s_ok)) { failed = true; break; }
            tc_fence_after_sync();
            float p[CW];
            tmem_ld32(t_lane + s_at + col0, *reinterpret_cast<uint32_t(*)[32]>(&p[0]));
            tmem_ld_wait();
            if (PASS != PASS_DV) {   // the scores are in registers: the next ones may come
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(sh.bar.s_free));
            }
            const bool clear = !padded && c0 >= lo && c0 + CW <= hi;
            if (!__all_sync(0xffffffffu, clear)) {
                // A row that sees none of these columns (it belongs to another sequence of the packed batch, or
                // its interval ends before them) needs no comparisons: where every row of the warp sees all or
                // none, those rows are simply set.
                const bool none = !padded && (hi <= c0 || lo >= c0 + CW || hi <= lo);
                if (__all_sync(0xffffffffu, clear || none)) {
                    if (none) {
#pragma unroll
                        for (int c = 0; c < CW; ++c) p[c] = -INFINITY;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < CW; ++c)
                        p[c] = (c0 + c >= lo && c0 + c < hi && !((pb >> c) & 1u)) ? p[c] : -INFINITY;
                }
            }
            const ColumnAux &aux = sh.aux[st];
#pragma unroll
            for (int c4 = 0; c4 < CW / 4; ++c4) {
                float4 l4 = make_float4(l2, l2, l2, l2);
                if (!ROWS_ARE_QUERIES) l4 = *reinterpret_cast<const float4 *>(&aux.lse2[col0 + 4 * c4]);
                p[4 * c4 + 0] = ex2(fmaf(p[4 * c4 + 0], a.scale_log2, -l4.x));
                p[4 * c4 + 1] = ex2(fmaf(p[4 * c4 + 1], a.scale_log2, -l4.y));
                p[4 * c4 + 2] = ex2(fmaf(p[4 * c4 + 2], a.scale_log2, -l4.z));
                p[4 * c4 + 3] = ex2(fmaf(p[4 * c4 + 3], a.scale_log2, -l4.w));
            }
            uint32_t out[CW / 2];
            if (PASS == PASS_DV) {
#pragma unroll
                for (int c2 = 0; c2 < CW / 2; ++c2) out[c2] = Pack<T>::two(p[2 * c2], p[2 * c2 + 1]);
                tmem_st16(t_lane + s_at + col0, out);   // P^T over the first half of the f32 columns just read
            } else {
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.dp_full), t & 1))) { failed = true; break; }
                tc_fence_after_sync();
                float dp[CW];
                tmem_ld32(t_lane + COL_DP + col0, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
                tmem_ld_wait();
#pragma unroll
                for (int c4 = 0; c4 < CW / 4; ++c4) {
                    float4 d4 = make_float4(dl, dl, dl, dl);
                    if (!ROWS_ARE_QUERIES) d4 = *reinterpret_cast<const float4 *>(&aux.delta[col0 + 4 * c4]);
                    out[2 * c4 + 0] = Pack<T>::two(p[4 * c4 + 0] * (dp[4 * c4 + 0] - d4.x), p[4 * c4 + 1] * (dp[4 * c4 + 1] - d4.y));
                    out[2 * c4 + 1] = Pack<T>::two(p[4 * c4 + 2] * (dp[4 * c4 + 2] - d4.z), p[4 * c4 + 3] * (dp[4 * c4 + 3] - d4.w));
                }
                tmem_st16(t_lane + COL_DP + col0, out);   // dS over the first half of the f32 columns just read
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(BAR(sh.bar.a_full[st]));
                if (!ROWS_ARE_QUERIES) mbar_arrive(BAR(sh.bar.aux_free[st]));
            }
        }
        // ---------------- epilogue: 64 columns of the row per thread ----------------
        T *dst;
        bool in_range;
        float factor = a.scale;
        if (PASS == PASS_DQ) {
            dst = static_cast<T *>(a.dq) + (((int64_t)b * a.tq + row) * a.hq + res_head) * HD;
            in_range = row < a.tq;
        } else {
            dst = static_cast<T *>(PASS == PASS_DK ? a.dk : a.dv) + (((int64_t)b * a.tk + row) * a.hkv + res_head) * HD;
            in_range = row < a.tk;
            if (PASS == PASS_DV) factor = 1.f;
        }
        dst += cg * 64;
        if (steps == 0 || failed) {
            if (in_range && !failed) {
                const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < 8; ++c) reinterpret_cast<uint4 *>(dst)[c] = z;
            }
        } else if (__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.acc_ready), 0))) {
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                tmem_ld32(t_lane + COL_ACC + cg * 64 + c * 32, o);
                tmem_ld_wait();
                if (in_range) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        uint4 v;
                        v.x = Pack<T>::two(__uint_as_float(o[8 * e + 0]) * factor, __uint_as_float(o[8 * e + 1]) * factor);
                        v.y = Pack<T>::two(__uint_as_float(o[8 * e + 2]) * factor, __uint_as_float(o[8 * e + 3]) * factor);
                        v.z = Pack<T>::two(__uint_as_float(o[8 * e + 4]) * factor, __uint_as_float(o[8 * e + 5]) * factor);
                        v.w = Pack<T>::two(__uint_as_float(o[8 * e + 6]) * factor, __uint_as_float(o[8 * e + 7]) * factor);
                        reinterpret_cast<uint4 *>(dst)[c * 4 + e] = v;
                    }
                }
            }
            tc_fence_before_sync();
        } else {
            failed = true;
        }
    }

    if (threadIdx.x == 0 && steps == 0 && !mbar_wait(BAR(sh.bar.res_full), 0)) failed = true;
    if (failed && !aborted) atomicOr(&g_sm100_bwd256_status, 16u);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

template <typename T>
__global__ void __launch_bounds__(THREADS, 1)
bwd256_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const Sm100BwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem256[];
    const int qt = gridDim.y - 1 - blockIdx.y;   // later (longer, under causality) tiles first
    bwd256_pass<T, PASS_DQ>(&tm_q, &tm_do, &tm_k, &tm_v, a, smem256, blockIdx.z, qt * ROWS, blockIdx.x);
}

// blockIdx.x: the (key block, key-value head) unit in the plan's order; blockIdx.y: 0 the dK pass (the
// longer one: three products a step), 1 the dV pass.
template <typename T>
__global__ void __launch_bounds__(THREADS, 1)
bwd256_dkdv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do, const Sm100BwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem256[];
    const int nkb = (a.tk + ROWS - 1) / ROWS;
    const int unit = a.order ? a.order[blockIdx.x] : (int)blockIdx.x;
    const int item = unit / a.hkv, hk = unit - item * a.hkv;
    const int b = item / nkb, kt = item - b * nkb;
    if (blockIdx.y == 0) bwd256_pass<T, PASS_DK>(&tm_k, &tm_v, &tm_q, &tm_do, a, smem256, b, kt * ROWS, hk);
    else bwd256_pass<T, PASS_DV>(&tm_k, &tm_v, &tm_q, &tm_do, a, smem256, b, kt * ROWS, hk);
}

namespace {
template <typename T>
cudaError_t launch256_t(const Sm100BwdMaps &m, Sm100BwdArgs a, cudaStream_t stream, int *launches) {
    constexpr size_t smem = smem_bytes(PASS_DQ);
    static_assert(smem_bytes(PASS_DK) == smem && smem_bytes(PASS_DV) <= smem, "one size for the three passes");
    cudaError_t e = cudaFuncSetAttribute(bwd256_dq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(bwd256_dkdv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 gq(a.hq, (a.tq + ROWS - 1) / ROWS, a.b);
    bwd256_dq_kernel<T><<<gq, THREADS, smem, stream>>>(m.q128, m.do128, m.k128, m.v128, a);
    *launches += 1;
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if ((e = launch_bwd_plan(a, stream, launches)) != cudaSuccess) return e;
    const long long units = (long long)a.b * ((a.tk + ROWS - 1) / ROWS) * a.hkv;
    if (units > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    dim3 gk((unsigned)units, 2, 1);
    bwd256_dkdv_kernel<T><<<gk, THREADS, smem, stream>>>(m.k128, m.v128, m.q128, m.do128, a);
    *launches += 1;
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_bwd256_sm100(int dtype, const Sm100BwdMaps &m, const Sm100BwdArgs &a, cudaStream_t stream, int *launches) {
    return dtype == DASH_ATTN_BF16 ? launch256_t<__nv_bfloat16>(m, a, stream, launches) : launch256_t<__half>(m, a, stream, launches);
}

cudaError_t read_sm100_bwd256_status(unsigned int *status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_sm100_bwd256_status, sizeof(unsigned int));
    if (e != cudaSuccess) return e;
    if (clear && *status) {
        unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_sm100_bwd256_status, &zero, sizeof(unsigned int));
    }
    return e;
}

}  // namespace dash
