// The training forward on the 5th-generation tensor cores, two query tiles per block: bf16 / f16,
// head dimension 128 or 64 (the text below gives the sizes at 128; at 64 the Q / K / V tiles and the O
// accumulators are half as wide and P V runs 128 x 64 x 16).
//
// A block owns TWO tiles of 128 queries that sweep the same keys - two query heads of one
// key-value group over the same rows (grouped heads, even group size), or two consecutive row
// tiles of one head - so that every K / V tile fetched from L2 feeds twice the arithmetic, and it
// runs two softmax warpgroups, one per tile, so that every scheduler has two warps of elementwise
// work to interleave.  384 threads:
//   warp 0, 10  one lane each issues the TMA tile loads: warp 0 both Q tiles once and then the K
//               tiles of 128 keys, warp 10 the V tiles, into two-stage rings of 128-byte-swizzled
//               shared memory;
//   warp 1, 11  one lane each issues the tcgen05 MMAs of tile 0 / tile 1 (warp 1 also owns tensor
//               memory: 512 columns, per tile TWO 64-column S buffers and the 128-column O
//               accumulator): S_t(u) = Q_t K_u^T (128 x 64 x 16) for sub-steps u of 64 keys into
//               buffer u & 1, O_t += P_t(u) V_u (128 x 128 x 16, P from tensor memory);
//   warps 2..5  softmax of tile 0, warps 6..9 of tile 1: one query row per thread (TMEM lane =
//               row): read S from tensor memory, mask what the row does not see, keep the online
//               softmax in f32 with the scale folded into an exp2, write P rounded to the input
//               dtype back into tensor memory over the first half of the columns of the S buffer
//               it was read from (two 16-bit values per 32-bit column: the A operand of P V comes
//               from tensor memory), and at the end normalise O and store it with the row's
//               log-sum-exp.
// K and V arrive 128 keys at a time; the products and the softmax go through them in two sub-steps
// of 64 keys, so that a tile has TWO S buffers in the 128 columns one buffer of 128 keys would take.
// S_t(u + 2) is issued right behind P_t(u) V_u, whose operand it overwrites (MMAs of one thread
// execute in issue order), which is one sub-step AHEAD of the softmax: when a softmax warp has
// written P_t(u), S_t(u + 1) is already in the other buffer, and no product sits between two
// sub-steps of a tile's softmax.  (With one buffer of 128 keys per tile the softmax, P V and the
// next Q K^T of a tile ran strictly one after another, and that chain, not the tensor cores, set
// the step.)  The two softmax warps of a scheduler - one per tile - take turns at their exponentials,
// which the special-function pipe would otherwise run at half speed for both, and idle after.  Lazy
// row maximum, masking, bounded waits and the status word as in the one-tile kernel (fwd_sm100.cu).
#include <cuda.h>

#include <cstddef>
#include <type_traits>

#include "common.cuh"
#include "sm100.h"
#include "sm100_kernels.h"
#include "sm100_ptx.cuh"

namespace dash {

using namespace ptx;

__device__ unsigned int g_sm100_fwd2_status = 0;  // sticky: non-zero once a bounded wait has run out

namespace {

constexpr int BM = 128;                   // queries per tile
constexpr int BN = 128;                   // keys per K / V tile (one stage of a ring)
constexpr int SN = 64;                    // keys per sub-step: one S buffer, one pass of the softmax
constexpr int NT = 2;                     // query tiles per block
constexpr int NS = 2;                     // stages of the K and of the V ring
constexpr int HALF_BYTES = 128 * 128;     // 128 rows of 64 features (128 bytes): what one TMA box brings
constexpr int Q_HALF = HALF_BYTES, KV_HALF = HALF_BYTES;
// A tile of 128 rows is HD / 64 such halves.
template <int HD> struct Geo {
    static constexpr int HALVES = HD / 64;
    static constexpr int Q_BYTES = HALVES * HALF_BYTES;    // 32 KiB per tile at HD = 128
    static constexpr int KV_BYTES = HALVES * HALF_BYTES;
    // 1 KiB slack | Q x 2 | K ring | V ring | Shared
    static constexpr size_t SMEM_BYTES = 1024 + NT * Q_BYTES + 2 * NS * KV_BYTES + 1024;
};
constexpr int THREADS = 384;
constexpr int V_WARP = 10;
constexpr int MMA_WARP0 = 1, MMA_WARP1 = 11;   // the issuers of tile 0 and of tile 1, on two schedulers
constexpr float RESCALE_LOG2 = 8.0f;
// A row that sees at most this many keys keeps the exact running maximum instead of the lazy one:
// with few keys one of them often carries most of the weight, and only against the exact maximum is
// that key's probability exactly 1 before P is rounded to the input dtype - as in the reference's
// kernels, whose error bounds were measured on such rows.  Long rows, where the weights spread and
// the roundings average out, keep the lazy maximum and its rare rescales.
constexpr int EXACT_KEYS = 512;

struct Barriers {
    uint64_t q_full, k_full[NS], k_empty[NS], v_full[NS], v_empty[NS];
    uint64_t s_full[NT][2], p_full[NT][2];   // per S buffer
    uint64_t o_tail[NT], o_done[NT];   // the last P V but one of the tile has completed / the last one has
    uint64_t turn[4][NT];              // per scheduler: which tile's softmax warp may run its exponentials
};

struct Shared {
    Barriers bar;
    uint32_t tmem_base;
    int red_lo[4 * NT], red_hi[4 * NT];
    unsigned int abort;
    int tile_bad[NT];   // a softmax warp of the tile gave up: its output is not stored
};

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
    static constexpr int FMT = 1;
    static __device__ __forceinline__ uint32_t two(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};
template <> struct Pack<__half> {
    static constexpr int FMT = 0;
    static __device__ __forceinline__ uint32_t two(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};

// This thread's row of an HD-column f32 accumulator in tensor memory times `factor`.  Rare (the
// lazy maximum moved) and out of line, so that its registers are not the softmax loop's.
template <int HD>
__device__ __noinline__ void rescale_accumulator(uint32_t taddr, float factor) {
    tc_fence_after_sync();
#pragma unroll 1
    for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(taddr + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
        tmem_st32(taddr + c * 32, o);
    }
    tmem_st_wait();
}

}  // namespace

template <typename T, int HD>
__global__ void __launch_bounds__(THREADS, 1)
fwd2_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const Sm100FwdArgs a) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int HALVES = Geo<HD>::HALVES, Q_BYTES = Geo<HD>::Q_BYTES, KV_BYTES = Geo<HD>::KV_BYTES;
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *q_s = smem;                       // [NT][Q_BYTES]
    uint8_t *k_s = q_s + NT * Q_BYTES;         // [NS][KV_BYTES]
    uint8_t *v_s = k_s + NS * KV_BYTES;        // [NS][KV_BYTES]
    Shared &sh = *reinterpret_cast<Shared *>(v_s + NS * KV_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = gridDim.y - 1 - blockIdx.y;  // later (longer, under causality) tiles first
    const int b = blockIdx.z;
    // Tile t of the block: head h0 + t over rows m0 (paired heads), or head h0 over rows m0 + 128 t.
    const int pair = a.pair_heads;
    const int h0 = pair ? 2 * blockIdx.x : blockIdx.x;
    const int hk = h0 / (a.hq / a.hkv);
    const int m_base = pair ? qt * BM : qt * NT * BM;
    auto tile_head = [&](int t) { return pair ? h0 + t : h0; };
    auto tile_row0 = [&](int t) { return pair ? m_base : m_base + t * BM; };
    auto BAR = [&](uint64_t &x) { return smem_u32(&x); };

    if (threadIdx.x == 0) {
        sh.abort = *reinterpret_cast<volatile unsigned int *>(&g_sm100_fwd2_status);
        sh.tile_bad[0] = sh.tile_bad[1] = 0;
        mbar_init(BAR(sh.bar.q_full), 1);
        for (int i = 0; i < NS; ++i) {
            mbar_init(BAR(sh.bar.k_full[i]), 1);
            mbar_init(BAR(sh.bar.k_empty[i]), NT);   // one commit per tile's issuer
            mbar_init(BAR(sh.bar.v_full[i]), 1);
            mbar_init(BAR(sh.bar.v_empty[i]), NT);
        }
        for (int t = 0; t < NT; ++t) {
            for (int buf = 0; buf < 2; ++buf) {
                mbar_init(BAR(sh.bar.s_full[t][buf]), 1);
                mbar_init(BAR(sh.bar.p_full[t][buf]), 4);   // one arrival per softmax warp
            }
            mbar_init(BAR(sh.bar.o_tail[t]), 1);
            mbar_init(BAR(sh.bar.o_done[t]), 1);
            for (int w = 0; w < 4; ++w) mbar_init(BAR(sh.bar.turn[w][t]), 1);
        }
        fence_mbar_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
        // Both Q tiles are on their way before the block knows which keys it sweeps: their flight
        // covers the rest of the setup.  (A block that turns out to have nothing to do waits for
        // them at the end: shared memory must not be written behind a block that has left.)
        const uint32_t qf = BAR(sh.bar.q_full);
        mbar_expect_tx(qf, NT * Q_BYTES);
        for (int t = 0; t < NT; ++t) {
            const uint32_t dst = smem_u32(q_s + t * Q_BYTES);
#pragma unroll
            for (int half = 0; half < HALVES; ++half)
                tma_load_4d(dst + half * Q_HALF, &tm_q, qf, 64 * half, tile_head(t), tile_row0(t), b);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
    }

    // Each softmax thread owns one query row of one tile; the block sweeps the union of all rows'
    // key intervals.
    const int sw = warp - 2;                       // 0..7 for softmax warps
    const int tile = (sw >> 2) & 1;                // which of the two tiles
    const int lane_base = 32 * (warp & 3);         // the TMEM lanes this warp may touch
    const int r = lane_base + lane;                // row of the tile
    int lo = a.tk, hi = 0;
    if (warp >= 2 && warp < 2 + 4 * NT) {
        row_bounds_warp(a.mask, tile_row0(tile) + r, a.tq, a.tk, lo, hi);
        int wlo = warp_min_i(hi > lo ? lo : a.tk), whi = warp_max_i(hi > lo ? hi : 0);
        if (lane == 0) { sh.red_lo[sw] = wlo; sh.red_hi[sw] = whi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    int kmin = a.tk, kmax = 0;
#pragma unroll
    for (int i = 0; i < 4 * NT; ++i) { kmin = min(kmin, sh.red_lo[i]); kmax = max(kmax, sh.red_hi[i]); }
    const bool aborted = sh.abort != 0;
    const int subs = (!aborted && kmax > kmin) ? (kmax - kmin + SN - 1) / SN : 0;   // sub-steps of 64 keys
    const int steps = (subs + 1) / 2;                                                // K / V tiles of 128 keys
    bool failed = aborted;
    // TMEM columns: S[tile][buffer] at 128 tile + 64 buffer (P over its first 32 columns), O[tile] at 256 + HD tile.
    auto COL_S = [](int t, int buf) { return static_cast<uint32_t>(t * BN + buf * SN); };
    auto COL_O = [](int t) { return static_cast<uint32_t>(256 + t * HD); };

    if (warp == 0) {
        // ---------------- TMA producer of the K ring (the Q tiles were issued during the setup) ----------------
        if (lane == 0 && steps > 0) {
            for (int j = 0; j < steps; ++j) {
                const int st = j % NS, ph = (j / NS) & 1, k0 = kmin + j * BN;
                if (!mbar_wait(BAR(sh.bar.k_empty[st]), ph ^ 1)) { failed = true; break; }
                const uint32_t full = BAR(sh.bar.k_full[st]), dst = smem_u32(k_s + st * KV_BYTES);
                mbar_expect_tx(full, KV_BYTES);
#pragma unroll
                for (int half = 0; half < HALVES; ++half) tma_load_4d(dst + half * KV_HALF, &tm_k, full, 64 * half, hk, k0, b);
            }
        }
    } else if (warp == V_WARP) {
        // ---------------- TMA producer of the V ring ----------------
        if (lane == 0 && steps > 0) {
            for (int j = 0; j < steps; ++j) {
                const int st = j % NS, ph = (j / NS) & 1, k0 = kmin + j * BN;
                if (!mbar_wait(BAR(sh.bar.v_empty[st]), ph ^ 1)) { failed = true; break; }
                const uint32_t full = BAR(sh.bar.v_full[st]), dst = smem_u32(v_s + st * KV_BYTES);
                mbar_expect_tx(full, KV_BYTES);
#pragma unroll
                for (int half = 0; half < HALVES; ++half) tma_load_4d(dst + half * KV_HALF, &tm_v, full, 64 * half, hk, k0, b);
            }
        }
    } else if (warp == MMA_WARP0 || warp == MMA_WARP1) {
        // ---------------- MMA issuers: one warp per tile, one elected lane issuing ----------------
        // The tensor pipe takes MMAs from a short queue: whatever the issuer does between two of them - a
        // poll of a barrier, address arithmetic - is time the pipe stands still unless another issuer's MMAs
        // fill it.  So each tile has an issuing warp of its own, on a scheduler of its own, whose waits fall
        // under the other tile's products.  The whole warp runs the (warp-uniform) code, so that barrier
        // addresses and descriptors are made in the uniform datapath; one elected lane issues.
        if (subs > 0) {
            const int t = __shfl_sync(0xffffffffu, warp, 0) == MMA_WARP0 ? 0 : 1;
            constexpr uint32_t IDESC_S = idesc_f16(BM, SN, Pack<T>::FMT, 0, 0);   // [128 q x 64 keys], A = Q, B = K K-major
            constexpr uint32_t IDESC_O = idesc_f16(BM, HD, Pack<T>::FMT, 0, 1);   // [128 q x HD], A = P (TMEM), B = V MN-major
            // Every address is a register plus a constant: barriers from one base, descriptors as a shared
            // high word and a low word (the address field) per operand, and the loop is unrolled four times
            // so that the stage and the half of a sub-step are constants.
            const uint64_t qk_desc = smem_desc_sw128(smem_u32(q_s + t * Q_BYTES), 16, 1024);
            // V rows are keys (the K of this product): 64-column halves KV_HALF apart, 8-key groups 1024 B apart.
            const uint64_t v_desc = smem_desc_sw128(smem_u32(v_s), KV_HALF, 1024);
            const uint32_t q_lo = static_cast<uint32_t>(qk_desc), qk_hi = static_cast<uint32_t>(qk_desc >> 32);
            const uint32_t k_lo = static_cast<uint32_t>(smem_desc_sw128(smem_u32(k_s), 16, 1024));
            const uint32_t v_lo = static_cast<uint32_t>(v_desc), v_hi = static_cast<uint32_t>(v_desc >> 32);
            const uint32_t col_s = tmem + COL_S(t, 0), col_o = tmem + COL_O(t);
            const uint32_t bars = BAR(sh.bar.q_full);
            auto bar_at = [&](size_t offset) { return bars + static_cast<uint32_t>(offset); };
#define FWD2_BAR(member) bar_at(offsetof(Barriers, member))
            // Keys 64 half .. of stage st: 64 rows of 128 bytes further down in each 64-feature half of the tile.
            auto tile_at = [](int st, int half) { return static_cast<uint32_t>((st * KV_BYTES + half * SN * 128) >> 4); };
            // S_t = Q_t K^T for the 64 keys of (st, half), into S buffer `half`
            auto qk = [&](int st, int half) {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma_f16_words(col_s + half * SN, q_lo + (((ks >> 2) * Q_HALF + (ks & 3) * 32) >> 4), qk_hi,
                                   k_lo + tile_at(st, half) + (((ks >> 2) * KV_HALF + (ks & 3) * 32) >> 4), qk_hi, IDESC_S, ks > 0 ? 1u : 0u);
            };
            // Sub-step u = 4 i + R: stage R / 2, half R % 2 - one uninterrupted run of MMAs (P V of the sub-step
            // and S of the next but one, which overwrites its operand, behind it), every wait before the run and
            // every commit after it.  Parities: P / S buffers are reused every second sub-step, stages every fourth.
            auto sub_step = [&](auto r_, int i, int u) -> bool {
                constexpr int R = decltype(r_)::value, st = R >> 1, half = R & 1;
                const bool more = u + 2 < subs;
                // (One vote over all the waits of the run: the lanes leave together, whatever a wait answers.)
                bool ok = mbar_wait(FWD2_BAR(p_full) + 8 * (2 * t + half), st);
                if (half == 0) {
                    ok = mbar_wait(FWD2_BAR(v_full) + 8 * st, i & 1) && ok;
                    if (more) ok = mbar_wait(FWD2_BAR(k_full) + 8 * (st ^ 1), (i + st) & 1) && ok;
                }
                if (!__all_sync(0xffffffffu, ok)) return false;
                tc_fence_after_sync();
                if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < SN / 16; ++ks)
                    umma_f16_ts_words(col_o, col_s + half * SN + ks * 8, v_lo + tile_at(st, half) + ((ks * 2048) >> 4), v_hi, IDESC_O,
                                      (u > 0 || ks > 0) ? 1u : 0u);
                if (more) {
                    qk(st ^ 1, half);
                    umma_commit(FWD2_BAR(s_full) + 8 * (2 * t + half));
                    // both issuers release a stage: behind the product on its second half, or on the last sub-step
                    if (half == 1 || u + 2 == subs - 1) umma_commit(FWD2_BAR(k_empty) + 8 * (st ^ 1));
                }
                // No commit per product for O: a row that has to rescale O (rare) learns that P V of u - 1
                // has completed from S of u + 1, which is issued behind it - or, at the last sub-step, from
                // o_tail; the epilogue waits for o_done.
                if (u >= subs - 2) umma_commit(u == subs - 1 ? FWD2_BAR(o_done) + 8 * t : FWD2_BAR(o_tail) + 8 * t);
                if (half == 1 || u == subs - 1) umma_commit(FWD2_BAR(v_empty) + 8 * st);
                }
                return true;
            };
            // Two sub-steps of S ahead ...
            if (!__all_sync(0xffffffffu, mbar_wait(FWD2_BAR(q_full), 0) && mbar_wait(FWD2_BAR(k_full), 0))) failed = true;
            if (!failed) {
                tc_fence_after_sync();
                if (elect_one()) {
                qk(0, 0);
                umma_commit(FWD2_BAR(s_full) + 8 * (2 * t));
                if (subs > 1) {
                    qk(0, 1);
                    umma_commit(FWD2_BAR(s_full) + 8 * (2 * t + 1));
                }
                umma_commit(FWD2_BAR(k_empty));
                }
                // ... then the sub-steps, four to a round of the two stages.
#pragma unroll 1
                for (int i = 0, u = 0; u < subs; ++i, u += 4) {
                    if (!sub_step(std::integral_constant<int, 0>{}, i, u)) { failed = true; break; }
                    if (u + 1 >= subs) break;
                    if (!sub_step(std::integral_constant<int, 1>{}, i, u + 1)) { failed = true; break; }
                    if (u + 2 >= subs) break;
                    if (!sub_step(std::integral_constant<int, 2>{}, i, u + 2)) { failed = true; break; }
                    if (u + 3 >= subs) break;
                    if (!sub_step(std::integral_constant<int, 3>{}, i, u + 3)) { failed = true; break; }
                }
            }
#undef FWD2_BAR
        }
    } else {
        // ---------------- softmax of one tile, one row per thread ----------------
        const int t = tile, h = tile_head(t);
        const int row = tile_row0(t) + r;
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(lane_base) << 16);
        const bool padded = a.mask.kind == 1;
        const float2 sl2 = make_float2(a.scale_log2, a.scale_log2);
        float m_ref = -INFINITY, l = 0.f;
        const float rescale_at = hi - lo <= EXACT_KEYS ? 0.f : RESCALE_LOG2;
        for (int u = 0; u < subs && !failed; ++u) {
            const int k0 = kmin + u * SN, buf = u & 1;
            uint32_t pb[SN / 32] = {0, 0};
            if (padded) {
#pragma unroll
                for (int i = 0; i < SN / 32; ++i) {
                    const int key = k0 + i * 32 + lane;
                    pb[i] = __ballot_sync(0xffffffffu, key >= a.tk || key_padded(a.mask, b, key));
                }
            }
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.s_full[t][buf]), (u >> 1) & 1))) { failed = true; break; }
            tc_fence_after_sync();
            float s[SN];
#pragma unroll
            for (int c = 0; c < SN / 32; ++c) tmem_ld32(t_lane + COL_S(t, buf) + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            tmem_ld_wait();

            const bool clear = !padded && k0 >= lo && k0 + SN <= hi;  // the row sees the whole sub-step
            // ... or nothing of it: a row of another sequence of the packed batch (a tile that straddles two
            // sequences sweeps the first one's keys for the second one's rows too), or one whose interval ends
            // before the sub-step.  Such a row needs no look at its scores: its maximum is -inf and its
            // exponentials are taken against -inf, which makes them exact zeros.
            const bool none = !padded && (hi <= k0 || lo >= k0 + SN || hi <= lo);
            if (!__all_sync(0xffffffffu, clear || none)) {
#pragma unroll
                for (int c = 0; c < SN; ++c) {
                    const int key = k0 + c;
                    const bool vis = key >= lo && key < hi && !((pb[c >> 5] >> (c & 31)) & 1u);
                    s[c] = vis ? s[c] : -INFINITY;
                }
            }
            // Row maximum: eight independent chains of three-input maxima, then a tree.
            float mx8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) mx8[e] = fmax3(s[e], s[8 + e], s[16 + e]);
#pragma unroll
            for (int c = 24; c < SN; c += 16)
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    mx8[e] = c + 8 + e < SN ? fmax3(mx8[e], s[c + e], s[c + 8 + e]) : fmaxf(mx8[e], s[c + e]);
            const float mx = none ? -INFINITY : fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(fmax3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
            // Lazy maximum: move the reference only when the row's maximum outgrew it by 2^8 - or by
            // anything at all, for a row of few keys (see EXACT_KEYS).
            float factor = 1.f;
            bool rescale = false;
            if (m_ref == -INFINITY) {
                m_ref = mx;  // nothing accumulated yet for this row (or exact zeros)
            } else if ((mx - m_ref) * a.scale_log2 > rescale_at) {
                // The difference of the two offsets as the exponentials use them (each product rounded on its
                // own), so that what was summed before and what is summed from here on share one reference.
                factor = ex2(__fsub_rn(__fmul_rn(m_ref, a.scale_log2), __fmul_rn(mx, a.scale_log2)));
                l *= factor;
                m_ref = mx;
                rescale = true;
            }
            const float neg = none ? -INFINITY : m_ref == -INFINITY ? 0.f : -__fmul_rn(m_ref, a.scale_log2);
            const float2 neg2 = make_float2(neg, neg);

            // Only a moved reference touches O, and it has to see sub-steps 0..u-1 in it.  P V of u - 2 has
            // completed (S of this sub-step was issued behind it); P V of u - 1 - whose P this warp arrived a
            // moment ago - may not have.  S of u + 1 is issued behind it, so the warp waits for that (the
            // barrier it waits on at the next sub-step anyway: of its phases, that of S(u - 1) has completed
            // and that of S(u + 3) cannot have), or for o_tail at the last sub-step.
            if (u > 0 && __any_sync(0xffffffffu, rescale)) {
                const bool ok = u + 1 < subs ? mbar_wait(BAR(sh.bar.s_full[t][buf ^ 1]), ((u + 1) >> 1) & 1)
                                             : mbar_wait(BAR(sh.bar.o_tail[t]), 0);
                if (!__all_sync(0xffffffffu, ok)) { failed = true; break; }
                rescale_accumulator<HD>(t_lane + COL_O(t), factor);
            }
            // The special-function pipe takes one warp instruction in eight cycles: the 64 exponentials of a
            // warp are 512 cycles of it, and the two softmax warps of a scheduler - one per tile - that run
            // them at the same time each take twice that, after which the pipe stands idle while both do the
            // rest of their sub-steps.  So the two take turns: tile 0's warp runs the exponentials of sub-step
            // u, then tile 1's, then tile 0's of u + 1 ..., each doing the rest of its sub-step (the wait for
            // S, the maximum, the store of P) under the other's turn.  (Bounded waits on barriers of the
            // block's own, like every other wait here; both tiles sweep the same sub-steps.)
            if (t == 1 || u > 0) {
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.turn[warp & 3][t]), (t == 1 ? u : u - 1) & 1))) { failed = true; break; }
            }
            // P over the first 32 columns of the buffer this thread has read (two 16-bit values a column).
            float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int cc = 0; cc < SN / 32; ++cc) {
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float2 x = fma2(make_float2(s[cc * 32 + 2 * e], s[cc * 32 + 2 * e + 1]), sl2, neg2);
                    const float p0 = ex2(x.x), p1 = ex2(x.y);
                    sum2[e & 3] = add2(sum2[e & 3], make_float2(p0, p1));
                    pk[e] = Pack<T>::two(p0, p1);
                }
                tmem_st16(t_lane + COL_S(t, buf) + cc * 16, pk);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(sh.bar.turn[warp & 3][t ^ 1]));   // the other tile's turn
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(sh.bar.p_full[t][buf]));
            {
                const float2 tsum = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
                l += tsum.x + tsum.y;
            }
        }
        // ---------------- epilogue ----------------
        T *out = static_cast<T *>(a.out);
        const int64_t base = ((int64_t)b * a.tq + row) * a.hq + h;
        if (subs == 0 || failed) {
            if (row < a.tq && !failed) {
                const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) reinterpret_cast<uint4 *>(out + base * HD)[c] = z;
                a.lse[base] = -INFINITY;
            }
        } else if (__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.o_done[t]), 0))) {
            // Every MMA has completed, so the tile's Q is dead: the normalised rows are staged over
            // it in the layout of the TMA box (two halves of 64 columns, 128-byte rows, 16-byte
            // chunks XOR-swizzled by the row) and leave as two bulk stores - whole lines instead of
            // 16 bytes per thread and row - which also drop the rows past the last query.
            tc_fence_after_sync();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            uint8_t *stage = q_s + t * Q_BYTES;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(t_lane + COL_O(t) + c * 32, o);
                tmem_ld_wait();
                uint8_t *half_row = stage + (c >> 1) * Q_HALF + r * 128;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint4 v;
                    v.x = Pack<T>::two(__uint_as_float(o[8 * e + 0]) * inv, __uint_as_float(o[8 * e + 1]) * inv);
                    v.y = Pack<T>::two(__uint_as_float(o[8 * e + 2]) * inv, __uint_as_float(o[8 * e + 3]) * inv);
                    v.z = Pack<T>::two(__uint_as_float(o[8 * e + 4]) * inv, __uint_as_float(o[8 * e + 5]) * inv);
                    v.w = Pack<T>::two(__uint_as_float(o[8 * e + 6]) * inv, __uint_as_float(o[8 * e + 7]) * inv);
                    const int chunk = (c & 1) * 4 + e;   // 16-byte chunk of the half row
                    *reinterpret_cast<uint4 *>(half_row + ((chunk ^ (r & 7)) << 4)) = v;
                }
            }
            // Once per row, so in f64: the product, the logarithm and their sum round once, to f32 at the end.
            // The exponentials were taken against -m_ref * scale_log2 ROUNDED to f32, a factor common to the
            // whole row that is not in m_ref * scale: its rounding error (in base-2 units) goes back in.
            if (row < a.tq) {
                const float used = __fmul_rn(m_ref, a.scale_log2);   // what the loop subtracted from every exponent
                const double slip = (double)used - (double)m_ref * (double)a.scale_log2;
                a.lse[base] = l > 0.f ? (float)((double)m_ref * (double)a.scale + slip * 0.6931471805599453 + log((double)l)) : -INFINITY;
            }
            tc_fence_before_sync();
        } else {
            failed = true;
        }
        if (steps > 0) {
            // Every warp of the tile gets here (all waits are bounded), whatever became of it: one
            // that gave up marks the tile, and nothing is stored from a tile that is not whole.
            if (failed && lane == 0) sh.tile_bad[t] = 1;
            fence_proxy_async_smem();
            named_barrier(1 + t, 128);   // the tile's four warps
            if ((warp & 3) == 2 && lane == 0 && sh.tile_bad[t] == 0) {
                uint8_t *stage = q_s + t * Q_BYTES;
#pragma unroll
                for (int half = 0; half < HALVES; ++half)
                    tma_store_4d(&tm_o, smem_u32(stage + half * Q_HALF), 64 * half, h, tile_row0(t), b);
                tma_store_commit();
                tma_store_wait_read();
            }
        }
    }

    if (threadIdx.x == 0 && steps == 0 && !mbar_wait(BAR(sh.bar.q_full), 0)) failed = true;
    if (failed && !aborted) atomicOr(&g_sm100_fwd2_status, 8u);
    // Teardown: every thread gets here (all waits are bounded); the allocating warp frees TMEM.
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

namespace {
template <typename T, int HD>
cudaError_t launch_fwd2_t(dim3 grid, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const CUtensorMap &to,
                          const Sm100FwdArgs &a, cudaStream_t stream) {
    constexpr size_t smem = Geo<HD>::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(fwd2_sm100_kernel<T, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    fwd2_sm100_kernel<T, HD><<<grid, THREADS, smem, stream>>>(tq, tk, tv, to, a);
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_fwd2_sm100(int dtype, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                              const CUtensorMap &to, const Sm100FwdArgs &a, cudaStream_t stream) {
    dim3 grid(a.pair_heads ? a.hq / 2 : a.hq, a.pair_heads ? (a.tq + BM - 1) / BM : (a.tq + NT * BM - 1) / (NT * BM), a.b);
    if (dtype == DASH_ATTN_BF16)
        return a.d == 64 ? launch_fwd2_t<__nv_bfloat16, 64>(grid, tq, tk, tv, to, a, stream)
                         : launch_fwd2_t<__nv_bfloat16, 128>(grid, tq, tk, tv, to, a, stream);
    return a.d == 64 ? launch_fwd2_t<__half, 64>(grid, tq, tk, tv, to, a, stream)
                     : launch_fwd2_t<__half, 128>(grid, tq, tk, tv, to, a, stream);
}

cudaError_t read_sm100_fwd2_status(unsigned int *status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_sm100_fwd2_status, sizeof(unsigned int));
    if (e != cudaSuccess) return e;
    if (clear && *status) {
        unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_sm100_fwd2_status, &zero, sizeof(unsigned int));
    }
    return e;
}

}  // namespace dash
