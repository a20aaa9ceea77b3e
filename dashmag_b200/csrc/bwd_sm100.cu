// The written-out backward on the 5th-generation tensor cores: bf16 / f16, head dimension 128.
//
// Two kernels, neither with atomics, so every gradient is summed in a fixed order and the bits
// repeat from run to run (the contract's default, crates/dash-contract/src/attention.rs:96-102):
//
//   dkdv   one block per (128 keys, key-value head).  K_j and V_j stay in shared memory; the block
//          sweeps the query heads of the group and, in steps of 128, the queries that see the key
//          block.  Per step:  S^T = K_j Q^T and dP^T = V_j dO^T on the tensor cores (TMEM lane =
//          key), P^T = exp2(S^T sl - lse) and dS^T = P^T (dP^T - delta) elementwise, rounded to the
//          input dtype back into tensor memory, then dV += P^T dO and dK += dS^T Q with the A
//          operand read from tensor memory, accumulated in TMEM over the whole sweep.
//   dq     one block per (128 queries, query head).  Q_i and dO_i stay in shared memory; the block
//          sweeps, in steps of 64, the keys its queries see.  Per step: S = Q_i K^T, dP = dO_i V^T,
//          dS = P (dP - delta), then dQ += dS K.
//
// Both recompute the scores tile by tile from the saved log-sum-exp (no T x T anywhere): seven
// 128-deep products per pair of tiles.  The streamed tiles serve twice from one copy in shared
// memory - K-major for the score products and MN-major for the gradient products - through two
// descriptors over the same 128-byte-swizzled bytes.  Warp roles as in the forward: warp 0 issues
// TMA loads, warp 1 issues the MMAs and owns TMEM, the next 8 (dq) or 16 (dkdv) warps do the
// elementwise work - two or four warps per quadrant of TMEM lanes, each thread one row (lane) and
// a slice of the step's columns, so that every scheduler has several warps of it to interleave -
// and in dkdv one more warp gathers the step's per-query log-sum-exp, delta and key interval, one
// step ahead of their use (its loads from global memory were the longest link of the step before
// they were issued early).  Every mbarrier wait is bounded (sm100_ptx.cuh).
#include <cuda.h>

#include "bwd_common.cuh"
#include "common.cuh"
#include "sm100.h"
#include "sm100_kernels.h"
#include "sm100_ptx.cuh"

namespace dash {

using namespace ptx;

// Sticky, like the forward's: non-zero once a bounded wait of these kernels has run out.  (Without
// relocatable device code every translation unit owns its device variables, so the backward has a
// word of its own and the host reads both.)
__device__ unsigned int g_sm100_bwd_status = 0;

namespace {

constexpr int BIG = 128;                   // rows of a tile: resident or streamed (and TMEM lanes)
constexpr int BIG_HALF = BIG * 128;        // 128 rows of 128 bytes: 64 columns of a tile, what one TMA box brings
// A tile of head dimension HD (128 or 64) is HD / 64 such halves: 32 KiB at 128.
template <int HD> constexpr int tile_bytes() { return (HD / 64) * BIG_HALF; }
constexpr int QS = BIG;                    // rows of a streamed tile: a step
constexpr int KCG = 4;                     // elementwise warps per TMEM lane quadrant
constexpr int KQW = QS / KCG;              // columns of a step per elementwise thread
constexpr int KAUX_WARP = 2 + 4 * KCG;     // dkdv: one more warp gathers the per-query vectors
constexpr int KTHREADS = 32 * (3 + 4 * KCG);
constexpr int KRED_WARP = KAUX_WARP + 1;   // fused dkdv: four more warps (one per TMEM lane quadrant) send dQ out
constexpr int KTHREADS_FUSED = KTHREADS + 128;
constexpr int RED_SLOT = 128 * 128;        // a staging slot of the dQ reduction: 128 rows of 32 f32 columns
static_assert(KQW == 32, "one 32-column TMEM load per thread and phase");
constexpr float LOG2E = 1.4426950408889634f;

// 2^x on the special-function pipe or, for a share of the elements, on the FMA pipe.
template <bool POLY> __device__ __forceinline__ float exp2_mixed(float x) { return POLY ? ex2_poly3(x) : ex2(x); }

// Of every four exponentials, how many run on the FMA pipe (ex2_poly3).  dkdv: one for bf16, whose rounding
// step (2^-9) is thirty times the cubic's error; none for f16, whose step (2^-12) is only four times it.  dq:
// none - its elementwise warps are not held up by the special-function pipe, and every cubic is ten
// instructions for one (measured on config 2: 35 us of 1 370 slower with a quarter as cubics).
template <typename T> constexpr int poly_of4() { return Pack<T>::FMT == 1 ? 1 : 0; }

// `groups` x 32 f32 accumulator columns of this thread's TMEM lane, scaled, rounded and stored as
// contiguous elements of the row.
template <typename T>
__device__ __forceinline__ void store_acc_cols(uint32_t taddr, T *dst, float scale, bool write, int groups) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (c >= groups) break;
        uint32_t o[32];
        tmem_ld32(taddr + c * 32, o);
        tmem_ld_wait();
        if (write) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                uint4 v;
                v.x = Pack<T>::two(__uint_as_float(o[8 * e + 0]) * scale, __uint_as_float(o[8 * e + 1]) * scale);
                v.y = Pack<T>::two(__uint_as_float(o[8 * e + 2]) * scale, __uint_as_float(o[8 * e + 3]) * scale);
                v.z = Pack<T>::two(__uint_as_float(o[8 * e + 4]) * scale, __uint_as_float(o[8 * e + 5]) * scale);
                v.w = Pack<T>::two(__uint_as_float(o[8 * e + 6]) * scale, __uint_as_float(o[8 * e + 7]) * scale);
                reinterpret_cast<uint4 *>(dst)[c * 4 + e] = v;
            }
        }
    }
}

// 8 * CHUNKS zero elements.
template <typename T, int CHUNKS>
__device__ __forceinline__ void store_zero_cols(T *dst) {
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) reinterpret_cast<uint4 *>(dst)[c] = z;
}

// Offsets of packed sequences kept in shared memory (dkdv); the fused form, whose tiles fill shared
// memory to the last kilobytes, keeps fewer.
template <bool FUSED> constexpr int cu_cache() { return FUSED ? 64 : 768; }

}  // namespace

// =================================================================================================
// Plan: the order in which the (key block, key-value head) units of dkdv are launched
// =================================================================================================
// Two things decide it.  The sweep of a key block is as long as the range of queries that may see it,
// which under causality and packing differs by two orders of magnitude between blocks, and blocks are
// scheduled in index order: long sweeps must start first or the kernel ends in a tail.  And what runs
// at the same time should touch the same memory: the key blocks of one sequence and one key-value
// head stream the same Q / dO tiles of that head's group (and, in the fused form, add to the same
// rows of the f32 dQ accumulator), one tile apart, so that side by side they find each other's tiles
// in L2 - where all heads of many sequences at once push each other's out.  So: sequences by
// falling work of their longest sweep; within a sequence one head after the other; within a head the
// key blocks by falling work.  One block of threads counts the steps of each key block, ranks them
// and writes, for every launch index, item * hkv + head (ties by index, so the order is a pure
// function of the inputs).
constexpr int PLAN_MAX = 2048;
constexpr int PLAN_THREADS = 1024;

__global__ void __launch_bounds__(PLAN_THREADS) bwd_plan_kernel(const Sm100BwdArgs a, int items) {
    // Items are (batch element, key block) in index order, so the items of one sequence are a run of
    // consecutive items: the runs are listed once, and each item then ranks its run among the runs
    // and itself within its run.
    __shared__ int work[PLAN_MAX], seq[PLAN_MAX], run_top[PLAN_MAX];
    __shared__ unsigned short run_of[PLAN_MAX], run_first[PLAN_MAX], run_len[PLAN_MAX];   // all below PLAN_MAX
    __shared__ int runs;
    const int nkb = (a.tk + BIG - 1) / BIG;
    if (threadIdx.x == 0) runs = 0;
    for (int i = threadIdx.x; i < items; i += PLAN_THREADS) {
        const int bi = i / nkb, kt = i - bi * nkb, k0 = kt * BIG;
        int first, end;
        query_range(a.mask, k0, min(k0 + BIG, a.tk), a.tq, a.tk, first, end);
        work[i] = end > first ? (end - first + QS - 1) / QS : 0;
        // The sequence a key block belongs to: the packed sequence of its first key, else its batch
        // element (kept apart per batch element so that a run never crosses one).
        seq[i] = a.mask.kind == 2 ? max(sequence_of(a.mask.cu_k, a.mask.idx_bytes, a.mask.seqs, k0), 0) : bi;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < items; i += PLAN_THREADS) {
        if (i == 0 || seq[i - 1] != seq[i]) {   // the head of a run measures it
            int n = 1, top = work[i];
            while (i + n < items && seq[i + n] == seq[i]) { top = max(top, work[i + n]); ++n; }
            const int r = atomicAdd(&runs, 1);
            run_first[r] = (unsigned short)i;
            run_len[r] = (unsigned short)n;
            run_top[r] = top;
            for (int j = 0; j < n; ++j) run_of[i + j] = (unsigned short)r;
        }
    }
    __syncthreads();
    const int nruns = runs;
    for (int i = threadIdx.x; i < items; i += PLAN_THREADS) {
        const int r = run_of[i], f = run_first[r], n = run_len[r], tp = run_top[r], w = work[i];
        int before = 0, ahead = 0;   // items of the runs that go first; items of this run ahead of i
        for (int j = 0; j < nruns; ++j)
            if (run_top[j] > tp || (run_top[j] == tp && run_first[j] < f)) before += run_len[j];
        for (int j = f; j < f + n; ++j) ahead += (work[j] > w) || (work[j] == w && j < i);
        for (int hk = 0; hk < a.hkv; ++hk) a.order[before * a.hkv + hk * n + ahead] = i * a.hkv + hk;
    }
}

// Launches the plan into a.order, or clears a.order when there is nothing to rank or too much to rank
// in one block (the units then run in index order).
cudaError_t launch_bwd_plan(Sm100BwdArgs &a, cudaStream_t stream, int *launches) {
    const long long items = (long long)a.b * ((a.tk + BIG - 1) / BIG);
    if (a.order && items > 1 && items <= PLAN_MAX && items * a.hkv <= 0x7fffffffLL / 4) {
        bwd_plan_kernel<<<1, PLAN_THREADS, 0, stream>>>(a, (int)items);
        *launches += 1;
        return cudaGetLastError();
    }
    a.order = nullptr;
    return cudaSuccess;
}

size_t bwd_sm100_order_bytes(int b, int tk, int hkv) {
    const long long units = (long long)b * ((tk + BIG - 1) / BIG) * hkv;
    return (size_t)((units * 4 + 255) & ~255LL);
}

// =================================================================================================
// dK, dV
// =================================================================================================
// Steps of 128 queries, so that all four products of a step are 128 x 128 x 128 (the width at which
// the tensor cores run at full rate).  The score tiles are single in tensor memory and P^T / dS^T are
// written over the f32 values they were made from (two 16-bit values per 32-bit column) and fed to
// dV += P^T dO and dK += dS^T Q as A operands straight from tensor memory; MMAs of one thread
// execute in issue order, which is what lets S^T of the next step be issued right behind the
// product that reads P^T from the same columns.  Issue order per step t:
//     dV(t)  S^T(t+1)  dK(t)  dP^T(t+1)
// so the P half of the elementwise work of step t+1 runs under dK(t) and dP^T(t+1), and its dS half
// under dV(t+1) and S^T(t+2).
//
// The FUSED form (AttentionOptions::deterministic off; the reference's backward_kernel with atomics,
// crates/dash-ops/src/attention/kernels.rs:1600) adds the fifth product to the same sweep, so that no
// dq kernel runs and the scores are computed once: dS^T is also written, in the input dtype, to a tile
// in shared memory, dQ(t) = dS K comes from it (A = dS, MN-major, straight from that tile; B = the
// resident K) into the columns dP^T has just left, and four more warps take dQ(t) out of tensor memory,
// stage it 32 columns at a time in shared memory and add it to an f32 accumulator in global memory
// with bulk tensor reductions (cp.reduce.async.bulk, whole lines added in L2) - in whatever order the
// key blocks get there, which is what makes this form's dQ differ in its last bits from run to run.
// Issue order per step t:
//     dV(t)  S^T(t+1)  dK(t)  dQ(t)  dP^T(t+1)
// dK(t) reads dS^T from the dP^T columns before dQ(t) overwrites them (MMAs execute in issue order).
// Shared memory: the dO ring gives up a stage for the dS tile and the staging slots (a dO tile is
// dead once dV has read it, and the next one is not needed before S^T, dK and dQ have run).
struct DkdvBarriers {
    uint64_t res_full;
    uint64_t q_full[2], q_empty[2], do_full[2], do_empty[2];
    uint64_t aux_full[2];
    uint64_t s_full, p_full[2], dp_full, ds_full[2];   // P^T and dS^T arrive in two halves (even, odd k-steps)
    uint64_t acc_ready;
    uint64_t dq_done, dq_taken;   // fused: dQ(t) is in tensor memory; the reduction warps have taken it out
};

struct alignas(16) QAux {   // what the elementwise threads need per query of a step
    float lse2[QS];        // log-sum-exp in base 2, +inf for a query that saw no key or is out of range
    float delta[QS];
};

template <bool FUSED> struct DkdvTail {
    DkdvBarriers bar;
    QAux aux[2];
    uint32_t tmem_base;
    unsigned int abort;
    int cu_q[cu_cache<FUSED>()], cu_k[cu_cache<FUSED>()];   // the packed sequences' offsets, when they fit
};

template <bool FUSED> constexpr size_t dkdv_tail() { return FUSED ? 3072 : 12288; }
static_assert(sizeof(DkdvTail<false>) <= dkdv_tail<false>() && sizeof(DkdvTail<true>) <= dkdv_tail<true>(),
              "the tail of the dkdv kernel's shared memory");
// 1 KiB slack | K, V resident (2 x 32 KiB) | Q ring 2 x 32 KiB | dO ring 2 x 32 KiB | tail, or fused
// (no slack: at D = 128 the tiles and the tail are the 227 KiB a block may have, and the kernel checks
// that its shared memory starts on a 1 KiB boundary)
//             K, V resident | Q ring 2 | dO 1 | dS^T tile 32 KiB | 2 staging slots of 16 KiB | tail
template <int HD, bool FUSED> constexpr size_t smem_dkdv() {
    return FUSED ? 5 * tile_bytes<HD>() + BIG * BIG * 2 + 2 * RED_SLOT + dkdv_tail<true>()
                 : 1024 + 6 * tile_bytes<HD>() + dkdv_tail<false>();
}

template <typename T, int HD, bool FUSED>
__global__ void __launch_bounds__(FUSED ? KTHREADS_FUSED : KTHREADS, 1)
bwd_dkdv_sm100_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_dq_acc, const Sm100BwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int BIG_BYTES = tile_bytes<HD>();
    constexpr int DOS = FUSED ? 1 : 2;        // stages of the dO ring
    uint8_t *smem = FUSED ? smem_raw : reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *k_s = smem, *v_s = k_s + BIG_BYTES;
    uint8_t *q_s = v_s + BIG_BYTES;           // [2][BIG_BYTES]
    uint8_t *do_s = q_s + 2 * BIG_BYTES;      // [DOS][BIG_BYTES]
    uint8_t *ds_s = do_s + DOS * BIG_BYTES;   // fused: dS^T of the step, [2 halves of 64 queries][128 keys][128 bytes]
    uint8_t *red_s = ds_s + BIG * BIG * 2;    // fused: [2][RED_SLOT]
    using Tail = DkdvTail<FUSED>;
    Tail &sh = *reinterpret_cast<Tail *>(FUSED ? red_s + 2 * RED_SLOT : do_s + DOS * BIG_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Units are taken in the order the plan kernel left (without one: in index order, the heads of a
    // key block side by side).
    const int nkb = (a.tk + BIG - 1) / BIG;
    const int unit = a.order ? a.order[blockIdx.x] : (int)blockIdx.x;
    const int item = unit / a.hkv, hk = unit - item * a.hkv;
    const int b = item / nkb, kt = item - b * nkb;
    const int group = a.hq / a.hkv;
    const int k0 = kt * BIG, k1 = min(k0 + BIG, a.tk);
    auto BAR = [&](uint64_t &x) { return smem_u32(&x); };

    if (threadIdx.x == 0) {
        sh.abort = *reinterpret_cast<volatile unsigned int *>(&g_sm100_bwd_status);
        // The fused form has no room to realign: a window that does not start on a 1 KiB boundary
        // (the swizzled tiles need it) is reported like a wait that ran out, and nothing runs.
        if (FUSED && (smem_u32(smem_raw) & 1023u) != 0) sh.abort = 1u;
        mbar_init(BAR(sh.bar.res_full), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(sh.bar.q_full[i]), 1);
            mbar_init(BAR(sh.bar.q_empty[i]), 1);
            mbar_init(BAR(sh.bar.do_full[i]), 1);
            mbar_init(BAR(sh.bar.do_empty[i]), 1);
            mbar_init(BAR(sh.bar.aux_full[i]), 1);
        }
        mbar_init(BAR(sh.bar.s_full), 1);
        mbar_init(BAR(sh.bar.dp_full), 1);
        mbar_init(BAR(sh.bar.p_full[0]), 4 * KCG);   // one arrival per elementwise warp
        mbar_init(BAR(sh.bar.p_full[1]), 4 * KCG);
        mbar_init(BAR(sh.bar.ds_full[0]), 4 * KCG);
        mbar_init(BAR(sh.bar.ds_full[1]), 4 * KCG);
        mbar_init(BAR(sh.bar.acc_ready), 1);
        mbar_init(BAR(sh.bar.dq_done), 1);
        mbar_init(BAR(sh.bar.dq_taken), 4);          // one arrival per reduction warp
        fence_mbar_init();
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_do);
        if constexpr (FUSED) prefetch_tensormap(&tm_dq_acc);
        // The resident tiles are on their way before the block knows which queries it sweeps: their
        // flight covers the rest of the setup.  (A block that turns out to have nothing to do waits
        // for them at the end: shared memory must not be written behind a block that has left.)
        const uint32_t rfull = BAR(sh.bar.res_full);
        mbar_expect_tx(rfull, 2 * BIG_BYTES);
        tma_load_4d(smem_u32(k_s), &tm_k, rfull, 0, hk, k0, b);
        if constexpr (HD > 64) tma_load_4d(smem_u32(k_s + BIG_HALF), &tm_k, rfull, 64, hk, k0, b);
        tma_load_4d(smem_u32(v_s), &tm_v, rfull, 0, hk, k0, b);
        if constexpr (HD > 64) tma_load_4d(smem_u32(v_s + BIG_HALF), &tm_v, rfull, 64, hk, k0, b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
    }
    int qfirst, qend;
    query_range(a.mask, k0, k1, a.tq, a.tk, qfirst, qend);
    // The per-query vectors of every step need each query's key interval, a binary search over the
    // sequences' offsets: from shared memory when they fit, so that it costs tens of cycles a probe
    // instead of a trip to L2.
    MaskArgs qmask = a.mask;
    if (a.mask.kind == 2 && a.mask.seqs + 1 <= cu_cache<FUSED>()) {
        for (int i = threadIdx.x; i <= a.mask.seqs; i += blockDim.x) {
            sh.cu_q[i] = load_index(a.mask.cu_q, a.mask.idx_bytes, i);
            sh.cu_k[i] = load_index(a.mask.cu_k, a.mask.idx_bytes, i);
        }
        qmask.cu_q = sh.cu_q;
        qmask.cu_k = sh.cu_k;
        qmask.idx_bytes = 4;
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    const bool aborted = sh.abort != 0;
    const int tiles = (!aborted && qend > qfirst) ? (qend - qfirst + QS - 1) / QS : 0;
    const int steps = tiles * group;
    bool failed = aborted;
    // TMEM columns: S^T at 0, dP^T at 128 (each with its 16-bit twin over the first half of every
    // group of 32 columns: columns 32 g + [0, 16) hold queries 32 g + [0, 32)), dV at 256, dK at 384.
    constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384;

    if (warp == 0) {
        // ---------------- producer: TMA loads ----------------
        if (lane == 0 && steps > 0) {
            for (int t = 0; t < steps; ++t) {
                const int st = t & 1, ph = (t >> 1) & 1;
                const int h = hk * group + t / tiles, q0 = qfirst + (t % tiles) * QS;
                // Q first (S^T of the step is issued before dP^T); its stage is also the later to come free.
                if (!mbar_wait(BAR(sh.bar.q_empty[st]), ph ^ 1)) { failed = true; break; }
                const uint32_t qf = BAR(sh.bar.q_full[st]), qd = smem_u32(q_s + st * BIG_BYTES);
                mbar_expect_tx(qf, BIG_BYTES);
                tma_load_4d(qd, &tm_q, qf, 0, h, q0, b);
                if constexpr (HD > 64) tma_load_4d(qd + BIG_HALF, &tm_q, qf, 64, h, q0, b);
                const int gst = t % DOS, gph = (t / DOS) & 1;
                if (!mbar_wait(BAR(sh.bar.do_empty[gst]), gph ^ 1)) { failed = true; break; }
                const uint32_t gf = BAR(sh.bar.do_full[gst]), gd = smem_u32(do_s + gst * BIG_BYTES);
                mbar_expect_tx(gf, BIG_BYTES);
                tma_load_4d(gd, &tm_do, gf, 0, h, q0, b);
                if constexpr (HD > 64) tma_load_4d(gd + BIG_HALF, &tm_do, gf, 64, h, q0, b);
            }
        }
    } else if (warp == KAUX_WARP) {
        // ---------------- the per-query vectors of each step: log-sum-exp, delta, key interval ----------------
        // The gathers of step t + 1 are issued (all of them, from clamped rows, before anything
        // looks at their values) ahead of the work on step t, so that no step waits for a trip to L2.
        constexpr int RPL = QS / 32;   // rows per lane
        float lse_n[RPL], dl_n[RPL];
        auto gather = [&](int t) {
            const int h = hk * group + t / tiles, q0 = qfirst + (t % tiles) * QS;
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
            const int st = t & 1, ph = (t >> 1) & 1;
            const int q0 = qfirst + (t % tiles) * QS;
            float lse_c[RPL], dl_c[RPL];
#pragma unroll
            for (int i = 0; i < RPL; ++i) { lse_c[i] = lse_n[i]; dl_c[i] = dl_n[i]; }
            if (t + 1 < steps) gather(t + 1);
            float l2v[RPL], dlv[RPL];
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const bool in = q0 + lane + 32 * i < a.tq;
                l2v[i] = (!in || lse_c[i] == -INFINITY) ? INFINITY : lse_c[i] * LOG2E;
                dlv[i] = in ? dl_c[i] : 0.f;
            }
            // aux[st] is free when the Q stage is: the elementwise threads of step t - 2 are done with it.
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.q_empty[st]), ph ^ 1))) { failed = true; break; }
            QAux &aux = sh.aux[st];
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int c = lane + 32 * i;
                aux.lse2[c] = l2v[i];
                aux.delta[c] = dlv[i];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(sh.bar.aux_full[st]));
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        if (steps > 0) {
            constexpr uint32_t IDESC_SC = idesc_f16(BIG, QS, Pack<T>::FMT, 0, 0);     // [128 keys x 128 queries]
            constexpr uint32_t IDESC_ACC = idesc_f16(BIG, HD, Pack<T>::FMT, 0, 1);    // [128 keys x 128 d], B MN-major
            const uint64_t k_desc = smem_desc_sw128(smem_u32(k_s), 16, 1024), v_desc = smem_desc_sw128(smem_u32(v_s), 16, 1024);
            // Fused: dQ = dS K with both operands MN-major: A = the dS^T tile (rows = keys = the product's K
            // dimension, 64 queries to a 128-byte row, the second 64 queries BIG_HALF further on), B = the
            // resident K read along its rows.
            constexpr uint32_t IDESC_DQ = idesc_f16(QS, HD, Pack<T>::FMT, 1, 1);   // [128 queries x HD]
            const uint64_t ds_desc = smem_desc_sw128(smem_u32(ds_s), BIG_HALF, 1024), k_mn = smem_desc_sw128(smem_u32(k_s), BIG_HALF, 1024);
            // The 16 queries of k-step ks of a gradient product, as 16-bit pairs in tensor memory.
            auto a_cols = [](int ks) { return static_cast<uint32_t>(32 * (ks >> 1) + 8 * (ks & 1)); };
            auto scores = [&](int t) -> bool {   // S^T(t) = K Q^T
                const int st = t & 1, ph = (t >> 1) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.q_full[st]), ph))) return false;
                tc_fence_after_sync();
                const uint64_t qk = smem_desc_sw128(smem_u32(q_s + st * BIG_BYTES), 16, 1024);
                const uint32_t full = BAR(sh.bar.s_full);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks)
                        umma_f16(tmem + COL_ST, desc_at(k_desc, (ks >> 2) * BIG_HALF + (ks & 3) * 32),
                                 desc_at(qk, (ks >> 2) * BIG_HALF + (ks & 3) * 32), IDESC_SC, ks > 0 ? 1u : 0u);
                    umma_commit(full);
                }
                __syncwarp();
                return true;
            };
            auto dscores = [&](int t) -> bool {  // dP^T(t) = V dO^T
                const int st = t % DOS, ph = (t / DOS) & 1;
                // Fused: dQ(t - 1) sits in these columns until the reduction warps have taken it out.
                if (FUSED && t > 0 && !__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.dq_taken), (t - 1) & 1))) return false;
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.do_full[st]), ph))) return false;
                tc_fence_after_sync();
                const uint64_t gk = smem_desc_sw128(smem_u32(do_s + st * BIG_BYTES), 16, 1024);
                const uint32_t full = BAR(sh.bar.dp_full);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks)
                        umma_f16(tmem + COL_DPT, desc_at(v_desc, (ks >> 2) * BIG_HALF + (ks & 3) * 32),
                                 desc_at(gk, (ks >> 2) * BIG_HALF + (ks & 3) * 32), IDESC_SC, ks > 0 ? 1u : 0u);
                    umma_commit(full);
                }
                __syncwarp();
                return true;
            };
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.res_full), 0))) failed = true;
            if (!failed && !(scores(0) && dscores(0))) failed = true;
            for (int t = 0; t < steps && !failed; ++t) {
                const int st = t & 1, ph = t & 1;
                // dV += P^T dO over the step's 128 queries, the even k-steps (the first half of every
                // elementwise thread's columns) as soon as they are written, the odd ones behind the
                // second half; the dO stage is free behind it.
                {
                    const uint64_t gm = smem_desc_sw128(smem_u32(do_s + (t % DOS) * BIG_BYTES), BIG_HALF, 1024);
                    const uint32_t e = BAR(sh.bar.do_empty[t % DOS]);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.p_full[half]), ph))) { failed = true; break; }
                        tc_fence_after_sync();
                        if (elect_one()) {
#pragma unroll
                            for (int ks = half; ks < QS / 16; ks += 2)
                                umma_f16_ts(tmem + COL_DV, tmem + COL_ST + a_cols(ks), desc_at(gm, ks * 2048), IDESC_ACC,
                                            (t > 0 || ks > 0) ? 1u : 0u);
                            if (half == 1) umma_commit(e);
                        }
                        __syncwarp();
                    }
                    if (failed) break;
                }
                if (t + 1 < steps && !scores(t + 1)) { failed = true; break; }
                // dK += dS^T Q likewise; the Q stage is free behind it.
                {
                    const uint64_t qm = smem_desc_sw128(smem_u32(q_s + st * BIG_BYTES), BIG_HALF, 1024);
                    const uint32_t e = BAR(sh.bar.q_empty[st]);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.ds_full[half]), ph))) { failed = true; break; }
                        tc_fence_after_sync();
                        if (elect_one()) {
#pragma unroll
                            for (int ks = half; ks < QS / 16; ks += 2)
                                umma_f16_ts(tmem + COL_DK, tmem + COL_DPT + a_cols(ks), desc_at(qm, ks * 2048), IDESC_ACC,
                                            (t > 0 || ks > 0) ? 1u : 0u);
                            if (half == 1) umma_commit(e);
                        }
                        __syncwarp();
                    }
                    if (failed) break;
                }
                if constexpr (FUSED) {
                    // dQ(t) = dS K over the step's 128 keys, into the columns of dP^T: both halves of dS^T
                    // are in the shared-memory tile (the waits of dK above), dK(t) has been issued.
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < BIG / 16; ++ks)
                            umma_f16(tmem + COL_DPT, desc_at(ds_desc, ks * 2048), desc_at(k_mn, ks * 2048), IDESC_DQ, ks > 0 ? 1u : 0u);
                        umma_commit(BAR(sh.bar.dq_done));
                    }
                    __syncwarp();
                }
                if (t + 1 < steps && !dscores(t + 1)) { failed = true; break; }
            }
            if (!failed && elect_one()) umma_commit(BAR(sh.bar.acc_ready));
        }
    } else if (FUSED && warp >= KRED_WARP) {
        // ---------------- fused: dQ(t) out of tensor memory and into the f32 accumulator ----------------
        // A thread owns a query row (TMEM lane); 64 columns at a time go through the two staging slots
        // (the layout of a 128-byte-swizzled TMA box of 32 f32 columns x 128 rows) and leave as two
        // bulk tensor reductions, which add whole lines in L2 and drop rows past the last query.
        const int lane_base = 32 * (warp & 3), r = lane_base + lane;
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(lane_base) << 16);
        const bool issuer = warp == KRED_WARP && lane == 0;
        for (int t = 0; t < steps && !failed; ++t) {
            const int h = hk * group + t / tiles, q0 = qfirst + (t % tiles) * QS;
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.dq_done), t & 1))) { failed = true; break; }
            tc_fence_after_sync();
#pragma unroll
            for (int pair = 0; pair < HD / 64; ++pair) {
                uint32_t x[2][32];
                tmem_ld32(t_lane + COL_DPT + pair * 64, x[0]);
                tmem_ld32(t_lane + COL_DPT + pair * 64 + 32, x[1]);
                tmem_ld_wait();
                if (pair == HD / 64 - 1) {   // all of dQ(t) is in registers or staged: dP^T(t+1) may overwrite it
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(sh.bar.dq_taken));
                }
                // The slots are free once the reductions issued from them have read them.
                if (issuer) tma_store_wait_read();
                named_barrier(1, 128);
#pragma unroll
                for (int sl = 0; sl < 2; ++sl) {
                    uint8_t *row = red_s + sl * RED_SLOT + r * 128;
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        *reinterpret_cast<uint4 *>(row + ((e ^ (r & 7)) << 4)) =
                            make_uint4(x[sl][4 * e + 0], x[sl][4 * e + 1], x[sl][4 * e + 2], x[sl][4 * e + 3]);
                }
                fence_proxy_async_smem();
                named_barrier(1, 128);
                if (issuer) {
                    tma_reduce_add_4d(&tm_dq_acc, smem_u32(red_s), pair * 64, h, q0, b);
                    tma_reduce_add_4d(&tm_dq_acc, smem_u32(red_s + RED_SLOT), pair * 64 + 32, h, q0, b);
                    tma_store_commit();
                }
            }
        }
        if (issuer) tma_store_wait_read();   // shared memory must not go while a reduction still reads it
    } else {
        // ---------------- elementwise: a key row and 32 of the step's queries per thread ----------------
        const int lane_base = 32 * (warp & 3);
        const int cg = (warp - 2) >> 2, col0 = cg * KQW;
        const int r = lane_base + lane;
        const int key = k0 + r;
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(lane_base) << 16);
        // The queries that see this thread's key: one interval for the whole sweep (empty for a
        // padded key), so a step needs masking only where its columns leave that interval.
        int qa = 0, qb = 0;
        if (key < a.tk && !key_padded(a.mask, b, key)) queries_of_key(qmask, key, a.tq, a.tk, qa, qb);
        for (int t = 0; t < steps && !failed; ++t) {
            const int st = t & 1, aph = (t >> 1) & 1, ph = t & 1;
            const int c0 = qfirst + (t % tiles) * QS + col0;   // the first query of this thread's columns
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.aux_full[st]), aph) && mbar_wait(BAR(sh.bar.s_full), ph))) {
                failed = true;
                break;
            }
            tc_fence_after_sync();
            float p[KQW];
            tmem_ld32(t_lane + COL_ST + col0, *reinterpret_cast<uint32_t(*)[32]>(&p[0]));
            tmem_ld_wait();
            const QAux &aux = sh.aux[st];
            const bool all_of_them = c0 >= qa && c0 + KQW <= qb;
            if (!__all_sync(0xffffffffu, all_of_them)) {
                // Some key of the warp is not seen by all of these queries: hide what it is not seen by
                // before the exponentials, in a pass of its own so that the common, unmasked step pays
                // nothing for it.  A key that is seen by NONE of them - a key of another sequence of the
                // packed batch, in a block of keys that straddles two - needs no comparisons: where every key
                // of the warp is seen by all or by none, those rows are simply set.
                const bool none_of_them = c0 + KQW <= qa || c0 >= qb || qb <= qa;
                if (__all_sync(0xffffffffu, all_of_them || none_of_them)) {
                    if (none_of_them) {
#pragma unroll
                        for (int c = 0; c < KQW; ++c) p[c] = -INFINITY;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < KQW; ++c) p[c] = (c0 + c >= qa && c0 + c < qb) ? p[c] : -INFINITY;
                }
            }
            // P^T over the first half of the f32 columns this thread has just read, in two halves of
            // 16 queries (8 columns): the tensor cores start on the first while the second is made.
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t pk[KQW / 4];
#pragma unroll
                for (int c4 = 0; c4 < KQW / 8; ++c4) {
                    const int c = half * (KQW / 2) + c4 * 4;
                    const float4 l2 = *reinterpret_cast<const float4 *>(&aux.lse2[col0 + c]);
                    p[c + 0] = exp2_mixed<(poly_of4<T>() > 3)>(fmaf(p[c + 0], a.scale_log2, -l2.x));
                    p[c + 1] = exp2_mixed<(poly_of4<T>() > 1)>(fmaf(p[c + 1], a.scale_log2, -l2.y));
                    p[c + 2] = exp2_mixed<(poly_of4<T>() > 2)>(fmaf(p[c + 2], a.scale_log2, -l2.z));
                    p[c + 3] = exp2_mixed<(poly_of4<T>() > 0)>(fmaf(p[c + 3], a.scale_log2, -l2.w));
                    pk[c4 * 2 + 0] = Pack<T>::two(p[c + 0], p[c + 1]);
                    pk[c4 * 2 + 1] = Pack<T>::two(p[c + 2], p[c + 3]);
                }
                tmem_st8(t_lane + COL_ST + col0 + half * (KQW / 4), pk);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(sh.bar.p_full[half]));
            }

            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.dp_full), ph))) { failed = true; break; }
            tc_fence_after_sync();
            {
                float dp[KQW];
                tmem_ld32(t_lane + COL_DPT + col0, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
                tmem_ld_wait();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t dk[KQW / 4];
#pragma unroll
                    for (int c4 = 0; c4 < KQW / 8; ++c4) {
                        const int c = half * (KQW / 2) + c4 * 4;
                        const float4 dl = *reinterpret_cast<const float4 *>(&aux.delta[col0 + c]);
                        dk[c4 * 2 + 0] = Pack<T>::two(p[c + 0] * (dp[c + 0] - dl.x), p[c + 1] * (dp[c + 1] - dl.y));
                        dk[c4 * 2 + 1] = Pack<T>::two(p[c + 2] * (dp[c + 2] - dl.z), p[c + 3] * (dp[c + 3] - dl.w));
                    }
                    tmem_st8(t_lane + COL_DPT + col0 + half * (KQW / 4), dk);   // dS^T likewise, in the same two halves
                    if constexpr (FUSED) {
                        // ... and into the shared-memory tile dQ reads it from: this key's row of the 64-query
                        // half that holds the thread's columns, two 16-byte chunks of 8 queries, XOR-swizzled by
                        // the row like a TMA tile.  The tile is free: dQ of the step before was issued ahead of
                        // this step's dP^T, whose completion (awaited above) means every earlier MMA has completed.
                        uint8_t *ds_row = ds_s + (cg >> 1) * BIG_HALF + r * 128;
#pragma unroll
                        for (int e2 = 0; e2 < 2; ++e2) {
                            const int chunk = (cg & 1) * 4 + half * 2 + e2;
                            *reinterpret_cast<uint4 *>(ds_row + ((chunk ^ (r & 7)) << 4)) =
                                make_uint4(dk[4 * e2 + 0], dk[4 * e2 + 1], dk[4 * e2 + 2], dk[4 * e2 + 3]);
                        }
                        fence_proxy_async_smem();
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(sh.bar.ds_full[half]));
                }
            }
        }
        // ---------------- epilogue: 32 columns of the row per thread (HD = 64: the first two of the four warps of a quadrant) ----------------
        constexpr int EC = 32;
        const bool mine = cg < HD / EC;
        T *dk = static_cast<T *>(a.dk) + (((int64_t)b * a.tk + key) * a.hkv + hk) * HD + cg * EC;
        T *dv = static_cast<T *>(a.dv) + (((int64_t)b * a.tk + key) * a.hkv + hk) * HD + cg * EC;
        if (steps == 0 || failed) {
            if (key < a.tk && !failed && mine) {
                store_zero_cols<T, EC / 8>(dk);
                store_zero_cols<T, EC / 8>(dv);
            }
        } else if (__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.acc_ready), 0))) {
            tc_fence_after_sync();
            if (mine) {
                store_acc_cols<T>(t_lane + COL_DV + cg * EC, dv, 1.f, key < a.tk, 1);
                store_acc_cols<T>(t_lane + COL_DK + cg * EC, dk, a.scale, key < a.tk, 1);
            }
            tc_fence_before_sync();
        } else {
            failed = true;
        }
    }

    if (threadIdx.x == 0 && steps == 0 && !mbar_wait(BAR(sh.bar.res_full), 0)) failed = true;
    if (failed && !aborted) atomicOr(&g_sm100_bwd_status, 2u);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// =================================================================================================
// dQ
// =================================================================================================
// Steps of 128 keys: S = Q_i K^T and dP = dO_i V^T are 128 x 128 x 128 products, dS is written over
// the f32 dP it was made from (two 16-bit values per 32-bit column) and dQ += dS K reads it from
// tensor memory.  S is single in tensor memory - the elementwise threads take it into registers at
// the start of a step, which frees it for the next step's product - and dP is double, so that both
// score products of step t + 1 are issued ahead of dQ of step t and the tensor cores never wait for
// the elementwise work of the step they feed.  With both scores of step t + 1 ready early, a fast
// warp can finish that step before a slow one has finished step t: the barrier the warps arrive on
// when dS is written is therefore double as well (one per buffer).
constexpr int DQ_KS = 3;   // stages of the K ring: a K tile serves S of its step and, a step and a half later, dQ

// dq: two elementwise warps per TMEM lane quadrant, 64 keys of a step per thread (measured on config 2: 573 us
// against 586 with four warps of 32 keys each; turns at the exponentials, as in the forward, cost 18 us here).
constexpr int QCG = 2;
constexpr int QW = BIG / QCG;
constexpr int QEW_THREADS = 32 * 4 * QCG;
static_assert(QW % 32 == 0, "whole 32-column TMEM loads per thread");

struct DqBarriers {
    uint64_t res_full;
    uint64_t k_full[DQ_KS], k_empty[DQ_KS], v_full[2], v_empty[2];
    uint64_t s_full, s_free, dp_full[2], ds_full[2];
    uint64_t acc_ready;
};

struct DqTail {
    DqBarriers bar;
    uint32_t tmem_base;
    unsigned int abort;
    int red_lo[4 * QCG], red_hi[4 * QCG];
    int tile_bad;   // an elementwise warp gave up: dQ of the tile is not stored
};

constexpr size_t DQ_TAIL = 1024;
static_assert(sizeof(DqTail) <= DQ_TAIL, "the tail of the dq kernel's shared memory");
// 1 KiB slack | Q, dO resident (2 x 32 KiB) | K ring 3 x 32 KiB | V ring 2 x 32 KiB | tail
template <int HD> constexpr size_t smem_dq() { return 1024 + (4 + DQ_KS) * tile_bytes<HD>() + DQ_TAIL; }
constexpr int DQ_THREADS = 32 * (2 + 4 * QCG);

template <typename T, int HD>
__global__ void __launch_bounds__(DQ_THREADS, 1)
bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_dq, const Sm100BwdArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int BIG_BYTES = tile_bytes<HD>();
    uint8_t *q_s = smem, *do_s = q_s + BIG_BYTES;
    uint8_t *k_s = do_s + BIG_BYTES;          // [DQ_KS][BIG_BYTES]
    uint8_t *v_s = k_s + DQ_KS * BIG_BYTES;   // [2][BIG_BYTES]
    DqTail &sh = *reinterpret_cast<DqTail *>(v_s + 2 * BIG_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x;
    const int qt = gridDim.y - 1 - blockIdx.y;
    const int b = blockIdx.z;
    const int hk = h / (a.hq / a.hkv);
    const int m0 = qt * BIG;
    auto BAR = [&](uint64_t &x) { return smem_u32(&x); };

    if (threadIdx.x == 0) {
        sh.abort = *reinterpret_cast<volatile unsigned int *>(&g_sm100_bwd_status);
        sh.tile_bad = 0;
        mbar_init(BAR(sh.bar.res_full), 1);
        for (int i = 0; i < DQ_KS; ++i) {
            mbar_init(BAR(sh.bar.k_full[i]), 1);
            mbar_init(BAR(sh.bar.k_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(sh.bar.v_full[i]), 1);
            mbar_init(BAR(sh.bar.v_empty[i]), 1);
            mbar_init(BAR(sh.bar.dp_full[i]), 1);
            mbar_init(BAR(sh.bar.ds_full[i]), 4 * QCG);
        }
        mbar_init(BAR(sh.bar.s_full), 1);
        mbar_init(BAR(sh.bar.s_free), 4 * QCG);    // one arrival per elementwise warp
        mbar_init(BAR(sh.bar.acc_ready), 1);
        fence_mbar_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_do);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_dq);
        // The resident tiles are on their way before the block knows which keys it sweeps: their
        // flight covers the rest of the setup.  (A block that turns out to have nothing to do waits
        // for them at the end: shared memory must not be written behind a block that has left.)
        const uint32_t full = BAR(sh.bar.res_full);
        mbar_expect_tx(full, 2 * BIG_BYTES);
        tma_load_4d(smem_u32(q_s), &tm_q, full, 0, h, m0, b);
        if constexpr (HD > 64) tma_load_4d(smem_u32(q_s + BIG_HALF), &tm_q, full, 64, h, m0, b);
        tma_load_4d(smem_u32(do_s), &tm_do, full, 0, h, m0, b);
        if constexpr (HD > 64) tma_load_4d(smem_u32(do_s + BIG_HALF), &tm_do, full, 64, h, m0, b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
    }
    const int sw = warp - 2;
    const int lane_base = 32 * (warp & 3);
    const int r = lane_base + lane;
    int lo = a.tk, hi = 0;
    if (warp >= 2) {
        row_bounds_warp(a.mask, m0 + r, a.tq, a.tk, lo, hi);
        int wlo = warp_min_i(hi > lo ? lo : a.tk), whi = warp_max_i(hi > lo ? hi : 0);
        if (lane == 0) { sh.red_lo[sw] = wlo; sh.red_hi[sw] = whi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    const bool aborted = sh.abort != 0;
    int kmin = a.tk, kmax = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { kmin = min(kmin, sh.red_lo[i]); kmax = max(kmax, sh.red_hi[i]); }  // the first four warps cover every row
    const int steps = (!aborted && kmax > kmin) ? (kmax - kmin + BIG - 1) / BIG : 0;
    bool failed = aborted;
    // TMEM columns: S at 0, dP[2] at 128 / 256 (dS over the first half of every group of 32 columns), dQ at 384.
    constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 384;

    if (warp == 0) {
        if (lane == 0 && steps > 0) {
            for (int t = 0; t < steps; ++t) {
                const int st = t & 1, ph = (t >> 1) & 1, c0 = kmin + t * BIG;
                const int ks = t % DQ_KS, kph = (t / DQ_KS) & 1;
                if (!mbar_wait(BAR(sh.bar.k_empty[ks]), kph ^ 1)) { failed = true; break; }
                const uint32_t kf = BAR(sh.bar.k_full[ks]), kd = smem_u32(k_s + ks * BIG_BYTES);
                mbar_expect_tx(kf, BIG_BYTES);
                tma_load_4d(kd, &tm_k, kf, 0, hk, c0, b);
                if constexpr (HD > 64) tma_load_4d(kd + BIG_HALF, &tm_k, kf, 64, hk, c0, b);
                if (!mbar_wait(BAR(sh.bar.v_empty[st]), ph ^ 1)) { failed = true; break; }
                const uint32_t vf = BAR(sh.bar.v_full[st]), vd = smem_u32(v_s + st * BIG_BYTES);
                mbar_expect_tx(vf, BIG_BYTES);
                tma_load_4d(vd, &tm_v, vf, 0, hk, c0, b);
                if constexpr (HD > 64) tma_load_4d(vd + BIG_HALF, &tm_v, vf, 64, hk, c0, b);
            }
        }
    } else if (warp == 1) {
        // MMA issuer: the whole warp runs the loop, one elected lane issues.
        if (steps > 0) {
            constexpr uint32_t IDESC_SC = idesc_f16(BIG, BIG, Pack<T>::FMT, 0, 0);    // [128 queries x 128 keys]
            constexpr uint32_t IDESC_ACC = idesc_f16(BIG, HD, Pack<T>::FMT, 0, 1);    // [128 queries x 128 d], B MN-major
            const uint64_t q_desc = smem_desc_sw128(smem_u32(q_s), 16, 1024), g_desc = smem_desc_sw128(smem_u32(do_s), 16, 1024);
            auto a_cols = [](int ks) { return static_cast<uint32_t>(32 * (ks >> 1) + 8 * (ks & 1)); };
            // S(t) = Q K^T once the elementwise threads have taken S(t - 1), and dP(t) = dO V^T into buffer t & 1.
            auto scores = [&](int t) -> bool {
                const int st = t & 1, ph = (t >> 1) & 1;
                if (t > 0 && !__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.s_free), (t - 1) & 1))) return false;
                const int kst = t % DQ_KS, kph = (t / DQ_KS) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.k_full[kst]), kph))) return false;
                tc_fence_after_sync();
                const uint64_t kk = smem_desc_sw128(smem_u32(k_s + kst * BIG_BYTES), 16, 1024);
                const uint32_t sf = BAR(sh.bar.s_full);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks)
                        umma_f16(tmem + COL_S, desc_at(q_desc, (ks >> 2) * BIG_HALF + (ks & 3) * 32),
                                 desc_at(kk, (ks >> 2) * BIG_HALF + (ks & 3) * 32), IDESC_SC, ks > 0 ? 1u : 0u);
                    umma_commit(sf);
                }
                __syncwarp();
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.v_full[st]), ph))) return false;
                tc_fence_after_sync();
                const uint64_t vk = smem_desc_sw128(smem_u32(v_s + st * BIG_BYTES), 16, 1024);
                const uint32_t df = BAR(sh.bar.dp_full[st]), ve = BAR(sh.bar.v_empty[st]);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks)
                        umma_f16(tmem + COL_DP + st * BIG, desc_at(g_desc, (ks >> 2) * BIG_HALF + (ks & 3) * 32),
                                 desc_at(vk, (ks >> 2) * BIG_HALF + (ks & 3) * 32), IDESC_SC, ks > 0 ? 1u : 0u);
                    umma_commit(df);
                    umma_commit(ve);
                }
                __syncwarp();
                return true;
            };
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.res_full), 0))) failed = true;
            if (!failed && !scores(0)) failed = true;
            for (int t = 0; t < steps && !failed; ++t) {
                const int st = t & 1;
                if (t + 1 < steps && !scores(t + 1)) { failed = true; break; }
                // dQ += dS K over the step's 128 keys; the K stage is free behind it.
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.ds_full[st]), (t >> 1) & 1))) { failed = true; break; }
                tc_fence_after_sync();
                const uint64_t km = smem_desc_sw128(smem_u32(k_s + (t % DQ_KS) * BIG_BYTES), BIG_HALF, 1024);
                const uint32_t ke = BAR(sh.bar.k_empty[t % DQ_KS]);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < BIG / 16; ++ks)
                        umma_f16_ts(tmem + COL_DQ, tmem + COL_DP + st * BIG + a_cols(ks), desc_at(km, ks * 2048), IDESC_ACC,
                                    (t > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(ke);
                }
                __syncwarp();
            }
            if (!failed && elect_one()) umma_commit(BAR(sh.bar.acc_ready));
        }
    } else {
        // ---------------- elementwise: a query row and QW of the step's keys per thread ----------------
        const int row = m0 + r;
        const int cg = sw >> 2, col0 = cg * QW;
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(lane_base) << 16);
        const bool padded = a.mask.kind == 1;
        float l2 = INFINITY, dl = 0.f;
        if (row < a.tq) {
            const int64_t at = ((int64_t)b * a.tq + row) * a.hq + h;
            const float x = a.lse[at];
            l2 = x == -INFINITY ? INFINITY : x * LOG2E;
            dl = a.delta[at];
        }
        for (int t = 0; t < steps && !failed; ++t) {
            const int st = t & 1, c0 = kmin + t * BIG + col0;
            uint32_t pb[QW / 32];
#pragma unroll
            for (int g = 0; g < QW / 32; ++g) {
                pb[g] = 0;
                if (padded) {
                    const int key = c0 + 32 * g + lane;
                    pb[g] = __ballot_sync(0xffffffffu, key >= a.tk || key_padded(a.mask, b, key));
                }
            }
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.s_full), t & 1))) { failed = true; break; }
            tc_fence_after_sync();
            float p[QW];
#pragma unroll
            for (int g = 0; g < QW / 32; ++g) tmem_ld32(t_lane + COL_S + col0 + 32 * g, *reinterpret_cast<uint32_t(*)[32]>(&p[32 * g]));
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(sh.bar.s_free));

            const bool clear = !padded && c0 >= lo && c0 + QW <= hi;
            // ... or sees none of them: a row of another sequence of the packed batch (a tile that straddles two
            // sequences sweeps the first one's keys for the second one's rows too), or one whose interval ends
            // before these keys.  Such a row needs no masking pass: against +inf its exponentials are exact zeros.
            const bool none = !padded && (hi <= c0 || lo >= c0 + QW || hi <= lo);
            if (!__all_sync(0xffffffffu, clear || none)) {
#pragma unroll
                for (int c = 0; c < QW; ++c) {
                    const int key = c0 + c;
                    p[c] = (key >= lo && key < hi && !((pb[c >> 5] >> (c & 31)) & 1u)) ? p[c] : -INFINITY;
                }
            }
            const float off = none ? INFINITY : l2;
#pragma unroll
            for (int c = 0; c < QW; ++c) p[c] = ex2(fmaf(p[c], a.scale_log2, -off));
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.dp_full[st]), (t >> 1) & 1))) { failed = true; break; }
            tc_fence_after_sync();
#pragma unroll
            for (int g = 0; g < QW / 32; ++g) {
                float dp[32];
                tmem_ld32(t_lane + COL_DP + st * BIG + col0 + 32 * g, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
                tmem_ld_wait();
                uint32_t ds[16];
#pragma unroll
                for (int c2 = 0; c2 < 16; ++c2)
                    ds[c2] = Pack<T>::two(p[32 * g + 2 * c2] * (dp[2 * c2] - dl), p[32 * g + 2 * c2 + 1] * (dp[2 * c2 + 1] - dl));
                tmem_st16(t_lane + COL_DP + st * BIG + col0 + 32 * g, ds);   // over the first half of the f32 columns just read
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(sh.bar.ds_full[st]));
        }
        // ---------------- epilogue: the row's HD columns over the quadrant's warps, 32 at a time ----------------
        constexpr int EC = 32;
        constexpr int PER = (HD / EC + QCG - 1) / QCG;   // 32-column chunks of the row per warp of the quadrant
        if (steps == 0 || failed) {
            if (row < a.tq && !failed) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int ch = cg * PER + i;
                    if (ch < HD / EC) store_zero_cols<T, EC / 8>(static_cast<T *>(a.dq) + (((int64_t)b * a.tq + row) * a.hq + h) * HD + ch * EC);
                }
            }
        } else if (__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.acc_ready), 0))) {
            // Every MMA has completed, so the resident Q is dead: the scaled rows of dQ are staged
            // over it in the layout of the TMA box and leave as two bulk stores (whole lines instead
            // of 64 bytes per thread and row; rows past the last query are dropped).
            tc_fence_after_sync();
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int ch = cg * PER + i;   // 32-column chunk of the row
                if (ch < HD / EC) {
                    uint32_t o[32];
                    tmem_ld32(t_lane + COL_DQ + ch * EC, o);
                    tmem_ld_wait();
                    uint8_t *half_row = q_s + (ch >> 1) * BIG_HALF + r * 128;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        uint4 v;
                        v.x = Pack<T>::two(__uint_as_float(o[8 * e + 0]) * a.scale, __uint_as_float(o[8 * e + 1]) * a.scale);
                        v.y = Pack<T>::two(__uint_as_float(o[8 * e + 2]) * a.scale, __uint_as_float(o[8 * e + 3]) * a.scale);
                        v.z = Pack<T>::two(__uint_as_float(o[8 * e + 4]) * a.scale, __uint_as_float(o[8 * e + 5]) * a.scale);
                        v.w = Pack<T>::two(__uint_as_float(o[8 * e + 6]) * a.scale, __uint_as_float(o[8 * e + 7]) * a.scale);
                        const int chunk = (ch & 1) * 4 + e;   // 16-byte chunk of the half row
                        *reinterpret_cast<uint4 *>(half_row + ((chunk ^ (r & 7)) << 4)) = v;
                    }
                }
            }
            tc_fence_before_sync();
        } else {
            failed = true;
        }
        if (steps > 0) {
            // Every elementwise warp gets here (all waits are bounded), whatever became of it: one
            // that gave up marks the tile, and nothing is stored from a tile that is not whole.
            if (failed && lane == 0) sh.tile_bad = 1;
            fence_proxy_async_smem();
            named_barrier(1, QEW_THREADS);
            if (sw == 0 && lane == 0 && sh.tile_bad == 0) {
                tma_store_4d(&tm_dq, smem_u32(q_s), 0, h, m0, b);
                if constexpr (HD > 64) tma_store_4d(&tm_dq, smem_u32(q_s + BIG_HALF), 64, h, m0, b);
                tma_store_commit();
                tma_store_wait_read();
            }
        }
    }

    if (threadIdx.x == 0 && steps == 0 && !mbar_wait(BAR(sh.bar.res_full), 0)) failed = true;
    if (failed && !aborted) atomicOr(&g_sm100_bwd_status, 4u);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// =================================================================================================
// The fused form's finish: the f32 accumulator, scaled, in the gradient's dtype
// =================================================================================================
template <typename T>
__global__ void __launch_bounds__(256) bwd_dq_finish_kernel(const float *__restrict__ acc, T *__restrict__ dq, float scale, long long n8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // eight elements per thread
    if (i >= n8) return;
    const float4 lo = reinterpret_cast<const float4 *>(acc)[2 * i], hi = reinterpret_cast<const float4 *>(acc)[2 * i + 1];
    uint4 v;
    v.x = Pack<T>::two(lo.x * scale, lo.y * scale);
    v.y = Pack<T>::two(lo.z * scale, lo.w * scale);
    v.z = Pack<T>::two(hi.x * scale, hi.y * scale);
    v.w = Pack<T>::two(hi.z * scale, hi.w * scale);
    reinterpret_cast<uint4 *>(dq)[i] = v;
}

// -------------------------------------------------------------------------------------------------
template <typename T, int HD, bool FUSED>
static cudaError_t launch_dkdv(const Sm100BwdMaps &m, const Sm100BwdArgs &a, long long items, cudaStream_t stream) {
    constexpr size_t smem = smem_dkdv<HD, FUSED>();
    cudaError_t e = cudaFuncSetAttribute(bwd_dkdv_sm100_kernel<T, HD, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 gk((unsigned)(items * a.hkv), 1, 1);
    bwd_dkdv_sm100_kernel<T, HD, FUSED><<<gk, FUSED ? KTHREADS_FUSED : KTHREADS, smem, stream>>>(m.k128, m.v128, m.q128, m.do128, m.dq_acc, a);
    return cudaGetLastError();
}

template <typename T, int HD>
static cudaError_t launch_t(const Sm100BwdMaps &m, Sm100BwdArgs a, cudaStream_t stream, int *launches) {
    const bool fused = a.dq_acc != nullptr;
    cudaError_t e;
    const long long dq_elems = (long long)a.b * a.tq * a.hq * HD;
    if (fused) {
        // The accumulator starts at zero; every key block adds its share as it gets there.
        if ((e = cudaMemsetAsync(a.dq_acc, 0, sizeof(float) * (size_t)dq_elems, stream)) != cudaSuccess) return e;
    } else {
        e = cudaFuncSetAttribute(bwd_dq_sm100_kernel<T, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq<HD>());
        if (e != cudaSuccess) return e;
        dim3 gq(a.hq, (a.tq + BIG - 1) / BIG, a.b);
        bwd_dq_sm100_kernel<T, HD><<<gq, DQ_THREADS, smem_dq<HD>(), stream>>>(m.q128, m.do128, m.k128, m.v128, m.dq128, a);
        *launches += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    const long long items = (long long)a.b * ((a.tk + BIG - 1) / BIG);
    if ((e = launch_bwd_plan(a, stream, launches)) != cudaSuccess) return e;
    if (items * a.hkv > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    e = fused ? launch_dkdv<T, HD, true>(m, a, items, stream) : launch_dkdv<T, HD, false>(m, a, items, stream);
    *launches += 1;
    if (e != cudaSuccess || !fused) return e;
    const long long n8 = dq_elems / 8;
    bwd_dq_finish_kernel<T><<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(a.dq_acc, static_cast<T *>(a.dq), a.scale, n8);
    *launches += 1;
    return cudaGetLastError();
}

size_t bwd_sm100_fused_shared_bytes(int d) { return d == 64 ? smem_dkdv<64, true>() : smem_dkdv<128, true>(); }

cudaError_t read_sm100_bwd_status(unsigned int *status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_sm100_bwd_status, sizeof(unsigned int));
    if (e != cudaSuccess) return e;
    if (clear && *status) {
        unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_sm100_bwd_status, &zero, sizeof(unsigned int));
    }
    return e;
}

cudaError_t launch_bwd_sm100(int dtype, const Sm100BwdMaps &m, const Sm100BwdArgs &a, cudaStream_t stream, int *launches) {
    if (dtype == DASH_ATTN_BF16)
        return a.d == 64 ? launch_t<__nv_bfloat16, 64>(m, a, stream, launches) : launch_t<__nv_bfloat16, 128>(m, a, stream, launches);
    return a.d == 64 ? launch_t<__half, 64>(m, a, stream, launches) : launch_t<__half, 128>(m, a, stream, launches);
}

}  // namespace dash
