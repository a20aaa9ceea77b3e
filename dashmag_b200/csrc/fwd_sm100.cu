// The training forward on the 5th-generation tensor cores: bf16 / f16, head dimension 128.
//
// One block of 224 threads per (tile of 128 queries, query head):
//   warp 0, 6   one lane each issues the TMA tile loads: warp 0 the Q tile once and then the K
//               tiles of 128 keys, warp 6 the V tiles, into two-stage rings of 128-byte-swizzled
//               shared memory;
//   warp 1      owns tensor memory (512 columns: two S buffers and the O accumulator) and one lane
//               issues the tcgen05 MMAs: S_j = Q K_j^T into the S buffer (j mod 2), O += P_j V_j;
//   warps 2..5  128 softmax threads, one query row each (TMEM lane = row): read S_j from tensor
//               memory, mask what the row does not see, keep the online softmax in f32 with the
//               scale folded into an exp2, write P_j rounded to the input dtype back into tensor
//               memory over the first half of the S buffer they read (two 16-bit values per
//               32-bit column: the A operand of P V comes from tensor memory), and at the end
//               normalise O and store it with the row's log-sum-exp.
// The S buffer is double, so QK^T of the next key tile runs under the softmax of the current one,
// and P V of the current one under the softmax of the next; a buffer is free for S_{j+2} once
// P_j V_j has completed.
//
// The running maximum is "lazy": the accumulator is rescaled only when a row's maximum grows by
// more than 2^8, otherwise the stale maximum stays the reference of the exponentials (their sum and
// the accumulator carry the same factor, which the final division removes).  The log-sum-exp is
// formed in f32 from that reference and the f32 sum.
//
// Masks: every query's visible keys are one interval (common.cuh); a block sweeps the key tiles of
// the union of its rows' intervals, elementwise masking runs only on tiles that cut some row's
// interval or carry key padding, and out-of-range rows and keys are zero-filled by the TMA loads.
// Every wait on an mbarrier is bounded; a wait that runs out raises a status flag the host can
// read and the block leaves through the common teardown, so a fault in the pipeline cannot hang.
#include <cuda.h>

#include "common.cuh"
#include "sm100.h"
#include "sm100_kernels.h"
#include "sm100_ptx.cuh"

namespace dash {

using namespace ptx;

__device__ unsigned int g_sm100_status = 0;  // sticky: non-zero once any bounded wait has run out

namespace {

constexpr int BM = 128;          // queries per block
constexpr int BN = 128;          // keys per tile
constexpr int HALF_BYTES = 128 * 128;  // one 64-column part of a tile: 128 rows of 128 bytes, what one TMA box brings
// Head dimension HD = 128, or 256 (this kernel only: two accumulators of 256 columns do not fit the
// two-tile kernel's tensor memory): a tile is HD / 64 parts, 32 KiB at 128, and at 256 the K and V
// rings have one stage each (Q + K + V = 192 KiB).
template <int HD> struct Geo1 {
    static constexpr int PARTS = HD / 64;
    static constexpr int TILE_BYTES = PARTS * HALF_BYTES;
    static constexpr int NS = HD > 128 ? 1 : 2;
    static constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + (1 + 2 * NS) * TILE_BYTES /*Q, K ring, V ring*/ + 1024 /*Shared*/;
};
constexpr int THREADS = 224;
constexpr float RESCALE_LOG2 = 8.0f;
// A row that sees at most this many keys keeps the exact running maximum instead of the lazy one:
// with few keys one of them often carries most of the weight, and only against the exact maximum is
// that key's probability exactly 1 before P is rounded to the input dtype - as in the reference's
// kernels, whose error bounds were measured on such rows.  Long rows, where the weights spread and
// the roundings average out, keep the lazy maximum and its rare rescales.
constexpr int EXACT_KEYS = 512;

struct Barriers {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2];
    uint64_t s_full[2], s_empty[2], p_full[2], o_ready;
};

struct Shared {
    Barriers bar;
    uint32_t tmem_base;
    int red_lo[4], red_hi[4];
    unsigned int abort;
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

}  // namespace

template <typename T, int HD>
__global__ void __launch_bounds__(THREADS, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Sm100FwdArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int PARTS = Geo1<HD>::PARTS, TILE_BYTES = Geo1<HD>::TILE_BYTES, NS = Geo1<HD>::NS;
    uint8_t *q_s = smem;
    uint8_t *k_s = q_s + TILE_BYTES;
    uint8_t *v_s = k_s + NS * TILE_BYTES;
    Shared &sh = *reinterpret_cast<Shared *>(v_s + NS * TILE_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x;
    const int qt = gridDim.y - 1 - blockIdx.y;  // later (longer, under causality) tiles first
    const int b = blockIdx.z;
    const int hk = h / (a.hq / a.hkv);
    const int m0 = qt * BM;

    const uint32_t q_full = smem_u32(&sh.bar.q_full), o_ready = smem_u32(&sh.bar.o_ready);
    auto BAR = [&](uint64_t (&arr)[2], int i) { return smem_u32(&arr[i]); };

    if (threadIdx.x == 0) {
        sh.abort = *reinterpret_cast<volatile unsigned int *>(&g_sm100_status);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(sh.bar.k_full, i), 1);
            mbar_init(BAR(sh.bar.k_empty, i), 1);
            mbar_init(BAR(sh.bar.v_full, i), 1);
            mbar_init(BAR(sh.bar.v_empty, i), 1);
            mbar_init(BAR(sh.bar.s_full, i), 1);
            mbar_init(BAR(sh.bar.s_empty, i), 1);
            mbar_init(BAR(sh.bar.p_full, i), 128);
        }
        mbar_init(o_ready, 1);
        fence_mbar_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
    }

    // Each softmax thread owns one query row; the block sweeps the union of its rows' intervals.
    const int sw = warp - 2;                       // 0..3 for softmax warps
    const int lane_base = 32 * (warp & 3);         // the TMEM lanes this warp may touch
    const int r = lane_base + lane;                // row of the tile (softmax threads)
    int lo = a.tk, hi = 0;
    if (warp >= 2 && warp < 6) {
        row_bounds_warp(a.mask, m0 + r, a.tq, a.tk, lo, hi);
        int wlo = warp_min_i(hi > lo ? lo : a.tk), whi = warp_max_i(hi > lo ? hi : 0);
        if (lane == 0) { sh.red_lo[sw] = wlo; sh.red_hi[sw] = whi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    int kmin = a.tk, kmax = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { kmin = min(kmin, sh.red_lo[i]); kmax = max(kmax, sh.red_hi[i]); }
    // Once a bounded wait has run out anywhere, later blocks do nothing: the call has failed and
    // the host will say so; there is no point in timing out thousands of times.
    const bool aborted = sh.abort != 0;
    const int n_tiles = (!aborted && kmax > kmin) ? (kmax - kmin + BN - 1) / BN : 0;
    bool failed = aborted;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_tiles > 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
            for (int part = 0; part < PARTS; ++part) tma_load_4d(smem_u32(q_s + part * HALF_BYTES), &tm_q, q_full, 64 * part, h, m0, b);
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int st = j % NS, ph = (j / NS) & 1, k0 = kmin + j * BN;
                if (!mbar_wait(BAR(sh.bar.k_empty, st), ph ^ 1)) { failed = true; break; }
                uint32_t full = BAR(sh.bar.k_full, st), dst = smem_u32(k_s + st * TILE_BYTES);
                mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
                for (int part = 0; part < PARTS; ++part) tma_load_4d(dst + part * HALF_BYTES, &tm_k, full, 64 * part, hk, k0, b);
            }
        }
    } else if (warp == 6) {
        // ---------------- TMA producer of the V ring (its own warp: a K tile is wanted long
        // before the V tile of the same keys, and neither load should queue behind the other) ----
        if (lane == 0 && n_tiles > 0) {
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int st = j % NS, ph = (j / NS) & 1, k0 = kmin + j * BN;
                if (!mbar_wait(BAR(sh.bar.v_empty, st), ph ^ 1)) { failed = true; break; }
                const uint32_t full = BAR(sh.bar.v_full, st), dst = smem_u32(v_s + st * TILE_BYTES);
                mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
                for (int part = 0; part < PARTS; ++part) tma_load_4d(dst + part * HALF_BYTES, &tm_v, full, 64 * part, hk, k0, b);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        if (n_tiles > 0) {
            constexpr uint32_t IDESC_S = idesc_f16(BM, BN, Pack<T>::FMT, 0, 0);   // A = Q, B = K, both K-major
            constexpr uint32_t IDESC_O = idesc_f16(BM, HD, Pack<T>::FMT, 0, 1);   // A = P K-major, B = V MN-major
            const uint64_t q_desc = smem_desc_sw128(smem_u32(q_s), 16, 1024);
            auto issue_pv = [&](int i) -> bool {
                const int st = i & 1, ph = (i >> 1) & 1;         // the S / P buffer of the tile
                const int vst = i % NS, vph = (i / NS) & 1;     // its V stage
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.v_full, vst), vph) && mbar_wait(BAR(sh.bar.p_full, st), ph)))
                    return false;
                tc_fence_after_sync();
                // A = P: 16 keys = 32 bytes along the swizzled row, the second 64 keys in the second half.
                // B = V: rows are keys (K of this product), 128 bytes of head dimension per row and half:
                // 64-column atoms HALF_BYTES apart (leading), 8-key groups 1024 bytes apart.
                const uint64_t v_desc = smem_desc_sw128(smem_u32(v_s + vst * TILE_BYTES), HALF_BYTES, 1024);
                const uint32_t v_empty = BAR(sh.bar.v_empty, vst), s_empty = BAR(sh.bar.s_empty, st);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < BN / 16; ++ks)
                        // A = P in tensor memory, over the S buffer it came from: 16 keys = 8 columns a step.
                        umma_f16_ts(tmem + 256, tmem + st * BN + ks * 8, desc_at(v_desc, ks * 2048), IDESC_O,
                                    (i > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(v_empty);
                    umma_commit(s_empty);   // the S buffer (now P) may be overwritten by S of tile i + 2
                    umma_commit(o_ready);
                }
                __syncwarp();
                return true;
            };
            if (!__all_sync(0xffffffffu, mbar_wait(q_full, 0))) failed = true;
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int st = j & 1, ph = (j >> 1) & 1;
                const int kst = j % NS, kph = (j / NS) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.k_full, kst), kph) && mbar_wait(BAR(sh.bar.s_empty, st), ph ^ 1))) {
                    failed = true;
                    break;
                }
                tc_fence_after_sync();
                const uint64_t k_desc = smem_desc_sw128(smem_u32(k_s + kst * TILE_BYTES), 16, 1024);
                const uint32_t k_empty = BAR(sh.bar.k_empty, kst), s_full = BAR(sh.bar.s_full, st);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        const uint32_t off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
                        umma_f16(tmem + st * BN, desc_at(q_desc, off), desc_at(k_desc, off), IDESC_S, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(k_empty);
                    umma_commit(s_full);
                }
                __syncwarp();
                if (j > 0 && !issue_pv(j - 1)) { failed = true; break; }
            }
            if (!failed && !issue_pv(n_tiles - 1)) failed = true;
        }
    } else {
        // ---------------- softmax, one row per thread ----------------
        const int row = m0 + r;
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(lane_base) << 16);
        const bool padded = a.mask.kind == 1;
        float m_ref = -INFINITY, l = 0.f;
        const float rescale_at = hi - lo <= EXACT_KEYS ? 0.f : RESCALE_LOG2;
        for (int j = 0; j < n_tiles && !failed; ++j) {
            const int st = j & 1, ph = (j >> 1) & 1, k0 = kmin + j * BN;
            uint32_t pb[4] = {0, 0, 0, 0};
            if (padded) {
                // The tile's 128 padding flags as four words; every warp gathers its own copy, so
                // that no softmax warp ever waits on another.
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = k0 + i * 32 + lane;
                    pb[i] = __ballot_sync(0xffffffffu, key >= a.tk || key_padded(a.mask, b, key));
                }
            }
            if (!__all_sync(0xffffffffu, mbar_wait(BAR(sh.bar.s_full, st), ph))) { failed = true; break; }
            tc_fence_after_sync();
            float s[BN];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(t_lane + st * BN + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            tmem_ld_wait();

            const bool clear = !padded && k0 >= lo && k0 + BN <= hi;  // the row sees the whole tile
            // ... or nothing of it (a row of another sequence of the packed batch, or one whose interval ends
            // before the tile): no look at its scores is needed, its maximum is -inf and its exponentials are
            // taken against -inf, which makes them exact zeros.
            const bool none = !padded && (hi <= k0 || lo >= k0 + BN || hi <= lo);
            if (!__all_sync(0xffffffffu, clear || none)) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
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
            for (int c = 24; c < BN; c += 16)
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    mx8[e] = c + 8 + e < BN ? fmax3(mx8[e], s[c + e], s[c + 8 + e]) : fmaxf(mx8[e], s[c + e]);
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

            uint32_t pk[BN / 2];  // P of this row, two keys per 32-bit column
            const float2 sl2 = make_float2(a.scale_log2, a.scale_log2), neg2 = make_float2(neg, neg);
            float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int cc = 0; cc < BN / 8; ++cc) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // two exponents per packed FMA, four independent packed sums
                    const float2 x = fma2(make_float2(s[cc * 8 + 2 * e], s[cc * 8 + 2 * e + 1]), sl2, neg2);
                    p[2 * e] = ex2(x.x);
                    p[2 * e + 1] = ex2(x.y);
                    sum2[e] = add2(sum2[e], make_float2(p[2 * e], p[2 * e + 1]));
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) pk[cc * 4 + e] = Pack<T>::two(p[2 * e], p[2 * e + 1]);
            }
            {
                const float2 t = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
                l += t.x + t.y;
            }

            // O holds tiles 0..j-1 once P V of tile j - 1 has completed; rescale it before P V of tile j.
            if (j > 0) {
                if (!__all_sync(0xffffffffu, mbar_wait(o_ready, (j - 1) & 1))) { failed = true; break; }
                if (__any_sync(0xffffffffu, rescale)) {
                    tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(t_lane + 256 + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
                        tmem_st32(t_lane + 256 + c * 32, o);
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                }
            }
            // P goes back into the first 64 columns of the S buffer it was read from.
            tmem_st32(t_lane + st * BN, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
            tmem_st32(t_lane + st * BN + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(BAR(sh.bar.p_full, st));
        }

        // ---------------- epilogue ----------------
        T *out = static_cast<T *>(a.out);
        const int64_t base = ((int64_t)b * a.tq + row) * a.hq + h;
        if (n_tiles == 0 || failed) {
            if (row < a.tq && !failed) {
                uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) reinterpret_cast<uint4 *>(out + base * HD)[c] = z;
                a.lse[base] = -INFINITY;
            }
        } else if (__all_sync(0xffffffffu, mbar_wait(o_ready, (n_tiles - 1) & 1))) {
            tc_fence_after_sync();
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(t_lane + 256 + c * 32, o);
                tmem_ld_wait();
                if (row < a.tq) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        uint4 v;
                        v.x = Pack<T>::two(__uint_as_float(o[8 * e + 0]) * inv, __uint_as_float(o[8 * e + 1]) * inv);
                        v.y = Pack<T>::two(__uint_as_float(o[8 * e + 2]) * inv, __uint_as_float(o[8 * e + 3]) * inv);
                        v.z = Pack<T>::two(__uint_as_float(o[8 * e + 4]) * inv, __uint_as_float(o[8 * e + 5]) * inv);
                        v.w = Pack<T>::two(__uint_as_float(o[8 * e + 6]) * inv, __uint_as_float(o[8 * e + 7]) * inv);
                        reinterpret_cast<uint4 *>(out + base * HD)[c * 4 + e] = v;
                    }
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
    }

    if (failed && !aborted) atomicOr(&g_sm100_status, 1u);
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
cudaError_t launch_fwd_t(dim3 grid, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const Sm100FwdArgs &a,
                         cudaStream_t stream) {
    constexpr size_t smem = Geo1<HD>::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(fwd_sm100_kernel<T, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    fwd_sm100_kernel<T, HD><<<grid, THREADS, smem, stream>>>(tq, tk, tv, a);
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_fwd_sm100(int dtype, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                             const Sm100FwdArgs &a, cudaStream_t stream) {
    dim3 grid(a.hq, (a.tq + BM - 1) / BM, a.b);
    if (dtype == DASH_ATTN_BF16)
        return a.d == 256 ? launch_fwd_t<__nv_bfloat16, 256>(grid, tq, tk, tv, a, stream)
                          : launch_fwd_t<__nv_bfloat16, 128>(grid, tq, tk, tv, a, stream);
    return a.d == 256 ? launch_fwd_t<__half, 256>(grid, tq, tk, tv, a, stream) : launch_fwd_t<__half, 128>(grid, tq, tk, tv, a, stream);
}

cudaError_t read_sm100_status(unsigned int *status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_sm100_status, sizeof(unsigned int));
    if (e != cudaSuccess) return e;
    if (clear && *status) {
        unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_sm100_status, &zero, sizeof(unsigned int));
        if (e != cudaSuccess) return e;
    }
    unsigned int bwd = 0, fwd2 = 0, bwd256 = 0;
    e = read_sm100_bwd_status(&bwd, clear);
    if (e != cudaSuccess) return e;
    e = read_sm100_bwd256_status(&bwd256, clear);
    if (e != cudaSuccess) return e;
    e = read_sm100_fwd2_status(&fwd2, clear);
    *status |= bwd | fwd2 | bwd256;
    return e;
}

}  // namespace dash
