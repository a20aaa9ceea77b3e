// Sampling the next token on the device, as crates/dash-contract/src/sample.rs:1-96 defines it:
// from the logits [B, V] of one position per sequence, one token per row and its log-probability
// under the model's distribution, the model's at the temperature, and the one it was drawn from;
// temperature, top-k, top-p and masked ids; greedy at temperature 0; Gumbel-max with
// Philox4x32-10 words, counter (i / 4, row, offset), word i % 4 (crates/dash-ops/src/sample/philox.rs).
//
// One thread-block cluster per row (1 to 8 blocks of 1024 threads, as many as fill the GPU at the
// call's batch; their partial results meet through distributed shared memory), the row read from
// L2 in each pass (a row of 128 Ki bf16 logits is 256 KiB):
//   1. the row's maximum over the unmasked tokens, 2. sum exp(z - m) -> the log-sum-exp,
//   3. the cuts as ONE threshold on the logits' order-preserving integer keys, found by a radix
//      search from the top byte down: top-k's is the largest key T with |{key >= T}| >= k, top-p's
//      the largest T (at or above top-k's) whose tempered mass reaches p of the mass top-k keeps -
//      every token tied with the last one is kept by construction, as the definition wants.  Two
//      passes for 16-bit logits (their keys are their own 16 bits), four for f32, and all but the
//      first look only at the tokens that share the bytes found so far;
//   4. argmax over the kept tokens of s_i + g_i, ties to the lowest id, four tokens per Philox call;
//   5. the three log-probabilities, taken from one another where the definition says they are one
//      number (tau = 1; nothing cut).
// Every sum is formed in a fixed order - each thread its strided elements in sequence, then a
// tree over the lanes and the warps, then the cluster's blocks in rank order - so the same call gives the same bits on every run, and the
// rounding grows with log V as in the reference's trees of pairs (reference.rs:198-214).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sample.h"

namespace dash {
namespace {

namespace cg = cooperative_groups;

constexpr int ST = 1024;   // threads per block; a row has 1 to 8 blocks (a cluster)

// A row's logits as f32 and as integers in the logits' order.
template <typename T> struct Key;
template <> struct Key<float> {
    static constexpr int BITS = 32;
    static __device__ __forceinline__ uint32_t of(float x) {
        const uint32_t u = __float_as_uint(x);
        return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    }
};
template <> struct Key<__nv_bfloat16> {
    static constexpr int BITS = 16;
    static __device__ __forceinline__ uint32_t of(__nv_bfloat16 x) {
        const uint32_t u = __bfloat16_as_ushort(x);
        return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
    }
};
template <> struct Key<__half> {
    static constexpr int BITS = 16;
    static __device__ __forceinline__ uint32_t of(__half x) {
        const uint32_t u = __half_as_ushort(x);
        return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
    }
};

struct MaxOp { __device__ float operator()(float a, float b) const { return fmaxf(a, b); } };
struct AddOp { template <typename X> __device__ X operator()(X a, X b) const { return a + b; } };
struct MinOp { __device__ int operator()(int a, int b) const { return min(a, b); } };

// The block's reduction of one value per thread, in a fixed order; every thread gets the result.
template <typename X, typename Op>
__device__ __forceinline__ X block_reduce(X x, Op op, X *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = op(x, __shfl_xor_sync(0xffffffffu, x, o));
    __syncthreads();   // the scratch of the reduction before is read
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    x = scratch[lane];   // ST / 32 = 32 warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = op(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

// The row's reduction: the block's, then the cluster's blocks in rank order through distributed
// shared memory (`slot` is one value per block).
template <typename X, typename Op>
__device__ __forceinline__ X row_reduce(X x, Op op, X *scratch, X *slot) {
    x = block_reduce(x, op, scratch);
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned blocks = cluster.num_blocks();
    if (blocks == 1) return x;
    if (threadIdx.x == 0) *slot = x;
    cluster.sync();
    X r = *cluster.map_shared_rank(slot, 0);
    for (unsigned b = 1; b < blocks; ++b) r = op(r, *cluster.map_shared_rank(slot, b));
    cluster.sync();   // every block has read before a slot is written again
    return r;
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                              uint32_t out[4]) {
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        if (round > 0) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
        const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
        const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
        c0 = h1 ^ c1 ^ k0;
        c1 = l1;
        c2 = h0 ^ c3 ^ k1;
        c3 = l0;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// The standard Gumbel variate of a Philox word (sample.rs "Random numbers"; the operations and
// their order are reference.rs:255-285's): u = (x + 1/2) / 2^32, E = -ln u computed from
// a = (2y + 1) / 2^33 as -ln a below one half and -ln_1p(-a), a = 1 - u, above; g = -ln E.
__device__ __forceinline__ float gumbel_of_word(uint32_t x) {
    const bool upper = (x >> 31) == 1;
    const uint32_t y = upper ? ~x : x;
    const float a = __fmul_rn(static_cast<float>((y << 1) | 1u), __uint_as_float(0x2F000000u));
    float e;
    if (!upper) {
        e = -logf(a);
    } else if (a <= 0.015625f) {
        e = __fmul_rn(a, __fdiv_rn(__fadd_rn(-a, 6.0f), __fadd_rn(__fmul_rn(a, -4.0f), 6.0f)));
    } else {
        const float w = __fadd_rn(-a, 1.0f);
        e = __fmul_rn(-logf(w), __fdiv_rn(a, __fadd_rn(-w, 1.0f)));
    }
    return -logf(e);
}

// Every token of the row once, thread by thread: 16 bytes of logits a load where the rows allow it
// (eight 16-bit logits or four f32 to a thread at a time), one logit a load otherwise.
template <typename T, typename F>
__device__ __forceinline__ void for_each_logit(const T *z, int v, int tid, int TS, bool vec, F f) {
    constexpr int E = 16 / sizeof(T);
    int done = 0;
    if (vec) {
        const int nv = v / E;
        for (int j = tid; j < nv; j += TS) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(z + (size_t)j * E);
            const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
            for (int k = 0; k < E; ++k) f(j * E + k, e[k]);
        }
        done = nv * E;
    }
    for (int i = done + tid; i < v; i += TS) f(i, z[i]);
}

// Shared memory of the threshold search: a histogram of 256 bins per warp (counts, and tempered
// masses in fixed point: integer sums do not depend on the order the atomics land in, so the search
// gives the same threshold on every run), and the block's totals, which the cluster's other blocks read.
struct RadixSmem {
    // 32 copies of each bin: copy c of bin d at [c / 4][d][c % 4]; a thread uses copy 4 (warp / 4) + lane % 4, so
    // that the lanes of a warp that meet in one bin (16-bit logits crowd into a few top bytes) spread over four words.
    uint32_t cnt[8][256][4];
    // A mass (41 bits of fixed point) as three pieces of 14, 14 and 13 bits in three 32-bit words: 32-bit
    // shared-memory atomics are native, 64-bit ones are not, and a copy's few thousand tokens cannot overflow a piece.
    uint32_t mass[3][8][256][4];
    uint32_t tcnt[256];
    unsigned long long tmass[256];
    uint32_t sel, above_cnt;
    unsigned long long above_mass, target;
};
constexpr float MASS_ONE = 1099511627776.0f;   // 2^40: a weight in (0, 1] as an integer

// The largest key T such that the tokens with key >= T (and >= floor_key) number at least `k`
// (MASS false), or hold at least p of the tempered mass of all tokens >= floor_key, and are at
// least one (MASS true): a radix search, eight bits of the key per pass from the top, in which only
// the tokens that share the bits found so far are looked at again.  Masked tokens count as -inf
// for top-k (they sort last, as in the reference) and take no part in the masses.
template <typename T, bool MASS>
__device__ uint32_t radix_threshold(const T *z, const SampleArgs &a, const uint32_t *bits, int tid, int TS, float m, uint32_t floor_key,
                                    RadixSmem &sm) {
    cg::cluster_group cluster = cg::this_cluster();
    const int blocks = (int)cluster.num_blocks();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t key_ninf = Key<T>::of(Num<T>::from_f32(-INFINITY));
    uint32_t prefix = 0, above_cnt = 0;
    unsigned long long above_mass = 0, target = 0;
    for (int level = 0; level < Key<T>::BITS / 8; ++level) {
        const int shift = Key<T>::BITS - 8 * (level + 1);
        for (int i = threadIdx.x; i < 32 * 256; i += ST) {
            (&sm.cnt[0][0][0])[i] = 0;
            if (MASS) { (&sm.mass[0][0][0][0])[i] = 0; (&sm.mass[1][0][0][0])[i] = 0; (&sm.mass[2][0][0][0])[i] = 0; }
        }
        __syncthreads();
        for_each_logit(z, a.v, tid, TS, a.vec != 0, [&](int i, T zi) {
            const bool gone = bits != nullptr && ((bits[i >> 5] >> (i & 31)) & 1u) != 0;
            if (MASS && gone) return;
            const uint32_t key = gone ? key_ninf : Key<T>::of(zi);
            if (key < floor_key) return;
            if (level > 0 && (key >> (shift + 8)) != prefix) return;
            const uint32_t d = (key >> shift) & 255u;
            if (MASS) {
                // Weights under 2^-41 round to nothing and are left out (the largest logit's is 1).
                const unsigned long long w = __float2ull_rn(expf(__fmul_rn(Num<T>::to_f32(zi) - m, a.tau)) * MASS_ONE);
                if (w == 0) return;
                atomicAdd(&sm.mass[0][warp >> 2][d][lane & 3], (uint32_t)(w & 0x3fffu));
                if (w >> 14) atomicAdd(&sm.mass[1][warp >> 2][d][lane & 3], (uint32_t)((w >> 14) & 0x3fffu));
                if (w >> 28) atomicAdd(&sm.mass[2][warp >> 2][d][lane & 3], (uint32_t)(w >> 28));
            }
            atomicAdd(&sm.cnt[warp >> 2][d][lane & 3], 1u);
        });
        __syncthreads();
        if (threadIdx.x < 256) {
            uint32_t c = 0;
            unsigned long long w = 0;
            for (int x = 0; x < 32; ++x) {
                c += sm.cnt[x >> 2][threadIdx.x][x & 3];
                if (MASS) w += (unsigned long long)sm.mass[0][x >> 2][threadIdx.x][x & 3] + ((unsigned long long)sm.mass[1][x >> 2][threadIdx.x][x & 3] << 14) +
                               ((unsigned long long)sm.mass[2][x >> 2][threadIdx.x][x & 3] << 28);
            }
            sm.tcnt[threadIdx.x] = c;
            sm.tmass[threadIdx.x] = w;
        }
        if (blocks > 1) {
            cluster.sync();
            uint32_t c = 0;
            unsigned long long w = 0;
            if (threadIdx.x < 256) {
                for (int r = 0; r < blocks; ++r) {
                    c += *cluster.map_shared_rank(&sm.tcnt[threadIdx.x], r);
                    if (MASS) w += *cluster.map_shared_rank(&sm.tmass[threadIdx.x], r);
                }
            }
            cluster.sync();   // every block has read the others' totals
            if (threadIdx.x < 256) { sm.tcnt[threadIdx.x] = c; sm.tmass[threadIdx.x] = w; }
        }
        __syncthreads();
        if (warp == 0) {
            // Lane l holds bins 255 - 8 l down to 248 - 8 l: the higher bins on the lower lanes.
            uint32_t c8 = 0;
            unsigned long long w8 = 0;
            for (int x = 0; x < 8; ++x) { c8 += sm.tcnt[255 - 8 * lane - x]; w8 += sm.tmass[255 - 8 * lane - x]; }
            uint32_t c_before = c8;
            unsigned long long w_before = w8;
            for (int o = 1; o < 32; o <<= 1) {   // inclusive sums over the lanes up to this one
                const uint32_t cu = __shfl_up_sync(0xffffffffu, c_before, o);
                const unsigned long long wu = __shfl_up_sync(0xffffffffu, w_before, o);
                if (lane >= o) { c_before += cu; w_before += wu; }
            }
            if (MASS && level == 0) {
                const unsigned long long total = __shfl_sync(0xffffffffu, w_before, 31);
                target = __double2ull_ru((double)a.p * (double)total);
            }
            uint32_t run_c = above_cnt + c_before - c8;
            unsigned long long run_w = above_mass + w_before - w8;
            int hit = -1;
            uint32_t hit_c = 0;
            unsigned long long hit_w = 0;
            for (int x = 0; x < 8 && hit < 0; ++x) {
                const int d = 255 - 8 * lane - x;
                const uint32_t nc = run_c + sm.tcnt[d];
                const unsigned long long nw = run_w + sm.tmass[d];
                if (MASS ? (nw >= target && nc >= 1u) : (nc >= (uint32_t)a.top_k)) { hit = d; hit_c = run_c; hit_w = run_w; }
                run_c = nc;
                run_w = nw;
            }
            const unsigned vote = __ballot_sync(0xffffffffu, hit >= 0);
            const int src = vote ? __ffs(vote) - 1 : 31;   // the lowest lane: the highest bin
            if (lane == src) {
                sm.sel = hit >= 0 ? (uint32_t)hit : 0u;
                sm.above_cnt = hit >= 0 ? hit_c : run_c;
                sm.above_mass = hit >= 0 ? hit_w : run_w;
                sm.target = target;
            }
        }
        __syncthreads();
        prefix = (prefix << 8) | sm.sel;
        above_cnt = sm.above_cnt;
        above_mass = sm.above_mass;
        target = sm.target;
        __syncthreads();   // read before the next level writes
    }
    return prefix;
}

template <typename T>
__global__ void __launch_bounds__(ST) sample_kernel(SampleArgs a) {
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ float fslot;
    __shared__ int islot;
    extern __shared__ __align__(16) uint8_t radix_raw[];
    RadixSmem &radix = *reinterpret_cast<RadixSmem *>(radix_raw);
    cg::cluster_group cluster = cg::this_cluster();
    const int blocks = (int)cluster.num_blocks();
    const int row = blockIdx.x / blocks, tid = (int)cluster.block_rank() * ST + threadIdx.x;
    const int TS = blocks * ST;   // the row's threads
    const T *z = static_cast<const T *>(a.logits) + (int64_t)row * a.stride;
    const uint32_t *bits = a.masked_bits;
    auto masked = [&](int i) { return bits != nullptr && ((bits[i >> 5] >> (i & 31)) & 1u) != 0; };
    const uint32_t key_ninf = Key<T>::of(Num<T>::from_f32(-INFINITY));

    // 1. m = max over the unmasked tokens; 2. sum exp(z - m) (and, tempered, sum exp((z - m) tau)).
    float m = -INFINITY;
    for_each_logit(z, a.v, tid, TS, a.vec != 0, [&](int i, T zi) {
        if (!masked(i)) m = fmaxf(m, Num<T>::to_f32(zi));
    });
    m = row_reduce(m, MaxOp(), fs, &fslot);
    const bool degenerate = m == -INFINITY;   // no finite unmasked logit: the lowest unmasked id, NaN
    const bool tempered_differs = !a.greedy && a.tau != 1.0f;
    float s1 = 0.f, wu = 0.f;
    int first = a.v;   // the lowest unmasked id holding the maximum
    for_each_logit(z, a.v, tid, TS, a.vec != 0, [&](int i, T zi) {
        if (masked(i)) return;
        const float x = Num<T>::to_f32(zi);
        s1 += expf(x - m);
        if (tempered_differs) wu += expf((x - m) * a.tau);
        if (x == m && i < first) first = i;
    });
    s1 = row_reduce(s1, AddOp(), fs, &fslot);
    if (tempered_differs) wu = row_reduce(wu, AddOp(), fs, &fslot);
    const float lse = m + logf(s1);

    int token = 0;
    float tempered = 0.f, sampling = 0.f;
    bool own_tempered = true, own_sampling = true;   // false: the value is another output's (same bits)
    if (a.greedy || degenerate) {
        token = row_reduce(first, MinOp(), is, &islot);
    } else {
        // 3. The cuts: one threshold T on the keys; 0 keeps every token.
        uint32_t t_keep = 0;
        const bool cut = a.top_k > 0 || a.has_p;
        if (a.top_k > 0) t_keep = radix_threshold<T, false>(z, a, bits, tid, TS, m, 0u, radix);
        if (a.has_p) t_keep = max(t_keep, radix_threshold<T, true>(z, a, bits, tid, TS, m, t_keep, radix));

        // 4. argmax of s + g over the kept tokens, ties to the lowest id; the kept tokens' mass.
        float best = -INFINITY, wp = 0.f, reach = -3.2f;
        int best_i = a.v;
        // g lies within [-3.13, 22.9] (the words' range) and the winner scores at least `reach` (this thread's
        // best so far; the row's largest logit, always kept, alone reaches -3.13), so a token with s < reach - 22.95
        // is never drawn - at the start that is 26.1 below the largest logit, the contract's own bound: it adds to
        // the mass and skips the generator and the logarithms.
        // Four tokens (one Philox call) at a time: `zs` their logits, read by the caller.
        auto draw4 = [&](int g, const T (&zs)[4]) {
            float s4[4];
            bool draw = false;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 4 * g + e;
                s4[e] = -INFINITY;
                if (i >= a.v || masked(i) || Key<T>::of(zs[e]) < t_keep) continue;
                s4[e] = __fmul_rn(Num<T>::to_f32(zs[e]) - m, a.tau);
                if (cut) wp += expf(s4[e]);
                draw = draw || s4[e] >= reach - 22.95f;
            }
            if (!draw) return;
            uint32_t w[4];
            philox4x32_10((uint32_t)g, (uint32_t)row, a.off_lo, a.off_hi, a.key0, a.key1, w);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 4 * g + e;
                if (!(s4[e] >= reach - 22.95f)) continue;
                // g rises with the word, so most tokens are out of the running by their word alone: the winner
                // scores at least `reach` (this thread's best so far; the row's largest logit alone reaches -3.13),
                // and g < c exactly when u < exp(-exp(-c)).  With c = reach - s - 0.001 > 0 and a thousandth off
                // the threshold, the two fast exponentials (relative error under 1e-5 here) can only let a token
                // through that the exact variate then weighs, never turn one away that could win or tie.
                const float c = reach - s4[e] - 1e-3f;
                if (c > 0.f) {
                    const float u = (static_cast<float>(w[e]) + 0.5f) * 2.3283064365386963e-10f;
                    if (u < __expf(-__expf(-c)) * 0.999f) continue;
                }
                const float score = __fadd_rn(s4[e], gumbel_of_word(w[e]));
                if (score > best || (score == best && i < best_i) || best_i == a.v) { best = score; best_i = i; }
                reach = fmaxf(reach, best);
            }
        };
        constexpr int E = 16 / sizeof(T);   // logits to a 16-byte load: one or two groups of four
        int g0 = 0;
        if (a.vec) {
            const int nv = a.v / E;
            for (int j = tid; j < nv; j += TS) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(z + (size_t)j * E);
                const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
                for (int sub = 0; sub < E / 4; ++sub) {
                    const T zs[4] = {e[4 * sub], e[4 * sub + 1], e[4 * sub + 2], e[4 * sub + 3]};
                    draw4(j * (E / 4) + sub, zs);
                }
            }
            g0 = nv * (E / 4);
        }
        for (int g = g0 + tid; g < (a.v + 3) / 4; g += TS) {
            T zs[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) zs[e] = 4 * g + e < a.v ? z[4 * g + e] : z[0];
            draw4(g, zs);
        }
        // (score, id) pairs: the larger score, then the lower id.
        {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            auto better = [](float sa, int ia, float sb, int ib) { return ib != INT_MAX && (ia == INT_MAX || sb > sa || (sb == sa && ib < ia)); };
            if (best_i == a.v) best_i = INT_MAX;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float sb = __shfl_xor_sync(0xffffffffu, best, o);
                const int ib = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (better(best, best_i, sb, ib)) { best = sb; best_i = ib; }
            }
            __syncthreads();
            if (lane == 0) { fs[warp] = best; is[warp] = best_i; }
            __syncthreads();
            best = fs[lane];
            best_i = is[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float sb = __shfl_xor_sync(0xffffffffu, best, o);
                const int ib = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (better(best, best_i, sb, ib)) { best = sb; best_i = ib; }
            }
            if (blocks > 1) {
                if (threadIdx.x == 0) { fslot = best; islot = best_i; }
                cluster.sync();
                best = *cluster.map_shared_rank(&fslot, 0);
                best_i = *cluster.map_shared_rank(&islot, 0);
                for (int b = 1; b < blocks; ++b) {
                    const float sb = *cluster.map_shared_rank(&fslot, b);
                    const int ib = *cluster.map_shared_rank(&islot, b);
                    if (better(best, best_i, sb, ib)) { best = sb; best_i = ib; }
                }
                cluster.sync();
            }
        }
        token = best_i == INT_MAX ? 0 : best_i;
        if (cut) wp = row_reduce(wp, AddOp(), fs, &fslot);
        const float s_t = __fmul_rn(Num<T>::to_f32(z[token]) - m, a.tau);
        if (tempered_differs) tempered = s_t - logf(wu); else own_tempered = false;
        if (cut) sampling = s_t - logf(wp); else own_sampling = false;
    }
    if (tid == 0) {   // the first thread of the row's first block
        const float logprob = Num<T>::to_f32(z[token]) - lse;
        if (!a.greedy || degenerate) {
            if (!own_tempered || degenerate) tempered = logprob;
            if (!own_sampling || degenerate) sampling = tempered;
        }
        if (degenerate) tempered = sampling = __int_as_float(0x7fc00000);
        if (a.token_bytes == 8) static_cast<int64_t *>(a.tokens)[row] = token;
        else static_cast<int32_t *>(a.tokens)[row] = token;
        a.logprob[row] = logprob;
        a.tempered[row] = tempered;
        a.sampling[row] = sampling;
    }
}

}  // namespace

template <typename T>
static cudaError_t launch_t(const SampleArgs &a, int blocks, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.b * blocks), 1, 1);
    cfg.blockDim = dim3(ST, 1, 1);
    cfg.stream = stream;
    cfg.dynamicSmemBytes = sizeof(RadixSmem);
    cudaError_t e = cudaFuncSetAttribute(sample_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(RadixSmem));
    if (e != cudaSuccess) return e;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)blocks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sample_kernel<T>, a);
}

cudaError_t launch_sample(int dtype, const SampleArgs &a, cudaStream_t stream, int *launches) {
    if (a.b == 0) return cudaSuccess;
    // As many blocks to a row as fill the multiprocessors at this batch (one block of 1024 threads
    // each), a power of two up to the portable cluster size; short rows take one.
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int blocks = 1;
    while (blocks < 8 && (int64_t)a.b * blocks * 2 <= sms && a.v >= blocks * 2 * ST * 4) blocks *= 2;
    cudaError_t e;
    switch (dtype) {
        case 0: e = launch_t<float>(a, blocks, stream); break;
        case 1: e = launch_t<__nv_bfloat16>(a, blocks, stream); break;
        default: e = launch_t<__half>(a, blocks, stream); break;
    }
    *launches += 1;
    return e;
}

}  // namespace dash
