// Sampling the next token on the device, as crates/dash-contract/src/sample.rs:1-96 defines it:
// from the logits [B, V] of one position per sequence, one token per row and its log-probability
// under the model's distribution, the model's at the temperature, and the one it was drawn from;
// temperature, top-k, top-p and masked ids; greedy at temperature 0; Gumbel-max with
// Philox4x32-10 words, counter (i / 4, row, offset), word i % 4 (crates/dash-ops/src/sample/philox.rs).
//
// One block per row, the row read from L2 in each pass (a row of 128 Ki bf16 logits is 256 KiB):
//   1. the row's maximum over the unmasked tokens, 2. sum exp(z - m) -> the log-sum-exp,
//   3. the cuts as ONE threshold on the logits' order-preserving integer keys, found by bisection
//      from the top bit down: top-k's is the largest key T with |{key >= T}| >= k, top-p's the
//      largest T (at or above top-k's) whose tempered mass reaches p of the mass top-k keeps - every
//      token tied with the last one is kept by construction, as the definition wants.  16 passes
//      for 16-bit logits (their keys are their own 16 bits), 32 for f32;
//   4. argmax over the kept tokens of s_i + g_i, ties to the lowest id, four tokens per Philox call;
//   5. the three log-probabilities, taken from one another where the definition says they are one
//      number (tau = 1; nothing cut).
// Every sum is formed in a fixed order - each thread its strided elements in sequence, then a
// tree over the lanes and the warps - so the same call gives the same bits on every run, and the
// rounding grows with log V as in the reference's trees of pairs (reference.rs:198-214).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sample.h"

namespace dash {
namespace {

constexpr int ST = 1024;   // threads per row

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

template <typename T>
__global__ void __launch_bounds__(ST) sample_kernel(SampleArgs a) {
    __shared__ float fs[32];
    __shared__ int is[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const T *z = static_cast<const T *>(a.logits) + (int64_t)row * a.stride;
    const uint32_t *bits = a.masked_bits;
    auto masked = [&](int i) { return bits != nullptr && ((bits[i >> 5] >> (i & 31)) & 1u) != 0; };
    const uint32_t key_ninf = Key<T>::of(Num<T>::from_f32(-INFINITY));

    // 1. m = max over the unmasked tokens; 2. sum exp(z - m) (and, tempered, sum exp((z - m) tau)).
    float m = -INFINITY;
    for (int i = tid; i < a.v; i += ST)
        if (!masked(i)) m = fmaxf(m, Num<T>::to_f32(z[i]));
    m = block_reduce(m, MaxOp(), fs);
    const bool degenerate = m == -INFINITY;   // no finite unmasked logit: the lowest unmasked id, NaN
    const bool tempered_differs = !a.greedy && a.tau != 1.0f;
    float s1 = 0.f, wu = 0.f;
    int first = a.v;   // the lowest unmasked id holding the maximum
    for (int i = tid; i < a.v; i += ST) {
        if (masked(i)) continue;
        const float x = Num<T>::to_f32(z[i]);
        s1 += expf(x - m);
        if (tempered_differs) wu += expf((x - m) * a.tau);
        if (x == m && i < first) first = i;
    }
    s1 = block_reduce(s1, AddOp(), fs);
    if (tempered_differs) wu = block_reduce(wu, AddOp(), fs);
    const float lse = m + logf(s1);

    int token = 0;
    float tempered = 0.f, sampling = 0.f;
    bool own_tempered = true, own_sampling = true;   // false: the value is another output's (same bits)
    if (a.greedy || degenerate) {
        token = block_reduce(first, MinOp(), is);
    } else {
        // 3. The cuts: one threshold T on the keys; 0 keeps every token.
        uint32_t t_keep = 0;
        const bool cut = a.top_k > 0 || a.has_p;
        if (a.top_k > 0) {
            for (int bit = Key<T>::BITS - 1; bit >= 0; --bit) {
                const uint32_t cand = t_keep | (1u << bit);
                int count = 0;
                for (int i = tid; i < a.v; i += ST) count += (masked(i) ? key_ninf : Key<T>::of(z[i])) >= cand ? 1 : 0;
                count = block_reduce(count, AddOp(), is);
                if (count >= a.top_k) t_keep = cand;
            }
        }
        if (a.has_p) {
            // The tempered mass of what top-k keeps, then the largest threshold whose mass reaches p of it.
            float wk = 0.f;
            for (int i = tid; i < a.v; i += ST)
                if (!masked(i) && Key<T>::of(z[i]) >= t_keep) wk += expf((Num<T>::to_f32(z[i]) - m) * a.tau);
            wk = block_reduce(wk, AddOp(), fs);
            const float target = __fmul_rn(wk, a.p);
            uint32_t t_p = 0;
            for (int bit = Key<T>::BITS - 1; bit >= 0; --bit) {
                const uint32_t cand = t_p | (1u << bit);
                float mass = 0.f;
                int any = 0;
                for (int i = tid; i < a.v; i += ST) {
                    if (masked(i)) continue;
                    const uint32_t k = Key<T>::of(z[i]);
                    if (k >= cand && k >= t_keep) {
                        mass += expf((Num<T>::to_f32(z[i]) - m) * a.tau);
                        any = 1;
                    }
                }
                mass = block_reduce(mass, AddOp(), fs);
                any = block_reduce(any, AddOp(), is);
                if (any > 0 && mass >= target) t_p = cand;
            }
            t_keep = max(t_keep, t_p);
        }

        // 4. argmax of s + g over the kept tokens, ties to the lowest id; the kept tokens' mass.
        float best = -INFINITY, wp = 0.f;
        int best_i = a.v;
        for (int g = tid; g < (a.v + 3) / 4; g += ST) {
            uint32_t w[4];
            philox4x32_10((uint32_t)g, (uint32_t)row, a.off_lo, a.off_hi, a.key0, a.key1, w);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 4 * g + e;
                if (i >= a.v || masked(i) || Key<T>::of(z[i]) < t_keep) continue;
                const float s = __fmul_rn(Num<T>::to_f32(z[i]) - m, a.tau);
                if (cut) wp += expf(s);
                const float score = __fadd_rn(s, gumbel_of_word(w[e]));
                if (score > best || (score == best && i < best_i) || best_i == a.v) { best = score; best_i = i; }
            }
        }
        // (score, id) pairs: the larger score, then the lower id.
        {
            const int lane = tid & 31, warp = tid >> 5;
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
        }
        token = best_i == INT_MAX ? 0 : best_i;
        if (cut) wp = block_reduce(wp, AddOp(), fs);
        const float s_t = __fmul_rn(Num<T>::to_f32(z[token]) - m, a.tau);
        if (tempered_differs) tempered = s_t - logf(wu); else own_tempered = false;
        if (cut) sampling = s_t - logf(wp); else own_sampling = false;
    }
    if (tid == 0) {
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

cudaError_t launch_sample(int dtype, const SampleArgs &a, cudaStream_t stream, int *launches) {
    if (a.b == 0) return cudaSuccess;
    switch (dtype) {
        case 0: sample_kernel<float><<<a.b, ST, 0, stream>>>(a); break;
        case 1: sample_kernel<__nv_bfloat16><<<a.b, ST, 0, stream>>>(a); break;
        default: sample_kernel<__half><<<a.b, ST, 0, stream>>>(a); break;
    }
    *launches += 1;
    return cudaGetLastError();
}

}  // namespace dash
