// Rotary position embedding from tables, the form of crates/dash-mag/src/rope.rs:94-107:
//
//     out = x * cos + rotate_half(x) * sin,   rotate_half(x) = (-x[half..dim], x[0..half])
//
// over the first `dim` features of every head, the features behind them unchanged.  The reference
// builds this from whole-tensor operations of the tensors' dtype, so each product and the sum is
// rounded once to that dtype; the kernel keeps exactly those three roundings (and, in f32, keeps
// the multiplications and the addition apart: no fused multiply-add), so its results are the
// reference's bit for bit.  One launch rotates two tensors that share their tokens' positions (the
// query and the key of a layer): the work is a read and a write of each, bound by HBM.
//
// The transpose (`inverse`) is what the gradient goes through:
//     dx[j]        = g[j] cos[j] + g[j + half] sin[j + half]
//     dx[j + half] = g[j + half] cos[j + half] - g[j] sin[j]
// with the same roundings (the reference's autograd multiplies the gradient by each table and adds
// the two parts).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "rope.h"

namespace dash {
namespace {

template <typename T> __device__ __forceinline__ float rnd(float x) { return Num<T>::to_f32(Num<T>::from_f32(x)); }
template <> __device__ __forceinline__ float rnd<float>(float x) { return x; }

template <typename T> struct Pair { using type = float2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Pair<__half> { using type = __half2; };

template <typename T> __device__ __forceinline__ T quiet_nan() { return Num<T>::from_f32(__int_as_float(0x7fc00000)); }

// x / d for non-negative x and a 32-bit d, in 32 bits when x fits.
__device__ __forceinline__ int64_t div_small(int64_t x, int d) {
    return (x >> 32) == 0 ? (int64_t)((uint32_t)x / (uint32_t)d) : x / d;
}

__device__ __forceinline__ int64_t mod_small(int64_t x, int64_t d) {
    return ((x | d) >> 32) == 0 ? (int64_t)((uint32_t)x % (uint32_t)d) : x % d;
}

__device__ __forceinline__ int64_t index_at(const void *p, int bytes, int64_t i) {
    return bytes == 8 ? static_cast<const int64_t *>(p)[i] : static_cast<int64_t>(static_cast<const int32_t *>(p)[i]);
}

// The position of token n; `rotate` false for a token of no sequence (packed tokens past the last
// offset), which passes through unchanged.
__device__ __forceinline__ int64_t position_of(const RopeArgs &a, int64_t n, bool &rotate) {
    rotate = true;
    if (a.positions) return index_at(a.positions, a.pos_bytes, n);
    if (a.cu) {
        // The last sequence whose offset is <= n.
        int lo = 0, hi = a.sequences;
        if (a.sequences <= 0 || n < index_at(a.cu, a.cu_bytes, 0) || n >= index_at(a.cu, a.cu_bytes, a.sequences)) {
            rotate = false;
            return 0;
        }
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (index_at(a.cu, a.cu_bytes, mid) <= n) lo = mid; else hi = mid;
        }
        return a.start + n - index_at(a.cu, a.cu_bytes, lo);
    }
    return a.start + (a.period > 0 ? mod_small(n, a.period) : 0);
}

// V elements of T moved as one 16-byte access (V = 1: as the element itself).
template <typename T, int V> struct alignas(sizeof(T) * V) VecOf { T e[V]; };
template <typename T, int V> __device__ __forceinline__ VecOf<T, V> load_vec(const T *p) {
    VecOf<T, V> v;
    if constexpr (sizeof(T) * V == 16) *reinterpret_cast<uint4 *>(&v) = *reinterpret_cast<const uint4 *>(p);
    else v.e[0] = *p;
    return v;
}
template <typename T, int V> __device__ __forceinline__ void store_vec(T *p, const VecOf<T, V> &v) {
    if constexpr (sizeof(T) * V == 16) *reinterpret_cast<uint4 *>(p) = *reinterpret_cast<const uint4 *>(&v);
    else *p = v.e[0];
}

// V = elements per thread and side of a pair: 16 bytes' worth, or 1 where the shapes or the
// addresses do not allow vectors.  A thread takes its columns of HG heads of one token (counted
// across both tensors): the position and the four table vectors are fetched once for them, and all
// of the heads' loads are issued before the first is used.  The heads of a thread are `hsub` apart
// and neighbouring threads take neighbouring heads, so that a warp's loads stay contiguous (the
// same heads dealt out in blocks of HG per thread measured 30-60 % slower: every load instruction
// of the GPU then strides through memory).
template <typename T, int V, int HG>
__global__ void __launch_bounds__(256) rope_kernel(RopeArgs a, int hsub) {
    const int half = a.dim / 2;
    const int pair_items = half / V, copy_items = (a.d - a.dim) / V;
    const int per_row = pair_items + copy_items;
    const int heads = a.a.heads + a.b.heads;
    const int chunk_heads = hsub * HG;
    const int chunks = (heads + chunk_heads - 1) / chunk_heads;
    // 64-bit divisions cost a hundred instructions each, and this kernel has few others: one at
    // most (none while the item count fits 32 bits), the rest in 32 bits.
    const int per_token = chunks * hsub * per_row;
    const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= a.tokens * per_token) return;
    const int64_t n = div_small(item, per_token);
    const int in_token = (int)(item - n * per_token);
    const int i = in_token % per_row;
    const int hs = (in_token / per_row) % hsub;
    const int h0 = (in_token / (per_row * hsub)) * chunk_heads + hs;

    using Vec = VecOf<T, V>;
    const bool pair = i < pair_items;
    const int c = pair ? i * V : a.dim + (i - pair_items) * V;
    const int c2 = pair ? c + half : c;   // the second column of the pair (a copied column has none)
    const T *src[HG];
    T *dst[HG];
    bool live[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
        const int hh = min(h0 + g * hsub, heads - 1);
        const RopeTensor &t = hh < a.a.heads ? a.a : a.b;
        const int h = hh < a.a.heads ? hh : hh - a.a.heads;
        src[g] = static_cast<const T *>(t.x) + n * t.st + h * t.sh;
        dst[g] = static_cast<T *>(t.out) + n * t.ost + h * t.osh;
        live[g] = h0 + g * hsub < heads && (pair || t.out != t.x);
    }
    Vec x1[HG], x2[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
        if (live[g]) {
            x1[g] = load_vec<T, V>(src[g] + c);
            if (pair) x2[g] = load_vec<T, V>(src[g] + c2);
        }
    }
    if (!pair) {
#pragma unroll
        for (int g = 0; g < HG; ++g)
            if (live[g]) store_vec<T, V>(dst[g] + c, x1[g]);
        return;
    }
    bool rotate;
    const int64_t pos = position_of(a, n, rotate);
    const bool known = pos >= 0 && pos < a.len;
    Vec c1, cc2, s1, s2;
    if (rotate && known) {
        const T *cs = static_cast<const T *>(a.cos) + pos * a.dim, *sn = static_cast<const T *>(a.sin) + pos * a.dim;
        c1 = load_vec<T, V>(cs + c);
        cc2 = load_vec<T, V>(cs + c2);
        s1 = load_vec<T, V>(sn + c);
        s2 = load_vec<T, V>(sn + c2);
    }
#pragma unroll
    for (int g = 0; g < HG; ++g) {
        if (!live[g]) continue;
        Vec y1, y2;
        if (!rotate) {
            y1 = x1[g];
            y2 = x2[g];
        } else if (!known) {
            // No such row in the tables: the reference leaves this to the caller; a NaN shows it.
#pragma unroll
            for (int e = 0; e < V; ++e) y1.e[e] = y2.e[e] = quiet_nan<T>();
        } else if constexpr (V > 1 && sizeof(T) == 2) {
            // Two columns at a time in the dtype's own arithmetic: a product of two 16-bit values and
            // a sum of two are each rounded once, which is what the f32 route below computes too.
            using P2 = typename Pair<T>::type;
            const P2 *u1 = reinterpret_cast<const P2 *>(&x1[g]), *u2 = reinterpret_cast<const P2 *>(&x2[g]);
            const P2 *k1 = reinterpret_cast<const P2 *>(&c1), *k2 = reinterpret_cast<const P2 *>(&cc2);
            const P2 *z1 = reinterpret_cast<const P2 *>(&s1), *z2 = reinterpret_cast<const P2 *>(&s2);
            P2 *r1 = reinterpret_cast<P2 *>(&y1), *r2 = reinterpret_cast<P2 *>(&y2);
#pragma unroll
            for (int e = 0; e < V / 2; ++e) {
                if (!a.inverse) {
                    r1[e] = __hadd2_rn(__hmul2_rn(u1[e], k1[e]), __hmul2_rn(__hneg2(u2[e]), z1[e]));
                    r2[e] = __hadd2_rn(__hmul2_rn(u2[e], k2[e]), __hmul2_rn(u1[e], z2[e]));
                } else {
                    r1[e] = __hadd2_rn(__hmul2_rn(u1[e], k1[e]), __hmul2_rn(u2[e], z2[e]));
                    r2[e] = __hadd2_rn(__hmul2_rn(u2[e], k2[e]), __hneg2(__hmul2_rn(u1[e], z1[e])));
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float a1 = Num<T>::to_f32(x1[g].e[e]), a2 = Num<T>::to_f32(x2[g].e[e]);
                const float k1 = Num<T>::to_f32(c1.e[e]), k2 = Num<T>::to_f32(cc2.e[e]);
                const float z1 = Num<T>::to_f32(s1.e[e]), z2 = Num<T>::to_f32(s2.e[e]);
                float r1, r2;
                if (!a.inverse) {
                    r1 = __fadd_rn(rnd<T>(__fmul_rn(a1, k1)), rnd<T>(__fmul_rn(-a2, z1)));
                    r2 = __fadd_rn(rnd<T>(__fmul_rn(a2, k2)), rnd<T>(__fmul_rn(a1, z2)));
                } else {
                    r1 = __fadd_rn(rnd<T>(__fmul_rn(a1, k1)), rnd<T>(__fmul_rn(a2, z2)));
                    r2 = __fadd_rn(rnd<T>(__fmul_rn(a2, k2)), -rnd<T>(__fmul_rn(a1, z1)));
                }
                y1.e[e] = Num<T>::from_f32(r1);
                y2.e[e] = Num<T>::from_f32(r2);
            }
        }
        store_vec<T, V>(dst[g] + c, y1);
        store_vec<T, V>(dst[g] + c2, y2);
    }
}

template <typename T>
cudaError_t launch_t(const RopeArgs &a, cudaStream_t stream, int *launches) {
    constexpr int V = 16 / sizeof(T);
#ifndef ROPE_HG
#define ROPE_HG 4
#endif
    constexpr int HG = ROPE_HG;
    const int half = a.dim / 2;
    const int heads = a.a.heads + a.b.heads;
    if (a.tokens == 0 || heads == 0 || a.d == 0) return cudaSuccess;
    auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    auto tensor_ok = [&](const RopeTensor &t) {
        return t.heads == 0 || (aligned(t.x) && aligned(t.out) && t.st % V == 0 && t.sh % V == 0 && t.ost % V == 0 && t.osh % V == 0);
    };
    const bool vec = half % V == 0 && a.d % V == 0 && aligned(a.cos) && aligned(a.sin) && tensor_ok(a.a) && tensor_ok(a.b);
    const int per_row = vec ? (half + a.d - a.dim) / V : half + a.d - a.dim;
    // Neighbouring threads: the columns of a head, then `hsub` neighbouring heads - a warp's worth.
    int hsub = 1;
    while (hsub * 2 * per_row <= 32 && hsub * 2 * HG <= heads) hsub *= 2;
    const int chunks = (heads + hsub * HG - 1) / (hsub * HG);
    const int64_t items = a.tokens * chunks * hsub * per_row;
    const int64_t blocks = (items + 255) / 256;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (vec) rope_kernel<T, V, HG><<<(unsigned)blocks, 256, 0, stream>>>(a, hsub);
    else rope_kernel<T, 1, HG><<<(unsigned)blocks, 256, 0, stream>>>(a, hsub);
    *launches += 1;
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_rope(int dtype, const RopeArgs &a, cudaStream_t stream, int *launches) {
    switch (dtype) {
        case 0: return launch_t<float>(a, stream, launches);
        case 1: return launch_t<__nv_bfloat16>(a, stream, launches);
        default: return launch_t<__half>(a, stream, launches);
    }
}

}  // namespace dash
