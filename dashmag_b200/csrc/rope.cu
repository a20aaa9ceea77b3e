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

template <typename T> __device__ __forceinline__ T quiet_nan() { return Num<T>::from_f32(__int_as_float(0x7fc00000)); }

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
    return a.start + (a.period > 0 ? n % a.period : 0);
}

// V = elements per thread and side of a pair: 16 bytes' worth, or 1 where the shapes or the
// addresses do not allow vectors.
template <typename T, int V>
__global__ void __launch_bounds__(256) rope_kernel(RopeArgs a) {
    const int half = a.dim / 2;
    const int pair_items = half / V, copy_items = (a.d - a.dim) / V;
    const int per_row = pair_items + copy_items;
    const int heads = a.a.heads + a.b.heads;
    const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= a.tokens * heads * per_row) return;
    const int i = (int)(item % per_row);
    const int64_t row = item / per_row;
    const int hh = (int)(row % heads);
    const int64_t n = row / heads;
    const RopeTensor &t = hh < a.a.heads ? a.a : a.b;
    const int h = hh < a.a.heads ? hh : hh - a.a.heads;
    const T *x = static_cast<const T *>(t.x) + n * t.st + h * t.sh;
    T *out = static_cast<T *>(t.out) + n * t.ost + h * t.osh;

    struct alignas(sizeof(T) * V) Vec { T e[V]; };
    if (i >= pair_items) {
        const int c = a.dim + (i - pair_items) * V;
        if (t.out != t.x) *reinterpret_cast<Vec *>(out + c) = *reinterpret_cast<const Vec *>(x + c);
        return;
    }
    const int c = i * V;
    const Vec x1 = *reinterpret_cast<const Vec *>(x + c), x2 = *reinterpret_cast<const Vec *>(x + c + half);
    bool rotate;
    const int64_t pos = position_of(a, n, rotate);
    Vec y1, y2;
    if (!rotate) {
        y1 = x1;
        y2 = x2;
    } else if (pos < 0 || pos >= a.len) {
        // No such row in the tables: the reference leaves this to the caller; a NaN shows it.
#pragma unroll
        for (int e = 0; e < V; ++e) y1.e[e] = y2.e[e] = quiet_nan<T>();
    } else {
        const T *cs = static_cast<const T *>(a.cos) + pos * a.dim, *sn = static_cast<const T *>(a.sin) + pos * a.dim;
        const Vec c1 = *reinterpret_cast<const Vec *>(cs + c), c2 = *reinterpret_cast<const Vec *>(cs + c + half);
        const Vec s1 = *reinterpret_cast<const Vec *>(sn + c), s2 = *reinterpret_cast<const Vec *>(sn + c + half);
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float a1 = Num<T>::to_f32(x1.e[e]), a2 = Num<T>::to_f32(x2.e[e]);
            const float cc1 = Num<T>::to_f32(c1.e[e]), cc2 = Num<T>::to_f32(c2.e[e]);
            const float ss1 = Num<T>::to_f32(s1.e[e]), ss2 = Num<T>::to_f32(s2.e[e]);
            float r1, r2;
            if (!a.inverse) {
                r1 = __fadd_rn(rnd<T>(__fmul_rn(a1, cc1)), rnd<T>(__fmul_rn(-a2, ss1)));
                r2 = __fadd_rn(rnd<T>(__fmul_rn(a2, cc2)), rnd<T>(__fmul_rn(a1, ss2)));
            } else {
                r1 = __fadd_rn(rnd<T>(__fmul_rn(a1, cc1)), rnd<T>(__fmul_rn(a2, ss2)));
                r2 = __fadd_rn(rnd<T>(__fmul_rn(a2, cc2)), -rnd<T>(__fmul_rn(a1, ss1)));
            }
            y1.e[e] = Num<T>::from_f32(r1);
            y2.e[e] = Num<T>::from_f32(r2);
        }
    }
    *reinterpret_cast<Vec *>(out + c) = y1;
    *reinterpret_cast<Vec *>(out + c + half) = y2;
}

template <typename T>
cudaError_t launch_t(const RopeArgs &a, cudaStream_t stream, int *launches) {
    constexpr int V = 16 / sizeof(T);
    const int half = a.dim / 2;
    const int heads = a.a.heads + a.b.heads;
    if (a.tokens == 0 || heads == 0 || a.d == 0) return cudaSuccess;
    auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    auto tensor_ok = [&](const RopeTensor &t) {
        return t.heads == 0 || (aligned(t.x) && aligned(t.out) && t.st % V == 0 && t.sh % V == 0 && t.ost % V == 0 && t.osh % V == 0);
    };
    const bool vec = half % V == 0 && a.d % V == 0 && aligned(a.cos) && aligned(a.sin) && tensor_ok(a.a) && tensor_ok(a.b);
    const int per_row = vec ? (half + a.d - a.dim) / V : half + a.d - a.dim;
    const int64_t items = a.tokens * heads * per_row;
    const int64_t blocks = (items + 255) / 256;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (vec) rope_kernel<T, V><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else rope_kernel<T, 1><<<(unsigned)blocks, 256, 0, stream>>>(a);
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
