// Pieces the backward kernels share: packing two f32 values into a 32-bit pair of the input dtype,
// and the inverse of the visible-key interval (which queries see a key, or a block of keys).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace dash {
namespace {

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

// The queries [first, end) that may see some key of [k0, k1): a superset cut from the closed form
// of the visible interval (query i of a sequence sees key c iff
// c - right - (Lk - Lq) <= i <= c + left - (Lk - Lq)); exact masking happens per element.
__device__ __forceinline__ void query_range(const MaskArgs &m, int k0, int k1, int tq, int tk, int &first, int &end) {
    first = 0;
    end = 0;
    if (k1 <= k0) return;
    if (m.kind == 2) {
        if (m.seqs <= 0) return;
        int sa = sequence_of(m.cu_k, m.idx_bytes, m.seqs, k0);
        int sb = sequence_of(m.cu_k, m.idx_bytes, m.seqs, k1 - 1);
        if (sb < 0 || sa >= m.seqs) return;
        sa = max(sa, 0);
        sb = min(sb, m.seqs - 1);
        const int qa0 = load_index(m.cu_q, m.idx_bytes, sa), qa1 = load_index(m.cu_q, m.idx_bytes, sa + 1);
        const int ka0 = load_index(m.cu_k, m.idx_bytes, sa), ka1 = load_index(m.cu_k, m.idx_bytes, sa + 1);
        const int qb0 = load_index(m.cu_q, m.idx_bytes, sb), qb1 = load_index(m.cu_q, m.idx_bytes, sb + 1);
        const int kb0 = load_index(m.cu_k, m.idx_bytes, sb), kb1 = load_index(m.cu_k, m.idx_bytes, sb + 1);
        const int off_a = (ka1 - ka0) - (qa1 - qa0), off_b = (kb1 - kb0) - (qb1 - qb0);
        first = qa0 + min(max(k0 - ka0 - m.right - off_a, 0), qa1 - qa0);
        end = qb0 + min(max(k1 - 1 - kb0 + m.left - off_b + 1, 0), qb1 - qb0);
    } else {
        const int off = tk - tq;
        first = min(max(k0 - m.right - off, 0), tq);
        end = min(max(k1 - 1 + m.left - off + 1, 0), tq);
    }
    first = min(max(first, 0), tq);
    end = min(max(end, 0), tq);
    if (end < first) end = first;
}

// The queries [first, end) that see key `key`: the inverse of the visible interval (both ends of a
// query's interval grow with the query, so the queries that see one key are an interval as well),
// from the same closed form as query_range and exact.  Key padding is the caller's to apply.
__device__ __forceinline__ void queries_of_key(const MaskArgs &m, int key, int tq, int tk, int &first, int &end) {
    first = 0;
    end = 0;
    if (key < 0 || key >= tk) return;
    if (m.kind == 2) {
        const int s = sequence_of(m.cu_k, m.idx_bytes, m.seqs, key);
        if (s < 0 || s >= m.seqs) return;
        const int q0 = load_index(m.cu_q, m.idx_bytes, s), q1 = load_index(m.cu_q, m.idx_bytes, s + 1);
        const int k0 = load_index(m.cu_k, m.idx_bytes, s), k1 = load_index(m.cu_k, m.idx_bytes, s + 1);
        if (key >= k1) return;   // between sequences
        const int off = (k1 - k0) - (q1 - q0), rel = key - k0;
        first = max(q0, q0 + rel - m.right - off);
        end = min(q1, q0 + rel + m.left - off + 1);
    } else {
        const int off = tk - tq;
        first = max(0, key - m.right - off);
        end = min(tq, key + m.left - off + 1);
    }
    first = max(first, 0);
    end = min(end, tq);
    if (end < first) end = first;
}

}  // namespace
}  // namespace dash
