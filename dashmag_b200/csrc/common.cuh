// Shared device-side pieces of the attention kernels: dtype conversion, strided tensor views, and
// the integer rule that says which keys a query sees.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dash {

// ---------------------------------------------------------------------------------------------
// dtypes
// ---------------------------------------------------------------------------------------------
template <typename T> struct Num;
template <> struct Num<float> {
    static __device__ __forceinline__ float to_f32(float x) { return x; }
    static __device__ __forceinline__ float from_f32(float x) { return x; }
};
template <> struct Num<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Num<__half> {
    static __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};

// A [batch, time, head, dim] view of caller-owned memory, strides in elements.
struct View4 {
    const void *ptr;
    int64_t sb, st, sh, sd;
};

template <typename T>
__device__ __forceinline__ float load_f32(const View4 &v, int64_t b, int64_t t, int64_t h, int64_t d) {
    return Num<T>::to_f32(static_cast<const T *>(v.ptr)[b * v.sb + t * v.st + h * v.sh + d * v.sd]);
}

// ---------------------------------------------------------------------------------------------
// Which keys a query sees
// ---------------------------------------------------------------------------------------------
// Every mask of the contract but key padding gives each query ONE interval of keys [lo, hi):
// the query's position is `row + Tk - Tq` (packed: `i + Lk - Lq` inside its own sequence) and it
// sees from `left` keys before that position to `right` after it
// (crates/dash-contract/src/attention.rs:33-54).  `left` and `right` arrive clamped to
// Tq + Tk + 1, which stands for "no bound" and keeps everything inside int32.
struct MaskArgs {
    int kind;              // 0 none, 1 key padding, 2 packed
    const void *kp;        // key padding [B,Tk]
    int kp_bytes;          // 1 or 4
    int64_t kp_sb, kp_st;  // element strides
    const void *cu_q;      // [seqs + 1]
    const void *cu_k;
    int seqs;
    int idx_bytes;         // 4 or 8
    int left, right;       // clamped reach; causal already folded into right = 0
};

__device__ __forceinline__ int load_index(const void *p, int bytes, int i) {
    if (bytes == 8) {
        long long v = static_cast<const long long *>(p)[i];
        v = v < -2147483647LL ? -2147483647LL : (v > 2147483647LL ? 2147483647LL : v);
        return static_cast<int>(v);
    }
    return static_cast<const int *>(p)[i];
}

// The last s with cu[s] <= pos over the non-decreasing offsets cu[0..seqs]: -1 before the first
// offset, `seqs` from the last one on (both: no sequence).
__device__ __forceinline__ int sequence_of(const void *cu, int bytes, int seqs, int pos) {
    int lo = 0, hi = seqs + 1;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (load_index(cu, bytes, mid) <= pos) lo = mid + 1; else hi = mid;
    }
    return lo - 1;
}

// The keys query `row` of packed sequence `s` sees, [lo, hi), or (tk, 0) when it sees none.
__device__ __forceinline__ void row_bounds_in_sequence(const MaskArgs &m, int s, int row, int tk, int &lo, int &hi) {
    lo = tk;
    hi = 0;
    if (s < 0 || s >= m.seqs) return;
    int q0 = load_index(m.cu_q, m.idx_bytes, s), q1 = load_index(m.cu_q, m.idx_bytes, s + 1);
    int k0 = load_index(m.cu_k, m.idx_bytes, s), k1 = load_index(m.cu_k, m.idx_bytes, s + 1);
    int lk = k1 - k0, lq = q1 - q0;
    int pos = row - q0 + lk - lq;
    int a = max(k0 + max(0, pos - m.left), 0);
    int c = min(k0 + min(lk, pos + m.right + 1), tk);
    if (c > a) { lo = a; hi = c; }
}

// The keys query `row` sees, [lo, hi), or (tk, 0) when it sees none or lies past the queries.
__device__ __forceinline__ void row_bounds(const MaskArgs &m, int row, int tq, int tk, int &lo, int &hi) {
    lo = tk;
    hi = 0;
    if (row < 0 || row >= tq) return;
    if (m.kind == 2) {
        row_bounds_in_sequence(m, sequence_of(m.cu_q, m.idx_bytes, m.seqs, row), row, tk, lo, hi);
    } else {
        int pos = row + tk - tq;
        int a = max(0, pos - m.left);
        int c = min(tk, pos + m.right + 1);
        if (c > a) { lo = a; hi = c; }
    }
}

// The same for the 32 rows of a (converged) warp at once.  A thread that places its row by itself walks
// the packed offsets by bisection - three or four DEPENDENT loads from global memory, some two thousand
// cycles of a block's set-up before its first tile load can be issued.  Here each lane fetches ONE pair of
// offsets (lane i: cu_q[i], cu_k[i]; batches of up to 31 sequences, else every lane falls back to
// row_bounds), the rows are placed by comparing against the lanes' values, and the four offsets of a row's
// sequence come by shuffle: one load latency instead of four.  All 32 lanes must call; results are
// identical to row_bounds.
__device__ __forceinline__ void row_bounds_warp(const MaskArgs &m, int row, int tq, int tk, int &lo, int &hi) {
    if (m.kind != 2 || m.seqs > 31) {
        row_bounds(m, row, tq, tk, lo, hi);
        return;
    }
    const int lane = threadIdx.x & 31;
    const int cq = lane <= m.seqs ? load_index(m.cu_q, m.idx_bytes, lane) : 2147483647;
    const int ck = lane <= m.seqs ? load_index(m.cu_k, m.idx_bytes, lane) : 2147483647;
    int s = -1;   // the last s with cu_q[s] <= row: the offsets do not decrease, so it is a count
    for (int i = 0; i <= m.seqs; ++i) s += __shfl_sync(0xffffffffu, cq, i) <= row ? 1 : 0;
    const int sc = min(max(s, 0), 30);
    const int q0 = __shfl_sync(0xffffffffu, cq, sc), q1 = __shfl_sync(0xffffffffu, cq, sc + 1);
    const int k0 = __shfl_sync(0xffffffffu, ck, sc), k1 = __shfl_sync(0xffffffffu, ck, sc + 1);
    lo = tk;
    hi = 0;
    if (row < 0 || row >= tq || s < 0 || s >= m.seqs) return;
    const int lk = k1 - k0, lq = q1 - q0;
    const int pos = row - q0 + lk - lq;
    const int a = max(k0 + max(0, pos - m.left), 0);
    const int c = min(k0 + min(lk, pos + m.right + 1), tk);
    if (c > a) { lo = a; hi = c; }
}

__device__ __forceinline__ bool key_padded(const MaskArgs &m, int b, int key) {
    if (m.kind != 1) return false;
    int64_t at = (int64_t)b * m.kp_sb + (int64_t)key * m.kp_st;
    return m.kp_bytes == 4 ? static_cast<const int *>(m.kp)[at] != 0
                           : static_cast<const unsigned char *>(m.kp)[at] != 0;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ int warp_min_i(int x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = min(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ int warp_max_i(int x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = max(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

// ---------------------------------------------------------------------------------------------
// Arguments of the generic kernels
// ---------------------------------------------------------------------------------------------
struct TrainArgs {
    int b, tq, tk, hq, hkv, d;
    float scale;
    View4 q, k, v, o, dout;     // o / dout: backward's inputs
    void *out;                  // forward: o (contiguous, q's dtype)
    float *lse;                 // forward: output; backward: input; contiguous [B,Tq,Hq]
    float *delta;               // backward scratch [B,Tq,Hq]
    void *dq, *dk, *dv;         // backward outputs, contiguous
    MaskArgs mask;
};

struct DecodeArgs {
    int b, s, hq, hkv, d;
    float scale;
    const void *q;
    int64_t q_sb, q_sh, q_sd;
    View4 k, v;
    const void *lengths;
    int len_bytes;
    int left;                   // clamped to s + 1 = no bound
    int chunk, splits;          // keys per split and splits per sequence
    float *part_o;              // [B,Hq,splits,D]
    float *part_lse;            // [B,Hq,splits]
    void *out;                  // [B,Hq,D]
    // The step that also appends: the new key and value rows [B,Hkv,D] (contiguous) go to
    // position lengths[b] of the cache, where the step already sees them.  Null otherwise.
    const void *k_new, *v_new;
};

// Where the appending step writes sequence b's new row: its length before the step, or -1 when
// the step does not append or the cache is full.
__device__ __forceinline__ int decode_append_at(const DecodeArgs &a, int b) {
    if (!a.k_new || !a.lengths) return -1;
    const int len = max(load_index(a.lengths, a.len_bytes, b), 0);
    return len < a.s ? len : -1;
}

// The visible keys of sequence b in a decoding step: [first, len); the appended row counts.
__device__ __forceinline__ void decode_range(const DecodeArgs &a, int b, int &first, int &len) {
    len = a.s;
    if (a.lengths) len = min(max(load_index(a.lengths, a.len_bytes, b), 0) + (a.k_new ? 1 : 0), a.s);
    first = max(0, len - 1 - a.left);
    if (a.left > a.s) first = 0;
}

}  // namespace dash
