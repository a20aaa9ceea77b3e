// The decoding step against a key-value cache: split-KV (flash-decoding) and an LSE merge.
//
// The step is a single scan of the cache, so it is bound by HBM bandwidth: the algorithmic bytes
// are (visible keys) x Hkv x D x element size x 2 (keys and values).  Layout of the work:
//
//   * the visible keys [first, len) of each sequence are cut into chunks of `chunk` keys; one WARP
//     owns one (chunk, key-value head) and all the query heads of that head's group, so that a
//     cache row is read once for the whole group; warps of a block take consecutive key-value
//     heads of the same chunk, so a block streams whole contiguous cache rows;
//   * D / 8 lanes share a key: each lane loads 16 bytes of the key row and 16 bytes of the value
//     row (bf16 / f16; two 16-byte loads each for f32) - fully coalesced 128-bit loads - and owns
//     eight head dimensions of the output; four keys per lane group are in flight at once;
//   * scores are reduced across the D / 8 lanes with shuffles, the softmax is kept online in f32
//     per query head, lane groups are merged with shuffles at the end, and each warp writes one
//     normalised partial output and its log-sum-exp;
//   * the merge kernel combines the partials of each (sequence, query head) by their log-sum-exp
//     and rounds to the queries' dtype.  Chunks past a sequence's length or before its window are
//     never touched.
//
// Inputs the vector path cannot read (head dimension not 64 / 128 / 256, last stride not 1, rows
// not 16-byte aligned) go through a slower scalar kernel with the same arithmetic.
#include <mutex>

#include "common.cuh"
#include "launch.h"

namespace dash {

constexpr int DEC_WARPS = 8;
constexpr int DEC_UNROLL = 4;

template <typename T>
__device__ __forceinline__ void load8(const T *p, bool valid, float (&x)[8]);

template <>
__device__ __forceinline__ void load8<float>(const float *p, bool valid, float (&x)[8]) {
    float4 a = make_float4(0, 0, 0, 0), b = a;
    if (valid) {
        a = __ldg(reinterpret_cast<const float4 *>(p));
        b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    }
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, bool valid, float (&x)[8]) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (valid) r = __ldg(reinterpret_cast<const uint4 *>(p));
    const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = __uint_as_float(u[i] << 16);
        x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half *p, bool valid, float (&x)[8]) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (valid) r = __ldg(reinterpret_cast<const uint4 *>(p));
    const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

// exp for the online softmax: the accurate one for f32 inputs, the fast one for 16-bit inputs,
// whose outputs round to 8 or 11 significant bits anyway.
template <typename T> __device__ __forceinline__ float soft_exp(float x) { return __expf(x); }
template <> __device__ __forceinline__ float soft_exp<float>(float x) { return expf(x); }
template <typename T> __device__ __forceinline__ float soft_log(float x) { return __logf(x); }
template <> __device__ __forceinline__ float soft_log<float>(float x) { return logf(x); }

// One warp per (chunk, key-value head, pass over GH query heads of the group).
template <typename T, int D, int GH>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_split_kernel(DecodeArgs a) {
    constexpr int LPK = D / 8;       // lanes per key
    constexpr int KPW = 32 / LPK;    // keys per warp step
    const int lane = threadIdx.x & 31;
    const int group = a.hq / a.hkv;
    const int passes = (group + GH - 1) / GH;
    const int b = blockIdx.y;
    long long unit = (long long)blockIdx.x * DEC_WARPS + (threadIdx.x >> 5);
    const int hk = (int)(unit % a.hkv);
    unit /= a.hkv;
    const int pass = (int)(unit % passes);
    const long long split = unit / passes;
    if (split >= a.splits) return;

    int first, len;
    decode_range(a, b, first, len);
    const long long c0l = (long long)first + split * a.chunk;
    if (c0l >= len) return;
    const int c0 = (int)c0l, c1 = min(len, c0 + a.chunk);

    const int sub = lane / LPK, dl = lane % LPK;
    const int g0 = pass * GH;
    float q[GH][8], acc[GH][8], m[GH], l[GH];
#pragma unroll
    for (int g = 0; g < GH; ++g) {
        const bool live = g0 + g < group;
        const int h = hk * group + min(g0 + g, group - 1);
        const T *qp = static_cast<const T *>(a.q) + (int64_t)b * a.q_sb + (int64_t)h * a.q_sh + dl * 8;
        load8<T>(qp, live, q[g]);
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[g][c] = 0.f;
    }
    const T *kbase = static_cast<const T *>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)hk * a.k.sh + dl * 8;
    const T *vbase = static_cast<const T *>(a.v.ptr) + (int64_t)b * a.v.sb + (int64_t)hk * a.v.sh + dl * 8;

    for (int base = c0; base < c1; base += KPW * DEC_UNROLL) {
        float kx[DEC_UNROLL][8], vx[DEC_UNROLL][8];
        bool valid[DEC_UNROLL];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            const int key = base + u * KPW + sub;
            valid[u] = key < c1;
            load8<T>(kbase + (int64_t)key * a.k.st, valid[u], kx[u]);
            load8<T>(vbase + (int64_t)key * a.v.st, valid[u], vx[u]);
        }
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            float s[DEC_UNROLL];
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                float d = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) d = fmaf(q[g][c], kx[u][c], d);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                s[u] = valid[u] ? d * a.scale : -INFINITY;
                mx = fmaxf(mx, s[u]);
            }
            const float mn = fmaxf(m[g], mx);
            if (mn != -INFINITY) {
                const float corr = soft_exp<T>(m[g] - mn);
                float sum = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[g][c] *= corr;
#pragma unroll
                for (int u = 0; u < DEC_UNROLL; ++u) {
                    const float p = soft_exp<T>(s[u] - mn);
                    sum += p;
#pragma unroll
                    for (int c = 0; c < 8; ++c) acc[g][c] = fmaf(p, vx[u][c], acc[g][c]);
                }
                l[g] = l[g] * corr + sum;
                m[g] = mn;
            }
        }
    }

    // Merge the lane groups (each saw different keys).
#pragma unroll
    for (int g = 0; g < GH; ++g) {
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
            const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
            const float mn = fmaxf(m[g], mo);
            const float wa = mn == -INFINITY ? 0.f : soft_exp<T>(m[g] - mn);
            const float wb = mn == -INFINITY ? 0.f : soft_exp<T>(mo - mn);
            l[g] = l[g] * wa + lo * wb;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[g][c], o);
                acc[g][c] = acc[g][c] * wa + ao * wb;
            }
            m[g] = mn;
        }
        if (sub == 0 && g0 + g < group) {
            const int h = hk * group + g0 + g;
            const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
            float *po = a.part_o + (((int64_t)b * a.hq + h) * a.splits + split) * D + dl * 8;
            reinterpret_cast<float4 *>(po)[0] = make_float4(acc[g][0] * inv, acc[g][1] * inv, acc[g][2] * inv, acc[g][3] * inv);
            reinterpret_cast<float4 *>(po)[1] = make_float4(acc[g][4] * inv, acc[g][5] * inv, acc[g][6] * inv, acc[g][7] * inv);
            if (dl == 0) a.part_lse[((int64_t)b * a.hq + h) * a.splits + split] = l[g] > 0.f ? m[g] + soft_log<T>(l[g]) : -INFINITY;
        }
    }
}

// The same split for inputs the vector loads cannot take: one warp per (chunk, query head), a
// lane owning the head dimensions `lane + 32 i`, keys in order.
template <typename T>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_split_scalar_kernel(DecodeArgs a) {
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    long long unit = (long long)blockIdx.x * DEC_WARPS + (threadIdx.x >> 5);
    const int h = (int)(unit % a.hq);
    const long long split = unit / a.hq;
    if (split >= a.splits) return;
    int first, len;
    decode_range(a, b, first, len);
    const long long c0l = (long long)first + split * a.chunk;
    if (c0l >= len) return;
    const int c0 = (int)c0l, c1 = min(len, c0 + a.chunk);
    const int hk = h / (a.hq / a.hkv);
    const int ni = (a.d + 31) / 32;
    float q[8], acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int c = lane + 32 * i;
        q[i] = (i < ni && c < a.d)
                   ? Num<T>::to_f32(static_cast<const T *>(a.q)[(int64_t)b * a.q_sb + (int64_t)h * a.q_sh + (int64_t)c * a.q_sd])
                   : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int key = c0; key < c1; ++key) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int c = lane + 32 * i;
            if (i < ni && c < a.d) d = fmaf(q[i], load_f32<T>(a.k, b, key, hk, c), d);
        }
        const float s = warp_sum(d) * a.scale;
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), p = expf(s - mn);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int c = lane + 32 * i;
            float v = (i < ni && c < a.d) ? load_f32<T>(a.v, b, key, hk, c) : 0.f;
            acc[i] = fmaf(p, v, acc[i] * corr);
        }
        m = mn;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float *po = a.part_o + (((int64_t)b * a.hq + h) * a.splits + split) * a.d;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int c = lane + 32 * i;
        if (i < ni && c < a.d) po[c] = acc[i] * inv;
    }
    if (lane == 0) a.part_lse[((int64_t)b * a.hq + h) * a.splits + split] = l > 0.f ? m + logf(l) : -INFINITY;
}

// Merges the partials of one (sequence, query head) by their log-sum-exp.
template <typename T>
__global__ void __launch_bounds__(128) decode_merge_kernel(DecodeArgs a) {
    const int bh = blockIdx.x;
    const int b = bh / a.hq;
    int first, len;
    decode_range(a, b, first, len);
    const int n = (len - first + a.chunk - 1) / a.chunk;  // splits that hold keys
    T *out = static_cast<T *>(a.out) + (int64_t)bh * a.d;
    if (n <= 0) {
        for (int c = threadIdx.x; c < a.d; c += blockDim.x) out[c] = Num<T>::from_f32(0.f);
        return;
    }
    const float *lse = a.part_lse + (int64_t)bh * a.splits;
    const float *po = a.part_o + (int64_t)bh * a.splits * a.d;
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) mx = fmaxf(mx, lse[i]);
    for (int c = threadIdx.x; c < a.d; c += blockDim.x) {
        float num = 0.f, den = 0.f;
        for (int i = 0; i < n; ++i) {
            const float w = expf(lse[i] - mx);
            den += w;
            num = fmaf(w, po[(int64_t)i * a.d + c], num);
        }
        out[c] = Num<T>::from_f32(den > 0.f ? num / den : 0.f);
    }
}

template <typename T, int D>
static cudaError_t split_vec(const DecodeArgs &a, cudaStream_t stream) {
    const int group = a.hq / a.hkv;
    const int gh = group >= 4 ? 4 : (group >= 2 ? 2 : 1);
    const int passes = (group + gh - 1) / gh;
    const long long units = (long long)a.splits * a.hkv * passes;
    dim3 grid((unsigned)((units + DEC_WARPS - 1) / DEC_WARPS), a.b);
    if (gh == 4) decode_split_kernel<T, D, 4><<<grid, DEC_WARPS * 32, 0, stream>>>(a);
    else if (gh == 2) decode_split_kernel<T, D, 2><<<grid, DEC_WARPS * 32, 0, stream>>>(a);
    else decode_split_kernel<T, D, 1><<<grid, DEC_WARPS * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t decode_t(const DecodeArgs &a, bool vector_ok, cudaStream_t stream, int *launches) {
    cudaError_t e;
    if (vector_ok && a.d == 64) e = split_vec<T, 64>(a, stream);
    else if (vector_ok && a.d == 128) e = split_vec<T, 128>(a, stream);
    else if (vector_ok && a.d == 256) e = split_vec<T, 256>(a, stream);
    else {
        const long long units = (long long)a.splits * a.hq;
        dim3 grid((unsigned)((units + DEC_WARPS - 1) / DEC_WARPS), a.b);
        decode_split_scalar_kernel<T><<<grid, DEC_WARPS * 32, 0, stream>>>(a);
        e = cudaGetLastError();
    }
    *launches += 1;
    if (e != cudaSuccess) return e;
    decode_merge_kernel<T><<<a.b * a.hq, 128, 0, stream>>>(a);
    *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_decode(int dtype, const DecodeArgs &a, bool vector_ok, cudaStream_t stream, int *launches) {
    switch (dtype) {
        case 0: return decode_t<float>(a, vector_ok, stream, launches);
        case 1: return decode_t<__nv_bfloat16>(a, vector_ok, stream, launches);
        default: return decode_t<__half>(a, vector_ok, stream, launches);
    }
}

// ---------------------------------------------------------------------------------------------
// The decoding step with its scratch inside the library (dash_attn_decode_static)
// ---------------------------------------------------------------------------------------------
// Some callers hold nothing but the raw input and output buffers they were handed and have no way
// to produce a workspace: an FFI shim under a tensor runtime whose memory pool owns all device
// memory and is not reachable from C, or a serving loop that has promised not to allocate once it
// is running.  For them the partial outputs of the split pass live in this file-scope array
// instead of a caller-provided workspace.  Every GPU that loads the library reserves it until the
// process exits, so it is kept modest: 4 Mi floats (16 MiB).
//
// In host code the array's name is only a stand-in; its device address is asked for once per
// device (with that device current) and cached.  All calls share the array and it keeps whatever
// the last call left in it: nothing in it needs to start at zero, because the merge pass reads
// only the partials the split pass of the same call has just written - but two calls whose kernels
// overlap on the GPU (different streams, or different host threads without ordering) would write
// over each other's partials.
constexpr size_t DECODE_STATIC_FLOATS = size_t(4) << 20;
static __device__ __align__(256) float g_decode_static_scratch[DECODE_STATIC_FLOATS];

size_t decode_static_capacity_floats() { return DECODE_STATIC_FLOATS; }

// The device address of the static scratch on the current device; the first call on each device
// resolves it (and should therefore come before any stream capture begins).
cudaError_t decode_static_scratch(float **out) {
    constexpr int MAX_DEVICES = 64;
    static float *cache[MAX_DEVICES] = {};
    static std::mutex lock;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(lock);
    if (!cache[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_decode_static_scratch);
        if (e != cudaSuccess) return e;
        cache[dev] = ptr;
    }
    *out = cache[dev];
    return cudaSuccess;
}

}  // namespace dash
