// The decoding step against a key-value cache: split-KV (flash-decoding) and an LSE merge.
//
// The step is a single scan of the cache, so it is bound by HBM bandwidth: the algorithmic bytes
// are (visible keys) x Hkv x D x element size x 2 (keys and values).  Layout of the work:
//
//   * the visible keys [first, len) of each sequence are cut into chunks of `chunk` keys; one WARP
//     owns one (chunk, key-value head) and all the query heads of that head's group, so that a
//     cache row is read once for the whole group; warps of a block take consecutive key-value
//     heads of the same chunk, so a block streams whole contiguous cache rows;
//   * D / 8 lanes share a key: each lane copies 16 bytes of the key row and 16 bytes of the value
//     row (bf16 / f16; two 16-byte vectors each for f32) - fully coalesced 128-bit accesses - and
//     owns eight head dimensions of the output; the copies are asynchronous, into a ring of
//     shared memory private to the lane, three steps of four keys ahead of the arithmetic;
//   * scores are reduced across the D / 8 lanes with shuffles, the softmax is kept online in f32
//     per query head, lane groups are merged with shuffles at the end, and each warp writes one
//     normalised partial output and its log-sum-exp;
//   * the merge kernel combines the partials of each (sequence, query head) by their log-sum-exp
//     and rounds to the queries' dtype.  Chunks past a sequence's length or before its window are
//     never touched.
//
// With 16-bit caches, head dimension 128 and four to sixteen query heads per key-value head the
// split pass runs on the tensor cores instead (decode_split_mma_kernel below): at that much
// arithmetic per cache row the FMA pipe, not HBM, bounds the pass above.
//
// Inputs the vector path cannot read (head dimension not 64 / 128 / 256, last stride not 1, rows
// not 16-byte aligned) go through a slower scalar kernel with the same arithmetic.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "launch.h"

namespace dash {

constexpr int DEC_WARPS = 4;    // warps per block, each with its own (chunk, key-value head)
constexpr int DEC_UNROLL = 4;   // keys per group of D / 8 lanes in one step
constexpr int DEC_STAGES = 4;   // steps of the per-lane ring (16-bit dtypes; two for f32)

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

// ---- 16-byte asynchronous copies, global -> this lane's slots of shared memory ------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    // An invalid (out of range) key copies nothing and fills its slot with zeros.
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Eight values of T from this lane's own 16-byte slots.
template <typename T>
__device__ __forceinline__ void slot8(const uint4 *slot, float (&x)[8]);
template <>
__device__ __forceinline__ void slot8<float>(const uint4 *slot, float (&x)[8]) {
    const uint4 a = slot[0], b = slot[32];
    x[0] = __uint_as_float(a.x); x[1] = __uint_as_float(a.y); x[2] = __uint_as_float(a.z); x[3] = __uint_as_float(a.w);
    x[4] = __uint_as_float(b.x); x[5] = __uint_as_float(b.y); x[6] = __uint_as_float(b.z); x[7] = __uint_as_float(b.w);
}
template <>
__device__ __forceinline__ void slot8<__nv_bfloat16>(const uint4 *slot, float (&x)[8]) {
    const uint4 r = slot[0];
    const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = __uint_as_float(u[i] << 16);
        x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void slot8<__half>(const uint4 *slot, float (&x)[8]) {
    const uint4 r = slot[0];
    const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

// One warp per (chunk, key-value head, pass over GH query heads of the group).
//
// The cache rows reach the arithmetic through a ring of shared memory that is private to each
// lane: a lane copies, with 16-byte asynchronous copies, exactly the bytes it will later read
// itself, DEC_STAGES - 1 steps ahead (a step is DEC_UNROLL keys for each group of D / 8 lanes).
// The bytes in flight therefore cost shared memory, not registers, no lane ever waits for
// another, and a multiprocessor keeps three blocks of four such warps resident: twelve warps
// with three steps each on the way from HBM.
template <typename T, int D, int GH>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_split_kernel(DecodeArgs a) {
    constexpr int LPK = D / 8;                    // lanes per key
    constexpr int KPW = 32 / LPK;                 // keys per warp in one load
    constexpr int VPK = sizeof(T) == 4 ? 2 : 1;   // 16-byte vectors per eight values
    constexpr int SLOTS = 2 * DEC_UNROLL * VPK;   // this lane's vectors per stage: K and V of DEC_UNROLL keys
    constexpr int NS = sizeof(T) == 4 ? 2 : DEC_STAGES;
    extern __shared__ uint4 ring[];               // [warp][stage][slot][lane]
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int group = a.hq / a.hkv;
    const int passes = (group + GH - 1) / GH;
    const int b = blockIdx.y;
    long long unit = (long long)blockIdx.x * DEC_WARPS + wib;
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
    // The appending step: the row at `pos` comes from the new rows, and the warp whose chunk holds
    // it (first pass only) also writes it into the cache.
    const int pos = decode_append_at(a, b);
    const T *knew = static_cast<const T *>(a.k_new) + ((int64_t)b * a.hkv + hk) * D + dl * 8;
    const T *vnew = static_cast<const T *>(a.v_new) + ((int64_t)b * a.hkv + hk) * D + dl * 8;
    if (pos >= c0 && pos < c1 && pass == 0 && sub == 0) {
#pragma unroll
        for (int x = 0; x < VPK; ++x) {
            reinterpret_cast<uint4 *>(const_cast<T *>(kbase) + (int64_t)pos * a.k.st)[x] = reinterpret_cast<const uint4 *>(knew)[x];
            reinterpret_cast<uint4 *>(const_cast<T *>(vbase) + (int64_t)pos * a.v.st)[x] = reinterpret_cast<const uint4 *>(vnew)[x];
        }
    }

    uint4 *mine = ring + (size_t)wib * NS * SLOTS * 32 + lane;
    const uint32_t mine_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(mine));
    constexpr int STEP_KEYS = KPW * DEC_UNROLL;
    const int iters = (c1 - c0 + STEP_KEYS - 1) / STEP_KEYS;

    auto issue = [&](int it) {
        if (it < iters) {
            const uint32_t dst = mine_u32 + (uint32_t)((it % NS) * SLOTS * 32 * 16);
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                const int key = c0 + it * STEP_KEYS + u * KPW + sub;
                const bool valid = key < c1;
                const T *kp = key == pos ? knew : kbase + (int64_t)(valid ? key : c0) * a.k.st;
                const T *vp = key == pos ? vnew : vbase + (int64_t)(valid ? key : c0) * a.v.st;
#pragma unroll
                for (int x = 0; x < VPK; ++x) {
                    cp_async16(dst + (uint32_t)(((2 * u) * VPK + x) * 32 * 16), reinterpret_cast<const char *>(kp) + 16 * x, valid);
                    cp_async16(dst + (uint32_t)(((2 * u + 1) * VPK + x) * 32 * 16), reinterpret_cast<const char *>(vp) + 16 * x, valid);
                }
            }
        }
        cp_async_commit();  // always, so that the group count stays in step with the iterations
    };

#pragma unroll
    for (int s = 0; s < NS - 1; ++s) issue(s);
    for (int it = 0; it < iters; ++it) {
        issue(it + NS - 1);
        cp_async_wait<NS - 1>();
        const uint4 *stage = mine + (size_t)(it % NS) * SLOTS * 32;
        const int key0 = c0 + it * STEP_KEYS + sub;
        float s[GH][DEC_UNROLL];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float kx[8];
            slot8<T>(stage + (2 * u) * VPK * 32, kx);
            const bool valid = key0 + u * KPW < c1;
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float d = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) d = fmaf(q[g][c], kx[c], d);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                s[g][u] = valid ? d * a.scale : -INFINITY;
            }
        }
        float corr[GH];
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            float mx = s[g][0];
#pragma unroll
            for (int u = 1; u < DEC_UNROLL; ++u) mx = fmaxf(mx, s[g][u]);
            const float mn = fmaxf(m[g], mx);
            const float base = mn == -INFINITY ? 0.f : mn;   // nothing seen yet: exponentiate against 0
            corr[g] = soft_exp<T>(m[g] - base);
            float sum = 0.f;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                s[g][u] = soft_exp<T>(s[g][u] - base);
                sum += s[g][u];
            }
            l[g] = l[g] * corr[g] + sum;
            m[g] = mn;
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[g][c] *= corr[g];
        }
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float vx[8];
            slot8<T>(stage + (2 * u + 1) * VPK * 32, vx);
#pragma unroll
            for (int g = 0; g < GH; ++g)
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[g][c] = fmaf(s[g][u], vx[c], acc[g][c]);
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

// ---------------------------------------------------------------------------------------------
// The split pass on the tensor cores (16-bit cache, head dimension 64, 128 or 256, groups of two heads or more)
// ---------------------------------------------------------------------------------------------
// With several query heads to a key-value head the scalar pass spends its time on FMA issue,
// not on HBM: a cache row of 512 bytes feeds 2048 multiply-adds.  Here the query heads of the group
// are the M dimension of warp-level MMAs (m16n8k16): S = Q K^T with the 16 keys of a tile as two
// N tiles, then O += P V with P taken straight from the accumulator registers of S as the A
// operand.  One warp per (chunk, key-value head) as before, with a ring of its own in shared memory:
// every lane copies 16-byte pieces of the tile's 16 key rows and 16 value rows asynchronously, two
// tiles ahead, into rows (256 bytes at D = 128) whose 16-byte chunks are XOR-swizzled by the row, and ldmatrix
// reads the fragments from there without bank conflicts (transposed for V).
constexpr int DM_WARPS = 8;     // warps per block
constexpr int DM_STAGES = 3;    // tiles of the per-warp ring
constexpr int DM_KEYS = 16;     // keys per tile

template <typename T> struct MmaType;
template <> struct MmaType<__nv_bfloat16> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
    static __device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
};
template <> struct MmaType<__half> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ float lo(uint32_t u) { return __low2float(*reinterpret_cast<const __half2 *>(&u)); }
    static __device__ __forceinline__ float hi(uint32_t u) { return __high2float(*reinterpret_cast<const __half2 *>(&u)); }
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// PARTS = 2 (head dimension 256): two neighbouring warps share a unit, each with D = 128 of the 256
// features - its half of the scores' sum over the features, which the two exchange through shared
// memory and add (in one order, so both hold the same bits), its half of Q, of every K and V row
// and of the output; the accumulators of a whole row of 256 would not fit a thread's registers.
template <typename T, int D, int PARTS>
__global__ void __launch_bounds__(DM_WARPS * 32) decode_split_mma_kernel(DecodeArgs a) {
    constexpr int DFULL = D * PARTS;            // the head dimension; D is what one warp takes of it
    constexpr int ROWB = 2 * D;                 // bytes of a warp's part of a cache row: 256 at D = 128, 128 at D = 64
    constexpr int CH = D / 8;                   // its 16-byte chunks
    constexpr int DM_TILE = DM_KEYS * ROWB;     // bytes of a K (or V) tile of 16 rows
    extern __shared__ __align__(128) uint8_t dm_ring[];   // [warp][stage][K tile | V tile], then the warps' score exchange
    float *dm_exchange = reinterpret_cast<float *>(dm_ring + (size_t)DM_WARPS * DM_STAGES * 2 * DM_KEYS * ROWB);   // [warp][lane][8]
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int group = a.hq / a.hkv;
    const int b = blockIdx.y;
    const long long unit = ((long long)blockIdx.x * DM_WARPS + wib) / PARTS;
    const int part = wib % PARTS, d0 = part * D;   // this warp's features [d0, d0 + D)
    // A unit: sixteen query heads of a group (the M rows of the MMAs; a group of more takes several
    // units side by side, whose warps read the same chunk of the cache at the same time: once from
    // HBM, the rest from L2), a key-value head, a chunk.
    const int hblocks = (group + 15) / 16;
    const int g_base = (int)(unit % hblocks) * 16;
    const int hk = (int)((unit / hblocks) % a.hkv);
    const long long split = unit / hblocks / a.hkv;
    if (split >= a.splits) return;
    int first, len;
    decode_range(a, b, first, len);
    const long long c0l = (long long)first + split * a.chunk;
    if (c0l >= len) return;
    const int c0 = (int)c0l, c1 = min(len, c0 + a.chunk);
    const int iters = (c1 - c0 + DM_KEYS - 1) / DM_KEYS;

    const int g = lane >> 2, t = lane & 3;   // fragment coordinates: row (head) g and g + 8, column pair t
    // Q as the A operand of every score MMA: [16 heads x 16 d] per k-step, rows past the group zero.
    uint32_t qa[D / 16][4];
    {
        const T *q0 = static_cast<const T *>(a.q) + (int64_t)b * a.q_sb + (int64_t)(hk * group + min(g_base + g, group - 1)) * a.q_sh + d0;
        const T *q1 = static_cast<const T *>(a.q) + (int64_t)b * a.q_sb + (int64_t)(hk * group + min(g_base + g + 8, group - 1)) * a.q_sh + d0;
        const bool live0 = g_base + g < group, live1 = g_base + g + 8 < group;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa[ks][0] = live0 ? *reinterpret_cast<const uint32_t *>(q0 + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = live1 ? *reinterpret_cast<const uint32_t *>(q1 + ks * 16 + 2 * t) : 0u;
            qa[ks][2] = live0 ? *reinterpret_cast<const uint32_t *>(q0 + ks * 16 + 8 + 2 * t) : 0u;
            qa[ks][3] = live1 ? *reinterpret_cast<const uint32_t *>(q1 + ks * 16 + 8 + 2 * t) : 0u;
        }
    }
    const T *kbase = static_cast<const T *>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)hk * a.k.sh + d0;
    const T *vbase = static_cast<const T *>(a.v.ptr) + (int64_t)b * a.v.sb + (int64_t)hk * a.v.sh + d0;
    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(dm_ring)) + (uint32_t)wib * DM_STAGES * 2 * DM_TILE;

    // This lane's pieces of a tile: chunk (lane % 16) of rows (lane / 16) + 2 j.
    const int cp_chunk = lane % CH, cp_row0 = lane / CH;
    constexpr int RPP = 32 / CH;                // rows the warp copies per pass
    // The appending step: the row at `pos` comes from the new rows, and the warp whose chunk holds
    // it also writes it into the cache (D / 8 lanes the key row, D / 8 the value row).
    const int pos = decode_append_at(a, b);
    const T *knew = static_cast<const T *>(a.k_new) + ((int64_t)b * a.hkv + hk) * DFULL + d0;
    const T *vnew = static_cast<const T *>(a.v_new) + ((int64_t)b * a.hkv + hk) * DFULL + d0;
    if (pos >= c0 && pos < c1 && lane < 2 * CH && g_base == 0) {
        const T *src = (lane < CH ? knew : vnew) + cp_chunk * 8;
        T *dst = const_cast<T *>(lane < CH ? kbase + (int64_t)pos * a.k.st : vbase + (int64_t)pos * a.v.st) + cp_chunk * 8;
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
    }
    const int pos_it = (pos >= c0 && pos < c1) ? (pos - c0) / DM_KEYS : -1;   // the tile of the new row, if this chunk holds it
    auto issue = [&](int it) {
        if (it < iters) {
            const uint32_t dst = ring + (uint32_t)(it % DM_STAGES) * 2 * DM_TILE;
#pragma unroll
            for (int j = 0; j < DM_KEYS / RPP; ++j) {
                const int row = cp_row0 + RPP * j, key = c0 + it * DM_KEYS + row;
                const bool valid = key < c1;
                const uint32_t at = (uint32_t)(row * ROWB + ((cp_chunk ^ (row & 7)) << 4));
                const T *kp = kbase + (int64_t)(valid ? key : c0) * a.k.st, *vp = vbase + (int64_t)(valid ? key : c0) * a.v.st;
                if (it == pos_it && key == pos) { kp = knew; vp = vnew; }   // only the tile that holds the new row looks for it
                cp_async16(dst + at, kp + cp_chunk * 8, valid);
                cp_async16(dst + DM_TILE + at, vp + cp_chunk * 8, valid);
            }
        }
        cp_async_commit();  // always, so that the group count stays in step with the tiles
    };

    const float sl = a.scale * 1.4426950408889634f;   // scores are exponentiated in base 2
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};   // rows g and g + 8; l is this lane's share
    // ldmatrix rows: lane -> (matrix lane / 8, row lane % 8)
    const int lm = lane >> 3, lr = lane & 7;

#pragma unroll
    for (int s = 0; s < DM_STAGES - 1; ++s) issue(s);
    for (int it = 0; it < iters; ++it) {
        __syncwarp();   // every lane is done with the stage about to be refilled
        issue(it + DM_STAGES - 1);
        cp_async_wait<DM_STAGES - 1>();
        __syncwarp();   // ... and sees the other lanes' pieces of this tile
        const uint32_t kt = ring + (uint32_t)(it % DM_STAGES) * 2 * DM_TILE, vt = kt + DM_TILE;
        const int key0 = c0 + it * DM_KEYS;

        // S[16 heads x 16 keys] as two N tiles of 8 keys.
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int row = nt * 8 + lr;
#pragma unroll
            for (int ks = 0; ks < D / 16; ks += 2) {
                uint32_t kb[4];   // b0, b1 of k-step ks, then of ks + 1
                ldmatrix_x4(kt + (uint32_t)(row * ROWB + (((2 * ks + lm) ^ (row & 7)) << 4)), kb);
                MmaType<T>::mma(sc[nt], qa[ks], kb[0], kb[1]);
                MmaType<T>::mma(sc[nt], qa[ks + 1], kb[2], kb[3]);
            }
        }
        if constexpr (PARTS == 2) {
            // The other half of the sum over the features is the neighbouring warp's: both write theirs, meet,
            // and add part 0's and part 1's in that order.
            float *mine = dm_exchange + ((size_t)wib * 32 + lane) * 8, *other = dm_exchange + ((size_t)(wib ^ 1) * 32 + lane) * 8;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
                *reinterpret_cast<float4 *>(mine + 4 * nt) = make_float4(sc[nt][0], sc[nt][1], sc[nt][2], sc[nt][3]);
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (wib >> 1)) : "memory");
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float4 o4 = *reinterpret_cast<const float4 *>(other + 4 * nt);
                const float theirs[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] = part == 0 ? sc[nt][e] + theirs[e] : theirs[e] + sc[nt][e];
            }
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (wib >> 1)) : "memory");   // both have read before the next tile's are written
        }
        // Online softmax of rows g (values 0, 1 of a tile) and g + 8 (values 2, 3); a tile's columns
        // are keys key0 + 8 nt + 2 t + {0, 1}.
        if (key0 + DM_KEYS > c1) {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (key0 + nt * 8 + 2 * t + (j & 1) >= c1) sc[nt][j] = -INFINITY;
        }
        // P goes to the tensor cores as the sum of two 16-bit values (what the rounding of the first
        // loses is the second), so that the products keep the f32 accuracy of the scalar pass.
        uint32_t pa[4], pl[4];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            float mx = fmaxf(fmaxf(sc[0][2 * rr], sc[0][2 * rr + 1]), fmaxf(sc[1][2 * rr], sc[1][2 * rr + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[rr], mx);
            if (__any_sync(0xffffffffu, mn > m[rr])) {
                // The row's maximum grew (in some row of the warp): bring the sum and the accumulator along.
                const float corr = mn == -INFINITY ? 1.f : exp2f((m[rr] - mn) * sl);   // exp2(-inf) = 0 for a first maximum
                l[rr] *= corr;
#pragma unroll
                for (int n = 0; n < D / 8; ++n) { o[n][2 * rr] *= corr; o[n][2 * rr + 1] *= corr; }
                m[rr] = mn;
            }
            const float base = m[rr] == -INFINITY ? 0.f : m[rr] * sl;
            const float p00 = exp2f(fmaf(sc[0][2 * rr], sl, -base)), p01 = exp2f(fmaf(sc[0][2 * rr + 1], sl, -base));
            const float p10 = exp2f(fmaf(sc[1][2 * rr], sl, -base)), p11 = exp2f(fmaf(sc[1][2 * rr + 1], sl, -base));
            l[rr] += (p00 + p01) + (p10 + p11);
            pa[rr] = MmaType<T>::pack(p00, p01);       // a0 / a1: keys 2t, 2t + 1
            pa[2 + rr] = MmaType<T>::pack(p10, p11);   // a2 / a3: keys 8 + 2t, 8 + 2t + 1
            pl[rr] = MmaType<T>::pack(p00 - MmaType<T>::lo(pa[rr]), p01 - MmaType<T>::hi(pa[rr]));
            pl[2 + rr] = MmaType<T>::pack(p10 - MmaType<T>::lo(pa[2 + rr]), p11 - MmaType<T>::hi(pa[2 + rr]));
        }
        // O[16 heads x 128 d] += P[16 x 16 keys] V[16 keys x 128 d], two N tiles of 8 d per load.
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            uint32_t vb[4];   // b0, b1 of d-tile n, then of n + 1
            const int row = (lm & 1) * 8 + lr, chunk = n + (lm >> 1);
            ldmatrix_x4_trans(vt + (uint32_t)(row * ROWB + ((chunk ^ (row & 7)) << 4)), vb);
            MmaType<T>::mma(o[n], pa, vb[0], vb[1]);
            MmaType<T>::mma(o[n], pl, vb[0], vb[1]);
            MmaType<T>::mma(o[n + 1], pa, vb[2], vb[3]);
            MmaType<T>::mma(o[n + 1], pl, vb[2], vb[3]);
        }
    }
    cp_async_wait<0>();

    // Each row's sum over the four lanes that share it, then the normalised partial and its log-sum-exp.
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
        const int hg = g_base + g + 8 * rr;
        if (hg < group) {
            const int h = hk * group + hg;
            const float inv = l[rr] > 0.f ? 1.f / l[rr] : 0.f;
            float *po = a.part_o + (((int64_t)b * a.hq + h) * a.splits + split) * DFULL + d0 + 2 * t;
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<float2 *>(po + n * 8) = make_float2(o[n][2 * rr] * inv, o[n][2 * rr + 1] * inv);
            if (t == 0 && part == 0) a.part_lse[((int64_t)b * a.hq + h) * a.splits + split] = l[rr] > 0.f ? m[rr] * a.scale + __logf(l[rr]) : -INFINITY;
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
    // The appending step: the row at `pos` comes from the new rows, and the warp of the group's
    // first head whose chunk holds it also writes it into the cache.
    const int pos = decode_append_at(a, b);
    const T *knew = static_cast<const T *>(a.k_new) + ((int64_t)b * a.hkv + hk) * a.d;
    const T *vnew = static_cast<const T *>(a.v_new) + ((int64_t)b * a.hkv + hk) * a.d;
    if (pos >= c0 && pos < c1 && h % (a.hq / a.hkv) == 0) {
        for (int c = lane; c < a.d; c += 32) {
            const_cast<T *>(static_cast<const T *>(a.k.ptr))[(int64_t)b * a.k.sb + (int64_t)pos * a.k.st + (int64_t)hk * a.k.sh + (int64_t)c * a.k.sd] = knew[c];
            const_cast<T *>(static_cast<const T *>(a.v.ptr))[(int64_t)b * a.v.sb + (int64_t)pos * a.v.st + (int64_t)hk * a.v.sh + (int64_t)c * a.v.sd] = vnew[c];
        }
    }
    float m = -INFINITY, l = 0.f;
    for (int key = c0; key < c1; ++key) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int c = lane + 32 * i;
            if (i < ni && c < a.d) d = fmaf(q[i], key == pos ? Num<T>::to_f32(knew[c]) : load_f32<T>(a.k, b, key, hk, c), d);
        }
        const float s = warp_sum(d) * a.scale;
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), p = expf(s - mn);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int c = lane + 32 * i;
            float v = (i < ni && c < a.d) ? (key == pos ? Num<T>::to_f32(vnew[c]) : load_f32<T>(a.v, b, key, hk, c)) : 0.f;
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

// Merges the partials of one (sequence, query head) by their log-sum-exp: the weights once into
// shared memory, then every thread its head dimensions over the splits.
constexpr int MERGE_MAX = 1024;  // splits whose weights fit the shared array; more are folded in passes

template <typename T>
__global__ void __launch_bounds__(128) decode_merge_kernel(DecodeArgs a) {
    __shared__ float w[MERGE_MAX];
    __shared__ float red[4];
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
    for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, lse[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));

    if (a.d % 4 == 0) {
        // Four head dimensions a thread (16-byte loads of the partials), the splits dealt over the
        // 128 / (d / 4) groups of threads, whose sums meet in shared memory in group order.
        __shared__ float4 part[128];
        __shared__ float dens[128];
        const int ct = a.d / 4, groups = 128 / ct;
        const int c4 = threadIdx.x % ct, sg = threadIdx.x / ct;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        float den = 0.f;
        for (int i0 = 0; i0 < n; i0 += MERGE_MAX) {
            const int m = min(MERGE_MAX, n - i0);
            __syncthreads();
            for (int i = threadIdx.x; i < m; i += blockDim.x) w[i] = expf(lse[i0 + i] - mx);
            __syncthreads();
            if (sg < groups) {
#pragma unroll 4
                for (int i = sg; i < m; i += groups) {
                    const float wi = w[i];
                    const float4 x = *reinterpret_cast<const float4 *>(po + (int64_t)(i0 + i) * a.d + 4 * c4);
                    den += wi;
                    num.x = fmaf(wi, x.x, num.x);
                    num.y = fmaf(wi, x.y, num.y);
                    num.z = fmaf(wi, x.z, num.z);
                    num.w = fmaf(wi, x.w, num.w);
                }
            }
        }
        part[threadIdx.x] = num;
        dens[threadIdx.x] = den;
        __syncthreads();
        if (sg == 0) {
            for (int g = 1; g < groups; ++g) {
                const float4 x = part[g * ct + c4];
                num.x += x.x; num.y += x.y; num.z += x.z; num.w += x.w;
                den += dens[g * ct + c4];
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            T *o = out + 4 * c4;
            o[0] = Num<T>::from_f32(num.x * inv);
            o[1] = Num<T>::from_f32(num.y * inv);
            o[2] = Num<T>::from_f32(num.z * inv);
            o[3] = Num<T>::from_f32(num.w * inv);
        }
        return;
    }
    float num[2] = {0.f, 0.f}, den = 0.f;  // a.d <= 256: two head dimensions per thread at most
    for (int i0 = 0; i0 < n; i0 += MERGE_MAX) {
        const int m = min(MERGE_MAX, n - i0);
        __syncthreads();
        for (int i = threadIdx.x; i < m; i += blockDim.x) w[i] = expf(lse[i0 + i] - mx);
        __syncthreads();
#pragma unroll 4
        for (int i = 0; i < m; ++i) {
            const float wi = w[i];
            den += wi;
            const float *row = po + (int64_t)(i0 + i) * a.d;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int c = threadIdx.x + 128 * k;
                if (c < a.d) num[k] = fmaf(wi, row[c], num[k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int c = threadIdx.x + 128 * k;
        if (c < a.d) out[c] = Num<T>::from_f32(den > 0.f ? num[k] / den : 0.f);
    }
}

template <typename T, int D, int GH>
static cudaError_t split_vec_g(const DecodeArgs &a, dim3 grid, cudaStream_t stream) {
    constexpr int VPK = sizeof(T) == 4 ? 2 : 1, NS = sizeof(T) == 4 ? 2 : DEC_STAGES;
    constexpr size_t smem = (size_t)DEC_WARPS * NS * (2 * DEC_UNROLL * VPK) * 32 * 16;
    cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<T, D, GH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    decode_split_kernel<T, D, GH><<<grid, DEC_WARPS * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

template <typename T, int D>
static cudaError_t split_vec(const DecodeArgs &a, cudaStream_t stream) {
    const int group = a.hq / a.hkv;
    const int gh = group >= 4 ? 4 : (group >= 2 ? 2 : 1);
    const int passes = (group + gh - 1) / gh;
    const long long units = (long long)a.splits * a.hkv * passes;
    dim3 grid((unsigned)((units + DEC_WARPS - 1) / DEC_WARPS), a.b);
    if (gh == 4) return split_vec_g<T, D, 4>(a, grid, stream);
    if (gh == 2) return split_vec_g<T, D, 2>(a, grid, stream);
    return split_vec_g<T, D, 1>(a, grid, stream);
}

template <typename T, int DFULL>
static cudaError_t split_mma(const DecodeArgs &a, cudaStream_t stream) {
    constexpr int PARTS = DFULL > 128 ? 2 : 1, D = DFULL / PARTS;
    constexpr size_t smem = (size_t)DM_WARPS * DM_STAGES * 2 * DM_KEYS * 2 * D + (PARTS == 2 ? (size_t)DM_WARPS * 32 * 8 * sizeof(float) : 0);
    cudaError_t e = cudaFuncSetAttribute(decode_split_mma_kernel<T, D, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long units = (long long)a.splits * a.hkv * PARTS * ((a.hq / a.hkv + 15) / 16);
    dim3 grid((unsigned)((units + DM_WARPS - 1) / DM_WARPS), a.b);
    decode_split_mma_kernel<T, D, PARTS><<<grid, DM_WARPS * 32, smem, stream>>>(a);
    return cudaGetLastError();
}
template <> cudaError_t split_mma<float, 128>(const DecodeArgs &, cudaStream_t) { return cudaErrorInvalidValue; }   // never taken: 16-bit caches only
template <> cudaError_t split_mma<float, 64>(const DecodeArgs &, cudaStream_t) { return cudaErrorInvalidValue; }
template <> cudaError_t split_mma<float, 256>(const DecodeArgs &, cudaStream_t) { return cudaErrorInvalidValue; }

// DASH_ATTN_DECODE_MMA=0 keeps the FMA pass (for comparison runs).
static bool decode_force_scalar_pass() {
    static const bool off = [] { const char *e = std::getenv("DASH_ATTN_DECODE_MMA"); return e && std::atoi(e) == 0; }();
    return off;
}

template <typename T>
static cudaError_t decode_t(const DecodeArgs &a, bool vector_ok, cudaStream_t stream, int *launches) {
    cudaError_t e;
    const bool mma = vector_ok && sizeof(T) == 2 && a.hq / a.hkv >= 2 && !decode_force_scalar_pass();
    if (mma && a.d == 128) e = split_mma<T, 128>(a, stream);
    else if (mma && a.d == 64) e = split_mma<T, 64>(a, stream);
    else if (mma && a.d == 256) e = split_mma<T, 256>(a, stream);
    else if (vector_ok && a.d == 64) e = split_vec<T, 64>(a, stream);
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
