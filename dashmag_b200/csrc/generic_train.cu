// The generic training kernels: forward, delta, query gradient, key/value gradients.
//
// They take every call of the contract (f32 / bf16 / f16, any head dimension up to 256, any
// strides, every mask, Tq != Tk, queries that see no key) with plain f32 FMAs on the CUDA cores:
// this is the IEEE-f32 path (no TF32, crates/dash-contract/src/lib.rs:69) and the path of the
// shapes the tensor-core kernels do not take.  No T x T matrix is ever held; the backward
// recomputes the scores tile by tile from the saved log-sum-exp, and sums every gradient in a
// fixed order (no atomics), so its results are the same bits on every run.
//
// Work split: a block of 256 threads owns 32 rows (queries, or keys in the key/value gradient
// kernel), four per warp; the other side streams through shared memory in tiles of 32, one per
// lane.  A lane forms the dot products of its tile row with the warp's four rows, the warp
// reduces the softmax statistics with shuffles, and for the second product each lane owns the
// head dimensions `lane + 32 i`.
#include "common.cuh"
#include "launch.h"

namespace dash {

constexpr int ROWS = 32;      // rows per block
constexpr int RPW = 4;        // rows per warp
constexpr int TILE = 32;      // streamed rows per tile (one per lane)
constexpr int THREADS = 256;
constexpr int MAXI = 8;       // ceil(256 / 32) owned head dimensions per lane

__host__ __device__ inline int padded_d(int d) { return (d + 3) & ~3; }

// Copies rows [r0, r0 + 32) of one head into shared memory as f32, zero past `limit` and past d.
template <typename T>
__device__ __forceinline__ void stage_rows(float *dst, int stride, const View4 &src, int b, int h,
                                           int r0, int limit, int d, int dp) {
    for (int idx = threadIdx.x; idx < TILE * dp; idx += THREADS) {
        int r = idx / dp, c = idx - r * dp;
        float x = 0.f;
        if (r0 + r < limit && c < d) x = load_f32<T>(src, b, r0 + r, h, c);
        dst[r * stride + c] = x;
    }
}

// dot[r] = sum_c rows[(w*4 + r)][c] * tile[lane][c], the four rows read as broadcast float4.
__device__ __forceinline__ void dots4(const float *rows, int row_stride, const float *tile_row,
                                      int dp, float (&acc)[RPW]) {
#pragma unroll
    for (int r = 0; r < RPW; ++r) acc[r] = 0.f;
    for (int c = 0; c < dp; c += 4) {
        float t0 = tile_row[c], t1 = tile_row[c + 1], t2 = tile_row[c + 2], t3 = tile_row[c + 3];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            float4 x = *reinterpret_cast<const float4 *>(rows + r * row_stride + c);
            acc[r] = fmaf(x.x, t0, acc[r]);
            acc[r] = fmaf(x.y, t1, acc[r]);
            acc[r] = fmaf(x.z, t2, acc[r]);
            acc[r] = fmaf(x.w, t3, acc[r]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) generic_forward_kernel(TrainArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int dp = padded_d(a.d);
    float *qs = smem;                          // [32][dp]
    float *ks = qs + ROWS * dp;                // [32][dp + 1]
    float *vs = ks + TILE * (dp + 1);          // [32][dp]
    float *ps = vs + TILE * dp;                // [8 warps][32 keys][4 rows]
    int *los = reinterpret_cast<int *>(ps + 8 * TILE * RPW);  // [32]
    int *his = los + ROWS;                     // [32]
    int *pad = his + ROWS;                     // [32] key padding flags of the tile
    __shared__ int span[2];

    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int qt = gridDim.x - 1 - blockIdx.x;  // long (late) causal rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (a.hq / a.hkv);
    const int row0 = qt * ROWS;

    stage_rows<T>(qs, dp, a.q, b, h, row0, a.tq, a.d, dp);
    if (threadIdx.x < ROWS) {
        int lo, hi;
        row_bounds(a.mask, row0 + threadIdx.x, a.tq, a.tk, lo, hi);
        los[threadIdx.x] = lo;
        his[threadIdx.x] = hi;
        int kmin = warp_min_i(hi > lo ? lo : a.tk);
        int kmax = warp_max_i(hi > lo ? hi : 0);
        if (threadIdx.x == 0) { span[0] = kmin; span[1] = kmax; }
    }
    __syncthreads();
    const int kmin = span[0], kmax = span[1];

    int lo[RPW], hi[RPW];
    int wlo = a.tk, whi = 0;
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        lo[r] = los[w * RPW + r];
        hi[r] = his[w * RPW + r];
        if (hi[r] > lo[r]) { wlo = min(wlo, lo[r]); whi = max(whi, hi[r]); }
    }
    float m[RPW], l[RPW], acc[RPW][MAXI];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < MAXI; ++i) acc[r][i] = 0.f;
    }
    const int ni = (dp + 31) / 32;

    for (int k0 = (kmin / TILE) * TILE; k0 < kmax; k0 += TILE) {
        __syncthreads();
        stage_rows<T>(ks, dp + 1, a.k, b, hk, k0, a.tk, a.d, dp);
        stage_rows<T>(vs, dp, a.v, b, hk, k0, a.tk, a.d, dp);
        if (threadIdx.x < TILE) {
            int key = k0 + threadIdx.x;
            pad[threadIdx.x] = key < a.tk ? (key_padded(a.mask, b, key) ? 1 : 0) : 1;
        }
        __syncthreads();
        if (k0 + TILE <= wlo || k0 >= whi) continue;  // no row of this warp sees the tile

        float s[RPW];
        dots4(qs + w * RPW * dp, dp, ks + lane * (dp + 1), dp, s);
        const int key = k0 + lane;
        const bool open = pad[lane] == 0;
        float4 p4;
        float *pp = reinterpret_cast<float *>(&p4);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            bool vis = open && key >= lo[r] && key < hi[r];
            float sr = vis ? s[r] * a.scale : -INFINITY;
            float mt = warp_max(sr);
            float mn = fmaxf(m[r], mt);
            float p = 0.f, alpha = 1.f;
            if (mn != -INFINITY) {
                alpha = expf(m[r] - mn);  // exp(-inf) = 0 on the first visible tile
                p = expf(sr - mn);
            }
            l[r] = l[r] * alpha + warp_sum(p);
#pragma unroll
            for (int i = 0; i < MAXI; ++i) acc[r][i] *= alpha;
            m[r] = mn;
            pp[r] = p;
        }
        float4 *pw = reinterpret_cast<float4 *>(ps) + w * TILE;
        pw[lane] = p4;
        __syncwarp();
        for (int j = 0; j < TILE; ++j) {
            float4 pj = pw[j];
#pragma unroll
            for (int i = 0; i < MAXI; ++i) {
                if (i < ni) {
                    int c = lane + 32 * i;
                    float v = c < dp ? vs[j * dp + c] : 0.f;
                    acc[0][i] = fmaf(pj.x, v, acc[0][i]);
                    acc[1][i] = fmaf(pj.y, v, acc[1][i]);
                    acc[2][i] = fmaf(pj.z, v, acc[2][i]);
                    acc[3][i] = fmaf(pj.w, v, acc[3][i]);
                }
            }
        }
        __syncwarp();
    }

    T *out = static_cast<T *>(a.out);
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        int row = row0 + w * RPW + r;
        if (row >= a.tq) continue;
        float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        int64_t base = (((int64_t)b * a.tq + row) * a.hq + h);
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            int c = lane + 32 * i;
            if (i < ni && c < a.d) out[base * a.d + c] = Num<T>::from_f32(acc[r][i] * inv);
        }
        if (lane == 0) a.lse[base] = l[r] > 0.f ? m[r] + logf(l[r]) : -INFINITY;
    }
}

// ---------------------------------------------------------------------------------------------
// delta = rowsum(dO * O), one warp per (batch, query, head); from the output as stored.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) generic_delta_kernel(TrainArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = (int64_t)a.b * a.tq * a.hq;
    int64_t row = (int64_t)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int h = (int)(row % a.hq);
    int64_t bt = row / a.hq;
    int t = (int)(bt % a.tq), b = (int)(bt / a.tq);
    float sum = 0.f;
    for (int c = lane; c < a.d; c += 32) sum = fmaf(load_f32<T>(a.dout, b, t, h, c), load_f32<T>(a.o, b, t, h, c), sum);
    sum = warp_sum(sum);
    if (lane == 0) a.delta[row] = sum;
}

// ---------------------------------------------------------------------------------------------
// dQ: each block of 32 queries sweeps, in order, the key tiles it sees.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) generic_dq_kernel(TrainArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int dp = padded_d(a.d);
    float *qs = smem;                          // [32][dp]
    float *gs = qs + ROWS * dp;                // [32][dp]   dO
    float *ks = gs + ROWS * dp;                // [32][dp + 1]
    float *vs = ks + TILE * (dp + 1);          // [32][dp + 1]
    float *ps = vs + TILE * (dp + 1);          // [8][32][4]  dS
    int *los = reinterpret_cast<int *>(ps + 8 * TILE * RPW);
    int *his = los + ROWS;
    int *pad = his + ROWS;
    __shared__ int span[2];

    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int qt = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (a.hq / a.hkv);
    const int row0 = qt * ROWS;

    stage_rows<T>(qs, dp, a.q, b, h, row0, a.tq, a.d, dp);
    stage_rows<T>(gs, dp, a.dout, b, h, row0, a.tq, a.d, dp);
    if (threadIdx.x < ROWS) {
        int lo, hi;
        row_bounds(a.mask, row0 + threadIdx.x, a.tq, a.tk, lo, hi);
        los[threadIdx.x] = lo;
        his[threadIdx.x] = hi;
        int kmin = warp_min_i(hi > lo ? lo : a.tk);
        int kmax = warp_max_i(hi > lo ? hi : 0);
        if (threadIdx.x == 0) { span[0] = kmin; span[1] = kmax; }
    }
    __syncthreads();
    const int kmin = span[0], kmax = span[1];

    int lo[RPW], hi[RPW];
    float lse[RPW], delta[RPW];
    int wlo = a.tk, whi = 0;
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        int row = row0 + w * RPW + r;
        lo[r] = los[w * RPW + r];
        hi[r] = his[w * RPW + r];
        if (hi[r] > lo[r]) { wlo = min(wlo, lo[r]); whi = max(whi, hi[r]); }
        float x = INFINITY, dl = 0.f;
        if (row < a.tq) {
            int64_t at = ((int64_t)b * a.tq + row) * a.hq + h;
            x = a.lse[at];
            dl = a.delta[at];
        }
        lse[r] = x == -INFINITY ? INFINITY : x;  // a query that saw no key: P = 0
        delta[r] = dl;
    }
    float acc[RPW][MAXI];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int i = 0; i < MAXI; ++i) acc[r][i] = 0.f;
    const int ni = (dp + 31) / 32;

    for (int k0 = (kmin / TILE) * TILE; k0 < kmax; k0 += TILE) {
        __syncthreads();
        stage_rows<T>(ks, dp + 1, a.k, b, hk, k0, a.tk, a.d, dp);
        stage_rows<T>(vs, dp + 1, a.v, b, hk, k0, a.tk, a.d, dp);
        if (threadIdx.x < TILE) {
            int key = k0 + threadIdx.x;
            pad[threadIdx.x] = key < a.tk ? (key_padded(a.mask, b, key) ? 1 : 0) : 1;
        }
        __syncthreads();
        if (k0 + TILE <= wlo || k0 >= whi) continue;

        float s[RPW], dpv[RPW];
        dots4(qs + w * RPW * dp, dp, ks + lane * (dp + 1), dp, s);
        dots4(gs + w * RPW * dp, dp, vs + lane * (dp + 1), dp, dpv);
        const int key = k0 + lane;
        const bool open = pad[lane] == 0;
        float4 d4;
        float *dd = reinterpret_cast<float *>(&d4);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            bool vis = open && key >= lo[r] && key < hi[r];
            float p = vis ? expf(s[r] * a.scale - lse[r]) : 0.f;
            dd[r] = p * (dpv[r] - delta[r]);
        }
        float4 *pw = reinterpret_cast<float4 *>(ps) + w * TILE;
        pw[lane] = d4;
        __syncwarp();
        for (int j = 0; j < TILE; ++j) {
            float4 dj = pw[j];
#pragma unroll
            for (int i = 0; i < MAXI; ++i) {
                if (i < ni) {
                    int c = lane + 32 * i;
                    float kv = c < dp ? ks[j * (dp + 1) + c] : 0.f;
                    acc[0][i] = fmaf(dj.x, kv, acc[0][i]);
                    acc[1][i] = fmaf(dj.y, kv, acc[1][i]);
                    acc[2][i] = fmaf(dj.z, kv, acc[2][i]);
                    acc[3][i] = fmaf(dj.w, kv, acc[3][i]);
                }
            }
        }
        __syncwarp();
    }

    T *dq = static_cast<T *>(a.dq);
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        int row = row0 + w * RPW + r;
        if (row >= a.tq) continue;
        int64_t base = (((int64_t)b * a.tq + row) * a.hq + h) * a.d;
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            int c = lane + 32 * i;
            if (i < ni && c < a.d) dq[base + c] = Num<T>::from_f32(acc[r][i] * a.scale);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// dK, dV: each block of 32 keys sweeps, in order, the query heads of its group and the query
// tiles that see it; a warp owns four keys, a lane one query of the tile.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) generic_dkdv_kernel(TrainArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int dp = padded_d(a.d);
    float *ks = smem;                          // [32][dp]
    float *vs = ks + ROWS * dp;                // [32][dp]
    float *qs = vs + ROWS * dp;                // [32][dp + 1]
    float *gs = qs + TILE * (dp + 1);          // [32][dp + 1]  dO
    float *ps = gs + TILE * (dp + 1);          // [8][32][4]  P
    float *ds = ps + 8 * TILE * RPW;           // [8][32][4]  dS
    float *lses = ds + 8 * TILE * RPW;         // [32]
    float *deltas = lses + TILE;               // [32]
    int *los = reinterpret_cast<int *>(deltas + TILE);
    int *his = los + TILE;
    __shared__ int span[2];
    __shared__ int red[2][THREADS / 32];

    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int group = a.hq / a.hkv;
    const int key0 = kt * ROWS;

    stage_rows<T>(ks, dp, a.k, b, hk, key0, a.tk, a.d, dp);
    stage_rows<T>(vs, dp, a.v, b, hk, key0, a.tk, a.d, dp);

    // The queries that see some key of [key0, key0 + 32): first and one past the last.
    {
        const int k1 = min(key0 + ROWS, a.tk);
        int first = a.tq, end = 0;
        for (int row = threadIdx.x; row < a.tq; row += THREADS) {
            int lo, hi;
            row_bounds(a.mask, row, a.tq, a.tk, lo, hi);
            if (hi > lo && lo < k1 && hi > key0) { first = min(first, row); end = max(end, row + 1); }
        }
        first = warp_min_i(first);
        end = warp_max_i(end);
        if (lane == 0) { red[0][w] = first; red[1][w] = end; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 1; i < THREADS / 32; ++i) { first = min(first, red[0][i]); end = max(end, red[1][i]); }
            span[0] = first;
            span[1] = end;
        }
        __syncthreads();
    }
    const int qfirst = span[0], qend = span[1];

    bool open[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        int key = key0 + w * RPW + r;
        open[r] = key < a.tk && !key_padded(a.mask, b, key);
    }
    float acck[RPW][MAXI], accv[RPW][MAXI];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int i = 0; i < MAXI; ++i) { acck[r][i] = 0.f; accv[r][i] = 0.f; }
    const int ni = (dp + 31) / 32;

    for (int g = 0; g < group; ++g) {
        const int h = hk * group + g;
        for (int q0 = (qfirst / TILE) * TILE; q0 < qend; q0 += TILE) {
            __syncthreads();
            stage_rows<T>(qs, dp + 1, a.q, b, h, q0, a.tq, a.d, dp);
            stage_rows<T>(gs, dp + 1, a.dout, b, h, q0, a.tq, a.d, dp);
            if (threadIdx.x < TILE) {
                int row = q0 + threadIdx.x;
                int lo, hi;
                row_bounds(a.mask, row, a.tq, a.tk, lo, hi);
                los[threadIdx.x] = lo;
                his[threadIdx.x] = hi;
                float x = INFINITY, dl = 0.f;
                if (row < a.tq) {
                    int64_t at = ((int64_t)b * a.tq + row) * a.hq + h;
                    x = a.lse[at];
                    dl = a.delta[at];
                }
                lses[threadIdx.x] = x == -INFINITY ? INFINITY : x;
                deltas[threadIdx.x] = dl;
            }
            __syncthreads();

            float s[RPW], dpv[RPW];
            dots4(ks + w * RPW * dp, dp, qs + lane * (dp + 1), dp, s);
            dots4(vs + w * RPW * dp, dp, gs + lane * (dp + 1), dp, dpv);
            const int lo = los[lane], hi = his[lane];
            const float lse = lses[lane], delta = deltas[lane];
            float4 p4, d4;
            float *pp = reinterpret_cast<float *>(&p4), *dd = reinterpret_cast<float *>(&d4);
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                int key = key0 + w * RPW + r;
                bool vis = open[r] && key >= lo && key < hi;
                float p = vis ? expf(s[r] * a.scale - lse) : 0.f;
                pp[r] = p;
                dd[r] = p * (dpv[r] - delta);
            }
            float4 *pw = reinterpret_cast<float4 *>(ps) + w * TILE;
            float4 *dw = reinterpret_cast<float4 *>(ds) + w * TILE;
            pw[lane] = p4;
            dw[lane] = d4;
            __syncwarp();
            for (int j = 0; j < TILE; ++j) {
                float4 pj = pw[j], dj = dw[j];
#pragma unroll
                for (int i = 0; i < MAXI; ++i) {
                    if (i < ni) {
                        int c = lane + 32 * i;
                        float gv = c < dp ? gs[j * (dp + 1) + c] : 0.f;
                        float qv = c < dp ? qs[j * (dp + 1) + c] : 0.f;
                        accv[0][i] = fmaf(pj.x, gv, accv[0][i]);
                        accv[1][i] = fmaf(pj.y, gv, accv[1][i]);
                        accv[2][i] = fmaf(pj.z, gv, accv[2][i]);
                        accv[3][i] = fmaf(pj.w, gv, accv[3][i]);
                        acck[0][i] = fmaf(dj.x, qv, acck[0][i]);
                        acck[1][i] = fmaf(dj.y, qv, acck[1][i]);
                        acck[2][i] = fmaf(dj.z, qv, acck[2][i]);
                        acck[3][i] = fmaf(dj.w, qv, acck[3][i]);
                    }
                }
            }
            __syncwarp();
        }
    }

    T *dk = static_cast<T *>(a.dk), *dv = static_cast<T *>(a.dv);
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        int key = key0 + w * RPW + r;
        if (key >= a.tk) continue;
        int64_t base = (((int64_t)b * a.tk + key) * a.hkv + hk) * a.d;
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            int c = lane + 32 * i;
            if (i < ni && c < a.d) {
                dk[base + c] = Num<T>::from_f32(acck[r][i] * a.scale);
                dv[base + c] = Num<T>::from_f32(accv[r][i]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------------------
static size_t forward_smem(int d) {
    int dp = padded_d(d);
    return sizeof(float) * (ROWS * dp + TILE * (dp + 1) + TILE * dp + 8 * TILE * RPW) + sizeof(int) * 3 * ROWS;
}
static size_t dq_smem(int d) {
    int dp = padded_d(d);
    return sizeof(float) * (2 * ROWS * dp + 2 * TILE * (dp + 1) + 8 * TILE * RPW) + sizeof(int) * 3 * ROWS;
}
static size_t dkdv_smem(int d) {
    int dp = padded_d(d);
    return sizeof(float) * (2 * ROWS * dp + 2 * TILE * (dp + 1) + 2 * 8 * TILE * RPW + 2 * TILE) + sizeof(int) * 2 * TILE;
}

template <typename T>
static cudaError_t forward_t(const TrainArgs &a, cudaStream_t stream, int *launches) {
    size_t smem = forward_smem(a.d);
    cudaError_t e = cudaFuncSetAttribute(generic_forward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((a.tq + ROWS - 1) / ROWS, a.hq, a.b);
    generic_forward_kernel<T><<<grid, THREADS, smem, stream>>>(a);
    *launches += 1;
    return cudaGetLastError();
}

template <typename T>
static cudaError_t backward_t(const TrainArgs &a, cudaStream_t stream, int *launches) {
    cudaError_t e;
    {
        int64_t rows = (int64_t)a.b * a.tq * a.hq;
        unsigned blocks = (unsigned)((rows + THREADS / 32 - 1) / (THREADS / 32));
        generic_delta_kernel<T><<<blocks, THREADS, 0, stream>>>(a);
        *launches += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    {
        size_t smem = dq_smem(a.d);
        e = cudaFuncSetAttribute(generic_dq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        dim3 grid((a.tq + ROWS - 1) / ROWS, a.hq, a.b);
        generic_dq_kernel<T><<<grid, THREADS, smem, stream>>>(a);
        *launches += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    {
        size_t smem = dkdv_smem(a.d);
        e = cudaFuncSetAttribute(generic_dkdv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        dim3 grid((a.tk + ROWS - 1) / ROWS, a.hkv, a.b);
        generic_dkdv_kernel<T><<<grid, THREADS, smem, stream>>>(a);
        *launches += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// The same for 16-bit rows of D = 64, 128 or 256 elements that can be read 16 bytes at a time: D / 8
// lanes a row (at 128: sixteen lanes a row, two rows a warp), the row's bytes of each tensor in one
// request.
template <typename T, int D>
__global__ void __launch_bounds__(THREADS) delta_rows_kernel(TrainArgs a) {
    constexpr int LPR = D / 8, RPW = 32 / LPR;   // lanes per row, rows per warp
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    const int64_t rows = (int64_t)a.b * a.tq * a.hq;
    const int64_t row = ((int64_t)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5)) * RPW + lane / LPR;
    float sum = 0.f;
    if (row < rows) {
        const int h = (int)(row % a.hq);
        const int64_t bt = row / a.hq;
        const int64_t t = bt % a.tq, b = bt / a.tq;
        const uint4 g = *reinterpret_cast<const uint4 *>(static_cast<const T *>(a.dout.ptr) + b * a.dout.sb + t * a.dout.st + h * a.dout.sh + sub * 8);
        const uint4 o = *reinterpret_cast<const uint4 *>(static_cast<const T *>(a.o.ptr) + b * a.o.sb + t * a.o.st + h * a.o.sh + sub * 8);
        const T *gv = reinterpret_cast<const T *>(&g), *ov = reinterpret_cast<const T *>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) sum = fmaf(Num<T>::to_f32(gv[i]), Num<T>::to_f32(ov[i]), sum);
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (row < rows && sub == 0) a.delta[row] = sum;
}

// Whether every row of the view starts on a 16-byte boundary and is contiguous.
static bool rows_16b(const View4 &v) {
    return v.sd == 1 && reinterpret_cast<uintptr_t>(v.ptr) % 16 == 0 && v.sb % 8 == 0 && v.st % 8 == 0 && v.sh % 8 == 0;
}

template <typename T>
static cudaError_t delta_t(const TrainArgs &a, cudaStream_t stream, int *launches) {
    int64_t rows = (int64_t)a.b * a.tq * a.hq;
    if (sizeof(T) == 2 && (a.d == 64 || a.d == 128 || a.d == 256) && rows_16b(a.dout) && rows_16b(a.o)) {
        const int64_t per_block = (32 / (a.d / 8)) * (THREADS / 32);
        const unsigned blocks = (unsigned)((rows + per_block - 1) / per_block);
        if (a.d == 64) delta_rows_kernel<T, 64><<<blocks, THREADS, 0, stream>>>(a);
        else if (a.d == 128) delta_rows_kernel<T, 128><<<blocks, THREADS, 0, stream>>>(a);
        else delta_rows_kernel<T, 256><<<blocks, THREADS, 0, stream>>>(a);
        *launches += 1;
        return cudaGetLastError();
    }
    unsigned blocks = (unsigned)((rows + THREADS / 32 - 1) / (THREADS / 32));
    generic_delta_kernel<T><<<blocks, THREADS, 0, stream>>>(a);
    *launches += 1;
    return cudaGetLastError();
}

// delta = rowsum(dO * O) alone, for the tensor-core backward.
cudaError_t launch_generic_delta(int dtype, const TrainArgs &a, cudaStream_t stream, int *launches) {
    switch (dtype) {
        case 0: return delta_t<float>(a, stream, launches);
        case 1: return delta_t<__nv_bfloat16>(a, stream, launches);
        default: return delta_t<__half>(a, stream, launches);
    }
}

cudaError_t launch_generic_forward(int dtype, const TrainArgs &a, cudaStream_t stream, int *launches) {
    switch (dtype) {
        case 0: return forward_t<float>(a, stream, launches);
        case 1: return forward_t<__nv_bfloat16>(a, stream, launches);
        default: return forward_t<__half>(a, stream, launches);
    }
}

cudaError_t launch_generic_backward(int dtype, const TrainArgs &a, cudaStream_t stream, int *launches) {
    switch (dtype) {
        case 0: return backward_t<float>(a, stream, launches);
        case 1: return backward_t<__nv_bfloat16>(a, stream, launches);
        default: return backward_t<__half>(a, stream, launches);
    }
}

}  // namespace dash
