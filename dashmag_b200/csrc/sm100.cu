// Host side of the tcgen05 path: which calls it takes, the TMA tensor maps over the caller's
// tensors, and the launches.
#include "sm100.h"

#include <cuda.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "launch.h"
#include "sm100_kernels.h"

namespace dash {

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library carries no
// link-time dependency on libcuda (it must load on machines without a driver).
EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    });
    return fn;
}

// Whether the current device is a compute-capability-10 part; -1 unknown, cached per device.
bool device_is_sm100() {
    static int cache[64];
    static std::once_flag once;
    std::call_once(once, [] { for (int &c : cache) c = -1; });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return false; }
    if (cache[dev] < 0) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        cache[dev] = major == 10 ? 1 : 0;
    }
    return cache[dev] == 1;
}

// The reference's in-place rule (crates/dash-ops/src/attention/cube.rs:428-461), which is also what
// a TMA tensor map needs: last stride 1, the others multiples of 16 bytes, base 16-byte aligned.
bool tma_readable(const void *ptr, const int64_t *stride) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || stride[3] != 1) return false;
    for (int i = 0; i < 3; ++i)
        if (stride[i] % 8 != 0 || stride[i] < 0) return false;
    return true;
}

// A [B, T, H, d] tensor of 16-bit elements (d = 64, 128 or 256) as a 4-D map (d, h, t, b) with boxes of
// 64 x 1 x 128 x 1 and the 128-byte swizzle: each load brings 128 rows of 128 bytes of one head.
// (dtype DASH_ATTN_F32: the fused backward's accumulator, 32 f32 columns to a 128-byte box row.)
bool encode_uncached(CUtensorMap *map, int dtype, const void *ptr, int b, int t, int h, const int64_t *stride, int rows, int d) {
    EncodeTiled fn = encoder();
    if (!fn) return false;
    const bool f32 = dtype == DASH_ATTN_F32;
    auto bytes = [f32](int64_t elems) { return static_cast<cuuint64_t>(elems) * (f32 ? 4 : 2); };
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)h, (cuuint64_t)t, (cuuint64_t)b};
    // A dimension of extent 1 never moves: give it any legal stride.
    cuuint64_t strides[3] = {h > 1 ? bytes(stride[2]) : 256, t > 1 ? bytes(stride[1]) : 256, b > 1 ? bytes(stride[0]) : 256};
    for (cuuint64_t s : strides)
        if (s == 0 || s % 16 != 0 || s >= (1ull << 40)) return false;
    cuuint32_t box[4] = {f32 ? 32u : 64u, 1, (cuuint32_t)rows, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == DASH_ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// A tensor map is a pure function of the address and the geometry it was encoded from, not of the
// bytes behind the address, and a training loop or a decoder calls with the same buffers step after
// step: the last maps are kept, keyed on everything the encoder reads, so that a repeated call costs
// a lookup instead of a trip through the driver per tensor (short calls are bound by exactly that
// host time, crates/dash-ops/src/attention.rs:123-127).
struct MapKey {
    const void *ptr;
    int dtype, b, t, h, rows, d;
    int64_t s0, s1, s2;
    bool operator==(const MapKey &o) const {
        return ptr == o.ptr && dtype == o.dtype && b == o.b && t == o.t && h == o.h && rows == o.rows && d == o.d &&
               s0 == o.s0 && s1 == o.s1 && s2 == o.s2;
    }
};
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int MAP_SLOTS = 64, MAP_WAYS = 4;
MapSlot g_maps[MAP_SLOTS];
unsigned g_map_turn[MAP_SLOTS / MAP_WAYS];
std::mutex g_map_mutex;
std::atomic<uint64_t> g_map_encodes{0};

bool encode(CUtensorMap *map, int dtype, const void *ptr, int b, int t, int h, const int64_t *stride, int rows = 128, int d = 128) {
    const MapKey key{ptr, dtype, b, t, h, rows, d, stride[0], stride[1], stride[2]};
    uint64_t x = reinterpret_cast<uintptr_t>(ptr) >> 4;
    x ^= (uint64_t)(unsigned)t * 0x9E3779B97F4A7C15ull + (uint64_t)(unsigned)h * 0xC2B2AE3D27D4EB4Full + (uint64_t)(unsigned)(rows + d + dtype);
    x ^= x >> 29;
    const int set = (int)(x % (MAP_SLOTS / MAP_WAYS));
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        for (int w = 0; w < MAP_WAYS; ++w) {
            const MapSlot &s = g_maps[set * MAP_WAYS + w];
            if (s.used && s.key == key) { *map = s.map; return true; }
        }
    }
    if (!encode_uncached(map, dtype, ptr, b, t, h, stride, rows, d)) return false;
    g_map_encodes.fetch_add(1, std::memory_order_relaxed);
    std::lock_guard<std::mutex> lock(g_map_mutex);
    MapSlot &s = g_maps[set * MAP_WAYS + (g_map_turn[set]++ % MAP_WAYS)];
    s.key = key;
    s.map = *map;
    s.used = true;
    return true;
}

float resolved_scale(const dash_attn_params *p) {
    return p->has_scale ? p->scale : (float)(1.0 / std::sqrt((double)p->d));
}

}  // namespace

uint64_t sm100_tensor_map_encodes() { return g_map_encodes.load(std::memory_order_relaxed); }

bool sm100_takes(const dash_attn_params *p, const void *q, const void *k, const void *v, int backward, bool any_size) {
    if (backward && !tma_readable(q, p->do_stride)) return false;  // dO's strides; its base is checked at launch
    if (p->dtype != DASH_ATTN_BF16 && p->dtype != DASH_ATTN_F16) return false;
    // Head dimensions 64 and 256 only from 128 queries and 128 keys on: below that there is a single
    // partial tile of queries or of keys (one block per head), the tensor cores gain nothing, and the
    // generic kernels' f32 FMA sums keep the log-sum-exp within the one or two units in the last place
    // that the reference's records allow at those sizes.  (`any_size`, a switch for tests, lifts the
    // size rule, so that the records themselves can be run through the tensor-core kernels.)
    // At 256 the forward is the one-tile kernel and the backward the three passes of bwd256_sm100.cu.
    const bool big = any_size || (p->tq >= 128 && p->tk >= 128);
    if (p->d != 128 && !((p->d == 64 || p->d == 256) && big)) return false;
    const float scale = resolved_scale(p);
    if (!(scale > 0.f) || !std::isfinite(scale)) return false;  // the row maximum is taken before scaling
    if (!q || !k || !v) return false;
    if (!tma_readable(q, p->q_stride) || !tma_readable(k, p->k_stride) || !tma_readable(v, p->v_stride)) return false;
    if (p->hq > 65535 || p->b > 65535) return false;   // grid extents
    if (!device_is_sm100() || !encoder()) return false;
    return true;
}

size_t sm100_forward_workspace(const dash_attn_params *) { return 0; }
// Whether a backward call takes the five-product form that adds dQ by reductions in L2: only when the
// caller gave up the fixed order of summation, and only where that form exists (D = 64, 128).
static bool fused_backward(const dash_attn_params *p) { return !p->deterministic && (p->d == 128 || p->d == 64); }
static size_t dq_acc_bytes(const dash_attn_params *p) {
    return (sizeof(float) * (size_t)p->b * p->tq * p->hq * p->d + 255) & ~size_t(255);
}
size_t sm100_backward_workspace(const dash_attn_params *p) {
    return bwd_sm100_order_bytes(p->b, p->tk, p->hkv) + (fused_backward(p) ? dq_acc_bytes(p) : 0);
}

cudaError_t sm100_forward(const dash_attn_params *p, const TrainArgs &a, void *, cudaStream_t stream, int *launches,
                          std::string &err) {
    // The two-tile kernel shares every K / V tile between two query tiles; DASH_ATTN_FWD_TILES=1
    // keeps the one-tile kernel (for comparison runs).
    static const bool one_tile = [] { const char *e = std::getenv("DASH_ATTN_FWD_TILES"); return e && std::atoi(e) == 1; }();
    const int kv_rows = 128;
    (void)one_tile;
    CUtensorMap tq, tk, tv, to;
    const int64_t o_stride[4] = {(int64_t)p->tq * p->hq * p->d, (int64_t)p->hq * p->d, p->d, 1};   // the output is contiguous
    if (!encode(&to, p->dtype, a.out, p->b, p->tq, p->hq, o_stride, 128, p->d) ||
        !encode(&tq, p->dtype, a.q.ptr, p->b, p->tq, p->hq, p->q_stride, 128, p->d) ||
        !encode(&tk, p->dtype, a.k.ptr, p->b, p->tk, p->hkv, p->k_stride, kv_rows, p->d) ||
        !encode(&tv, p->dtype, a.v.ptr, p->b, p->tk, p->hkv, p->v_stride, kv_rows, p->d)) {
        err = "attention: the driver refused a TMA tensor map over the inputs";
        return cudaSuccess;
    }
    Sm100FwdArgs f{};
    f.b = p->b; f.tq = p->tq; f.tk = p->tk; f.hq = p->hq; f.hkv = p->hkv; f.d = p->d;
    f.scale = a.scale;
    f.scale_log2 = a.scale * 1.4426950408889634f;
    f.out = a.out;
    f.lse = a.lse;
    f.mask = a.mask;
    f.pair_heads = ((p->hq / p->hkv) % 2 == 0) ? 1 : 0;
    cudaError_t e = ((one_tile && p->d == 128) || p->d == 256) ? launch_fwd_sm100(p->dtype, tq, tk, tv, f, stream) : launch_fwd2_sm100(p->dtype, tq, tk, tv, to, f, stream);
    *launches += 1;
    return e;
}

cudaError_t sm100_backward(const dash_attn_params *p, const TrainArgs &a, void *workspace, cudaStream_t stream, int *launches,
                           bool *atomic, std::string &err) {
    const bool fused = fused_backward(p);
    *atomic = fused;
    Sm100BwdMaps m;
    float *dq_acc = fused ? reinterpret_cast<float *>(static_cast<char *>(workspace) + bwd_sm100_order_bytes(p->b, p->tk, p->hkv)) : nullptr;
    const void *q = a.q.ptr, *k = a.k.ptr, *v = a.v.ptr, *g = a.dout.ptr;
    const int64_t dq_stride[4] = {(int64_t)p->tq * p->hq * p->d, (int64_t)p->hq * p->d, p->d, 1};   // the gradients are contiguous
    bool ok = encode(&m.dq128, p->dtype, a.dq, p->b, p->tq, p->hq, dq_stride, 128, p->d) &&
              encode(&m.q128, p->dtype, q, p->b, p->tq, p->hq, p->q_stride, 128, p->d) &&
              encode(&m.do128, p->dtype, g, p->b, p->tq, p->hq, p->do_stride, 128, p->d) &&
              encode(&m.k128, p->dtype, k, p->b, p->tk, p->hkv, p->k_stride, 128, p->d) &&
              encode(&m.v128, p->dtype, v, p->b, p->tk, p->hkv, p->v_stride, 128, p->d);
    if (ok && fused) ok = encode(&m.dq_acc, DASH_ATTN_F32, dq_acc, p->b, p->tq, p->hq, dq_stride, 128, p->d);
    else if (ok) m.dq_acc = m.dq128;   // not read
    if (!ok) {
        err = "attention_backward: the driver refused a TMA tensor map over the inputs";
        return cudaSuccess;
    }
    cudaError_t e = launch_generic_delta(p->dtype, a, stream, launches);
    if (e != cudaSuccess) return e;
    Sm100BwdArgs f{};
    f.b = p->b; f.tq = p->tq; f.tk = p->tk; f.hq = p->hq; f.hkv = p->hkv; f.d = p->d;
    f.scale = a.scale;
    f.scale_log2 = a.scale * 1.4426950408889634f;
    f.lse = a.lse;
    f.delta = a.delta;
    f.dq = a.dq; f.dk = a.dk; f.dv = a.dv;
    f.mask = a.mask;
    f.order = static_cast<int *>(workspace);
    f.dq_acc = dq_acc;
    if (p->d == 256) return launch_bwd256_sm100(p->dtype, m, f, stream, launches);
    return launch_bwd_sm100(p->dtype, m, f, stream, launches);
}

}  // namespace dash
