// The C ABI: refusals with the reference's wording, stride rules, workspace plans, path choice,
// probes.  Everything here is host code; nothing is launched when a call is refused.
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <algorithm>
#include <string>
#include <vector>

#include "../../include/dash_attn.h"
#include "common.cuh"
#include "launch.h"
#include "rope.h"
#include "sample.h"
#include "sm100.h"
#include "sm100_kernels.h"

namespace {

thread_local std::string g_error;
std::atomic<uint64_t> g_probe[DASH_ATTN_PROBE_COUNT];
std::atomic<int> g_force_generic{0};
std::atomic<int> g_force_tensor{0};

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

int cuda_fail(const char *op, cudaError_t e) {
    return fail(DASH_ATTN_CUDA, "%s: CUDA error: %s", op, cudaGetErrorString(e));
}

size_t elem_bytes(int dtype) { return dtype == DASH_ATTN_F32 ? 4 : 2; }
size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// crates/dash-contract/src/attention.rs:157-159
float scale_for(int has_scale, float scale, int d) {
    return has_scale ? scale : (float)(1.0 / std::sqrt((double)d));
}

dash::View4 view(const void *p, const int64_t s[4]) { return dash::View4{p, s[0], s[1], s[2], s[3]}; }

// The checks of check_shapes (crates/dash-ops/src/attention.rs:551-590), same order, same words.
int check_train(const char *op, const dash_attn_params *p) {
    if (!p) return fail(DASH_ATTN_INVALID, "%s: null parameters", op);
    if (p->dtype != DASH_ATTN_F32 && p->dtype != DASH_ATTN_BF16 && p->dtype != DASH_ATTN_F16)
        return fail(DASH_ATTN_INVALID, "%s: the dtype must be f32, bf16 or f16, got code %d", op, p->dtype);
    if (p->b < 0 || p->tq < 0 || p->tk < 0 || p->hq < 0 || p->hkv < 0 || p->d < 0)
        return fail(DASH_ATTN_INVALID, "%s: query is [B, Tq, Hq, D] and key is [B, Tk, Hkv, D], no dimension negative", op);
    if (p->v_tk != p->tk || p->v_hkv != p->hkv || p->v_d != p->k_d)
        return fail(DASH_ATTN_INVALID, "%s: key and value must have one shape", op);
    if (p->k_b != p->b) return fail(DASH_ATTN_INVALID, "%s: query and key must have one batch size", op);
    if (p->k_d != p->d) return fail(DASH_ATTN_INVALID, "%s: query and key must have one head dimension", op);
    if (!(p->hkv > 0 && p->hq % p->hkv == 0))
        return fail(DASH_ATTN_INVALID, "%s: the query heads (%d) must be a multiple of the key-value heads (%d)", op, p->hq, p->hkv);
    switch (p->mask_kind) {
        case DASH_ATTN_MASK_NONE: break;
        case DASH_ATTN_MASK_KEY_PADDING:
            if (p->key_padding_shape[0] != p->b || p->key_padding_shape[1] != p->tk)
                return fail(DASH_ATTN_INVALID, "%s: the key padding mask is [B, Tk] = [%d, %d]", op, p->b, p->tk);
            if (p->key_padding_elem_bytes != 1 && p->key_padding_elem_bytes != 4)
                return fail(DASH_ATTN_INVALID, "%s: the key padding mask holds 1-byte booleans or 4-byte integers", op);
            if (!p->key_padding && (int64_t)p->b * p->tk > 0)
                return fail(DASH_ATTN_INVALID, "%s: the key padding mask is null", op);
            break;
        case DASH_ATTN_MASK_PACKED:
            if (p->b != 1) return fail(DASH_ATTN_INVALID, "%s: packed sequences lie along the time, B = 1", op);
            if (!(p->cu_seqlens_q_len == p->cu_seqlens_k_len && p->cu_seqlens_q_len >= 1))
                return fail(DASH_ATTN_INVALID, "%s: cu_seqlens_q and cu_seqlens_k are [S + 1], one S, got [%d], [%d]", op,
                            p->cu_seqlens_q_len, p->cu_seqlens_k_len);
            if (p->index_elem_bytes != 4 && p->index_elem_bytes != 8)
                return fail(DASH_ATTN_INVALID, "%s: cu_seqlens hold 4- or 8-byte integers", op);
            if (!p->cu_seqlens_q || !p->cu_seqlens_k)
                return fail(DASH_ATTN_INVALID, "%s: cu_seqlens_q or cu_seqlens_k is null", op);
            break;
        default: return fail(DASH_ATTN_INVALID, "%s: unknown mask kind %d", op, p->mask_kind);
    }
    if (p->d > 256) return fail(DASH_ATTN_UNSUPPORTED, "%s: head dimension %d: this library takes up to 256", op, p->d);
    if ((int64_t)p->tq + p->tk + 1 > 0x3fffffff)
        return fail(DASH_ATTN_UNSUPPORTED, "%s: Tq + Tk = %lld: this library takes up to 2^30", op, (long long)p->tq + p->tk);
    return DASH_ATTN_OK;
}

bool degenerate(const dash_attn_params *p) {  // crates/dash-ops/src/attention/reference.rs:316, :386
    return (int64_t)p->b * p->tq * p->hq * p->d == 0 || p->tk == 0;
}

dash::MaskArgs mask_args(const dash_attn_params *p) {
    dash::MaskArgs m{};
    m.kind = p->mask_kind;
    m.kp = p->key_padding;
    m.kp_bytes = p->key_padding_elem_bytes;
    m.kp_sb = p->key_padding_stride[0];
    m.kp_st = p->key_padding_stride[1];
    m.cu_q = p->cu_seqlens_q;
    m.cu_k = p->cu_seqlens_k;
    m.seqs = p->cu_seqlens_q_len - 1;
    m.idx_bytes = p->index_elem_bytes;
    // crates/dash-ops/src/attention/cube.rs:520-531: Tq + Tk + 1 stands for "no bound".
    const int64_t none = (int64_t)p->tq + p->tk + 1;
    int64_t left = none, right = none;
    if (p->has_window) {
        if (p->window_left >= 0) left = p->window_left < none ? p->window_left : none;
        if (p->window_right >= 0) right = p->window_right < none ? p->window_right : none;
    }
    if (p->causal) right = 0;
    m.left = (int)left;
    m.right = (int)right;
    return m;
}

dash::TrainArgs train_args(const dash_attn_params *p, const void *q, const void *k, const void *v) {
    dash::TrainArgs a{};
    a.b = p->b; a.tq = p->tq; a.tk = p->tk; a.hq = p->hq; a.hkv = p->hkv; a.d = p->d;
    a.scale = scale_for(p->has_scale, p->scale, p->d);
    a.q = view(q, p->q_stride);
    a.k = view(k, p->k_stride);
    a.v = view(v, p->v_stride);
    a.mask = mask_args(p);
    return a;
}

// The reference's rule for reading an input in place with 16-byte vectors
// (crates/dash-ops/src/attention/cube.rs:428-461): last stride 1, the others whole vectors, the
// first element 16-byte aligned.
bool vector_readable(const void *ptr, const int64_t *stride, int n, size_t elem) {
    const int64_t per = (int64_t)(16 / elem);
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return false;
    if (stride[n - 1] != 1) return false;
    for (int i = 0; i < n - 1; ++i)
        if (stride[i] % per != 0) return false;
    return true;
}

int check_workspace(const char *op, void *ws, size_t have, size_t need) {
    if (need == 0) return DASH_ATTN_OK;
    if (!ws) return fail(DASH_ATTN_WORKSPACE, "%s: workspace is null, %zu bytes are needed", op, need);
    if (reinterpret_cast<uintptr_t>(ws) % 256 != 0) return fail(DASH_ATTN_WORKSPACE, "%s: workspace must be 256-byte aligned", op);
    if (have < need) return fail(DASH_ATTN_WORKSPACE, "%s: workspace holds %zu bytes, %zu are needed", op, have, need);
    return DASH_ATTN_OK;
}

int train_path(const dash_attn_params *p, const void *q, const void *k, const void *v, int backward) {
    if (g_force_generic.load()) return 0;
    return dash::sm100_takes(p, q, k, v, backward, g_force_tensor.load() != 0) ? 1 : 0;
}

// The tensor-core kernels write their outputs (and read dO) through TMA tiles and 16-byte vectors:
// a call whose output is not 16-byte aligned goes to the generic kernels, like one whose input is not.
bool aligned16(std::initializer_list<const void *> ptrs) {
    for (const void *x : ptrs)
        if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return false;
    return true;
}

// ---- decode ---------------------------------------------------------------------------------

int check_decode(const dash_attn_decode_params *p, const char *op = "attention_decode") {
    if (!p) return fail(DASH_ATTN_INVALID, "%s: null parameters", op);
    if (p->dtype != DASH_ATTN_F32 && p->dtype != DASH_ATTN_BF16 && p->dtype != DASH_ATTN_F16)
        return fail(DASH_ATTN_INVALID, "%s: the dtype must be f32, bf16 or f16, got code %d", op, p->dtype);
    if (p->b < 0 || p->s < 0 || p->hq < 0 || p->hkv < 0 || p->d < 0)
        return fail(DASH_ATTN_INVALID, "%s: query is [B, Hq, D] and key is [B, S, Hkv, D], no dimension negative", op);
    // check_decode_shapes runs check_shapes on [B, 1, Hq, D] (crates/dash-ops/src/attention.rs:629).
    if (p->v_b != p->k_b || p->v_s != p->s || p->v_hkv != p->hkv || p->v_d != p->k_d)
        return fail(DASH_ATTN_INVALID, "attention: key and value must have one shape");
    if (p->k_b != p->b) return fail(DASH_ATTN_INVALID, "attention: query and key must have one batch size");
    if (p->k_d != p->d) return fail(DASH_ATTN_INVALID, "attention: query and key must have one head dimension");
    if (!(p->hkv > 0 && p->hq % p->hkv == 0))
        return fail(DASH_ATTN_INVALID, "attention: the query heads (%d) must be a multiple of the key-value heads (%d)", p->hq, p->hkv);
    if (p->lengths) {
        if (p->lengths_len != p->b)
            return fail(DASH_ATTN_INVALID, "%s: the cache lengths are [B] = [%d]", op, p->b);
        if (p->lengths_elem_bytes != 4 && p->lengths_elem_bytes != 8)
            return fail(DASH_ATTN_INVALID, "%s: the cache lengths are 4- or 8-byte integers", op);
    }
    if (p->d > 256) return fail(DASH_ATTN_UNSUPPORTED, "%s: head dimension %d: this library takes up to 256", op, p->d);
    if (p->b > 65535) return fail(DASH_ATTN_UNSUPPORTED, "%s: batch %d: this library takes up to 65535", op, p->b);
    return DASH_ATTN_OK;
}

// Keys per split and splits per sequence: enough warps to fill the 148 multiprocessors of a B200
// several times over (16 resident warps each, 4 waves), between 64 and 512 keys a split so that
// the partial outputs stay a few percent of the cache traffic.  A pure function of the shape, so
// the workspace query and the launch agree without looking at the device.
void decode_plan(const dash_attn_decode_params *p, int *chunk, int *splits) {
    // DASH_ATTN_DECODE_CHUNK (read once, when the first plan is made) fixes the chunk for comparison runs.
    static const long long fixed = [] {
        const char *env = std::getenv("DASH_ATTN_DECODE_CHUNK");
        return env ? std::atoll(env) : 0LL;
    }();
    long long c = 512;
    if (fixed > 0) {
        c = fixed;
    } else {
        // Chunks of 128 to 512 keys, as long as they still leave units (a chunk of a key-value head;
        // a group of more than sixteen query heads counts once per sixteen) to fill the warps of the GPU:
        // under 128 keys a warp's set-up outweighs its tiles.
        const long long want = 148LL * 16 * 4;
        const long long head_blocks = p->hkv > 0 ? (p->hq / p->hkv + 15) / 16 : 1;
        long long per = (long long)p->s * p->b * p->hkv * head_blocks / want;
        c = 128;
        while (c * 2 <= per && c < 512) c *= 2;
    }
    if (c < 8) c = 8;
    *chunk = (int)c;
    *splits = p->s > 0 ? (int)((p->s + c - 1) / c) : 1;
}

__global__ void fill_kernel(float *dst, float value, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value;
}

}  // namespace

namespace dash {
cudaError_t launch_fill_f32(float *dst, float value, long long n, cudaStream_t stream, int *launches) {
    if (n <= 0) return cudaSuccess;
    fill_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(dst, value, n);
    *launches += 1;
    return cudaGetLastError();
}
}  // namespace dash

extern "C" {

const char *dash_attn_last_error(void) { return g_error.c_str(); }

uint64_t dash_attn_probe(int which) {
    if (which < 0 || which >= DASH_ATTN_PROBE_COUNT) return 0;
    if (which == DASH_ATTN_PROBE_TENSOR_MAP_ENCODES) return dash::sm100_tensor_map_encodes();
    return g_probe[which].load();
}

void dash_attn_force_generic(int on) { g_force_generic.store(on ? 1 : 0); }
void dash_attn_force_tensor(int on) { g_force_tensor.store(on ? 1 : 0); }

int dash_attn_device_status(int clear) {
    g_error.clear();
    unsigned int status = 0;
    cudaError_t e = dash::read_sm100_status(&status, clear != 0);
    if (e != cudaSuccess) return -cuda_fail("device_status", e);
    return (int)status;
}

int dash_attn_kernels_take(const dash_attn_params *p, const void *q, const void *k, const void *v, int backward) {
    g_error.clear();
    int rc = check_train(backward ? "attention_backward" : "attention", p);
    if (rc != DASH_ATTN_OK) return -rc;
    return train_path(p, q, k, v, backward);
}

size_t dash_attn_forward_workspace(const dash_attn_params *p) {
    if (!p || check_train("attention", p) != DASH_ATTN_OK || degenerate(p)) return 0;
    return dash::sm100_forward_workspace(p);
}

size_t dash_attn_backward_workspace(const dash_attn_params *p) {
    if (!p || check_train("attention_backward", p) != DASH_ATTN_OK || degenerate(p)) return 0;
    // delta [B,Tq,Hq] f32 for either path, then whatever the tensor-core path adds.
    size_t delta = align256(sizeof(float) * (size_t)p->b * p->tq * p->hq);
    return delta + dash::sm100_backward_workspace(p);
}

size_t dash_attn_decode_workspace(const dash_attn_decode_params *p) {
    if (!p || check_decode(p) != DASH_ATTN_OK) return 0;
    if ((int64_t)p->b * p->hq * p->d == 0 || p->s == 0) return 0;
    int chunk, splits;
    decode_plan(p, &chunk, &splits);
    size_t part_o = align256(sizeof(float) * (size_t)p->b * p->hq * splits * p->d);
    size_t part_lse = align256(sizeof(float) * (size_t)p->b * p->hq * splits);
    return part_o + part_lse;
}

int dash_attn_forward(const dash_attn_params *p, const void *q, const void *k, const void *v, void *o,
                      float *lse, void *workspace, size_t workspace_bytes, dash_attn_stream_t stream_) {
    const char *op = "attention";
    g_error.clear();
    int rc = check_train(op, p);
    if (rc != DASH_ATTN_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int launches = 0;
    if (degenerate(p)) {
        // No key at all: zeros, and a log-sum-exp of -inf (reference.rs:316-327).
        size_t ob = (size_t)p->b * p->tq * p->hq * p->d * elem_bytes(p->dtype);
        if (ob) {
            if (!o) return fail(DASH_ATTN_INVALID, "%s: the output is null", op);
            cudaError_t e = cudaMemsetAsync(o, 0, ob, stream);
            if (e != cudaSuccess) return cuda_fail(op, e);
        }
        long long n = (long long)p->b * p->tq * p->hq;
        if (n) {
            if (!lse) return fail(DASH_ATTN_INVALID, "%s: the log-sum-exp is null", op);
            cudaError_t e = dash::launch_fill_f32(lse, -INFINITY, n, stream, &launches);
            if (e != cudaSuccess) return cuda_fail(op, e);
        }
        g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
        return DASH_ATTN_OK;
    }
    if (!q || !k || !v || !o || !lse) return fail(DASH_ATTN_INVALID, "%s: a tensor pointer is null", op);
    size_t need = dash_attn_forward_workspace(p);
    if ((rc = check_workspace(op, workspace, workspace_bytes, need)) != DASH_ATTN_OK) return rc;

    dash::TrainArgs a = train_args(p, q, k, v);
    a.out = o;
    a.lse = lse;
    cudaError_t e;
    if (train_path(p, q, k, v, 0) == 1 && aligned16({o})) {
        e = dash::sm100_forward(p, a, workspace, stream, &launches, g_error);
        if (e == cudaSuccess && !g_error.empty()) return DASH_ATTN_CUDA;
        g_probe[DASH_ATTN_PROBE_TENSOR_CORE_RUNS] += 1;
    } else {
        e = dash::launch_generic_forward(p->dtype, a, stream, &launches);
        g_probe[DASH_ATTN_PROBE_GENERIC_RUNS] += 1;
    }
    g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
    if (e != cudaSuccess) return cuda_fail(op, e);
    return DASH_ATTN_OK;
}

int dash_attn_backward(const dash_attn_params *p, const void *q, const void *k, const void *v, const void *o,
                       const float *lse, const void *dout, void *dq, void *dk, void *dv, void *workspace,
                       size_t workspace_bytes, dash_attn_stream_t stream_) {
    const char *op = "attention_backward";
    g_error.clear();
    int rc = check_train(op, p);
    if (rc != DASH_ATTN_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int launches = 0;
    const size_t eb = elem_bytes(p->dtype);
    if (degenerate(p)) {  // reference.rs:386-395: zeros
        size_t qb = (size_t)p->b * p->tq * p->hq * p->d * eb, kb = (size_t)p->b * p->tk * p->hkv * p->d * eb;
        cudaError_t e = cudaSuccess;
        if (qb && dq) e = cudaMemsetAsync(dq, 0, qb, stream);
        if (e == cudaSuccess && kb && dk) e = cudaMemsetAsync(dk, 0, kb, stream);
        if (e == cudaSuccess && kb && dv) e = cudaMemsetAsync(dv, 0, kb, stream);
        if (e != cudaSuccess) return cuda_fail(op, e);
        return DASH_ATTN_OK;
    }
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv)
        return fail(DASH_ATTN_INVALID, "%s: a tensor pointer is null", op);
    size_t need = dash_attn_backward_workspace(p);
    if ((rc = check_workspace(op, workspace, workspace_bytes, need)) != DASH_ATTN_OK) return rc;

    dash::TrainArgs a = train_args(p, q, k, v);
    a.o = view(o, p->o_stride);
    a.dout = view(dout, p->do_stride);
    a.lse = const_cast<float *>(lse);
    a.delta = static_cast<float *>(workspace);
    a.dq = dq; a.dk = dk; a.dv = dv;
    void *extra = static_cast<char *>(workspace) + align256(sizeof(float) * (size_t)p->b * p->tq * p->hq);
    cudaError_t e;
    if (train_path(p, q, k, v, 1) == 1 && aligned16({dout, dq, dk, dv})) {
        bool atomic = false;
        e = dash::sm100_backward(p, a, extra, stream, &launches, &atomic, g_error);
        if (e == cudaSuccess && !g_error.empty()) return DASH_ATTN_CUDA;
        g_probe[DASH_ATTN_PROBE_TENSOR_CORE_RUNS] += 1;
        if (atomic) g_probe[DASH_ATTN_PROBE_ATOMIC_RUNS] += 1;
    } else {
        e = dash::launch_generic_backward(p->dtype, a, stream, &launches);
        g_probe[DASH_ATTN_PROBE_GENERIC_RUNS] += 1;
    }
    g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
    g_probe[DASH_ATTN_PROBE_BACKWARD_RUNS] += 1;
    if (e != cudaSuccess) return cuda_fail(op, e);
    return DASH_ATTN_OK;
}

// The decoding step, with (k_new, v_new set) or without the new row written into the cache first.
// The split pass's partial outputs go to the caller's workspace, or (`library_array`) to the array the
// library itself holds on the device.
static int decode_impl(const char *op, const dash_attn_decode_params *p, const void *q, const void *k_new, const void *v_new,
                       const void *k_cache, const void *v_cache, void *out, void *workspace, size_t workspace_bytes,
                       dash_attn_stream_t stream_, bool library_array = false) {
    g_error.clear();
    int rc = check_decode(p, op);
    if (rc != DASH_ATTN_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const size_t eb = elem_bytes(p->dtype);
    size_t ob = (size_t)p->b * p->hq * p->d * eb;
    if (ob == 0) return DASH_ATTN_OK;
    if (!out) return fail(DASH_ATTN_INVALID, "%s: the output is null", op);
    if (p->s == 0) {  // a sequence holding no key gets zeros
        cudaError_t e = cudaMemsetAsync(out, 0, ob, stream);
        return e == cudaSuccess ? DASH_ATTN_OK : cuda_fail(op, e);
    }
    if (!q || !k_cache || !v_cache) return fail(DASH_ATTN_INVALID, "%s: a tensor pointer is null", op);

    dash::DecodeArgs a{};
    decode_plan(p, &a.chunk, &a.splits);
    if (library_array) {
        // Fewer, longer splits until the partials fit the library's array.
        const size_t capacity = dash::decode_static_capacity_floats();
        const size_t per_split = (size_t)p->b * p->hq * ((size_t)p->d + 1) + 64;
        if (per_split > capacity)
            return fail(DASH_ATTN_UNSUPPORTED,
                        "%s: B * Hq * (D + 1) = %zu floats of partial output exceed the library's %zu-float (16 MiB) "
                        "scratch; use dash_attn_decode with a workspace", op, per_split - 64, capacity);
        while ((size_t)a.splits * per_split > capacity) {
            a.chunk *= 2;
            a.splits = (p->s + a.chunk - 1) / a.chunk;
        }
        float *scratch = nullptr;
        cudaError_t e = dash::decode_static_scratch(&scratch);
        if (e != cudaSuccess) return cuda_fail(op, e);
        a.part_o = scratch;
        a.part_lse = scratch + (((size_t)p->b * p->hq * a.splits * p->d + 63) & ~size_t(63));
    } else {
        size_t need = dash_attn_decode_workspace(p);
        if ((rc = check_workspace(op, workspace, workspace_bytes, need)) != DASH_ATTN_OK) return rc;
        a.part_o = static_cast<float *>(workspace);
        a.part_lse = reinterpret_cast<float *>(static_cast<char *>(workspace) +
                                               align256(sizeof(float) * (size_t)p->b * p->hq * a.splits * p->d));
    }
    a.b = p->b; a.s = p->s; a.hq = p->hq; a.hkv = p->hkv; a.d = p->d;
    a.scale = scale_for(p->has_scale, p->scale, p->d);
    a.q = q;
    a.q_sb = p->q_stride[0]; a.q_sh = p->q_stride[1]; a.q_sd = p->q_stride[2];
    a.k = view(k_cache, p->k_stride);
    a.v = view(v_cache, p->v_stride);
    a.lengths = p->lengths;
    a.len_bytes = p->lengths_elem_bytes;
    a.k_new = k_new;
    a.v_new = v_new;
    // The window's left side binds only within S + 1 positions (reference.rs:445).
    int64_t none = (int64_t)p->s + 1;
    a.left = (int)((p->has_window && p->window_left >= 0 && p->window_left < none) ? p->window_left : none);
    a.out = out;
    bool vec = (p->d == 64 || p->d == 128 || p->d == 256) && vector_readable(q, p->q_stride, 3, eb) &&
               vector_readable(k_cache, p->k_stride, 4, eb) && vector_readable(v_cache, p->v_stride, 4, eb) &&
               (!k_new || (reinterpret_cast<uintptr_t>(k_new) % 16 == 0 && reinterpret_cast<uintptr_t>(v_new) % 16 == 0));
    int launches = 0;
    cudaError_t e = dash::launch_decode(p->dtype, a, vec, stream, &launches);
    g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
    g_probe[DASH_ATTN_PROBE_GENERIC_RUNS] += 1;
    if (e != cudaSuccess) return cuda_fail(op, e);
    return DASH_ATTN_OK;
}

int dash_attn_decode(const dash_attn_decode_params *p, const void *q, const void *k_cache, const void *v_cache,
                     void *out, void *workspace, size_t workspace_bytes, dash_attn_stream_t stream_) {
    return decode_impl("attention_decode", p, q, nullptr, nullptr, k_cache, v_cache, out, workspace, workspace_bytes, stream_);
}

int dash_attn_decode_append(const dash_attn_decode_params *p, const void *q, const void *k_new, const void *v_new,
                            void *k_cache, void *v_cache, void *out, void *workspace, size_t workspace_bytes,
                            dash_attn_stream_t stream_) {
    const char *op = "attention_decode_append";
    g_error.clear();
    int rc = check_decode(p, op);
    if (rc != DASH_ATTN_OK) return rc;
    if (!p->lengths) return fail(DASH_ATTN_INVALID, "%s: the lengths are needed: they say where each sequence's new row goes", op);
    if ((size_t)p->b * p->hkv * p->d != 0 && p->s != 0 && (!k_new || !v_new))
        return fail(DASH_ATTN_INVALID, "%s: a new row is null", op);
    return decode_impl(op, p, q, k_new, v_new, k_cache, v_cache, out, workspace, workspace_bytes, stream_);
}

// The checks of Rope::new and Rope::check_features (crates/dash-mag/src/rope.rs:27-32, 76-91).
static int check_rope(const char *op, const dash_rope_tables *r, int d) {
    if (!r) return fail(DASH_ATTN_INVALID, "%s: null rotation tables", op);
    if (r->dtype != DASH_ATTN_F32 && r->dtype != DASH_ATTN_BF16 && r->dtype != DASH_ATTN_F16)
        return fail(DASH_ATTN_INVALID, "Rope: dtype code %d is not floating", r->dtype);
    if (r->dim <= 0 || r->dim % 2 != 0) return fail(DASH_ATTN_INVALID, "Rope: %d features; an even number is rotated", r->dim);
    if (d < r->dim) return fail(DASH_ATTN_INVALID, "Rope: %d features to rotate, of %d", r->dim, d);
    if (r->len < 0) return fail(DASH_ATTN_INVALID, "Rope: %lld positions", (long long)r->len);
    if (r->len > 0 && (!r->cos || !r->sin)) return fail(DASH_ATTN_INVALID, "%s: a rotation table is null", op);
    return DASH_ATTN_OK;
}

int dash_rope_apply(const dash_rope_tables *r, const dash_rope_params *p, const void *x_a, void *out_a, const void *x_b,
                    void *out_b, dash_attn_stream_t stream_) {
    const char *op = "rope_apply";
    g_error.clear();
    if (!p) return fail(DASH_ATTN_INVALID, "%s: null parameters", op);
    int rc = check_rope(op, r, p->d);
    if (rc != DASH_ATTN_OK) return rc;
    if (p->tokens < 0 || p->heads_a < 0 || p->heads_b < 0)
        return fail(DASH_ATTN_INVALID, "%s: no dimension may be negative", op);
    if (p->positions && p->positions_elem_bytes != 4 && p->positions_elem_bytes != 8)
        return fail(DASH_ATTN_INVALID, "Rope: positions of %d bytes; i32 or i64", p->positions_elem_bytes);
    if (!p->positions && p->cu_seqlens && (p->index_elem_bytes != 4 && p->index_elem_bytes != 8))
        return fail(DASH_ATTN_INVALID, "Rope: offsets of %d bytes; i32 or i64", p->index_elem_bytes);
    if (!p->positions && p->cu_seqlens && p->cu_seqlens_len < 1)
        return fail(DASH_ATTN_INVALID, "Rope: the offsets hold at least the first 0");
    const int64_t work = p->tokens * ((int64_t)p->heads_a + p->heads_b) * p->d;
    if (!p->positions && !p->cu_seqlens && work != 0) {
        // apply_range's refusal (:111-117): T positions, all inside the tables.
        const int64_t t = p->period > 0 ? (p->period < p->tokens ? p->period : p->tokens) : 1;
        if (p->start < 0 || p->period < 0 || (p->period > 0 && p->tokens % p->period != 0) || p->start + t > r->len)
            return fail(DASH_ATTN_INVALID, "Rope: positions %lld..%lld of %lld for %lld tokens", (long long)p->start,
                        (long long)(p->start + t), (long long)r->len, (long long)p->tokens);
    }
    if (work == 0) return DASH_ATTN_OK;
    if ((p->heads_a && (!x_a || !out_a)) || (p->heads_b && (!x_b || !out_b)))
        return fail(DASH_ATTN_INVALID, "%s: a tensor pointer is null", op);
    dash::RopeArgs a{};
    a.a = dash::RopeTensor{x_a, out_a, p->heads_a, p->stride_a[0], p->stride_a[1], p->stride_a[0], p->stride_a[1]};
    a.b = dash::RopeTensor{x_b, out_b, p->heads_b, p->stride_b[0], p->stride_b[1], p->stride_b[0], p->stride_b[1]};
    a.tokens = p->tokens; a.d = p->d; a.dim = r->dim;
    a.cos = r->cos; a.sin = r->sin; a.len = r->len;
    a.inverse = p->inverse ? 1 : 0;
    a.positions = p->positions; a.pos_bytes = p->positions_elem_bytes;
    if (!p->positions && p->cu_seqlens) {
        a.cu = p->cu_seqlens; a.cu_bytes = p->index_elem_bytes; a.sequences = p->cu_seqlens_len - 1;
    }
    a.start = p->start; a.period = p->period;
    int launches = 0;
    cudaError_t e = dash::launch_rope(r->dtype, a, reinterpret_cast<cudaStream_t>(stream_), &launches);
    g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
    if (e != cudaSuccess) return cuda_fail(op, e);
    return DASH_ATTN_OK;
}

// The rotated query and key sit behind the decoding step's own scratch.
static size_t rope_scratch_offset(const dash_attn_decode_params *p) { return align256(dash_attn_decode_workspace(p)); }

size_t dash_attn_decode_append_rope_workspace(const dash_attn_decode_params *p) {
    if (!p || p->b < 0 || p->hq < 0 || p->hkv < 0 || p->d < 0) return 0;
    const size_t eb = elem_bytes(p->dtype);
    return rope_scratch_offset(p) + align256((size_t)p->b * p->hq * p->d * eb) + align256((size_t)p->b * p->hkv * p->d * eb);
}

int dash_attn_decode_append_rope(const dash_attn_decode_params *p, const dash_rope_tables *r, const void *positions,
                                 int32_t positions_elem_bytes, const void *q, const void *k_new, const void *v_new,
                                 void *k_cache, void *v_cache, void *out, void *workspace, size_t workspace_bytes,
                                 dash_attn_stream_t stream_) {
    const char *op = "attention_decode_append_rope";
    g_error.clear();
    int rc = check_decode(p, op);
    if (rc != DASH_ATTN_OK) return rc;
    if ((rc = check_rope(op, r, p->d)) != DASH_ATTN_OK) return rc;
    if (r->dtype != p->dtype) return fail(DASH_ATTN_INVALID, "Rope: dtype code %d under a rotation of code %d", p->dtype, r->dtype);
    if (!p->lengths) return fail(DASH_ATTN_INVALID, "%s: the lengths are needed: they say where each sequence's new row goes", op);
    if (positions && positions_elem_bytes != 4 && positions_elem_bytes != 8)
        return fail(DASH_ATTN_INVALID, "Rope: positions of %d bytes; i32 or i64", positions_elem_bytes);
    const size_t eb = elem_bytes(p->dtype);
    if ((size_t)p->b * p->hq * p->d == 0 || p->s == 0)   // nothing to rotate for, or no cache to append to
        return decode_impl(op, p, q, k_new, v_new, k_cache, v_cache, out, workspace, workspace_bytes, stream_);
    if (!q || !k_new || !v_new) return fail(DASH_ATTN_INVALID, "%s: a tensor pointer is null", op);
    if (p->q_stride[2] != 1) return fail(DASH_ATTN_UNSUPPORTED, "%s: the query's features must be contiguous", op);
    const size_t need = dash_attn_decode_append_rope_workspace(p);
    if ((rc = check_workspace(op, workspace, workspace_bytes, need)) != DASH_ATTN_OK) return rc;
    char *q_rot = static_cast<char *>(workspace) + rope_scratch_offset(p);
    char *k_rot = q_rot + align256((size_t)p->b * p->hq * p->d * eb);

    dash::RopeArgs a{};
    // The rotated rows are written contiguous, whatever the query's strides.
    a.a = dash::RopeTensor{q, q_rot, p->hq, p->q_stride[0], p->q_stride[1], (int64_t)p->hq * p->d, (int64_t)p->d};
    a.b = dash::RopeTensor{k_new, k_rot, p->hkv, (int64_t)p->hkv * p->d, (int64_t)p->d, (int64_t)p->hkv * p->d, (int64_t)p->d};
    a.tokens = p->b; a.d = p->d; a.dim = r->dim;
    a.cos = r->cos; a.sin = r->sin; a.len = r->len;
    a.positions = positions ? positions : p->lengths;
    a.pos_bytes = positions ? positions_elem_bytes : p->lengths_elem_bytes;
    int launches = 0;
    cudaError_t e = dash::launch_rope(p->dtype, a, reinterpret_cast<cudaStream_t>(stream_), &launches);
    g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
    if (e != cudaSuccess) return cuda_fail(op, e);
    dash_attn_decode_params rotated = *p;
    rotated.q_stride[0] = (int64_t)p->hq * p->d; rotated.q_stride[1] = p->d; rotated.q_stride[2] = 1;
    return decode_impl(op, &rotated, q_rot, k_rot, v_new, k_cache, v_cache, out, workspace, workspace_bytes, stream_);
}

// ------------------------------------------------------------------------------------------------
// Sampling (crates/dash-ops/src/sample.rs:300-342: the checks, same words)
// ------------------------------------------------------------------------------------------------
static int check_sample(const dash_sample_params *p, std::vector<uint32_t> *masked) {
    const char *op = "sample";
    if (!p) return fail(DASH_ATTN_INVALID, "%s: null parameters", op);
    if (p->dtype != DASH_ATTN_F32 && p->dtype != DASH_ATTN_BF16 && p->dtype != DASH_ATTN_F16)
        return fail(DASH_ATTN_INVALID, "%s: logits must be f32, bf16 or f16, got code %d", op, p->dtype);
    if (p->b < 0 || p->v < 0) return fail(DASH_ATTN_INVALID, "%s: logits must be [B, V], got [%d, %d]", op, p->b, p->v);
    if (p->v == 0) return fail(DASH_ATTN_INVALID, "%s: the vocabulary is empty", op);
    // The top-p search sums 14-bit pieces of the weights in 32-bit words, a thirty-second of a row to a word.
    if (p->v > (1 << 22)) return fail(DASH_ATTN_UNSUPPORTED, "%s: a vocabulary of %d tokens; up to 4194304 are taken", op, p->v);
    if (!(std::isfinite(p->temperature) && p->temperature >= 0.f))
        return fail(DASH_ATTN_INVALID, "%s: the temperature must be finite and >= 0, got %g", op, (double)p->temperature);
    if (!(p->top_p >= 0.f && p->top_p <= 1.f))
        return fail(DASH_ATTN_INVALID, "%s: top_p must be within 0..=1, got %g", op, (double)p->top_p);
    if (p->top_k < 0) return fail(DASH_ATTN_INVALID, "%s: top_k must not be negative", op);
    if (p->masked_len < 0 || (p->masked_len > 0 && !p->masked)) return fail(DASH_ATTN_INVALID, "%s: the masked ids are null", op);
    if (p->token_elem_bytes != 4 && p->token_elem_bytes != 8)
        return fail(DASH_ATTN_INVALID, "%s: tokens of %d bytes; i32 or i64", op, p->token_elem_bytes);
    masked->assign(p->masked, p->masked + p->masked_len);
    std::sort(masked->begin(), masked->end());
    masked->erase(std::unique(masked->begin(), masked->end()), masked->end());
    if (!masked->empty()) {
        if (masked->back() >= (uint32_t)p->v)
            return fail(DASH_ATTN_INVALID, "%s: masked token id %u is outside the vocabulary of %d", op, masked->back(), p->v);
        if (masked->size() >= (size_t)p->v) return fail(DASH_ATTN_INVALID, "%s: every token of the vocabulary is masked", op);
    }
    return DASH_ATTN_OK;
}

size_t dash_sample_workspace(const dash_sample_params *p) {
    if (!p || p->masked_len <= 0 || p->v <= 0) return 0;
    return align256(sizeof(uint32_t) * (((size_t)p->v + 31) / 32));
}

int dash_sample(const dash_sample_params *p, const void *logits, void *tokens, float *logprob, float *tempered_logprob,
                float *sampling_logprob, void *workspace, size_t workspace_bytes, dash_attn_stream_t stream_) {
    const char *op = "sample";
    g_error.clear();
    std::vector<uint32_t> masked;
    int rc = check_sample(p, &masked);
    if (rc != DASH_ATTN_OK) return rc;
    if (p->b == 0) return DASH_ATTN_OK;
    if (!logits || !tokens || !logprob || !tempered_logprob || !sampling_logprob)
        return fail(DASH_ATTN_INVALID, "%s: a tensor pointer is null", op);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if ((rc = check_workspace(op, workspace, workspace_bytes, dash_sample_workspace(p))) != DASH_ATTN_OK) return rc;
    dash::SampleArgs a{};
    a.logits = logits; a.b = p->b; a.v = p->v; a.stride = p->row_stride;
    a.vec = reinterpret_cast<uintptr_t>(logits) % 16 == 0 && (p->b == 1 || (p->row_stride * (int64_t)elem_bytes(p->dtype)) % 16 == 0);
    a.greedy = p->temperature == 0.f;
    a.tau = a.greedy ? 1.f : std::min(1.0f / p->temperature, 3.4028234663852886e38f);   // Cuts::inverse_temperature (:89-91)
    const size_t unmasked = (size_t)p->v - masked.size();
    a.top_k = (p->top_k > 0 && (uint64_t)p->top_k < unmasked) ? (int)p->top_k : 0;        // Cuts::top_k_cut (:93-95)
    a.has_p = p->top_p < 1.f;                                                              // Cuts::top_p_cut (:97-99)
    a.p = p->top_p;
    a.key0 = (uint32_t)p->seed; a.key1 = (uint32_t)(p->seed >> 32);
    a.off_lo = (uint32_t)p->offset; a.off_hi = (uint32_t)(p->offset >> 32);
    if (!masked.empty()) {
        std::vector<uint32_t> bits(((size_t)p->v + 31) / 32, 0u);
        for (uint32_t id : masked) bits[id >> 5] |= 1u << (id & 31);
        // From pageable memory: the copy is staged before the call returns, so `bits` may go.
        cudaError_t e = cudaMemcpyAsync(workspace, bits.data(), bits.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(op, e);
        a.masked_bits = static_cast<const uint32_t *>(workspace);
    }
    a.tokens = tokens; a.token_bytes = p->token_elem_bytes;
    a.logprob = logprob; a.tempered = tempered_logprob; a.sampling = sampling_logprob;
    int launches = 0;
    cudaError_t e = dash::launch_sample(p->dtype, a, stream, &launches);
    g_probe[DASH_ATTN_PROBE_KERNEL_LAUNCHES] += launches;
    if (e != cudaSuccess) return cuda_fail(op, e);
    return DASH_ATTN_OK;
}

int dash_attn_decode_static(const dash_attn_decode_params *p, const void *q, const void *k_cache,
                            const void *v_cache, void *out, dash_attn_stream_t stream_) {
    return decode_impl("attention_decode (static scratch)", p, q, nullptr, nullptr, k_cache, v_cache, out, nullptr, 0,
                       stream_, true);
}

}  // extern "C"
