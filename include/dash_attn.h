/*
 * dash_attn.h - C ABI of the B200 (sm_100a) attention library.
 *
 * Scaled dot-product attention with grouped key-value heads in its three forms: the packed /
 * masked training forward with saved log-sum-exp, its written-out backward, and the decoding step
 * against a key-value cache, as crates/dash-contract/src/attention.rs defines them.  These entry
 * points are what a Rust `extern "C"` block would bind to sit behind dash-ops' backend-extension
 * trait `AttentionBackend` (crates/dash-ops/src/attention.rs:289-352).
 *
 * Conventions (crates/dash-contract/src/lib.rs, crates/dash-ops/src/attention.rs:85-93):
 *   - every pointer except the parameter structs is DEVICE memory owned by the caller; the library
 *     allocates nothing; scratch comes in through `workspace` (dash_attn_decode_static, which uses
 *     an array of the library's own, is the one exception and says so);
 *   - work is enqueued on `stream` and the call returns without synchronising;
 *   - layouts: q, o, do, dq [B,Tq,Hq,D]; k, v, dk, dv [B,Tk,Hkv,D]; lse [B,Tq,Hq] f32; decode
 *     q / out [B,Hq,D], cache [B,S,Hkv,D], lengths [B];
 *   - inputs may have any strides (given in ELEMENTS, order batch, time, head, dim); outputs are
 *     written contiguous.  The tensor-core paths read an input in place when its last stride is 1,
 *     its other strides are multiples of 8 elements (16-bit dtypes) and its base is 16-byte
 *     aligned - the reference's own rule (crates/dash-ops/src/attention/cube.rs:428-461) - and any
 *     other input is read, also in place, by the generic kernels: no input is ever copied;
 *   - every function returning `int` gives DASH_ATTN_OK or an error code, and then
 *     dash_attn_last_error() names the operation and the argument, with the reference's own
 *     wording where it panics (crates/dash-ops/src/attention.rs:551-638).  Nothing is launched
 *     when a call is refused.  There is no CPU fallback.
 *   - re-entrant.  What the library does keep between calls, all of it process-wide: atomic counters
 *     (dash_attn_probe), the test switches (dash_attn_force_*), a thread-local error string, a small
 *     cache of TMA tensor maps keyed on address and geometry (never on contents), one sticky status
 *     word per device that a bounded wait inside a tensor-core kernel raises when it runs out
 *     (dash_attn_device_status), and the 16 MiB device array of dash_attn_decode_static.
 */
#ifndef DASH_ATTN_H
#define DASH_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling the CUDA headers into the caller. */
typedef struct CUstream_st *dash_attn_stream_t;

/* crates/dash-contract/src/lib.rs:107-115 (DType): the dtype q, k and v share. */
enum { DASH_ATTN_F32 = 0, DASH_ATTN_BF16 = 1, DASH_ATTN_F16 = 2 };

/* crates/dash-contract/src/attention.rs:162-183 (AttentionMask). */
enum { DASH_ATTN_MASK_NONE = 0, DASH_ATTN_MASK_KEY_PADDING = 1, DASH_ATTN_MASK_PACKED = 2 };

enum {
    DASH_ATTN_OK = 0,
    DASH_ATTN_INVALID = 1,     /* the shapes do not fit together: where dash-ops panics */
    DASH_ATTN_UNSUPPORTED = 2, /* a well-formed call this library does not take (conformance's Unsupported) */
    DASH_ATTN_WORKSPACE = 3,   /* workspace missing, misaligned or smaller than *_workspace() says */
    DASH_ATTN_CUDA = 4         /* a CUDA runtime or driver call failed; the message carries its text */
};

/* A window side with no bound (`usize::MAX` in crates/dash-contract/src/attention.rs:71-80). */
#define DASH_ATTN_UNBOUNDED ((int64_t)-1)

/*
 * One training call: shapes, strides, mask and options as plain data.
 * Mirrors the arguments of AttentionBackend::attention_forward / attention_backward
 * (crates/dash-ops/src/attention.rs:307-337) with AttentionOptions
 * (crates/dash-contract/src/attention.rs:88-103) flattened in.
 */
typedef struct dash_attn_params {
    int32_t dtype;           /* DASH_ATTN_F32 / BF16 / F16 */
    int32_t b, tq, tk, hq, hkv, d;
    int32_t v_tk, v_hkv, v_d; /* value's own [Tk, Hkv, D]: "key and value must have one shape" */
    int32_t k_b, k_d;        /* key's own batch size and head dimension, checked against q's */
    int64_t q_stride[4], k_stride[4], v_stride[4]; /* elements: batch, time, head, dim */
    int64_t o_stride[4], do_stride[4];             /* backward's inputs o and do (ignored by forward) */

    int32_t mask_kind;       /* DASH_ATTN_MASK_* */
    const void *key_padding; /* [B,Tk], non-zero = key left out */
    int32_t key_padding_elem_bytes; /* 1 (bool / u8) or 4 (i32) */
    int32_t key_padding_shape[2];   /* must equal [B, Tk] */
    int64_t key_padding_stride[2];  /* elements */
    const void *cu_seqlens_q; /* [S+1] */
    const void *cu_seqlens_k; /* [S+1] */
    int32_t cu_seqlens_q_len, cu_seqlens_k_len; /* S+1 each, one S */
    int32_t index_elem_bytes; /* 4 (i32) or 8 (i64): the offsets' integer type */

    int32_t causal;          /* 0 / 1 */
    int32_t has_window;      /* 0: no window; 1: window_left / window_right apply */
    int64_t window_left, window_right; /* DASH_ATTN_UNBOUNDED (any negative) = no bound */
    int32_t has_scale;       /* 0: 1/sqrt(D), as (1.0 / (d as f64).sqrt()) as f32 */
    float scale;
    int32_t deterministic;   /* 1: the query gradient sums in a fixed order (default) */
} dash_attn_params;

/*
 * One decoding step.  Mirrors AttentionBackend::attention_decode
 * (crates/dash-ops/src/attention.rs:343-351) and check_decode_shapes (:617-638).  Of the options
 * only the scale and the window's left side apply.
 */
typedef struct dash_attn_decode_params {
    int32_t dtype;
    int32_t b, s, hq, hkv, d;
    int32_t k_b, k_d, v_b, v_s, v_hkv, v_d; /* the caches' own dims, checked against each other */
    int64_t q_stride[3];                    /* elements: batch, head, dim */
    int64_t k_stride[4], v_stride[4];       /* elements: batch, time, head, dim */
    const void *lengths;       /* [B] or NULL: every sequence holds all S keys */
    int32_t lengths_len;       /* must equal B when lengths != NULL */
    int32_t lengths_elem_bytes; /* 4 or 8 */
    int32_t has_window;
    int64_t window_left;       /* DASH_ATTN_UNBOUNDED = no bound */
    int32_t has_scale;
    float scale;
} dash_attn_decode_params;

/* Bytes of device scratch each call needs (0 is possible).  256-byte aligned workspace. */
size_t dash_attn_forward_workspace(const dash_attn_params *p);
size_t dash_attn_backward_workspace(const dash_attn_params *p);
size_t dash_attn_decode_workspace(const dash_attn_decode_params *p);

/*
 * Replaces AttentionBackend::attention_forward (crates/dash-ops/src/attention.rs:307-315; the
 * reference's launch glue is crates/dash-ops/src/attention/cube.rs:562-684).
 * o [B,Tq,Hq,D] in q's dtype and lse [B,Tq,Hq] f32, both contiguous.  A query that sees no key
 * gives zeros and -inf.
 */
int dash_attn_forward(const dash_attn_params *p, const void *q, const void *k, const void *v,
                      void *o, float *lse, void *workspace, size_t workspace_bytes,
                      dash_attn_stream_t stream);

/*
 * Replaces AttentionBackend::attention_backward (crates/dash-ops/src/attention.rs:326-337; glue
 * crates/dash-ops/src/attention/cube.rs:850-1120).  dq, dk, dv contiguous, each in its input's
 * dtype.  lse is the forward's, contiguous [B,Tq,Hq] f32.
 */
int dash_attn_backward(const dash_attn_params *p, const void *q, const void *k, const void *v,
                       const void *o, const float *lse, const void *dout, void *dq, void *dk,
                       void *dv, void *workspace, size_t workspace_bytes,
                       dash_attn_stream_t stream);

/*
 * Replaces AttentionBackend::attention_decode (crates/dash-ops/src/attention.rs:343-351; glue
 * crates/dash-ops/src/attention/cube.rs:1126-1216).  out [B,Hq,D] contiguous in q's dtype; zeros
 * for a sequence that holds no key.
 */
int dash_attn_decode(const dash_attn_decode_params *p, const void *q, const void *k_cache,
                     const void *v_cache, void *out, void *workspace, size_t workspace_bytes,
                     dash_attn_stream_t stream);

/*
 * The decoding step that first appends: the step's new key and value rows k_new, v_new [B,Hkv,D]
 * (contiguous, the cache's dtype) are written to position lengths[b] of sequence b's cache, and the
 * query sees the keys up to and including that row - what the reference's caller gets from
 * Tensor::put_along_axis_owned on the cache (crates/dash-mag/src/tensor.rs:732-744, the arm's
 * crates/dash-mag/src/arm/mod.rs:188-199) followed by attention_decode with lengths + 1, in the
 * launches of the decoding step alone: the warp that owns the chunk holding the position takes
 * the row from k_new / v_new and stores it into the cache on its way.  p->lengths are the lengths
 * BEFORE the step and are required (they are not changed: the caller advances them).  A sequence
 * whose cache is full (lengths[b] >= S) gets no row written and sees all S keys.
 */
int dash_attn_decode_append(const dash_attn_decode_params *p, const void *q, const void *k_new,
                            const void *v_new, void *k_cache, void *v_cache, void *out,
                            void *workspace, size_t workspace_bytes, dash_attn_stream_t stream);

/*
 * Rotary position embedding from tables, transformers' form `x cos + rotate_half(x) sin` over the
 * first `dim` features of every head (crates/dash-mag/src/rope.rs:11-24: Rope's cosines and sines
 * [len, dim], each angle rounded once to f32 and once to `dtype`; the caller builds them as
 * Rope::new does, :43-56).  The reference rotates with whole-tensor operations of the tensors'
 * dtype (Rope::rotate, :94-107): each product and the sum rounds once to that dtype, and so does
 * this library, bit for bit.
 */
typedef struct dash_rope_tables {
    int32_t dtype;         /* of cos and sin, and of every tensor rotated with them (:76-83) */
    int32_t dim;           /* features rotated: even, not 0, at most D (:27-29, :84-91) */
    int64_t len;           /* positions 0..len the tables hold */
    const void *cos, *sin; /* [len, dim] contiguous, device memory */
} dash_rope_tables;

/*
 * One rotation of up to two tensors [tokens, heads, D] that share their tokens' positions (a
 * layer's query and key: one launch instead of two).  The position of token n is, first rule that
 * applies: positions[n]; start + n - cu_seqlens[s] for the packed sequence s that holds n (tokens
 * of no sequence pass through unchanged); start + n % period - Rope::apply_range on [B,T,H,D] is
 * tokens = B * T, period = T, start = positions.start (:110-135), Rope::apply_at on [B,H,D] is
 * tokens = B with positions [B] (:141-165).  A range past the tables is refused as the reference
 * refuses it; positions read on the device cannot be, and one outside the tables gives NaN in the
 * rotated features instead of the reference's "garbage" (:137-140) - nothing is read out of bounds.
 */
typedef struct dash_rope_params {
    int64_t tokens;
    int32_t d;
    int32_t heads_a, heads_b;           /* heads_b = 0: one tensor */
    int64_t stride_a[2], stride_b[2];   /* elements: token, head; the features are contiguous */
    int32_t inverse;                    /* 1: the transpose of the rotation, which the gradient goes through */
    const void *positions;              /* [tokens] or NULL */
    int32_t positions_elem_bytes;       /* 4 or 8 */
    const void *cu_seqlens;             /* [cu_seqlens_len] or NULL */
    int32_t cu_seqlens_len;
    int32_t index_elem_bytes;           /* 4 or 8 */
    int64_t start, period;
} dash_rope_params;

/* out_a / out_b have x_a / x_b's strides and may be x_a / x_b themselves (in place). */
int dash_rope_apply(const dash_rope_tables *rope, const dash_rope_params *p, const void *x_a, void *out_a,
                    const void *x_b, void *out_b, dash_attn_stream_t stream);

/*
 * The appending decoding step with the rotation in front: q [B,Hq,D] and k_new [B,Hkv,D] are
 * rotated at each sequence's position lengths[b] (`positions` [B], when not NULL, gives other
 * positions, e.g. for a cache that slides), then the step is dash_attn_decode_append with the
 * rotated query and key - the reference's caller does Rope::apply_at on the query, Rope::apply_at
 * on the key, two put_along_axis_owned and attention_decode, five dispatches, where this is one
 * call that launches the rotation (both tensors at once, into the workspace) and the decoding
 * step's own kernels.  The result is bit-identical to dash_rope_apply followed by
 * dash_attn_decode_append.  q's last stride must be 1.
 */
size_t dash_attn_decode_append_rope_workspace(const dash_attn_decode_params *p);
int dash_attn_decode_append_rope(const dash_attn_decode_params *p, const dash_rope_tables *rope,
                                 const void *positions, int32_t positions_elem_bytes, const void *q,
                                 const void *k_new, const void *v_new, void *k_cache, void *v_cache,
                                 void *out, void *workspace, size_t workspace_bytes,
                                 dash_attn_stream_t stream);

/*
 * Sampling the next token on the device, the step on the far side of the decoding loop: from the
 * logits [B, V] of one position per sequence, one token id per row with its log-probability under
 * the model's distribution, the model's at the temperature, and the one it was drawn from - the
 * definition of crates/dash-contract/src/sample.rs:1-96 (temperature, top-k, then top-p over what
 * top-k keeps, ties kept, masked ids taking part in nothing; greedy at temperature 0; Gumbel-max
 * over Philox4x32-10 words with the key (seed) and the counter (i / 4, row, offset)).  Mirrors
 * dash-ops' `sample` (crates/dash-ops/src/sample.rs) with SampleOptions
 * (crates/dash-contract/src/sample.rs:98-150) flattened in, and refuses what it refuses
 * (crates/dash-ops/src/sample.rs:300-342), in its words.  The same seed, offset and logits give
 * the same bits on every run.  Not differentiable.
 */
typedef struct dash_sample_params {
    int32_t dtype;            /* of the logits: DASH_ATTN_F32 / BF16 / F16 */
    int32_t b, v;             /* rows, vocabulary */
    int64_t row_stride;       /* elements between rows; the vocabulary is contiguous */
    float temperature;        /* >= 0, finite; 0 = greedy */
    int64_t top_k;            /* 0 keeps all */
    float top_p;              /* 0..=1; 1 keeps all */
    uint64_t seed, offset;    /* the generator's key and counter: advance the offset every step */
    const uint32_t *masked;   /* HOST memory (they are options, a Vec<u32> in the reference): ids in any order, each < V */
    int32_t masked_len;
    int32_t token_elem_bytes; /* 4 (i32) or 8 (i64): the tokens' integer type */
} dash_sample_params;

/* Bytes of device scratch (the masked ids as a bit per token; 0 without any). */
size_t dash_sample_workspace(const dash_sample_params *p);
/* tokens [B] of token_elem_bytes; logprob, tempered_logprob, sampling_logprob [B] f32; all device memory. */
int dash_sample(const dash_sample_params *p, const void *logits, void *tokens, float *logprob,
                float *tempered_logprob, float *sampling_logprob, void *workspace,
                size_t workspace_bytes, dash_attn_stream_t stream);

/*
 * The decoding step for callers that cannot hand over a workspace.  It has no counterpart in the
 * reference, whose launch glue always allocates its partial outputs from Burn's memory pool.
 *
 * Who needs it: code that is given raw device pointers and nothing else - an FFI shim sitting
 * under a tensor runtime whose pool owns all device memory, a serving loop that must not allocate
 * once it is running - and so can neither call cudaMalloc nor ask anyone for scratch.  The split
 * pass's partial outputs live in a 16 MiB array inside the library (reserved on every GPU that
 * loads it, until the process exits), and this call allocates nothing, on the device or through
 * any library.  The result is dash_attn_decode's up to f32 rounding (the cache may be cut into
 * fewer, longer splits so that the partials fit).
 *
 * Limits: B * Hq * (D + 1) floats per split must fit the array at least once, i.e.
 * B * Hq * (D + 1) <= 4 Mi; larger calls return DASH_ATTN_UNSUPPORTED and say so.  All calls
 * share the one array: calls whose kernels may overlap on the GPU (different streams, or threads
 * without ordering between them) race on it - keep them on one stream.  The first call on each
 * device looks up the array's device address; make that call before starting any stream capture.
 */
int dash_attn_decode_static(const dash_attn_decode_params *p, const void *q, const void *k_cache,
                            const void *v_cache, void *out, dash_attn_stream_t stream);

/*
 * Which kernels a call would run: 0 = the generic f32-FMA kernels (any dtype, any D <= 256, any
 * strides), 1 = the tcgen05 tensor-core path, negative = refused (dash_attn_last_error() says
 * why).  `backward` selects the pass.  The analogue of dash-ops' `kernels_take`
 * (crates/dash-ops/src/attention.rs:814-821), for tests.
 */
int dash_attn_kernels_take(const dash_attn_params *p, const void *q, const void *k, const void *v,
                           int backward);

/*
 * Every wait inside the tensor-core kernels is bounded; one that runs out raises a sticky word on
 * the device instead of hanging, and later blocks and launches of those kernels then do nothing.
 * This reads that word (0 = healthy) and, with `clear` non-zero, resets it.  It synchronises with
 * the device, so it is for tests and for error paths, not for the hot loop.  Returns a negative
 * DASH_ATTN_* code if the word cannot be read.  The reference has no counterpart: its kernels
 * have no device-side waits.
 */
int dash_attn_device_status(int clear);

/* Thread-local text of the last refusal or failure on this thread ("" when none). */
const char *dash_attn_last_error(void);

/*
 * Process-wide counters, the analogue of dash-ops' `probe` module
 * (crates/dash-ops/src/attention.rs:158-221).
 */
enum {
    DASH_ATTN_PROBE_KERNEL_LAUNCHES = 0, /* kernels this library launched */
    DASH_ATTN_PROBE_BACKWARD_RUNS = 1,   /* calls of dash_attn_backward that launched */
    DASH_ATTN_PROBE_INPUT_COPIES = 2,    /* always 0: every input is read in place */
    DASH_ATTN_PROBE_ATOMIC_RUNS = 3,     /* backward passes that summed dq with atomics */
    DASH_ATTN_PROBE_TENSOR_CORE_RUNS = 4, /* calls that took the tcgen05 path */
    DASH_ATTN_PROBE_GENERIC_RUNS = 5,    /* calls that took the generic kernels */
    DASH_ATTN_PROBE_TENSOR_MAP_ENCODES = 6, /* TMA tensor maps encoded through the driver (repeated calls reuse theirs) */
    DASH_ATTN_PROBE_COUNT = 7
};
uint64_t dash_attn_probe(int which);

/* For tests: 0 = choose by the call (default), 1 = always the generic kernels. */
void dash_attn_force_generic(int on);
/*
 * For tests: 1 = the tensor-core kernels also take the calls they leave to the generic kernels by
 * SIZE alone (head dimension 64 or 256 with fewer than 128 queries or keys - a single partial
 * tile), so that the reference's small recorded cases can be run through them; every other
 * precondition (dtype, strides, alignment, scale) still decides.  dash_attn_force_generic wins.
 */
void dash_attn_force_tensor(int on);

#ifdef __cplusplus
}
#endif
#endif /* DASH_ATTN_H */
