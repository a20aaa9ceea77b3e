/*
 * CPU oracle for the attention path: TEST INFRASTRUCTURE, not product code.
 *
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may load this file's
 * library; the product (the CUDA library under dashmag_b200/csrc) never links, loads or calls it.
 *
 * It restates, in plain C, the algorithm of the reference's CPU path
 * (crates/dash-ops/src/attention/reference.rs): everything in one real type whatever the inputs'
 * dtype, the key-value heads expanded to the query heads, the Tq x Tk scores and the boolean
 * "hidden" mask materialised per head, a softmax with the no-key guards, and plain matrix
 * products.  The arithmetic underneath the reference (matmul, exp, reductions) belongs to
 * burn-flex 0.22.1, a third-party crate that is not part of the reference checkout; what pins
 * this restatement is therefore the reference's own recorded fixtures (torch float64 / fp32
 * scaled_dot_product_attention, crates/dash-ops/tests/fixtures/attention), which
 * tests/test_oracle_golden.py checks it against.  Parity is pinned by those ten records.
 *
 * Every entry point exists twice: `_f64` computes in double (the parity oracle: agrees with
 * torch's float64 records to f32 rounding) and `_f32` computes in float exactly as the
 * reference's Flex path does (the timed CPU baseline).  Inputs and outputs are contiguous f32 in
 * the contract's layouts: q, o, do, dq [B,Tq,Hq,D]; k, v, dk, dv [B,Tk,Hkv,D]; lse [B,Tq,Hq].
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    int32_t b, tq, tk, hq, hkv, d;
    int32_t mask_kind;          /* 0 none, 1 key padding, 2 packed */
    const uint8_t *key_padding; /* [B,Tk], non-zero = key left out */
    const int64_t *cu_q;        /* [seqs+1] */
    const int64_t *cu_k;        /* [seqs+1] */
    int32_t seqs;
    int32_t causal;
    int64_t window_left;        /* < 0: unbounded */
    int64_t window_right;       /* < 0: unbounded */
    float scale;
} oracle_attn_params;

int oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* reference.rs:231-242 (Reach) and :75-77 (bound): a side binds only when it is shorter than
 * `span`; causality sets the right reach to 0. */
typedef struct { int left_binds, right_binds; int64_t left, right; } reach_t;

static reach_t reach_of(const oracle_attn_params *p, int64_t span) {
    reach_t r;
    int64_t left = p->window_left, right = p->causal ? 0 : p->window_right;
    r.left_binds = left >= 0 && left < span;
    r.right_binds = right >= 0 && right < span;
    r.left = left;
    r.right = right;
    return r;
}

/* reference.rs:99-116 outside_window: rel > pos + right or rel < pos - left. */
static int outside_window(const reach_t *r, int64_t pos, int64_t rel) {
    if (r->right_binds && rel > pos + r->right) return 1;
    if (r->left_binds && rel < pos - r->left) return 1;
    return 0;
}

/* reference.rs:120-162 sequences: the number of ends at or before the position, clamped into
 * 0..S-1, and whether the position lies inside [cu[0], cu[S]). */
static void sequence_at(const int64_t *cu, int32_t s, int64_t at, int64_t *index, int *inside) {
    int64_t passed = 0;
    for (int32_t e = 1; e <= s; ++e) passed += at >= cu[e];
    if (passed > s - 1) passed = s - 1;
    if (passed < 0) passed = 0;
    *index = passed;
    *inside = at >= cu[0] && at < cu[s];
}

/* The boolean mask of reference.rs:228-272 (hidden) for batch element `bi`: hidden[i*tk+j] = 1
 * where key j is hidden from query i. */
static void build_hidden(const oracle_attn_params *p, int32_t bi, uint8_t *hidden) {
    const int64_t tq = p->tq, tk = p->tk;
    reach_t r = reach_of(p, tq + tk + 1);
    if (p->mask_kind == 2) {
        /* reference.rs:177-223 packed_hidden */
        const int32_t s = p->seqs;
        if (s == 0 || tq == 0 || tk == 0) {
            memset(hidden, 1, (size_t)(tq * tk));
            return;
        }
        int64_t *seq_k = (int64_t *)malloc(sizeof(int64_t) * (size_t)tk);
        int64_t *rel = (int64_t *)malloc(sizeof(int64_t) * (size_t)tk);
        uint8_t *inside_k = (uint8_t *)malloc((size_t)tk);
        for (int64_t j = 0; j < tk; ++j) {
            int in;
            sequence_at(p->cu_k, s, j, &seq_k[j], &in);
            inside_k[j] = (uint8_t)in;
            rel[j] = j - p->cu_k[seq_k[j]];
        }
        for (int64_t i = 0; i < tq; ++i) {
            int64_t sq;
            int inside_q;
            sequence_at(p->cu_q, s, i, &sq, &inside_q);
            int64_t q_start = p->cu_q[sq], q_len = p->cu_q[sq + 1] - q_start;
            int64_t k_len = p->cu_k[sq + 1] - p->cu_k[sq];
            int64_t pos = (i - q_start) + (k_len - q_len);
            for (int64_t j = 0; j < tk; ++j) {
                int h = sq != seq_k[j] || !(inside_q && inside_k[j]);
                h = h || outside_window(&r, pos, rel[j]);
                hidden[i * tk + j] = (uint8_t)h;
            }
        }
        free(seq_k);
        free(rel);
        free(inside_k);
        return;
    }
    /* reference.rs:237-259: query i sits at key position i + Tk - Tq; key padding is OR-ed in. */
    for (int64_t i = 0; i < tq; ++i) {
        int64_t pos = i + tk - tq;
        for (int64_t j = 0; j < tk; ++j) {
            int h = outside_window(&r, pos, j);
            if (p->mask_kind == 1) h = h || p->key_padding[(int64_t)bi * tk + j] != 0;
            hidden[i * tk + j] = (uint8_t)h;
        }
    }
}

#define REAL double
#define SUFFIX(name) name##_f64
#define EXP exp
#define LOG log
#include "attention_oracle_body.inc"
#undef REAL
#undef SUFFIX
#undef EXP
#undef LOG

#define REAL float
#define SUFFIX(name) name##_f32
#define EXP expf
#define LOG logf
#include "attention_oracle_body.inc"
#undef REAL
#undef SUFFIX
#undef EXP
#undef LOG

/* The seeded inputs of the reference's tests (crates/dash-conformance/src/attention.rs:433-452,
 * crates/dash-ops/tests/attention_masks.rs:354-384): xorshift64 from seed * 0x9E3779B97F4A7C15 | 1,
 * the top 24 bits as a uniform in [0, 1), mapped to about [-2, 2] and rounded to bf16. */
static float round_to_bf16(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    bits = (bits + 0x7fffu + ((bits >> 16) & 1u)) & 0xffff0000u;
    memcpy(&x, &bits, 4);
    return x;
}

void oracle_seeded(float *out, int64_t n, uint64_t seed) {
    uint64_t state = (seed * 0x9E3779B97F4A7C15ull) | 1ull;
    for (int64_t i = 0; i < n; ++i) {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        float uniform = (float)(state >> 40) / (float)(1ull << 24);
        out[i] = round_to_bf16((uniform - 0.5f) * 4.0f);
    }
}

/* Deterministic booleans, true with probability p (attention_masks.rs:373-384). */
void oracle_coins(uint8_t *out, int64_t n, float p, uint64_t seed) {
    uint64_t state = (seed * 0x2545F4914F6CDD1Dull) | 1ull;
    for (int64_t i = 0; i < n; ++i) {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        out[i] = ((float)(state >> 40) / (float)(1ull << 24)) < p;
    }
}
