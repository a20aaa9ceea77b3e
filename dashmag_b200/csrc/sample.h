// Sampling the next token from a decoder's logits (crates/dash-contract/src/sample.rs): arguments and launcher.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dash {

struct SampleArgs {
    const void *logits;      // [B, V], rows `stride` elements apart, the vocabulary contiguous
    int b, v;
    int64_t stride;
    int vec;                 // every row starts on a 16-byte boundary
    int greedy;              // temperature 0
    float tau;               // 1 / temperature as f32, at most f32::MAX
    int top_k;               // 0: top-k cuts nothing (k = 0 or k >= the unmasked tokens)
    int has_p;               // top-p cuts (p < 1)
    float p;
    uint32_t key0, key1, off_lo, off_hi;   // Philox key (seed) and the counter's upper words (offset)
    const uint32_t *masked_bits;           // bit i set: token i is masked; null: none
    void *tokens;            // [B] i32 or i64
    int token_bytes;
    float *logprob, *tempered, *sampling;  // [B]
};

cudaError_t launch_sample(int dtype, const SampleArgs &a, cudaStream_t stream, int *launches);

}  // namespace dash
