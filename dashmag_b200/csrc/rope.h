// Rotary position embedding from tables (crates/dash-mag/src/rope.rs:94-107): arguments and launcher.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dash {

// One tensor [tokens, heads, d]: token and head strides in elements of the input and of the output
// (the features are contiguous in both).
struct RopeTensor {
    const void *x;
    void *out;   // may be x: every element is read before its pair is written
    int heads;
    int64_t st, sh, ost, osh;
};

struct RopeArgs {
    RopeTensor a, b;       // b.heads == 0: one tensor only.  Both share the tokens' positions.
    int64_t tokens;
    int d, dim;            // the first `dim` of `d` features are rotated, the rest pass through
    const void *cos, *sin; // [len, dim], the tensors' dtype
    int64_t len;
    int inverse;           // 1: the transpose of the rotation (what the gradient goes through)
    // The position of token n, first rule that applies:
    const void *positions; // [tokens] i32 / i64
    int pos_bytes;
    const void *cu;        // [sequences + 1] i32 / i64: start + n - cu[s] for cu[s] <= n < cu[s + 1]
    int cu_bytes, sequences;
    int64_t start, period; // start + n % period
};

cudaError_t launch_rope(int dtype, const RopeArgs &a, cudaStream_t stream, int *launches);

}  // namespace dash
