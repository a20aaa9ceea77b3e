// Arguments and launchers of the tcgen05 kernels (device side in fwd_sm100.cu, host side in
// sm100.cu, which encodes the TMA tensor maps).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace dash {

struct Sm100FwdArgs {
    int b, tq, tk, hq, hkv;
    int d;             // head dimension: 128, or 64 (two-tile kernel only)
    float scale;       // the factor on the scores
    float scale_log2;  // scale * log2(e): the exponentials are base 2
    void *out;         // [B,Tq,Hq,D] contiguous, the inputs' dtype
    float *lse;        // [B,Tq,Hq]
    MaskArgs mask;
    int pair_heads;    // two-tile kernel: the block's tiles are two heads of one group (else two row tiles)
};

struct Sm100BwdArgs {
    int b, tq, tk, hq, hkv;
    int d;               // head dimension: 128 or 64
    float scale, scale_log2;
    const float *lse;    // [B,Tq,Hq], the forward's
    const float *delta;  // [B,Tq,Hq], rowsum(dO * O)
    void *dq, *dk, *dv;  // contiguous, the inputs' dtype
    MaskArgs mask;
    int *order;          // scratch: the (key block, key-value head) units in launch order, [B * ceil(Tk / 128) * Hkv]
    float *dq_acc;       // scratch [B,Tq,Hq,D] f32, or null: the query gradient summed by reductions in L2 (the fused form)
};

// Tensor maps of the backward: every tensor with boxes of 128 rows, resident or streamed.
struct Sm100BwdMaps {
    CUtensorMap q128, do128, k128, v128;
    CUtensorMap dq128;                   // dq kernel's output
    CUtensorMap dq_acc;                  // the fused form's f32 accumulator, boxes of 32 columns x 128 rows
};

// Adds the kernels it launched to *launches.
cudaError_t launch_bwd_sm100(int dtype, const Sm100BwdMaps &m, const Sm100BwdArgs &a, cudaStream_t stream, int *launches);
size_t bwd_sm100_order_bytes(int b, int tk, int hkv);
cudaError_t launch_bwd_plan(Sm100BwdArgs &a, cudaStream_t stream, int *launches);
// Head dimension 256: the dq pass, the plan, and the dk and dv passes as one launch (bwd256_sm100.cu).
cudaError_t launch_bwd256_sm100(int dtype, const Sm100BwdMaps &m, const Sm100BwdArgs &a, cudaStream_t stream, int *launches);
cudaError_t read_sm100_bwd256_status(unsigned int *status, bool clear);
size_t bwd_sm100_fused_shared_bytes(int d);

cudaError_t launch_fwd_sm100(int dtype, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                             const Sm100FwdArgs &a, cudaStream_t stream);
// The two-tile forward: tq with boxes of 128 rows, tk / tv with boxes of 64 rows.
cudaError_t launch_fwd2_sm100(int dtype, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                              const CUtensorMap &to, const Sm100FwdArgs &a, cudaStream_t stream);
cudaError_t read_sm100_fwd2_status(unsigned int *status, bool clear);
// Reads (and optionally clears) the sticky device word the kernels raise when a bounded wait ran
// out.  Synchronises with the device.
cudaError_t read_sm100_status(unsigned int *status, bool clear);
cudaError_t read_sm100_bwd_status(unsigned int *status, bool clear);

}  // namespace dash
