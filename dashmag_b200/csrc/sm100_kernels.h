// Arguments and launchers of the tcgen05 kernels (device side in fwd_sm100.cu, host side in
// sm100.cu, which encodes the TMA tensor maps).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace dash {

struct Sm100FwdArgs {
    int b, tq, tk, hq, hkv;
    float scale;       // the factor on the scores
    float scale_log2;  // scale * log2(e): the exponentials are base 2
    void *out;         // [B,Tq,Hq,128] contiguous, the inputs' dtype
    float *lse;        // [B,Tq,Hq]
    MaskArgs mask;
};

cudaError_t launch_fwd_sm100(int dtype, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                             const Sm100FwdArgs &a, cudaStream_t stream);
// Reads (and optionally clears) the sticky device word the kernels raise when a bounded wait ran
// out.  Synchronises with the device.
cudaError_t read_sm100_status(unsigned int *status, bool clear);

}  // namespace dash
