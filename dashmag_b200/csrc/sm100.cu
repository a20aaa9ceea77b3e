#include "sm100.h"

#include "common.cuh"

namespace dash {
bool sm100_takes(const dash_attn_params *, const void *, const void *, const void *, int) { return false; }
size_t sm100_forward_workspace(const dash_attn_params *) { return 0; }
size_t sm100_backward_workspace(const dash_attn_params *) { return 0; }
cudaError_t sm100_forward(const dash_attn_params *, const TrainArgs &, void *, cudaStream_t, int *, std::string &err) {
    err = "attention: the tensor-core path is not built";
    return cudaSuccess;
}
cudaError_t sm100_backward(const dash_attn_params *, const TrainArgs &, void *, cudaStream_t, int *, bool *,
                           std::string &err) {
    err = "attention_backward: the tensor-core path is not built";
    return cudaSuccess;
}
}  // namespace dash
