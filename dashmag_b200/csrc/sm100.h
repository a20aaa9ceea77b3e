// The tcgen05 tensor-core path (bf16 / f16, head dimension 128): interface to the C ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/dash_attn.h"

namespace dash {
struct TrainArgs;

// Whether the tensor-core kernels take the call (dtype, head dimension, strides, alignment).
// `any_size` lifts the rule that keeps single-tile problems of head dimension 64 / 256 on the generic
// kernels (a switch for tests).
bool sm100_takes(const dash_attn_params *p, const void *q, const void *k, const void *v, int backward, bool any_size = false);
// How many tensor maps the driver has encoded for this process (repeated calls reuse theirs).
uint64_t sm100_tensor_map_encodes();
// Extra scratch the tensor-core path needs beyond what the C ABI layer itself plans.
size_t sm100_forward_workspace(const dash_attn_params *p);
size_t sm100_backward_workspace(const dash_attn_params *p);
// Launchers: add to *launches; a failure that is not a CUDA error code is reported through `err`.
cudaError_t sm100_forward(const dash_attn_params *p, const TrainArgs &a, void *workspace, cudaStream_t stream,
                          int *launches, std::string &err);
cudaError_t sm100_backward(const dash_attn_params *p, const TrainArgs &a, void *workspace, cudaStream_t stream,
                           int *launches, bool *atomic, std::string &err);
}  // namespace dash
