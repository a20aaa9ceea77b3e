// Host-side launchers of the kernels, one per translation unit.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace dash {
struct TrainArgs;
struct DecodeArgs;

// Each adds the kernels it launched to *launches and returns the first launch error.
cudaError_t launch_generic_forward(int dtype, const TrainArgs &a, cudaStream_t stream, int *launches);
cudaError_t launch_generic_backward(int dtype, const TrainArgs &a, cudaStream_t stream, int *launches);
cudaError_t launch_generic_delta(int dtype, const TrainArgs &a, cudaStream_t stream, int *launches);
cudaError_t launch_decode(int dtype, const DecodeArgs &a, bool vector_ok, cudaStream_t stream, int *launches);
// The library's own decode scratch: its size in floats, and its address on the current device.
size_t decode_static_capacity_floats();
cudaError_t decode_static_scratch(float **out);
cudaError_t launch_fill_f32(float *dst, float value, long long n, cudaStream_t stream, int *launches);
}  // namespace dash
