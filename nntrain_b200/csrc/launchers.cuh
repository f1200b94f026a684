// Launchers defined in tensor_norm.cu and used by the other entry points.
#pragma once

#include "common.cuh"

namespace ngb {

cudaError_t launch_f32_squared_sum(const float* values, long long length, double* result, cudaStream_t stream);
cudaError_t launch_bf16_squared_sum(const unsigned short* values, long long length, double* result,
                                    cudaStream_t stream);
cudaError_t launch_bfp8_squared_sum(const signed char* payload, const float* scales, long long length,
                                    long long block, double* result, int* finite_status, cudaStream_t stream);
cudaError_t launch_f32_scale(float* values, long long length, float multiplier, cudaStream_t stream,
                             const float* coefficient = nullptr);
cudaError_t launch_bf16_scale(unsigned short* values, long long length, float multiplier, cudaStream_t stream,
                              const float* coefficient = nullptr);
cudaError_t launch_f32_to_bf16(const float* source, unsigned short* destination, long long length,
                               cudaStream_t stream);
cudaError_t launch_bf16_to_f32(const unsigned short* source, float* destination, long long length,
                               cudaStream_t stream);
cudaError_t launch_f32_copy(const float* source, float* destination, long long length, cudaStream_t stream);
cudaError_t launch_bfp8_scale_scales(float* scales, long long count, float multiplier,
                                     const float* coefficient, cudaStream_t stream);
cudaError_t launch_clip_coefficient(const double* squared_sum, float max_norm, float* norm_and_coefficient,
                                    cudaStream_t stream);

}  // namespace ngb
