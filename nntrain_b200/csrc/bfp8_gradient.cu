// Tensor-wide BFP8 gradient publication and the two-device reduce / broadcast
// of the pure-BFP8 reducer.
//
// Replaces, signature for signature:
//   nntrain_bfp8_gradient_quantize             NNtrain.Cuda/native/tensor_kernels.cu:3876-3889
//   nntrain_bfp8_gradient_quantize_accumulate  :3891-3905
//   nntrain_bfp8_gradient_squared_sum          :3907-3921
//   nntrain_bfp8_gradient_scale                :3923-3933
//   nntrain_bfp8_gradient_reduce               :3935-4002
//   nntrain_bfp8_gradient_broadcast            :4004-4038
// The reference publishes a tensor with a memset and five or six launches
// (:1114-1146: per-element atomic maximum, finalize, quantize, decode, sum of
// squares); here it is a memset and three: maximum + finite flag (one atomic
// per CTA), payload + decode write-back + sum of squares in one pass, and the
// scale finalize.
#include "bfp8_kernels.cuh"
#include "reduce_kernels.cuh"
#include "launchers.cuh"

namespace ngb {
namespace {

// Raises *finite_status when the finished tensor-wide scale is not finite and
// positive (the reference's sum-of-squares kernel does this, :1051-1054).
__global__ void check_scale_kernel(const float* scale, int* finite_status) {
    if (bad_scale(scale[0])) atomicExch(finite_status, 1);
}

// OR of the peer's finite flag into ours (:1108-1112).
__global__ void merge_status_kernel(int* destination, const int* remote) {
    if (*remote != 0) *destination = 1;
}

__global__ void __launch_bounds__(kThreads)
bfp8_decode_gated_kernel(const signed char* __restrict__ payload, const float* __restrict__ scale,
                         float* __restrict__ destination, long long length, const int* skip_flag,
                         bool vector_ok) {
    if (*skip_flag != 0) return;
    const float s = scale[0];
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long words = vector_ok ? length / 4 : 0;
    for (long long w = thread; w < words; w += threads) {
        const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(payload) + w) ^ 0x80808080u;
        store_f4(destination + w * 4,
                 make_float4(__fmul_rn(byte_to_float(biased, 0), s), __fmul_rn(byte_to_float(biased, 1), s),
                             __fmul_rn(byte_to_float(biased, 2), s), __fmul_rn(byte_to_float(biased, 3), s)));
    }
    for (long long i = words * 4 + thread; i < length; i += threads)
        destination[i] = __fmul_rn(static_cast<float>(payload[i]), s);
}

// Publishes one tensor: payload + tensor-wide scale, the fp32 gradient
// overwritten with its decode, optional sum of squares.  A NaN/Inf anywhere
// (or an already raised flag) publishes nothing and leaves scale = 1.
cudaError_t publish_tensor(float* gradient, signed char* payload, float* scale, long long length,
                           int* finite_status, double* squared_sum, cudaStream_t stream) {
    const int flags = kEncWriteBack | kEncFiniteFlag | (squared_sum ? kEncSquares : 0);
    cudaError_t status = launch_bfp8_encode(gradient, gradient, payload, scale, length, length, flags,
                                            squared_sum, finite_status, true, stream);
    if (status != cudaSuccess || !squared_sum) return status;
    check_scale_kernel<<<1, 1, 0, stream>>>(scale, finite_status);
    return cudaPeekAtLastError();
}

}  // namespace
}  // namespace ngb

using namespace ngb;

NNTRAIN_EXPORT int nntrain_bfp8_gradient_quantize(int device, float* source, signed char* payload,
                                                  float* scale, int length, int* finite_status,
                                                  cudaStream_t stream) {
    if (device < 0 || !source || !payload || !scale || length <= 0 || !finite_status)
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(publish_tensor(source, payload, scale, length, finite_status, nullptr, stream));
}

NNTRAIN_EXPORT int nntrain_bfp8_gradient_quantize_accumulate(int device, float* source, signed char* payload,
                                                             float* scale, int length, int* finite_status,
                                                             double* squared_sum, cudaStream_t stream) {
    if (device < 0 || !source || !payload || !scale || length <= 0 || !finite_status || !squared_sum)
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(publish_tensor(source, payload, scale, length, finite_status, squared_sum, stream));
}

NNTRAIN_EXPORT int nntrain_bfp8_gradient_squared_sum(int device, const signed char* payload, const float* scale,
                                                     int length, double* squared_sum, int* finite_status,
                                                     cudaStream_t stream) {
    if (device < 0 || !payload || !scale || length <= 0 || !squared_sum || !finite_status)
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(launch_bfp8_squared_sum(payload, scale, length, length, squared_sum, finite_status, stream));
}

// Scale-only clip of one tensor: scale = fmaxf(scale * multiplier, FLT_MIN).
NNTRAIN_EXPORT int nntrain_bfp8_gradient_scale(int device, float* scale, float multiplier, cudaStream_t stream) {
    if (device < 0 || !scale || !std::isfinite(multiplier) || !(multiplier > 0.0f))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(launch_bfp8_scale_scales(scale, 1, multiplier, nullptr, stream));
}

// Two-device all-reduce of one tensor, primary side: pull the peer's payload,
// scale and finite flag, r = reduction_scale * (l*ls + r*rs) with every
// operation rounded separately, re-encode r tensor-wide, leave decode(encode r)
// in `reduced`, add its sum of squares, record `reduced_ready`.
NNTRAIN_EXPORT int nntrain_bfp8_gradient_reduce(
    int primary_device, int secondary_device, const signed char* local_payload, const float* local_scale,
    const signed char* remote_payload, const float* remote_scale, signed char* remote_payload_staging,
    float* remote_scale_staging, float* reduced, signed char* output_payload, float* output_scale,
    int length, float reduction_scale, int* finite_status, const int* remote_finite_status,
    int* remote_status_staging, double* squared_sum, cudaStream_t communication_stream,
    cudaEvent_t local_ready, cudaEvent_t remote_ready, cudaEvent_t reduced_ready) {
    if (primary_device < 0 || secondary_device < 0 || primary_device == secondary_device || !local_payload ||
        !local_scale || !remote_payload || !remote_scale || !remote_payload_staging || !remote_scale_staging ||
        !reduced || !output_payload || !output_scale || length <= 0 || !std::isfinite(reduction_scale) ||
        !finite_status || !remote_finite_status || !remote_status_staging || !squared_sum ||
        !communication_stream || !local_ready || !remote_ready || !reduced_ready)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t status = static_cast<cudaError_t>(select_device(primary_device));
    if (status != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaStreamWaitEvent(communication_stream, local_ready, 0)) != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaStreamWaitEvent(communication_stream, remote_ready, 0)) != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(remote_payload_staging, primary_device, remote_payload, secondary_device,
                                      static_cast<size_t>(length), communication_stream)) != cudaSuccess)
        return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(remote_scale_staging, primary_device, remote_scale, secondary_device,
                                      sizeof(float), communication_stream)) != cudaSuccess)
        return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(remote_status_staging, primary_device, remote_finite_status, secondary_device,
                                      sizeof(int), communication_stream)) != cudaSuccess)
        return static_cast<int>(status);
    merge_status_kernel<<<1, 1, 0, communication_stream>>>(finite_status, remote_status_staging);
    if ((status = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(status);

    EncodedInputs in{};
    in.inputs = 2;
    in.payload[0] = local_payload;           in.scales[0] = local_scale;
    in.payload[1] = remote_payload_staging;  in.scales[1] = remote_scale_staging;
    status = launch_bfp8_sum_to_f32(in, reduced, length, length, reduction_scale, nullptr, finite_status,
                                    nullptr, communication_stream);
    if (status != cudaSuccess) return static_cast<int>(status);
    status = publish_tensor(reduced, output_payload, output_scale, length, finite_status, squared_sum,
                            communication_stream);
    if (status != cudaSuccess) return static_cast<int>(status);
    return static_cast<int>(cudaEventRecord(reduced_ready, communication_stream));
}

// Secondary side: pull the reduced payload + scale and decode into the fp32
// gradient (skipped when this device's finite flag is raised).
NNTRAIN_EXPORT int nntrain_bfp8_gradient_broadcast(
    int destination_device, int source_device, const signed char* source_payload, const float* source_scale,
    signed char* destination_payload, float* destination_scale, float* destination_float, int length,
    int* destination_finite_status, cudaStream_t destination_stream, cudaEvent_t source_ready) {
    if (destination_device < 0 || source_device < 0 || destination_device == source_device || !source_payload ||
        !source_scale || !destination_payload || !destination_scale || !destination_float || length <= 0 ||
        !destination_finite_status || !destination_stream || !source_ready)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t status = static_cast<cudaError_t>(select_device(destination_device));
    if (status != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaStreamWaitEvent(destination_stream, source_ready, 0)) != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(destination_payload, destination_device, source_payload, source_device,
                                      static_cast<size_t>(length), destination_stream)) != cudaSuccess)
        return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(destination_scale, destination_device, source_scale, source_device,
                                      sizeof(float), destination_stream)) != cudaSuccess)
        return static_cast<int>(status);
    const bool vector_ok = (reinterpret_cast<std::uintptr_t>(destination_payload) & 3u) == 0 &&
                           (reinterpret_cast<std::uintptr_t>(destination_float) & 15u) == 0;
    const int grid = grid_for((length / 4 + kThreads) / kThreads, kCtasPerSm);
    bfp8_decode_gated_kernel<<<grid, kThreads, 0, destination_stream>>>(
        destination_payload, destination_scale, destination_float, length, destination_finite_status, vector_ok);
    return static_cast<int>(cudaPeekAtLastError());
}
