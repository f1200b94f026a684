// Block / tensor-wide BFP8 codec entry points.
//
// Replaces, signature for signature, the reference's
//   nntrain_cuda_bfp8_quantize_f32            NNtrain.Cuda/native/cuda_runtime_bridge.cu:1540-1622
//   nntrain_cuda_bfp8_dequantize_f32          NNtrain.Cuda/native/cuda_runtime_bridge.cu:1720-1768
//   nntrain_cuda_bfp8_quantize_f32_roundtrip  NNtrain.Cuda/native/cuda_runtime_bridge.cu:1770-1826
// and adds the 64-bit-length block codec used by the N-rank reducers.
#include "bfp8_kernels.cuh"

namespace ngb {
namespace {

inline bool aligned_to(const void* p, std::uintptr_t bytes) {
    return (reinterpret_cast<std::uintptr_t>(p) & (bytes - 1)) == 0;
}

// Pass 3: turn the raw maxima into scales.  With a finite flag raised every
// scale becomes 1 (tensor_kernels.cu:1011-1021).
__global__ void bfp8_finalize_scales_kernel(float* maxima, long long count, const int* finite_status) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    if (finite_status != nullptr && *finite_status != 0) { maxima[i] = 1.0f; return; }
    maxima[i] = scale_from_maximum(maxima[i]);
}

// Any alignment, any block size.
__global__ void __launch_bounds__(kThreads)
bfp8_decode_scalar_kernel(const signed char* __restrict__ payload, const float* __restrict__ scales,
                          float* __restrict__ destination, long long length, long long block) {
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < length; i += threads)
        destination[i] = __fmul_rn(static_cast<float>(payload[i]), scales[i / block]);
}


template <int kBlock, int kFlags>
cudaError_t run_fast(const float* source, float* writeback, signed char* payload, float* scales,
                     long long length, double* squared_sum, int* finite_status, cudaStream_t stream) {
    const long long tiles = (length + kWarpTile - 1) / kWarpTile;
    const int grid = codec_grid_for((tiles + kWarpsPerCta - 1) / kWarpsPerCta,
                                    resident_ctas_per_sm<bfp8_encode_blocks_kernel<kBlock, kFlags>>());
    bfp8_encode_blocks_kernel<kBlock, kFlags><<<grid, kThreads, 0, stream>>>(
        source, writeback, payload, scales, length, squared_sum, finite_status);
    return cudaPeekAtLastError();
}

template <int kBlock>
cudaError_t dispatch_fast(int flags, const float* source, float* writeback, signed char* payload,
                          float* scales, long long length, double* squared_sum, int* finite_status,
                          cudaStream_t stream) {
#define NGB_CASE(F) \
    case F: return run_fast<kBlock, F>(source, writeback, payload, scales, length, squared_sum, finite_status, stream);
    switch (flags) {
        NGB_CASE(0) NGB_CASE(1) NGB_CASE(2) NGB_CASE(3)
        NGB_CASE(4) NGB_CASE(5) NGB_CASE(6) NGB_CASE(7)
        NGB_CASE(8)
        default: return cudaErrorInvalidValue;
    }
#undef NGB_CASE
}

template <int kFlags>
cudaError_t run_warp(const float* source, float* writeback, signed char* payload, float* scales,
                     long long length, long long block, double* squared_sum, int* finite_status,
                     cudaStream_t stream) {
    const long long count = (length + block - 1) / block;
    const int grid = codec_grid_for((count + kWarpsPerCta - 1) / kWarpsPerCta,
                                    resident_ctas_per_sm<bfp8_encode_warp_per_block_kernel<kFlags>>());
    bfp8_encode_warp_per_block_kernel<kFlags><<<grid, kThreads, 0, stream>>>(
        source, writeback, payload, scales, length, block, count, squared_sum, finite_status);
    return cudaPeekAtLastError();
}

cudaError_t dispatch_warp(int flags, const float* source, float* writeback, signed char* payload,
                          float* scales, long long length, long long block, double* squared_sum,
                          int* finite_status, cudaStream_t stream) {
#define NGB_CASE(F) \
    case F: return run_warp<F>(source, writeback, payload, scales, length, block, squared_sum, finite_status, stream);
    switch (flags) {
        NGB_CASE(0) NGB_CASE(1) NGB_CASE(2) NGB_CASE(3)
        NGB_CASE(4) NGB_CASE(5) NGB_CASE(6) NGB_CASE(7)
        NGB_CASE(8)
        default: return cudaErrorInvalidValue;
    }
#undef NGB_CASE
}

template <int kFlags>
void run_segment_payload(int grid, cudaStream_t stream, const float* source, float* writeback,
                         signed char* payload, const float* maxima, long long length, long long block,
                         const int* finite_status, double* squared_sum, int ctas_per_segment) {
    bfp8_segment_payload_kernel<kFlags><<<grid, kThreads, 0, stream>>>(
        source, writeback, payload, maxima, length, block, finite_status, squared_sum, ctas_per_segment);
}

// Three passes: zero + maxima, payload, finalize.  The scale slots double as
// the maxima accumulators between the passes, as in the reference's
// tensor-wide path (cuda_runtime_bridge.cu:1573-1595).
cudaError_t run_segments(int flags, const float* source, float* writeback, signed char* payload,
                         float* scales, long long length, long long block, double* squared_sum,
                         int* finite_status, bool skip_if_non_finite, cudaStream_t stream) {
    if (flags & kEncNanScale) return cudaErrorInvalidValue;
    const long long segments = (length + block - 1) / block;
    const long long span = block < length ? block : length;
    // ~4096 values per CTA pass keeps enough CTAs in flight without flooding
    // the atomics; never more CTAs in total than fill the machine 8 times.
    long long per_segment = (span + 16383) / 16384;
    const long long cap = static_cast<long long>(sm_count()) * kCtasPerSm;
    if (per_segment * segments > cap) per_segment = cap / segments;
    if (per_segment < 1) per_segment = 1;
    if (per_segment * segments > 2147483647ll) return cudaErrorInvalidConfiguration;
    const int grid = static_cast<int>(per_segment * segments);
    const int ctas_per_segment = static_cast<int>(per_segment);

    cudaError_t status = cudaMemsetAsync(scales, 0, sizeof(float) * static_cast<size_t>(segments), stream);
    if (status != cudaSuccess) return status;
    const bool finite = (flags & kEncFiniteFlag) != 0;
    if (finite) {
        bfp8_segment_max_kernel<true><<<grid, kThreads, 0, stream>>>(
            source, length, block, reinterpret_cast<unsigned*>(scales), finite_status, ctas_per_segment);
    } else {
        bfp8_segment_max_kernel<false><<<grid, kThreads, 0, stream>>>(
            source, length, block, reinterpret_cast<unsigned*>(scales), nullptr, ctas_per_segment);
    }
    status = cudaPeekAtLastError();
    if (status != cudaSuccess) return status;
    const int* gate = (finite && skip_if_non_finite) ? finite_status : nullptr;
    switch (flags & (kEncWriteBack | kEncSquares)) {
        case 0: run_segment_payload<0>(grid, stream, source, writeback, payload, scales, length, block, gate, squared_sum, ctas_per_segment); break;
        case 1: run_segment_payload<1>(grid, stream, source, writeback, payload, scales, length, block, gate, squared_sum, ctas_per_segment); break;
        case 2: run_segment_payload<2>(grid, stream, source, writeback, payload, scales, length, block, gate, squared_sum, ctas_per_segment); break;
        default: run_segment_payload<3>(grid, stream, source, writeback, payload, scales, length, block, gate, squared_sum, ctas_per_segment); break;
    }
    status = cudaPeekAtLastError();
    if (status != cudaSuccess) return status;
    const int finalize_grid = static_cast<int>((segments + kThreads - 1) / kThreads);
    bfp8_finalize_scales_kernel<<<finalize_grid, kThreads, 0, stream>>>(scales, segments, gate);
    return cudaPeekAtLastError();
}

}  // namespace

cudaError_t launch_bfp8_encode(const float* source, float* writeback, signed char* payload,
                               float* scales, long long length, long long block, int flags,
                               double* squared_sum, int* finite_status, bool skip_if_non_finite,
                               cudaStream_t stream) {
    if (!source || !payload || !scales || length <= 0 || block <= 0) return cudaErrorInvalidValue;
    if ((flags & kEncWriteBack) && !writeback) return cudaErrorInvalidValue;
    if ((flags & kEncSquares) && !squared_sum) return cudaErrorInvalidValue;
    if ((flags & kEncFiniteFlag) && !finite_status) return cudaErrorInvalidValue;
    if (block > length) block = length;
    const bool skip_semantics = skip_if_non_finite && (flags & kEncFiniteFlag);
    const bool fast_aligned = aligned_to(source, 16) && aligned_to(payload, 4) &&
                              (!(flags & kEncWriteBack) || aligned_to(writeback, 16));
    if (!skip_semantics && fast_aligned && block < length) {
        if (block == 32) return dispatch_fast<32>(flags, source, writeback, payload, scales, length, squared_sum, finite_status, stream);
        if (block == 64) return dispatch_fast<64>(flags, source, writeback, payload, scales, length, squared_sum, finite_status, stream);
        if (block == 128) return dispatch_fast<128>(flags, source, writeback, payload, scales, length, squared_sum, finite_status, stream);
    }
    if (!skip_semantics && block <= kMaxWarpBlock)
        return dispatch_warp(flags, source, writeback, payload, scales, length, block, squared_sum, finite_status, stream);
    return run_segments(flags, source, writeback, payload, scales, length, block, squared_sum,
                        finite_status, skip_if_non_finite, stream);
}

cudaError_t launch_bfp8_decode(const signed char* payload, const float* scales, float* destination,
                               long long length, long long block, cudaStream_t stream) {
    if (!payload || !scales || !destination || length <= 0 || block <= 0) return cudaErrorInvalidValue;
    if (block > length) block = length;
    const long long words = (length + 3) / 4;
    if (aligned_to(payload, 4) && aligned_to(destination, 16)) {
        const int grid = codec_grid_for((words + kThreads * kDecodeUnroll - 1) / (kThreads * kDecodeUnroll), kCtasPerSm);
        if (block == 32) bfp8_decode_blocks_kernel<5><<<grid, kThreads, 0, stream>>>(payload, scales, destination, length, block);
        else if (block == 64) bfp8_decode_blocks_kernel<6><<<grid, kThreads, 0, stream>>>(payload, scales, destination, length, block);
        else if (block == 128) bfp8_decode_blocks_kernel<7><<<grid, kThreads, 0, stream>>>(payload, scales, destination, length, block);
        else bfp8_decode_blocks_kernel<-1><<<grid, kThreads, 0, stream>>>(payload, scales, destination, length, block);
    } else {
        const int grid = grid_for((length + kThreads - 1) / kThreads, kCtasPerSm);
        bfp8_decode_scalar_kernel<<<grid, kThreads, 0, stream>>>(payload, scales, destination, length, block);
    }
    return cudaPeekAtLastError();
}

}  // namespace ngb

using namespace ngb;

// quantization_block_size >= length means tensor-wide (one scale).
NNTRAIN_EXPORT int nntrain_cuda_bfp8_quantize_f32(int device, const float* source, signed char* payload,
                                                  float* scales, int length, int quantization_block_size,
                                                  void* stream) {
    if (!source || !payload || !scales || length <= 0 || quantization_block_size <= 0)
        return complete(kOpBfp8Quantize, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpBfp8Quantize, device, status);
    return complete(kOpBfp8Quantize, device, static_cast<int>(launch_bfp8_encode(
        source, nullptr, payload, scales, length, quantization_block_size, 0, nullptr, nullptr, false,
        reinterpret_cast<cudaStream_t>(stream))));
}

NNTRAIN_EXPORT int nntrain_cuda_bfp8_dequantize_f32(int device, const signed char* payload,
                                                    const float* scales, float* destination, int length,
                                                    int quantization_block_size, void* stream) {
    if (!payload || !scales || !destination || length <= 0 || quantization_block_size <= 0)
        return complete(kOpBfp8DequantizeF32, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpBfp8DequantizeF32, device, status);
    return complete(kOpBfp8DequantizeF32, device, static_cast<int>(launch_bfp8_decode(
        payload, scales, destination, length, quantization_block_size,
        reinterpret_cast<cudaStream_t>(stream))));
}

// Encodes and overwrites the source with its decode in one pass.  The
// reference rejects the tensor-wide case here (block >= length).
NNTRAIN_EXPORT int nntrain_cuda_bfp8_quantize_f32_roundtrip(int device, float* source, signed char* payload,
                                                            float* scales, int length,
                                                            int quantization_block_size, void* stream) {
    if (!source || !payload || !scales || length <= 0 || quantization_block_size <= 0 ||
        quantization_block_size >= length)
        return complete(kOpBfp8Quantize, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpBfp8Quantize, device, status);
    return complete(kOpBfp8Quantize, device, static_cast<int>(launch_bfp8_encode(
        source, source, payload, scales, length, quantization_block_size, kEncWriteBack, nullptr, nullptr,
        false, reinterpret_cast<cudaStream_t>(stream))));
}

// ---- 64-bit-length block codec (ABI minor 36; no counterpart in the
// reference, whose lengths are 32-bit) ------------------------------------------
// Encodes `length` fp32 values in blocks of `block_size` values (0 or
// >= length: tensor-wide).  Optional outputs, each enabled by a non-null
// pointer: `roundtrip` receives code*scale (may alias `source`);
// `squared_sum` accumulates the sum of squares of the decoded values in
// binary64; `finite_status` is set to 1 when any input is NaN or Inf.
NNTRAIN_EXPORT int nntrain_bfp8_block_encode(int device, const float* source, signed char* payload,
                                             float* scales, long long length, int block_size,
                                             float* roundtrip, double* squared_sum, int* finite_status,
                                             void* stream) {
    if (!source || !payload || !scales || length <= 0 || block_size < 0)
        return complete(kOpBfp8Quantize, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpBfp8Quantize, device, status);
    const long long block = block_size == 0 ? length : block_size;
    const int flags = (roundtrip ? kEncWriteBack : 0) | (squared_sum ? kEncSquares : 0) |
                      (finite_status ? kEncFiniteFlag : 0);
    return complete(kOpBfp8Quantize, device, static_cast<int>(launch_bfp8_encode(
        source, roundtrip, payload, scales, length, block, flags, squared_sum, finite_status, false,
        reinterpret_cast<cudaStream_t>(stream))));
}

NNTRAIN_EXPORT int nntrain_bfp8_block_decode(int device, const signed char* payload, const float* scales,
                                             float* destination, long long length, int block_size,
                                             void* stream) {
    if (!payload || !scales || !destination || length <= 0 || block_size < 0)
        return complete(kOpBfp8DequantizeF32, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpBfp8DequantizeF32, device, status);
    const long long block = block_size == 0 ? length : block_size;
    return complete(kOpBfp8DequantizeF32, device, static_cast<int>(launch_bfp8_decode(
        payload, scales, destination, length, block, reinterpret_cast<cudaStream_t>(stream))));
}
