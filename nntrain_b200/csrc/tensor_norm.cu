// Sum-of-squares, scaling and bf16 conversion entry points of the clip-norm
// path, plus the device-side clip coefficient.
//
// Replaces:
//   nntrain_tensor_squared_sum / _scale / _encode_bf16 / _decode_bf16
//       NNtrain.Cuda/native/tensor_kernels.cu:910-914,931-936,968-986,2876-2881,3177-3231,3870-3874
//       (these use the thread's implicit stream, tensor_kernels.cu:26,2888-2891)
//   nntrain_tensor_bf16_gradient_squared_sum / _scale
//       NNtrain.Cuda/native/pure_bfloat16_gradients.cu:315-348,546-570
// Clip arithmetic: NNtrain.Core/Torch/nn.cs:62-81.
#include "reduce_kernels.cuh"
#include "launchers.cuh"

namespace ngb {
namespace {

inline bool aligned_to(const void* p, std::uintptr_t bytes) {
    return (reinterpret_cast<std::uintptr_t>(p) & (bytes - 1)) == 0;
}

// Sum of (double)v*v over fp32 values; 128-bit loads when aligned.
__global__ void __launch_bounds__(kThreads)
f32_squared_sum_kernel(const float* __restrict__ values, long long length, double* result, bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long vectors = vector_ok ? length / 4 : 0;
    double squares = 0.0;
    for (long long i = thread; i < vectors; i += threads) {
        const float4 x = load_f4_stream(values + i * 4);
        squares += static_cast<double>(x.x) * static_cast<double>(x.x);
        squares += static_cast<double>(x.y) * static_cast<double>(x.y);
        squares += static_cast<double>(x.z) * static_cast<double>(x.z);
        squares += static_cast<double>(x.w) * static_cast<double>(x.w);
    }
    for (long long i = vectors * 4 + thread; i < length; i += threads)
        squares += static_cast<double>(values[i]) * static_cast<double>(values[i]);
    cta_accumulate(squares, result);
}

__global__ void __launch_bounds__(kThreads)
bf16_squared_sum_kernel(const unsigned short* __restrict__ values, long long length, double* result,
                        bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long groups = vector_ok ? length / 8 : 0;
    double squares = 0.0;
    for (long long g = thread; g < groups; g += threads) {
        const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(values + g * 8));
        const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            const double lo = static_cast<double>(__uint_as_float(w[q] << 16));
            const double hi = static_cast<double>(__uint_as_float(w[q] & 0xffff0000u));
            squares += lo * lo;
            squares += hi * hi;
        }
    }
    for (long long i = groups * 8 + thread; i < length; i += threads) {
        const double v = static_cast<double>(bf16_bits_to_float(values[i]));
        squares += v * v;
    }
    cta_accumulate(squares, result);
}

// Sum of squares of decoded BFP8 values; a block whose scale is not finite
// and positive contributes nothing and raises the flag
// (NNtrain.Cuda/native/tensor_kernels.cu:1047-1073).
__global__ void __launch_bounds__(kThreads)
bfp8_squared_sum_kernel(const signed char* __restrict__ payload, const float* __restrict__ scales,
                        long long length, long long block, double* result, int* finite_status,
                        bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long words = vector_ok ? length / 4 : 0;
    double squares = 0.0;
    int invalid = 0;
    for (long long w = thread; w < words; w += threads) {
        const float scale = __ldg(scales + (w * 4) / block);
        if (bad_scale(scale)) { invalid = 1; continue; }
        const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(payload) + w) ^ 0x80808080u;
        #pragma unroll
        for (int b = 0; b < 4; ++b) {
            const double d = static_cast<double>(__fmul_rn(byte_to_float(biased, b), scale));
            squares += d * d;
        }
    }
    for (long long i = words * 4 + thread; i < length; i += threads) {
        const float scale = scales[i / block];
        if (bad_scale(scale)) { invalid = 1; continue; }
        const double d = static_cast<double>(__fmul_rn(static_cast<float>(payload[i]), scale));
        squares += d * d;
    }
    if (finite_status != nullptr) {
        if (__any_sync(0xffffffffu, invalid) && (threadIdx.x & 31) == 0) atomicExch(finite_status, 1);
    }
    cta_accumulate(squares, result);
}

__global__ void __launch_bounds__(kThreads)
f32_scale_kernel(float* values, long long length, float multiplier, const float* coefficient, bool vector_ok) {
    // with a device-resident coefficient nothing is touched when it is 1
    if (coefficient != nullptr) {
        multiplier = coefficient[1];
        if (multiplier == 1.0f) return;
    }
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long vectors = vector_ok ? length / 4 : 0;
    for (long long i = thread; i < vectors; i += threads) {
        float4 x = load_f4(values + i * 4);
        x.x = __fmul_rn(x.x, multiplier); x.y = __fmul_rn(x.y, multiplier);
        x.z = __fmul_rn(x.z, multiplier); x.w = __fmul_rn(x.w, multiplier);
        store_f4(values + i * 4, x);
    }
    for (long long i = vectors * 4 + thread; i < length; i += threads)
        values[i] = __fmul_rn(values[i], multiplier);
}

// g = bf16_rn(f32(g) * multiplier)  (pure_bfloat16_gradients.cu:337-348)
__global__ void __launch_bounds__(kThreads)
bf16_scale_kernel(unsigned short* values, long long length, float multiplier, const float* coefficient,
                  bool vector_ok) {
    if (coefficient != nullptr) {
        multiplier = coefficient[1];
        if (multiplier == 1.0f) return;
    }
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long groups = vector_ok ? length / 8 : 0;
    for (long long g = thread; g < groups; g += threads) {
        uint4 raw = *reinterpret_cast<const uint4*>(values + g * 8);
        unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            const unsigned lo = float_to_bf16_bits(__fmul_rn(__uint_as_float(w[q] << 16), multiplier));
            const unsigned hi = float_to_bf16_bits(__fmul_rn(__uint_as_float(w[q] & 0xffff0000u), multiplier));
            w[q] = lo | (hi << 16);
        }
        *reinterpret_cast<uint4*>(values + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (long long i = groups * 8 + thread; i < length; i += threads)
        values[i] = float_to_bf16_bits(__fmul_rn(bf16_bits_to_float(values[i]), multiplier));
}

// fp32 -> bf16 into destination[destination_offset + i]
// (gradient_collectives.cu:11-22; tensor_kernels.cu:931-936).
__global__ void __launch_bounds__(kThreads)
f32_to_bf16_kernel(const float* __restrict__ source, unsigned short* __restrict__ destination,
                   long long length, bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long vectors = vector_ok ? length / 4 : 0;
    for (long long i = thread; i < vectors; i += threads) {
        const float4 x = load_f4_stream(source + i * 4);
        uint2 packed;
        packed.x = float_to_bf16_bits(x.x) | (static_cast<unsigned>(float_to_bf16_bits(x.y)) << 16);
        packed.y = float_to_bf16_bits(x.z) | (static_cast<unsigned>(float_to_bf16_bits(x.w)) << 16);
        *reinterpret_cast<uint2*>(destination + i * 4) = packed;
    }
    for (long long i = vectors * 4 + thread; i < length; i += threads)
        destination[i] = float_to_bf16_bits(source[i]);
}

__global__ void __launch_bounds__(kThreads)
bf16_to_f32_kernel(const unsigned short* __restrict__ source, float* __restrict__ destination,
                   long long length, bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long vectors = vector_ok ? length / 4 : 0;
    for (long long i = thread; i < vectors; i += threads) {
        const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(source + i * 4));
        store_f4(destination + i * 4,
                 make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                             __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u)));
    }
    for (long long i = vectors * 4 + thread; i < length; i += threads)
        destination[i] = bf16_bits_to_float(source[i]);
}

__global__ void __launch_bounds__(kThreads)
f32_copy_kernel(const float* __restrict__ source, float* __restrict__ destination, long long length,
                bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long vectors = vector_ok ? length / 4 : 0;
    for (long long i = thread; i < vectors; i += threads)
        store_f4(destination + i * 4, load_f4_stream(source + i * 4));
    for (long long i = vectors * 4 + thread; i < length; i += threads) destination[i] = source[i];
}

// Clip coefficient from the device-resident sum of squares, no host round
// trip:  norm = (float)sqrt(sum); c = norm > max_norm ? max_norm/(norm+1e-6f) : 1.
// out[0] = norm (pre-clip), out[1] = c.
__global__ void clip_coefficient_kernel(const double* squared_sum, float max_norm, float* out) {
    const float norm = static_cast<float>(sqrt(*squared_sum));
    float c = 1.0f;
    if (norm > max_norm) c = __fdiv_rn(max_norm, __fadd_rn(norm, 1e-6f));
    out[0] = norm;
    out[1] = c;
}

// scales[i] = fmaxf(scales[i] * c, FLT_MIN), payload untouched
// (tensor_kernels.cu:1075-1082).  The multiplier is either the argument or,
// when `coefficient` is given, coefficient[1] read on the device.
__global__ void __launch_bounds__(kThreads)
bfp8_scale_scales_kernel(float* scales, long long count, float multiplier, const float* coefficient) {
    const float c = coefficient != nullptr ? coefficient[1] : multiplier;
    if (coefficient != nullptr && c == 1.0f) return;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += threads)
        scales[i] = fmaxf(__fmul_rn(scales[i], c), FLT_MIN);
}

int elementwise_grid(long long items_per_thread_units) {
    return grid_for((items_per_thread_units + kThreads - 1) / kThreads, kCtasPerSm);
}

}  // namespace

cudaError_t launch_f32_squared_sum(const float* values, long long length, double* result, cudaStream_t stream) {
    f32_squared_sum_kernel<<<elementwise_grid(length / 4 + 1), kThreads, 0, stream>>>(
        values, length, result, aligned_to(values, 16));
    return cudaPeekAtLastError();
}

cudaError_t launch_bf16_squared_sum(const unsigned short* values, long long length, double* result,
                                    cudaStream_t stream) {
    bf16_squared_sum_kernel<<<elementwise_grid(length / 8 + 1), kThreads, 0, stream>>>(
        values, length, result, aligned_to(values, 16));
    return cudaPeekAtLastError();
}

cudaError_t launch_bfp8_squared_sum(const signed char* payload, const float* scales, long long length,
                                    long long block, double* result, int* finite_status, cudaStream_t stream) {
    if (block > length) block = length;
    // a 4-value word must not straddle two blocks on the vector path
    const bool vector_ok = aligned_to(payload, 4) && (block % 4 == 0 || block >= length);
    bfp8_squared_sum_kernel<<<elementwise_grid(length / 4 + 1), kThreads, 0, stream>>>(
        payload, scales, length, block, result, finite_status, vector_ok);
    return cudaPeekAtLastError();
}

cudaError_t launch_f32_scale(float* values, long long length, float multiplier, cudaStream_t stream,
                             const float* coefficient) {
    f32_scale_kernel<<<elementwise_grid(length / 4 + 1), kThreads, 0, stream>>>(
        values, length, multiplier, coefficient, aligned_to(values, 16));
    return cudaPeekAtLastError();
}

cudaError_t launch_bf16_scale(unsigned short* values, long long length, float multiplier, cudaStream_t stream,
                              const float* coefficient) {
    bf16_scale_kernel<<<elementwise_grid(length / 8 + 1), kThreads, 0, stream>>>(
        values, length, multiplier, coefficient, aligned_to(values, 16));
    return cudaPeekAtLastError();
}

cudaError_t launch_f32_to_bf16(const float* source, unsigned short* destination, long long length,
                               cudaStream_t stream) {
    f32_to_bf16_kernel<<<elementwise_grid(length / 4 + 1), kThreads, 0, stream>>>(
        source, destination, length, aligned_to(source, 16) && aligned_to(destination, 8));
    return cudaPeekAtLastError();
}

cudaError_t launch_bf16_to_f32(const unsigned short* source, float* destination, long long length,
                               cudaStream_t stream) {
    bf16_to_f32_kernel<<<elementwise_grid(length / 4 + 1), kThreads, 0, stream>>>(
        source, destination, length, aligned_to(source, 8) && aligned_to(destination, 16));
    return cudaPeekAtLastError();
}

cudaError_t launch_f32_copy(const float* source, float* destination, long long length, cudaStream_t stream) {
    f32_copy_kernel<<<elementwise_grid(length / 4 + 1), kThreads, 0, stream>>>(
        source, destination, length, aligned_to(source, 16) && aligned_to(destination, 16));
    return cudaPeekAtLastError();
}

cudaError_t launch_bfp8_scale_scales(float* scales, long long count, float multiplier,
                                     const float* coefficient, cudaStream_t stream) {
    bfp8_scale_scales_kernel<<<elementwise_grid(count), kThreads, 0, stream>>>(scales, count, multiplier, coefficient);
    return cudaPeekAtLastError();
}

cudaError_t launch_clip_coefficient(const double* squared_sum, float max_norm, float* norm_and_coefficient,
                                    cudaStream_t stream) {
    clip_coefficient_kernel<<<1, 1, 0, stream>>>(squared_sum, max_norm, norm_and_coefficient);
    return cudaPeekAtLastError();
}

}  // namespace ngb

using namespace ngb;

// ---- exports that run on the thread's implicit stream -------------------------
NNTRAIN_EXPORT int nntrain_tensor_squared_sum(const float* values, int length, double* result) {
    if (!values || length <= 0 || !result) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(launch_f32_squared_sum(values, length, result, implicit_stream()));
}

NNTRAIN_EXPORT int nntrain_tensor_scale(float* values, int length, float scale) {
    if (!values || length <= 0) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(launch_f32_scale(values, length, scale, implicit_stream()));
}

NNTRAIN_EXPORT int nntrain_tensor_encode_bf16(const float* source, unsigned short* destination, int length) {
    if (!source || !destination || length <= 0) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(launch_f32_to_bf16(source, destination, length, implicit_stream()));
}

NNTRAIN_EXPORT int nntrain_tensor_decode_bf16(const unsigned short* source, float* destination, int length) {
    if (!source || !destination || length <= 0) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(launch_bf16_to_f32(source, destination, length, implicit_stream()));
}

// ---- bf16 gradient arena norm / clip ------------------------------------------
NNTRAIN_EXPORT int nntrain_tensor_bf16_gradient_squared_sum(const unsigned short* values, int length,
                                                            double* result, cudaStream_t stream) {
    if (!values || length <= 0 || !result) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(launch_bf16_squared_sum(values, length, result, stream));
}

NNTRAIN_EXPORT int nntrain_tensor_bf16_gradient_scale(unsigned short* values, int length, float multiplier,
                                                      cudaStream_t stream) {
    if (!values || length <= 0 || !std::isfinite(multiplier)) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(launch_bf16_scale(values, length, multiplier, stream));
}

// ---- 64-bit-length / device-resident clip (ABI minor 36; no counterpart in
// the reference, which reads the sum of squares back to the host and clips
// with one launch per tensor) ---------------------------------------------------
// kind: 0 = fp32, 1 = bf16, 2 = BFP8 (values = payload, scales/block required).
static int gradient_squared_sum_impl(int device, int kind, const void* values, const float* scales,
                                                long long length, int block_size, double* squared_sum,
                                                int* finite_status, cudaStream_t stream) {
    if (!values || length <= 0 || !squared_sum || kind < 0 || kind > 2 || (kind == 2 && (!scales || block_size < 0)))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    if (kind == 0) return static_cast<int>(launch_f32_squared_sum(static_cast<const float*>(values), length, squared_sum, stream));
    if (kind == 1) return static_cast<int>(launch_bf16_squared_sum(static_cast<const unsigned short*>(values), length, squared_sum, stream));
    return static_cast<int>(launch_bfp8_squared_sum(static_cast<const signed char*>(values), scales, length,
                                                    block_size == 0 ? length : block_size, squared_sum,
                                                    finite_status, stream));
}

// norm_and_coefficient[0] = (float)sqrt(*squared_sum), [1] = clip coefficient
// (1 when the norm does not exceed max_norm).  Runs on the device so the
// clip can be enqueued behind the reduction without a host read.
static int gradient_clip_coefficient_impl(int device, const double* squared_sum, float max_norm,
                                                     float* norm_and_coefficient, cudaStream_t stream) {
    if (!squared_sum || !norm_and_coefficient || !(max_norm > 0.0f))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(launch_clip_coefficient(squared_sum, max_norm, norm_and_coefficient, stream));
}

// Applies a clip multiplier to a whole arena.  kind 0: fp32 values *= c;
// kind 1: bf16 values = bf16_rn(f32 * c); kind 2: BFP8 scale sidecar
// scales[i] = fmaxf(scales[i] * c, FLT_MIN), payload untouched.  When
// `coefficient` is non-null the multiplier is coefficient[1] read on the
// device (the output of nntrain_gradient_clip_coefficient), `multiplier` is
// ignored, and a coefficient of exactly 1 leaves the arena untouched.
static int gradient_clip_apply_impl(int device, int kind, void* values, long long count,
                                               float multiplier, const float* coefficient, cudaStream_t stream) {
    if (!values || count <= 0 || kind < 0 || kind > 2) return static_cast<int>(cudaErrorInvalidValue);
    if (!coefficient && (!std::isfinite(multiplier) || !(multiplier > 0.0f)))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    if (kind == 0) return static_cast<int>(launch_f32_scale(static_cast<float*>(values), count, multiplier, stream, coefficient));
    if (kind == 1) return static_cast<int>(launch_bf16_scale(static_cast<unsigned short*>(values), count, multiplier, stream, coefficient));
    return static_cast<int>(launch_bfp8_scale_scales(static_cast<float*>(values), count, multiplier, coefficient, stream));
}

// failures of the ABI-minor-36 norm / clip exports are recorded in the error ring
NNTRAIN_EXPORT int nntrain_gradient_squared_sum(int device, int kind, const void* values, const float* scales, long long length, int block_size, double* squared_sum, int* finite_status, cudaStream_t stream) {
    return complete(kOpGradientNorm, device, gradient_squared_sum_impl(device, kind, values, scales, length, block_size, squared_sum, finite_status, stream));
}

NNTRAIN_EXPORT int nntrain_gradient_clip_coefficient(int device, const double* squared_sum, float max_norm, float* norm_and_coefficient, cudaStream_t stream) {
    return complete(kOpGradientNorm, device, gradient_clip_coefficient_impl(device, squared_sum, max_norm, norm_and_coefficient, stream));
}

NNTRAIN_EXPORT int nntrain_gradient_clip_apply(int device, int kind, void* values, long long count, float multiplier, const float* coefficient, cudaStream_t stream) {
    return complete(kOpGradientNorm, device, gradient_clip_apply_impl(device, kind, values, count, multiplier, coefficient, stream));
}
