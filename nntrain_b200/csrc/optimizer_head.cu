// AdamW that reads the reduced BFP8 gradient directly (ABI minor 36).
//
// After the all-reduce the authoritative gradient is payload x (clipped)
// scales.  The reference decodes it into an fp32 cache and its AdamW kernel
// reads that cache (NNtrain.Cuda/native/tensor_kernels.cu:1148-1174,
// 3233-3241); its BFP8-native optimizers skip the cache
// (tensor_kernels.cu:3282-3365).  This entry point is the plain fp32-state
// AdamW with the decode folded into its head: g = code * scale is formed in
// registers, so the step never needs the 5.125 B/value decode pass nor the
// 4 B/value gradient read.  HBM traffic per value: 1.125 read for the
// gradient, 12 read + 12 written for parameter and moments (+2 for the
// optional bf16 compute copy).
//
// Arithmetic is adamw_kernel's, operation by operation, each one a separate
// IEEE binary32 operation (no contraction, no fast division or square root):
//   first  = beta1 * m + (1 - beta1) * g
//   second = beta2 * v + ((1 - beta2) * g) * g
//   p      = apply_weight_decay ? p * (1 - lr * wd) : p
//   p      = p - (update_scale * first) / (sqrt(second) + scaled_epsilon)
#include "reduce_kernels.cuh"

namespace ngb {
namespace {

constexpr Operation kOpOptimizerHead = static_cast<Operation>(217);

struct AdamWConstants {
    float beta1, beta2, one_minus_beta1, one_minus_beta2, decay, update_scale, scaled_epsilon;
    int apply_weight_decay;
};

__device__ __forceinline__ void adamw_one(float g, float& p, float& m, float& v, const AdamWConstants& c) {
    m = __fadd_rn(__fmul_rn(c.beta1, m), __fmul_rn(c.one_minus_beta1, g));
    v = __fadd_rn(__fmul_rn(c.beta2, v), __fmul_rn(__fmul_rn(c.one_minus_beta2, g), g));
    if (c.apply_weight_decay) p = __fmul_rn(p, c.decay);
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(c.update_scale, m), __fadd_rn(__fsqrt_rn(v), c.scaled_epsilon)));
}

template <int kShift>   // block = 1 << kShift, or < 0: runtime block
__global__ void __launch_bounds__(kThreads)
adamw_bfp8_gradient_kernel(float* __restrict__ data, const signed char* __restrict__ payload,
                           const float* __restrict__ scales, float* __restrict__ first_moment,
                           float* __restrict__ second_moment, unsigned short* __restrict__ compute_bf16,
                           long long length, long long block, AdamWConstants c, bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long words = vector_ok ? length / 4 : 0;
    for (long long w = thread; w < words; w += threads) {
        const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(payload) + w) ^ 0x80808080u;
        const float scale = __ldg(scales + (kShift >= 0 ? (w * 4) >> (kShift >= 0 ? kShift : 0) : (w * 4) / block));
        float4 p = load_f4(data + w * 4), m = load_f4(first_moment + w * 4), v = load_f4(second_moment + w * 4);
        adamw_one(__fmul_rn(byte_to_float(biased, 0), scale), p.x, m.x, v.x, c);
        adamw_one(__fmul_rn(byte_to_float(biased, 1), scale), p.y, m.y, v.y, c);
        adamw_one(__fmul_rn(byte_to_float(biased, 2), scale), p.z, m.z, v.z, c);
        adamw_one(__fmul_rn(byte_to_float(biased, 3), scale), p.w, m.w, v.w, c);
        store_f4(data + w * 4, p);
        store_f4(first_moment + w * 4, m);
        store_f4(second_moment + w * 4, v);
        if (compute_bf16 != nullptr) {
            uint2 out;
            out.x = float_to_bf16_bits(p.x) | (static_cast<unsigned>(float_to_bf16_bits(p.y)) << 16);
            out.y = float_to_bf16_bits(p.z) | (static_cast<unsigned>(float_to_bf16_bits(p.w)) << 16);
            *reinterpret_cast<uint2*>(compute_bf16 + w * 4) = out;
        }
    }
    for (long long i = words * 4 + thread; i < length; i += threads) {
        const float scale = scales[kShift >= 0 ? i >> (kShift >= 0 ? kShift : 0) : i / block];
        float p = data[i], m = first_moment[i], v = second_moment[i];
        adamw_one(__fmul_rn(static_cast<float>(payload[i]), scale), p, m, v, c);
        data[i] = p;
        first_moment[i] = m;
        second_moment[i] = v;
        if (compute_bf16 != nullptr) compute_bf16[i] = float_to_bf16_bits(p);
    }
}

inline bool aligned_to(const void* p, std::uintptr_t bytes) {
    return (reinterpret_cast<std::uintptr_t>(p) & (bytes - 1)) == 0;
}

}  // namespace
}  // namespace ngb

using namespace ngb;

// One AdamW step over `length` parameters whose gradient is the encoded arena
// (payload, one fp32 scale per `block_size` values; 0 = one scale for all).
// compute_bf16 (optional): the bf16 working copy of the updated parameters.
NNTRAIN_EXPORT int nntrain_optimizer_adamw_bfp8_gradient(
    int device, float* data, const signed char* gradient_payload, const float* gradient_scales, int block_size,
    float* first_moment, float* second_moment, unsigned short* compute_bf16, long long length, float beta1,
    float beta2, float learning_rate, float weight_decay, float update_scale, float scaled_epsilon,
    int apply_weight_decay, cudaStream_t stream) {
    if (!data || !gradient_payload || !gradient_scales || !first_moment || !second_moment || length <= 0 ||
        block_size < 0)
        return complete(kOpOptimizerHead, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpOptimizerHead, device, status);
    long long block = block_size == 0 || block_size > length ? length : block_size;
    AdamWConstants c{beta1, beta2, 1.0f - beta1, 1.0f - beta2, 1.0f - learning_rate * weight_decay, update_scale,
                     scaled_epsilon, apply_weight_decay};
    const bool vector_ok = aligned_to(data, 16) && aligned_to(first_moment, 16) && aligned_to(second_moment, 16) &&
                           aligned_to(gradient_payload, 4) && (!compute_bf16 || aligned_to(compute_bf16, 8)) &&
                           (block % 4 == 0 || block >= length);
    const int grid = grid_for((length / 4 + kThreads) / kThreads, kCtasPerSm);
    if (block == 32)
        adamw_bfp8_gradient_kernel<5><<<grid, kThreads, 0, stream>>>(data, gradient_payload, gradient_scales, first_moment, second_moment, compute_bf16, length, block, c, vector_ok);
    else if (block == 128)
        adamw_bfp8_gradient_kernel<7><<<grid, kThreads, 0, stream>>>(data, gradient_payload, gradient_scales, first_moment, second_moment, compute_bf16, length, block, c, vector_ok);
    else
        adamw_bfp8_gradient_kernel<-1><<<grid, kThreads, 0, stream>>>(data, gradient_payload, gradient_scales, first_moment, second_moment, compute_bf16, length, block, c, vector_ok);
    return complete(kOpOptimizerHead, device, static_cast<int>(cudaPeekAtLastError()));
}
