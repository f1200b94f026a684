// BFP8 block codec with a bf16 tensor on the other side:
//   nntrain_cuda_bfp8_quantize_bf16     NNtrain.Cuda/native/cuda_runtime_bridge.cu:868-935,2024-2118
//   nntrain_cuda_bfp8_dequantize_bf16   NNtrain.Cuda/native/cuda_runtime_bridge.cu:769-806,1964-2022
// The arithmetic is the fp32 codec's on the widened value (a bf16 is an fp32
// with a zero low half): scale = max|x| / 127, code = clamp(rne(x / scale),
// +-127); the decode is bf16_rn(code * scale).  With these a gradient kept in
// bf16 is encoded straight from its storage, and an optimizer whose working
// copy is bf16 reads the reduced BFP8 gradient without an fp32 decode pass.
//
// Fast path (blocks of 32 / 64 / 128, 8-byte aligned bf16, 4-byte aligned
// payload): a lane owns four consecutive values per row (one 64-bit bf16 access,
// one 32-bit payload access), four independent rows per step; the block
// maximum is an integer max over the block's lanes.  Everything else goes
// through a warp-per-block kernel, the tensor-wide case through a maximum pass
// and a payload pass.
#include "bfp8_kernels.cuh"
#include "reduce_kernels.cuh"

namespace ngb {
namespace {

constexpr Operation kOpDequantizeBf16 = static_cast<Operation>(28);   // the reference's numbering
constexpr Operation kOpQuantizeBf16 = static_cast<Operation>(29);

__device__ __forceinline__ float4 widen4(uint2 raw) {
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

template <int kBlock>
__global__ void __launch_bounds__(kThreads)
bf16_encode_blocks_kernel(const unsigned short* __restrict__ source, signed char* __restrict__ payload,
                          float* __restrict__ scales, long long length) {
    constexpr int kLanesPerBlock = kBlock / 4;
    constexpr int kRows = 4;
    constexpr int kTile = 128 * kRows;
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long tiles = length / kTile;               // whole tiles only; the rest is done by the generic kernel
    const unsigned mask = group_mask<kLanesPerBlock>(lane);
    const bool leader = (lane & (kLanesPerBlock - 1)) == 0;
    for (long long tile = warp; tile < tiles; tile += warps) {
        const long long base = tile * kTile + lane * 4;
        uint2 raw[kRows];
        #pragma unroll
        for (int j = 0; j < kRows; ++j) raw[j] = __ldcs(reinterpret_cast<const uint2*>(source + base + j * 128));
        #pragma unroll
        for (int j = 0; j < kRows; ++j) {
            const float4 x = widen4(raw[j]);
            const float lane_max = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
            const bool odd = is_non_finite(x.x) | is_non_finite(x.y) | is_non_finite(x.z) | is_non_finite(x.w);
            const unsigned bits = group_max_bits<kLanesPerBlock>(mask, odd ? 0xffffffffu : __float_as_uint(lane_max));
            float scale, t0, t1, t2, t3;
            if (bits < 0x7f800000u) {
                scale = scale_from_maximum_fast(__uint_as_float(bits));
                biased_codes_of(x, block_scale(scale), t0, t1, t2, t3);
            } else {
                // NaN / Inf in the block: fmaxf drops NaN, the quotient rules apply per value
                const float m = group_max_masked<kLanesPerBlock>(
                    mask, fmaxf(fmaxf(fmaxf(0.0f, fabsf(x.x)), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
                scale = scale_from_maximum(m);
                t0 = biased_code_of(x.x, scale); t1 = biased_code_of(x.y, scale);
                t2 = biased_code_of(x.z, scale); t3 = biased_code_of(x.w, scale);
            }
            *reinterpret_cast<unsigned*>(payload + base + j * 128) = pack_codes(t0, t1, t2, t3);
            if (leader) scales[(base + j * 128) / kBlock] = scale;
        }
    }
}

// One warp per block: any block size, any alignment, [first_block, block_count).
__global__ void __launch_bounds__(kThreads)
bf16_encode_generic_kernel(const unsigned short* __restrict__ source, signed char* __restrict__ payload,
                           float* __restrict__ scales, long long length, long long block,
                           long long first_block, long long block_count) {
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    for (long long b = first_block + warp; b < block_count; b += warps) {
        const long long start = b * block;
        const long long end = start + block < length ? start + block : length;
        float m = 0.0f;
        for (long long i = start + lane; i < end; i += 32) m = fmaxf(m, fabsf(bf16_bits_to_float(source[i])));
        m = group_max<32>(m);
        const float scale = scale_from_maximum(m);
        if (lane == 0) scales[b] = scale;
        for (long long i = start + lane; i < end; i += 32)
            payload[i] = code_byte(biased_code_of(bf16_bits_to_float(source[i]), scale));
    }
}

__global__ void __launch_bounds__(kThreads)
bf16_tensor_max_kernel(const unsigned short* __restrict__ source, long long length, unsigned* maximum_bits) {
    __shared__ float warp_max[kWarpsPerCta];
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    float m = 0.0f;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < length; i += threads)
        m = fmaxf(m, fabsf(bf16_bits_to_float(source[i])));
    m = group_max<32>(m);
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kWarpsPerCta; ++w) m = fmaxf(m, warp_max[w]);
        if (m > 0.0f) atomicMax(maximum_bits, __float_as_uint(m));
    }
}

// Tensor-wide payload pass: scales[0] still holds the raw maximum (the bits the
// maximum pass left there); a one-thread kernel turns it into the scale
// afterwards.
__global__ void __launch_bounds__(kThreads)
bf16_tensor_payload_kernel(const unsigned short* __restrict__ source, signed char* __restrict__ payload,
                           const float* maximum, long long length) {
    const float scale = scale_from_maximum(maximum[0]);
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < length; i += threads)
        payload[i] = code_byte(biased_code_of(bf16_bits_to_float(source[i]), scale));
}

__global__ void finalize_tensor_scale_kernel(float* scale) { scale[0] = scale_from_maximum(scale[0]); }

template <int kShift>   // block = 1 << kShift, or < 0: runtime block
__global__ void __launch_bounds__(kThreads)
bfp8_decode_to_bf16_kernel(const signed char* __restrict__ payload, const float* __restrict__ scales,
                           unsigned short* __restrict__ destination, long long length, long long block,
                           bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long words = vector_ok ? length / 4 : 0;
    for (long long w = thread; w < words; w += threads) {
        const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(payload) + w) ^ 0x80808080u;
        const float scale = __ldg(scales + (kShift >= 0 ? (w * 4) >> (kShift >= 0 ? kShift : 0) : (w * 4) / block));
        uint2 out;
        out.x = float_to_bf16_bits(__fmul_rn(byte_to_float(biased, 0), scale)) |
                (static_cast<unsigned>(float_to_bf16_bits(__fmul_rn(byte_to_float(biased, 1), scale))) << 16);
        out.y = float_to_bf16_bits(__fmul_rn(byte_to_float(biased, 2), scale)) |
                (static_cast<unsigned>(float_to_bf16_bits(__fmul_rn(byte_to_float(biased, 3), scale))) << 16);
        *reinterpret_cast<uint2*>(destination + w * 4) = out;
    }
    for (long long i = words * 4 + thread; i < length; i += threads) {
        const float scale = scales[kShift >= 0 ? i >> (kShift >= 0 ? kShift : 0) : i / block];
        destination[i] = float_to_bf16_bits(__fmul_rn(static_cast<float>(payload[i]), scale));
    }
}

inline bool aligned_to(const void* p, std::uintptr_t bytes) {
    return (reinterpret_cast<std::uintptr_t>(p) & (bytes - 1)) == 0;
}

template <int kBlock>
cudaError_t encode_fast(const unsigned short* source, signed char* payload, float* scales, long long length,
                        cudaStream_t stream) {
    const long long tiles = length / 512;
    if (tiles > 0) {
        const int grid = codec_grid_for((tiles + kWarpsPerCta - 1) / kWarpsPerCta, kCtasPerSm);
        bf16_encode_blocks_kernel<kBlock><<<grid, kThreads, 0, stream>>>(source, payload, scales, length);
    }
    const long long blocks = (length + kBlock - 1) / kBlock, done = tiles * 512 / kBlock;
    if (done < blocks) {
        const int grid = grid_for((blocks - done + kWarpsPerCta - 1) / kWarpsPerCta, kCtasPerSm);
        bf16_encode_generic_kernel<<<grid, kThreads, 0, stream>>>(source, payload, scales, length, kBlock, done, blocks);
    }
    return cudaPeekAtLastError();
}

}  // namespace
}  // namespace ngb

using namespace ngb;

// quantization_block_size >= length means tensor-wide (one scale).
NNTRAIN_EXPORT int nntrain_cuda_bfp8_quantize_bf16(int device, const unsigned short* source, signed char* payload,
                                                   float* scales, int length, int quantization_block_size,
                                                   void* stream) {
    if (!source || !payload || !scales || length <= 0 || quantization_block_size <= 0)
        return complete(kOpQuantizeBf16, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpQuantizeBf16, device, status);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const long long n = length, block = quantization_block_size;
    cudaError_t e;
    if (block >= n) {
        e = cudaMemsetAsync(scales, 0, sizeof(float), s);
        if (e == cudaSuccess) {
            const int grid = grid_for((n + kThreads - 1) / kThreads, kCtasPerSm);
            bf16_tensor_max_kernel<<<grid, kThreads, 0, s>>>(source, n, reinterpret_cast<unsigned*>(scales));
            bf16_tensor_payload_kernel<<<grid, kThreads, 0, s>>>(source, payload, scales, n);
            finalize_tensor_scale_kernel<<<1, 1, 0, s>>>(scales);
            e = cudaPeekAtLastError();
        }
    } else if ((block == 32 || block == 64 || block == 128) && aligned_to(source, 8) && aligned_to(payload, 4)) {
        e = block == 32 ? encode_fast<32>(source, payload, scales, n, s)
          : block == 64 ? encode_fast<64>(source, payload, scales, n, s)
                        : encode_fast<128>(source, payload, scales, n, s);
    } else {
        const long long blocks = (n + block - 1) / block;
        const int grid = grid_for((blocks + kWarpsPerCta - 1) / kWarpsPerCta, kCtasPerSm);
        bf16_encode_generic_kernel<<<grid, kThreads, 0, s>>>(source, payload, scales, n, block, 0, blocks);
        e = cudaPeekAtLastError();
    }
    return complete(kOpQuantizeBf16, device, static_cast<int>(e));
}

NNTRAIN_EXPORT int nntrain_cuda_bfp8_dequantize_bf16(int device, const signed char* payload, const float* scales,
                                                     unsigned short* destination, int length,
                                                     int quantization_block_size, void* stream) {
    if (!payload || !scales || !destination || length <= 0 || quantization_block_size <= 0)
        return complete(kOpDequantizeBf16, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpDequantizeBf16, device, status);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const long long n = length;
    long long block = quantization_block_size;
    if (block > n) block = n;
    // a 4-value word must not straddle two blocks on the vector path
    const bool vector_ok = aligned_to(payload, 4) && aligned_to(destination, 8) && (block % 4 == 0 || block >= n);
    const int grid = codec_grid_for((n / 4 + kThreads * 4) / (kThreads * 4), kCtasPerSm);
    if (block == 32) bfp8_decode_to_bf16_kernel<5><<<grid, kThreads, 0, s>>>(payload, scales, destination, n, block, vector_ok);
    else if (block == 128) bfp8_decode_to_bf16_kernel<7><<<grid, kThreads, 0, s>>>(payload, scales, destination, n, block, vector_ok);
    else bfp8_decode_to_bf16_kernel<-1><<<grid, kThreads, 0, s>>>(payload, scales, destination, n, block, vector_ok);
    return complete(kOpDequantizeBf16, device, static_cast<int>(cudaPeekAtLastError()));
}
