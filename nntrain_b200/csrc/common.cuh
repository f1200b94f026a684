// Shared plumbing for the gradient-path library: export macro, status
// recording, per-thread device selection, launch geometry, and the small
// device helpers every kernel uses (IEEE scale / code arithmetic, vector
// access, block-wide reductions).
//
// All translation units are compiled for sm_100a WITHOUT fast-math and with
// -fmad=false: the codec must agree bit for bit with the reference's CPU codec
// (NNtrain.Core/Tensors/Bfp8Quantization.cs:188-274), which neither flushes
// subnormals nor fuses a multiply into an add.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cfloat>
#include <cmath>
#include <cstddef>
#include <cstdint>

#define NNTRAIN_EXPORT extern "C" __attribute__((visibility("default")))

namespace ngb {

constexpr int kCtasPerSmDefault = 8;
constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;
constexpr int kCtasPerSm = 8;

// ---- ABI / status ---------------------------------------------------------
// Same numbering as the reference's native layer
// (NNtrain.Cuda/native/cuda_runtime_bridge.cu:18-21,23-72).
constexpr std::uint32_t kAbiMajor = 1;
constexpr std::uint32_t kAbiMinor = 36;   // 35 = reference; 36 adds the N-rank exports
constexpr std::uint32_t kAbiVersion = (kAbiMajor << 16) | kAbiMinor;

enum Operation : std::uint32_t {
    kOpNone = 0,
    kOpSetDevice = 3,
    kOpCapabilities = 25,
    kOpBfp8Quantize = 26,
    kOpBfp8DequantizeF32 = 27,
    // ABI minor 36 (no counterpart in the reference's numbering)
    // 200: the allocation-free owner reduce (no_alloc.cu)
    kOpGradientPeerMemory = 210,
    kOpGradientGroup = 211,
    kOpGradientReduceShards = 212,
    kOpGradientAllReduce = 213,
    kOpGradientLocalGroup = 214,
    kOpGradientLocalAllReduce = 215,
    kOpGradientPublishTensors = 216,
    // 217: the AdamW head that reads the encoded gradient (optimizer_head.cu)
    kOpGradientNorm = 218,
};

struct ErrorInfo {            // layout of nntrain_native_error_info (:74-82)
    std::uint32_t struct_size;
    std::uint32_t abi_version;
    std::uint64_t sequence;
    std::int32_t status;
    std::int32_t device;
    std::uint32_t operation;
    std::uint32_t reserved;
};

// Records a failed status in the error ring and returns it unchanged; the
// success path takes no lock.
int complete(Operation operation, int device, int status);

// Thread-local device cache: cudaSetDevice only when the thread's selection
// changes (cuda_runtime_bridge.cu:122-131).
int select_device(int device);

// Thread-local "current stream" used by the exports that take no stream
// argument (NNtrain.Cuda/native/tensor_kernels.cu:26,2888-2891).
cudaStream_t& implicit_stream();

// Number of SMs of the current device (cached per device).
int sm_count();

// Launch shape policy (process-wide, set by nntrain_gradient_configure):
//   codec_iterations_per_cta  n > 0 (default 2): every CTA of an encode /
//       decode kernel does n loop iterations and retires; a kernel on another
//       stream (the collective) then finds free SM slots while a codec kernel
//       runs.  0: persistent grids (one resident wave looping over the input).
//   codec_ctas  n > 0 (with codec_iterations_per_cta == 0): persistent codec
//       grids of at most n CTAs, which bounds the share of HBM bandwidth and
//       of SM slots a codec kernel takes while the collective runs.
//   collective_ctas  0: the all-reduce kernels also fill the machine.  n > 0:
//       they use at most n CTAs and leave the rest of the SMs' capacity to the
//       codec kernels of the neighbouring chunks.
struct LaunchPolicy {
    int codec_iterations_per_cta;
    int collective_ctas;
    int collective_async;     // 1: all-reduce kernels stage their inputs with cp.async rings
    int codec_ctas;           // > 0: persistent codec grids of at most this many CTAs
};
LaunchPolicy launch_policy();
void set_launch_policy(int codec_iterations_per_cta, int collective_ctas);
void set_collective_async(int enabled);
void set_codec_ctas(int ctas);

// Persistent grid for `work_items` CTA-sized loop iterations: fill every SM
// `per_sm` times, never more than the work needs.
inline int grid_for(long long work_items, int per_sm) {
    if (work_items < 1) work_items = 1;
    long long cap = static_cast<long long>(sm_count()) * per_sm;
    return static_cast<int>(work_items < cap ? work_items : cap);
}

// Grid for the encode / decode kernels under the launch policy: short-lived
// CTAs of a few iterations each (the default, and the fastest measured: the
// CTAs drift apart, which mixes DRAM reads and writes better than one resident
// wave marching in step), or a persistent grid, optionally capped.
inline int codec_grid_for(long long work_items, int per_sm) {
    if (work_items < 1) work_items = 1;
    const LaunchPolicy policy = launch_policy();
    if (policy.codec_iterations_per_cta > 0) {
        const long long ctas = (work_items + policy.codec_iterations_per_cta - 1) / policy.codec_iterations_per_cta;
        return static_cast<int>(ctas < 2147483647ll ? ctas : 2147483647ll);
    }
    long long cap = static_cast<long long>(sm_count()) * per_sm;
    if (policy.codec_ctas > 0 && policy.codec_ctas < cap) cap = policy.codec_ctas;
    return static_cast<int>(work_items < cap ? work_items : cap);
}

// CTAs of `kKernel` (kThreads threads, no dynamic shared memory) that fit on
// one SM.  A persistent grid must be exactly one resident wave: with more CTAs
// than fit, the surplus runs as a second, partly empty wave (a 48-register
// kernel fits 5 CTAs per SM, so a grid of 8 per SM ran at 80 % of its speed).
#ifdef __CUDACC__
template <auto kKernel>
int resident_ctas_per_sm() {
    static int cached = 0;
    if (cached == 0) {
        int fit = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, kKernel, kThreads, 0) != cudaSuccess || fit < 1)
            fit = 4;
        cached = fit;
    }
    return cached;
}
#endif

// ---- device helpers -------------------------------------------------------
#ifdef __CUDACC__

// scale = max == 0 ? 1 : max / 127, one IEEE division
// (Bfp8Quantization.cs:217; cuda_runtime_bridge.cu:138-140).
__device__ __forceinline__ float scale_from_maximum(float maximum) {
    return maximum == 0.0f ? 1.0f : __fdiv_rn(maximum, 127.0f);
}

// The same value in three FP32 instructions when the maximum lies in
// [2^-90, 2^100]: q0 = m * r, e = fma(-127, q0, m), q = fma(e, r, q0) with
// r = fl(1/127).  For the divisor 127 this sequence returns the correctly
// rounded quotient for every binary32 significand (checked exhaustively over
// all 2^23 of them; scaling by a power of two carries the result to every
// exponent at which nothing underflows, hence the range test).  Outside the
// range, and for zero, the IEEE division above is used.
__device__ __forceinline__ float scale_from_maximum_fast(float maximum) {
    if (maximum >= 8.0779356694631609e-28f && maximum <= 1.2676506002282294e30f) {
        constexpr float kReciprocal = 1.0f / 127.0f;
        const float q0 = __fmul_rn(maximum, kReciprocal);
        const float e = __fmaf_rn(-127.0f, q0, maximum);
        return __fmaf_rn(e, kReciprocal, q0);
    }
    return scale_from_maximum(maximum);
}

// Round-half-even of a quotient to an integer in [-127,127], NaN -> 0
// (Bfp8Quantization.cs:220-227), kept in "biased" form: the returned float is
// code + 1.5 * 2^23, whose low mantissa byte is the two's-complement int8
// code.  Adding 1.5 * 2^23 performs the binary32 round-to-nearest-even to an
// integer exactly for |q| <= 2^22; the quotient is clamped first, which
// commutes with the rounding because the bounds are integers.  Everything
// stays on the FP32/integer pipes (no F2I / I2F conversions).
constexpr float kRoundMagic = 12582912.0f;

__device__ __forceinline__ float biased_code(float quotient) {
    float q = (quotient == quotient) ? quotient : 0.0f;
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return __fadd_rn(q, kRoundMagic);
}

__device__ __forceinline__ float biased_code_of(float value, float scale) {
    return biased_code(__fdiv_rn(value, scale));
}

// The same result without an IEEE division per value.  The rounded code only
// depends on which integer the quotient is nearest to, so an approximate
// quotient q0 = value * (1/scale) decides it whenever q0 is not within a guard
// band of a rounding boundary (a half-integer).  Error budget at |q| <= 127:
// approximate reciprocal (<= 1 ulp) and the multiply give |q0 - value/scale|
// <= 127 * 1.8e-7 = 2.3e-5, rounding the true quotient to binary32 moves it by
// <= 3.9e-6; the band is 1e-4.  Inside the band, for NaN / Inf, and for scales
// outside [2^-100, 2^100] (where the approximate reciprocal would flush or
// overflow) the exact division is used.  Rare: ~2e-4 of the values.
struct BlockScale {
    float scale;
    float inverse;
    bool fast;
};

__device__ __forceinline__ BlockScale block_scale(float scale) {
    BlockScale b;
    b.scale = scale;
    b.fast = scale >= 7.8886090522101181e-31f && scale <= 1.2676506002282294e30f;
    float inverse;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inverse) : "f"(scale));
    b.inverse = inverse;
    return b;
}

__device__ __forceinline__ float biased_code_of(float value, const BlockScale& b) {
    const float raw = __fmul_rn(value, b.inverse);
    const float q = fminf(fmaxf(raw, -127.0f), 127.0f);
    const float t = __fadd_rn(q, kRoundMagic);
    const float distance = fabsf(__fadd_rn(raw, -__fadd_rn(t, -kRoundMagic)));
    if (b.fast && distance < 0.4999f) return t;
    return biased_code_of(value, b.scale);
}

// Four values of one block at once: one decision for the (rare) exact path.
__device__ __forceinline__ void biased_codes_of(const float4& x, const BlockScale& b,
                                                float& t0, float& t1, float& t2, float& t3) {
    const float r0 = __fmul_rn(x.x, b.inverse), r1 = __fmul_rn(x.y, b.inverse),
                r2 = __fmul_rn(x.z, b.inverse), r3 = __fmul_rn(x.w, b.inverse);
    t0 = __fadd_rn(r0, kRoundMagic);
    t1 = __fadd_rn(r1, kRoundMagic);
    t2 = __fadd_rn(r2, kRoundMagic);
    t3 = __fadd_rn(r3, kRoundMagic);
    // The scale is the block maximum / 127, so |r| <= 127.00003 and no clamp
    // is needed here; a NaN or Inf value makes its distance NaN, fails the
    // comparison and takes the exact path.
    const float d0 = fabsf(__fadd_rn(r0, -__fadd_rn(t0, -kRoundMagic)));
    const float d1 = fabsf(__fadd_rn(r1, -__fadd_rn(t1, -kRoundMagic)));
    const float d2 = fabsf(__fadd_rn(r2, -__fadd_rn(t2, -kRoundMagic)));
    const float d3 = fabsf(__fadd_rn(r3, -__fadd_rn(t3, -kRoundMagic)));
    const bool ok = b.fast && (d0 < 0.4999f) && (d1 < 0.4999f) && (d2 < 0.4999f) && (d3 < 0.4999f);
    if (!ok) {
        t0 = biased_code_of(x.x, b.scale);
        t1 = biased_code_of(x.y, b.scale);
        t2 = biased_code_of(x.z, b.scale);
        t3 = biased_code_of(x.w, b.scale);
    }
}

// The code as an integer-valued float (for decode = code * scale).
__device__ __forceinline__ float code_value(float biased) {
    return __fadd_rn(biased, -kRoundMagic);
}

__device__ __forceinline__ signed char code_byte(float biased) {
    return static_cast<signed char>(__float_as_uint(biased) & 0xffu);
}

// Four biased codes -> four int8 in one word (element 0 in the low byte).
__device__ __forceinline__ unsigned pack_codes(float t0, float t1, float t2, float t3) {
    unsigned lo = __byte_perm(__float_as_uint(t0), __float_as_uint(t1), 0x0040);
    unsigned hi = __byte_perm(__float_as_uint(t2), __float_as_uint(t3), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

// int8 byte `index` of `word` -> float, exactly, on the integer/FP32 pipes
// only: (byte ^ 0x80) placed in the mantissa of 2^23 * 1.5 and the bias
// subtracted.  `biased` must already be word ^ 0x80808080.
__device__ __forceinline__ float byte_to_float(unsigned biased, int index) {
    unsigned bits = __byte_perm(biased, 0x4B400000u, 0x7650 + index);   // 0x4B4000bb
    return __fadd_rn(__uint_as_float(bits), -12583040.0f);              // -(1.5*2^23 + 128)
}

__device__ __forceinline__ bool is_non_finite(float v) {
    return (__float_as_uint(v) & 0x7fffffffu) >= 0x7f800000u;
}

__device__ __forceinline__ float4 load_f4(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
// Streaming load: read once, do not keep in L1.
__device__ __forceinline__ float4 load_f4_stream(const float* p) {
    return __ldcs(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ void store_f4(float* p, float4 v) {
    *reinterpret_cast<float4*>(p) = v;
}

__device__ __forceinline__ double warp_sum(double v) {
    #pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// Adds every thread's `partial` into *target with one atomic per CTA.
// Must be reached by all threads of the CTA.
__device__ __forceinline__ void cta_accumulate(double partial, double* target) {
    __shared__ double warp_partials[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    partial = warp_sum(partial);
    if (lane == 0) warp_partials[warp] = partial;
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        double v = lane < warps ? warp_partials[lane] : 0.0;
        v = warp_sum(v);
        if (lane == 0 && v != 0.0) atomicAdd(target, v);
    }
}

// Same, but the CTA's total goes to partials[blockIdx.x] (no atomics), for a
// fixed-order second stage.
__device__ __forceinline__ void cta_store_partial(double partial, double* partials) {
    __shared__ double warp_partials_det[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    partial = warp_sum(partial);
    if (lane == 0) warp_partials_det[warp] = partial;
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        double v = lane < warps ? warp_partials_det[lane] : 0.0;
        v = warp_sum(v);
        if (lane == 0) partials[blockIdx.x] = v;
    }
}

#endif  // __CUDACC__

}  // namespace ngb
