// BFP8 block codec kernels (signed int8 payload + one fp32 scale per block).
//
// Arithmetic contract (NNtrain.Core/Tensors/Bfp8Quantization.cs:188-274):
//   scale = max|x| == 0 ? 1 : max|x| / 127        one IEEE division
//   code  = clamp(round_half_even(x / scale), +-127)
//   x'    = code * scale                           one IEEE multiply
//
// Layout of the fast path (blocks of 32, 64 or 128 values): a warp owns a
// tile of 512 consecutive values per step.  Every lane issues four
// independent 128-bit loads (the warp reads 4 x 512 contiguous bytes), the
// block maximum is a shuffle-xor reduction over the block's lanes
// (block / 4 of them), codes are packed four to a 32-bit word so each warp
// store instruction writes one full 128-byte line of payload, and the 4..16
// scales of the tile are gathered into the low lanes and written with one
// store.  HBM traffic is the algorithmic minimum: 4 B read, 1 B + 4/block B
// written per value (+4 B when the decoded value is written back).
#pragma once

#include "common.cuh"

namespace ngb {

enum EncodeFlags : int {
    kEncWriteBack = 1,     // write code*scale as fp32 (may alias the source)
    kEncSquares = 2,       // accumulate sum of (double)(code*scale)^2
    kEncFiniteFlag = 4,    // set *finite_status = 1 when any input is NaN/Inf
    kEncNanScale = 8,      // non-finite block -> scale bits 0x7fffffff, payload 0
                           // (NNtrain.Cuda/native/gradient_collectives.cu:49-58)
};

constexpr int kEncodeUnroll = 4;
constexpr int kWarpTile = 128 * kEncodeUnroll;   // values per warp per step

template <int kLanes>
__device__ __forceinline__ float group_max(float v) {
    #pragma unroll
    for (int offset = kLanes / 2; offset > 0; offset >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

template <int kLanes>
__device__ __forceinline__ int group_or(int v) {
    #pragma unroll
    for (int offset = kLanes / 2; offset > 0; offset >>= 1)
        v |= __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// One block handled by one warp with scalar accesses: ragged tails, unaligned
// pointers and block sizes without a fast path.  Two passes over the block;
// the second one hits L1/L2.
template <int kFlags>
__device__ __forceinline__ void encode_block_scalar(
    const float* __restrict__ source, float* writeback, signed char* __restrict__ payload,
    float* __restrict__ scales, long long start, long long end, long long scale_index,
    int lane, double& squares, int& non_finite) {
    float maximum = 0.0f;
    int bad = 0;
    for (long long i = start + lane; i < end; i += 32) {
        const float v = source[i];
        const bool nf = is_non_finite(v);
        if ((kFlags & (kEncFiniteFlag | kEncNanScale)) && nf) bad = 1;
        maximum = fmaxf(maximum, (kFlags & kEncNanScale) && nf ? 0.0f : fabsf(v));
    }
    maximum = group_max<32>(maximum);
    if (kFlags & (kEncFiniteFlag | kEncNanScale)) bad = __any_sync(0xffffffffu, bad);
    if (kFlags & kEncFiniteFlag) non_finite |= bad;
    float scale = scale_from_maximum(maximum);
    const bool poison = (kFlags & kEncNanScale) && bad;
    if (poison) scale = __uint_as_float(0x7fffffffu);
    if (lane == 0) scales[scale_index] = scale;
    const BlockScale divisor = block_scale(scale);
    for (long long i = start + lane; i < end; i += 32) {
        const float t = poison ? kRoundMagic : biased_code_of(source[i], divisor);
        payload[i] = code_byte(t);
        if (kFlags & (kEncWriteBack | kEncSquares)) {
            const float decoded = __fmul_rn(code_value(t), scale);
            if (kFlags & kEncWriteBack) writeback[i] = decoded;
            if (kFlags & kEncSquares) squares += static_cast<double>(decoded) * static_cast<double>(decoded);
        }
    }
}

// Lanes of the warp that share a block of kLanes * 4 values with this lane.
template <int kLanes>
__device__ __forceinline__ unsigned group_mask(int lane) {
    if constexpr (kLanes == 32) {
        return 0xffffffffu;
    } else {
        return ((1u << kLanes) - 1u) << (lane & ~(kLanes - 1));
    }
}

template <int kLanes>
__device__ __forceinline__ float group_max_masked(unsigned mask, float v) {
    #pragma unroll
    for (int offset = kLanes / 2; offset > 0; offset >>= 1)
        v = fmaxf(v, __shfl_xor_sync(mask, v, offset));
    return v;
}

// Maximum of an unsigned value over the block's lanes: one hardware
// reduction when the block is the whole warp, a shuffle butterfly for 8- and
// 16-lane blocks (a reduction with a partial mask costs one pass per distinct
// mask in the warp).
template <int kLanes>
__device__ __forceinline__ unsigned group_max_bits(unsigned mask, unsigned v) {
    if constexpr (kLanes == 32) {
        return __reduce_max_sync(0xffffffffu, v);
    } else {
        #pragma unroll
        for (int offset = kLanes / 2; offset > 0; offset >>= 1)
            v = max(v, __shfl_xor_sync(mask, v, offset));
        return v;
    }
}

// Fast path.  Requires: source (and writeback) 16-byte aligned, payload
// 4-byte aligned.  `length` may be ragged: the last partial warp tile falls
// back to encode_block_scalar.
//
// Per row of 128 values each lane holds four.  The block maximum is one
// integer max-reduction over the block's lanes on the bit patterns (|x| >= 0
// orders like an unsigned integer).  A lane whose four values contain a NaN
// or Inf (their sum is then not finite) contributes 0xffffffff instead, so a
// reduced value >= 0x7f800000 marks a block that needs the exact, per-value
// treatment of non-finite input; finite blocks never pay for it.
template <int kBlock, int kFlags>
__global__ void __launch_bounds__(kThreads)
bfp8_encode_blocks_kernel(const float* __restrict__ source, float* writeback,
                          signed char* __restrict__ payload, float* __restrict__ scales,
                          long long length, double* squared_sum, int* finite_status) {
    static_assert(kBlock == 32 || kBlock == 64 || kBlock == 128, "fast path block sizes");
    constexpr int kLanesPerBlock = kBlock / 4;

    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long tiles = (length + kWarpTile - 1) / kWarpTile;
    const unsigned mask = group_mask<kLanesPerBlock>(lane);
    const bool leader = (lane & (kLanesPerBlock - 1)) == 0;

    double squares = 0.0;
    int non_finite = 0;

    for (long long tile = warp; tile < tiles; tile += warps) {
        const long long base = tile * kWarpTile;
        if (base + kWarpTile <= length) {
            const float* in = source + base + lane * 4;
            signed char* out = payload + base + lane * 4;
            float* back = (kFlags & kEncWriteBack) ? writeback + base + lane * 4 : nullptr;
            float* scale_out = scales + base / kBlock + lane / kLanesPerBlock;
            float4 v[kEncodeUnroll];
            #pragma unroll
            for (int j = 0; j < kEncodeUnroll; ++j) v[j] = load_f4_stream(in + j * 128);

            #pragma unroll
            for (int j = 0; j < kEncodeUnroll; ++j) {
                const float4 x = v[j];
                const float lane_max = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
                const float lane_sum = __fadd_rn(__fadd_rn(x.x, x.y), __fadd_rn(x.z, x.w));
                const unsigned lane_bits = fabsf(lane_sum) < __int_as_float(0x7f800000)
                                               ? __float_as_uint(lane_max) : 0xffffffffu;
                const unsigned block_bits = group_max_bits<kLanesPerBlock>(mask, lane_bits);
                float scale;
                float t0, t1, t2, t3;
                if (block_bits < 0x7f800000u) {
                    scale = scale_from_maximum_fast(__uint_as_float(block_bits));
                    biased_codes_of(x, block_scale(scale), t0, t1, t2, t3);
                } else {
                    // a NaN / Inf in the block, or four finite values whose sum
                    // overflowed: the reference's per-value rules
                    const bool n0 = is_non_finite(x.x), n1 = is_non_finite(x.y),
                               n2 = is_non_finite(x.z), n3 = is_non_finite(x.w);
                    const int bad = n0 | n1 | n2 | n3;
                    float m;
                    if (kFlags & kEncNanScale) {
                        m = fmaxf(fmaxf(n0 ? 0.0f : fabsf(x.x), n1 ? 0.0f : fabsf(x.y)),
                                  fmaxf(n2 ? 0.0f : fabsf(x.z), n3 ? 0.0f : fabsf(x.w)));
                    } else {
                        m = fmaxf(fmaxf(fmaxf(0.0f, fabsf(x.x)), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
                    }
                    if (kFlags & kEncFiniteFlag) non_finite |= bad;
                    m = group_max_masked<kLanesPerBlock>(mask, m);
                    scale = scale_from_maximum(m);
                    bool poison = false;
                    if (kFlags & kEncNanScale) {
                        poison = __reduce_or_sync(mask, static_cast<unsigned>(bad)) != 0;
                        if (poison) scale = __uint_as_float(0x7fffffffu);
                    }
                    if (poison) {
                        t0 = t1 = t2 = t3 = kRoundMagic;
                    } else {
                        t0 = biased_code_of(x.x, scale);
                        t1 = biased_code_of(x.y, scale);
                        t2 = biased_code_of(x.z, scale);
                        t3 = biased_code_of(x.w, scale);
                    }
                }
                *reinterpret_cast<unsigned*>(out + j * 128) = pack_codes(t0, t1, t2, t3);
                if (leader) scale_out[j * (128 / kBlock)] = scale;
                if (kFlags & (kEncWriteBack | kEncSquares)) {
                    float4 d;
                    d.x = __fmul_rn(code_value(t0), scale);
                    d.y = __fmul_rn(code_value(t1), scale);
                    d.z = __fmul_rn(code_value(t2), scale);
                    d.w = __fmul_rn(code_value(t3), scale);
                    if (kFlags & kEncWriteBack) store_f4(back + j * 128, d);
                    if (kFlags & kEncSquares) {
                        squares += static_cast<double>(d.x) * static_cast<double>(d.x);
                        squares += static_cast<double>(d.y) * static_cast<double>(d.y);
                        squares += static_cast<double>(d.z) * static_cast<double>(d.z);
                        squares += static_cast<double>(d.w) * static_cast<double>(d.w);
                    }
                }
            }
        } else {
            for (long long start = base; start < length; start += kBlock) {
                const long long end = start + kBlock < length ? start + kBlock : length;
                encode_block_scalar<kFlags>(source, writeback, payload, scales, start, end,
                                            start / kBlock, lane, squares, non_finite);
            }
        }
    }
    if (kFlags & kEncFiniteFlag) {
        if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(finite_status, 1);
    }
    if (kFlags & kEncSquares) cta_accumulate(squares, squared_sum);
}

// Any block size up to kMaxWarpBlock, any alignment: one warp per block.
constexpr long long kMaxWarpBlock = 8192;

template <int kFlags>
__global__ void __launch_bounds__(kThreads)
bfp8_encode_warp_per_block_kernel(const float* __restrict__ source, float* writeback,
                                  signed char* __restrict__ payload, float* __restrict__ scales,
                                  long long length, long long block, long long block_count,
                                  double* squared_sum, int* finite_status) {
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    double squares = 0.0;
    int non_finite = 0;
    for (long long b = warp; b < block_count; b += warps) {
        const long long start = b * block;
        const long long end = start + block < length ? start + block : length;
        encode_block_scalar<kFlags>(source, writeback, payload, scales, start, end, b, lane,
                                    squares, non_finite);
    }
    if (kFlags & kEncFiniteFlag) {
        if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(finite_status, 1);
    }
    if (kFlags & kEncSquares) cta_accumulate(squares, squared_sum);
}

// ---- large blocks and tensor-wide: maximum pass + payload pass -------------
// Pass 1: maximum of |x| over [0,length) of each "segment" (a block, or the
// whole tensor), accumulated with atomicMax on the float's bit pattern, which
// orders like the value for non-negative floats.  The slot must be zeroed
// first.  Optionally raises the finite flag
// (NNtrain.Cuda/native/tensor_kernels.cu:988-999 does this with one atomic per
// element; here it is one per CTA).
template <bool kFinite>
__global__ void __launch_bounds__(kThreads)
bfp8_segment_max_kernel(const float* __restrict__ source, long long length, long long block,
                        unsigned* __restrict__ maximum_bits, int* finite_status,
                        int ctas_per_segment) {
    __shared__ float warp_max[kWarpsPerCta];
    const long long segment = blockIdx.x / ctas_per_segment;
    const int part = blockIdx.x % ctas_per_segment;
    const long long start = segment * block;
    const long long end = start + block < length ? start + block : length;
    const long long span = end - start;
    const float* base = source + start;
    float m = 0.0f;
    int bad = 0;
    // 128-bit body when the segment start is 16-byte aligned, scalar edges.
    const bool aligned = (reinterpret_cast<std::uintptr_t>(base) & 15u) == 0;
    const long long vectors = aligned ? span / 4 : 0;
    const long long stride = static_cast<long long>(ctas_per_segment) * kThreads;
    for (long long i = static_cast<long long>(part) * kThreads + threadIdx.x; i < vectors; i += stride) {
        const float4 x = load_f4(base + i * 4);
        if (kFinite) bad |= is_non_finite(x.x) | is_non_finite(x.y) | is_non_finite(x.z) | is_non_finite(x.w);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
    }
    for (long long i = vectors * 4 + static_cast<long long>(part) * kThreads + threadIdx.x; i < span; i += stride) {
        const float x = base[i];
        if (kFinite) bad |= is_non_finite(x);
        m = fmaxf(m, fabsf(x));
    }
    m = group_max<32>(m);
    if (kFinite && __any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(finite_status, 1);
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        #pragma unroll
        for (int w = 1; w < kWarpsPerCta; ++w) m = fmaxf(m, warp_max[w]);
        // A NaN maximum cannot occur (fmaxf drops NaN); +Inf orders above
        // every finite pattern, as it must.
        if (m > 0.0f) atomicMax(maximum_bits + segment, __float_as_uint(m));
    }
}

// Pass 2: payload (and optional write-back / squares) from the raw maxima
// left in `maxima` by pass 1.  When `finite_status` is given and non-zero
// nothing is written (tensor_kernels.cu:1023-1042: a non-finite gradient
// publishes no payload and no decode).
template <int kFlags>
__global__ void __launch_bounds__(kThreads)
bfp8_segment_payload_kernel(const float* __restrict__ source, float* writeback,
                            signed char* __restrict__ payload, const float* __restrict__ maxima,
                            long long length, long long block, const int* finite_status,
                            double* squared_sum, int ctas_per_segment) {
    const bool skip = finite_status != nullptr && *finite_status != 0;
    double squares = 0.0;
    if (!skip) {
        const long long segment = blockIdx.x / ctas_per_segment;
        const int part = blockIdx.x % ctas_per_segment;
        const long long start = segment * block;
        const long long end = start + block < length ? start + block : length;
        const long long span = end - start;
        const float scale = scale_from_maximum(maxima[segment]);
        const BlockScale divisor = block_scale(scale);
        const float* base = source + start;
        signed char* out = payload + start;
        float* back = (kFlags & kEncWriteBack) ? writeback + start : nullptr;
        const bool aligned = ((reinterpret_cast<std::uintptr_t>(base) & 15u) == 0) &&
                             ((reinterpret_cast<std::uintptr_t>(out) & 3u) == 0) &&
                             (!(kFlags & kEncWriteBack) || (reinterpret_cast<std::uintptr_t>(back) & 15u) == 0);
        const long long vectors = aligned ? span / 4 : 0;
        const long long stride = static_cast<long long>(ctas_per_segment) * kThreads;
        for (long long i = static_cast<long long>(part) * kThreads + threadIdx.x; i < vectors; i += stride) {
            const float4 x = load_f4_stream(base + i * 4);
            const float t0 = biased_code_of(x.x, divisor), t1 = biased_code_of(x.y, divisor),
                        t2 = biased_code_of(x.z, divisor), t3 = biased_code_of(x.w, divisor);
            *reinterpret_cast<unsigned*>(out + i * 4) = pack_codes(t0, t1, t2, t3);
            if (kFlags & (kEncWriteBack | kEncSquares)) {
                float4 d;
                d.x = __fmul_rn(code_value(t0), scale);
                d.y = __fmul_rn(code_value(t1), scale);
                d.z = __fmul_rn(code_value(t2), scale);
                d.w = __fmul_rn(code_value(t3), scale);
                if (kFlags & kEncWriteBack) store_f4(back + i * 4, d);
                if (kFlags & kEncSquares) {
                    squares += static_cast<double>(d.x) * static_cast<double>(d.x);
                    squares += static_cast<double>(d.y) * static_cast<double>(d.y);
                    squares += static_cast<double>(d.z) * static_cast<double>(d.z);
                    squares += static_cast<double>(d.w) * static_cast<double>(d.w);
                }
            }
        }
        for (long long i = vectors * 4 + static_cast<long long>(part) * kThreads + threadIdx.x; i < span; i += stride) {
            const float t = biased_code_of(base[i], divisor);
            out[i] = code_byte(t);
            if (kFlags & (kEncWriteBack | kEncSquares)) {
                const float d = __fmul_rn(code_value(t), scale);
                if (kFlags & kEncWriteBack) back[i] = d;
                if (kFlags & kEncSquares) squares += static_cast<double>(d) * static_cast<double>(d);
            }
        }
    }
    if (kFlags & kEncSquares) cta_accumulate(squares, squared_sum);
}

// ---- decode ----------------------------------------------------------------
// Fast path: payload 4-byte aligned, destination 16-byte aligned.  Each lane
// reads one 32-bit payload word and writes one 128-bit fp32 vector; eight
// independent rows per step keep the loads in flight.
constexpr int kDecodeUnroll = 8;

template <int kShift>   // block = 1 << kShift, or kShift < 0: runtime block
__global__ void __launch_bounds__(kThreads)
bfp8_decode_blocks_kernel(const signed char* __restrict__ payload, const float* __restrict__ scales,
                          float* __restrict__ destination, long long length, long long block) {
    const long long words = length / 4;
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const unsigned* in = reinterpret_cast<const unsigned*>(payload);
    long long w = thread;
    for (; w + (kDecodeUnroll - 1) * threads < words; w += kDecodeUnroll * threads) {
        unsigned word[kDecodeUnroll];
        float scale[kDecodeUnroll];
        #pragma unroll
        for (int j = 0; j < kDecodeUnroll; ++j) {
            const long long at = w + j * threads;
            word[j] = __ldcs(in + at);
            scale[j] = __ldg(scales + (kShift >= 0 ? (at * 4) >> (kShift >= 0 ? kShift : 0) : (at * 4) / block));
        }
        #pragma unroll
        for (int j = 0; j < kDecodeUnroll; ++j) {
            const unsigned biased = word[j] ^ 0x80808080u;
            float4 d;
            d.x = __fmul_rn(byte_to_float(biased, 0), scale[j]);
            d.y = __fmul_rn(byte_to_float(biased, 1), scale[j]);
            d.z = __fmul_rn(byte_to_float(biased, 2), scale[j]);
            d.w = __fmul_rn(byte_to_float(biased, 3), scale[j]);
            __stcs(reinterpret_cast<float4*>(destination + (w + j * threads) * 4), d);
        }
    }
    for (; w < words; w += threads) {
        const unsigned biased = __ldcs(in + w) ^ 0x80808080u;
        const float scale = __ldg(scales + (kShift >= 0 ? (w * 4) >> (kShift >= 0 ? kShift : 0) : (w * 4) / block));
        float4 d;
        d.x = __fmul_rn(byte_to_float(biased, 0), scale);
        d.y = __fmul_rn(byte_to_float(biased, 1), scale);
        d.z = __fmul_rn(byte_to_float(biased, 2), scale);
        d.w = __fmul_rn(byte_to_float(biased, 3), scale);
        __stcs(reinterpret_cast<float4*>(destination + w * 4), d);
    }
    // ragged tail (< 4 values)
    for (long long i = words * 4 + thread; i < length; i += threads) {
        const float scale = scales[kShift >= 0 ? i >> (kShift >= 0 ? kShift : 0) : i / block];
        destination[i] = __fmul_rn(static_cast<float>(payload[i]), scale);
    }
}

// ---- host-side launchers (bfp8_codec.cu) -------------------------------------
// Encodes `length` values in blocks of `block` (block >= length: one block).
// `flags` is a combination of EncodeFlags; `scales` must hold
// ceil(length / block) floats.  Picks the fast path when block is 32/64/128
// and the pointers are aligned; otherwise the warp-per-block or the
// three-pass segment path.  When `skip_if_non_finite` is set together with
// kEncFiniteFlag on the segment path, a non-finite input publishes nothing.
cudaError_t launch_bfp8_encode(const float* source, float* writeback, signed char* payload,
                               float* scales, long long length, long long block, int flags,
                               double* squared_sum, int* finite_status, bool skip_if_non_finite,
                               cudaStream_t stream);

cudaError_t launch_bfp8_decode(const signed char* payload, const float* scales, float* destination,
                               long long length, long long block, cudaStream_t stream);

}  // namespace ngb
