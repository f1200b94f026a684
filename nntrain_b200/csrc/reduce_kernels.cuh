// Reduction kernels of the gradient path.
//
//   bfp8_reduce_reencode_kernel  N encoded shards -> fp32 accumulate in rank
//       order -> x reduction_scale -> re-encode -> M destinations.  The
//       pointers may be local or peer (NVLink-mapped) device memory: with
//       peer pointers one launch is the reduce-scatter, the owner's
//       arithmetic and the all-gather of the owned shard.
//   bfp8_sum_to_f32_kernel       N encoded inputs -> fp32 sum (no re-encode):
//       the block transport of the reference's bucketed reducer
//       (NNtrain.Cuda/native/gradient_collectives.cu:92-129).
//   bf16_reduce_kernel           N bf16 inputs -> fp32 accumulate -> fp32
//       and/or bf16 outputs (gradient_collectives.cu:62-90 for N = 2).
//
// Arithmetic: every product payload*scale, every add and the final multiply
// by reduction_scale is a separate IEEE binary32 operation (__fmul_rn /
// __fadd_rn), summed left to right in ascending rank order, so every rank
// that repeats the computation gets identical bits.
#pragma once

#include "common.cuh"
#include "bfp8_kernels.cuh"

namespace ngb {

constexpr int kMaxRanks = 16;

struct EncodedShards {                    // passed by value to the kernels
    const signed char* payload[kMaxRanks];
    const float* scales[kMaxRanks];
    signed char* out_payload[kMaxRanks];
    float* out_scales[kMaxRanks];
    int inputs;                           // N
    int outputs;                          // M
};

__device__ __forceinline__ bool bad_scale(float s) {
    return !(s > 0.0f) || is_non_finite(s);
}

// Decodes 16 int8 codes (one uint4) times `scale` and adds them into acc[16].
template <bool kFirst>
__device__ __forceinline__ void accumulate16(const uint4& words, float scale, float (&acc)[16]) {
    const unsigned w[4] = {words.x ^ 0x80808080u, words.y ^ 0x80808080u,
                           words.z ^ 0x80808080u, words.w ^ 0x80808080u};
    #pragma unroll
    for (int q = 0; q < 4; ++q) {
        #pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float term = __fmul_rn(byte_to_float(w[q], b), scale);
            acc[q * 4 + b] = kFirst ? term : __fadd_rn(acc[q * 4 + b], term);
        }
    }
}

// Fast path: every lane owns 16 consecutive values (one 128-bit payload load
// per input rank, one 128-bit payload store per destination); a block of
// kBlock values is kBlock/16 adjacent lanes.  A warp step covers 512 values.
// Requirements: all payload pointers 16-byte aligned, first_value a multiple
// of 16; the ragged end (< 512 values) is done with scalar accesses by the
// same kernel, as is everything when vector_ok is false.
// kRanks > 0: number of inputs known at compile time.  The loads of the NEXT
// tile are issued before the current tile's arithmetic, so every warp always
// has one tile of every rank in flight: with peer pointers that hides the
// NVLink round trip even when only a few CTAs are given to the kernel.
// kRanks == 0: runtime count, no prefetch.
template <int kRanks>
struct ShardTile {
    uint4 words[kRanks > 0 ? kRanks : 1];
    float scale[kRanks > 0 ? kRanks : 1];
};

template <int kBlock, int kRanks>
__device__ __forceinline__ void load_shard_tile(const EncodedShards& shards, long long base, int lane,
                                                ShardTile<kRanks>& tile) {
    const long long at = base + lane * 16;
    const long long block_index = at / kBlock;
    #pragma unroll
    for (int k = 0; k < kRanks; ++k) {
        tile.words[k] = __ldcs(reinterpret_cast<const uint4*>(shards.payload[k] + at));
        tile.scale[k] = __ldcs(shards.scales[k] + block_index);
    }
}

// Re-encodes acc[16] (the rank-ordered sums): x reduction_scale, block scale,
// 16 codes packed into one 128-bit word; optional sum of squares of the
// decoded result.
template <int kBlock, bool kSquares>
__device__ __forceinline__ void reencode16(float (&acc)[16], float reduction_scale, double& squares,
                                           int& non_finite, uint4& packed, float& scale) {
    constexpr int kLanesPerBlock = kBlock / 16;
    float m = 0.0f;
    #pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc[i] = __fmul_rn(reduction_scale, acc[i]);
        non_finite |= is_non_finite(acc[i]);
        m = fmaxf(m, fabsf(acc[i]));
    }
    m = group_max<kLanesPerBlock>(m);
    // a NaN sum is dropped by fmaxf and an Inf one gives scale = Inf; both are
    // flagged above and take the exact per-value path inside biased_codes_of
    scale = scale_from_maximum_fast(m);
    const BlockScale divisor = block_scale(scale);
    float t[16];
    #pragma unroll
    for (int i = 0; i < 16; i += 4)
        biased_codes_of(make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]), divisor,
                        t[i], t[i + 1], t[i + 2], t[i + 3]);
    packed.x = pack_codes(t[0], t[1], t[2], t[3]);
    packed.y = pack_codes(t[4], t[5], t[6], t[7]);
    packed.z = pack_codes(t[8], t[9], t[10], t[11]);
    packed.w = pack_codes(t[12], t[13], t[14], t[15]);
    if (kSquares) {
        #pragma unroll
        for (int i = 0; i < 16; ++i) {
            const double d = static_cast<double>(__fmul_rn(code_value(t[i]), scale));
            squares += d * d;
        }
    }
}

// Re-encodes acc[16] and stores payload + scale to every destination.
template <int kBlock, bool kSquares>
__device__ __forceinline__ void reencode_and_store(const EncodedShards& shards, long long base, int lane,
                                                   float (&acc)[16], float reduction_scale,
                                                   double& squares, int& non_finite) {
    constexpr int kLanesPerBlock = kBlock / 16;
    const long long at = base + lane * 16;
    uint4 packed;
    float scale;
    reencode16<kBlock, kSquares>(acc, reduction_scale, squares, non_finite, packed, scale);
    // Gather the tile's scales (one per kLanesPerBlock lanes) into the low
    // lanes so each destination gets one contiguous store.
    constexpr int kScalesPerTile = 512 / kBlock;
    const float routed = __shfl_sync(0xffffffffu, scale, (lane * kLanesPerBlock) & 31);
    for (int d = 0; d < shards.outputs; ++d) {
        *reinterpret_cast<uint4*>(shards.out_payload[d] + at) = packed;
        if (lane < kScalesPerTile) shards.out_scales[d][base / kBlock + lane] = routed;
    }
}

// One (possibly partial) tile with scalar accesses: one block at a time, the
// warp's lanes stride over it.
template <int kBlock, bool kSquares>
__device__ __forceinline__ void reduce_tile_scalar(const EncodedShards& shards, int ranks, long long base,
                                                   long long end_value, int lane, float reduction_scale,
                                                   double& squares, int& non_finite) {
    const long long tile_end = base + 512 < end_value ? base + 512 : end_value;
    for (long long start = base; start < tile_end; start += kBlock) {
        const long long stop = start + kBlock < end_value ? start + kBlock : end_value;
        const long long block_index = start / kBlock;
        constexpr int kPerLane = kBlock / 32;
        float value[kPerLane];
        float m = 0.0f;
        #pragma unroll
        for (int e = 0; e < kPerLane; ++e) {
            const long long i = start + lane + e * 32;
            float sum = 0.0f;
            if (i < stop) {
                for (int k = 0; k < ranks; ++k) {
                    const float s = shards.scales[k][block_index];
                    non_finite |= bad_scale(s);
                    const float term = __fmul_rn(static_cast<float>(shards.payload[k][i]), s);
                    sum = k == 0 ? term : __fadd_rn(sum, term);
                }
                sum = __fmul_rn(reduction_scale, sum);
                non_finite |= is_non_finite(sum);
                m = fmaxf(m, fabsf(sum));
            }
            value[e] = sum;
        }
        m = group_max<32>(m);
        const float scale = scale_from_maximum(m);
        #pragma unroll
        for (int e = 0; e < kPerLane; ++e) {
            const long long i = start + lane + e * 32;
            if (i < stop) {
                const float t = biased_code_of(value[e], scale);
                if (kSquares) {
                    const double d = static_cast<double>(__fmul_rn(code_value(t), scale));
                    squares += d * d;
                }
                for (int d = 0; d < shards.outputs; ++d) shards.out_payload[d][i] = code_byte(t);
            }
        }
        if (lane == 0)
            for (int d = 0; d < shards.outputs; ++d) shards.out_scales[d][block_index] = scale;
    }
}

// At most 96 registers per thread: one 256-thread CTA per SM then leaves
// room for three CTAs of a codec kernel working on the neighbouring chunk.
template <int kBlock, int kRanks, bool kSquares>
__global__ void __maxnreg__(96)
bfp8_reduce_reencode_kernel(EncodedShards shards, long long first_value, long long end_value,
                            float reduction_scale, double* squared_sum, int* finite_status,
                            bool vector_ok) {
    static_assert(kBlock == 32 || kBlock == 64 || kBlock == 128, "fast path block sizes");
    const int ranks = kRanks > 0 ? kRanks : shards.inputs;
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long tiles = (end_value - first_value + 511) / 512;
    double squares = 0.0;
    int non_finite = 0;

    auto is_fast = [&](long long tile) {
        return vector_ok && tile < tiles && first_value + tile * 512 + 512 <= end_value;
    };

    if (kRanks > 0) {
        ShardTile<kRanks> current, next;
        long long tile = warp;
        bool current_fast = is_fast(tile);
        if (current_fast) load_shard_tile<kBlock, kRanks>(shards, first_value + tile * 512, lane, current);
        while (tile < tiles) {
            const long long following = tile + warps;
            const bool next_fast = is_fast(following);
            if (next_fast) load_shard_tile<kBlock, kRanks>(shards, first_value + following * 512, lane, next);
            const long long base = first_value + tile * 512;
            if (current_fast) {
                float acc[16];
                #pragma unroll
                for (int k = 0; k < kRanks; ++k) {
                    non_finite |= bad_scale(current.scale[k]);
                    if (k == 0) accumulate16<true>(current.words[k], current.scale[k], acc);
                    else accumulate16<false>(current.words[k], current.scale[k], acc);
                }
                reencode_and_store<kBlock, kSquares>(shards, base, lane, acc, reduction_scale, squares, non_finite);
            } else {
                reduce_tile_scalar<kBlock, kSquares>(shards, ranks, base, end_value, lane, reduction_scale,
                                                     squares, non_finite);
            }
            current = next;
            current_fast = next_fast;
            tile = following;
        }
    } else {
        for (long long tile = warp; tile < tiles; tile += warps) {
            const long long base = first_value + tile * 512;
            if (is_fast(tile)) {
                const long long at = base + lane * 16;
                const long long block_index = at / kBlock;
                float acc[16];
                for (int k = 0; k < ranks; ++k) {
                    const uint4 words = __ldcs(reinterpret_cast<const uint4*>(shards.payload[k] + at));
                    const float scale = __ldcs(shards.scales[k] + block_index);
                    non_finite |= bad_scale(scale);
                    if (k == 0) accumulate16<true>(words, scale, acc);
                    else accumulate16<false>(words, scale, acc);
                }
                reencode_and_store<kBlock, kSquares>(shards, base, lane, acc, reduction_scale, squares, non_finite);
            } else {
                reduce_tile_scalar<kBlock, kSquares>(shards, ranks, base, end_value, lane, reduction_scale,
                                                     squares, non_finite);
            }
        }
    }
    if (finite_status != nullptr) {
        if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(finite_status, 1);
    }
    if (kSquares) cta_accumulate(squares, squared_sum);
}

// ---- encode + all-gather: fp32 shard -> encoded shard in every arena -------------
// The publication of updated parameters after an optimizer step that is
// sharded over the ranks (every rank updates the fp32 master of its own shard
// only): rank r encodes shard r of its fp32 arena and stores payload + scales
// into EVERY rank's encoded arena with 128-bit (peer) stores -- the all-gather
// half of the fused all-reduce kernel with the encode in front of it.  Same
// tiling: a lane owns 16 consecutive values (four 128-bit fp32 loads, issued
// for the next tile before the current one is encoded), a warp 512.
struct Fp32Tile {
    float4 v[4];
};

__device__ __forceinline__ void load_fp32_tile(const float* __restrict__ source, long long base, int lane,
                                               Fp32Tile& tile) {
    const float* p = source + base + lane * 16;
    #pragma unroll
    for (int q = 0; q < 4; ++q) tile.v[q] = load_f4_stream(p + q * 4);
}

template <int kBlock>
__global__ void __launch_bounds__(kThreads)
bfp8_encode_to_all_kernel(const float* __restrict__ source, EncodedShards shards, long long first_value,
                          long long end_value, int* finite_status, bool vector_ok) {
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long tiles = (end_value - first_value + 511) / 512;
    double unused = 0.0;
    int non_finite = 0;
    auto is_fast = [&](long long tile) {
        return vector_ok && tile < tiles && first_value + tile * 512 + 512 <= end_value;
    };
    Fp32Tile current, next;
    long long tile = warp;
    bool current_fast = is_fast(tile);
    if (current_fast) load_fp32_tile(source, first_value + tile * 512, lane, current);
    while (tile < tiles) {
        const long long following = tile + warps;
        const bool next_fast = is_fast(following);
        if (next_fast) load_fp32_tile(source, first_value + following * 512, lane, next);
        const long long base = first_value + tile * 512;
        if (current_fast) {
            float acc[16];
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[q * 4 + 0] = current.v[q].x; acc[q * 4 + 1] = current.v[q].y;
                acc[q * 4 + 2] = current.v[q].z; acc[q * 4 + 3] = current.v[q].w;
            }
            // x * 1 is x: the shared tail re-encodes "reduction_scale * sum"
            reencode_and_store<kBlock, false>(shards, base, lane, acc, 1.0f, unused, non_finite);
        } else {
            // ragged end / unaligned pointers: one block at a time, scalar
            const long long tile_end = base + 512 < end_value ? base + 512 : end_value;
            for (long long start = base; start < tile_end; start += kBlock) {
                const long long stop = start + kBlock < end_value ? start + kBlock : end_value;
                constexpr int kPerLane = kBlock / 32;
                float value[kPerLane];
                float m = 0.0f;
                #pragma unroll
                for (int e = 0; e < kPerLane; ++e) {
                    const long long i = start + lane + e * 32;
                    value[e] = i < stop ? source[i] : 0.0f;
                    non_finite |= is_non_finite(value[e]);
                    m = fmaxf(m, fabsf(value[e]));
                }
                m = group_max<32>(m);
                const float scale = scale_from_maximum(m);
                #pragma unroll
                for (int e = 0; e < kPerLane; ++e) {
                    const long long i = start + lane + e * 32;
                    if (i < stop) {
                        const signed char code = code_byte(biased_code_of(value[e], scale));
                        for (int d = 0; d < shards.outputs; ++d) shards.out_payload[d][i] = code;
                    }
                }
                if (lane == 0)
                    for (int d = 0; d < shards.outputs; ++d) shards.out_scales[d][start / kBlock] = scale;
            }
        }
        current = next;
        current_fast = next_fast;
        tile = following;
    }
    if (finite_status != nullptr) {
        if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(finite_status, 1);
    }
}

// ---- asynchronous-copy variant ------------------------------------------------
// Same arithmetic; the inputs travel global -> shared memory with cp.async
// (16-byte payload pieces, 4-byte scales) through a ring of kStages tiles per
// warp.  Every lane copies exactly the bytes it will consume, so completion is
// tracked by the lane's own cp.async groups (wait_group is a scoreboard wait:
// nothing here can spin forever) and no cross-lane synchronisation is needed.
// The bytes in flight live in shared memory, not in registers: a single
// 256-thread CTA per SM keeps kStages - 1 tiles of every rank outstanding
// (N = 8: 3 x 4.6 KB per warp, 110 KB per SM), which rides out the longer
// NVLink / HBM latency seen while codec kernels saturate the memory system,
// and leaves most of the register file to those kernels.
__device__ __forceinline__ void async_copy_16(void* shared_destination, const void* source) {
    const unsigned address = static_cast<unsigned>(__cvta_generic_to_shared(shared_destination));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(address), "l"(source) : "memory");
}
__device__ __forceinline__ void async_copy_4(void* shared_destination, const void* source) {
    const unsigned address = static_cast<unsigned>(__cvta_generic_to_shared(shared_destination));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(address), "l"(source) : "memory");
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

template <int kRanks, int kStages, int kWarps>
constexpr size_t reduce_ring_bytes() {
    return static_cast<size_t>(kWarps) * kStages * kRanks * 32 * (sizeof(uint4) + sizeof(float));
}

// Dynamic shared memory that makes a CTA the only one its SM can hold: every
// CTA also reserves 1 KB for the system, and an SM has 228 KB, so a CTA asking
// for all but 512 bytes of the 227 KB a CTA may have leaves less than that
// 1 KB to anyone else.  An all-reduce kernel launched this way on G CTAs owns
// G SMs outright; the codec kernels of the neighbouring chunks get the other
// SMs and never share a memory request path with it.
constexpr size_t kExclusiveSharedBytes = 227 * 1024 - 512;

template <int kBlock, int kRanks, bool kSquares, int kStages, int kWarps>
__global__ void __launch_bounds__(kWarps * 32)
bfp8_reduce_reencode_async_kernel(EncodedShards shards, long long first_value, long long end_value,
                                  float reduction_scale, double* squared_sum, int* finite_status) {
    static_assert(kRanks > 0 && kStages >= 2, "compile-time rank count, at least two stages");
    extern __shared__ uint4 ring[];
    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    // payload ring: [warp][stage][rank][lane] uint4; scale ring behind it: same shape, float
    uint4* payload_ring = ring + static_cast<size_t>(warp_in_cta) * kStages * kRanks * 32;
    float* scale_ring = reinterpret_cast<float*>(ring + static_cast<size_t>(kWarps) * kStages * kRanks * 32) +
                        static_cast<size_t>(warp_in_cta) * kStages * kRanks * 32;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarps + warp_in_cta;
    const long long warps = static_cast<long long>(gridDim.x) * kWarps;
    const long long tiles = (end_value - first_value + 511) / 512;
    double squares = 0.0;
    int non_finite = 0;

    auto is_fast = [&](long long tile) { return tile < tiles && first_value + tile * 512 + 512 <= end_value; };
    auto issue = [&](long long tile, int stage) {
        if (is_fast(tile)) {
            const long long at = first_value + tile * 512 + lane * 16;
            const long long block_index = at / kBlock;
            #pragma unroll
            for (int k = 0; k < kRanks; ++k) {
                async_copy_16(payload_ring + (stage * kRanks + k) * 32 + lane, shards.payload[k] + at);
                async_copy_4(scale_ring + (stage * kRanks + k) * 32 + lane, shards.scales[k] + block_index);
            }
        }
        async_commit();      // one group per tile slot, empty when there is nothing to copy
    };

    #pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(warp + s * warps, s);
    int stage = 0;
    for (long long tile = warp; tile < tiles; tile += warps) {
        // The slot being refilled was consumed in the previous iteration.
        issue(tile + (kStages - 1) * warps, (stage + kStages - 1) % kStages);
        async_wait<kStages - 1>();
        const long long base = first_value + tile * 512;
        if (is_fast(tile)) {
            float acc[16];
            #pragma unroll
            for (int k = 0; k < kRanks; ++k) {
                const uint4 words = payload_ring[(stage * kRanks + k) * 32 + lane];
                const float scale = scale_ring[(stage * kRanks + k) * 32 + lane];
                non_finite |= bad_scale(scale);
                if (k == 0) accumulate16<true>(words, scale, acc);
                else accumulate16<false>(words, scale, acc);
            }
            reencode_and_store<kBlock, kSquares>(shards, base, lane, acc, reduction_scale, squares, non_finite);
        } else {
            reduce_tile_scalar<kBlock, kSquares>(shards, kRanks, base, end_value, lane, reduction_scale,
                                                 squares, non_finite);
        }
        stage = (stage + 1) % kStages;
    }
    async_wait<0>();
    if (finite_status != nullptr) {
        if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(finite_status, 1);
    }
    if (kSquares) cta_accumulate(squares, squared_sum);
}

// N encoded inputs -> fp32 sum, rank order, optional x reduction_scale,
// optional sum of squares of the fp32 result, optional finite flag with the
// tensor-wide reducer's rule: an invalid input scale or a non-finite result
// raises the flag and that element is not written
// (NNtrain.Cuda/native/tensor_kernels.cu:1084-1106).  kShift: block = 1 <<
// kShift, or -1 for a runtime block size.  kMaximum additionally folds the
// maximum |result| into *maximum_bits (for a tensor-wide re-encode).
struct EncodedInputs {
    const signed char* payload[kMaxRanks];
    const float* scales[kMaxRanks];
    int inputs;
};

template <int kShift, bool kGuard, bool kSquares, bool kMaximum>
__global__ void __launch_bounds__(kThreads)
bfp8_sum_to_f32_kernel(EncodedInputs in, float* __restrict__ reduced, long long length, long long block,
                       float reduction_scale, double* squared_sum, int* finite_status,
                       unsigned* maximum_bits, bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long words = vector_ok ? length / 4 : 0;
    double squares = 0.0;
    int non_finite = 0;
    float m = 0.0f;
    auto scale_index = [&](long long i) -> long long {
        return kShift >= 0 ? i >> (kShift >= 0 ? kShift : 0) : i / block;
    };
    for (long long w = thread; w < words; w += threads) {
        float4 sum;
        bool bad = false;
        for (int k = 0; k < in.inputs; ++k) {
            const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(in.payload[k]) + w) ^ 0x80808080u;
            const float s = __ldg(in.scales[k] + scale_index(w * 4));
            if (kGuard) bad |= bad_scale(s);
            const float t0 = __fmul_rn(byte_to_float(biased, 0), s), t1 = __fmul_rn(byte_to_float(biased, 1), s),
                        t2 = __fmul_rn(byte_to_float(biased, 2), s), t3 = __fmul_rn(byte_to_float(biased, 3), s);
            if (k == 0) { sum.x = t0; sum.y = t1; sum.z = t2; sum.w = t3; }
            else {
                sum.x = __fadd_rn(sum.x, t0); sum.y = __fadd_rn(sum.y, t1);
                sum.z = __fadd_rn(sum.z, t2); sum.w = __fadd_rn(sum.w, t3);
            }
        }
        sum.x = __fmul_rn(reduction_scale, sum.x); sum.y = __fmul_rn(reduction_scale, sum.y);
        sum.z = __fmul_rn(reduction_scale, sum.z); sum.w = __fmul_rn(reduction_scale, sum.w);
        if (kGuard) {
            const bool n0 = bad | is_non_finite(sum.x), n1 = bad | is_non_finite(sum.y),
                       n2 = bad | is_non_finite(sum.z), n3 = bad | is_non_finite(sum.w);
            if (n0 | n1 | n2 | n3) {
                non_finite = 1;
                if (!n0) reduced[w * 4 + 0] = sum.x;
                if (!n1) reduced[w * 4 + 1] = sum.y;
                if (!n2) reduced[w * 4 + 2] = sum.z;
                if (!n3) reduced[w * 4 + 3] = sum.w;
                continue;
            }
        }
        store_f4(reduced + w * 4, sum);
        if (kMaximum) m = fmaxf(m, fmaxf(fmaxf(fabsf(sum.x), fabsf(sum.y)), fmaxf(fabsf(sum.z), fabsf(sum.w))));
        if (kSquares) {
            squares += static_cast<double>(sum.x) * static_cast<double>(sum.x);
            squares += static_cast<double>(sum.y) * static_cast<double>(sum.y);
            squares += static_cast<double>(sum.z) * static_cast<double>(sum.z);
            squares += static_cast<double>(sum.w) * static_cast<double>(sum.w);
        }
    }
    for (long long i = words * 4 + thread; i < length; i += threads) {
        float sum = 0.0f;
        bool bad = false;
        for (int k = 0; k < in.inputs; ++k) {
            const float s = in.scales[k][scale_index(i)];
            if (kGuard) bad |= bad_scale(s);
            const float term = __fmul_rn(static_cast<float>(in.payload[k][i]), s);
            sum = k == 0 ? term : __fadd_rn(sum, term);
        }
        sum = __fmul_rn(reduction_scale, sum);
        if (kGuard && (bad || is_non_finite(sum))) { non_finite = 1; continue; }
        reduced[i] = sum;
        if (kMaximum) m = fmaxf(m, fabsf(sum));
        if (kSquares) squares += static_cast<double>(sum) * static_cast<double>(sum);
    }
    if (kGuard) {
        if (__any_sync(0xffffffffu, non_finite) && (threadIdx.x & 31) == 0) atomicExch(finite_status, 1);
    }
    if (kMaximum) {
        __shared__ float warp_max[kWarpsPerCta];
        m = group_max<32>(m);
        if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0) {
            #pragma unroll
            for (int w = 1; w < kWarpsPerCta; ++w) m = fmaxf(m, warp_max[w]);
            if (m > 0.0f) atomicMax(maximum_bits, __float_as_uint(m));
        }
    }
    if (kSquares) cta_accumulate(squares, squared_sum);
}

// ---- bf16 ------------------------------------------------------------------
struct Bf16Inputs {
    const unsigned short* values[kMaxRanks];
    unsigned short* out_bf16[kMaxRanks];   // optional re-encoded outputs (M of them)
    int inputs;
    int outputs;
};

__device__ __forceinline__ float bf16_bits_to_float(unsigned short bits) {
    return __uint_as_float(static_cast<unsigned>(bits) << 16);
}

// fp32 -> bf16 round-to-nearest-even, every NaN -> 0x7FFF: what CUDA's
// __float2bfloat16_rn produces (the reference's pack kernel,
// gradient_collectives.cu:11-22), written out so it is identical on every
// toolchain.
__device__ __forceinline__ unsigned short float_to_bf16_bits(float value) {
    const unsigned bits = __float_as_uint(value);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
    return static_cast<unsigned short>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

// N bf16 inputs -> fp32 accumulate in rank order (x reduction_scale) ->
// optional fp32 output, optional bf16 outputs to M destinations, optional sum
// of squares (of the bf16-rounded value when kSquareOfBf16, else of the fp32
// sum).  Eight values (one 128-bit load per input) per lane per step when
// `vector_ok`, scalar otherwise.
// kRanks > 0: number of inputs known at compile time; the loads of the NEXT
// group of every rank are issued before the current group's arithmetic, so
// with peer pointers a lane always has one NVLink round trip per rank in
// flight.  kRanks == 0: runtime count, loads and arithmetic alternate.
template <int kRanks>
struct Bf16Group {
    uint4 raw[kRanks > 0 ? kRanks : 1];
};

template <int kRanks>
__device__ __forceinline__ void load_bf16_group(const Bf16Inputs& io, long long at, Bf16Group<kRanks>& group) {
    #pragma unroll
    for (int k = 0; k < kRanks; ++k) group.raw[k] = __ldcs(reinterpret_cast<const uint4*>(io.values[k] + at));
}

template <bool kFirst>
__device__ __forceinline__ void accumulate_bf16x8(const uint4& raw, float (&acc)[8]) {
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
    #pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float lo = __uint_as_float(w[q] << 16), hi = __uint_as_float(w[q] & 0xffff0000u);
        acc[2 * q] = kFirst ? lo : __fadd_rn(acc[2 * q], lo);
        acc[2 * q + 1] = kFirst ? hi : __fadd_rn(acc[2 * q + 1], hi);
    }
}

template <bool kSquares, bool kSquareOfBf16>
__device__ __forceinline__ void finish_bf16x8(const Bf16Inputs& io, float* reduced, long long at, float (&acc)[8],
                                              float reduction_scale, double& squares) {
    #pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fmul_rn(reduction_scale, acc[i]);
    if (reduced != nullptr) {
        store_f4(reduced + at, make_float4(acc[0], acc[1], acc[2], acc[3]));
        store_f4(reduced + at + 4, make_float4(acc[4], acc[5], acc[6], acc[7]));
    }
    unsigned short e[8];
    if (io.outputs > 0 || (kSquares && kSquareOfBf16)) {
        #pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = float_to_bf16_bits(acc[i]);
    }
    if (io.outputs > 0) {
        uint4 packed;
        packed.x = e[0] | (static_cast<unsigned>(e[1]) << 16);
        packed.y = e[2] | (static_cast<unsigned>(e[3]) << 16);
        packed.z = e[4] | (static_cast<unsigned>(e[5]) << 16);
        packed.w = e[6] | (static_cast<unsigned>(e[7]) << 16);
        for (int d = 0; d < io.outputs; ++d)
            *reinterpret_cast<uint4*>(io.out_bf16[d] + at) = packed;
    }
    if (kSquares) {
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const double v = static_cast<double>(kSquareOfBf16 ? bf16_bits_to_float(e[i]) : acc[i]);
            squares += v * v;
        }
    }
}

template <int kRanks, bool kSquares, bool kSquareOfBf16>
__global__ void __launch_bounds__(kThreads)
bf16_reduce_kernel(Bf16Inputs io, float* reduced, long long first_value, long long end_value,
                   float reduction_scale, double* squared_sum, bool vector_ok) {
    const long long thread = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long span = end_value - first_value;
    const long long groups = vector_ok ? span / 8 : 0;
    double squares = 0.0;
    if (kRanks > 0) {
        Bf16Group<kRanks> current, next;
        long long g = thread;
        if (g < groups) load_bf16_group<kRanks>(io, first_value + g * 8, current);
        while (g < groups) {
            const long long following = g + threads;
            if (following < groups) load_bf16_group<kRanks>(io, first_value + following * 8, next);
            float acc[8];
            #pragma unroll
            for (int k = 0; k < kRanks; ++k) {
                if (k == 0) accumulate_bf16x8<true>(current.raw[k], acc);
                else accumulate_bf16x8<false>(current.raw[k], acc);
            }
            finish_bf16x8<kSquares, kSquareOfBf16>(io, reduced, first_value + g * 8, acc, reduction_scale, squares);
            current = next;
            g = following;
        }
    } else {
        for (long long g = thread; g < groups; g += threads) {
            const long long at = first_value + g * 8;
            float acc[8];
            for (int k = 0; k < io.inputs; ++k) {
                const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(io.values[k] + at));
                if (k == 0) accumulate_bf16x8<true>(raw, acc);
                else accumulate_bf16x8<false>(raw, acc);
            }
            finish_bf16x8<kSquares, kSquareOfBf16>(io, reduced, at, acc, reduction_scale, squares);
        }
    }
    for (long long i = first_value + groups * 8 + thread; i < end_value; i += threads) {
        float sum = 0.0f;
        for (int k = 0; k < io.inputs; ++k) {
            const float term = bf16_bits_to_float(io.values[k][i]);
            sum = k == 0 ? term : __fadd_rn(sum, term);
        }
        sum = __fmul_rn(reduction_scale, sum);
        if (reduced != nullptr) reduced[i] = sum;
        const unsigned short e = float_to_bf16_bits(sum);
        for (int d = 0; d < io.outputs; ++d) io.out_bf16[d][i] = e;
        if (kSquares) {
            const double v = static_cast<double>(kSquareOfBf16 ? bf16_bits_to_float(e) : sum);
            squares += v * v;
        }
    }
    if (kSquares) cta_accumulate(squares, squared_sum);
}

// How an all-reduce kernel is launched.  ctas: 0 = fill the machine, n > 0 =
// at most n CTAs.  asynchronous: 0 = register prefetch, 1 = cp.async rings in
// shared memory, 2 = bulk asynchronous copies of whole tiles (reduce_bulk.cuh).
// exclusive: 1 (with asynchronous) = big CTAs that take a whole SM each (see
// kExclusiveSharedBytes), so `ctas` is then the number of SMs the collective
// owns while it runs; the bulk variant is always launched that way.
struct CollectiveShape {
    int ctas;
    int asynchronous;
    int exclusive;
};

// The process-wide default (nntrain_gradient_configure*).
CollectiveShape default_collective_shape();

// What every group handle starts with, so one configure call serves both the
// one-process-per-GPU group and the in-process group.
constexpr int kKindProcessGroup = 0x47524f55;
constexpr int kKindLocalGroup = 0x4c4f4341;
struct GroupHeader {
    int kind;
    CollectiveShape shape;
};

// ---- launchers (reduce_launch.cu) --------------------------------------------
cudaError_t launch_bfp8_reduce_reencode(const EncodedShards& shards, long long first_value,
                                        long long end_value, int block, float reduction_scale,
                                        double* squared_sum, int* finite_status, cudaStream_t stream,
                                        const CollectiveShape* shape = nullptr);

// fp32 [first_value, end_value) of `source` -> payload + scales in every output
// of `shards` (inputs unused).  first_value must be a multiple of `block`.
cudaError_t launch_bfp8_encode_to_all(const float* source, const EncodedShards& shards, long long first_value,
                                      long long end_value, int block, int* finite_status, cudaStream_t stream,
                                      const CollectiveShape* shape = nullptr);

cudaError_t launch_bfp8_sum_to_f32(const EncodedInputs& in, float* reduced, long long length,
                                   long long block, float reduction_scale, double* squared_sum,
                                   int* finite_status, unsigned* maximum_bits, cudaStream_t stream);

cudaError_t launch_bf16_reduce(const Bf16Inputs& io, float* reduced, long long first_value,
                               long long end_value, float reduction_scale, double* squared_sum,
                               bool square_of_bf16, cudaStream_t stream,
                               const CollectiveShape* shape = nullptr);

}  // namespace ngb
