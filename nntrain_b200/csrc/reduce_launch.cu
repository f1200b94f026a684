// Host-side launchers for the reduction kernels in reduce_kernels.cuh.
#include "reduce_kernels.cuh"
#include "reduce_bulk.cuh"

namespace ngb {
namespace {

inline bool aligned_to(const void* p, std::uintptr_t bytes) {
    return (reinterpret_cast<std::uintptr_t>(p) & (bytes - 1)) == 0;
}

int capped_grid(long long work_items, int cap_ctas, int per_sm_default) {
    if (work_items < 1) work_items = 1;
    long long cap = cap_ctas;
    if (cap <= 0) cap = static_cast<long long>(sm_count()) * per_sm_default;
    return static_cast<int>(work_items < cap ? work_items : cap);
}

template <int kBlock, int kRanks>
cudaError_t run_reencode(const EncodedShards& shards, long long first_value, long long end_value,
                         float reduction_scale, double* squared_sum, int* finite_status,
                         bool vector_ok, const CollectiveShape& shape, cudaStream_t stream) {
    const long long tiles = (end_value - first_value + 511) / 512;
    const int grid = capped_grid((tiles + kWarpsPerCta - 1) / kWarpsPerCta, shape.ctas, kCtasPerSmDefault);
    if (squared_sum != nullptr) {
        bfp8_reduce_reencode_kernel<kBlock, kRanks, true><<<grid, kThreads, 0, stream>>>(
            shards, first_value, end_value, reduction_scale, squared_sum, finite_status, vector_ok);
    } else {
        bfp8_reduce_reencode_kernel<kBlock, kRanks, false><<<grid, kThreads, 0, stream>>>(
            shards, first_value, end_value, reduction_scale, nullptr, finite_status, vector_ok);
    }
    return cudaPeekAtLastError();
}

// cp.async ring variant: needs 16-byte aligned arenas and a compile-time rank
// count.  Shared: 8 warps per CTA, one CTA per SM when it runs beside codec
// kernels, as many as the ring's shared memory lets an SM hold when alone.
// Exclusive (kWarps > 8 and the whole SM's shared memory): `shape.ctas` SMs
// belong to the kernel while it runs.
template <int kBlock, int kRanks, int kStages, int kWarps>
cudaError_t run_reencode_async(const EncodedShards& shards, long long first_value, long long end_value,
                               float reduction_scale, double* squared_sum, int* finite_status,
                               const CollectiveShape& shape, cudaStream_t stream) {
    constexpr size_t ring_bytes = reduce_ring_bytes<kRanks, kStages, kWarps>();
    static_assert(ring_bytes <= kExclusiveSharedBytes, "ring does not fit in one SM");
    const size_t bytes = shape.exclusive ? kExclusiveSharedBytes : ring_bytes;
    const long long tiles = (end_value - first_value + 511) / 512;
    const long long work = (tiles + kWarps - 1) / kWarps;
    long long cap = shape.ctas;
    if (cap <= 0) cap = static_cast<long long>(sm_count()) * ((shape.exclusive || bytes > 100 * 1024) ? 1 : 2);
    if (shape.exclusive && cap > sm_count()) cap = sm_count();
    const int grid = static_cast<int>(work < cap ? work : cap);
    cudaError_t e;
    if (squared_sum != nullptr) {
        auto kernel = bfp8_reduce_reencode_async_kernel<kBlock, kRanks, true, kStages, kWarps>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (e != cudaSuccess) return e;
        kernel<<<grid, kWarps * 32, bytes, stream>>>(shards, first_value, end_value, reduction_scale, squared_sum,
                                                    finite_status);
    } else {
        auto kernel = bfp8_reduce_reencode_async_kernel<kBlock, kRanks, false, kStages, kWarps>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (e != cudaSuccess) return e;
        kernel<<<grid, kWarps * 32, bytes, stream>>>(shards, first_value, end_value, reduction_scale, nullptr,
                                                    finite_status);
    }
    return cudaPeekAtLastError();
}

// Bulk-copy variant: whole tiles travel as cp.async.bulk transfers; launched
// either with big CTAs that own their SM or with small ones that share it.
// Needs a compile-time rank count,
// 16-byte aligned payload AND scale arenas and a 512-aligned first value.
template <int kBlock, int kRanks, int kStages, int kWarps, int kTile>
cudaError_t run_reencode_bulk(const EncodedShards& shards, long long first_value, long long end_value,
                              float reduction_scale, double* squared_sum, int* finite_status,
                              const CollectiveShape& shape, cudaStream_t stream) {
    constexpr size_t needed = kWarps * bulk_warp_bytes<kBlock, kRanks, kStages, kTile>();
    static_assert(needed <= kExclusiveSharedBytes, "the rings do not fit in one SM");
    const size_t bytes = shape.exclusive ? kExclusiveSharedBytes : needed;
    const long long tiles = (end_value - first_value + kTile - 1) / kTile;
    const long long work = (tiles + kWarps - 1) / kWarps;
    long long cap = shape.ctas > 0 ? shape.ctas : sm_count();
    if (shape.exclusive && cap > sm_count()) cap = sm_count();
    const int grid = static_cast<int>(work < cap ? work : cap);
    cudaError_t e;
    if (squared_sum != nullptr) {
        auto kernel = bfp8_reduce_reencode_bulk_kernel<kBlock, kRanks, true, kStages, kWarps, kTile>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (e != cudaSuccess) return e;
        kernel<<<grid, kWarps * 32, bytes, stream>>>(shards, first_value, end_value, reduction_scale, squared_sum,
                                                    finite_status);
    } else {
        auto kernel = bfp8_reduce_reencode_bulk_kernel<kBlock, kRanks, false, kStages, kWarps, kTile>;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (e != cudaSuccess) return e;
        kernel<<<grid, kWarps * 32, bytes, stream>>>(shards, first_value, end_value, reduction_scale, nullptr,
                                                    finite_status);
    }
    return cudaPeekAtLastError();
}

template <int kBlock>
cudaError_t dispatch_reencode(const EncodedShards& shards, long long first_value, long long end_value,
                              float reduction_scale, double* squared_sum, int* finite_status,
                              bool vector_ok, const CollectiveShape& shape, cudaStream_t stream) {
    if (vector_ok && shape.asynchronous == 2 && first_value % 512 == 0) {
        bool scales_aligned = true;
        for (int k = 0; k < shards.inputs; ++k) scales_aligned = scales_aligned && aligned_to(shards.scales[k], 16);
        for (int d = 0; d < shards.outputs; ++d) scales_aligned = scales_aligned && aligned_to(shards.out_scales[d], 16);
        if (scales_aligned && !shape.exclusive) {
            // small CTAs (4 warps, ~80 KB of rings) that share their SM with codec CTAs
            switch (shards.inputs) {
                case 2: return run_reencode_bulk<kBlock, 2, 8, 4, 1024>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream);
                case 4: return run_reencode_bulk<kBlock, 4, 4, 4, 1024>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream);
                case 8: return run_reencode_bulk<kBlock, 8, 4, 4, 512>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream);
                default: break;
            }
        }
        if (scales_aligned) {
            switch (shards.inputs) {
                case 2: return run_reencode_bulk<kBlock, 2, 8, 11, 1024>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream);
                case 4: return run_reencode_bulk<kBlock, 4, 4, 11, 1024>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream);
                case 8: return run_reencode_bulk<kBlock, 8, 4, 11, 512>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream);
                default: break;
            }
        }
    }
#define NGB_RING(R, S, W) \
    return run_reencode_async<kBlock, R, S, W>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, shape, stream)
    if (vector_ok && shape.asynchronous != 0 && shape.exclusive) {
        // rings sized for an SM of their own: ~130-150 KB of loads in flight per SM
        switch (shards.inputs) {
            case 2: NGB_RING(2, 8, 16);
            case 4: NGB_RING(4, 5, 16);
            case 8: NGB_RING(8, 3, 12);
            default: break;
        }
    }
    if (vector_ok && shape.asynchronous != 0) {
        switch (shards.inputs) {
            case 2: NGB_RING(2, 8, 8);
            case 4: NGB_RING(4, 6, 8);
            case 8: NGB_RING(8, 4, 8);
            default: break;
        }
    }
#undef NGB_RING
#define NGB_PREFETCH(R) \
    case R: return run_reencode<kBlock, R>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, vector_ok, shape, stream)
    switch (shards.inputs) {
        NGB_PREFETCH(2); NGB_PREFETCH(3); NGB_PREFETCH(4); NGB_PREFETCH(5);
        NGB_PREFETCH(6); NGB_PREFETCH(7); NGB_PREFETCH(8);
        default: return run_reencode<kBlock, 0>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, vector_ok, shape, stream);
    }
#undef NGB_PREFETCH
}

template <int kShift, bool kGuard, bool kSquares, bool kMaximum>
void run_sum(int grid, cudaStream_t stream, const EncodedInputs& in, float* reduced, long long length,
             long long block, float reduction_scale, double* squared_sum, int* finite_status,
             unsigned* maximum_bits, bool vector_ok) {
    bfp8_sum_to_f32_kernel<kShift, kGuard, kSquares, kMaximum><<<grid, kThreads, 0, stream>>>(
        in, reduced, length, block, reduction_scale, squared_sum, finite_status, maximum_bits, vector_ok);
}

template <int kShift>
void dispatch_sum(int grid, cudaStream_t stream, const EncodedInputs& in, float* reduced, long long length,
                  long long block, float reduction_scale, double* squared_sum, int* finite_status,
                  unsigned* maximum_bits, bool vector_ok) {
    const int key = (finite_status ? 4 : 0) | (squared_sum ? 2 : 0) | (maximum_bits ? 1 : 0);
#define NGB_SUM(K, G, S, M) \
    case K: run_sum<kShift, G, S, M>(grid, stream, in, reduced, length, block, reduction_scale, squared_sum, finite_status, maximum_bits, vector_ok); break;
    switch (key) {
        NGB_SUM(0, false, false, false) NGB_SUM(1, false, false, true)
        NGB_SUM(2, false, true, false) NGB_SUM(3, false, true, true)
        NGB_SUM(4, true, false, false) NGB_SUM(5, true, false, true)
        NGB_SUM(6, true, true, false) NGB_SUM(7, true, true, true)
    }
#undef NGB_SUM
}

}  // namespace

CollectiveShape default_collective_shape() {
    const LaunchPolicy policy = launch_policy();
    // process-wide mode: 0 register prefetch, 1 cp.async rings, 2 rings in CTAs that own
    // their SM, 3 bulk copies in CTAs that own their SM, 4 bulk copies in small CTAs
    const int mode = policy.collective_async;
    return CollectiveShape{policy.collective_ctas, mode >= 3 ? 2 : (mode != 0 ? 1 : 0),
                           (mode == 2 || mode == 3) ? 1 : 0};
}

cudaError_t launch_bfp8_reduce_reencode(const EncodedShards& shards, long long first_value,
                                        long long end_value, int block, float reduction_scale,
                                        double* squared_sum, int* finite_status, cudaStream_t stream,
                                        const CollectiveShape* shape_or_null) {
    const CollectiveShape shape = shape_or_null ? *shape_or_null : default_collective_shape();
    if (shards.inputs < 1 || shards.inputs > kMaxRanks || shards.outputs < 1 || shards.outputs > kMaxRanks)
        return cudaErrorInvalidValue;
    if (first_value < 0 || end_value <= first_value) return cudaErrorInvalidValue;
    if (block != 32 && block != 64 && block != 128) return cudaErrorInvalidValue;
    if (first_value % block != 0) return cudaErrorInvalidValue;
    bool vector_ok = first_value % 16 == 0;
    for (int k = 0; k < shards.inputs; ++k) {
        if (!shards.payload[k] || !shards.scales[k]) return cudaErrorInvalidValue;
        vector_ok = vector_ok && aligned_to(shards.payload[k], 16);
    }
    for (int d = 0; d < shards.outputs; ++d) {
        if (!shards.out_payload[d] || !shards.out_scales[d]) return cudaErrorInvalidValue;
        vector_ok = vector_ok && aligned_to(shards.out_payload[d], 16);
    }
    switch (block) {
        case 32: return dispatch_reencode<32>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, vector_ok, shape, stream);
        case 64: return dispatch_reencode<64>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, vector_ok, shape, stream);
        default: return dispatch_reencode<128>(shards, first_value, end_value, reduction_scale, squared_sum, finite_status, vector_ok, shape, stream);
    }
}

cudaError_t launch_bfp8_encode_to_all(const float* source, const EncodedShards& shards, long long first_value,
                                      long long end_value, int block, int* finite_status, cudaStream_t stream,
                                      const CollectiveShape* shape_or_null) {
    const CollectiveShape shape = shape_or_null ? *shape_or_null : default_collective_shape();
    if (!source || shards.outputs < 1 || shards.outputs > kMaxRanks) return cudaErrorInvalidValue;
    if (first_value < 0 || end_value <= first_value) return cudaErrorInvalidValue;
    if ((block != 32 && block != 64 && block != 128) || first_value % block != 0) return cudaErrorInvalidValue;
    bool vector_ok = first_value % 16 == 0 && aligned_to(source, 16);
    for (int d = 0; d < shards.outputs; ++d) {
        if (!shards.out_payload[d] || !shards.out_scales[d]) return cudaErrorInvalidValue;
        vector_ok = vector_ok && aligned_to(shards.out_payload[d], 16);
    }
    const long long tiles = (end_value - first_value + 511) / 512;
    const int grid = capped_grid((tiles + kWarpsPerCta - 1) / kWarpsPerCta, shape.ctas, kCtasPerSmDefault);
    if (block == 32)
        bfp8_encode_to_all_kernel<32><<<grid, kThreads, 0, stream>>>(source, shards, first_value, end_value, finite_status, vector_ok);
    else if (block == 64)
        bfp8_encode_to_all_kernel<64><<<grid, kThreads, 0, stream>>>(source, shards, first_value, end_value, finite_status, vector_ok);
    else
        bfp8_encode_to_all_kernel<128><<<grid, kThreads, 0, stream>>>(source, shards, first_value, end_value, finite_status, vector_ok);
    return cudaPeekAtLastError();
}

cudaError_t launch_bfp8_sum_to_f32(const EncodedInputs& in, float* reduced, long long length,
                                   long long block, float reduction_scale, double* squared_sum,
                                   int* finite_status, unsigned* maximum_bits, cudaStream_t stream) {
    if (in.inputs < 1 || in.inputs > kMaxRanks || !reduced || length <= 0 || block <= 0)
        return cudaErrorInvalidValue;
    if (block > length) block = length;
    bool vector_ok = aligned_to(reduced, 16);
    for (int k = 0; k < in.inputs; ++k) {
        if (!in.payload[k] || !in.scales[k]) return cudaErrorInvalidValue;
        vector_ok = vector_ok && aligned_to(in.payload[k], 4);
    }
    const int grid = grid_for((length / 4 + kThreads - 1) / kThreads, kCtasPerSm);
    if (block == 32) dispatch_sum<5>(grid, stream, in, reduced, length, block, reduction_scale, squared_sum, finite_status, maximum_bits, vector_ok);
    else if (block == 128) dispatch_sum<7>(grid, stream, in, reduced, length, block, reduction_scale, squared_sum, finite_status, maximum_bits, vector_ok);
    else dispatch_sum<-1>(grid, stream, in, reduced, length, block, reduction_scale, squared_sum, finite_status, maximum_bits, vector_ok);
    return cudaPeekAtLastError();
}

template <int kRanks>
void run_bf16_reduce(int grid, cudaStream_t stream, const Bf16Inputs& io, float* reduced, long long first_value,
                     long long end_value, float reduction_scale, double* squared_sum, bool square_of_bf16,
                     bool vector_ok) {
    if (!squared_sum)
        bf16_reduce_kernel<kRanks, false, false><<<grid, kThreads, 0, stream>>>(io, reduced, first_value, end_value, reduction_scale, nullptr, vector_ok);
    else if (square_of_bf16)
        bf16_reduce_kernel<kRanks, true, true><<<grid, kThreads, 0, stream>>>(io, reduced, first_value, end_value, reduction_scale, squared_sum, vector_ok);
    else
        bf16_reduce_kernel<kRanks, true, false><<<grid, kThreads, 0, stream>>>(io, reduced, first_value, end_value, reduction_scale, squared_sum, vector_ok);
}

cudaError_t launch_bf16_reduce(const Bf16Inputs& io, float* reduced, long long first_value,
                               long long end_value, float reduction_scale, double* squared_sum,
                               bool square_of_bf16, cudaStream_t stream, const CollectiveShape* shape_or_null) {
    const CollectiveShape shape = shape_or_null ? *shape_or_null : default_collective_shape();
    if (io.inputs < 1 || io.inputs > kMaxRanks || io.outputs < 0 || io.outputs > kMaxRanks)
        return cudaErrorInvalidValue;
    if (first_value < 0 || end_value <= first_value || (!reduced && io.outputs == 0 && !squared_sum))
        return cudaErrorInvalidValue;
    bool vector_ok = first_value % 8 == 0 && (!reduced || aligned_to(reduced, 16));
    for (int k = 0; k < io.inputs; ++k) {
        if (!io.values[k]) return cudaErrorInvalidValue;
        vector_ok = vector_ok && aligned_to(io.values[k], 16);
    }
    for (int d = 0; d < io.outputs; ++d) {
        if (!io.out_bf16[d]) return cudaErrorInvalidValue;
        vector_ok = vector_ok && aligned_to(io.out_bf16[d], 16);
    }
    const long long groups = (end_value - first_value + 7) / 8;
    const int grid = capped_grid((groups + kThreads - 1) / kThreads, shape.ctas, kCtasPerSmDefault);
#define NGB_BF16(R) \
    case R: run_bf16_reduce<R>(grid, stream, io, reduced, first_value, end_value, reduction_scale, squared_sum, square_of_bf16, vector_ok); break
    switch (io.inputs) {
        NGB_BF16(2); NGB_BF16(3); NGB_BF16(4); NGB_BF16(5); NGB_BF16(6); NGB_BF16(7); NGB_BF16(8);
        default: run_bf16_reduce<0>(grid, stream, io, reduced, first_value, end_value, reduction_scale, squared_sum, square_of_bf16, vector_ok); break;
    }
#undef NGB_BF16
    return cudaPeekAtLastError();
}

}  // namespace ngb
