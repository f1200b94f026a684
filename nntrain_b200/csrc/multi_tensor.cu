// Whole-bucket launches for the tensor-wide BFP8 gradient reducer (ABI minor 36).
//
// The reference publishes, reduces and broadcasts ONE TENSOR per call
// (NNtrain.Cuda/native/tensor_kernels.cu:1114-1146 publish: a memset and five
// or six launches; :3935-4038 reduce / broadcast: five peer copies and about
// thirteen launches), and its single-GPU publication scope walks the leaves
// the same way (NNtrain.Core/Tensors/CudaBfp8GradientPublicationScope.cs:
// 12-521).  A model has hundreds of tensors, so a step pays thousands of
// launches.  Here the tensors of a bucket sit in one contiguous arena at
// running-sum offsets (the reference's own arena layout,
// NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1572-1601) and a table
// of those offsets, resident on the device, lets one kernel serve them all:
//
//   publish  memset(maxima) + maxima/finite pass + payload/write-back/squares
//            pass: 3 operations per BUCKET, whatever the number of tensors;
//   reduce   memset + (N inputs -> fp32 sum + maxima) pass + payload pass;
//   decode   one pass (the receiving side of a broadcast).
//
// Arithmetic per tensor is the reference's: scale = max|x| / 127 over the whole
// tensor (1 for an all-zero tensor), code = clamp(rne(x / scale), +-127), the
// fp32 gradient overwritten with code * scale, sum of squares of that in
// binary64; r = reduction_scale * (rank-ordered sum of code * scale).  A NaN or
// Inf anywhere in the bucket (or a flag already raised) publishes nothing: the
// flag is set, every scale of the bucket becomes 1, payload and gradient stay
// as they were -- the reference's rule (tensor_kernels.cu:1015-1018,1027,1038)
// applied to the launch's unit, the bucket.
//
// Traversal: a warp owns a contiguous chunk of 4096 values of the flat arena
// and walks it in rows of 128 (each lane four consecutive values, one 128-bit
// access).  The tensor under the row is tracked incrementally from the offset
// table (one uniform, cached load per row); a row that lies inside one tensor
// -- nearly all of them -- takes the vector path (four such rows at a time, so
// four independent 128-bit loads per lane are in flight), a row that straddles
// a boundary is done value by value.  Per-tensor maxima are folded in registers
// while the tensor stays the same and flushed with one atomic per change.
#include "bfp8_kernels.cuh"
#include "reduce_kernels.cuh"

namespace ngb {
namespace {

constexpr int kChunkValues = 4096;     // per warp
constexpr int kRowValues = 128;
constexpr int kBatchRows = 4;          // rows whose loads are issued together when one tensor holds them all

// Index t with offsets[t] <= position < offsets[t + 1] (offsets ascending,
// offsets[0] = 0, offsets[tensors] = total).
__device__ __forceinline__ int find_tensor(const long long* __restrict__ offsets, int tensors, long long position) {
    int lo = 0, hi = tensors - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(offsets + mid) <= position) lo = mid; else hi = mid - 1;
    }
    return lo;
}

struct TensorCursor {
    const long long* offsets;
    int tensors;
    int current;
    long long current_end;

    __device__ __forceinline__ void seek(long long position) {
        while (current + 1 < tensors && current_end <= position) {
            ++current;
            current_end = __ldg(offsets + current + 1);
        }
    }
};

__device__ __forceinline__ TensorCursor cursor_at(const long long* offsets, int tensors, long long position) {
    TensorCursor c{offsets, tensors, 0, 0};
    c.current = find_tensor(offsets, tensors, position);
    c.current_end = __ldg(offsets + c.current + 1);
    return c;
}

__device__ __forceinline__ void flush_maximum(float m, unsigned* maxima, int tensor, int lane) {
    m = group_max<32>(m);
    if (lane == 0 && m > 0.0f) atomicMax(maxima + tensor, __float_as_uint(m));
}

// ---- pass 1 of publish: per-tensor max|x| and the finite flag ---------------
__global__ void __launch_bounds__(kThreads)
tensors_maxima_kernel(const float* __restrict__ arena, const long long* __restrict__ offsets, int tensors,
                      long long total, unsigned* __restrict__ maxima, int* finite_status) {
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long chunks = (total + kChunkValues - 1) / kChunkValues;
    int bad = 0;
    for (long long chunk = warp; chunk < chunks; chunk += warps) {
        const long long chunk_start = chunk * kChunkValues;
        const long long chunk_end = chunk_start + kChunkValues < total ? chunk_start + kChunkValues : total;
        TensorCursor cursor = cursor_at(offsets, tensors, chunk_start);
        int owner = cursor.current;
        float m = 0.0f;
        for (long long row = chunk_start; row < chunk_end; row += kRowValues) {
            const long long row_end = row + kRowValues < chunk_end ? row + kRowValues : chunk_end;
            cursor.seek(row);
            if (cursor.current != owner) {
                flush_maximum(m, maxima, owner, lane);
                owner = cursor.current;
                m = 0.0f;
            }
            const long long at = row + lane * 4;
            if (row + kBatchRows * kRowValues <= chunk_end && cursor.current_end >= row + kBatchRows * kRowValues) {
                // kBatchRows rows inside one tensor: all their loads in flight together
                float4 x[kBatchRows];
                #pragma unroll
                for (int j = 0; j < kBatchRows; ++j) x[j] = load_f4_stream(arena + at + j * kRowValues);
                #pragma unroll
                for (int j = 0; j < kBatchRows; ++j) {
                    bad |= is_non_finite(x[j].x) | is_non_finite(x[j].y) | is_non_finite(x[j].z) | is_non_finite(x[j].w);
                    m = fmaxf(m, fmaxf(fmaxf(fabsf(x[j].x), fabsf(x[j].y)), fmaxf(fabsf(x[j].z), fabsf(x[j].w))));
                }
                row += (kBatchRows - 1) * kRowValues;
            } else if (row + kRowValues <= total && cursor.current_end >= row + kRowValues) {
                const float4 x = load_f4_stream(arena + at);
                bad |= is_non_finite(x.x) | is_non_finite(x.y) | is_non_finite(x.z) | is_non_finite(x.w);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
            } else {
                // the row crosses a tensor boundary (or the arena's ragged end)
                TensorCursor mine = cursor;
                for (int e = 0; e < 4; ++e) {
                    const long long i = at + e;
                    if (i >= row_end) break;
                    mine.seek(i);
                    const float x = arena[i];
                    bad |= is_non_finite(x);
                    // (a non-finite value raises the flag; nothing is published then)
                    if (fabsf(x) > 0.0f && !is_non_finite(x)) atomicMax(maxima + mine.current, __float_as_uint(fabsf(x)));
                }
            }
        }
        flush_maximum(m, maxima, owner, lane);
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicExch(finite_status, 1);
}

// ---- pass 2 of publish / reduce: payload, write-back, squares, scales ---------
// `source` holds the values to encode (the gradient itself, or the fp32 sum of
// a reduce); the decode is written back into it.
template <bool kSquares>
__global__ void __launch_bounds__(kThreads)
tensors_payload_kernel(float* source, signed char* __restrict__ payload, float* __restrict__ scales,
                       const long long* __restrict__ offsets, int tensors, long long total,
                       const unsigned* __restrict__ maxima, const int* finite_status, double* squared_sum) {
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long chunks = (total + kChunkValues - 1) / kChunkValues;
    const bool skip = *finite_status != 0;
    double squares = 0.0;
    if (skip) {
        // nothing is published: every scale of the bucket reads 1
        for (long long t = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; t < tensors;
             t += static_cast<long long>(gridDim.x) * kThreads)
            scales[t] = 1.0f;
    } else {
        for (long long chunk = warp; chunk < chunks; chunk += warps) {
            const long long chunk_start = chunk * kChunkValues;
            const long long chunk_end = chunk_start + kChunkValues < total ? chunk_start + kChunkValues : total;
            TensorCursor cursor = cursor_at(offsets, tensors, chunk_start);
            int owner = -1;
            float scale = 1.0f;
            BlockScale divisor = block_scale(1.0f);
            for (long long row = chunk_start; row < chunk_end; row += kRowValues) {
                const long long row_end = row + kRowValues < chunk_end ? row + kRowValues : chunk_end;
                cursor.seek(row);
                if (cursor.current != owner) {
                    owner = cursor.current;
                    scale = scale_from_maximum(__uint_as_float(maxima[owner]));
                    divisor = block_scale(scale);
                    // the row that holds a tensor's first value stores its scale
                    if (lane == 0 && __ldg(offsets + owner) >= row && __ldg(offsets + owner) < row + kRowValues)
                        scales[owner] = scale;
                }
                const long long at = row + lane * 4;
                if (row + kBatchRows * kRowValues <= chunk_end && cursor.current_end >= row + kBatchRows * kRowValues) {
                    float4 x[kBatchRows];
                    #pragma unroll
                    for (int j = 0; j < kBatchRows; ++j) x[j] = load_f4_stream(source + at + j * kRowValues);
                    #pragma unroll
                    for (int j = 0; j < kBatchRows; ++j) {
                        float t0, t1, t2, t3;
                        biased_codes_of(x[j], divisor, t0, t1, t2, t3);
                        *reinterpret_cast<unsigned*>(payload + at + j * kRowValues) = pack_codes(t0, t1, t2, t3);
                        float4 d;
                        d.x = __fmul_rn(code_value(t0), scale);
                        d.y = __fmul_rn(code_value(t1), scale);
                        d.z = __fmul_rn(code_value(t2), scale);
                        d.w = __fmul_rn(code_value(t3), scale);
                        store_f4(source + at + j * kRowValues, d);
                        if (kSquares) {
                            squares += static_cast<double>(d.x) * static_cast<double>(d.x);
                            squares += static_cast<double>(d.y) * static_cast<double>(d.y);
                            squares += static_cast<double>(d.z) * static_cast<double>(d.z);
                            squares += static_cast<double>(d.w) * static_cast<double>(d.w);
                        }
                    }
                    row += (kBatchRows - 1) * kRowValues;
                } else if (row + kRowValues <= total && cursor.current_end >= row + kRowValues) {
                    const float4 x = load_f4_stream(source + at);
                    float t0, t1, t2, t3;
                    biased_codes_of(x, divisor, t0, t1, t2, t3);
                    *reinterpret_cast<unsigned*>(payload + at) = pack_codes(t0, t1, t2, t3);
                    float4 d;
                    d.x = __fmul_rn(code_value(t0), scale);
                    d.y = __fmul_rn(code_value(t1), scale);
                    d.z = __fmul_rn(code_value(t2), scale);
                    d.w = __fmul_rn(code_value(t3), scale);
                    store_f4(source + at, d);
                    if (kSquares) {
                        squares += static_cast<double>(d.x) * static_cast<double>(d.x);
                        squares += static_cast<double>(d.y) * static_cast<double>(d.y);
                        squares += static_cast<double>(d.z) * static_cast<double>(d.z);
                        squares += static_cast<double>(d.w) * static_cast<double>(d.w);
                    }
                } else {
                    TensorCursor mine = cursor;
                    for (int e = 0; e < 4; ++e) {
                        const long long i = at + e;
                        if (i >= row_end) break;
                        mine.seek(i);
                        const float s = scale_from_maximum(__uint_as_float(maxima[mine.current]));
                        if (i == __ldg(offsets + mine.current)) scales[mine.current] = s;
                        const float t = biased_code_of(source[i], s);
                        payload[i] = code_byte(t);
                        const float d = __fmul_rn(code_value(t), s);
                        source[i] = d;
                        if (kSquares) squares += static_cast<double>(d) * static_cast<double>(d);
                    }
                }
            }
        }
    }
    if (kSquares) cta_accumulate(squares, squared_sum);
}

// ---- reduce: N encoded inputs -> fp32 sum (+ maxima, + flag) ------------------
struct TensorInputs {
    const signed char* payload[kMaxRanks];
    const float* scales[kMaxRanks];       // one scale per tensor
    int inputs;
};

__global__ void __launch_bounds__(kThreads)
tensors_sum_kernel(TensorInputs in, float* __restrict__ reduced, const long long* __restrict__ offsets,
                   int tensors, long long total, float reduction_scale, unsigned* __restrict__ maxima,
                   int* finite_status) {
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long chunks = (total + kChunkValues - 1) / kChunkValues;
    int bad = 0;
    for (long long chunk = warp; chunk < chunks; chunk += warps) {
        const long long chunk_start = chunk * kChunkValues;
        const long long chunk_end = chunk_start + kChunkValues < total ? chunk_start + kChunkValues : total;
        TensorCursor cursor = cursor_at(offsets, tensors, chunk_start);
        int owner = cursor.current;
        float m = 0.0f;
        for (long long row = chunk_start; row < chunk_end; row += kRowValues) {
            const long long row_end = row + kRowValues < chunk_end ? row + kRowValues : chunk_end;
            cursor.seek(row);
            if (cursor.current != owner) {
                flush_maximum(m, maxima, owner, lane);
                owner = cursor.current;
                m = 0.0f;
            }
            const long long at = row + lane * 4;
            if (row + kBatchRows * kRowValues <= chunk_end && cursor.current_end >= row + kBatchRows * kRowValues) {
                float4 sum[kBatchRows];
                for (int k = 0; k < in.inputs; ++k) {
                    const float s = __ldg(in.scales[k] + owner);
                    bad |= bad_scale(s);
                    unsigned word[kBatchRows];
                    #pragma unroll
                    for (int j = 0; j < kBatchRows; ++j)
                        word[j] = __ldcs(reinterpret_cast<const unsigned*>(in.payload[k] + at + j * kRowValues)) ^ 0x80808080u;
                    #pragma unroll
                    for (int j = 0; j < kBatchRows; ++j) {
                        const float t0 = __fmul_rn(byte_to_float(word[j], 0), s), t1 = __fmul_rn(byte_to_float(word[j], 1), s),
                                    t2 = __fmul_rn(byte_to_float(word[j], 2), s), t3 = __fmul_rn(byte_to_float(word[j], 3), s);
                        if (k == 0) { sum[j].x = t0; sum[j].y = t1; sum[j].z = t2; sum[j].w = t3; }
                        else {
                            sum[j].x = __fadd_rn(sum[j].x, t0); sum[j].y = __fadd_rn(sum[j].y, t1);
                            sum[j].z = __fadd_rn(sum[j].z, t2); sum[j].w = __fadd_rn(sum[j].w, t3);
                        }
                    }
                }
                #pragma unroll
                for (int j = 0; j < kBatchRows; ++j) {
                    float4 r = sum[j];
                    r.x = __fmul_rn(reduction_scale, r.x); r.y = __fmul_rn(reduction_scale, r.y);
                    r.z = __fmul_rn(reduction_scale, r.z); r.w = __fmul_rn(reduction_scale, r.w);
                    bad |= is_non_finite(r.x) | is_non_finite(r.y) | is_non_finite(r.z) | is_non_finite(r.w);
                    store_f4(reduced + at + j * kRowValues, r);
                    m = fmaxf(m, fmaxf(fmaxf(fabsf(r.x), fabsf(r.y)), fmaxf(fabsf(r.z), fabsf(r.w))));
                }
                row += (kBatchRows - 1) * kRowValues;
            } else if (row + kRowValues <= total && cursor.current_end >= row + kRowValues) {
                float4 sum;
                for (int k = 0; k < in.inputs; ++k) {
                    const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(in.payload[k] + at)) ^ 0x80808080u;
                    const float s = __ldg(in.scales[k] + owner);
                    bad |= bad_scale(s);
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
                bad |= is_non_finite(sum.x) | is_non_finite(sum.y) | is_non_finite(sum.z) | is_non_finite(sum.w);
                store_f4(reduced + at, sum);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(sum.x), fabsf(sum.y)), fmaxf(fabsf(sum.z), fabsf(sum.w))));
            } else {
                TensorCursor mine = cursor;
                for (int e = 0; e < 4; ++e) {
                    const long long i = at + e;
                    if (i >= row_end) break;
                    mine.seek(i);
                    float sum = 0.0f;
                    for (int k = 0; k < in.inputs; ++k) {
                        const float s = in.scales[k][mine.current];
                        bad |= bad_scale(s);
                        const float term = __fmul_rn(static_cast<float>(in.payload[k][i]), s);
                        sum = k == 0 ? term : __fadd_rn(sum, term);
                    }
                    sum = __fmul_rn(reduction_scale, sum);
                    bad |= is_non_finite(sum);
                    reduced[i] = sum;
                    if (fabsf(sum) > 0.0f && !is_non_finite(sum)) atomicMax(maxima + mine.current, __float_as_uint(fabsf(sum)));
                }
            }
        }
        flush_maximum(m, maxima, owner, lane);
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicExch(finite_status, 1);
}

// ---- decode: payload + per-tensor scales -> fp32 -------------------------------
__global__ void __launch_bounds__(kThreads)
tensors_decode_kernel(const signed char* __restrict__ payload, const float* __restrict__ scales,
                      float* __restrict__ destination, const long long* __restrict__ offsets, int tensors,
                      long long total, const int* skip_flag) {
    if (skip_flag != nullptr && *skip_flag != 0) return;
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    const long long chunks = (total + kChunkValues - 1) / kChunkValues;
    for (long long chunk = warp; chunk < chunks; chunk += warps) {
        const long long chunk_start = chunk * kChunkValues;
        const long long chunk_end = chunk_start + kChunkValues < total ? chunk_start + kChunkValues : total;
        TensorCursor cursor = cursor_at(offsets, tensors, chunk_start);
        int owner = -1;
        float scale = 1.0f;
        for (long long row = chunk_start; row < chunk_end; row += kRowValues) {
            const long long row_end = row + kRowValues < chunk_end ? row + kRowValues : chunk_end;
            cursor.seek(row);
            if (cursor.current != owner) {
                owner = cursor.current;
                scale = __ldg(scales + owner);
            }
            const long long at = row + lane * 4;
            if (row + kBatchRows * kRowValues <= chunk_end && cursor.current_end >= row + kBatchRows * kRowValues) {
                unsigned word[kBatchRows];
                #pragma unroll
                for (int j = 0; j < kBatchRows; ++j)
                    word[j] = __ldcs(reinterpret_cast<const unsigned*>(payload + at + j * kRowValues)) ^ 0x80808080u;
                #pragma unroll
                for (int j = 0; j < kBatchRows; ++j)
                    store_f4(destination + at + j * kRowValues,
                             make_float4(__fmul_rn(byte_to_float(word[j], 0), scale), __fmul_rn(byte_to_float(word[j], 1), scale),
                                         __fmul_rn(byte_to_float(word[j], 2), scale), __fmul_rn(byte_to_float(word[j], 3), scale)));
                row += (kBatchRows - 1) * kRowValues;
            } else if (row + kRowValues <= total && cursor.current_end >= row + kRowValues) {
                const unsigned biased = __ldcs(reinterpret_cast<const unsigned*>(payload + at)) ^ 0x80808080u;
                store_f4(destination + at,
                         make_float4(__fmul_rn(byte_to_float(biased, 0), scale), __fmul_rn(byte_to_float(biased, 1), scale),
                                     __fmul_rn(byte_to_float(biased, 2), scale), __fmul_rn(byte_to_float(biased, 3), scale)));
            } else {
                TensorCursor mine = cursor;
                for (int e = 0; e < 4; ++e) {
                    const long long i = at + e;
                    if (i >= row_end) break;
                    mine.seek(i);
                    destination[i] = __fmul_rn(static_cast<float>(payload[i]), scales[mine.current]);
                }
            }
        }
    }
}

inline bool aligned_to(const void* p, std::uintptr_t bytes) {
    return (reinterpret_cast<std::uintptr_t>(p) & (bytes - 1)) == 0;
}

int bucket_grid(long long total) {
    const long long chunks = (total + kChunkValues - 1) / kChunkValues;
    return grid_for((chunks + kWarpsPerCta - 1) / kWarpsPerCta, kCtasPerSm);
}

cudaError_t run_payload_pass(float* source, signed char* payload, float* scales, const long long* offsets,
                             int tensors, long long total, const unsigned* maxima, const int* finite_status,
                             double* squared_sum, cudaStream_t stream) {
    if (squared_sum != nullptr)
        tensors_payload_kernel<true><<<bucket_grid(total), kThreads, 0, stream>>>(
            source, payload, scales, offsets, tensors, total, maxima, finite_status, squared_sum);
    else
        tensors_payload_kernel<false><<<bucket_grid(total), kThreads, 0, stream>>>(
            source, payload, scales, offsets, tensors, total, maxima, finite_status, nullptr);
    return cudaPeekAtLastError();
}

}  // namespace
}  // namespace ngb

using namespace ngb;

// Publishes every tensor of a bucket arena in three stream operations.
// `tensor_offsets` is a DEVICE array of tensors + 1 strictly ascending element
// offsets (first 0, last = total_elements): tensor t is arena[offsets[t],
// offsets[t+1]).  `payload` has the arena's element layout, `scales` one entry
// per tensor, `maxima_scratch` is tensors words the caller owns (cleared
// here).  arena must be 16-byte aligned and payload 4-byte aligned (bucket
// bases are); the tensors themselves may start anywhere.  *squared_sum (may be
// null) += the sum of squares of the decoded values; *finite_status (required)
// is raised on NaN / Inf, in which case nothing else is published and every
// scale of the bucket is 1.
NNTRAIN_EXPORT int nntrain_bfp8_gradient_publish_tensors(
    int device, float* arena, signed char* payload, float* scales, const long long* tensor_offsets, int tensors,
    long long total_elements, unsigned* maxima_scratch, int* finite_status, double* squared_sum,
    cudaStream_t stream) {
    if (!arena || !payload || !scales || !tensor_offsets || tensors <= 0 || total_elements <= 0 ||
        !maxima_scratch || !finite_status || !aligned_to(arena, 16) || !aligned_to(payload, 4))
        return complete(kOpGradientPublishTensors, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpGradientPublishTensors, device, status);
    cudaError_t e = cudaMemsetAsync(maxima_scratch, 0, sizeof(unsigned) * static_cast<size_t>(tensors), stream);
    if (e == cudaSuccess) {
        tensors_maxima_kernel<<<bucket_grid(total_elements), kThreads, 0, stream>>>(
            arena, tensor_offsets, tensors, total_elements, maxima_scratch, finite_status);
        e = cudaPeekAtLastError();
    }
    if (e == cudaSuccess)
        e = run_payload_pass(arena, payload, scales, tensor_offsets, tensors, total_elements, maxima_scratch,
                             finite_status, squared_sum, stream);
    return complete(kOpGradientPublishTensors, device, static_cast<int>(e));
}

// The primary's arithmetic of the tensor-wide reducer for a whole bucket and N
// encoded inputs (host tables of device pointers, local or peer-mapped; scales
// are per-tensor arrays): reduced = reduction_scale * (rank-ordered fp32 sum
// of code * scale), then published as above -- out_payload / out_scales get
// the re-encoded result, `reduced` ends as its decode, *squared_sum += its sum
// of squares.  An invalid input scale or a non-finite sum raises the flag and
// publishes nothing (`reduced` then holds the raw sums).  Three stream
// operations per bucket.
NNTRAIN_EXPORT int nntrain_bfp8_gradient_reduce_tensors(
    int device, int inputs, const signed char* const* payloads, const float* const* scales, float* reduced,
    signed char* out_payload, float* out_scales, const long long* tensor_offsets, int tensors,
    long long total_elements, float reduction_scale, unsigned* maxima_scratch, int* finite_status,
    double* squared_sum, cudaStream_t stream) {
    if (inputs < 1 || inputs > kMaxRanks || !payloads || !scales || !reduced || !out_payload || !out_scales ||
        !tensor_offsets || tensors <= 0 || total_elements <= 0 || !std::isfinite(reduction_scale) ||
        !maxima_scratch || !finite_status || !aligned_to(reduced, 16) || !aligned_to(out_payload, 4))
        return complete(kOpGradientPublishTensors, device, static_cast<int>(cudaErrorInvalidValue));
    TensorInputs in{};
    in.inputs = inputs;
    for (int k = 0; k < inputs; ++k) {
        if (!payloads[k] || !scales[k] || !aligned_to(payloads[k], 4))
            return complete(kOpGradientPublishTensors, device, static_cast<int>(cudaErrorInvalidValue));
        in.payload[k] = payloads[k];
        in.scales[k] = scales[k];
    }
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpGradientPublishTensors, device, status);
    cudaError_t e = cudaMemsetAsync(maxima_scratch, 0, sizeof(unsigned) * static_cast<size_t>(tensors), stream);
    if (e == cudaSuccess) {
        tensors_sum_kernel<<<bucket_grid(total_elements), kThreads, 0, stream>>>(
            in, reduced, tensor_offsets, tensors, total_elements, reduction_scale, maxima_scratch, finite_status);
        e = cudaPeekAtLastError();
    }
    if (e == cudaSuccess)
        e = run_payload_pass(reduced, out_payload, out_scales, tensor_offsets, tensors, total_elements,
                             maxima_scratch, finite_status, squared_sum, stream);
    return complete(kOpGradientPublishTensors, device, static_cast<int>(e));
}

// destination = payload * scales[tensor] for a whole bucket (the receiving side
// of a broadcast).  Skipped when *skip_flag (optional) is non-zero, as the
// reference skips the decode of a failed step (tensor_kernels.cu:4034-4036).
NNTRAIN_EXPORT int nntrain_bfp8_gradient_decode_tensors(
    int device, const signed char* payload, const float* scales, float* destination,
    const long long* tensor_offsets, int tensors, long long total_elements, const int* skip_flag,
    cudaStream_t stream) {
    if (!payload || !scales || !destination || !tensor_offsets || tensors <= 0 || total_elements <= 0 ||
        !aligned_to(destination, 16) || !aligned_to(payload, 4))
        return complete(kOpGradientPublishTensors, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpGradientPublishTensors, device, status);
    tensors_decode_kernel<<<bucket_grid(total_elements), kThreads, 0, stream>>>(
        payload, scales, destination, tensor_offsets, tensors, total_elements, skip_flag);
    return complete(kOpGradientPublishTensors, device, static_cast<int>(cudaPeekAtLastError()));
}
