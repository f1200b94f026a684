// Owner arithmetic for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they
// reduce gradients: code running inside a memory-pool owner that forbids
// foreign allocations, a step that is being recorded for replay, or a
// real-time loop that must not touch the allocator.  The regular all-reduce
// keeps its per-shard sum of squares and finite flag in scratch memory that
// nntrain_gradient_group_create allocates; this entry point does the same
// owner arithmetic (N encoded shards -> fp32 accumulate in rank order ->
// re-encode -> M destinations, sum of squares, finite flag) with its scratch
// in a fixed array that is part of the library image.  It calls no
// allocating routine of the CUDA runtime or of any other library.
//
// The scratch holds one partial sum of squares per 65,536-value span, so the
// sum is also reproducible: spans are summed in a fixed order, with no
// atomics.  Size limit: kMaxSpans spans = 2^30 values per call; longer ranges
// are rejected.  The array (128 KiB + 256 B) is resident on every GPU that
// loads the library, until the process exits.
//
// Every call on a device shares that one array and the array keeps the last
// call's contents: the flag word is cleared at the start of each call and every
// partial slot a call reads is first written by that call.  Two calls whose
// kernels overlap on the same GPU (different streams, or different threads)
// race on it: serialise them.
#include "reduce_kernels.cuh"

#include <mutex>

namespace ngb {
namespace {

constexpr int kSpanValues = 65536;                 // values per CTA = per partial slot
constexpr int kMaxSpans = 16384;                   // 2^30 values per call
constexpr int kFlagSlot = kMaxSpans;               // int flag lives behind the partials
constexpr int kTilesPerWarp = kSpanValues / (kWarpsPerCta * 512);

static __device__ __align__(256) double g_no_alloc_scratch[kMaxSpans + 32];

constexpr int kKnownDevices = 64;
std::mutex g_setup_mutex;
double* g_scratch_address[kKnownDevices] = {};     // device address of the array, per device

// The array's name is only a host-side stand-in in host code; the device
// address comes from the runtime, once per device, with that device current.
cudaError_t scratch_for_current_device(int device, double** address) {
    if (device < 0 || device >= kKnownDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* found = nullptr;
        const cudaError_t status = cudaGetSymbolAddress(&found, g_no_alloc_scratch);
        if (status != cudaSuccess) return status;
        g_scratch_address[device] = static_cast<double*>(found);
    }
    *address = g_scratch_address[device];
    return cudaSuccess;
}

// One CTA per span.  Same per-tile arithmetic as the regular owner kernel
// (runtime rank count), then the CTA's sum of squares goes to its own slot.
template <int kBlock>
__global__ void __launch_bounds__(kThreads)
bfp8_reduce_reencode_spans_kernel(EncodedShards shards, long long first_value, long long end_value,
                                  float reduction_scale, double* partials, int* flag, bool vector_ok) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int ranks = shards.inputs;
    const long long span_first = first_value + static_cast<long long>(blockIdx.x) * kSpanValues;
    double squares = 0.0;
    int non_finite = 0;
    for (int i = 0; i < kTilesPerWarp; ++i) {
        const long long base = span_first + (static_cast<long long>(i) * kWarpsPerCta + warp) * 512;
        if (base >= end_value) break;
        if (vector_ok && base + 512 <= end_value) {
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
            reencode_and_store<kBlock, true>(shards, base, lane, acc, reduction_scale, squares, non_finite);
        } else {
            reduce_tile_scalar<kBlock, true>(shards, ranks, base, end_value, lane, reduction_scale,
                                             squares, non_finite);
        }
    }
    if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(flag, 1);
    cta_store_partial(squares, partials);
}

// Fixed-order sum of the partials; publishes the totals into the caller's
// outputs.  One CTA.
__global__ void __launch_bounds__(kThreads)
sum_spans_kernel(const double* partials, int spans, const int* flag, double* squared_sum, int* finite_status) {
    __shared__ double lanes[kThreads];
    double total = 0.0;
    for (int i = threadIdx.x; i < spans; i += kThreads) total += partials[i];
    lanes[threadIdx.x] = total;
    __syncthreads();
    for (int stride = kThreads / 2; stride > 0; stride >>= 1) {
        if (threadIdx.x < stride) lanes[threadIdx.x] += lanes[threadIdx.x + stride];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (squared_sum != nullptr) *squared_sum += lanes[0];
        if (finite_status != nullptr && *flag != 0) *finite_status = 1;
    }
}

constexpr Operation kOpReduceNoAlloc = static_cast<Operation>(200);

}  // namespace
}  // namespace ngb

using namespace ngb;

// Same arguments and results as nntrain_gradient_reduce_shards_bfp8: pointer
// tables are host arrays of device pointers; r = reduction_scale *
// (rank-ordered fp32 sum of the decoded inputs) over [first_value, end_value),
// re-encoded in blocks of block_size (32 / 64 / 128) into every output;
// *squared_sum += the sum of squares of the decoded result (fixed summation
// order); *finite_status = 1 on an invalid input scale or a non-finite sum.
// Allocates nothing.  At most 2^30 values per call (cudaErrorInvalidValue
// beyond, recorded in the error ring under operation 200).  The first call on
// a device looks up the scratch array's device address; make that first call
// before any stream capture begins on the device.  Calls that overlap on one
// GPU race on the shared scratch.
NNTRAIN_EXPORT int nntrain_gradient_reduce_shards_bfp8_no_alloc(
    int device, int inputs, const signed char* const* payloads, const float* const* scales, int outputs,
    signed char* const* out_payloads, float* const* out_scales, long long first_value, long long end_value,
    int block_size, float reduction_scale, double* squared_sum, int* finite_status, cudaStream_t stream) {
    if (inputs < 1 || inputs > kMaxRanks || outputs < 1 || outputs > kMaxRanks || !payloads || !scales ||
        !out_payloads || !out_scales || !std::isfinite(reduction_scale) || first_value < 0 ||
        end_value <= first_value || (block_size != 32 && block_size != 64 && block_size != 128) ||
        first_value % block_size != 0)
        return complete(kOpReduceNoAlloc, device, static_cast<int>(cudaErrorInvalidValue));
    const long long spans = (end_value - first_value + kSpanValues - 1) / kSpanValues;
    if (spans > kMaxSpans)      // beyond the fixed scratch: refuse rather than overrun it
        return complete(kOpReduceNoAlloc, device, static_cast<int>(cudaErrorInvalidValue));
    int status = select_device(device);
    if (status != cudaSuccess) return complete(kOpReduceNoAlloc, device, status);
    double* scratch = nullptr;
    cudaError_t e = scratch_for_current_device(device, &scratch);
    if (e != cudaSuccess) return complete(kOpReduceNoAlloc, device, static_cast<int>(e));

    EncodedShards shards{};
    shards.inputs = inputs;
    shards.outputs = outputs;
    bool vector_ok = first_value % 16 == 0;
    for (int k = 0; k < inputs; ++k) {
        if (!payloads[k] || !scales[k]) return complete(kOpReduceNoAlloc, device, static_cast<int>(cudaErrorInvalidValue));
        shards.payload[k] = payloads[k];
        shards.scales[k] = scales[k];
        vector_ok = vector_ok && (reinterpret_cast<std::uintptr_t>(payloads[k]) & 15u) == 0;
    }
    for (int d = 0; d < outputs; ++d) {
        if (!out_payloads[d] || !out_scales[d]) return complete(kOpReduceNoAlloc, device, static_cast<int>(cudaErrorInvalidValue));
        shards.out_payload[d] = out_payloads[d];
        shards.out_scales[d] = out_scales[d];
        vector_ok = vector_ok && (reinterpret_cast<std::uintptr_t>(out_payloads[d]) & 15u) == 0;
    }
    int* flag = reinterpret_cast<int*>(scratch + kFlagSlot);
    e = cudaMemsetAsync(flag, 0, sizeof(int), stream);      // the only word that must start at zero
    if (e != cudaSuccess) return complete(kOpReduceNoAlloc, device, static_cast<int>(e));
    const int grid = static_cast<int>(spans);
    if (block_size == 32)
        bfp8_reduce_reencode_spans_kernel<32><<<grid, kThreads, 0, stream>>>(shards, first_value, end_value, reduction_scale, scratch, flag, vector_ok);
    else if (block_size == 64)
        bfp8_reduce_reencode_spans_kernel<64><<<grid, kThreads, 0, stream>>>(shards, first_value, end_value, reduction_scale, scratch, flag, vector_ok);
    else
        bfp8_reduce_reencode_spans_kernel<128><<<grid, kThreads, 0, stream>>>(shards, first_value, end_value, reduction_scale, scratch, flag, vector_ok);
    if ((e = cudaPeekAtLastError()) != cudaSuccess) return complete(kOpReduceNoAlloc, device, static_cast<int>(e));
    sum_spans_kernel<<<1, kThreads, 0, stream>>>(scratch, grid, flag, squared_sum, finite_status);
    return complete(kOpReduceNoAlloc, device, static_cast<int>(cudaPeekAtLastError()));
}
