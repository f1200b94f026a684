// In-process N-rank gradient all-reduce (ABI minor 36): ONE host process
// drives all N devices, the way the reference's data-parallel engine does
// (one worker thread per device, NNtrain.Core/Training/CudaReplicaExecutor.cs:
// 29-116,339-369; whichever worker arrives last enqueues the cross-device
// work, NNtrain.Core/Training/CudaBfp8GradientAllReduce.cs:352-363).  The
// reference's reducers stop at two devices; this carries the same flow to N.
//
// Buffers are plain cudaMalloc pointers (no IPC): peer access between the
// devices is enabled when the group is created.  Ranks are ordered by CUDA
// events only -- every rank's stream waits for the other ranks' "arrived"
// events before its kernel reads their arenas, and for their "reduced" events
// before anything reads the gathered result -- so no kernel ever waits on
// memory another kernel writes, the whole step can be enqueued by one thread,
// and several ranks may even share one device (which is how the N-rank path is
// exercised on a single GPU).
//
// The kernel per rank is the same fused one as in the one-process-per-GPU
// path: 128-bit loads of the owned shard from every rank's arena, fp32
// accumulate in rank order, re-encode, 128-bit stores into every rank's arena.
#include "reduce_kernels.cuh"

#include <cstring>
#include <new>

namespace ngb {
namespace {

struct LocalGroup : GroupHeader {
    LocalGroup() : GroupHeader{kKindLocalGroup, CollectiveShape{0, 1, 0}} {}
    int ranks = 0;
    int device[kMaxRanks] = {};
    // per rank, on its device: [0] shard sum of squares, [1] flag carried as a
    // double, [3] the owner kernel's int flag
    double* scratch[kMaxRanks] = {};
    double** scratch_table[kMaxRanks] = {};   // per rank, on its device: the N scratch pointers
    cudaEvent_t arrived[kMaxRanks] = {};
    cudaEvent_t reduced[kMaxRanks] = {};
    cudaEvent_t published[kMaxRanks] = {};
};

constexpr int kPhaseBegin = 1;
constexpr int kPhaseEnd = 2;

__global__ void local_clear_partials_kernel(double* scratch, const int* finite_status) {
    scratch[0] = 0.0;
    scratch[1] = (finite_status != nullptr && *finite_status != 0) ? 1.0 : 0.0;
    *reinterpret_cast<int*>(scratch + 3) = 0;
}

__global__ void local_fold_flags_kernel(double* scratch, const int* finite_status) {
    if (*reinterpret_cast<const int*>(scratch + 3) != 0) scratch[1] += 1.0;
    if (finite_status != nullptr && *finite_status != 0) scratch[1] += 1.0;
}

// Sum of the ranks' partials in rank order (identical on every rank).
__global__ void local_publish_totals_kernel(double* const* scratch_by_rank, int ranks, double* squared_sum,
                                            int* finite_status) {
    double total = 0.0, flags = 0.0;
    for (int k = 0; k < ranks; ++k) {
        total += scratch_by_rank[k][0];
        flags += scratch_by_rank[k][1];
    }
    if (squared_sum != nullptr) *squared_sum += total;
    if (finite_status != nullptr && flags != 0.0) *finite_status = 1;
}

inline long long shard_size(long long length, int world) {
    const long long per = (length + world - 1) / world;
    return (per + 511) / 512 * 512;
}

inline void shard_range(long long length, int world, int rank, long long* first, long long* end) {
    const long long size = shard_size(length, world);
    long long a = size * rank, b = a + size;
    if (a > length) a = length;
    if (b > length) b = length;
    *first = a;
    *end = b;
}

int destroy_impl(LocalGroup* g) {
    if (!g) return 0;
    int first = 0;
    for (int r = 0; r < g->ranks; ++r) {
        int s = select_device(g->device[r]);
        if (s == 0) s = static_cast<int>(cudaDeviceSynchronize());
        if (first == 0) first = s;
        if (g->scratch[r]) cudaFree(g->scratch[r]);
        if (g->scratch_table[r]) cudaFree(g->scratch_table[r]);
        if (g->arrived[r]) cudaEventDestroy(g->arrived[r]);
        if (g->reduced[r]) cudaEventDestroy(g->reduced[r]);
        if (g->published[r]) cudaEventDestroy(g->published[r]);
    }
    delete g;
    return first;
}

int create_impl(int ranks, const int* devices, void** group) {
    if (!group || !devices || ranks < 1 || ranks > kMaxRanks) return static_cast<int>(cudaErrorInvalidValue);
    *group = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return static_cast<int>(e);
    for (int r = 0; r < ranks; ++r)
        if (devices[r] < 0 || devices[r] >= count) return static_cast<int>(cudaErrorInvalidDevice);
    LocalGroup* g = new (std::nothrow) LocalGroup();
    if (!g) return static_cast<int>(cudaErrorMemoryAllocation);
    g->ranks = ranks;
    g->shape = default_collective_shape();
    for (int r = 0; r < ranks; ++r) g->device[r] = devices[r];
    int status = 0;
    for (int r = 0; status == 0 && r < ranks; ++r) {
        status = select_device(devices[r]);
        for (int q = 0; status == 0 && q < ranks; ++q) {
            if (devices[q] == devices[r]) continue;
            int can = 0;
            e = cudaDeviceCanAccessPeer(&can, devices[r], devices[q]);
            if (e == cudaSuccess && !can) e = cudaErrorPeerAccessUnsupported;
            if (e == cudaSuccess) {
                e = cudaDeviceEnablePeerAccess(devices[q], 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) { e = cudaSuccess; cudaGetLastError(); }
            }
            status = static_cast<int>(e);
        }
        if (status == 0) e = cudaMalloc(reinterpret_cast<void**>(&g->scratch[r]), 4 * sizeof(double));
        if (status == 0 && e == cudaSuccess) e = cudaMemset(g->scratch[r], 0, 4 * sizeof(double));
        if (status == 0 && e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&g->scratch_table[r]), kMaxRanks * sizeof(double*));
        if (status == 0 && e == cudaSuccess) e = cudaEventCreateWithFlags(&g->arrived[r], cudaEventDisableTiming);
        if (status == 0 && e == cudaSuccess) e = cudaEventCreateWithFlags(&g->reduced[r], cudaEventDisableTiming);
        if (status == 0 && e == cudaSuccess) e = cudaEventCreateWithFlags(&g->published[r], cudaEventDisableTiming);
        if (status == 0) status = static_cast<int>(e);
    }
    for (int r = 0; status == 0 && r < ranks; ++r) {
        status = select_device(devices[r]);
        if (status == 0)
            status = static_cast<int>(cudaMemcpy(g->scratch_table[r], g->scratch, ranks * sizeof(double*),
                                                 cudaMemcpyHostToDevice));
    }
    if (status != 0) { destroy_impl(g); return status; }
    *group = g;
    return 0;
}

// Everything both all-reduce flavours share: the event choreography around
// one launch per rank.  `launch(r, first, end, squares, flag, stream)` enqueues
// rank r's owner kernel.
template <typename Launch>
int run_step(LocalGroup* g, long long length, int phase, double* const* squared_sum_by_rank,
             int* const* finite_status_by_rank, const cudaStream_t* streams, Launch launch) {
    const int ranks = g->ranks;
    cudaError_t e = cudaSuccess;
    int status = 0;
    // 1. every rank: (first chunk) reset its partials once nobody still reads
    //    them, then say "my encoded arena is ready".
    for (int r = 0; r < ranks; ++r) {
        if ((status = select_device(g->device[r])) != 0) return status;
        if (phase & kPhaseBegin) {
            for (int q = 0; q < ranks; ++q)
                if (q != r && (e = cudaStreamWaitEvent(streams[r], g->published[q], 0)) != cudaSuccess)
                    return static_cast<int>(e);
            local_clear_partials_kernel<<<1, 1, 0, streams[r]>>>(
                g->scratch[r], finite_status_by_rank ? finite_status_by_rank[r] : nullptr);
            if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
        }
        if ((e = cudaEventRecord(g->arrived[r], streams[r])) != cudaSuccess) return static_cast<int>(e);
    }
    // 2. every rank: wait for all arenas, reduce the owned shard into all arenas.
    for (int r = 0; r < ranks; ++r) {
        if ((status = select_device(g->device[r])) != 0) return status;
        for (int q = 0; q < ranks; ++q)
            if (q != r && (e = cudaStreamWaitEvent(streams[r], g->arrived[q], 0)) != cudaSuccess)
                return static_cast<int>(e);
        long long first = 0, end = 0;
        shard_range(length, ranks, r, &first, &end);
        if (end > first) {
            e = launch(r, first, end, g->scratch[r], reinterpret_cast<int*>(g->scratch[r] + 3), streams[r]);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        if (phase & kPhaseEnd) {
            local_fold_flags_kernel<<<1, 1, 0, streams[r]>>>(
                g->scratch[r], finite_status_by_rank ? finite_status_by_rank[r] : nullptr);
            if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
        }
        if ((e = cudaEventRecord(g->reduced[r], streams[r])) != cudaSuccess) return static_cast<int>(e);
    }
    // 3. every rank: its arena is complete once every owner has stored; (last
    //    chunk) add up the partials in rank order.
    for (int r = 0; r < ranks; ++r) {
        if ((status = select_device(g->device[r])) != 0) return status;
        for (int q = 0; q < ranks; ++q)
            if (q != r && (e = cudaStreamWaitEvent(streams[r], g->reduced[q], 0)) != cudaSuccess)
                return static_cast<int>(e);
        if (phase & kPhaseEnd) {
            local_publish_totals_kernel<<<1, 1, 0, streams[r]>>>(
                g->scratch_table[r], ranks, squared_sum_by_rank ? squared_sum_by_rank[r] : nullptr,
                finite_status_by_rank ? finite_status_by_rank[r] : nullptr);
            if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
            if ((e = cudaEventRecord(g->published[r], streams[r])) != cudaSuccess) return static_cast<int>(e);
        }
    }
    return 0;
}

// Restores the calling thread's device when the call ends.
struct DeviceScope {
    int original = -1;
    DeviceScope() { if (cudaGetDevice(&original) != cudaSuccess) original = -1; }
    ~DeviceScope() { if (original >= 0) select_device(original); }
};

}  // namespace
}  // namespace ngb

using namespace ngb;

// ranks devices of this process (a device may appear more than once: those
// ranks then share it).  Enables peer access between distinct devices.
NNTRAIN_EXPORT int nntrain_gradient_local_group_create(int ranks, const int* devices, void** group) {
    DeviceScope scope;
    return complete(kOpGradientLocalGroup, devices && ranks > 0 ? devices[0] : -1, create_impl(ranks, devices, group));
}

// Waits for the devices to go idle, then frees the group's scratch and events.
NNTRAIN_EXPORT int nntrain_gradient_local_group_destroy(void* group) {
    LocalGroup* g = static_cast<LocalGroup*>(group);
    if (!g) return 0;
    if (g->kind != kKindLocalGroup) return complete(kOpGradientLocalGroup, -1, static_cast<int>(cudaErrorInvalidValue));
    DeviceScope scope;
    const int device = g->device[0];
    return complete(kOpGradientLocalGroup, device, destroy_impl(g));
}

// In-place BFP8 all-reduce of one encoded arena (or one chunk of it) on every
// rank of the group, enqueued by the calling thread on streams[r] (rank r's
// communication stream; anything rank r's encode runs on must already be
// ordered before it).  On completion, in stream order on streams[r], rank r's
// arena holds encode(reduction_scale * rank-ordered sum) for every shard,
// bit-identical on all ranks.  phase as in nntrain_gradient_allreduce_bfp8;
// with bit 1, *squared_sum_by_rank[r] += the sum of squares of the decoded
// result and *finite_status_by_rank[r] = 1 when any rank saw a bad scale, a
// non-finite sum or had its flag raised (both tables optional).  All tables
// are host arrays.
NNTRAIN_EXPORT int nntrain_gradient_local_allreduce_bfp8(
    void* group, signed char* const* payload_by_rank, float* const* scales_by_rank, long long length,
    int block_size, float reduction_scale, double* const* squared_sum_by_rank, int* const* finite_status_by_rank,
    int phase, const cudaStream_t* streams) {
    LocalGroup* g = static_cast<LocalGroup*>(group);
    if (!g || g->kind != kKindLocalGroup || !payload_by_rank || !scales_by_rank || !streams || length <= 0 ||
        !std::isfinite(reduction_scale) || (block_size != 32 && block_size != 64 && block_size != 128) ||
        phase < 0 || phase > 3)
        return complete(kOpGradientLocalAllReduce, -1, static_cast<int>(cudaErrorInvalidValue));
    EncodedShards shards{};
    shards.inputs = shards.outputs = g->ranks;
    for (int k = 0; k < g->ranks; ++k) {
        if (!payload_by_rank[k] || !scales_by_rank[k])
            return complete(kOpGradientLocalAllReduce, g->device[k], static_cast<int>(cudaErrorInvalidValue));
        shards.payload[k] = shards.out_payload[k] = payload_by_rank[k];
        shards.scales[k] = shards.out_scales[k] = scales_by_rank[k];
    }
    DeviceScope scope;
    const CollectiveShape shape = g->shape;
    const int status = run_step(g, length, phase, squared_sum_by_rank, finite_status_by_rank, streams,
        [&](int, long long first, long long end, double* squares, int* flag, cudaStream_t stream) {
            return launch_bfp8_reduce_reencode(shards, first, end, block_size, reduction_scale, squares, flag,
                                               stream, &shape);
        });
    return complete(kOpGradientLocalAllReduce, g->device[0], status);
}

// bf16 twin: fp32 accumulate in rank order, bf16 (nearest even) result in
// every rank's arena, sum of squares of the bf16 result.
NNTRAIN_EXPORT int nntrain_gradient_local_allreduce_bf16(
    void* group, unsigned short* const* values_by_rank, long long length, float reduction_scale,
    double* const* squared_sum_by_rank, int phase, const cudaStream_t* streams) {
    LocalGroup* g = static_cast<LocalGroup*>(group);
    if (!g || g->kind != kKindLocalGroup || !values_by_rank || !streams || length <= 0 ||
        !std::isfinite(reduction_scale) || phase < 0 || phase > 3)
        return complete(kOpGradientLocalAllReduce, -1, static_cast<int>(cudaErrorInvalidValue));
    Bf16Inputs io{};
    io.inputs = io.outputs = g->ranks;
    for (int k = 0; k < g->ranks; ++k) {
        if (!values_by_rank[k])
            return complete(kOpGradientLocalAllReduce, g->device[k], static_cast<int>(cudaErrorInvalidValue));
        io.values[k] = io.out_bf16[k] = values_by_rank[k];
    }
    DeviceScope scope;
    const CollectiveShape shape = g->shape;
    const int status = run_step(g, length, phase, squared_sum_by_rank, nullptr, streams,
        [&](int, long long first, long long end, double* squares, int*, cudaStream_t stream) {
            return launch_bf16_reduce(io, nullptr, first, end, reduction_scale, squares, true, stream, &shape);
        });
    return complete(kOpGradientLocalAllReduce, g->device[0], status);
}

// Publication of parameters whose optimizer step is sharded over the ranks
// (the reference re-publishes every BFP8 data replica after a step,
// NNtrain.Core/Tensors/Tensor.Device.Bfp8.cs:593-649, with every device
// updating everything; here rank r updates and encodes shard r only): rank r
// encodes [shard r) of source_by_rank[r] (its fp32 master arena) and stores
// payload + scales into EVERY rank's encoded arena.  On completion, in stream
// order on streams[r], every rank holds encode(assembled parameters),
// bit-identical everywhere.  *finite_status_by_rank[r] (optional) is raised on
// every rank when any shard held a NaN / Inf.
NNTRAIN_EXPORT int nntrain_gradient_local_publish_shards_bfp8(
    void* group, const float* const* source_by_rank, signed char* const* payload_by_rank,
    float* const* scales_by_rank, long long length, int block_size, int* const* finite_status_by_rank,
    const cudaStream_t* streams) {
    LocalGroup* g = static_cast<LocalGroup*>(group);
    if (!g || g->kind != kKindLocalGroup || !source_by_rank || !payload_by_rank || !scales_by_rank || !streams ||
        length <= 0 || (block_size != 32 && block_size != 64 && block_size != 128))
        return complete(kOpGradientLocalAllReduce, -1, static_cast<int>(cudaErrorInvalidValue));
    EncodedShards shards{};
    shards.inputs = 0;
    shards.outputs = g->ranks;
    for (int k = 0; k < g->ranks; ++k) {
        if (!source_by_rank[k] || !payload_by_rank[k] || !scales_by_rank[k])
            return complete(kOpGradientLocalAllReduce, g->device[k], static_cast<int>(cudaErrorInvalidValue));
        shards.out_payload[k] = payload_by_rank[k];
        shards.out_scales[k] = scales_by_rank[k];
    }
    DeviceScope scope;
    const CollectiveShape shape{g->shape.ctas, 0, 0};
    const int status = run_step(g, length, 3, nullptr, finite_status_by_rank, streams,
        [&](int rank, long long first, long long end, double*, int* flag, cudaStream_t stream) {
            return launch_bfp8_encode_to_all(source_by_rank[rank], shards, first, end, block_size, flag, stream,
                                             &shape);
        });
    return complete(kOpGradientLocalAllReduce, g->device[0], status);
}
