// N-rank gradient all-reduce (ABI minor 36).  None of this has a counterpart
// in the reference, whose compressed reducers accept exactly two devices of
// one process (NNtrain.Core/Training/CudaBfp8GradientAllReduce.cs:44-49,
// CudaBFloat16GradientAllReduce.cs:119-124) and move whole buckets with
// cudaMemcpyPeerAsync.  The arithmetic is the reference's two-device reducer
// extended left to right over ranks 0..N-1.
//
// One process per GPU.  A "group" holds this rank's view of the job: world
// size, rank, device, an NCCL communicator (loaded at run time) and a few
// bytes of device scratch.  The encoded gradient arena of every rank
// (payload + scale sidecar, or bf16) lives in memory the other ranks can map
// (nntrain_gradient_peer_alloc / _open, CUDA IPC).  The arena is cut into N
// contiguous shards on 512-value boundaries; rank r owns shard r.
//
// Two transports:
//   peer (mode 0): after a stream-ordered barrier, ONE kernel per rank reads
//     its shard from every rank's arena over NVLink (128-bit peer loads),
//     accumulates in fp32 in rank order, re-encodes, and stores the result
//     into every rank's arena (128-bit peer stores).  Reduce-scatter, owner
//     arithmetic and all-gather are the same launch; nothing is staged.  A
//     second tiny collective both fences the stores and sums the per-shard
//     sum of squares / finite flag.
//   nccl (mode 1): grouped ncclSend/ncclRecv of encoded shards into local
//     staging, the same owner kernel on local memory, grouped send/recv of the
//     reduced shard.
//   copy engine (mode 2): the encoded shards are pulled from the peers' arenas
//     into local staging and the reduced shard is pushed into the peers'
//     arenas by the GPU's copy engines (cudaMemcpyAsync on peer-mapped
//     memory); the owner kernel runs on local memory.  No SM is spent on the
//     wire, so the codec kernels of neighbouring chunks overlap it freely.
// No kernel here spins on memory another rank writes: ordering between ranks
// comes only from collectives enqueued on the stream.
#include "reduce_kernels.cuh"
#include "launchers.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <type_traits>

namespace ngb {
namespace {

// ---- NCCL, resolved at run time ----------------------------------------------
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

constexpr int kNcclStatusBase = 10000;   // returned status = kNcclStatusBase + ncclResult_t
constexpr int kNcclMissing = 10099;

void load_nccl() {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* name : names) {
        g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) return;
    bool all = true;
    auto bind = [&](auto& slot, const char* symbol) {
        slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(dlsym(g_nccl.handle, symbol));
        if (!slot) all = false;
    };
    bind(g_nccl.GetUniqueId, "ncclGetUniqueId");
    bind(g_nccl.CommInitRank, "ncclCommInitRank");
    bind(g_nccl.CommDestroy, "ncclCommDestroy");
    bind(g_nccl.CommAbort, "ncclCommAbort");
    bind(g_nccl.CommGetAsyncError, "ncclCommGetAsyncError");
    bind(g_nccl.AllReduce, "ncclAllReduce");
    bind(g_nccl.AllGather, "ncclAllGather");
    bind(g_nccl.Send, "ncclSend");
    bind(g_nccl.Recv, "ncclRecv");
    bind(g_nccl.GroupStart, "ncclGroupStart");
    bind(g_nccl.GroupEnd, "ncclGroupEnd");
    g_nccl.ok = all;
}

const NcclApi* nccl() {
    std::call_once(g_nccl_once, load_nccl);
    return g_nccl.ok ? &g_nccl : nullptr;
}

inline int nccl_status(ncclResult_t r) { return r == ncclSuccess ? 0 : kNcclStatusBase + static_cast<int>(r); }

// ---- group ---------------------------------------------------------------------
struct Group : GroupHeader {
    Group() : GroupHeader{kKindProcessGroup, CollectiveShape{0, 1, 0}} {}
    int world = 1;
    int rank = 0;
    int device = 0;
    ncclComm_t comm = nullptr;
    double* scratch = nullptr;     // [0] shard sum of squares, [1] shard flag, [2] barrier token
    // copy-engine transport: two streams that carry the peer copies, and the
    // events that tie them to the caller's stream
    cudaStream_t wire[2] = {nullptr, nullptr};
    cudaEvent_t fork = nullptr;
    cudaEvent_t join[2] = {nullptr, nullptr};
};

// Makes both wire streams wait for everything enqueued on `stream` so far.
cudaError_t fork_wire(Group* g, cudaStream_t stream) {
    cudaError_t e = cudaEventRecord(g->fork, stream);
    for (int w = 0; e == cudaSuccess && w < 2; ++w) e = cudaStreamWaitEvent(g->wire[w], g->fork, 0);
    return e;
}

// Makes `stream` wait for everything enqueued on the wire streams so far.
cudaError_t join_wire(Group* g, cudaStream_t stream) {
    cudaError_t e = cudaSuccess;
    for (int w = 0; e == cudaSuccess && w < 2; ++w) {
        e = cudaEventRecord(g->join[w], g->wire[w]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, g->join[w], 0);
    }
    return e;
}

constexpr int kPhaseBegin = 1;   // first chunk of a step: reset the group's partials
constexpr int kPhaseEnd = 2;     // last chunk: fence + sum the partials over ranks, publish

// Start of a step: shard sum of squares = 0, shard flag = 0, and the flag
// that travels with the sum carries this rank's entry flag.
__global__ void clear_partials_kernel(double* scratch, const int* finite_status) {
    scratch[0] = 0.0;
    scratch[1] = (finite_status != nullptr && *finite_status != 0) ? 1.0 : 0.0;
    *reinterpret_cast<int*>(scratch + 3) = 0;
}

// Before the sum over ranks: fold the owner kernels' int flag, and a flag the
// caller raised since the step began (its encode kernels), into the double
// that travels with the sum of squares.
__global__ void fold_flags_kernel(double* scratch, const int* finite_status) {
    if (*reinterpret_cast<const int*>(scratch + 3) != 0) scratch[1] += 1.0;
    if (finite_status != nullptr && *finite_status != 0) scratch[1] += 1.0;
}

// After the sum over ranks: add the job-wide sum of squares, raise the flag.
__global__ void publish_totals_kernel(const double* scratch, double* squared_sum, int* finite_status) {
    if (squared_sum != nullptr) *squared_sum += scratch[0];
    if (finite_status != nullptr && scratch[1] != 0.0) *finite_status = 1;
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

int barrier(const Group* g, cudaStream_t stream) {
    const NcclApi* api = nccl();
    if (!api) return kNcclMissing;
    return nccl_status(api->AllReduce(g->scratch + 2, g->scratch + 2, 1, ncclDouble, ncclSum, g->comm, stream));
}

int sum_partials(const Group* g, cudaStream_t stream) {
    const NcclApi* api = nccl();
    if (!api) return kNcclMissing;
    return nccl_status(api->AllReduce(g->scratch, g->scratch, 2, ncclDouble, ncclSum, g->comm, stream));
}

}  // namespace
}  // namespace ngb

using namespace ngb;

// ---- peer-visible memory (CUDA IPC) ----------------------------------------------
// Allocates `bytes` on `device` with cudaMalloc and writes the 64-byte IPC
// handle other processes open with nntrain_gradient_peer_open.
static int gradient_peer_alloc_impl(int device, long long bytes, void** pointer, void* handle64) {
    if (!pointer || !handle64 || bytes <= 0) return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaIpcMemHandle_t handle;
    e = cudaIpcGetMemHandle(&handle, p);
    if (e != cudaSuccess) { cudaFree(p); return static_cast<int>(e); }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    std::memcpy(handle64, &handle, 64);
    *pointer = p;
    return 0;
}

static int gradient_peer_free_impl(int device, void* pointer) {
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(cudaFree(pointer));
}

// Maps another process's allocation into this process on `device` (peer
// access is enabled lazily by the runtime).
static int gradient_peer_open_impl(int device, const void* handle64, void** pointer) {
    if (!handle64 || !pointer) return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    cudaIpcMemHandle_t handle;
    std::memcpy(&handle, handle64, 64);
    return static_cast<int>(cudaIpcOpenMemHandle(pointer, handle, cudaIpcMemLazyEnablePeerAccess));
}

static int gradient_peer_close_impl(int device, void* pointer) {
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    return static_cast<int>(cudaIpcCloseMemHandle(pointer));
}

// ---- group -------------------------------------------------------------------------
// 128-byte NCCL unique id; rank 0 creates it and hands it to the other ranks
// by whatever channel the host has.
NNTRAIN_EXPORT int nntrain_gradient_group_unique_id(void* id128) {
    if (!id128) return static_cast<int>(cudaErrorInvalidValue);
    const NcclApi* api = nccl();
    if (!api) return kNcclMissing;
    ncclUniqueId id;
    int status = nccl_status(api->GetUniqueId(&id));
    if (status == 0) std::memcpy(id128, &id, sizeof(id));
    return status;
}

namespace {

int group_destroy_impl(Group* g) {
    if (!g) return 0;
    int first = select_device(g->device);
    if (g->comm) {
        const NcclApi* api = nccl();
        if (api) { int s = nccl_status(api->CommDestroy(g->comm)); if (first == 0) first = s; }
    }
    if (g->scratch) { int s = static_cast<int>(cudaFree(g->scratch)); if (first == 0) first = s; }
    for (int w = 0; w < 2; ++w) {
        if (g->wire[w]) { cudaStreamSynchronize(g->wire[w]); cudaStreamDestroy(g->wire[w]); }
        if (g->join[w]) cudaEventDestroy(g->join[w]);
    }
    if (g->fork) cudaEventDestroy(g->fork);
    delete g;
    return first;
}

int group_create_impl(const void* id128, int world, int rank, int device, void** group) {
    if (!group || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || (world > 1 && !id128))
        return static_cast<int>(cudaErrorInvalidValue);
    *group = nullptr;
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    Group* g = new (std::nothrow) Group();
    if (!g) return static_cast<int>(cudaErrorMemoryAllocation);
    g->world = world;
    g->rank = rank;
    g->device = device;
    g->shape = default_collective_shape();
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&g->scratch), 4 * sizeof(double));
    if (e == cudaSuccess) e = cudaMemset(g->scratch, 0, 4 * sizeof(double));
    for (int w = 0; e == cudaSuccess && w < 2; ++w) {
        e = cudaStreamCreateWithFlags(&g->wire[w], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&g->join[w], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&g->fork, cudaEventDisableTiming);
    status = static_cast<int>(e);
    if (status == 0 && world > 1) {
        const NcclApi* api = nccl();
        if (!api) status = kNcclMissing;
        else {
            ncclUniqueId id;
            std::memcpy(&id, id128, sizeof(id));
            status = nccl_status(api->CommInitRank(&g->comm, world, id, rank));
            if (status != 0) g->comm = nullptr;
        }
    }
    // one way out for every failure: whatever was created is released
    if (status != 0) { group_destroy_impl(g); return status; }
    *group = g;
    return 0;
}

}  // namespace

// Collective over all ranks.  world == 1 needs no id and no NCCL.  The
// group's launch shape for its all-reduce kernels starts as the process-wide
// default and is changed with nntrain_gradient_group_configure.
NNTRAIN_EXPORT int nntrain_gradient_group_create(const void* id128, int world, int rank, int device, void** group) {
    return complete(kOpGradientGroup, device, group_create_impl(id128, world, rank, device, group));
}

NNTRAIN_EXPORT int nntrain_gradient_group_destroy(void* group) {
    Group* g = static_cast<Group*>(group);
    if (!g) return 0;
    const int device = g->device;
    return complete(kOpGradientGroup, device, group_destroy_impl(g));
}

// Launch shape of this group's all-reduce kernels (peer transport).
// collective_ctas: 0 = fill the machine, n > 0 = at most n CTAs.
// asynchronous_copies: 0 = register prefetch, 1 = cp.async rings, 2 = bulk
// asynchronous copies of whole tiles.
// exclusive_sms: 1 (with asynchronous_copies) = every CTA takes a whole SM, so
// collective_ctas SMs belong to the all-reduce while it runs and the codec
// kernels of the neighbouring chunks keep the rest to themselves.
NNTRAIN_EXPORT int nntrain_gradient_group_configure(void* group, int collective_ctas, int asynchronous_copies,
                                                    int exclusive_sms) {
    GroupHeader* header = static_cast<GroupHeader*>(group);
    if (!header || (header->kind != kKindProcessGroup && header->kind != kKindLocalGroup) || collective_ctas < 0)
        return complete(kOpGradientGroup, -1, static_cast<int>(cudaErrorInvalidValue));
    if (asynchronous_copies < 0 || asynchronous_copies > 2)
        return complete(kOpGradientGroup, -1, static_cast<int>(cudaErrorInvalidValue));
    header->shape = CollectiveShape{collective_ctas, asynchronous_copies,
                                    (exclusive_sms != 0 && asynchronous_copies != 0) ? 1 : 0};
    return 0;
}

// Host-side liveness check: 0 = healthy, otherwise the communicator's
// asynchronous error (kNcclStatusBase + code).  Never blocks.
NNTRAIN_EXPORT int nntrain_gradient_group_poll(void* group) {
    Group* g = static_cast<Group*>(group);
    if (!g) return static_cast<int>(cudaErrorInvalidValue);
    if (!g->comm) return 0;
    const NcclApi* api = nccl();
    if (!api) return kNcclMissing;
    ncclResult_t async = ncclSuccess;
    int status = nccl_status(api->CommGetAsyncError(g->comm, &async));
    if (status != 0) return status;
    return nccl_status(async == ncclInProgress ? ncclSuccess : async);
}

// Tears the communicator down without waiting for outstanding work (after a
// peer was declared lost by the host).
NNTRAIN_EXPORT int nntrain_gradient_group_abort(void* group) {
    Group* g = static_cast<Group*>(group);
    if (!g || !g->comm) return 0;
    const NcclApi* api = nccl();
    if (!api) return kNcclMissing;
    int status = nccl_status(api->CommAbort(g->comm));
    g->comm = nullptr;
    return status;
}

// Shard r of an arena of `length` values split over `world` ranks.
NNTRAIN_EXPORT int nntrain_gradient_shard_range(long long length, int world, int rank, long long* first,
                                                long long* end) {
    if (length < 0 || world < 1 || rank < 0 || rank >= world || !first || !end)
        return static_cast<int>(cudaErrorInvalidValue);
    shard_range(length, world, rank, first, end);
    return 0;
}

// ---- the owner kernels on caller-supplied pointer tables ----------------------------
// Pointer tables are HOST arrays of device pointers (local or peer-mapped).
// r = reduction_scale * (rank-ordered fp32 sum of decoded inputs) over
// [first_value, end_value), re-encoded in blocks of block_size (32/64/128)
// and stored to every output.  first_value must be a multiple of block_size.
static int gradient_reduce_shards_bfp8_impl(
    int device, int inputs, const signed char* const* payloads, const float* const* scales, int outputs,
    signed char* const* out_payloads, float* const* out_scales, long long first_value, long long end_value,
    int block_size, float reduction_scale, double* squared_sum, int* finite_status, cudaStream_t stream) {
    if (inputs < 1 || inputs > kMaxRanks || outputs < 1 || outputs > kMaxRanks || !payloads || !scales ||
        !out_payloads || !out_scales || !std::isfinite(reduction_scale))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    EncodedShards shards{};
    shards.inputs = inputs;
    shards.outputs = outputs;
    for (int k = 0; k < inputs; ++k) { shards.payload[k] = payloads[k]; shards.scales[k] = scales[k]; }
    for (int d = 0; d < outputs; ++d) { shards.out_payload[d] = out_payloads[d]; shards.out_scales[d] = out_scales[d]; }
    return static_cast<int>(launch_bfp8_reduce_reencode(shards, first_value, end_value, block_size,
                                                        reduction_scale, squared_sum, finite_status, stream));
}

// bf16 twin: fp32 accumulate in rank order, optional fp32 output (local),
// bf16 round-to-nearest-even outputs, optional sum of squares of the bf16
// result (square_of_bf16 != 0) or of the fp32 sum.
static int gradient_reduce_shards_bf16_impl(
    int device, int inputs, const unsigned short* const* values, int outputs, unsigned short* const* out_values,
    float* reduced, long long first_value, long long end_value, float reduction_scale, double* squared_sum,
    int square_of_bf16, cudaStream_t stream) {
    if (inputs < 1 || inputs > kMaxRanks || outputs < 0 || outputs > kMaxRanks || !values ||
        (outputs > 0 && !out_values) || !std::isfinite(reduction_scale))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(device);
    if (status != cudaSuccess) return status;
    Bf16Inputs io{};
    io.inputs = inputs;
    io.outputs = outputs;
    for (int k = 0; k < inputs; ++k) io.values[k] = values[k];
    for (int d = 0; d < outputs; ++d) io.out_bf16[d] = out_values[d];
    return static_cast<int>(launch_bf16_reduce(io, reduced, first_value, end_value, reduction_scale, squared_sum,
                                               square_of_bf16 != 0, stream));
}

// ---- the all-reduce ---------------------------------------------------------------------
// BFP8 all-reduce of one arena (or one chunk of it), in place: on entry
// payload_by_rank[k] / scales_by_rank[k] address rank k's encoded arena as
// mapped in this process (entry `rank` is this rank's own); on completion (in
// stream order) this rank's arena holds encode(reduction_scale * sum) for
// every shard, bit-identical on all ranks.  *squared_sum += the sum of
// squares of the whole reduced arena's decoded values; *finite_status = 1 if
// any rank saw an invalid scale or a non-finite sum, or had its flag raised
// (by its encode kernels) when the step ended.  `phase` lets a caller cut one
// step into chunks that overlap with its encode / decode kernels: bit 0 on the
// first chunk (reset the group's partials), bit 1 on the last (fence, sum the
// partials over ranks, publish); 3 for a whole arena in one call.  Without
// bit 1 the chunk's result must not be read before a later collective on the
// group has completed (the next chunk's leading barrier is one): when
// `previous_final` is given it is recorded on `stream` right behind this
// call's leading barrier, i.e. at the point where every EARLIER chunk of the
// step is complete on this rank.  mode 0 = peer memory, one fused kernel; mode 2 = copy engines through the same staging; mode 1 = NCCL send/recv
// through staging_payload / staging_scales (capacity: world shards).
// Collective: every rank must call it with the same length / block / mode, in
// the same order relative to other calls on the group.
static int gradient_allreduce_bfp8_impl(
    void* group, signed char* const* payload_by_rank, float* const* scales_by_rank, long long length,
    int block_size, float reduction_scale, double* squared_sum, int* finite_status, int mode, int phase,
    signed char* staging_payload, float* staging_scales, cudaEvent_t previous_final, cudaStream_t stream) {
    Group* g = static_cast<Group*>(group);
    if (!g || !payload_by_rank || !scales_by_rank || length <= 0 || !std::isfinite(reduction_scale) ||
        (block_size != 32 && block_size != 64 && block_size != 128) || mode < 0 || mode > 2 ||
        phase < 0 || phase > 3)
        return static_cast<int>(cudaErrorInvalidValue);
    if (mode != 0 && g->world > 1 && (!staging_payload || !staging_scales))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(g->device);
    if (status != cudaSuccess) return status;
    const int world = g->world, rank = g->rank;
    long long first = 0, end = 0;
    shard_range(length, world, rank, &first, &end);
    const long long shard = shard_size(length, world);

    cudaError_t e = cudaSuccess;
    int* shard_flag = reinterpret_cast<int*>(g->scratch + 3);
    if (phase & kPhaseBegin) {
        clear_partials_kernel<<<1, 1, 0, stream>>>(g->scratch, finite_status);
        if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
    }

    // owner kernels that read staged (local) shards are short: they fill the machine
    const CollectiveShape local_shape{0, g->shape.asynchronous, 0};
    EncodedShards shards{};
    shards.inputs = world;
    if (mode == 0 || world == 1) {
        // Every rank's encode must have finished before anyone reads it.
        if (world > 1 && (status = barrier(g, stream)) != 0) return status;
        if (previous_final != nullptr && (e = cudaEventRecord(previous_final, stream)) != cudaSuccess)
            return static_cast<int>(e);
        shards.outputs = world;
        for (int k = 0; k < world; ++k) {
            if (!payload_by_rank[k] || !scales_by_rank[k]) return static_cast<int>(cudaErrorInvalidValue);
            shards.payload[k] = payload_by_rank[k];
            shards.scales[k] = scales_by_rank[k];
            // own arena first in the store order is irrelevant; all get the same bytes
            shards.out_payload[k] = payload_by_rank[k];
            shards.out_scales[k] = scales_by_rank[k];
        }
        if (end > first) {
            e = launch_bfp8_reduce_reencode(shards, first, end, block_size, reduction_scale, g->scratch,
                                            shard_flag, stream, &g->shape);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
    } else if (mode == 2) {
        // Copy-engine transport: the SMs stay free for the codec kernels of
        // the neighbouring chunks.  Pull my shard from every peer into staging,
        // reduce locally, push the reduced shard into every peer's arena.  The
        // leading barrier says every rank's encode of this chunk is done (and
        // that the previous chunk's pushes have landed); the pushes of this
        // chunk are fenced by the next collective on the group.
        signed char* own_payload = payload_by_rank[rank];
        float* own_scales = scales_by_rank[rank];
        if (!own_payload || !own_scales) return static_cast<int>(cudaErrorInvalidValue);
        for (int k = 0; k < world; ++k)
            if (!payload_by_rank[k] || !scales_by_rank[k]) return static_cast<int>(cudaErrorInvalidValue);
        const long long shard_scales = shard / block_size;
        if ((status = barrier(g, stream)) != 0) return status;
        if (previous_final != nullptr && (e = cudaEventRecord(previous_final, stream)) != cudaSuccess)
            return static_cast<int>(e);
        if (end > first) {
            const long long sa = first / block_size, sb = (end + block_size - 1) / block_size;
            if ((e = fork_wire(g, stream)) != cudaSuccess) return static_cast<int>(e);
            for (int step = 1; step < world; ++step) {
                const int peer = (rank + step) % world;
                cudaStream_t lane = g->wire[step & 1];
                e = cudaMemcpyAsync(staging_payload + shard * peer, payload_by_rank[peer] + first,
                                    static_cast<size_t>(end - first), cudaMemcpyDeviceToDevice, lane);
                if (e == cudaSuccess)
                    e = cudaMemcpyAsync(staging_scales + shard_scales * peer, scales_by_rank[peer] + sa,
                                        static_cast<size_t>(sb - sa) * sizeof(float), cudaMemcpyDeviceToDevice, lane);
                if (e != cudaSuccess) return static_cast<int>(e);
            }
            if ((e = join_wire(g, stream)) != cudaSuccess) return static_cast<int>(e);
            shards.outputs = 1;
            for (int k = 0; k < world; ++k) {
                if (k == rank) { shards.payload[k] = own_payload; shards.scales[k] = own_scales; }
                else {
                    shards.payload[k] = staging_payload + shard * k - first;
                    shards.scales[k] = staging_scales + shard_scales * k - sa;
                }
            }
            shards.out_payload[0] = own_payload;
            shards.out_scales[0] = own_scales;
            e = launch_bfp8_reduce_reencode(shards, first, end, block_size, reduction_scale, g->scratch,
                                            shard_flag, stream, &local_shape);
            if (e != cudaSuccess) return static_cast<int>(e);
            if ((e = fork_wire(g, stream)) != cudaSuccess) return static_cast<int>(e);
            for (int step = 1; step < world; ++step) {
                const int peer = (rank + step) % world;
                cudaStream_t lane = g->wire[step & 1];
                e = cudaMemcpyAsync(payload_by_rank[peer] + first, own_payload + first,
                                    static_cast<size_t>(end - first), cudaMemcpyDeviceToDevice, lane);
                if (e == cudaSuccess)
                    e = cudaMemcpyAsync(scales_by_rank[peer] + sa, own_scales + sa,
                                        static_cast<size_t>(sb - sa) * sizeof(float), cudaMemcpyDeviceToDevice, lane);
                if (e != cudaSuccess) return static_cast<int>(e);
            }
            if ((e = join_wire(g, stream)) != cudaSuccess) return static_cast<int>(e);
        }
    } else {
        const NcclApi* api = nccl();
        if (!api) return kNcclMissing;
        // with send/recv every earlier chunk is already final in stream order
        if (previous_final != nullptr && (e = cudaEventRecord(previous_final, stream)) != cudaSuccess)
            return static_cast<int>(e);
        signed char* own_payload = payload_by_rank[rank];
        float* own_scales = scales_by_rank[rank];
        if (!own_payload || !own_scales) return static_cast<int>(cudaErrorInvalidValue);
        const long long shard_scales = shard / block_size;
        // reduce-scatter: my copy of shard p goes to rank p; rank p's copy of
        // my shard lands in staging slot p.
        if ((status = nccl_status(api->GroupStart())) != 0) return status;
        for (int step = 1; step < world; ++step) {
            const int to = (rank + step) % world, from = (rank - step + world) % world;
            long long a = 0, b = 0;
            shard_range(length, world, to, &a, &b);
            if (b > a) {
                const long long sa = a / block_size, sb = (b + block_size - 1) / block_size;
                status = nccl_status(api->Send(own_payload + a, b - a, ncclInt8, to, g->comm, stream));
                if (status == 0) status = nccl_status(api->Send(own_scales + sa, sb - sa, ncclFloat, to, g->comm, stream));
            }
            if (status == 0 && end > first) {
                const long long sa = first / block_size, sb = (end + block_size - 1) / block_size;
                status = nccl_status(api->Recv(staging_payload + shard * from, end - first, ncclInt8, from, g->comm, stream));
                if (status == 0) status = nccl_status(api->Recv(staging_scales + shard_scales * from, sb - sa, ncclFloat, from, g->comm, stream));
            }
            if (status != 0) { api->GroupEnd(); return status; }
        }
        if ((status = nccl_status(api->GroupEnd())) != 0) return status;
        if (end > first) {
            // staging slot k holds rank k's shard starting at value index
            // `first`; bias the pointers so the kernel indexes them like arenas.
            shards.outputs = 1;
            for (int k = 0; k < world; ++k) {
                if (k == rank) { shards.payload[k] = own_payload; shards.scales[k] = own_scales; }
                else {
                    shards.payload[k] = staging_payload + shard * k - first;
                    shards.scales[k] = staging_scales + shard_scales * k - first / block_size;
                }
            }
            shards.out_payload[0] = own_payload;
            shards.out_scales[0] = own_scales;
            e = launch_bfp8_reduce_reencode(shards, first, end, block_size, reduction_scale, g->scratch,
                                            shard_flag, stream, &local_shape);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        // all-gather of the reduced shards, in place in the arena
        if ((status = nccl_status(api->GroupStart())) != 0) return status;
        for (int step = 1; step < world; ++step) {
            const int to = (rank + step) % world, from = (rank - step + world) % world;
            if (end > first) {
                const long long sa = first / block_size, sb = (end + block_size - 1) / block_size;
                status = nccl_status(api->Send(own_payload + first, end - first, ncclInt8, to, g->comm, stream));
                if (status == 0) status = nccl_status(api->Send(own_scales + sa, sb - sa, ncclFloat, to, g->comm, stream));
            }
            long long a = 0, b = 0;
            shard_range(length, world, from, &a, &b);
            if (status == 0 && b > a) {
                const long long sa = a / block_size, sb = (b + block_size - 1) / block_size;
                status = nccl_status(api->Recv(own_payload + a, b - a, ncclInt8, from, g->comm, stream));
                if (status == 0) status = nccl_status(api->Recv(own_scales + sa, sb - sa, ncclFloat, from, g->comm, stream));
            }
            if (status != 0) { api->GroupEnd(); return status; }
        }
        if ((status = nccl_status(api->GroupEnd())) != 0) return status;
    }

    if (!(phase & kPhaseEnd)) return 0;
    fold_flags_kernel<<<1, 1, 0, stream>>>(g->scratch, finite_status);
    if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
    // Sum of the shards' partials over ranks; in peer mode this collective is
    // also the fence after which every rank's arena is complete.
    if (world > 1 && (status = sum_partials(g, stream)) != 0) return status;
    publish_totals_kernel<<<1, 1, 0, stream>>>(g->scratch, squared_sum, finite_status);
    return static_cast<int>(cudaPeekAtLastError());
}

// bf16 arena all-reduce, in place: fp32 accumulate in rank order, result
// rounded to bf16 (nearest even) and stored into every rank's arena;
// *squared_sum += sum of squares of the bf16 result.  Modes as above
// (staging: world shards of bf16).
static int gradient_allreduce_bf16_impl(
    void* group, unsigned short* const* values_by_rank, long long length, float reduction_scale,
    double* squared_sum, int mode, int phase, unsigned short* staging, cudaStream_t stream) {
    Group* g = static_cast<Group*>(group);
    if (!g || !values_by_rank || length <= 0 || !std::isfinite(reduction_scale) || (mode != 0 && mode != 1) ||
        phase < 0 || phase > 3)
        return static_cast<int>(cudaErrorInvalidValue);
    if (mode == 1 && g->world > 1 && !staging) return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(g->device);
    if (status != cudaSuccess) return status;
    const int world = g->world, rank = g->rank;
    long long first = 0, end = 0;
    shard_range(length, world, rank, &first, &end);
    const long long shard = shard_size(length, world);

    cudaError_t e = cudaSuccess;
    if (phase & kPhaseBegin) {
        clear_partials_kernel<<<1, 1, 0, stream>>>(g->scratch, nullptr);
        if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
    }

    Bf16Inputs io{};
    io.inputs = world;
    if (mode == 0 || world == 1) {
        if (world > 1 && (status = barrier(g, stream)) != 0) return status;
        io.outputs = world;
        for (int k = 0; k < world; ++k) {
            if (!values_by_rank[k]) return static_cast<int>(cudaErrorInvalidValue);
            io.values[k] = values_by_rank[k];
            io.out_bf16[k] = values_by_rank[k];
        }
        if (end > first) {
            e = launch_bf16_reduce(io, nullptr, first, end, reduction_scale, g->scratch, true, stream, &g->shape);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
    } else {
        const NcclApi* api = nccl();
        if (!api) return kNcclMissing;
        unsigned short* own = values_by_rank[rank];
        if (!own) return static_cast<int>(cudaErrorInvalidValue);
        if ((status = nccl_status(api->GroupStart())) != 0) return status;
        for (int step = 1; step < world; ++step) {
            const int to = (rank + step) % world, from = (rank - step + world) % world;
            long long a = 0, b = 0;
            shard_range(length, world, to, &a, &b);
            if (b > a) status = nccl_status(api->Send(own + a, b - a, ncclBfloat16, to, g->comm, stream));
            if (status == 0 && end > first)
                status = nccl_status(api->Recv(staging + shard * from, end - first, ncclBfloat16, from, g->comm, stream));
            if (status != 0) { api->GroupEnd(); return status; }
        }
        if ((status = nccl_status(api->GroupEnd())) != 0) return status;
        if (end > first) {
            io.outputs = 1;
            for (int k = 0; k < world; ++k) io.values[k] = k == rank ? own : staging + shard * k - first;
            io.out_bf16[0] = own;
            e = launch_bf16_reduce(io, nullptr, first, end, reduction_scale, g->scratch, true, stream);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        if ((status = nccl_status(api->GroupStart())) != 0) return status;
        for (int step = 1; step < world; ++step) {
            const int to = (rank + step) % world, from = (rank - step + world) % world;
            if (end > first) status = nccl_status(api->Send(own + first, end - first, ncclBfloat16, to, g->comm, stream));
            long long a = 0, b = 0;
            shard_range(length, world, from, &a, &b);
            if (status == 0 && b > a) status = nccl_status(api->Recv(own + a, b - a, ncclBfloat16, from, g->comm, stream));
            if (status != 0) { api->GroupEnd(); return status; }
        }
        if ((status = nccl_status(api->GroupEnd())) != 0) return status;
    }
    if (!(phase & kPhaseEnd)) return 0;
    if (world > 1 && (status = sum_partials(g, stream)) != 0) return status;
    publish_totals_kernel<<<1, 1, 0, stream>>>(g->scratch, squared_sum, nullptr);
    return static_cast<int>(cudaPeekAtLastError());
}

// Publication of parameters whose optimizer step is sharded over the ranks:
// this rank encodes its shard of `source` (its fp32 master arena) and stores
// payload + scales into every rank's encoded arena (peer stores); a leading
// barrier makes sure nobody still reads the previous publication, the closing
// collective fences the stores and spreads the finite flag.  Collective.
static int gradient_publish_shards_bfp8_impl(void* group, const float* source, signed char* const* payload_by_rank,
                                             float* const* scales_by_rank, long long length, int block_size,
                                             int* finite_status, cudaStream_t stream) {
    Group* g = static_cast<Group*>(group);
    if (!g || !source || !payload_by_rank || !scales_by_rank || length <= 0 ||
        (block_size != 32 && block_size != 64 && block_size != 128))
        return static_cast<int>(cudaErrorInvalidValue);
    int status = select_device(g->device);
    if (status != cudaSuccess) return status;
    const int world = g->world, rank = g->rank;
    long long first = 0, end = 0;
    shard_range(length, world, rank, &first, &end);
    clear_partials_kernel<<<1, 1, 0, stream>>>(g->scratch, finite_status);
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    if (world > 1 && (status = barrier(g, stream)) != 0) return status;
    EncodedShards shards{};
    shards.outputs = world;
    for (int k = 0; k < world; ++k) {
        if (!payload_by_rank[k] || !scales_by_rank[k]) return static_cast<int>(cudaErrorInvalidValue);
        shards.out_payload[k] = payload_by_rank[k];
        shards.out_scales[k] = scales_by_rank[k];
    }
    if (end > first) {
        const CollectiveShape shape{g->shape.ctas, 0, 0};
        e = launch_bfp8_encode_to_all(source, shards, first, end, block_size, reinterpret_cast<int*>(g->scratch + 3),
                                      stream, &shape);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    fold_flags_kernel<<<1, 1, 0, stream>>>(g->scratch, finite_status);
    if ((e = cudaPeekAtLastError()) != cudaSuccess) return static_cast<int>(e);
    if (world > 1 && (status = sum_partials(g, stream)) != 0) return status;
    publish_totals_kernel<<<1, 1, 0, stream>>>(g->scratch, nullptr, finite_status);
    return static_cast<int>(cudaPeekAtLastError());
}

NNTRAIN_EXPORT int nntrain_gradient_publish_shards_bfp8(void* group, const float* source,
                                                        signed char* const* payload_by_rank,
                                                        float* const* scales_by_rank, long long length,
                                                        int block_size, int* finite_status, cudaStream_t stream) {
    return complete(kOpGradientAllReduce, group ? static_cast<Group*>(group)->device : -1,
                    gradient_publish_shards_bfp8_impl(group, source, payload_by_rank, scales_by_rank, length,
                                                      block_size, finite_status, stream));
}

// Sums `count` doubles over the ranks in place (stream-ordered); with
// count == 0 it is a pure barrier.  For host-side quantities that ride along
// with a step (global norm pieces, flags).
static int gradient_group_sum_impl(void* group, double* values, int count, cudaStream_t stream) {
    Group* g = static_cast<Group*>(group);
    if (!g || count < 0 || (count > 0 && !values)) return static_cast<int>(cudaErrorInvalidValue);
    if (g->world == 1) return 0;
    int status = select_device(g->device);
    if (status != cudaSuccess) return status;
    if (count == 0) return barrier(g, stream);
    const NcclApi* api = nccl();
    if (!api) return kNcclMissing;
    return nccl_status(api->AllReduce(values, values, static_cast<size_t>(count), ncclDouble, ncclSum, g->comm, stream));
}

// cudaStreamWaitEvent for hosts that hold only the opaque handles (the
// reference's exchange entry points do this internally,
// NNtrain.Cuda/native/gradient_collectives.cu:284-291).
NNTRAIN_EXPORT int nntrain_gradient_stream_wait_event(cudaStream_t stream, cudaEvent_t event) {
    if (!event) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(cudaStreamWaitEvent(stream, event, 0));
}

// ---- exports: every failure is recorded in the error ring (nntrain_last_error) -----------
NNTRAIN_EXPORT int nntrain_gradient_peer_alloc(int device, long long bytes, void** pointer, void* handle64) {
    return complete(kOpGradientPeerMemory, device,
                    gradient_peer_alloc_impl(device, bytes, pointer, handle64));
}

NNTRAIN_EXPORT int nntrain_gradient_peer_free(int device, void* pointer) {
    return complete(kOpGradientPeerMemory, device,
                    gradient_peer_free_impl(device, pointer));
}

NNTRAIN_EXPORT int nntrain_gradient_peer_open(int device, const void* handle64, void** pointer) {
    return complete(kOpGradientPeerMemory, device,
                    gradient_peer_open_impl(device, handle64, pointer));
}

NNTRAIN_EXPORT int nntrain_gradient_peer_close(int device, void* pointer) {
    return complete(kOpGradientPeerMemory, device,
                    gradient_peer_close_impl(device, pointer));
}

NNTRAIN_EXPORT int nntrain_gradient_reduce_shards_bfp8(int device, int inputs, const signed char* const* payloads, const float* const* scales, int outputs, signed char* const* out_payloads, float* const* out_scales, long long first_value, long long end_value, int block_size, float reduction_scale, double* squared_sum, int* finite_status, cudaStream_t stream) {
    return complete(kOpGradientReduceShards, device,
                    gradient_reduce_shards_bfp8_impl(device, inputs, payloads, scales, outputs, out_payloads, out_scales, first_value, end_value, block_size, reduction_scale, squared_sum, finite_status, stream));
}

NNTRAIN_EXPORT int nntrain_gradient_reduce_shards_bf16(int device, int inputs, const unsigned short* const* values, int outputs, unsigned short* const* out_values, float* reduced, long long first_value, long long end_value, float reduction_scale, double* squared_sum, int square_of_bf16, cudaStream_t stream) {
    return complete(kOpGradientReduceShards, device,
                    gradient_reduce_shards_bf16_impl(device, inputs, values, outputs, out_values, reduced, first_value, end_value, reduction_scale, squared_sum, square_of_bf16, stream));
}

NNTRAIN_EXPORT int nntrain_gradient_allreduce_bfp8(void* group, signed char* const* payload_by_rank, float* const* scales_by_rank, long long length, int block_size, float reduction_scale, double* squared_sum, int* finite_status, int mode, int phase, signed char* staging_payload, float* staging_scales, cudaEvent_t previous_final, cudaStream_t stream) {
    return complete(kOpGradientAllReduce, group ? static_cast<Group*>(group)->device : -1,
                    gradient_allreduce_bfp8_impl(group, payload_by_rank, scales_by_rank, length, block_size, reduction_scale, squared_sum, finite_status, mode, phase, staging_payload, staging_scales, previous_final, stream));
}

NNTRAIN_EXPORT int nntrain_gradient_allreduce_bf16(void* group, unsigned short* const* values_by_rank, long long length, float reduction_scale, double* squared_sum, int mode, int phase, unsigned short* staging, cudaStream_t stream) {
    return complete(kOpGradientAllReduce, group ? static_cast<Group*>(group)->device : -1,
                    gradient_allreduce_bf16_impl(group, values_by_rank, length, reduction_scale, squared_sum, mode, phase, staging, stream));
}

NNTRAIN_EXPORT int nntrain_gradient_group_sum(void* group, double* values, int count, cudaStream_t stream) {
    return complete(kOpGradientGroup, group ? static_cast<Group*>(group)->device : -1,
                    gradient_group_sum_impl(group, values, count, stream));
}
