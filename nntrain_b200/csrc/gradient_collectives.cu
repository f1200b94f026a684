// Bucketed BF16 / block-BFP8 gradient transport between two devices of one
// process: communication streams and ready events, bucket pack kernels, the
// peer-copy exchange, the pinned-host fallback pipeline and the fp32 unpack.
//
// Replaces, signature for signature, NNtrain.Cuda/native/gradient_collectives.cu:
//   nntrain_gradient_comm_create / _event_create                 :213-227
//   nntrain_gradient_pack_bf16 / _pack_bfp8_block                :229-252
//   nntrain_gradient_record_ready / _record_ready_external       :254-270
//   nntrain_gradient_exchange_bf16 / _exchange_bfp8_block        :272-357
//   nntrain_gradient_host_pipeline_{create,create_bfp8_block,
//       exchange_bf16,exchange_bfp8_block,destroy}               :359-709
//   nntrain_gradient_unpack_float                                :711-721
//   nntrain_gradient_comm_synchronize / _event_destroy / _comm_destroy  :723-739
// The transport block of the block-BFP8 bucket path is 128 values (:9).
#include "bfp8_kernels.cuh"
#include "reduce_kernels.cuh"
#include "launchers.cuh"

#include <new>

namespace ngb {
namespace {

constexpr int kTransportBlock = 128;

// Two pinned-host slots and two device slots: chunk k downloads into slot
// k & 1 on the source device's stream while chunk k-1 uploads and is summed on
// the destination's stream.
struct HostPipeline {
    int source_device = -1;
    int destination_device = -1;
    int capacity = 0;
    bool bfp8_block = false;
    void* host[2] = {nullptr, nullptr};
    void* device[2] = {nullptr, nullptr};
    float* host_scales[2] = {nullptr, nullptr};
    float* device_scales[2] = {nullptr, nullptr};
    cudaStream_t download_stream = nullptr;
    cudaStream_t upload_stream = nullptr;
    cudaEvent_t download_done[2] = {nullptr, nullptr};
    cudaEvent_t upload_done[2] = {nullptr, nullptr};
};

struct FirstError {
    cudaError_t value = cudaSuccess;
    void operator()(cudaError_t status) { if (value == cudaSuccess && status != cudaSuccess) value = status; }
};

cudaError_t destroy_pipeline(HostPipeline* p) {
    if (!p) return cudaSuccess;
    FirstError keep;
    if (p->source_device >= 0) {
        keep(static_cast<cudaError_t>(select_device(p->source_device)));
        if (p->download_stream) keep(cudaStreamSynchronize(p->download_stream));
        for (int s = 0; s < 2; ++s) if (p->download_done[s]) keep(cudaEventDestroy(p->download_done[s]));
        if (p->download_stream) keep(cudaStreamDestroy(p->download_stream));
    }
    if (p->destination_device >= 0) {
        keep(static_cast<cudaError_t>(select_device(p->destination_device)));
        if (p->upload_stream) keep(cudaStreamSynchronize(p->upload_stream));
        for (int s = 0; s < 2; ++s) {
            if (p->upload_done[s]) keep(cudaEventDestroy(p->upload_done[s]));
            if (p->device[s]) keep(cudaFree(p->device[s]));
            if (p->device_scales[s]) keep(cudaFree(p->device_scales[s]));
        }
        if (p->upload_stream) keep(cudaStreamDestroy(p->upload_stream));
    }
    for (int s = 0; s < 2; ++s) {
        if (p->host[s]) keep(cudaFreeHost(p->host[s]));
        if (p->host_scales[s]) keep(cudaFreeHost(p->host_scales[s]));
    }
    delete p;
    return keep.value;
}

cudaError_t create_pipeline(int source_device, int destination_device, int chunk_elements, bool bfp8_block,
                            void** out) {
    *out = nullptr;
    HostPipeline* p = new (std::nothrow) HostPipeline();
    if (!p) return cudaErrorMemoryAllocation;
    p->source_device = source_device;
    p->destination_device = destination_device;
    p->capacity = chunk_elements;
    p->bfp8_block = bfp8_block;
    const size_t payload_bytes = static_cast<size_t>(chunk_elements) * (bfp8_block ? 1 : sizeof(unsigned short));
    const size_t scale_bytes = bfp8_block ? static_cast<size_t>(chunk_elements / kTransportBlock) * sizeof(float) : 0;
    cudaError_t status = static_cast<cudaError_t>(select_device(source_device));
    if (status == cudaSuccess) status = cudaStreamCreateWithFlags(&p->download_stream, cudaStreamNonBlocking);
    for (int s = 0; status == cudaSuccess && s < 2; ++s)
        status = cudaEventCreateWithFlags(&p->download_done[s], cudaEventDisableTiming);
    if (status == cudaSuccess) status = static_cast<cudaError_t>(select_device(destination_device));
    if (status == cudaSuccess) status = cudaStreamCreateWithFlags(&p->upload_stream, cudaStreamNonBlocking);
    for (int s = 0; status == cudaSuccess && s < 2; ++s) {
        status = cudaEventCreateWithFlags(&p->upload_done[s], cudaEventDisableTiming);
        if (status == cudaSuccess) status = cudaMalloc(&p->device[s], payload_bytes);
        if (status == cudaSuccess) status = cudaMallocHost(&p->host[s], payload_bytes);
        if (status == cudaSuccess && bfp8_block) status = cudaMalloc(reinterpret_cast<void**>(&p->device_scales[s]), scale_bytes);
        if (status == cudaSuccess && bfp8_block) status = cudaMallocHost(reinterpret_cast<void**>(&p->host_scales[s]), scale_bytes);
    }
    if (status != cudaSuccess) { (void)destroy_pipeline(p); return status; }
    *out = p;
    return cudaSuccess;
}

// Shared chunk loop of both host-pipeline exchanges.  Blocks the calling
// thread, as the reference's does.
template <typename SumChunk>
cudaError_t run_pipeline(HostPipeline* p, const void* remote_source, const float* remote_scales, int length,
                         cudaEvent_t local_ready, cudaEvent_t remote_ready, SumChunk&& sum_chunk) {
    const size_t element_bytes = p->bfp8_block ? 1 : sizeof(unsigned short);
    cudaError_t status = static_cast<cudaError_t>(select_device(p->source_device));
    if (status == cudaSuccess) status = cudaEventSynchronize(remote_ready);
    if (status == cudaSuccess) status = static_cast<cudaError_t>(select_device(p->destination_device));
    if (status == cudaSuccess) status = cudaEventSynchronize(local_ready);
    if (status != cudaSuccess) return status;

    const int chunks = (length + p->capacity - 1) / p->capacity;
    auto download = [&](int chunk) -> cudaError_t {
        const int slot = chunk & 1;
        const int offset = chunk * p->capacity;
        const int count = length - offset < p->capacity ? length - offset : p->capacity;
        cudaError_t s = static_cast<cudaError_t>(select_device(p->source_device));
        if (s == cudaSuccess)
            s = cudaMemcpyAsync(p->host[slot], static_cast<const char*>(remote_source) + offset * element_bytes,
                                count * element_bytes, cudaMemcpyDeviceToHost, p->download_stream);
        if (s == cudaSuccess && p->bfp8_block) {
            const int scale_count = (count + kTransportBlock - 1) / kTransportBlock;
            s = cudaMemcpyAsync(p->host_scales[slot], remote_scales + offset / kTransportBlock,
                                scale_count * sizeof(float), cudaMemcpyDeviceToHost, p->download_stream);
        }
        if (s == cudaSuccess) s = cudaEventRecord(p->download_done[slot], p->download_stream);
        return s;
    };

    status = download(0);
    if (status == cudaSuccess && chunks > 1) status = download(1);
    for (int chunk = 0; status == cudaSuccess && chunk < chunks; ++chunk) {
        const int slot = chunk & 1;
        const int offset = chunk * p->capacity;
        const int count = length - offset < p->capacity ? length - offset : p->capacity;
        status = static_cast<cudaError_t>(select_device(p->source_device));
        if (status == cudaSuccess) status = cudaEventSynchronize(p->download_done[slot]);
        if (status != cudaSuccess) break;
        status = static_cast<cudaError_t>(select_device(p->destination_device));
        if (status == cudaSuccess)
            status = cudaMemcpyAsync(p->device[slot], p->host[slot], count * element_bytes,
                                     cudaMemcpyHostToDevice, p->upload_stream);
        if (status == cudaSuccess && p->bfp8_block) {
            const int scale_count = (count + kTransportBlock - 1) / kTransportBlock;
            status = cudaMemcpyAsync(p->device_scales[slot], p->host_scales[slot], scale_count * sizeof(float),
                                     cudaMemcpyHostToDevice, p->upload_stream);
        }
        if (status == cudaSuccess) status = sum_chunk(slot, offset, count);
        if (status == cudaSuccess) status = cudaEventRecord(p->upload_done[slot], p->upload_stream);
        if (status == cudaSuccess && chunk + 2 < chunks) {
            status = cudaEventSynchronize(p->upload_done[slot]);
            if (status == cudaSuccess) status = download(chunk + 2);
        }
    }
    if (status == cudaSuccess) status = static_cast<cudaError_t>(select_device(p->destination_device));
    if (status == cudaSuccess) status = cudaStreamSynchronize(p->upload_stream);
    return status;
}

cudaError_t sum_bf16_pair(const unsigned short* local, const unsigned short* remote, float* reduced, int length,
                          double* squared_sum, cudaStream_t stream) {
    Bf16Inputs io{};
    io.inputs = 2;
    io.values[0] = local;
    io.values[1] = remote;
    io.outputs = 0;
    return launch_bf16_reduce(io, reduced, 0, length, 1.0f, squared_sum, false, stream);
}

cudaError_t sum_bfp8_pair(const signed char* local, const float* local_scales, const signed char* remote,
                          const float* remote_scales, float* reduced, int length, double* squared_sum,
                          cudaStream_t stream) {
    EncodedInputs in{};
    in.inputs = 2;
    in.payload[0] = local;   in.scales[0] = local_scales;
    in.payload[1] = remote;  in.scales[1] = remote_scales;
    return launch_bfp8_sum_to_f32(in, reduced, length, kTransportBlock, 1.0f, squared_sum, nullptr, nullptr, stream);
}

}  // namespace
}  // namespace ngb

using namespace ngb;

NNTRAIN_EXPORT int nntrain_gradient_comm_create(int device, cudaStream_t* stream) {
    if (!stream) return static_cast<int>(cudaErrorInvalidValue);
    (void)device;
    return static_cast<int>(cudaStreamCreateWithFlags(stream, cudaStreamNonBlocking));
}

NNTRAIN_EXPORT int nntrain_gradient_event_create(int device, cudaEvent_t* event) {
    if (!event) return static_cast<int>(cudaErrorInvalidValue);
    (void)device;
    return static_cast<int>(cudaEventCreateWithFlags(event, cudaEventDisableTiming));
}

// fp32 -> bf16 (round to nearest even) into destination[destination_offset + i].
NNTRAIN_EXPORT int nntrain_gradient_pack_bf16(int device, const float* source, __nv_bfloat16* destination,
                                              int destination_offset, int length, cudaStream_t compute_stream) {
    if (!source || !destination || destination_offset < 0 || length <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    (void)device;
    return static_cast<int>(launch_f32_to_bf16(
        source, reinterpret_cast<unsigned short*>(destination) + destination_offset, length, compute_stream));
}

// Block-128 encode of a bucket; a block holding NaN/Inf gets the scale bit
// pattern 0x7fffffff and an all-zero payload so the NaN reaches the fp32 sum.
NNTRAIN_EXPORT int nntrain_gradient_pack_bfp8_block(int device, const float* source, signed char* destination,
                                                    float* scales, int length, cudaStream_t compute_stream) {
    if (!source || !destination || !scales || length <= 0) return static_cast<int>(cudaErrorInvalidValue);
    (void)device;
    return static_cast<int>(launch_bfp8_encode(source, nullptr, destination, scales, length, kTransportBlock,
                                               kEncNanScale, nullptr, nullptr, false, compute_stream));
}

NNTRAIN_EXPORT int nntrain_gradient_record_ready(int device, cudaEvent_t event, cudaStream_t compute_stream) {
    (void)device;
    return static_cast<int>(cudaEventRecord(event, compute_stream));
}

// For use inside stream capture: the record becomes an external-event node,
// visible to a communication stream outside the graph.
NNTRAIN_EXPORT int nntrain_gradient_record_ready_external(int device, cudaEvent_t event,
                                                          cudaStream_t compute_stream) {
    if (device < 0 || !event) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(cudaEventRecordWithFlags(event, compute_stream, cudaEventRecordExternal));
}

// Pull the peer's bf16 bucket into local staging, reduced = f32(local) +
// f32(remote), optional sum of squares of the fp32 result.
NNTRAIN_EXPORT int nntrain_gradient_exchange_bf16(
    int destination_device, int source_device, const __nv_bfloat16* local, const __nv_bfloat16* remote_source,
    __nv_bfloat16* remote_staging, float* reduced, int length, double* squared_sum,
    cudaStream_t communication_stream, cudaEvent_t local_ready, cudaEvent_t remote_ready) {
    if (!local || !remote_source || !remote_staging || !reduced || length <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t status = cudaStreamWaitEvent(communication_stream, local_ready, 0);
    if (status != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaStreamWaitEvent(communication_stream, remote_ready, 0)) != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(remote_staging, destination_device, remote_source, source_device,
                                      static_cast<size_t>(length) * sizeof(__nv_bfloat16),
                                      communication_stream)) != cudaSuccess)
        return static_cast<int>(status);
    return static_cast<int>(sum_bf16_pair(reinterpret_cast<const unsigned short*>(local),
                                          reinterpret_cast<const unsigned short*>(remote_staging), reduced, length,
                                          squared_sum, communication_stream));
}

// Same for a block-128 BFP8 bucket: payload + scale sidecar are pulled, the
// fp32 result is fl(fl(q0*s0) + fl(q1*s1)) on both replicas, never re-encoded.
NNTRAIN_EXPORT int nntrain_gradient_exchange_bfp8_block(
    int destination_device, int source_device, const signed char* local, const float* local_scales,
    const signed char* remote_source, const float* remote_source_scales, signed char* remote_staging,
    float* remote_staging_scales, float* reduced, int length, double* squared_sum,
    cudaStream_t communication_stream, cudaEvent_t local_ready, cudaEvent_t remote_ready) {
    if (!local || !local_scales || !remote_source || !remote_source_scales || !remote_staging ||
        !remote_staging_scales || !reduced || length <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t status = cudaStreamWaitEvent(communication_stream, local_ready, 0);
    if (status != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaStreamWaitEvent(communication_stream, remote_ready, 0)) != cudaSuccess) return static_cast<int>(status);
    if ((status = cudaMemcpyPeerAsync(remote_staging, destination_device, remote_source, source_device,
                                      static_cast<size_t>(length), communication_stream)) != cudaSuccess)
        return static_cast<int>(status);
    const int scale_count = (length + kTransportBlock - 1) / kTransportBlock;
    if ((status = cudaMemcpyPeerAsync(remote_staging_scales, destination_device, remote_source_scales, source_device,
                                      static_cast<size_t>(scale_count) * sizeof(float),
                                      communication_stream)) != cudaSuccess)
        return static_cast<int>(status);
    return static_cast<int>(sum_bfp8_pair(local, local_scales, remote_staging, remote_staging_scales, reduced,
                                          length, squared_sum, communication_stream));
}

NNTRAIN_EXPORT int nntrain_gradient_host_pipeline_create(int source_device, int destination_device,
                                                         int chunk_elements, void** pipeline_pointer) {
    if (!pipeline_pointer || source_device == destination_device || chunk_elements <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(create_pipeline(source_device, destination_device, chunk_elements, false, pipeline_pointer));
}

NNTRAIN_EXPORT int nntrain_gradient_host_pipeline_create_bfp8_block(int source_device, int destination_device,
                                                                    int chunk_elements, void** pipeline_pointer) {
    if (!pipeline_pointer || source_device == destination_device || chunk_elements <= 0 ||
        chunk_elements % kTransportBlock != 0)
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(create_pipeline(source_device, destination_device, chunk_elements, true, pipeline_pointer));
}

NNTRAIN_EXPORT int nntrain_gradient_host_pipeline_exchange_bf16(
    void* pipeline_pointer, const __nv_bfloat16* local, const __nv_bfloat16* remote_source, float* reduced,
    int length, double* squared_sum, cudaEvent_t local_ready, cudaEvent_t remote_ready) {
    HostPipeline* p = static_cast<HostPipeline*>(pipeline_pointer);
    if (!p || p->bfp8_block || !local || !remote_source || !reduced || length <= 0 || !local_ready || !remote_ready)
        return static_cast<int>(cudaErrorInvalidValue);
    const unsigned short* local_bits = reinterpret_cast<const unsigned short*>(local);
    return static_cast<int>(run_pipeline(p, remote_source, nullptr, length, local_ready, remote_ready,
        [&](int slot, int offset, int count) {
            return sum_bf16_pair(local_bits + offset, static_cast<const unsigned short*>(p->device[slot]),
                                 reduced + offset, count, squared_sum, p->upload_stream);
        }));
}

NNTRAIN_EXPORT int nntrain_gradient_host_pipeline_exchange_bfp8_block(
    void* pipeline_pointer, const signed char* local, const float* local_scales, const signed char* remote_source,
    const float* remote_source_scales, float* reduced, int length, double* squared_sum, cudaEvent_t local_ready,
    cudaEvent_t remote_ready) {
    HostPipeline* p = static_cast<HostPipeline*>(pipeline_pointer);
    if (!p || !p->bfp8_block || !local || !local_scales || !remote_source || !remote_source_scales || !reduced ||
        length <= 0 || !local_ready || !remote_ready)
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(run_pipeline(p, remote_source, remote_source_scales, length, local_ready, remote_ready,
        [&](int slot, int offset, int count) {
            return sum_bfp8_pair(local + offset, local_scales + offset / kTransportBlock,
                                 static_cast<const signed char*>(p->device[slot]), p->device_scales[slot],
                                 reduced + offset, count, squared_sum, p->upload_stream);
        }));
}

NNTRAIN_EXPORT int nntrain_gradient_host_pipeline_destroy(void* pipeline_pointer) {
    return static_cast<int>(destroy_pipeline(static_cast<HostPipeline*>(pipeline_pointer)));
}

// destination[i] = source[source_offset + i]
NNTRAIN_EXPORT int nntrain_gradient_unpack_float(int device, const float* source, int source_offset,
                                                 float* destination, int length,
                                                 cudaStream_t communication_stream) {
    if (!source || !destination || source_offset < 0 || length <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    (void)device;
    return static_cast<int>(launch_f32_copy(source + source_offset, destination, length, communication_stream));
}

NNTRAIN_EXPORT int nntrain_gradient_comm_synchronize(int device, cudaStream_t communication_stream) {
    (void)device;
    return static_cast<int>(cudaStreamSynchronize(communication_stream));
}

NNTRAIN_EXPORT int nntrain_gradient_event_destroy(int device, cudaEvent_t event) {
    (void)device;
    return static_cast<int>(cudaEventDestroy(event));
}

NNTRAIN_EXPORT int nntrain_gradient_comm_destroy(int device, cudaStream_t communication_stream) {
    (void)device;
    return static_cast<int>(cudaStreamDestroy(communication_stream));
}
