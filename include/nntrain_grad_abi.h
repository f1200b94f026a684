/*
 * C ABI of libnntrain_grad_b200.so: the compressed data-parallel gradient
 * path (BFP8 block codec, BFP8 / BF16 gradient reducers, fused clip-norm) as
 * hand-written sm_100a CUDA kernels.
 *
 * Conventions (those of the reference's native layer, NNtrain.Cuda/native):
 *   - every entry point returns an int cudaError_t (0 = success; bad
 *     arguments = cudaErrorInvalidValue = 1);
 *   - kernel launches are asynchronous; the return value is the launch status;
 *   - pointers are raw device addresses unless stated otherwise; streams and
 *     events are the CUDA runtime's handles passed as opaque pointers;
 *   - the caller owns every buffer; the library owns only what one of its
 *     create calls returned and frees it only in the paired destroy call;
 *   - NaN / Inf in the data is not a status: it raises a device-side flag the
 *     caller reads once per step.
 *
 * Each declaration cites the reference interface it replaces (path within the
 * reference project : lines).  Entry points marked "ABI minor 36" have no
 * counterpart in the reference, whose compressed reducers take exactly two
 * devices of one process; they carry the same path to N ranks.
 */
#ifndef NNTRAIN_GRAD_ABI_H
#define NNTRAIN_GRAD_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* nntrain_stream_t;   /* cudaStream_t */
typedef void* nntrain_event_t;    /* cudaEvent_t  */

/* NNtrain.Cuda/native/cuda_runtime_bridge.cu:74-82 */
typedef struct nntrain_native_error_info {
    uint32_t struct_size;
    uint32_t abi_version;
    uint64_t sequence;
    int32_t status;
    int32_t device;
    uint32_t operation;
    uint32_t reserved;
} nntrain_native_error_info;

/* ---- process-level ------------------------------------------------------ */

/* (major << 16) | minor; major 1, minor 36.
 * cuda_runtime_bridge.cu:18-21,1436-1438 */
uint32_t nntrain_abi_version(void);
/* cuda_runtime_bridge.cu:1440-1450 */
int nntrain_last_error(nntrain_native_error_info* destination, size_t destination_size);
/* cuda_runtime_bridge.cu:1452-1481 */
int nntrain_error_snapshot(int status, int device, uint32_t operation,
                           nntrain_native_error_info* destination, size_t destination_size);
/* Bits 1 (bfloat16), 6 (asynchronous gradient reduction), 7 (CUDA graphs),
 * 8 (BFP8 quantization) on compute capability >= 10.
 * cuda_runtime_bridge.cu:1483-1536 */
int nntrain_capability_bitmap(int device, unsigned long long* bitmap,
                              int* compute_capability_major, int* compute_capability_minor);
/* Thread-local device selection cache.  cuda_runtime_bridge.cu:122-131,2336-2339 */
int nntrain_cuda_set_device(int device);
/* Thread-local stream used by the entry points that take none.
 * NNtrain.Cuda/native/tensor_kernels.cu:26,2888-2891 */
int nntrain_cuda_use_external_stream(void* stream);

/* ABI minor 36; no counterpart in the reference (its kernels use fixed
 * grids).  Process-wide defaults of the launch shapes.
 * codec_iterations_per_cta: n > 0 = short-lived CTAs of n iterations each for
 * the encode / decode kernels (default 2, also the fastest for a kernel
 * running alone), 0 = persistent grids.  collective_ctas: what a group created
 * afterwards starts with (see nntrain_gradient_group_configure); default 0. */
int nntrain_gradient_configure(int codec_iterations_per_cta, int collective_ctas);
/* ABI minor 36; no counterpart in the reference.  How the owner / all-reduce
 * kernels fetch their inputs when no group says otherwise: 1 (default) =
 * cp.async rings in shared memory, 0 = register prefetch, 2 = cp.async rings
 * in CTAs that take a whole SM each, 3 = bulk asynchronous copies of whole
 * tiles in CTAs that own their SM, 4 = the same in small CTAs that share it.
 * Same results either way. */
int nntrain_gradient_configure_collective(int asynchronous_copies);
/* ABI minor 36; no counterpart in the reference.  Most CTAs a persistent
 * encode / decode grid may use (only with codec_iterations_per_cta == 0);
 * 0 = no cap. */
int nntrain_gradient_configure_codec_cap(int ctas);

/* ---- BFP8 block codec ---------------------------------------------------
 * payload: signed int8 per value; scales: one fp32 per block,
 * scale = max|x| == 0 ? 1 : max|x| / 127; code = clamp(rne(x / scale), +-127).
 * quantization_block_size >= length selects one tensor-wide scale. */

/* cuda_runtime_bridge.cu:1540-1622 */
int nntrain_cuda_bfp8_quantize_f32(int device, const float* source, signed char* payload,
                                   float* scales, int length, int quantization_block_size,
                                   void* stream);
/* cuda_runtime_bridge.cu:1720-1768 */
int nntrain_cuda_bfp8_dequantize_f32(int device, const signed char* payload, const float* scales,
                                     float* destination, int length, int quantization_block_size,
                                     void* stream);
/* Encode and overwrite the source with its decode; rejects the tensor-wide
 * case.  cuda_runtime_bridge.cu:1770-1826 */
int nntrain_cuda_bfp8_quantize_f32_roundtrip(int device, float* source, signed char* payload,
                                             float* scales, int length, int quantization_block_size,
                                             void* stream);
/* The codec with a bf16 tensor as the source: the fp32 rules on the widened
 * value.  cuda_runtime_bridge.cu:868-935,2024-2118 */
int nntrain_cuda_bfp8_quantize_bf16(int device, const unsigned short* source, signed char* payload,
                                    float* scales, int length, int quantization_block_size,
                                    void* stream);
/* destination = bf16_rn(code * scale).  cuda_runtime_bridge.cu:769-806,1964-2022 */
int nntrain_cuda_bfp8_dequantize_bf16(int device, const signed char* payload, const float* scales,
                                      unsigned short* destination, int length,
                                      int quantization_block_size, void* stream);
/* ABI minor 36.  64-bit length; block_size 0 = tensor-wide.  Optional
 * outputs, each enabled by a non-null pointer: roundtrip (decode, may alias
 * source), squared_sum (+= sum of squares of the decoded values, binary64),
 * finite_status (= 1 when any input is NaN/Inf). */
int nntrain_bfp8_block_encode(int device, const float* source, signed char* payload, float* scales,
                              long long length, int block_size, float* roundtrip,
                              double* squared_sum, int* finite_status, void* stream);
/* ABI minor 36. */
int nntrain_bfp8_block_decode(int device, const signed char* payload, const float* scales,
                              float* destination, long long length, int block_size, void* stream);

/* ---- tensor-wide BFP8 gradient publication and 2-device reducer ----------- */

/* Finite check, tensor-wide scale, payload, fp32 gradient overwritten with
 * its decode.  NaN/Inf: *finite_status = 1, scale = 1, nothing else written.
 * tensor_kernels.cu:988-1042,1114-1146,3876-3889 */
int nntrain_bfp8_gradient_quantize(int device, float* source, signed char* payload, float* scale,
                                   int length, int* finite_status, nntrain_stream_t stream);
/* Same plus *squared_sum += sum of squares of the decoded values.
 * tensor_kernels.cu:1044-1073,3891-3905 */
int nntrain_bfp8_gradient_quantize_accumulate(int device, float* source, signed char* payload,
                                              float* scale, int length, int* finite_status,
                                              double* squared_sum, nntrain_stream_t stream);
/* tensor_kernels.cu:1044-1073,3907-3921 */
int nntrain_bfp8_gradient_squared_sum(int device, const signed char* payload, const float* scale,
                                      int length, double* squared_sum, int* finite_status,
                                      nntrain_stream_t stream);
/* Scale-only clip: scale = fmaxf(scale * multiplier, FLT_MIN).
 * tensor_kernels.cu:1075-1082,3923-3933 */
int nntrain_bfp8_gradient_scale(int device, float* scale, float multiplier, nntrain_stream_t stream);
/* tensor_kernels.cu:3935-4002 */
int nntrain_bfp8_gradient_reduce(
    int primary_device, int secondary_device, const signed char* local_payload,
    const float* local_scale, const signed char* remote_payload, const float* remote_scale,
    signed char* remote_payload_staging, float* remote_scale_staging, float* reduced,
    signed char* output_payload, float* output_scale, int length, float reduction_scale,
    int* finite_status, const int* remote_finite_status, int* remote_status_staging,
    double* squared_sum, nntrain_stream_t communication_stream, nntrain_event_t local_ready,
    nntrain_event_t remote_ready, nntrain_event_t reduced_ready);
/* tensor_kernels.cu:4004-4038 */
int nntrain_bfp8_gradient_broadcast(
    int destination_device, int source_device, const signed char* source_payload,
    const float* source_scale, signed char* destination_payload, float* destination_scale,
    float* destination_float, int length, int* destination_finite_status,
    nntrain_stream_t destination_stream, nntrain_event_t source_ready);

/* ABI minor 36: the three calls above for EVERY tensor of a bucket at once.
 * The reference publishes, reduces and broadcasts one tensor per call
 * (tensor_kernels.cu:1114-1146: a memset and five or six launches per tensor;
 * :3935-4038: about thirteen; NNtrain.Core/Tensors/
 * CudaBfp8GradientPublicationScope.cs:12-521 walks the leaves the same way).
 * The tensors of a bucket lie in one contiguous arena at running-sum offsets
 * (NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1572-1601);
 * tensor_offsets is a DEVICE array of tensors + 1 strictly ascending element
 * offsets (first 0, last total_elements); payload has the arena's layout,
 * scales one entry per tensor; maxima_scratch is tensors words owned by the
 * caller.  Each call is three stream operations per bucket.  A NaN / Inf
 * anywhere in the bucket raises *finite_status and publishes nothing (every
 * scale of the bucket = 1). */
int nntrain_bfp8_gradient_publish_tensors(
    int device, float* arena, signed char* payload, float* scales, const long long* tensor_offsets,
    int tensors, long long total_elements, unsigned* maxima_scratch, int* finite_status,
    double* squared_sum, nntrain_stream_t stream);
/* reduced = reduction_scale * (rank-ordered fp32 sum of code * scale) over N
 * encoded inputs (host tables of device pointers; per-tensor scale arrays),
 * then published as above into out_payload / out_scales; `reduced` ends as the
 * decode of the result. */
int nntrain_bfp8_gradient_reduce_tensors(
    int device, int inputs, const signed char* const* payloads, const float* const* scales,
    float* reduced, signed char* out_payload, float* out_scales, const long long* tensor_offsets,
    int tensors, long long total_elements, float reduction_scale, unsigned* maxima_scratch,
    int* finite_status, double* squared_sum, nntrain_stream_t stream);
/* destination = payload * scales[tensor] for a whole bucket; skipped when
 * *skip_flag (optional) is non-zero (tensor_kernels.cu:4034-4036). */
int nntrain_bfp8_gradient_decode_tensors(
    int device, const signed char* payload, const float* scales, float* destination,
    const long long* tensor_offsets, int tensors, long long total_elements, const int* skip_flag,
    nntrain_stream_t stream);

/* ---- bucketed BF16 / block-128 BFP8 transport (two devices, one process) --- */

/* NNtrain.Cuda/native/gradient_collectives.cu:213-219 */
int nntrain_gradient_comm_create(int device, nntrain_stream_t* stream);
/* gradient_collectives.cu:221-227 */
int nntrain_gradient_event_create(int device, nntrain_event_t* event);
/* gradient_collectives.cu:11-22,229-239 */
int nntrain_gradient_pack_bf16(int device, const float* source, void* destination_bf16,
                               int destination_offset, int length, nntrain_stream_t compute_stream);
/* gradient_collectives.cu:24-60,241-252 */
int nntrain_gradient_pack_bfp8_block(int device, const float* source, signed char* destination,
                                     float* scales, int length, nntrain_stream_t compute_stream);
/* gradient_collectives.cu:254-258 */
int nntrain_gradient_record_ready(int device, nntrain_event_t event, nntrain_stream_t compute_stream);
/* gradient_collectives.cu:260-270 */
int nntrain_gradient_record_ready_external(int device, nntrain_event_t event,
                                           nntrain_stream_t compute_stream);
/* gradient_collectives.cu:62-90,272-309 */
int nntrain_gradient_exchange_bf16(int destination_device, int source_device, const void* local_bf16,
                                   const void* remote_source_bf16, void* remote_staging_bf16,
                                   float* reduced, int length, double* squared_sum,
                                   nntrain_stream_t communication_stream, nntrain_event_t local_ready,
                                   nntrain_event_t remote_ready);
/* gradient_collectives.cu:92-129,311-357 */
int nntrain_gradient_exchange_bfp8_block(
    int destination_device, int source_device, const signed char* local, const float* local_scales,
    const signed char* remote_source, const float* remote_source_scales, signed char* remote_staging,
    float* remote_staging_scales, float* reduced, int length, double* squared_sum,
    nntrain_stream_t communication_stream, nntrain_event_t local_ready, nntrain_event_t remote_ready);
/* gradient_collectives.cu:359-414 */
int nntrain_gradient_host_pipeline_create(int source_device, int destination_device,
                                          int chunk_elements, void** pipeline_pointer);
/* gradient_collectives.cu:416-474 */
int nntrain_gradient_host_pipeline_create_bfp8_block(int source_device, int destination_device,
                                                     int chunk_elements, void** pipeline_pointer);
/* gradient_collectives.cu:476-578 */
int nntrain_gradient_host_pipeline_exchange_bf16(void* pipeline_pointer, const void* local_bf16,
                                                 const void* remote_source_bf16, float* reduced,
                                                 int length, double* squared_sum,
                                                 nntrain_event_t local_ready,
                                                 nntrain_event_t remote_ready);
/* gradient_collectives.cu:580-703 */
int nntrain_gradient_host_pipeline_exchange_bfp8_block(
    void* pipeline_pointer, const signed char* local, const float* local_scales,
    const signed char* remote_source, const float* remote_source_scales, float* reduced, int length,
    double* squared_sum, nntrain_event_t local_ready, nntrain_event_t remote_ready);
/* gradient_collectives.cu:705-709 */
int nntrain_gradient_host_pipeline_destroy(void* pipeline_pointer);
/* gradient_collectives.cu:131-141,711-721 */
int nntrain_gradient_unpack_float(int device, const float* source, int source_offset,
                                  float* destination, int length,
                                  nntrain_stream_t communication_stream);
/* gradient_collectives.cu:723-727 */
int nntrain_gradient_comm_synchronize(int device, nntrain_stream_t communication_stream);
/* gradient_collectives.cu:729-733 */
int nntrain_gradient_event_destroy(int device, nntrain_event_t event);
/* gradient_collectives.cu:735-739 */
int nntrain_gradient_comm_destroy(int device, nntrain_stream_t communication_stream);

/* ---- norm / clip ---------------------------------------------------------- */

/* These four run on the thread's implicit stream.
 * tensor_kernels.cu:968-986,3229-3231 */
int nntrain_tensor_squared_sum(const float* values, int length, double* result);
/* tensor_kernels.cu:910-914,3177-3180 */
int nntrain_tensor_scale(float* values, int length, float scale);
/* tensor_kernels.cu:931-936,3208-3211 */
int nntrain_tensor_encode_bf16(const float* source, unsigned short* destination, int length);
/* tensor_kernels.cu:2876-2881,3870-3874 */
int nntrain_tensor_decode_bf16(const unsigned short* source, float* destination, int length);
/* NNtrain.Cuda/native/pure_bfloat16_gradients.cu:315-335,546-557 */
int nntrain_tensor_bf16_gradient_squared_sum(const unsigned short* values, int length, double* result,
                                             nntrain_stream_t stream);
/* pure_bfloat16_gradients.cu:337-348,559-570 */
int nntrain_tensor_bf16_gradient_scale(unsigned short* values, int length, float multiplier,
                                       nntrain_stream_t stream);
/* ABI minor 36.  kind 0 = fp32, 1 = bf16, 2 = BFP8 payload (+scales, block
 * size; 0 = tensor-wide).  *squared_sum += sum of squares in binary64. */
int nntrain_gradient_squared_sum(int device, int kind, const void* values, const float* scales,
                                 long long length, int block_size, double* squared_sum,
                                 int* finite_status, nntrain_stream_t stream);
/* ABI minor 36.  Device-side clip coefficient (NNtrain.Core/Torch/nn.cs:69-72):
 * out[0] = norm = (float)sqrt(*squared_sum); out[1] = norm > max_norm ?
 * max_norm / (norm + 1e-6f) : 1. */
int nntrain_gradient_clip_coefficient(int device, const double* squared_sum, float max_norm,
                                      float* norm_and_coefficient, nntrain_stream_t stream);
/* ABI minor 36.  Whole-arena clip.  kind 0: fp32 *= c (nn.cs:72-78); kind 1:
 * bf16 = rn(f32 * c) (pure_bfloat16_gradients.cu:337-348); kind 2: values is
 * the fp32 scale sidecar, scale = fmaxf(scale * c, FLT_MIN), payload untouched
 * (tensor_kernels.cu:1075-1082).  With a non-null `coefficient` the multiplier
 * is coefficient[1] read on the device (the output of
 * nntrain_gradient_clip_coefficient) and a value of exactly 1 touches nothing. */
int nntrain_gradient_clip_apply(int device, int kind, void* values, long long count, float multiplier,
                                const float* coefficient, nntrain_stream_t stream);

/* ABI minor 36.  AdamW that reads the reduced BFP8 gradient directly: the
 * arithmetic of the reference's adamw_kernel (NNtrain.Cuda/native/
 * tensor_kernels.cu:1148-1174, export :3233-3241) with g = code * scale formed
 * in registers, so the step needs no fp32 decode pass (the reference's
 * BFP8-native optimizers do the same, tensor_kernels.cu:3282-3365).  Every
 * operation is a separate IEEE binary32 operation.  block_size 0 = one scale
 * for all; compute_bf16 (optional) receives the bf16 working copy. */
int nntrain_optimizer_adamw_bfp8_gradient(
    int device, float* data, const signed char* gradient_payload, const float* gradient_scales,
    int block_size, float* first_moment, float* second_moment, unsigned short* compute_bf16,
    long long length, float beta1, float beta2, float learning_rate, float weight_decay,
    float update_scale, float scaled_epsilon, int apply_weight_decay, nntrain_stream_t stream);

/* ---- N-rank all-reduce, one process per GPU (ABI minor 36) -------------------
 * The reference's compressed reducers accept exactly two devices of one
 * process (NNtrain.Core/Training/CudaBfp8GradientAllReduce.cs:44-49,
 * CudaBFloat16GradientAllReduce.cs:119-124); these carry the same arithmetic,
 * summed left to right over ranks 0..N-1, to N ranks.  Status values of
 * 10000 + n are NCCL results (10099: NCCL could not be loaded). */

/* Peer-visible device memory (CUDA IPC): cudaMalloc + the 64-byte handle
 * other processes map. */
int nntrain_gradient_peer_alloc(int device, long long bytes, void** pointer, void* handle64);
/* Frees memory from nntrain_gradient_peer_alloc. */
int nntrain_gradient_peer_free(int device, void* pointer);
/* Maps a peer's handle into this process (peer access enabled lazily). */
int nntrain_gradient_peer_open(int device, const void* handle64, void** pointer);
/* Unmaps a pointer from nntrain_gradient_peer_open. */
int nntrain_gradient_peer_close(int device, void* pointer);
/* 128-byte NCCL unique id (rank 0 creates, host distributes). */
int nntrain_gradient_group_unique_id(void* id128);
/* Collective.  world == 1 needs neither an id nor NCCL. */
int nntrain_gradient_group_create(const void* id128, int world, int rank, int device, void** group);
/* Destroys the communicator and the group's device scratch. */
int nntrain_gradient_group_destroy(void* group);
/* Launch shape of ONE group's all-reduce kernels (either kind of group), so
 * that two reducers in a process do not retune each other.  collective_ctas:
 * 0 = fill the machine, n > 0 = at most n CTAs.  asynchronous_copies: 0 =
 * register prefetch, 1 = cp.async rings, 2 = bulk asynchronous copies of whole
 * tiles.  exclusive_sms (needs asynchronous_copies): every
 * CTA asks for a whole SM's shared memory, so
 * collective_ctas SMs belong to the all-reduce while it runs and the encode /
 * decode kernels of neighbouring chunks never share an SM with it. */
int nntrain_gradient_group_configure(void* group, int collective_ctas, int asynchronous_copies,
                                     int exclusive_sms);
/* Host-side liveness: 0 or the communicator's asynchronous error; never blocks. */
int nntrain_gradient_group_poll(void* group);
/* Abandon the communicator without waiting (a peer was declared lost). */
int nntrain_gradient_group_abort(void* group);
/* In-place sum of `count` doubles over the ranks; count 0 = barrier. */
int nntrain_gradient_group_sum(void* group, double* values, int count, nntrain_stream_t stream);
/* Shard `rank` of an arena of `length` values: contiguous, 512-value aligned. */
int nntrain_gradient_shard_range(long long length, int world, int rank, long long* first, long long* end);
/* Owner arithmetic on host tables of device pointers (local or peer):
 * r = reduction_scale * (rank-ordered fp32 sum of decoded inputs) over
 * [first_value, end_value), re-encoded (block 32/64/128), stored to every
 * output; optional sum of squares of the decoded result and finite flag.
 * Extends NNtrain.Cuda/native/tensor_kernels.cu:1084-1106 + 1114-1146. */
int nntrain_gradient_reduce_shards_bfp8(
    int device, int inputs, const signed char* const* payloads, const float* const* scales, int outputs,
    signed char* const* out_payloads, float* const* out_scales, long long first_value,
    long long end_value, int block_size, float reduction_scale, double* squared_sum,
    int* finite_status, nntrain_stream_t stream);
/* No counterpart in the reference.  nntrain_gradient_reduce_shards_bfp8 for
 * hosts that must not allocate device memory where they reduce (inside a
 * pool that forbids foreign allocations, while a step is recorded for replay,
 * in a loop that must stay off the allocator): same arguments and results,
 * but the per-span sums of squares and the flag word live in a fixed 128 KiB
 * array inside the library image, and no allocating routine is called.  The
 * sum of squares is added in a fixed order (reproducible).  At most 2^30
 * values per call: longer ranges return cudaErrorInvalidValue (error ring
 * operation 200).  The first call on a device looks up the array's device
 * address; make it before any stream capture starts there.  All calls on a
 * GPU share the array: calls whose kernels overlap on that GPU race. */
int nntrain_gradient_reduce_shards_bfp8_no_alloc(
    int device, int inputs, const signed char* const* payloads, const float* const* scales, int outputs,
    signed char* const* out_payloads, float* const* out_scales, long long first_value,
    long long end_value, int block_size, float reduction_scale, double* squared_sum,
    int* finite_status, nntrain_stream_t stream);
/* bf16 twin (extends NNtrain.Cuda/native/gradient_collectives.cu:62-90). */
int nntrain_gradient_reduce_shards_bf16(
    int device, int inputs, const unsigned short* const* values, int outputs,
    unsigned short* const* out_values, float* reduced, long long first_value, long long end_value,
    float reduction_scale, double* squared_sum, int square_of_bf16, nntrain_stream_t stream);
/* In-place BFP8 all-reduce of an encoded arena (or one chunk of it).
 * mode 0: peer memory, one fused reduce-scatter + accumulate + re-encode +
 * all-gather kernel; mode 1: NCCL send/recv through staging (world shards);
 * mode 2: copy engines pull the peers' shards into the same staging and push
 * the reduced shard back, the owner kernel runs on local memory.
 * phase: bit 0 = first chunk of a step, bit 1 = last chunk (fence, sum of
 * squares and finite flag summed over ranks and published); 3 = whole arena.
 * previous_final (optional event): recorded behind the call's leading barrier,
 * the point at which every earlier chunk of the step is complete here. */
int nntrain_gradient_allreduce_bfp8(
    void* group, signed char* const* payload_by_rank, float* const* scales_by_rank, long long length,
    int block_size, float reduction_scale, double* squared_sum, int* finite_status, int mode,
    int phase, signed char* staging_payload, float* staging_scales, nntrain_event_t previous_final,
    nntrain_stream_t stream);
/* Parameter publication after an optimizer step that is sharded over the
 * ranks (the reference re-publishes every BFP8 data replica after a step with
 * every device updating everything, NNtrain.Core/Tensors/
 * Tensor.Device.Bfp8.cs:593-649): this rank encodes its shard of `source` (its
 * fp32 master arena) into EVERY rank's encoded arena; afterwards all ranks
 * hold encode(assembled parameters), bit-identical.  Collective. */
int nntrain_gradient_publish_shards_bfp8(
    void* group, const float* source, signed char* const* payload_by_rank, float* const* scales_by_rank,
    long long length, int block_size, int* finite_status, nntrain_stream_t stream);
/* Makes `stream` wait for `event` (cudaStreamWaitEvent on opaque handles; the
 * reference does this inside its exchange entry points,
 * NNtrain.Cuda/native/gradient_collectives.cu:284-291). */
int nntrain_gradient_stream_wait_event(nntrain_stream_t stream, nntrain_event_t event);
/* In-place bf16 arena all-reduce (fp32 accumulate, bf16 result); mode and
 * phase as above. */
int nntrain_gradient_allreduce_bf16(
    void* group, unsigned short* const* values_by_rank, long long length, float reduction_scale,
    double* squared_sum, int mode, int phase, unsigned short* staging, nntrain_stream_t stream);

/* ---- N-rank all-reduce, ONE process driving all devices (ABI minor 36) ------
 * The host model of the reference's engine: one worker thread per device
 * (NNtrain.Core/Training/CudaReplicaExecutor.cs:29-116,339-369), the worker
 * that arrives last enqueues the cross-device work
 * (NNtrain.Core/Training/CudaBfp8GradientAllReduce.cs:352-363).  Buffers are
 * plain device allocations; peer access is enabled at creation; ranks are
 * ordered by events only, so one thread can enqueue the whole step. */

/* devices[r] is rank r's device; a device may repeat (those ranks share it). */
int nntrain_gradient_local_group_create(int ranks, const int* devices, void** group);
/* Waits for the devices to go idle, then frees the group's scratch and events. */
int nntrain_gradient_local_group_destroy(void* group);
/* In-place BFP8 all-reduce of one encoded arena (or chunk) on every rank;
 * streams[r] is rank r's communication stream.  All tables are host arrays
 * with one entry per rank; squared_sum_by_rank / finite_status_by_rank may be
 * null.  phase as in nntrain_gradient_allreduce_bfp8.  Replaces the pull /
 * reduce / push of NNtrain.Cuda/native/tensor_kernels.cu:3935-4038 and
 * NNtrain.Cuda/native/gradient_collectives.cu:311-357 for N devices. */
int nntrain_gradient_local_allreduce_bfp8(
    void* group, signed char* const* payload_by_rank, float* const* scales_by_rank, long long length,
    int block_size, float reduction_scale, double* const* squared_sum_by_rank,
    int* const* finite_status_by_rank, int phase, const nntrain_stream_t* streams);
/* bf16 twin (gradient_collectives.cu:272-309 for N devices). */
int nntrain_gradient_local_allreduce_bf16(
    void* group, unsigned short* const* values_by_rank, long long length, float reduction_scale,
    double* const* squared_sum_by_rank, int phase, const nntrain_stream_t* streams);

/* The in-process form of nntrain_gradient_publish_shards_bfp8:
 * source_by_rank[r] is rank r's fp32 master arena. */
int nntrain_gradient_local_publish_shards_bfp8(
    void* group, const float* const* source_by_rank, signed char* const* payload_by_rank,
    float* const* scales_by_rank, long long length, int block_size, int* const* finite_status_by_rank,
    const nntrain_stream_t* streams);

#ifdef __cplusplus
}
#endif
#endif /* NNTRAIN_GRAD_ABI_H */
