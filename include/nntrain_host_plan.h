/*
 * Host-side bookkeeping of the gradient reducers as C-ABI objects (part of
 * libnntrain_grad_b200.so; no device work).  The reference keeps this logic in
 * managed code; it is restated here so an N-rank managed reducer, or any other
 * host, asks one implementation whether a transition is legal.
 *
 * Status: 0 = ok; 1 = bad argument (the managed ArgumentException family);
 * 3000 = invalid operation (the managed InvalidOperationException), with the
 * message available per thread through nntrain_host_last_message.
 */
#ifndef NNTRAIN_HOST_PLAN_H
#define NNTRAIN_HOST_PLAN_H

#ifdef __cplusplus
extern "C" {
#endif

/* This thread's last failure message, NUL-terminated. */
int nntrain_host_last_message(char* buffer, int capacity);

/* Bucket layout; tensors are never split.
 * NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1647-1678 */
int nntrain_plan_build_buckets(const long long* numels, int count, long long target_elements,
                               int* bucket_of, long long* offset_of, int* bucket_count);

/* ---- exactly-once publication state machine ------------------------------
 * NNtrain.Core/Training/CudaCapturedGradientPublicationState.cs:9-337; one
 * entry point per method, same order of checks and same messages. */

/* constructor, CudaCapturedGradientPublicationState.cs:26-32 */
int nntrain_publication_state_create(int device_count, void** state);
/* no managed counterpart (garbage collected there) */
int nntrain_publication_state_destroy(void* state);
/* CudaCapturedGradientPublicationState.cs:34-48 */
int nntrain_publication_begin_step(void* state, long long step);
/* CudaCapturedGradientPublicationState.cs:50-67 */
int nntrain_publication_mark_device_begun(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:69-79 */
int nntrain_publication_enter_notification_path(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:81-101 */
int nntrain_publication_begin_capture_recording(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:103-108 */
int nntrain_publication_is_capture_recording(void* state, long long step, int slot, int* recording);
/* CudaCapturedGradientPublicationState.cs:110-123 */
int nntrain_publication_enter_capture_notification_path(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:125-142 */
int nntrain_publication_end_capture_recording(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:144-173 */
int nntrain_publication_validate_capture_discard(void* state, long long step);
/* CudaCapturedGradientPublicationState.cs:175-206 */
int nntrain_publication_begin_captured_publication(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:208-224 */
int nntrain_publication_complete_captured_publication(void* state, long long step, int slot, int device);
/* CudaCapturedGradientPublicationState.cs:226-237 */
int nntrain_publication_fail_captured_publication(void* state, long long step, int slot);
/* CudaCapturedGradientPublicationState.cs:239-267 */
int nntrain_publication_validate_complete(void* state, long long step);
/* CudaCapturedGradientPublicationState.cs:269-278 */
int nntrain_publication_end_step(void* state, long long step);

/* ---- per-rank step plan ---------------------------------------------------
 * One rank's view of an N-rank reducer: buckets, exactly-once notifications,
 * the fixed bucket order collectives are enqueued in on every rank, reduction
 * stamps and the optimizer guard.  Lifecycle as
 * NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:330-615,912-1089 and
 * CudaBfp8GradientAllReduce.cs:225-364,535-646; `devices` lists the job's
 * device ids in rank order. */

/* constructor; buckets per CudaBFloat16GradientAllReduce.cs:1647-1678, a new
 * reducer generation per CudaGradientCoherence.cs:31-43 */
int nntrain_plan_create(const long long* numels, int count, long long target_bucket_elements,
                        const int* devices, int world, int block_size, void** plan);
/* Dispose, CudaBFloat16GradientAllReduce.cs:1680-1729 */
int nntrain_plan_destroy(void* plan);
/* BucketCount, CudaBFloat16GradientAllReduce.cs:269 */
int nntrain_plan_bucket_count(void* plan, int* count);
/* BucketElementCounts, CudaBFloat16GradientAllReduce.cs:271-272 */
int nntrain_plan_bucket_elements(void* plan, int bucket, long long* elements);
/* segment location, CudaBFloat16GradientAllReduce.cs:1572-1601 */
int nntrain_plan_locate(void* plan, int tensor, int* bucket, long long* offset);
/* TransportBytesPerStep, CudaBFloat16GradientAllReduce.cs:292-297, for N ranks */
int nntrain_plan_transport_bytes_per_step(void* plan, long long* bytes);
/* BeginStep, CudaBFloat16GradientAllReduce.cs:330-399 */
int nntrain_plan_begin_step(void* plan, long long* step_id);
/* BeginDeviceStep, CudaBFloat16GradientAllReduce.cs:401-447 */
int nntrain_plan_begin_device_step(void* plan, long long step);
/* NotifyGradientReady, CudaBFloat16GradientAllReduce.cs:449-537; *bucket_ready
 * = the bucket this notification completed, or -1 */
int nntrain_plan_notify_gradient_ready(void* plan, long long step, int tensor, int* bucket_ready);
/* Next bucket to enqueue in the fixed cross-rank order (descending index), or
 * -1; the captured bucket order plays this role in the reference,
 * CudaBFloat16GradientAllReduce.cs:739-910 */
int nntrain_plan_next_enqueueable(void* plan, long long step, int* bucket);
/* Complete, CudaBFloat16GradientAllReduce.cs:912-1029 */
int nntrain_plan_complete(void* plan, long long step, int non_finite);
/* Abort, CudaBFloat16GradientAllReduce.cs:1031-1089 */
int nntrain_plan_abort(void* plan, long long step);
/* CompletedSteps, CudaBFloat16GradientAllReduce.cs:302 */
int nntrain_plan_completed_steps(void* plan, long long* steps);
/* CudaGradientCoherenceSnapshot, CudaGradientCoherence.cs:45-53: kind,
 * stamp generation, stamp step, pending step, version, consumed version */
int nntrain_plan_coherence_snapshot(void* plan, int tensor, long long* out6);
/* CudaGradientOptimizerGuard.ValidateAndConsume, CudaGradientCoherence.cs:61-173 */
int nntrain_plan_optimizer_validate_and_consume(void* plan, const int* devices, int device_count);

/* PublishGradientSquaredSum, NNtrain.Core/Tensors/Tensor.CudaKernels.cs:768-798 */
int nntrain_plan_publish_squared_sum(void* plan, const int* devices, int device_count, double squared_sum);
/* TryConsumeGradientSquaredSum, Tensor.CudaKernels.cs:800-829,831-848 */
int nntrain_plan_try_consume_squared_sum(void* plan, const int* devices, int device_count,
                                         double* squared_sum, int* hit);
/* clip decision of clip_grad_norm_, NNtrain.Core/Torch/nn.cs:41-47,69-72 */
int nntrain_gradient_clip_decision(double squared_sum, float max_norm, float* norm, float* coefficient);

#ifdef __cplusplus
}
#endif
#endif /* NNTRAIN_HOST_PLAN_H */
