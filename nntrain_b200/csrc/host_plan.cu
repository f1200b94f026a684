// Host-side bookkeeping of the gradient reducers, as C-ABI objects: bucket
// layout, the exactly-once publication state machine, reduction stamps with
// the optimizer guard, and the per-rank step plan.  No device work happens
// here; a managed reducer (or the Python mirror) drives the kernels and asks
// these objects whether each transition is legal.
//
// Restates, in C++, the behaviour of
//   BuildBuckets                         NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1647-1678
//   CudaCapturedGradientPublicationState NNtrain.Core/Training/CudaCapturedGradientPublicationState.cs:9-337
//   CudaGradientReductionStamp / -Source / CudaGradientOptimizerGuard
//                                        NNtrain.Core/Training/CudaGradientCoherence.cs:19-173
//   step lifecycle of the reducer plans  CudaBFloat16GradientAllReduce.cs:330-615,912-1089
//                                        CudaBfp8GradientAllReduce.cs:225-364,535-646
// Status: 0 = ok, 1 = bad argument (the managed code's ArgumentException
// family), 3000 = the managed code's InvalidOperationException; the message is
// kept per thread and read with nntrain_host_last_message.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

namespace ngb {
namespace {

constexpr int kOk = 0;
constexpr int kBadArgument = 1;
constexpr int kInvalidOperation = 3000;

thread_local std::string t_message;

int fail(int status, const char* format, ...) {
    char buffer[512];
    va_list arguments;
    va_start(arguments, format);
    std::vsnprintf(buffer, sizeof(buffer), format, arguments);
    va_end(arguments);
    t_message = buffer;
    return status;
}

// ---- exactly-once publication state ---------------------------------------------
struct PublicationState {
    enum Path : int { kPathNone = 0, kPathNotifications = 1, kPathCaptured = 2, kPathCaptureRecording = 3 };
    enum Device : int { kDeviceNone = 0, kDevicePublishing = 1, kDevicePublished = 2, kDeviceFailed = 3 };

    explicit PublicationState(int devices)
        : begin_steps(devices), captured(devices), recording(devices) {
        for (int i = 0; i < devices; ++i) { begin_steps[i] = 0; captured[i] = 0; recording[i] = 0; }
    }

    std::vector<std::atomic<long long>> begin_steps;
    std::vector<std::atomic<int>> captured;
    std::vector<std::atomic<int>> recording;
    std::atomic<long long> active_step{0};
    std::atomic<int> path{kPathNone};

    int slots() const { return static_cast<int>(begin_steps.size()); }

    int require_active(long long step) const {
        const long long active = active_step.load();
        if (step == 0 || active != step)
            return fail(kInvalidOperation, "Captured gradient step %lld is not active; active step is %lld.", step, active);
        return kOk;
    }
    int validate_slot(int slot) const {
        if (slot < 0 || slot >= slots()) return fail(kBadArgument, "deviceSlot %d is out of range.", slot);
        return kOk;
    }
    int require_begun(long long step, int slot, int device) const {
        int status = require_active(step);
        if (status == kOk) status = validate_slot(slot);
        if (status != kOk) return status;
        if (begin_steps[slot].load() != step)
            return fail(kInvalidOperation, "CUDA device %d was not begun for captured gradient step %lld.", device, step);
        return kOk;
    }
    int claim_path(int requested, const char* requested_name, const char* conflicting_name) {
        for (;;) {
            int current = path.load();
            if (current == requested) return kOk;
            if (current != kPathNone)
                return fail(kInvalidOperation, "Cannot mix %s with %s in one CUDA gradient reduction step.",
                            requested_name, conflicting_name);
            if (path.compare_exchange_strong(current, requested)) return kOk;
        }
    }
    bool is_capture_recording(long long step, int slot) const {
        return active_step.load() == step && slot >= 0 && slot < slots() &&
               path.load() == kPathCaptureRecording && recording[slot].load() == kDevicePublishing;
    }
};

// ---- stamps and coherence ---------------------------------------------------------
std::atomic<long long> g_reducer_generation{0};

struct Stamp {
    long long generation = 0;
    long long step = 0;
    bool valid() const { return generation > 0 && step > 0; }
    bool operator==(const Stamp& other) const { return generation == other.generation && step == other.step; }
};

enum CoherenceKind : int { kHost = 0, kLocal = 1, kReduced = 2 };

struct GradientRecord {
    int kind = kHost;
    int local_device = -1;
    std::vector<int> reduced_devices;
    Stamp reduction_stamp;
    Stamp pending_stamp;
    long long version = 0;
    long long consumed_version = 0;
    Stamp consumed_stamp;
};

// ---- per-rank step plan -------------------------------------------------------------
struct Segment { int tensor; long long offset; long long length; };
struct Bucket { std::vector<Segment> segments; long long elements = 0; };

struct StepPlan {
    std::vector<long long> numels;
    std::vector<Bucket> buckets;
    std::vector<int> bucket_of;            // per tensor
    std::vector<long long> offset_of;      // per tensor, within its bucket
    std::vector<GradientRecord> records;   // per tensor
    std::vector<long long> notified_step;  // per tensor: step of the last notification
    std::vector<int> remaining;            // per bucket: segments not yet notified
    std::vector<int> bucket_state;         // per bucket: 0 waiting, 1 ready, 2 enqueued
    std::vector<int> devices;              // the device set of the job (rank -> device id)
    int world = 1;
    int block_size = 32;
    long long generation = 0;
    long long step_sequence = 0;
    long long active_step = 0;
    long long device_begun_step = 0;
    long long completed_steps = 0;
    int next_in_order = 0;                 // buckets are enqueued in descending index order
    // one-shot cache of the step's fused sum of squares, valid for exactly the
    // gradient versions it was published with
    bool cache_valid = false;
    double cache_value = 0.0;
    std::vector<long long> cache_versions;
    std::vector<int> cache_devices;
    std::mutex mutex;
};

void build_buckets(const std::vector<long long>& numels, long long target, std::vector<Bucket>& buckets,
                   std::vector<int>& bucket_of, std::vector<long long>& offset_of) {
    buckets.clear();
    bucket_of.assign(numels.size(), 0);
    offset_of.assign(numels.size(), 0);
    Bucket current;
    auto finish = [&]() {
        if (current.segments.empty()) return;
        buckets.push_back(current);
        current = Bucket();
    };
    for (size_t i = 0; i < numels.size(); ++i) {
        const long long length = numels[i];
        if (!current.segments.empty() && current.elements + length > target) finish();
        bucket_of[i] = static_cast<int>(buckets.size());
        offset_of[i] = current.elements;
        current.segments.push_back(Segment{static_cast<int>(i), current.elements, length});
        current.elements += length;
        if (current.elements >= target) finish();
    }
    finish();
}

}  // namespace
}  // namespace ngb

using namespace ngb;

// Copies this thread's last host-logic failure message (NUL-terminated).
NNTRAIN_EXPORT int nntrain_host_last_message(char* buffer, int capacity) {
    if (!buffer || capacity <= 0) return kBadArgument;
    std::snprintf(buffer, static_cast<size_t>(capacity), "%s", t_message.c_str());
    return kOk;
}

// Bucket layout: tensors in order, a bucket closes when the next tensor would
// exceed `target_elements` or the bucket has reached it; a tensor is never
// split (an oversize tensor is a bucket of its own).  bucket_of / offset_of
// receive, per tensor, its bucket and its element offset inside the bucket.
NNTRAIN_EXPORT int nntrain_plan_build_buckets(const long long* numels, int count, long long target_elements,
                                              int* bucket_of, long long* offset_of, int* bucket_count) {
    if (!numels || count <= 0 || target_elements <= 0 || !bucket_of || !offset_of || !bucket_count)
        return fail(kBadArgument, "build_buckets: bad argument.");
    std::vector<long long> lengths(numels, numels + count);
    for (long long n : lengths)
        if (n <= 0) return fail(kBadArgument, "build_buckets: tensor lengths must be positive.");
    std::vector<Bucket> buckets;
    std::vector<int> of;
    std::vector<long long> offsets;
    build_buckets(lengths, target_elements, buckets, of, offsets);
    std::memcpy(bucket_of, of.data(), sizeof(int) * count);
    std::memcpy(offset_of, offsets.data(), sizeof(long long) * count);
    *bucket_count = static_cast<int>(buckets.size());
    return kOk;
}

// ---- publication state exports -----------------------------------------------------
NNTRAIN_EXPORT int nntrain_publication_state_create(int device_count, void** state) {
    if (device_count <= 0 || !state) return fail(kBadArgument, "deviceCount must be positive.");
    *state = new (std::nothrow) PublicationState(device_count);
    return *state ? kOk : fail(kBadArgument, "out of memory.");
}

NNTRAIN_EXPORT int nntrain_publication_state_destroy(void* state) {
    delete static_cast<PublicationState*>(state);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_begin_step(void* state, long long step) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    if (step == 0) return fail(kBadArgument, "stepId must not be zero.");
    if (s->active_step.load() != 0)
        return fail(kInvalidOperation, "The previous captured-gradient publication step is still active.");
    for (int i = 0; i < s->slots(); ++i) { s->begin_steps[i] = 0; s->captured[i] = 0; s->recording[i] = 0; }
    s->path = PublicationState::kPathNone;
    s->active_step = step;
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_mark_device_begun(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_active(step);
    if (status == kOk) status = s->validate_slot(slot);
    if (status != kOk) return status;
    long long expected = 0;
    if (!s->begin_steps[slot].compare_exchange_strong(expected, step))
        return fail(kInvalidOperation, "CUDA device %d was begun twice for captured gradient step %lld.", device, step);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_enter_notification_path(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_begun(step, slot, device);
    if (status != kOk) return status;
    return s->claim_path(PublicationState::kPathNotifications, "leaf notification", "captured device publication");
}

NNTRAIN_EXPORT int nntrain_publication_begin_capture_recording(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_begun(step, slot, device);
    if (status == kOk)
        status = s->claim_path(PublicationState::kPathCaptureRecording, "captured backward recording",
                               "normal or replay publication");
    if (status != kOk) return status;
    int expected = PublicationState::kDeviceNone;
    if (!s->recording[slot].compare_exchange_strong(expected, PublicationState::kDevicePublishing))
        return fail(kInvalidOperation, "CUDA device %d began captured backward recording twice for step %lld.", device, step);
    return kOk;
}

// *recording = 1 when the step is a capture-recording generation and this
// device slot is currently recording.
NNTRAIN_EXPORT int nntrain_publication_is_capture_recording(void* state, long long step, int slot, int* recording) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s || !recording) return fail(kBadArgument, "null argument.");
    *recording = s->is_capture_recording(step, slot) ? 1 : 0;
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_enter_capture_notification_path(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_begun(step, slot, device);
    if (status != kOk) return status;
    if (!s->is_capture_recording(step, slot))
        return fail(kInvalidOperation, "CUDA device %d is not recording captured backward gradients for step %lld.", device, step);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_end_capture_recording(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_active(step);
    if (status == kOk) status = s->validate_slot(slot);
    if (status != kOk) return status;
    int expected = PublicationState::kDevicePublishing;
    if (!s->recording[slot].compare_exchange_strong(expected, PublicationState::kDevicePublished))
        return fail(kInvalidOperation, "CUDA device %d has no captured backward recording to end for step %lld.", device, step);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_validate_capture_discard(void* state, long long step) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_active(step);
    if (status != kOk) return status;
    if (s->path.load() != PublicationState::kPathCaptureRecording)
        return fail(kInvalidOperation, "Gradient step %lld is not a captured backward recording generation.", step);
    bool recorded = false;
    for (int slot = 0; slot < s->slots(); ++slot) {
        const int st = s->recording[slot].load();
        if (st == PublicationState::kDevicePublishing)
            return fail(kInvalidOperation, "Captured backward recording is still active on device slot %d for step %lld.", slot, step);
        recorded |= st == PublicationState::kDevicePublished;
    }
    if (!recorded)
        return fail(kInvalidOperation, "Captured backward recording step %lld recorded no device graph.", step);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_begin_captured_publication(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_begun(step, slot, device);
    if (status == kOk)
        status = s->claim_path(PublicationState::kPathCaptured, "captured device publication", "leaf notification");
    if (status != kOk) return status;
    for (int i = 0; i < s->slots(); ++i)
        if (s->captured[i].load() == PublicationState::kDeviceFailed)
            return fail(kInvalidOperation, "Captured gradient step %lld already failed and must be aborted before reuse.", step);
    int previous = PublicationState::kDeviceNone;
    if (!s->captured[slot].compare_exchange_strong(previous, PublicationState::kDevicePublishing)) {
        const char* what = previous == PublicationState::kDevicePublishing ? "is already being published"
                           : previous == PublicationState::kDevicePublished ? "was published twice"
                           : previous == PublicationState::kDeviceFailed    ? "previously failed"
                                                                            : "has an invalid publication state";
        return fail(kInvalidOperation, "CUDA device %d %s for captured gradient step %lld.", device, what, step);
    }
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_complete_captured_publication(void* state, long long step, int slot, int device) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_active(step);
    if (status == kOk) status = s->validate_slot(slot);
    if (status != kOk) return status;
    int expected = PublicationState::kDevicePublishing;
    if (!s->captured[slot].compare_exchange_strong(expected, PublicationState::kDevicePublished))
        return fail(kInvalidOperation, "CUDA device %d has no captured gradient publication to complete for step %lld.", device, step);
    return kOk;
}

// Never fails: a stale step or slot is ignored.
NNTRAIN_EXPORT int nntrain_publication_fail_captured_publication(void* state, long long step, int slot) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s || s->active_step.load() != step || slot < 0 || slot >= s->slots()) return kOk;
    int expected = PublicationState::kDevicePublishing;
    s->captured[slot].compare_exchange_strong(expected, PublicationState::kDeviceFailed);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_validate_complete(void* state, long long step) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    int status = s->require_active(step);
    if (status != kOk) return status;
    const int path = s->path.load();
    if (path == PublicationState::kPathCaptureRecording)
        return fail(kInvalidOperation, "Captured backward recording step %lld must be discarded, not completed as a reduction.", step);
    if (path != PublicationState::kPathCaptured) return kOk;
    for (int slot = 0; slot < s->slots(); ++slot) {
        const int st = s->captured[slot].load();
        if (st == PublicationState::kDeviceFailed)
            return fail(kInvalidOperation, "Captured gradient publication failed on device slot %d for step %lld; abort is required.", slot, step);
        if (st != PublicationState::kDevicePublished)
            return fail(kInvalidOperation, "Captured gradients were not published on device slot %d for step %lld.", slot, step);
    }
    return kOk;
}

NNTRAIN_EXPORT int nntrain_publication_end_step(void* state, long long step) {
    auto* s = static_cast<PublicationState*>(state);
    if (!s) return fail(kBadArgument, "null state.");
    long long expected = step;
    if (s->active_step.compare_exchange_strong(expected, 0)) s->path = PublicationState::kPathNone;
    return kOk;
}

// ---- per-rank step plan ----------------------------------------------------------------
// One rank's view of an N-rank reducer over a list of tensors: buckets, the
// exactly-once notification bookkeeping, the fixed bucket order every rank
// enqueues its collectives in, reduction stamps and the optimizer guard.
// `devices` lists the job's device ids in rank order (the coherence records
// keep them, as the reference's tensors keep their reduced-device set).
NNTRAIN_EXPORT int nntrain_plan_create(const long long* numels, int count, long long target_bucket_elements,
                                       const int* devices, int world, int block_size, void** plan) {
    if (!numels || count <= 0 || target_bucket_elements <= 0 || !devices || world < 1 || !plan ||
        (block_size != 32 && block_size != 64 && block_size != 128))
        return fail(kBadArgument, "plan_create: bad argument.");
    for (int i = 0; i < count; ++i)
        if (numels[i] <= 0) return fail(kBadArgument, "plan_create: tensor lengths must be positive.");
    for (int a = 0; a < world; ++a) {
        if (devices[a] < 0) return fail(kInvalidOperation, "CUDA reducer devices must be unique and non-negative.");
        for (int b = 0; b < a; ++b)
            if (devices[a] == devices[b])
                return fail(kInvalidOperation, "CUDA reducer devices must be unique and non-negative.");
    }
    StepPlan* p = new (std::nothrow) StepPlan();
    if (!p) return fail(kBadArgument, "out of memory.");
    p->numels.assign(numels, numels + count);
    build_buckets(p->numels, target_bucket_elements, p->buckets, p->bucket_of, p->offset_of);
    p->records.resize(count);
    p->notified_step.assign(count, 0);
    p->remaining.assign(p->buckets.size(), 0);
    p->bucket_state.assign(p->buckets.size(), 0);
    p->devices.assign(devices, devices + world);
    p->world = world;
    p->block_size = block_size;
    p->generation = ++g_reducer_generation;      // a rebuilt reducer invalidates older stamps
    *plan = p;
    return kOk;
}

NNTRAIN_EXPORT int nntrain_plan_destroy(void* plan) {
    delete static_cast<StepPlan*>(plan);
    return kOk;
}

NNTRAIN_EXPORT int nntrain_plan_bucket_count(void* plan, int* count) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !count) return fail(kBadArgument, "null argument.");
    *count = static_cast<int>(p->buckets.size());
    return kOk;
}

NNTRAIN_EXPORT int nntrain_plan_bucket_elements(void* plan, int bucket, long long* elements) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !elements || bucket < 0 || bucket >= static_cast<int>(p->buckets.size()))
        return fail(kBadArgument, "bucket index out of range.");
    *elements = p->buckets[bucket].elements;
    return kOk;
}

// Where a tensor's gradient lives: its bucket and element offset in the
// bucket's arena (running sum of the lengths before it, no padding).
NNTRAIN_EXPORT int nntrain_plan_locate(void* plan, int tensor, int* bucket, long long* offset) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !bucket || !offset || tensor < 0 || tensor >= static_cast<int>(p->numels.size()))
        return fail(kBadArgument, "tensor index out of range.");
    *bucket = p->bucket_of[tensor];
    *offset = p->offset_of[tensor];
    return kOk;
}

// Bytes this rank sends per step: 2 (N-1)/N * sum over buckets of
// (elements + 4 ceil(elements / block)).  For N = 2 and block 128 this is the
// reference's 2 (E + 4 ceil(E / 128)) per pair of devices
// (NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:267-270).
NNTRAIN_EXPORT int nntrain_plan_transport_bytes_per_step(void* plan, long long* bytes) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !bytes) return fail(kBadArgument, "null argument.");
    long long total = 0;
    for (const Bucket& b : p->buckets) total += b.elements + 4 * ((b.elements + p->block_size - 1) / p->block_size);
    *bytes = 2 * (p->world - 1) * total / p->world;
    return kOk;
}

NNTRAIN_EXPORT int nntrain_plan_begin_step(void* plan, long long* step_id) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !step_id) return fail(kBadArgument, "null argument.");
    std::lock_guard<std::mutex> guard(p->mutex);
    if (p->active_step != 0) return fail(kInvalidOperation, "The previous gradient reduction step is still active.");
    long long step = ++p->step_sequence;
    if (step == 0) step = ++p->step_sequence;
    for (GradientRecord& r : p->records) {
        r.pending_stamp.generation = p->generation;
        r.pending_stamp.step = step;
    }
    for (size_t b = 0; b < p->buckets.size(); ++b) {
        p->remaining[b] = static_cast<int>(p->buckets[b].segments.size());
        p->bucket_state[b] = 0;
    }
    p->next_in_order = static_cast<int>(p->buckets.size()) - 1;
    p->device_begun_step = 0;
    p->active_step = step;
    *step_id = step;
    return kOk;
}

NNTRAIN_EXPORT int nntrain_plan_begin_device_step(void* plan, long long step) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p) return fail(kBadArgument, "null plan.");
    std::lock_guard<std::mutex> guard(p->mutex);
    if (p->active_step != step || step == 0) return fail(kInvalidOperation, "Gradient step %lld is not active.", step);
    if (p->device_begun_step == step)
        return fail(kInvalidOperation, "This rank's device was begun twice for step %lld.", step);
    p->device_begun_step = step;
    return kOk;
}

// A tensor's gradient is final on this rank.  *bucket_ready = the bucket that
// this notification completed, or -1.
NNTRAIN_EXPORT int nntrain_plan_notify_gradient_ready(void* plan, long long step, int tensor, int* bucket_ready) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !bucket_ready) return fail(kBadArgument, "null argument.");
    *bucket_ready = -1;
    std::lock_guard<std::mutex> guard(p->mutex);
    if (p->active_step != step || step == 0) return fail(kInvalidOperation, "Gradient step %lld is not active.", step);
    if (tensor < 0 || tensor >= static_cast<int>(p->numels.size())) return fail(kBadArgument, "tensor index out of range.");
    if (p->device_begun_step != step)
        return fail(kInvalidOperation, "This rank's device was not begun for step %lld.", step);
    if (p->notified_step[tensor] == step)
        return fail(kInvalidOperation, "Gradient %d was notified twice for step %lld.", tensor, step);
    p->notified_step[tensor] = step;
    GradientRecord& record = p->records[tensor];
    record.kind = kLocal;                 // a fresh local gradient: a new version exists
    record.local_device = p->devices[0];
    ++record.version;
    const int bucket = p->bucket_of[tensor];
    if (--p->remaining[bucket] == 0) {
        p->bucket_state[bucket] = 1;
        *bucket_ready = bucket;
    }
    return kOk;
}

// The next bucket this rank may enqueue, or -1.  Collectives must be issued
// in the same order on every rank; the order is fixed (descending bucket
// index: backward produces the last layers first), so a ready bucket waits
// for the ready buckets ordered before it.  Calling this marks the returned
// bucket as enqueued.
NNTRAIN_EXPORT int nntrain_plan_next_enqueueable(void* plan, long long step, int* bucket) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !bucket) return fail(kBadArgument, "null argument.");
    *bucket = -1;
    std::lock_guard<std::mutex> guard(p->mutex);
    if (p->active_step != step || step == 0) return fail(kInvalidOperation, "Gradient step %lld is not active.", step);
    if (p->next_in_order >= 0 && p->bucket_state[p->next_in_order] == 1) {
        p->bucket_state[p->next_in_order] = 2;
        *bucket = p->next_in_order--;
    }
    return kOk;
}

// Ends a step whose every bucket was enqueued: `non_finite` is the step's
// device flag as read by the caller.  Marks every gradient Reduced with this
// step's stamp.  A step with a bucket left fails and stays active (abort it).
NNTRAIN_EXPORT int nntrain_plan_complete(void* plan, long long step, int non_finite) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p) return fail(kBadArgument, "null plan.");
    std::lock_guard<std::mutex> guard(p->mutex);
    if (p->active_step != step || step == 0) return fail(kInvalidOperation, "Gradient step %lld is not active.", step);
    for (size_t b = 0; b < p->buckets.size(); ++b)
        if (p->bucket_state[b] != 2)
            return fail(kInvalidOperation, "Gradient bucket %d was not completed for step %lld.", static_cast<int>(b), step);
    if (non_finite != 0)
        return fail(kInvalidOperation, "Gradient reduction step %lld produced a non-finite gradient.", step);
    for (GradientRecord& r : p->records) {
        r.kind = kReduced;
        r.reduced_devices = p->devices;
        r.reduction_stamp = r.pending_stamp;
        r.pending_stamp = Stamp();
        ++r.version;
    }
    p->active_step = 0;
    ++p->completed_steps;
    return kOk;
}

// Fail-closed end of a step: pending stamps are dropped, nothing becomes Reduced.
NNTRAIN_EXPORT int nntrain_plan_abort(void* plan, long long step) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p) return fail(kBadArgument, "null plan.");
    std::lock_guard<std::mutex> guard(p->mutex);
    if (p->active_step != step) return kOk;
    for (GradientRecord& r : p->records) r.pending_stamp = Stamp();
    p->active_step = 0;
    return kOk;
}

NNTRAIN_EXPORT int nntrain_plan_completed_steps(void* plan, long long* steps) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !steps) return fail(kBadArgument, "null argument.");
    *steps = p->completed_steps;
    return kOk;
}

// out[0] = kind (0 host, 1 local, 2 reduced), out[1] = reduction stamp
// generation, out[2] = reduction stamp step, out[3] = pending step,
// out[4] = gradient version, out[5] = consumed version.
NNTRAIN_EXPORT int nntrain_plan_coherence_snapshot(void* plan, int tensor, long long* out6) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !out6 || tensor < 0 || tensor >= static_cast<int>(p->numels.size()))
        return fail(kBadArgument, "tensor index out of range.");
    std::lock_guard<std::mutex> guard(p->mutex);
    const GradientRecord& r = p->records[tensor];
    out6[0] = r.kind; out6[1] = r.reduction_stamp.generation; out6[2] = r.reduction_stamp.step;
    out6[3] = r.pending_stamp.step; out6[4] = r.version; out6[5] = r.consumed_version;
    return kOk;
}

// The optimizer guard: every gradient must carry the same completed stamp of
// the NEWEST reducer generation over exactly `devices`, not be pending, and
// not have been consumed; then all are claimed.  Validation runs over the
// whole set before anything is claimed (fail-closed).
NNTRAIN_EXPORT int nntrain_plan_optimizer_validate_and_consume(void* plan, const int* devices, int device_count) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !devices) return fail(kBadArgument, "null argument.");
    if (device_count <= 0) return fail(kInvalidOperation, "A CUDA optimizer requires at least one execution device.");
    for (int a = 0; a < device_count; ++a) {
        if (devices[a] < 0) return fail(kInvalidOperation, "CUDA optimizer devices must be unique and non-negative.");
        for (int b = 0; b < a; ++b)
            if (devices[a] == devices[b])
                return fail(kInvalidOperation, "CUDA optimizer devices must be unique and non-negative.");
    }
    std::lock_guard<std::mutex> guard(p->mutex);
    Stamp expected;
    const long long newest = g_reducer_generation.load();
    for (size_t i = 0; i < p->records.size(); ++i) {
        const GradientRecord& r = p->records[i];
        if (r.pending_stamp.valid())
            return fail(kInvalidOperation, "CUDA gradient %d belongs to an incomplete reduction step %lld.",
                        static_cast<int>(i), r.pending_stamp.step);
        if (r.version == r.consumed_version)
            return fail(kInvalidOperation, "CUDA gradient %d was already consumed by an optimizer update.", static_cast<int>(i));
        if (device_count == 1) {
            const bool local = r.kind == kLocal && r.local_device == devices[0];
            bool reduced = false;
            if (r.kind == kReduced)
                for (int d : r.reduced_devices) reduced |= d == devices[0];
            if (!local && !reduced)
                return fail(kInvalidOperation, "CUDA gradient %d is not current on device %d.", static_cast<int>(i), devices[0]);
            continue;
        }
        bool same_devices = r.reduced_devices.size() == static_cast<size_t>(device_count);
        for (int d = 0; same_devices && d < device_count; ++d) same_devices = r.reduced_devices[d] == devices[d];
        if (r.kind != kReduced || !r.reduction_stamp.valid() || !same_devices ||
            r.reduction_stamp.generation != newest)
            return fail(kInvalidOperation, "CUDA gradient %d has not been reduced across the active device set.", static_cast<int>(i));
        if (r.reduction_stamp == r.consumed_stamp)
            return fail(kInvalidOperation, "CUDA gradient %d reduction step was already consumed by an optimizer update.", static_cast<int>(i));
        if (!expected.valid()) expected = r.reduction_stamp;
        else if (!(r.reduction_stamp == expected))
            return fail(kInvalidOperation, "CUDA optimizer parameters do not share one completed gradient reduction step.");
    }
    for (GradientRecord& r : p->records) {
        r.consumed_version = r.version;
        if (device_count > 1) r.consumed_stamp = expected;
    }
    return kOk;
}

// ---- fused sum-of-squares cache and the clip decision ------------------------------------
// The reducer publishes the sum of squares it fused into the reduction; the
// clip consumes it once, and only if no gradient changed since
// (NNtrain.Core/Tensors/Tensor.CudaKernels.cs:768-854).  A non-finite or
// negative value is not cached.
NNTRAIN_EXPORT int nntrain_plan_publish_squared_sum(void* plan, const int* devices, int device_count,
                                                    double squared_sum) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !devices || device_count <= 0) return fail(kBadArgument, "null argument.");
    if (!std::isfinite(squared_sum) || squared_sum < 0.0) return kOk;
    std::lock_guard<std::mutex> guard(p->mutex);
    p->cache_versions.clear();
    for (const GradientRecord& r : p->records) p->cache_versions.push_back(r.version);
    p->cache_devices.assign(devices, devices + device_count);
    p->cache_value = squared_sum;
    p->cache_valid = true;
    return kOk;
}

// *hit = 1 and *squared_sum = the cached value when the cache matches the
// device set and every gradient version; the entry is dropped either way.
NNTRAIN_EXPORT int nntrain_plan_try_consume_squared_sum(void* plan, const int* devices, int device_count,
                                                        double* squared_sum, int* hit) {
    auto* p = static_cast<StepPlan*>(plan);
    if (!p || !devices || device_count <= 0 || !squared_sum || !hit) return fail(kBadArgument, "null argument.");
    std::lock_guard<std::mutex> guard(p->mutex);
    *hit = 0;
    *squared_sum = 0.0;
    if (!p->cache_valid) return kOk;
    p->cache_valid = false;
    if (static_cast<int>(p->cache_devices.size()) != device_count) return kOk;
    for (int d = 0; d < device_count; ++d)
        if (p->cache_devices[d] != devices[d]) return kOk;
    for (size_t i = 0; i < p->records.size(); ++i)
        if (p->records[i].version != p->cache_versions[i]) return kOk;
    *hit = 1;
    *squared_sum = p->cache_value;
    return kOk;
}

// norm = (float)sqrt(squared_sum); coefficient = norm > max_norm ?
// max_norm / (norm + 1e-6f) : 1 (NNtrain.Core/Torch/nn.cs:69-72).  max_norm
// must be positive (nn.cs:41-47).
NNTRAIN_EXPORT int nntrain_gradient_clip_decision(double squared_sum, float max_norm, float* norm,
                                                  float* coefficient) {
    if (!norm || !coefficient) return fail(kBadArgument, "null argument.");
    if (!(max_norm > 0.0f)) return fail(kBadArgument, "The maximum gradient norm must be positive.");
    const float total = static_cast<float>(std::sqrt(squared_sum));
    *norm = total;
    *coefficient = total > max_norm ? max_norm / (total + 1e-6f) : 1.0f;
    return kOk;
}
