// ABI gate, error ring, per-thread device / stream selection and the
// capability bitmap: the few process-level exports the reference's managed
// gateway probes before it uses the gradient path
// (NNtrain.Cuda/native/cuda_runtime_bridge.cu:74-131,1436-1536,2336-2339;
//  NNtrain.Cuda/native/tensor_kernels.cu:2888-2891).
#include "common.cuh"

#include <array>
#include <atomic>
#include <mutex>

namespace ngb {
namespace {

constexpr std::size_t kRingCapacity = 64;
std::mutex g_error_mutex;
std::uint64_t g_error_sequence = 0;
std::array<ErrorInfo, kRingCapacity> g_error_ring{};
ErrorInfo g_last_error{sizeof(ErrorInfo), kAbiVersion, 0, 0, -1, kOpNone, 0};

thread_local int t_selected_device = -1;
thread_local cudaStream_t t_implicit_stream = nullptr;

constexpr int kMaxDevices = 64;
int g_sm_counts[kMaxDevices] = {};

std::atomic<int> g_codec_iterations_per_cta{2};
std::atomic<int> g_collective_ctas{0};
std::atomic<int> g_collective_async{1};
std::atomic<int> g_codec_ctas{0};

}  // namespace

int complete(Operation operation, int device, int status) {
    if (status == static_cast<int>(cudaSuccess)) return status;
    std::lock_guard<std::mutex> guard(g_error_mutex);
    const std::uint64_t sequence = ++g_error_sequence;
    ErrorInfo entry{sizeof(ErrorInfo), kAbiVersion, sequence, status, device,
                    static_cast<std::uint32_t>(operation), 0};
    g_last_error = entry;
    g_error_ring[(sequence - 1) % kRingCapacity] = entry;
    return status;
}

int select_device(int device) {
    // The cached selection is trusted only when the runtime agrees: another
    // library in the process (the host's tensor library, a second gateway) may
    // have switched the thread's device since the last call.
    int current = -1;
    if (t_selected_device == device && cudaGetDevice(&current) == cudaSuccess && current == device)
        return static_cast<int>(cudaSuccess);
    cudaError_t status = cudaSetDevice(device);
    if (status == cudaSuccess) t_selected_device = device;
    return static_cast<int>(status);
}

cudaStream_t& implicit_stream() { return t_implicit_stream; }

LaunchPolicy launch_policy() {
    return LaunchPolicy{g_codec_iterations_per_cta.load(std::memory_order_relaxed),
                        g_collective_ctas.load(std::memory_order_relaxed),
                        g_collective_async.load(std::memory_order_relaxed),
                        g_codec_ctas.load(std::memory_order_relaxed)};
}

void set_codec_ctas(int ctas) { g_codec_ctas.store(ctas > 0 ? ctas : 0, std::memory_order_relaxed); }

void set_collective_async(int mode) { g_collective_async.store(mode < 0 ? 0 : (mode > 4 ? 4 : mode), std::memory_order_relaxed); }

void set_launch_policy(int codec_iterations_per_cta, int collective_ctas) {
    g_codec_iterations_per_cta.store(codec_iterations_per_cta, std::memory_order_relaxed);
    g_collective_ctas.store(collective_ctas, std::memory_order_relaxed);
}

int sm_count() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 148;
    int cached = g_sm_counts[device];
    if (cached > 0) return cached;
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
        count = 148;
    g_sm_counts[device] = count;
    return count;
}

}  // namespace ngb

using namespace ngb;

NNTRAIN_EXPORT std::uint32_t nntrain_abi_version() { return kAbiVersion; }

NNTRAIN_EXPORT int nntrain_last_error(ErrorInfo* destination, size_t destination_size) {
    if (!destination || destination_size < sizeof(ErrorInfo))
        return static_cast<int>(cudaErrorInvalidValue);
    std::lock_guard<std::mutex> guard(g_error_mutex);
    *destination = g_last_error;
    return static_cast<int>(cudaSuccess);
}

// Finds the newest ring entry matching (status, device, operation).
NNTRAIN_EXPORT int nntrain_error_snapshot(int status, int device, std::uint32_t operation,
                                          ErrorInfo* destination, size_t destination_size) {
    if (!destination || destination_size < sizeof(ErrorInfo))
        return static_cast<int>(cudaErrorInvalidValue);
    std::lock_guard<std::mutex> guard(g_error_mutex);
    const std::uint64_t live = g_error_sequence < kRingCapacity ? g_error_sequence : kRingCapacity;
    for (std::uint64_t back = 0; back < live; ++back) {
        const std::uint64_t sequence = g_error_sequence - back;
        const ErrorInfo& entry = g_error_ring[(sequence - 1) % kRingCapacity];
        if (entry.sequence == sequence && entry.status == status && entry.device == device &&
            entry.operation == operation) {
            *destination = entry;
            return static_cast<int>(cudaSuccess);
        }
    }
    return static_cast<int>(cudaErrorInvalidValue);
}

// Bits as the reference defines them (cuda_runtime_bridge.cu:1505-1516); this
// library implements only the gradient path, so it reports bit 1 (bfloat16),
// bit 6 (asynchronous gradient reduction), bit 7 (CUDA graphs: every local
// kernel here is capturable) and bit 8 (BFP8 quantization).
NNTRAIN_EXPORT int nntrain_capability_bitmap(int device, unsigned long long* bitmap,
                                             int* compute_capability_major,
                                             int* compute_capability_minor) {
    if (!bitmap || !compute_capability_major || !compute_capability_minor)
        return complete(kOpCapabilities, device, static_cast<int>(cudaErrorInvalidValue));
    int major = 0, minor = 0;
    cudaError_t status = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (status == cudaSuccess)
        status = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
    if (status != cudaSuccess) return complete(kOpCapabilities, device, static_cast<int>(status));
    unsigned long long features = 0;
    if (major >= 10) features = (1ull << 1) | (1ull << 6) | (1ull << 7) | (1ull << 8);
    *bitmap = features;
    *compute_capability_major = major;
    *compute_capability_minor = minor;
    return static_cast<int>(cudaSuccess);
}

NNTRAIN_EXPORT int nntrain_cuda_set_device(int device) {
    return complete(kOpSetDevice, device, select_device(device));
}

// Launch shapes for overlapping the collective with the codec kernels of
// neighbouring chunks (ABI minor 36; the reference has no counterpart: its
// kernels use fixed grids).  codec_iterations_per_cta: n > 0 = short-lived CTAs
// of n iterations each (default 2), 0 = persistent grids.  collective_ctas: 0 = fill the
// machine, n > 0 = at most n CTAs for the all-reduce kernels.
NNTRAIN_EXPORT int nntrain_gradient_configure(int codec_iterations_per_cta, int collective_ctas) {
    if (codec_iterations_per_cta < 0 || collective_ctas < 0) return static_cast<int>(cudaErrorInvalidValue);
    set_launch_policy(codec_iterations_per_cta, collective_ctas);
    return static_cast<int>(cudaSuccess);
}

// Process-wide default for how the owner / all-reduce kernels fetch their
// inputs (ABI minor 36, no counterpart in the reference): 1 (default) =
// cp.async rings in shared memory, 0 = register prefetch, 2 = cp.async rings
// in CTAs that take a whole SM each, 3 = bulk asynchronous copies (whole
// tiles per request) in CTAs that own their SM, 4 = the same in small CTAs that
// share it.  Same results either way; a group's own shape
// (nntrain_gradient_group_configure) overrides it.
NNTRAIN_EXPORT int nntrain_gradient_configure_collective(int asynchronous_copies) {
    if (asynchronous_copies < 0 || asynchronous_copies > 4) return static_cast<int>(cudaErrorInvalidValue);
    set_collective_async(asynchronous_copies);
    return static_cast<int>(cudaSuccess);
}

// Caps the CTAs of a persistent encode / decode grid (only used when
// codec_iterations_per_cta is 0): bounds the share of HBM bandwidth and SM
// slots a codec kernel takes while the collective runs.  0 = no cap.
NNTRAIN_EXPORT int nntrain_gradient_configure_codec_cap(int ctas) {
    if (ctas < 0) return static_cast<int>(cudaErrorInvalidValue);
    set_codec_ctas(ctas);
    return static_cast<int>(cudaSuccess);
}

NNTRAIN_EXPORT int nntrain_cuda_use_external_stream(void* stream) {
    implicit_stream() = reinterpret_cast<cudaStream_t>(stream);
    return static_cast<int>(cudaSuccess);
}
