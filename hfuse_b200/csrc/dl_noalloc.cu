// Batch-norm statistics for callers that cannot allocate device memory.
//
// hfuse_bnstats_f32 needs a scratch buffer from its caller whenever a channel is
// cut into slices.  Some callers have no way to provide one: code running inside a
// framework's memory-planning phase, plugins that are handed fixed input and output
// buffers and nothing else, and hosts whose allocator must not be entered from the
// calling thread.  For them this file keeps the scratch inside the library itself, in
// a file-scope device array that every GPU loading the library holds until exit.
#include "dl_host.cuh"

namespace {

// Largest channel count the built-in scratch serves: tickets plus kBnMaxSlices slice
// moments per channel = 3,149,824 bytes per GPU.
constexpr int kNoAllocMaxChannels = HFUSE_NOALLOC_MAX_CHANNELS;
constexpr size_t kNoAllocBytes =
    ((((size_t)kNoAllocMaxChannels * sizeof(unsigned)) + 255) & ~(size_t)255) +
    (size_t)kNoAllocMaxChannels * hfuse::kBnMaxSlices * 3 * sizeof(float);

static __device__ __align__(256) unsigned char g_bn_scratch[kNoAllocBytes];

// In host code `g_bn_scratch` is only a handle for the runtime, not a device address;
// the address is asked for once per device, with that device current.
constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

int scratch_for_current_device(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return HFUSE_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_bn_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return HFUSE_ERR_LAUNCH;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return HFUSE_OK;
}

}  // namespace

extern "C" int hfuse_bnstats_noalloc_f32(const float* x, int N, int C, int HW, float eps, float* mean,
                                         float* invstd, double* moments, hfuse_stream_t stream) {
    if (C > kNoAllocMaxChannels) return HFUSE_ERR_NOALLOC_LIMIT;
    void* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    BnStatsArgs a;
    if (int rc = prep_bnstats(x, N, C, HW, eps, mean, invstd, moments, scratch, kNoAllocBytes, a)) return rc;
    // The array is shared by every call and keeps what the last one left: the tickets
    // must be zero when the kernel starts, so clear them here on the caller's stream
    // (a kernel that was cut short could otherwise poison every later call).
    if (cudaMemsetAsync(scratch, 0, hfuse::bn_ticket_bytes(C), S_(stream)) != cudaSuccess) return HFUSE_ERR_LAUNCH;
    return dispatch_solo<BnStatsRole>("bnstats", kDefaultSolo_bnstats, a, S_(stream));
}
