// Memory-traffic probe: the denominator for kernels whose traffic is mostly writes.
//
// The measured copy bandwidth is taken with equal reads and writes.  The DL kernels here write
// four to nine times what they read, and HBM3e turns out to sustain less for such a mix, however
// the stores are issued.  This kernel moves a given number of bytes in and a given number out
// with 16-byte loads and 32-byte streaming stores and nothing else, so a caller can time the
// same mix as the kernel it wants to judge.
#include "launch.cuh"

namespace hfuse {
namespace {

// Writes n_out8 groups of eight floats; the first n_in4 * 4 floats read come from `in` (each
// 16-byte load feeds one 32-byte store, repeated), the rest of the output is a constant.
__global__ void __launch_bounds__(512, 2) hbm_probe_kernel(const float4* __restrict__ in, size_t n_in4, float* out,
                                                           size_t n_out8) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_out8; i += stride) {
        float4 v = make_float4(1.f, 2.f, 3.f, 4.f);
        if (i < n_in4) v = ldg_stream4(reinterpret_cast<const float*>(in + i));
        const float o[8] = {v.x, v.y, v.z, v.w, v.x, v.y, v.z, v.w};
        stg_stream8(out + 8 * i, o);
    }
}

}  // namespace
}  // namespace hfuse

extern "C" int hfuse_hbm_probe(const void* src, size_t read_bytes, void* dst, size_t write_bytes, hfuse_stream_t stream_) {
    using namespace hfuse;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!dst || write_bytes == 0 || write_bytes % 32 || read_bytes % 16 || (read_bytes && !src)) return HFUSE_ERR_BAD_ARG;
    if (read_bytes / 16 > write_bytes / 32) return HFUSE_ERR_BAD_ARG;     // one load per store at most
    if (((uintptr_t)dst & 31) || ((uintptr_t)src & 15)) return HFUSE_ERR_ALIGNMENT;
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    hbm_probe_kernel<<<f.sms * 2, 512, 0, stream>>>(static_cast<const float4*>(src), read_bytes / 16,
                                                    static_cast<float*>(dst), write_bytes / 32);
    return check_launch();
}
