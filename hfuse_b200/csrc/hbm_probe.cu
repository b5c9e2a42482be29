// Memory-traffic probe: the denominator for kernels whose traffic is mostly writes.
//
// The measured copy bandwidth is taken with equal reads and writes.  The DL kernels here write
// four to nine times what they read, and HBM3e turns out to sustain less for such a mix, however
// the stores are issued.  This kernel moves a given number of bytes in and a given number out
// with 16-byte loads and 32-byte streaming stores and nothing else, so a caller can time the
// same mix as the kernel it is to be compared with.
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

// The same traffic with the writes leaving as bulk (TMA) copies from shared memory: every block
// fills an 8 KB buffer (the part that is read comes through 16-byte loads, the rest is a
// constant) and one thread sends it off; two buffers, so a copy drains while the next is filled.
constexpr int kProbeChunk = 8192;
__global__ void __launch_bounds__(256, 4) hbm_probe_bulk_kernel(const float4* __restrict__ in, size_t n_in4, float* out,
                                                                size_t n_chunks, size_t in4_per_chunk) {
    __shared__ __align__(128) float4 buf[2][kProbeChunk / 16];
    int b = 0;
    for (size_t c = blockIdx.x; c < n_chunks; c += gridDim.x, b ^= 1) {
        if (threadIdx.x == 0) bulk_wait_read<1>();
        __syncthreads();
        for (int i = threadIdx.x; i < kProbeChunk / 16; i += blockDim.x) {
            float4 v = make_float4(1.f, 2.f, 3.f, 4.f);
            const size_t src = c * in4_per_chunk + (size_t)i;
            if ((size_t)i < in4_per_chunk && src < n_in4) v = ldg_stream4(reinterpret_cast<const float*>(in + src));
            buf[b][i] = v;
        }
        fence_proxy_async_shared();
        __syncthreads();
        if (threadIdx.x == 0) {
            bulk_store(out + c * (kProbeChunk / 4), buf[b], kProbeChunk);
            bulk_commit();
        }
    }
    if (threadIdx.x == 0) bulk_wait<0>();
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

extern "C" int hfuse_hbm_probe_bulk(const void* src, size_t read_bytes, void* dst, size_t write_bytes, hfuse_stream_t stream_) {
    using namespace hfuse;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!dst || write_bytes == 0 || write_bytes % kProbeChunk || read_bytes % 16 || (read_bytes && !src)) return HFUSE_ERR_BAD_ARG;
    if (read_bytes > write_bytes) return HFUSE_ERR_BAD_ARG;
    if (((uintptr_t)dst & 31) || ((uintptr_t)src & 15)) return HFUSE_ERR_ALIGNMENT;
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    const size_t chunks = write_bytes / kProbeChunk;
    const size_t in4_per_chunk = (read_bytes / 16 + chunks - 1) / chunks;
    hbm_probe_bulk_kernel<<<f.sms * 4, 256, 0, stream>>>(static_cast<const float4*>(src), read_bytes / 16,
                                                         static_cast<float*>(dst), chunks, in4_per_chunk);
    return check_launch();
}
