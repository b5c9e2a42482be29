// Integer-throughput probe: the denominator for the ALU-bound hash searches.
//
// The 32-bit hashes (BLAKE-256, SHA-256d, and BLAKE2b as pairs of 32-bit halves) are
// chains of add / xor / rotate.  Their ceiling is not a memory rate but the rate at which an
// SM can issue such operations, and no published figure covers this mix.  The kernel below runs
// the same three operations on sixteen independent chains per thread with nothing else in the
// loop, so that neither dependencies nor memory limit it; the caller times it and divides.
//
//   mix 0  xor + rotate                      (logic and funnel shift only)
//   mix 1  add + xor + rotate                (all three on the integer pipe)
//   mix 2  add + xor + rotate, the add written as a multiply-add by one so that it issues to
//          the FMA pipe, the arrangement the hash roles use
#include "launch.cuh"

namespace hfuse {
namespace {

constexpr int kChains = 16;
constexpr int kProbeThreads = 256;

template <int MIX>
__global__ void __launch_bounds__(kProbeThreads) int_probe_kernel(uint32_t iters, uint32_t one, uint32_t salt, uint32_t* sink) {
    uint32_t x[kChains], y[kChains];
#pragma unroll
    for (int c = 0; c < kChains; ++c) {
        x[c] = (threadIdx.x + blockIdx.x * blockDim.x) * 0x9E3779B9u + c * salt;
        y[c] = x[c] ^ (salt >> (c & 7));
    }
    for (uint32_t i = 0; i < iters; ++i) {
#pragma unroll
        for (int c = 0; c < kChains; ++c) {
            if (MIX == 1) x[c] = x[c] + y[c];
            if (MIX == 2) asm volatile("mad.lo.u32 %0, %1, %2, %3;" : "=r"(x[c]) : "r"(x[c]), "r"(one), "r"(y[c]));
            y[c] ^= x[c];
            y[c] = __funnelshift_r(y[c], y[c], 7 + (c & 3));
        }
    }
    uint32_t acc = 0;
#pragma unroll
    for (int c = 0; c < kChains; ++c) acc ^= x[c] + y[c];
    if (acc == 0x5EEDF00Du && one == 2) *sink = acc;   // never true: keeps the chains alive without a store
}

}  // namespace
}  // namespace hfuse

extern "C" int hfuse_int32_probe(int mix, uint32_t iters, uint32_t* sink, uint64_t* lane_ops, hfuse_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    using namespace hfuse;
    if (mix < 0 || mix > 2 || iters == 0 || !sink || !lane_ops) return HFUSE_ERR_BAD_ARG;
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    const int grid = f.sms * 8;   // 8 x 256 threads fill every SM's 2048 thread slots
    const uint32_t one = 1, salt = 0x85EBCA6Bu;
    switch (mix) {
    case 0: int_probe_kernel<0><<<grid, kProbeThreads, 0, stream>>>(iters, one, salt, sink); break;
    case 1: int_probe_kernel<1><<<grid, kProbeThreads, 0, stream>>>(iters, one, salt, sink); break;
    default: int_probe_kernel<2><<<grid, kProbeThreads, 0, stream>>>(iters, one, salt, sink); break;
    }
    if (cudaGetLastError() != cudaSuccess) return HFUSE_ERR_LAUNCH;
    *lane_ops = (uint64_t)grid * kProbeThreads * iters * kChains * (mix == 0 ? 2 : 3);
    return HFUSE_OK;
}
