// Shared device helpers for the horizontally fused kernels (sm_100a only).
//
// A fused kernel splits one thread block into two contiguous thread ranges
// ("roles").  The shape follows what aoli-al/HFuse emits: range guards
// (lib/KernelFuser/KernelFusion.cpp:5-10), thread ids re-derived from the
// range start (lib/KernelFuser/ThreadInfoRewriter.cpp:38-58) and every
// block-wide barrier replaced by a named partial barrier `bar.sync id, count`
// with one id per original kernel, counting from 1
// (lib/KernelFuser/BarrierRewriter.cpp:12-28).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "hfuse_b200 kernels are written for sm_100a only"
#endif

namespace hfuse {

// Barrier 0 belongs to __syncthreads(); roles use ids 1 and 2 so that one
// role can never release or block the other.
template <int ID, int COUNT>
__device__ __forceinline__ void role_sync() {
    static_assert(ID >= 1 && ID <= 15, "named barrier id out of range");
    static_assert(COUNT % 32 == 0 && COUNT > 0, "a role is a whole number of warps");
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory");
}

// ---- streaming global accesses -------------------------------------------------
// Inputs are read once and outputs written once, so loads bypass L1
// allocation and stores are marked evict-first.
__device__ __forceinline__ float4 ldg_stream4(const float* p) {
    float4 v;
    // not volatile: the data is read-only for the kernel, so the compiler may hoist and batch these loads
    asm("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void stg_stream4(float* p, float4 v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
// 256-bit stores (sm_100): half as many store instructions for the write-dominated kernels;
// measured 7 % faster than two 128-bit stores on the x2 upsample.  The address must be 32-byte aligned.
__device__ __forceinline__ void stg_stream8(float* p, const float* o) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(o[0]), "f"(o[1]), "f"(o[2]),
                 "f"(o[3]), "f"(o[4]), "f"(o[5]), "f"(o[6]), "f"(o[7])
                 : "memory");
}
__device__ __forceinline__ void stg_stream_4xi64(long long* p, long long a, long long b, long long c, long long d) {
    asm volatile("st.global.cs.v4.s64 [%0], {%1,%2,%3,%4};" ::"l"(p), "l"(a), "l"(b), "l"(c), "l"(d) : "memory");
}
__device__ __forceinline__ void stg_stream1(float* p, float v) {
    asm volatile("st.global.cs.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void stg_stream_2xi64(long long* p, long long a, long long b) {
    asm volatile("st.global.cs.v2.s64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

// ---- bulk (TMA) copies from shared to global memory ----------------------------------------
// Untiled form: both addresses 16-byte aligned, size a multiple of 16 bytes.  The shared-memory
// source is read by the async proxy, so the threads that filled it with ordinary stores run
// fence_proxy_async_shared() before the barrier that precedes the copy.  Groups are per thread:
// the thread that issued and committed the copies is the one that waits for them.
__device__ __forceinline__ void fence_proxy_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(__cvta_generic_to_global(gdst)),
                 "r"((uint32_t)__cvta_generic_to_shared(ssrc)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest N groups of this thread have finished READING their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// all but the newest N groups of this thread are complete (written)
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// ---- bulk (TMA) copies from global to shared memory, completion counted on an mbarrier -----------
// Untiled form again: both addresses 16-byte aligned, size a multiple of 16 bytes.  The thread that
// issues the copies first announces their bytes on the barrier (mbar_expect_tx, which is also its one
// arrival); the phase completes when all of them have landed, and the data is then visible to every
// thread that saw the phase flip (mbar_wait).  The wait is bounded in time: it gives up after
// `timeout_ns` and returns false, so a copy that never lands cannot hang the kernel.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
// makes freshly initialised barriers visible to the async proxy (the copies that will signal them)
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// before the barrier's shared memory is used for anything else
__device__ __forceinline__ void mbar_inval(unsigned long long* bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one arrival without bytes (a consumer saying that it has read a buffer)
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_load(void* sdst, const void* gsrc, uint32_t bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(sdst)),
                 "l"(__cvta_generic_to_global(gsrc)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity, unsigned long long timeout_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > timeout_ns) return false;
    }
}

// ---- division by a launch-time constant --------------------------------------------------
// q = n / d for n < 2^31 as one multiply-high, one add and one shift
// (m = floor(2^32 * (2^s - d) / d) + 1, s = ceil(log2 d); the sum cannot overflow for n < 2^31).
struct FastDiv {
    uint32_t d, m, s;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    f.s = s;
    f.m = (uint32_t)((((1ull << 32) * ((1ull << s) - d)) / d) + 1);
    return f;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) { return (__umulhi(n, f.m) + n) >> f.s; }
// n -> (n / d, n % d)
__device__ __forceinline__ uint32_t fast_divmod(uint32_t n, const FastDiv& f, uint32_t& rem) {
    const uint32_t q = fast_div(n, f);
    rem = n - q * f.d;
    return q;
}

// ---- role context ----------------------------------------------------------------
// What a role body sees instead of threadIdx / blockDim: its own thread id
// inside the range and the range size T (a compile-time constant).  blockIdx
// and gridDim are shared by both roles, exactly as in the reference's output
// (ThreadInfoRewriter rewrites threadIdx and blockDim only).
struct RoleCtx {
    int tid;        // 0 .. T-1 inside the role's thread range
    int block;      // blockIdx.x
    int nblocks;    // gridDim.x
    unsigned char* smem;   // this role's private slice of dynamic shared memory
};

}  // namespace hfuse
