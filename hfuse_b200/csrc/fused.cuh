// Kernel shells: one role over a whole block (the unfused baseline) and two
// roles side by side in one block (the horizontally fused pair).
//
// The fused shell is the hand-written form of what the reference prints for
// its `hfuse` presets: `__launch_bounds__(T1+T2, minBlocks)`
// (lib/KernelFuser/KernelPrinter.cpp:44-65), parameter lists concatenated
// (KernelPrinter.cpp:107-114), body 1 guarded by `tid < T1` and body 2 by
// `T1 <= tid < T1+T2` (lib/KernelFuser/KernelFusion.cpp:5-10,
// lib/KernelFuser/KernelFuseTool.cpp:56-62).  The split T1:T2 is a template
// parameter so that the sweep of tools/llvm-smart-fuser/main.cpp:215-227
// (128-thread steps) becomes a list of instantiations.
#pragma once
#include "common.cuh"

namespace hfuse {

template <class Role, int T, int MINB>
__global__ void __launch_bounds__(T, MINB) solo_kernel(const __grid_constant__ typename Role::Args a) {
    extern __shared__ __align__(16) unsigned char smem[];
    RoleCtx ctx{(int)threadIdx.x, (int)blockIdx.x, (int)gridDim.x, smem};
    Role::template run<T, 1>(a, ctx);
}

// One work-queue role over the whole block (the nonce searches): every warp draws chunks of nonces
// from the role's cursor until the range is used up, instead of walking a fixed grid-stride share.
template <class Role, int T, int MINB>
__global__ void __launch_bounds__(T, MINB) solo_queue_kernel(const __grid_constant__ typename Role::Args a, unsigned chunk) {
    Role::drain(a, chunk);
}

template <class RoleA, class RoleB, int TA, int TB, int MINB>
__global__ void __launch_bounds__(TA + TB, MINB)
fused_kernel(const __grid_constant__ typename RoleA::Args a, const __grid_constant__ typename RoleB::Args b,
             int smem_off_b) {
    static_assert(TA % 32 == 0 && TB % 32 == 0, "ranges are whole warps, so the guard never splits a warp");
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = (int)threadIdx.x;
    if (tid < TA) {
        RoleCtx ctx{tid, (int)blockIdx.x, (int)gridDim.x, smem};
        RoleA::template run<TA, 1>(a, ctx);
    } else {
        RoleCtx ctx{tid - TA, (int)blockIdx.x, (int)gridDim.x, smem + smem_off_b};
        RoleB::template run<TB, 2>(b, ctx);
    }
}

// Fused pair whose second role has a wait in the middle (the cross-GPU exchange of the
// batch-norm moments): role B's range runs the first half of its own work (compute and send),
// then takes over items [split, items) of role A's work, and only then runs its second half
// (collect), so the wait for the peers is covered by useful work instead of ending the kernel.
// Role A's range works on items [0, split).
template <class RoleA, class RoleB, int TA, int TB, int MINB>
__global__ void __launch_bounds__(TA + TB, MINB)
fused_share_kernel(const __grid_constant__ typename RoleA::Args a, const __grid_constant__ typename RoleB::Args b,
                   int smem_off_b, unsigned split, unsigned items) {
    static_assert(TA % 32 == 0 && TB % 32 == 0, "ranges are whole warps, so the guard never splits a warp");
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = (int)threadIdx.x;
    if (tid < TA) {
        RoleCtx ctx{tid, (int)blockIdx.x, (int)gridDim.x, smem};
        RoleA::template run_range<TA>(a, ctx, 0u, split);
    } else {
        RoleCtx ctx{tid - TA, (int)blockIdx.x, (int)gridDim.x, smem + smem_off_b};
        const auto token = RoleB::template run_early<TB, 2>(b, ctx);
        RoleA::template run_range<TB>(a, ctx, split, items);
        RoleB::template run_late<TB, 2>(b, ctx, token);
    }
}

// The same pair with the split of role A's items decided while the kernel runs: every warp of
// the block, whichever range it belongs to, draws 32-item chunks of role A's work from one cursor
// in shared memory.  Role A's range draws from the start; role B's range runs the first half of
// its own work (compute and send) and then joins the draw, except for its first warp, which
// first runs the second half (collect) and joins when the peers' answers are in.  Role B's range
// can therefore be given many threads (it sends early) without leaving those threads idle
// afterwards, and the wait for the peers is off the kernel's critical path, whatever the number of
// ranks.  A role A whose shape has no chunked path keeps
// all of its work in its own range.
template <class RoleA, class RoleB, int TA, int TB, int MINB>
__global__ void __launch_bounds__(TA + TB, MINB)
fused_pool_kernel(const __grid_constant__ typename RoleA::Args a, const __grid_constant__ typename RoleB::Args b,
                  int smem_off_b) {
    static_assert(TA % 32 == 0 && TB % 32 == 0, "ranges are whole warps, so the guard never splits a warp");
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned pool_cursor;
    const int tid = (int)threadIdx.x;
    if (tid == 0) pool_cursor = 0u;
    __syncthreads();          // the only use of barrier 0: before either role has started
    const bool pooled = RoleA::splittable(a);
    if (tid < TA) {
        RoleCtx ctx{tid, (int)blockIdx.x, (int)gridDim.x, smem};
        if (pooled) RoleA::run_pool(a, ctx.block, ctx.nblocks, &pool_cursor, (unsigned)tid & 31u);
        else RoleA::template run<TA, 1>(a, ctx);
    } else {
        RoleCtx ctx{tid - TA, (int)blockIdx.x, (int)gridDim.x, smem + smem_off_b};
        const auto token = RoleB::template run_early<TB, 2>(b, ctx);
        // The second half is the business of the range's first warp only: it waits for the peers
        // while the range's other warps are already drawing chunks, and joins them afterwards, so
        // the wait is neither at the end of the kernel nor in anybody's way.
        RoleB::template run_late<TB, 2>(b, ctx, token);
        if (pooled) RoleA::run_pool(a, ctx.block, ctx.nblocks, &pool_cursor, (unsigned)tid & 31u);
    }
}

// Vertical fusion, the reference's `vfuse` presets (tools/llvm-smart-fuser/main.cpp:182-193,
// include/KernelFusion.h:75-78): every thread range starts at 0, i.e. the SAME threads run
// body 1 and then body 2, block = max(T1, T2).  Kept as the third column of the comparison
// (standalone back to back, vertical, horizontal), like the reference's own analysis.
template <class RoleA, class RoleB, int T, int MINB>
__global__ void __launch_bounds__(T, MINB)
vfused_kernel(const __grid_constant__ typename RoleA::Args a, const __grid_constant__ typename RoleB::Args b) {
    extern __shared__ __align__(16) unsigned char smem[];
    RoleCtx ctx{(int)threadIdx.x, (int)blockIdx.x, (int)gridDim.x, smem};
    RoleA::template run<T, 1>(a, ctx);
    // body 2 reuses the shared memory: everyone must be done with body 1's first
    role_sync<2, T>();
    RoleB::template run<T, 1>(b, ctx);
}

// Fused pair of two work-queue roles (the nonce searches).  The block is still split into
// role A's and role B's thread ranges; each range drains its own queue first and then helps
// with the other one, so no range idles while the other still has nonces left.
template <class RoleA, class RoleB, int TA, int TB, int MINB>
__global__ void __launch_bounds__(TA + TB, MINB)
fused_queue_kernel(const __grid_constant__ typename RoleA::Args a, const __grid_constant__ typename RoleB::Args b,
                   unsigned chunk_a, unsigned chunk_b) {
    static_assert(TA % 32 == 0 && TB % 32 == 0, "ranges are whole warps, so the guard never splits a warp");
    int which = ((int)threadIdx.x < TA) ? 0 : 1;
#pragma unroll 1
    for (int phase = 0; phase < 2; ++phase, which ^= 1) {
        if (which == 0) RoleA::drain(a, chunk_a);
        else RoleB::drain(b, chunk_b);
    }
}

}  // namespace hfuse
