// Host-side launch plumbing shared by the DL and crypto entry points:
// per-device facts, occupancy cache, the per-pair tuning table and the
// variant dispatchers.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "../../include/hfuse_b200.h"
#include "fused.cuh"

namespace hfuse {

struct DeviceFacts {
    int sms = 0;
    int cc_major = 0;
};

inline int device_facts(DeviceFacts& out) {
    static std::mutex mu;
    static std::map<int, DeviceFacts> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return HFUSE_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(dev);
    if (it == cache.end()) {
        DeviceFacts f;
        if (cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&f.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
            return HFUSE_ERR_NO_DEVICE;
        if (f.cc_major != 10) return HFUSE_ERR_NO_DEVICE;   // sm_100a code only
        it = cache.emplace(dev, f).first;
    }
    out = it->second;
    return HFUSE_OK;
}

// more than 48 KB of dynamic shared memory has to be asked for once per kernel and device
inline void allow_dynamic_smem(const void* func, size_t smem) {
    if (smem <= 48 * 1024) return;
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, size_t> granted;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    size_t& g = granted[{dev, func}];
    if (g >= smem) return;
    if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) g = smem;
    else (void)cudaGetLastError();
}

// resident blocks per SM of (kernel, block size, dynamic smem) on the current device; the occupancy
// query only counts shared memory that the kernel has been allowed, so that comes first
inline int resident_blocks(const void* func, int block, size_t smem) {
    allow_dynamic_smem(func, smem);
    static std::mutex mu;
    static std::map<std::tuple<int, const void*, int, size_t>, int> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    auto key = std::make_tuple(dev, func, block, smem);
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, func, block, smem) != cudaSuccess || n < 1) n = 1;
    cache[key] = n;
    return n;
}

// ---- tuning table ------------------------------------------------------------------
struct Tune {
    int variant = -1;         // -1: the pair's compiled default
    int blocks_per_sm = 0;    // 0: as many as are resident
    int share_permille = -1;  // -1: the pair's compiled default (pairs launched through launch_pair_share)
};

inline std::map<std::string, Tune>& tune_table() {
    static std::map<std::string, Tune> t;
    return t;
}
inline std::mutex& tune_mutex() {
    static std::mutex m;
    return m;
}
inline Tune tune_get(const char* name) {
    std::lock_guard<std::mutex> lk(tune_mutex());
    auto it = tune_table().find(name);
    return it == tune_table().end() ? Tune{} : it->second;
}

// ---- options: named integer switches between alternative code paths -----------------------
// "im2col_store_path": -1 (unset) = the compiled choice of each kernel and pair, 0 = register tiles
// and streaming stores everywhere, 1 = shared-memory tile and bulk (TMA) stores wherever the shape
// allows it.
// "exchange_pair_pool": -1 (unset) = the compiled choice, 1 = the exchange pair draws the upsample's
// items from a cursor shared by both thread ranges (fused_pool_kernel), 0 = it hands a fixed share
// of them to the statistics range (fused_share_kernel, hfuse_tune_set_share).
// "bnstats_load_path": -1 (unset) = the compiled choice of each kernel and pair, 0 = 16-byte loads into
// registers everywhere, 1 = bulk (TMA) copies into shared memory wherever the shape allows it.
// "histc_load_path": the same choice for the histogram role (up to 256 bins): 0 = 16-byte loads into registers,
// 1 = bulk (TMA) copies into a ring of shared-memory buffers with "full" and "empty" mbarriers.
inline std::map<std::string, int>& option_table() {
    static std::map<std::string, int> t;
    return t;
}
inline int option_get(const char* name, int unset) {
    std::lock_guard<std::mutex> lk(tune_mutex());
    auto it = option_table().find(name);
    return it == option_table().end() ? unset : it->second;
}

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? HFUSE_OK : HFUSE_ERR_LAUNCH; }

// One kernel launch.  `dependent` marks the kernel as the programmatic dependent of the launch
// before it on the stream: it may start while that kernel is still running and meets it only at
// its own `griddepcontrol.wait` (used by the roles whose output buffer is cleared by a small
// kernel just ahead: the clearing then costs no gap on the stream).
template <class... KArgs, class... Args>
int launch_kernel(void (*kern)(KArgs...), int grid, int block, size_t smem, cudaStream_t s, bool dependent,
                  Args&&... args) {
    allow_dynamic_smem((const void*)kern, smem);
    if (!dependent) {
        kern<<<grid, block, smem, s>>>(args...);
        return check_launch();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...) != cudaSuccess) {
        (void)cudaGetLastError();
        return HFUSE_ERR_LAUNCH;
    }
    return check_launch();
}

// ---- one role over the whole block ----------------------------------------------------
template <class Role, int T, int MINB>
int launch_solo(typename Role::Args a, int blocks_per_sm, cudaStream_t s, bool dependent = false) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = solo_kernel<Role, T, MINB>;
    // shared memory of every role on this path does not depend on the grid
    if (int rc = Role::plan(a, T, f.sms * (blocks_per_sm > 0 ? blocks_per_sm : MINB))) return rc;
    const size_t smem = (size_t)Role::smem_bytes(a, T);
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, T, smem);
    const int grid = f.sms * bps;
    if (int rc = Role::plan(a, T, grid)) return rc;
    return launch_kernel(kern, grid, T, smem, s, dependent, a);
}

// ---- two roles side by side ------------------------------------------------------------
template <class RA, class RB, int TA, int TB, int MINB>
int launch_pair(typename RA::Args a, typename RB::Args b, int blocks_per_sm, cudaStream_t s, bool dependent = false) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = fused_kernel<RA, RB, TA, TB, MINB>;
    if (int rc = RA::plan(a, TA, f.sms * MINB)) return rc;
    if (int rc = RB::plan(b, TB, f.sms * MINB)) return rc;
    const int smem_a = (RA::smem_bytes(a, TA) + 15) & ~15;
    const size_t smem = (size_t)smem_a + (size_t)RB::smem_bytes(b, TB);
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, TA + TB, smem);
    const int grid = f.sms * bps;
    if (int rc = RA::plan(a, TA, grid)) return rc;
    if (int rc = RB::plan(b, TB, grid)) return rc;
    return launch_kernel(kern, grid, TA + TB, smem, s, dependent, a, b, smem_a);
}

// ---- two roles side by side, the second one taking over a share of the first one's items -----
// share_permille of role A's items (rounded down to whole rows) go to role B's thread range.
template <class RA, class RB, int TA, int TB, int MINB>
int launch_pair_share(typename RA::Args a, typename RB::Args b, int blocks_per_sm, int share_permille, cudaStream_t s,
                      bool dependent = false) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = fused_share_kernel<RA, RB, TA, TB, MINB>;
    if (int rc = RA::plan(a, TA, f.sms * MINB)) return rc;
    if (int rc = RB::plan(b, TB, f.sms * MINB)) return rc;
    const int smem_a = (RA::smem_bytes(a, TA) + 15) & ~15;
    const size_t smem = (size_t)smem_a + (size_t)RB::smem_bytes(b, TB);
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, TA + TB, smem);
    const int grid = f.sms * bps;
    if (int rc = RA::plan(a, TA, grid)) return rc;
    if (int rc = RB::plan(b, TB, grid)) return rc;
    unsigned items = 1, split = 1;          // scalar path: role A keeps everything
    if (RA::splittable(a)) {
        items = RA::vec_items(a);
        const unsigned row = RA::vec_row_items(a);
        const unsigned long long given = (unsigned long long)items * (unsigned)share_permille / 1000ull;
        split = items - (unsigned)(given / row * row);
    }
    return launch_kernel(kern, grid, TA + TB, smem, s, dependent, a, b, smem_a, split, items);
}

// ---- two roles side by side, role A's items drawn from a cursor by the warps of both ranges -----
template <class RA, class RB, int TA, int TB, int MINB>
int launch_pair_pool(typename RA::Args a, typename RB::Args b, int blocks_per_sm, cudaStream_t s, bool dependent = false) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = fused_pool_kernel<RA, RB, TA, TB, MINB>;
    if (int rc = RA::plan(a, TA, f.sms * MINB)) return rc;
    if (int rc = RB::plan(b, TB, f.sms * MINB)) return rc;
    const int smem_a = (RA::smem_bytes(a, TA) + 15) & ~15;
    const size_t smem = (size_t)smem_a + (size_t)RB::smem_bytes(b, TB);
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, TA + TB, smem);
    const int grid = f.sms * bps;
    if (int rc = RA::plan(a, TA, grid)) return rc;
    if (int rc = RB::plan(b, TB, grid)) return rc;
    return launch_kernel(kern, grid, TA + TB, smem, s, dependent, a, b, smem_a);
}

// ---- the same threads run both roles one after the other (vertical fusion) ------------------
template <class RA, class RB, int T, int MINB>
int launch_vpair(typename RA::Args a, typename RB::Args b, int blocks_per_sm, cudaStream_t s, bool dependent = false) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = vfused_kernel<RA, RB, T, MINB>;
    if (int rc = RA::plan(a, T, f.sms * MINB)) return rc;
    if (int rc = RB::plan(b, T, f.sms * MINB)) return rc;
    const int sa = RA::smem_bytes(a, T), sb = RB::smem_bytes(b, T);
    const size_t smem = (size_t)(sa > sb ? sa : sb);
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, T, smem);
    const int grid = f.sms * bps;
    if (int rc = RA::plan(a, T, grid)) return rc;
    if (int rc = RB::plan(b, T, grid)) return rc;
    return launch_kernel(kern, grid, T, smem, s, dependent, a, b);
}

// chunk of nonces a warp takes from a queue at a time: about 16 chunks per resident warp,
// a multiple of 32, at least 128, and large enough that the 32-bit cursor cannot wrap
inline unsigned queue_chunk(unsigned long long count, long long warps) {
    unsigned long long c = count / (unsigned long long)(warps * 16 > 0 ? warps * 16 : 1);
    if (c > 8192) c = 8192;
    if (c < 128) c = 128;
    const unsigned long long floor_c = (count >> 30) + 1;
    if (c < floor_c) c = floor_c;
    return (unsigned)((c + 31) / 32 * 32);
}

template <class R, int T, int MINB>
int launch_solo_queue(typename R::Args a, int blocks_per_sm, cudaStream_t s) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = solo_queue_kernel<R, T, MINB>;
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, T, 0);
    const int grid = f.sms * bps;
    kern<<<grid, T, 0, s>>>(a, queue_chunk(a.c.count, (long long)grid * (T / 32)));
    return check_launch();
}

template <class RA, class RB, int TA, int TB, int MINB>
int launch_pair_queue(typename RA::Args a, typename RB::Args b, int blocks_per_sm, cudaStream_t s) {
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    auto kern = fused_queue_kernel<RA, RB, TA, TB, MINB>;
    const int bps = blocks_per_sm > 0 ? blocks_per_sm : resident_blocks((const void*)kern, TA + TB, 0);
    const int grid = f.sms * bps;
    const long long warps = (long long)grid * ((TA + TB) / 32);
    kern<<<grid, TA + TB, 0, s>>>(a, b, queue_chunk(a.c.count, warps), queue_chunk(b.c.count, warps));
    return check_launch();
}

}  // namespace hfuse
