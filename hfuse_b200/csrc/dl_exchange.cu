// Batch-norm statistics whose cross-GPU sum happens INSIDE the kernel, over peer memory:
// the warp that finishes a channel stores its moments into every rank's exchange buffer with
// plain NVLink stores whose 8-byte words carry their own validity tag, then collects every rank's
// row for that channel and folds them in rank order (dl_roles.cuh, BnXchg).  No collective library
// call, no second launch; the wait for the other ranks is bounded in time.  In the fused pair the
// statistics range sends, its first warp collects, and all its warps then draw upsample work from the
// cursor that the upsample range draws from too (fused_pool_kernel), so neither the wait nor the
// statistics threads' spare time costs anything; fused_share_kernel is the older form with a fixed share.
// The reference is single-GPU, so none of this has a counterpart there.
#include "dl_host.cuh"

struct hfuse_exchange {
    int world = 0, rank = 0, C = 0;
    size_t bytes = 0;
    unsigned char* local = nullptr;
    unsigned char* peer[hfuse::kXchgMaxRanks] = {};
    bool opened[hfuse::kXchgMaxRanks] = {};
    unsigned long long timeout_ns = 5ull * 1000 * 1000 * 1000;   // 5 s per exchange wait unless changed
    bool connected = false;
};

namespace {

// What a launch needs to know about the exchange.  Nothing here changes from call to call: the
// slot and epoch of a call are derived on the device from the counter in the buffer's header,
// which the kernel itself advances, so a launch that fails after this point (or is captured in a
// graph and replayed) cannot put this rank out of step with the others.
int describe_exchange(hfuse_exchange* ex, int C, BnXchg& x) {
    if (!ex || !ex->connected) return HFUSE_ERR_BAD_ARG;
    if (C != ex->C) return HFUSE_ERR_BAD_ARG;
    x.world = ex->world;
    x.rank = ex->rank;
    x.timeout_ns = ex->timeout_ns;
    for (int r = 0; r < hfuse::kXchgMaxRanks; ++r) x.peer[r] = ex->peer[r];
    return HFUSE_OK;
}

}  // namespace

extern "C" {

int hfuse_exchange_create(int world, int rank, int channels, hfuse_exchange** out) {
    if (!out || world < 1 || world > hfuse::kXchgMaxRanks || rank < 0 || rank >= world || channels < 1)
        return HFUSE_ERR_BAD_ARG;
    auto* ex = new hfuse_exchange();
    ex->world = world; ex->rank = rank; ex->C = channels;
    ex->bytes = sizeof(XchgLayout) + (size_t)hfuse::kXchgSlots * hfuse::kXchgMaxRanks * channels *
                                         hfuse::kXchgRowWords * sizeof(unsigned long long);
    if (cudaMalloc(&ex->local, ex->bytes) != cudaSuccess || cudaMemset(ex->local, 0, ex->bytes) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
        (void)cudaGetLastError();
        if (ex->local) cudaFree(ex->local);
        delete ex;
        return HFUSE_ERR_LAUNCH;
    }
    ex->peer[rank] = ex->local;
    ex->connected = (world == 1);
    *out = ex;
    return HFUSE_OK;
}

int hfuse_exchange_local_handle(hfuse_exchange* ex, uint8_t handle[HFUSE_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == HFUSE_IPC_HANDLE_BYTES, "handle size");
    if (!ex || !handle) return HFUSE_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, ex->local) != cudaSuccess) { (void)cudaGetLastError(); return HFUSE_ERR_LAUNCH; }
    memcpy(handle, &h, sizeof h);
    return HFUSE_OK;
}

int hfuse_exchange_connect(hfuse_exchange* ex, const uint8_t* handles) {
    if (!ex || (!handles && ex->world > 1)) return HFUSE_ERR_BAD_ARG;
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank || ex->opened[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * HFUSE_IPC_HANDLE_BYTES, sizeof h);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !p) {
            (void)cudaGetLastError();
            return HFUSE_ERR_LAUNCH;
        }
        ex->peer[r] = static_cast<unsigned char*>(p);
        ex->opened[r] = true;
    }
    ex->connected = true;
    return HFUSE_OK;
}

int hfuse_exchange_local_pointer(hfuse_exchange* ex, void** buffer) {
    if (!ex || !buffer) return HFUSE_ERR_BAD_ARG;
    *buffer = ex->local;
    return HFUSE_OK;
}

int hfuse_exchange_connect_pointers(hfuse_exchange* ex, void* const* buffers) {
    if (!ex || (!buffers && ex->world > 1)) return HFUSE_ERR_BAD_ARG;
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank) continue;
        if (!buffers[r] || ex->opened[r]) return HFUSE_ERR_BAD_ARG;      // not after an IPC connect
        ex->peer[r] = static_cast<unsigned char*>(buffers[r]);
    }
    ex->connected = true;
    return HFUSE_OK;
}

int hfuse_exchange_set_timeout(hfuse_exchange* ex, uint64_t nanoseconds) {
    if (!ex || nanoseconds == 0) return HFUSE_ERR_BAD_ARG;
    ex->timeout_ns = nanoseconds;
    return HFUSE_OK;
}

int hfuse_exchange_status(hfuse_exchange* ex, int* timed_out) {
    if (!ex || !timed_out) return HFUSE_ERR_BAD_ARG;
    unsigned st = 0;
    if (cudaMemcpy(&st, ex->local + offsetof(XchgLayout, status), sizeof st, cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return HFUSE_ERR_LAUNCH;
    }
    *timed_out = st != 0;
    return HFUSE_OK;
}

int hfuse_exchange_clear_status(hfuse_exchange* ex, hfuse_stream_t stream) {
    if (!ex) return HFUSE_ERR_BAD_ARG;
    if (cudaMemsetAsync(ex->local + offsetof(XchgLayout, status), 0, sizeof(unsigned), S_(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        return HFUSE_ERR_LAUNCH;
    }
    return HFUSE_OK;
}

int hfuse_exchange_destroy(hfuse_exchange* ex) {
    if (!ex) return HFUSE_OK;
    for (int r = 0; r < ex->world; ++r)
        if (ex->opened[r]) cudaIpcCloseMemHandle(ex->peer[r]);
    if (ex->local) cudaFree(ex->local);
    (void)cudaGetLastError();
    delete ex;
    return HFUSE_OK;
}

int hfuse_bnstats_allreduce_f32(HFUSE_BNSTATS_PARAMS(), hfuse_exchange* ex, hfuse_stream_t stream) {
    BnStatsArgs a;
    if (int rc = prep_bnstats(BNSTATS_NAMES(), a)) return rc;
    if (int rc = describe_exchange(ex, C, a.xchg)) return rc;
    return dispatch_solo<BnStatsXchgRole>("bnstats", kDefaultSolo_bnstats, a, S_(stream));
}

int hfuse_upsample_bnstats_allreduce_f32(HFUSE_UPSAMPLE_PARAMS(a_), HFUSE_BNSTATS_PARAMS(b_), hfuse_exchange* ex,
                                         hfuse_stream_t stream) {
    UpsampleArgs a;
    BnStatsArgs b;
    if (int rc = prep_upsample(UPSAMPLE_NAMES(a_), a)) return rc;
    if (int rc = prep_bnstats(BNSTATS_NAMES(b_), b)) return rc;
    if (int rc = describe_exchange(ex, b_C, b.xchg)) return rc;
    // Its own tuning entry.  By default the upsample's items are drawn from a cursor by the warps of
    // both thread ranges (the statistics range joins once it has sent its moments; its first warp
    // collects the peers' before it joins), so the statistics range can be large, send early, and
    // still leave nobody idle.  The older form (a fixed share of the upsample handed to the
    // statistics range, hfuse_tune_set_share) runs when a share has been set or the option
    // "exchange_pair_pool" is 0.
    const Tune t = tune_get("upsample_bnstats_allreduce");
    const int opt = option_get("exchange_pair_pool", -1);
    const bool pool = t.share_permille < 0 && (opt >= 0 ? opt == 1 : kDefaultPool_upsample_bnstats_allreduce == 1);
    if (pool)      // thread split measured at 1, 2, 4 and at 8 ranks (bench.py --tune-share)
        return dispatch_pair_pool<UpsampleRole, BnStatsXchgRole>(
            "upsample_bnstats_allreduce",
            ex->world > 4 ? kDefaultPoolPair_upsample_bnstats_allreduce_wide : kDefaultPoolPair_upsample_bnstats_allreduce, a,
            b, S_(stream));
    const bool wide = ex->world > 2;      // measured at 2 and at 8 ranks (bench.py --tune-share)
    return dispatch_pair_share<UpsampleRole, BnStatsXchgRole>(
        "upsample_bnstats_allreduce",
        wide ? kDefaultPair_upsample_bnstats_allreduce_wide : kDefaultPair_upsample_bnstats_allreduce,
        wide ? kDefaultShare_upsample_bnstats_allreduce_wide : kDefaultShare_upsample_bnstats_allreduce, a, b, S_(stream));
}

}  // extern "C"
