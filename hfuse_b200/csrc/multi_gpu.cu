// Multi-GPU entry points for hosts that are not Python: an NCCL communicator behind the C ABI,
// the two small reductions of the batch-sharded DL pairs (batch-norm moments, histogram counts),
// the DAG broadcast of the nonce-sharded ethash pairs, and sharded forms of the two benchmark
// searches.  One process (or host thread) per GPU; the reference is single-GPU, so none of this
// has a counterpart there.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2), so the library still loads, and every
// other entry point still works, on a host without NCCL.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "../../include/hfuse_b200.h"

#define S_(x) static_cast<cudaStream_t>(x)

struct hfuse_comm {
    ncclComm_t comm = nullptr;
    int world = 0, rank = 0;
};

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!a.handle) return a;
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
        a.Broadcast = reinterpret_cast<decltype(a.Broadcast)>(dlsym(a.handle, "ncclBroadcast"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.Broadcast;
        return a;
    }();
    return api;
}

inline int nccl_rc(ncclResult_t r) { return r == ncclSuccess ? HFUSE_OK : HFUSE_ERR_COMM; }

}  // namespace

extern "C" {

int hfuse_comm_unique_id(uint8_t id[HFUSE_COMM_ID_BYTES]) {
    static_assert(sizeof(ncclUniqueId) == HFUSE_COMM_ID_BYTES, "id size");
    if (!id) return HFUSE_ERR_BAD_ARG;
    if (!nccl().ok) return HFUSE_ERR_COMM;
    ncclUniqueId u;
    if (int rc = nccl_rc(nccl().GetUniqueId(&u))) return rc;
    memcpy(id, &u, sizeof u);
    return HFUSE_OK;
}

int hfuse_comm_create(int world, int rank, const uint8_t id[HFUSE_COMM_ID_BYTES], hfuse_comm** out) {
    if (!out || !id || world < 1 || rank < 0 || rank >= world) return HFUSE_ERR_BAD_ARG;
    if (!nccl().ok) return HFUSE_ERR_COMM;
    ncclUniqueId u;
    memcpy(&u, id, sizeof u);
    auto* c = new hfuse_comm();
    c->world = world;
    c->rank = rank;
    if (nccl().CommInitRank(&c->comm, world, u, rank) != ncclSuccess) {
        delete c;
        return HFUSE_ERR_COMM;
    }
    *out = c;
    return HFUSE_OK;
}

int hfuse_comm_destroy(hfuse_comm* c) {
    if (!c) return HFUSE_OK;
    int rc = HFUSE_OK;
    if (c->comm && nccl().ok) rc = nccl_rc(nccl().CommDestroy(c->comm));
    delete c;
    return rc;
}

int hfuse_bnstats_allreduce_nccl_f64(hfuse_comm* c, double* moments, int C, float eps, float* mean, float* invstd,
                                     hfuse_stream_t stream) {
    if (!c || !moments || !mean || !invstd || C <= 0) return HFUSE_ERR_BAD_ARG;
    if (int rc = nccl_rc(nccl().AllReduce(moments, moments, (size_t)3 * C, ncclFloat64, ncclSum, c->comm, S_(stream))))
        return rc;
    return hfuse_bnstats_finalize_f64(moments, C, eps, mean, invstd, stream);
}

int hfuse_histc_allreduce_counts(hfuse_comm* c, uint32_t* counts, int nbins, hfuse_stream_t stream) {
    if (!c || !counts || nbins <= 0) return HFUSE_ERR_BAD_ARG;
    return nccl_rc(nccl().AllReduce(counts, counts, (size_t)nbins, ncclUint32, ncclSum, c->comm, S_(stream)));
}

int hfuse_dag_broadcast(hfuse_comm* c, void* dag, size_t bytes, int root, hfuse_stream_t stream) {
    if (!c || !dag || root < 0 || root >= c->world) return HFUSE_ERR_BAD_ARG;
    if (bytes == 0) return HFUSE_OK;
    return nccl_rc(nccl().Broadcast(dag, dag, bytes, ncclUint8, root, c->comm, S_(stream)));
}

// Sharded searches: rank's contiguous share of [start, start + count) for BOTH halves (the
// benchmark gives both halves the same range).  Hits stay in the rank's own records; the host
// merges them (sort by nonce).
int hfuse_blake256_sha256d_search_sharded(HFUSE_BLAKE256_PARAMS(a_), HFUSE_SHA256D_PARAMS(b_), int rank, int world,
                                          hfuse_stream_t stream) {
    uint64_t oa = 0, na = 0, ob = 0, nb = 0;
    if (int rc = hfuse_shard_range(a_count, rank, world, &oa, &na)) return rc;
    if (int rc = hfuse_shard_range(b_count, rank, world, &ob, &nb)) return rc;
    return hfuse_blake256_sha256d_search(a_header80, a_start + oa, na, a_target32, a_hits, b_header80, b_start + ob, nb,
                                         b_target32, b_hits, stream);
}

int hfuse_sia_ethash_search_sharded(HFUSE_SIA_PARAMS(a_), HFUSE_ETHASH_PARAMS(b_), int rank, int world,
                                    hfuse_stream_t stream) {
    uint64_t oa = 0, na = 0, ob = 0, nb = 0;
    if (int rc = hfuse_shard_range(a_count, rank, world, &oa, &na)) return rc;
    if (int rc = hfuse_shard_range(b_count, rank, world, &ob, &nb)) return rc;
    return hfuse_sia_ethash_search(a_header80, a_start + oa, na, a_target32, a_hits, b_dag, b_dag_items, b_header_hash32,
                                   b_start + ob, nb, b_target32, b_hits, stream);
}

}  // extern "C"
