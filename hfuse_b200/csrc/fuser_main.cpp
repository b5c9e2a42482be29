// C++ host program over the C ABI, in the role of the reference's `build/fuse/fuser` binary
// (README.md:101 of aoli-al/HFuse): build a DAG, then run each nonce-search kernel and each
// fused pair over one block of nonces and print what was found and how long it took.
//
//   fuser [--nonces N] [--dag-nodes M] [--cache-nodes K] [--bits B]
//
// Output: one JSON object per line (kernel or pair name, milliseconds, hit counts, nonces).
// Only the C ABI (include/hfuse_b200.h) and the CUDA runtime are used: no PyTorch, no Python.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/hfuse_b200.h"

#define CK(x)                                                                      \
    do {                                                                           \
        cudaError_t e_ = (x);                                                      \
        if (e_ != cudaSuccess) {                                                   \
            fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));               \
            return 2;                                                              \
        }                                                                          \
    } while (0)
#define HK(x)                                                                      \
    do {                                                                           \
        int r_ = (x);                                                              \
        if (r_ != HFUSE_OK) {                                                      \
            fprintf(stderr, "%s: %s (%d)\n", #x, hfuse_error_string(r_), r_);      \
            return 3;                                                              \
        }                                                                          \
    } while (0)

static std::string hits_json(const hfuse_hits& h) {
    std::vector<uint64_t> n(h.nonce, h.nonce + std::min<uint32_t>(h.count, HFUSE_MAX_HITS));
    std::sort(n.begin(), n.end());
    std::string s = "{\"count\": " + std::to_string(h.count) + ", \"nonces\": [";
    for (size_t i = 0; i < n.size(); ++i) s += (i ? ", " : "") + std::to_string(n[i]);
    return s + "]}";
}

int main(int argc, char** argv) {
    uint64_t nonces = 1ull << 22;
    uint32_t dag_nodes = 1u << 20, cache_nodes = 16381;
    int bits = 16;
    for (int i = 1; i + 1 < argc; i += 2) {
        if (!strcmp(argv[i], "--nonces")) nonces = strtoull(argv[i + 1], nullptr, 10);
        else if (!strcmp(argv[i], "--dag-nodes")) dag_nodes = (uint32_t)strtoul(argv[i + 1], nullptr, 10);
        else if (!strcmp(argv[i], "--cache-nodes")) cache_nodes = (uint32_t)strtoul(argv[i + 1], nullptr, 10);
        else if (!strcmp(argv[i], "--bits")) bits = atoi(argv[i + 1]);
    }
    dag_nodes &= ~1u;                                   // a 128-byte DAG item is two nodes
    uint8_t seed[32], header_hash[32], hdr_a[80], hdr_b[80], target[32] = {};
    uint8_t stream_bytes[32 + 32 + 160];
    hfuse_xoshiro256ss_fill(2024, stream_bytes, sizeof stream_bytes);
    memcpy(seed, stream_bytes, 32); memcpy(header_hash, stream_bytes + 32, 32);
    memcpy(hdr_a, stream_bytes + 64, 80); memcpy(hdr_b, stream_bytes + 144, 80);
    if (bits < 1 || bits > 255) bits = 16;
    // target = 2^(256-bits), big-endian: counting bits from the top, that is bit number bits-1
    target[(bits - 1) / 8] = (uint8_t)(0x80u >> ((bits - 1) % 8));

    // ---- DAG: light cache on the host, nodes on the GPU in 16 launches like the reference
    std::vector<uint8_t> cache((size_t)cache_nodes * 64);
    HK(hfuse_ethash_make_cache(seed, cache_nodes, cache.data()));
    void *d_cache, *d_dag;
    CK(cudaMalloc(&d_cache, cache.size()));
    CK(cudaMalloc(&d_dag, (size_t)dag_nodes * 64));
    CK(cudaMemcpy(d_cache, cache.data(), cache.size(), cudaMemcpyHostToDevice));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    CK(cudaEventRecord(e0));
    const uint32_t per = (dag_nodes + 15) / 16;
    for (uint32_t first = 0; first < dag_nodes; first += per)
        HK(hfuse_ethash_generate_dag(d_cache, cache_nodes, d_dag, first, std::min(per, dag_nodes - first), nullptr));
    CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1));
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    printf("{\"step\": \"ethash_calculate_dag_item\", \"nodes\": %u, \"ms\": %.3f}\n", dag_nodes, ms);

    hfuse_hits *d_ha, *d_hb, h_a, h_b;
    CK(cudaMalloc(&d_ha, sizeof(hfuse_hits))); CK(cudaMalloc(&d_hb, sizeof(hfuse_hits)));
    const uint32_t items = dag_nodes / 2;
    auto reset = [&]() { return hfuse_hits_reset(d_ha, nullptr) | hfuse_hits_reset(d_hb, nullptr); };
    auto report = [&](const char* name, bool two) -> int {
        CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1));
        CK(cudaEventElapsedTime(&ms, e0, e1));
        CK(cudaMemcpy(&h_a, d_ha, sizeof h_a, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(&h_b, d_hb, sizeof h_b, cudaMemcpyDeviceToHost));
        printf("{\"kernel\": \"%s\", \"nonces\": %llu, \"ms\": %.3f, \"first\": %s", name, (unsigned long long)nonces, ms,
               hits_json(h_a).c_str());
        if (two) printf(", \"second\": %s", hits_json(h_b).c_str());
        printf("}\n");
        return 0;
    };
#define RUN(NAME, TWO, CALL)                       \
    HK(reset());                                   \
    CK(cudaEventRecord(e0));                       \
    HK(CALL);                                      \
    if (int rc = report(NAME, TWO)) return rc;

    RUN("ethash_search", false, hfuse_ethash_search(d_dag, items, header_hash, 0, nonces, target, d_ha, nullptr))
    RUN("blake256", false, hfuse_blake256_search(hdr_a, 0, nonces, target, d_ha, nullptr))
    RUN("sha256d", false, hfuse_sha256d_search(hdr_b, 0, nonces, target, d_ha, nullptr))
    RUN("sia_blake2b", false, hfuse_sia_blake2b_search(hdr_b, 0, nonces, target, d_ha, nullptr))
    RUN("ethash_blake256", true, hfuse_ethash_blake256_search(d_dag, items, header_hash, 0, nonces, target, d_ha, hdr_a, 0, nonces, target, d_hb, nullptr))
    RUN("sha256d_ethash", true, hfuse_sha256d_ethash_search(hdr_b, 0, nonces, target, d_ha, d_dag, items, header_hash, 0, nonces, target, d_hb, nullptr))
    RUN("sia_ethash", true, hfuse_sia_ethash_search(hdr_b, 0, nonces, target, d_ha, d_dag, items, header_hash, 0, nonces, target, d_hb, nullptr))
    RUN("blake256_sha256d", true, hfuse_blake256_sha256d_search(hdr_a, 0, nonces, target, d_ha, hdr_b, 0, nonces, target, d_hb, nullptr))
    RUN("blake256_sia", true, hfuse_blake256_sia_search(hdr_a, 0, nonces, target, d_ha, hdr_b, 0, nonces, target, d_hb, nullptr))
    RUN("sha256d_sia", true, hfuse_sha256d_sia_search(hdr_b, 0, nonces, target, d_ha, hdr_b, 0, nonces, target, d_hb, nullptr))
    cudaFree(d_ha); cudaFree(d_hb); cudaFree(d_dag); cudaFree(d_cache);
    return 0;
}
