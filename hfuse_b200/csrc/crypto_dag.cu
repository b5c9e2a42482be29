// ethash DAG generation: the step before the search (the reference's fuser binary runs 16
// launches of ethash_calculate_dag_item before any search, scripts/data/miner.json:10052).
// The light cache is sequential by construction and is built on the host; the DAG nodes are
// independent and are built on the GPU, four lanes per 64-byte node so that every one of
// the 256 parent reads is one coalesced 64-byte access.
#include "crypto_host.cuh"

namespace {

// ---- host Keccak-512 (cache generation only) ------------------------------------------------
void keccak_f_host(uint64_t a[25]) {
    static const uint64_t RC[24] = HFUSE_KECCAKRC_INIT;
    static const int ROT[25] = {0, 1, 62, 28, 27, 36, 44, 6, 55, 20, 3, 10, 43, 25, 39, 41, 45, 15, 21, 8, 18, 2, 61, 56, 14};
    for (int r = 0; r < 24; ++r) {
        uint64_t c[5], b[25];
        for (int x = 0; x < 5; ++x) c[x] = a[x] ^ a[x + 5] ^ a[x + 10] ^ a[x + 15] ^ a[x + 20];
        for (int x = 0; x < 5; ++x) {
            const uint64_t d = c[(x + 4) % 5] ^ ((c[(x + 1) % 5] << 1) | (c[(x + 1) % 5] >> 63));
            for (int y = 0; y < 25; y += 5) a[y + x] ^= d;
        }
        for (int x = 0; x < 5; ++x)
            for (int y = 0; y < 5; ++y) {
                const int src = x + 5 * y, dst = y + 5 * ((2 * x + 3 * y) % 5), rot = ROT[src];
                b[dst] = rot ? ((a[src] << rot) | (a[src] >> (64 - rot))) : a[src];
            }
        for (int y = 0; y < 25; y += 5)
            for (int x = 0; x < 5; ++x) a[y + x] = b[y + x] ^ (~b[y + (x + 1) % 5] & b[y + (x + 2) % 5]);
        a[0] ^= RC[r];
    }
}
// Keccak-512 (rate 72, original padding) of `len` bytes, len = 32 or 64
void keccak512_host(const uint8_t* in, int len, uint8_t out[64]) {
    uint64_t a[25] = {};
    for (int i = 0; i < len / 8; ++i) a[i] = le64(in + 8 * i);
    a[len / 8] ^= 0x01ull;                       // first padding byte right after the message
    a[8] ^= 0x8000000000000000ull;               // last bit of the 72-byte block
    keccak_f_host(a);
    for (int i = 0; i < 8; ++i)
        for (int k = 0; k < 8; ++k) out[8 * i + k] = (uint8_t)(a[i] >> (8 * k));
}

// ---- device: Keccak-512 of a 64-byte block held as 16 words ---------------------------------
__device__ __forceinline__ void keccak512_words(uint32_t w[16]) {
    unsigned long long st[25];
#pragma unroll
    for (int i = 0; i < 8; ++i) st[i] = ((unsigned long long)w[2 * i + 1] << 32) | w[2 * i];
    st[8] = 0x8000000000000001ull;
#pragma unroll
    for (int i = 9; i < 25; ++i) st[i] = 0;
    keccak_f1600(st);
#pragma unroll
    for (int i = 0; i < 8; ++i) { w[2 * i] = (uint32_t)st[i]; w[2 * i + 1] = (uint32_t)(st[i] >> 32); }
}

// One thread owns one node; groups of four lanes walk the parents of each other's nodes.
__global__ void __launch_bounds__(128) dag_nodes_kernel(const uint4* __restrict__ cache, uint32_t cache_nodes,
                                                        unsigned long long magic, uint4* __restrict__ dag,
                                                        uint32_t first, uint32_t count) {
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    const int g = threadIdx.x & 3;
    const bool live = gid < count;
    const uint32_t node = first + (live ? gid : 0);
    uint32_t mix[16];
    {
        const uint4* src = cache + (size_t)fastmod(node, magic, cache_nodes) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = __ldg(src + q);
            mix[4 * q] = v.x; mix[4 * q + 1] = v.y; mix[4 * q + 2] = v.z; mix[4 * q + 3] = v.w;
        }
    }
    mix[0] ^= node;
    keccak512_words(mix);
#pragma unroll 1
    for (int t = 0; t < 4; ++t) {
        // lane g takes words 4g..4g+3 of lane t's mix
        uint32_t sh[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) sh[k] = __shfl_sync(0xffffffffu, mix[k], t, 4);
        const uint32_t tnode = __shfl_sync(0xffffffffu, node, t, 4);
        uint4 q = g == 0 ? make_uint4(sh[0], sh[1], sh[2], sh[3]) : g == 1 ? make_uint4(sh[4], sh[5], sh[6], sh[7])
                : g == 2 ? make_uint4(sh[8], sh[9], sh[10], sh[11]) : make_uint4(sh[12], sh[13], sh[14], sh[15]);
#pragma unroll 4
        for (uint32_t j = 0; j < 256; ++j) {
            // word j % 16 of the mix lives in lane (j % 16) / 4, component j % 4
            const uint32_t word = (j & 3) == 0 ? q.x : (j & 3) == 1 ? q.y : (j & 3) == 2 ? q.z : q.w;
            uint32_t parent = fastmod(fnv1(tnode ^ j, word), magic, cache_nodes);
            parent = __shfl_sync(0xffffffffu, parent, (j & 15) >> 2, 4);
            const uint4 c = __ldg(cache + (size_t)parent * 4 + g);
            q.x = fnv1(q.x, c.x); q.y = fnv1(q.y, c.y); q.z = fnv1(q.z, c.z); q.w = fnv1(q.w, c.w);
        }
        // hand the four quarters back to lane t
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t x = __shfl_sync(0xffffffffu, q.x, s, 4), y = __shfl_sync(0xffffffffu, q.y, s, 4);
            const uint32_t z = __shfl_sync(0xffffffffu, q.z, s, 4), w = __shfl_sync(0xffffffffu, q.w, s, 4);
            if (g == t) { mix[4 * s] = x; mix[4 * s + 1] = y; mix[4 * s + 2] = z; mix[4 * s + 3] = w; }
        }
    }
    keccak512_words(mix);
    if (live) {
        uint4* dst = dag + (size_t)(first + gid) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(mix[4 * q], mix[4 * q + 1], mix[4 * q + 2], mix[4 * q + 3]);
    }
}

}  // namespace

extern "C" {

int hfuse_ethash_make_cache(const uint8_t seed32[32], uint32_t cache_nodes, void* host_cache) {
    if (!seed32 || !host_cache || cache_nodes == 0) return HFUSE_ERR_BAD_ARG;
    uint8_t* c = static_cast<uint8_t*>(host_cache);
    keccak512_host(seed32, 32, c);
    for (uint32_t i = 1; i < cache_nodes; ++i) keccak512_host(c + 64 * (size_t)(i - 1), 64, c + 64 * (size_t)i);
    for (int round = 0; round < 3; ++round)
        for (uint32_t i = 0; i < cache_nodes; ++i) {
            const uint8_t* self = c + 64 * (size_t)i;
            const uint32_t v = ((uint32_t)self[0] | ((uint32_t)self[1] << 8) | ((uint32_t)self[2] << 16) |
                                ((uint32_t)self[3] << 24)) % cache_nodes;
            const uint8_t* a = c + 64 * (size_t)((i + cache_nodes - 1) % cache_nodes);
            const uint8_t* b = c + 64 * (size_t)v;
            uint8_t x[64];
            for (int k = 0; k < 64; ++k) x[k] = a[k] ^ b[k];
            keccak512_host(x, 64, c + 64 * (size_t)i);
        }
    return HFUSE_OK;
}

int hfuse_ethash_generate_dag(const void* cache, uint32_t cache_nodes, void* dag, uint32_t first_node,
                              uint32_t node_count, hfuse_stream_t stream) {
    if (!cache || !dag || cache_nodes == 0) return HFUSE_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(dag)) & 15u) return HFUSE_ERR_ALIGNMENT;
    if ((unsigned long long)first_node + node_count > (1ull << 32)) return HFUSE_ERR_TOO_LARGE;
    if (node_count == 0) return HFUSE_OK;
    DeviceFacts f;
    if (int rc = device_facts(f)) return rc;
    const unsigned blocks = (node_count + 127) / 128;
    dag_nodes_kernel<<<blocks, 128, 0, S_(stream)>>>(static_cast<const uint4*>(cache), cache_nodes,
                                                     ~0ull / cache_nodes + 1, static_cast<uint4*>(dag), first_node,
                                                     node_count);
    return check_launch();
}

}  // extern "C"
