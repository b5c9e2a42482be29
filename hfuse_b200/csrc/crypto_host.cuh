// Host side shared by the crypto entry points: first-block midstates, argument
// checks and variant dispatch.  Included by crypto_api.cu (standalone searches)
// and by one small translation unit per fused pair, so that the pairs compile
// in parallel.
#pragma once
#include "crypto_roles.cuh"
#include "launch.cuh"

using namespace hfuse;

#define SEARCH_NAMES(P) P##header80, P##start, P##count, P##target32, P##hits
#define ETHASH_NAMES(P) P##dag, P##dag_items, P##header_hash32, P##start, P##count, P##target32, P##hits

namespace {

using Sha = SearchRole<Sha256dRole>;
using Blake = SearchRole<Blake256Role>;
using Sia = SearchRole<SiaRole>;
using Eth = SearchRole<EthashRole>;

inline uint32_t be32(const uint8_t* p) {
    return ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | p[3];
}
inline uint64_t le64(const uint8_t* p) {
    uint64_t v = 0;
    for (int i = 7; i >= 0; --i) v = (v << 8) | p[i];
    return v;
}
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

// ---- host midstates: one compression of the first 64 header bytes ---------------------
void sha256_first_block(const uint8_t* blk, uint32_t h[8]) {
    static const uint32_t iv[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                   0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = be32(blk + 4 * i);
    for (int i = 16; i < 64; ++i)
        w[i] = w[i - 16] + (rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3)) + w[i - 7] +
               (rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10));
    uint32_t s[8];
    for (int i = 0; i < 8; ++i) s[i] = iv[i];
    for (int i = 0; i < 64; ++i) {
        const uint32_t t1 = s[7] + (rotr(s[4], 6) ^ rotr(s[4], 11) ^ rotr(s[4], 25)) + ((s[4] & s[5]) ^ (~s[4] & s[6])) +
                            kShaKLit[i] + w[i];
        const uint32_t t2 = (rotr(s[0], 2) ^ rotr(s[0], 13) ^ rotr(s[0], 22)) +
                            ((s[0] & s[1]) ^ (s[0] & s[2]) ^ (s[1] & s[2]));
        s[7] = s[6]; s[6] = s[5]; s[5] = s[4]; s[4] = s[3] + t1; s[3] = s[2]; s[2] = s[1]; s[1] = s[0]; s[0] = t1 + t2;
    }
    for (int i = 0; i < 8; ++i) h[i] = iv[i] + s[i];
}

void blake256_first_block(const uint8_t* blk, uint32_t h[8]) {
    static const uint32_t iv[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                   0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    uint32_t m[16], v[16];
    for (int i = 0; i < 16; ++i) m[i] = be32(blk + 4 * i);
    for (int i = 0; i < 8; ++i) v[i] = iv[i];
    for (int i = 0; i < 4; ++i) v[8 + i] = kBlakeC[i];
    v[12] = 512u ^ kBlakeC[4]; v[13] = 512u ^ kBlakeC[5]; v[14] = kBlakeC[6]; v[15] = kBlakeC[7];
    static const int q[8][4] = {{0, 4, 8, 12}, {1, 5, 9, 13}, {2, 6, 10, 14}, {3, 7, 11, 15},
                                {0, 5, 10, 15}, {1, 6, 11, 12}, {2, 7, 8, 13}, {3, 4, 9, 14}};
    for (int r = 0; r < 14; ++r)
        for (int i = 0; i < 8; ++i) {
            const int a = q[i][0], b = q[i][1], c = q[i][2], d = q[i][3];
            const int j = kSigma[r % 10][2 * i], k = kSigma[r % 10][2 * i + 1];
            v[a] += v[b] + (m[j] ^ kBlakeC[k]); v[d] = rotr(v[d] ^ v[a], 16);
            v[c] += v[d]; v[b] = rotr(v[b] ^ v[c], 12);
            v[a] += v[b] + (m[k] ^ kBlakeC[j]); v[d] = rotr(v[d] ^ v[a], 8);
            v[c] += v[d]; v[b] = rotr(v[b] ^ v[c], 7);
        }
    for (int i = 0; i < 8; ++i) h[i] = iv[i] ^ v[i] ^ v[i + 8];
}

// ---- argument checking ---------------------------------------------------------------------
int prep_common(uint64_t start, uint64_t count, const uint8_t* target32, hfuse_hits* hits, bool nonce32,
                SearchCommon& c) {
    if (!target32 || !hits) return HFUSE_ERR_BAD_ARG;
    if (nonce32 && count > (1ull << 32)) return HFUSE_ERR_TOO_LARGE;   // the nonce space itself
    if (count > (1ull << 61)) return HFUSE_ERR_TOO_LARGE;                // a work-queue chunk must fit 32 bits
    c.start = start; c.count = count; c.hits = hits; c.out32 = nullptr; c.mix32 = nullptr; c.one = 1u;
    for (int i = 0; i < 8; ++i) c.target[i] = be32(target32 + 4 * i);
    return HFUSE_OK;
}

int fill_sha(const uint8_t* header80, Sha256dArgs& a) {
    if (!header80) return HFUSE_ERR_BAD_ARG;
    sha256_first_block(header80, a.mid);
    a.w0 = be32(header80 + 64); a.w1 = be32(header80 + 68); a.w2 = be32(header80 + 72);
    return HFUSE_OK;
}
int fill_blake(const uint8_t* header80, Blake256Args& a) {
    if (!header80) return HFUSE_ERR_BAD_ARG;
    blake256_first_block(header80, a.mid);
    a.m0 = be32(header80 + 64); a.m1 = be32(header80 + 68); a.m2 = be32(header80 + 72);
    return HFUSE_OK;
}
int fill_sia(const uint8_t* header80, SiaArgs& a) {
    if (!header80) return HFUSE_ERR_BAD_ARG;
    for (int i = 0; i < 10; ++i) a.m[i] = le64(header80 + 8 * i);
    return HFUSE_OK;
}
int fill_eth(const void* dag, uint32_t dag_items, const uint8_t* header_hash32, EthashArgs& a) {
    if (!dag || !header_hash32 || dag_items == 0) return HFUSE_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(dag) & 15u) return HFUSE_ERR_ALIGNMENT;
    a.dag = static_cast<const uint4*>(dag);
    a.dag_items = dag_items;
    a.pow2_mask = (dag_items > 1 && (dag_items & (dag_items - 1)) == 0) ? dag_items - 1 : 0;
    a.mod_magic = ~0ull / dag_items + 1;
    for (int i = 0; i < 4; ++i) a.header[i] = le64(header_hash32 + 8 * i);
    return HFUSE_OK;
}

int prep_sha(HFUSE_SHA256D_PARAMS(), Sha256dArgs& a) {
    if (int rc = fill_sha(header80, a)) return rc;
    return prep_common(start, count, target32, hits, true, a.c);
}
int prep_blake(HFUSE_BLAKE256_PARAMS(), Blake256Args& a) {
    if (int rc = fill_blake(header80, a)) return rc;
    return prep_common(start, count, target32, hits, true, a.c);
}
int prep_sia(HFUSE_SIA_PARAMS(), SiaArgs& a) {
    if (int rc = fill_sia(header80, a)) return rc;
    return prep_common(start, count, target32, hits, false, a.c);
}
int prep_eth(HFUSE_ETHASH_PARAMS(), EthashArgs& a) {
    if (int rc = fill_eth(dag, dag_items, header_hash32, a)) return rc;
    return prep_common(start, count, target32, hits, false, a.c);
}

// ---- variants: (index, T1, T2, minBlocks/SM).  The reference has a single 128:128 split for
// the crypto pairs (all four kernels use 128-thread blocks, configs/crypto_kernels.yaml);
// unequal splits, down to one warp in eight, are added because the halves are far from equally
// expensive: next to ethash, an ALU-bound hash is best given a small range that fills the ALU gaps
// while ethash keeps nearly all of its loads in flight.
#define CRYPTO_PAIR_VARIANTS(X)                                                                       \
    X(0, 128, 128, 2) X(1, 128, 128, 3) X(2, 128, 128, 4) X(3, 256, 128, 2) X(4, 128, 256, 2)         \
    X(5, 384, 128, 1) X(6, 128, 384, 1) X(7, 256, 256, 1) X(8, 256, 256, 2) X(9, 128, 128, 1)         \
    X(10, 384, 128, 2) X(11, 128, 384, 2) X(12, 256, 128, 1) X(13, 128, 256, 1)         \
    X(14, 64, 448, 1) X(15, 448, 64, 1) X(16, 64, 192, 2) X(17, 192, 64, 2) X(18, 32, 224, 4) X(19, 224, 32, 4)         \
    X(20, 32, 352, 2) X(21, 352, 32, 2) X(22, 64, 320, 2) X(23, 320, 64, 2) X(24, 32, 224, 3) X(25, 224, 32, 3)
constexpr int kCryptoPairVariants = 26;
#define CRYPTO_SOLO_VARIANTS(X) \
    X(0, 128, 4) X(1, 128, 6) X(2, 128, 8) X(3, 256, 2) X(4, 256, 3) X(5, 256, 4) X(6, 128, 3) X(7, 128, 5) X(8, 128, 2)
// the same sweep in work-queue form (warps draw chunks of nonces from the cursor in the hits record)
#define CRYPTO_SOLO_QUEUE_VARIANTS(X) \
    X(9, 256, 3) X(10, 384, 2) X(11, 128, 6) X(12, 256, 2) X(13, 192, 4) X(14, 512, 1)
constexpr int kCryptoSoloVariants = 15;

template <class RA, class RB>
int dispatch_pair(const char* name, int default_variant, typename RA::Args a, typename RB::Args b, cudaStream_t s) {
    const Tune t = tune_get(name);
    // each half draws its nonces from the cursor in its own record: one record for both halves
    // would make them share a cursor and skip nonces
    if (a.c.hits == b.c.hits) return HFUSE_ERR_BAD_ARG;
    // the work-queue cursors must start at zero whatever the caller left in the records
    if (cudaMemsetAsync(&a.c.hits->reserved, 0, sizeof(uint32_t), s) != cudaSuccess ||
        cudaMemsetAsync(&b.c.hits->reserved, 0, sizeof(uint32_t), s) != cudaSuccess)
        return HFUSE_ERR_LAUNCH;
    switch (t.variant >= 0 ? t.variant : default_variant) {
#define X(I, TA, TB, MB) \
    case I: return launch_pair_queue<RA, RB, TA, TB, MB>(a, b, t.blocks_per_sm, s);
        CRYPTO_PAIR_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}
template <class R>
int dispatch_solo(const char* name, int default_variant, typename R::Args a, cudaStream_t s) {
    const Tune t = tune_get(name);
    switch (t.variant >= 0 ? t.variant : default_variant) {
#define X(I, T, MB) \
    case I: return launch_solo<R, T, MB>(a, t.blocks_per_sm, s);
        CRYPTO_SOLO_VARIANTS(X)
#undef X
#define X(I, T, MB)                                                                                         \
    case I:                                                                                                 \
        if (cudaMemsetAsync(&a.c.hits->reserved, 0, sizeof(uint32_t), s) != cudaSuccess) return HFUSE_ERR_LAUNCH; \
        return launch_solo_queue<R, T, MB>(a, t.blocks_per_sm, s);
        CRYPTO_SOLO_QUEUE_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}

#include "crypto_tuned.inc"

}  // namespace

#define S_(x) static_cast<cudaStream_t>(x)

#define DEFINE_CPAIR(NAME, RA, PA, NA, prepA, ArgsA, RB, PB, NB, prepB, ArgsB)                         \
    extern "C" int hfuse_##NAME##_search(PA(a_), PB(b_), hfuse_stream_t stream) {                     \
        ArgsA a;                                                                                       \
        ArgsB b;                                                                                       \
        if (int rc = prepA(NA(a_), a)) return rc;                                                      \
        if (int rc = prepB(NB(b_), b)) return rc;                                                      \
        return dispatch_pair<RA, RB>(#NAME, kDefaultPair_##NAME, a, b, S_(stream));                    \
    }
#define BLAKE_ Blake, HFUSE_BLAKE256_PARAMS, SEARCH_NAMES, prep_blake, Blake256Args
#define SHA_ Sha, HFUSE_SHA256D_PARAMS, SEARCH_NAMES, prep_sha, Sha256dArgs
#define SIA_ Sia, HFUSE_SIA_PARAMS, SEARCH_NAMES, prep_sia, SiaArgs
#define ETH_ Eth, HFUSE_ETHASH_PARAMS, ETHASH_NAMES, prep_eth, EthashArgs
#define DEFINE_CPAIR_(NAME, A, B) DEFINE_CPAIR_X(NAME, A, B)
#define DEFINE_CPAIR_X(NAME, ...) DEFINE_CPAIR(NAME, __VA_ARGS__)
