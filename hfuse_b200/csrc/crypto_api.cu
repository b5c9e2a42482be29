// C-ABI entry points of the standalone nonce searches, the batch hasher used by
// tests and the variant descriptions.  The fused pairs live in crypto_pair_*.cu.
#include "crypto_host.cuh"


extern "C" {

int hfuse_hits_reset(hfuse_hits* hits, hfuse_stream_t stream) {
    if (!hits) return HFUSE_ERR_BAD_ARG;
    return cudaMemsetAsync(hits, 0, sizeof(hfuse_hits), S_(stream)) == cudaSuccess ? HFUSE_OK : HFUSE_ERR_LAUNCH;
}

int hfuse_blake256_search(HFUSE_BLAKE256_PARAMS(), hfuse_stream_t stream) {
    Blake256Args a;
    if (int rc = prep_blake(SEARCH_NAMES(), a)) return rc;
    return dispatch_solo<Blake>("blake256", kDefaultSolo_blake256, a, S_(stream));
}
int hfuse_sha256d_search(HFUSE_SHA256D_PARAMS(), hfuse_stream_t stream) {
    Sha256dArgs a;
    if (int rc = prep_sha(SEARCH_NAMES(), a)) return rc;
    return dispatch_solo<Sha>("sha256d", kDefaultSolo_sha256d, a, S_(stream));
}
int hfuse_sia_blake2b_search(HFUSE_SIA_PARAMS(), hfuse_stream_t stream) {
    SiaArgs a;
    if (int rc = prep_sia(SEARCH_NAMES(), a)) return rc;
    return dispatch_solo<Sia>("sia", kDefaultSolo_sia, a, S_(stream));
}
int hfuse_ethash_search(HFUSE_ETHASH_PARAMS(), hfuse_stream_t stream) {
    EthashArgs a;
    if (int rc = prep_eth(ETHASH_NAMES(), a)) return rc;
    return dispatch_solo<Eth>("ethash", kDefaultSolo_ethash, a, S_(stream));
}

int hfuse_hash_batch(int kind, const uint8_t* header, const void* dag, uint32_t dag_items, uint64_t start,
                     uint32_t count, uint8_t* out32, uint8_t* mix32, hfuse_stream_t stream) {
    if (!header || !out32) return HFUSE_ERR_BAD_ARG;
    if (count == 0) return HFUSE_OK;
    static const uint8_t zero_target[32] = {0};
    hfuse_hits* no_hits = reinterpret_cast<hfuse_hits*>(out32);   // never dereferenced in batch mode
    switch (kind) {
    case 0: {
        Blake256Args a;
        if (int rc = fill_blake(header, a)) return rc;
        if (int rc = prep_common(start, count, zero_target, no_hits, true, a.c)) return rc;
        a.c.out32 = out32;
        return launch_solo<Blake, 128, 4>(a, 0, S_(stream));
    }
    case 1: {
        Sha256dArgs a;
        if (int rc = fill_sha(header, a)) return rc;
        if (int rc = prep_common(start, count, zero_target, no_hits, true, a.c)) return rc;
        a.c.out32 = out32;
        return launch_solo<Sha, 128, 4>(a, 0, S_(stream));
    }
    case 2: {
        SiaArgs a;
        if (int rc = fill_sia(header, a)) return rc;
        if (int rc = prep_common(start, count, zero_target, no_hits, false, a.c)) return rc;
        a.c.out32 = out32;
        return launch_solo<Sia, 128, 4>(a, 0, S_(stream));
    }
    case 3: {
        EthashArgs a;
        if (int rc = fill_eth(dag, dag_items, header, a)) return rc;
        if (int rc = prep_common(start, count, zero_target, no_hits, false, a.c)) return rc;
        a.c.out32 = out32;
        a.c.mix32 = mix32;
        return launch_solo<Eth, 128, 4>(a, 0, S_(stream));
    }
    }
    return HFUSE_ERR_BAD_ARG;
}

}  // extern "C"

namespace hfuse {
int crypto_describe(const char* name, int variant, char* buf, size_t n) {
    static const char* solos[] = {"blake256", "sha256d", "sia", "ethash"};
    static const char* pairs[] = {"ethash_blake256", "sha256d_ethash", "sia_ethash",
                                  "blake256_sha256d", "blake256_sia", "sha256d_sia"};
    for (const char* s : solos)
        if (!strcmp(s, name)) {
            switch (variant) {
#define X(I, T, MB) \
    case I: snprintf(buf, n, "%d:0:%d", T, MB); return kCryptoSoloVariants;
                CRYPTO_SOLO_VARIANTS(X)
#undef X
#define X(I, T, MB) \
    case I: snprintf(buf, n, "%d:0:%d queue", T, MB); return kCryptoSoloVariants;
                CRYPTO_SOLO_QUEUE_VARIANTS(X)
#undef X
            }
            return HFUSE_ERR_BAD_ARG;
        }
    for (const char* p : pairs)
        if (!strcmp(p, name)) {
            switch (variant) {
#define X(I, TA, TB, MB) \
    case I: snprintf(buf, n, "%d:%d:%d", TA, TB, MB); return kCryptoPairVariants;
                CRYPTO_PAIR_VARIANTS(X)
#undef X
            }
            return HFUSE_ERR_BAD_ARG;
        }
    return HFUSE_ERR_UNKNOWN_PAIR;
}
int crypto_default_variant(const char* name) {
#define D(kind, n) if (!strcmp(name, #n)) return kDefault##kind##_##n;
    D(Solo, blake256) D(Solo, sha256d) D(Solo, sia) D(Solo, ethash)
    D(Pair, ethash_blake256) D(Pair, sha256d_ethash) D(Pair, sia_ethash) D(Pair, blake256_sha256d)
    D(Pair, blake256_sia) D(Pair, sha256d_sia)
#undef D
    return HFUSE_ERR_UNKNOWN_PAIR;
}
}  // namespace hfuse
