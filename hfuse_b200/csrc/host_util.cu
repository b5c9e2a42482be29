// Host-side utilities of the C ABI: error strings, the tuning table and the
// seeded byte generator the synthetic workloads are drawn from.
#include <cstring>
#include "launch.cuh"

namespace hfuse {
int dl_describe(const char* name, int variant, char* buf, size_t n);
int crypto_describe(const char* name, int variant, char* buf, size_t n);
int dl_default_variant(const char* name);
int crypto_default_variant(const char* name);
}  // namespace hfuse

extern "C" {

const char* hfuse_error_string(int code) {
    switch (code) {
    case HFUSE_OK: return "ok";
    case HFUSE_ERR_BAD_ARG: return "bad argument (null pointer, non-positive extent or inconsistent shape)";
    case HFUSE_ERR_ALIGNMENT: return "buffer not 16-byte aligned";
    case HFUSE_ERR_TOO_LARGE: return "extent exceeds the kernels' index range";
    case HFUSE_ERR_WORKSPACE: return "scratch buffer missing or too small";
    case HFUSE_ERR_LAUNCH: return "CUDA reported an error at launch";
    case HFUSE_ERR_NO_DEVICE: return "no usable sm_100 device";
    case HFUSE_ERR_UNKNOWN_PAIR: return "unknown kernel or pair name";
    case HFUSE_ERR_COMM: return "NCCL could not be loaded or one of its calls failed";
    case HFUSE_ERR_NOALLOC_LIMIT:
        return "more channels than the built-in scratch of the no-allocation entry point serves (HFUSE_NOALLOC_MAX_CHANNELS)";
    }
    return "unknown error code";
}

int hfuse_version(void) { return 100; }

int hfuse_tune_describe(const char* pair, int variant, char* buf, size_t buflen) {
    if (!pair || !buf || buflen == 0) return HFUSE_ERR_BAD_ARG;
    int rc = hfuse::dl_describe(pair, variant, buf, buflen);
    if (rc == HFUSE_ERR_UNKNOWN_PAIR) rc = hfuse::crypto_describe(pair, variant, buf, buflen);
    return rc;
}

int hfuse_tune_default(const char* pair) {
    if (!pair) return HFUSE_ERR_BAD_ARG;
    int rc = hfuse::dl_default_variant(pair);
    if (rc == HFUSE_ERR_UNKNOWN_PAIR) rc = hfuse::crypto_default_variant(pair);
    return rc;
}

int hfuse_tune_set(const char* pair, int variant, int blocks_per_sm) {
    if (!pair || blocks_per_sm < 0) return HFUSE_ERR_BAD_ARG;
    if (variant >= 0) {
        char tmp[32];
        const int rc = hfuse_tune_describe(pair, variant, tmp, sizeof tmp);
        if (rc < 0) return rc;
    } else {
        char tmp[32];
        if (hfuse_tune_describe(pair, 0, tmp, sizeof tmp) == HFUSE_ERR_UNKNOWN_PAIR) return HFUSE_ERR_UNKNOWN_PAIR;
    }
    std::lock_guard<std::mutex> lk(hfuse::tune_mutex());
    hfuse::Tune& t = hfuse::tune_table()[pair];      // a share set through hfuse_tune_set_share stays
    t.variant = variant < 0 ? -1 : variant;
    t.blocks_per_sm = blocks_per_sm;
    return HFUSE_OK;
}

int hfuse_tune_set_share(const char* pair, int permille) {
    if (!pair || permille < -1 || permille > 1000) return HFUSE_ERR_BAD_ARG;
    if (strcmp(pair, "upsample_bnstats_allreduce") != 0) return HFUSE_ERR_UNKNOWN_PAIR;
    std::lock_guard<std::mutex> lk(hfuse::tune_mutex());
    hfuse::tune_table()[pair].share_permille = permille;
    return HFUSE_OK;
}

int hfuse_tune_option(const char* name, int value) {
    if (!name) return HFUSE_ERR_BAD_ARG;
    if (strcmp(name, "im2col_store_path") != 0 && strcmp(name, "exchange_pair_pool") != 0 &&
        strcmp(name, "bnstats_load_path") != 0 && strcmp(name, "histc_load_path") != 0) return HFUSE_ERR_UNKNOWN_PAIR;
    if (value < -1 || value > 1) return HFUSE_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lk(hfuse::tune_mutex());
    if (value < 0) hfuse::option_table().erase(name);
    else hfuse::option_table()[name] = value;
    return HFUSE_OK;
}

int hfuse_shard_range(uint64_t total, int rank, int world, uint64_t* offset, uint64_t* length) {
    if (world <= 0 || rank < 0 || rank >= world || !offset || !length) return HFUSE_ERR_BAD_ARG;
    const uint64_t base = total / (uint64_t)world, extra = total % (uint64_t)world;
    const uint64_t r = (uint64_t)rank;
    *length = base + (r < extra ? 1 : 0);
    *offset = r * base + (r < extra ? r : extra);
    return HFUSE_OK;
}

static inline uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

void hfuse_xoshiro256ss_fill(uint64_t seed, void* host_dst, size_t nbytes) {
    uint64_t s[4];
    for (int i = 0; i < 4; ++i) {          // splitmix64 expands the seed into the state
        seed += 0x9E3779B97F4A7C15ull;
        uint64_t z = seed;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        s[i] = z ^ (z >> 31);
    }
    unsigned char* out = static_cast<unsigned char*>(host_dst);
    for (size_t off = 0; off < nbytes; off += 8) {
        const uint64_t r = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
        s[2] ^= t; s[3] = rotl(s[3], 45);
        const size_t n = nbytes - off < 8 ? nbytes - off : 8;
        for (size_t b = 0; b < n; ++b) out[off + b] = (unsigned char)(r >> (8 * b));
    }
}

}  // extern "C"
