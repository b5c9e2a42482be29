/*
 * CPU oracle for the crypto nonce-search paths.  TEST INFRASTRUCTURE ONLY:
 * only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may load this library; the CUDA product never does.
 *
 * Parity status: "parity unpinned" by the reference.  The reference
 * (aoli-al/HFuse) ships neither the hash kernels nor any known-answer
 * vectors; it only names them (configs/crypto_kernels.yaml:1-32,
 * configs/crypto_fusion.yaml:1-24) and records their launch signatures
 * (scripts/data/ethminer_event.csv:2-27).  The kernels live in the
 * un-vendored third-party repository aoli-al/ethminer (branch "ae",
 * scripts/docker/Dockerfile:30-35, no commit pin).  Every function below is
 * therefore a restatement of the *published* algorithm:
 *   SHA-256            FIPS 180-4
 *   BLAKE-256          SHA-3 finalist specification (14 rounds)
 *   BLAKE2b            RFC 7693
 *   Keccak-f[1600]     Keccak reference (original 0x01 padding for ethash,
 *                      0x06 selectable so hashlib's SHA-3 can check it)
 *   ethash hashimoto   public ethash specification, over a supplied DAG
 *   xoshiro256**       Blackman & Vigna, seeded by splitmix64
 * and is pinned by the tests against hashlib (SHA-256, BLAKE2b, SHA-3), the
 * specification's own BLAKE-256 / Keccak digests, and a second independent
 * pure-Python restatement (oracle/crypto_py.py).
 *
 * Conventions shared with the CUDA library:
 *   - a digest is a hit iff its 32 bytes, read as a 256-bit big-endian
 *     integer, are strictly below the 32-byte big-endian target;
 *   - BLAKE-256 / SHA-256d: 80-byte header, 32-bit little-endian nonce at
 *     bytes 76..79;  Sia BLAKE2b-256: 80-byte header, 64-bit little-endian
 *     nonce at bytes 32..39;  ethash: Keccak-512(header_hash[32] || nonce LE64).
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define EXPORT __attribute__((visibility("default")))

static inline uint32_t rotr32(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
static inline uint64_t rotr64(uint64_t x, int n) { return (x >> n) | (x << (64 - n)); }
static inline uint64_t rotl64(uint64_t x, int n) { return (x << n) | (x >> (64 - n)); }
static inline uint32_t load_be32(const uint8_t *p) {
    return ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | p[3];
}
static inline void store_be32(uint8_t *p, uint32_t v) {
    p[0] = v >> 24; p[1] = v >> 16; p[2] = v >> 8; p[3] = v;
}
static inline uint64_t load_le64(const uint8_t *p) {
    uint64_t v = 0;
    for (int i = 7; i >= 0; --i) v = (v << 8) | p[i];
    return v;
}
static inline void store_le64(uint8_t *p, uint64_t v) {
    for (int i = 0; i < 8; ++i) { p[i] = (uint8_t)v; v >>= 8; }
}
static inline uint32_t load_le32(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static inline void store_le32(uint8_t *p, uint32_t v) {
    p[0] = v; p[1] = v >> 8; p[2] = v >> 16; p[3] = v >> 24;
}

/* digest < target as 256-bit big-endian integers */
EXPORT int oracle_below_target(const uint8_t digest[32], const uint8_t target[32]) {
    return memcmp(digest, target, 32) < 0;
}

/* ------------------------------------------------------------------ */
/* xoshiro256** seeded by four splitmix64 outputs; little-endian u64 stream */
static uint64_t splitmix64(uint64_t *x) {
    uint64_t z = (*x += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

EXPORT void oracle_xoshiro256ss_fill(uint64_t seed, uint8_t *out, size_t nbytes) {
    uint64_t s[4], x = seed;
    for (int i = 0; i < 4; ++i) s[i] = splitmix64(&x);
    size_t off = 0;
    while (off < nbytes) {
        uint64_t r = rotl64(s[1] * 5, 7) * 9;
        uint64_t t = s[1] << 17;
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
        s[2] ^= t; s[3] = rotl64(s[3], 45);
        uint8_t b[8];
        store_le64(b, r);
        size_t n = nbytes - off < 8 ? nbytes - off : 8;
        memcpy(out + off, b, n);
        off += n;
    }
}

/* ------------------------------------------------------------------ */
/* SHA-256 (FIPS 180-4) */
static const uint32_t SHA_K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
static const uint32_t SHA_IV[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                   0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};

static void sha256_compress(uint32_t h[8], const uint8_t block[64]) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = load_be32(block + 4 * i);
    for (int i = 16; i < 64; ++i) {
        uint32_t s0 = rotr32(w[i - 15], 7) ^ rotr32(w[i - 15], 18) ^ (w[i - 15] >> 3);
        uint32_t s1 = rotr32(w[i - 2], 17) ^ rotr32(w[i - 2], 19) ^ (w[i - 2] >> 10);
        w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
        uint32_t S1 = rotr32(e, 6) ^ rotr32(e, 11) ^ rotr32(e, 25);
        uint32_t ch = (e & f) ^ (~e & g);
        uint32_t t1 = hh + S1 + ch + SHA_K[i] + w[i];
        uint32_t S0 = rotr32(a, 2) ^ rotr32(a, 13) ^ rotr32(a, 22);
        uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
        uint32_t t2 = S0 + mj;
        hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}

EXPORT void oracle_sha256(const uint8_t *msg, size_t len, uint8_t out[32]) {
    uint32_t h[8];
    memcpy(h, SHA_IV, sizeof h);
    size_t off = 0;
    for (; off + 64 <= len; off += 64) sha256_compress(h, msg + off);
    uint8_t buf[128];
    size_t rem = len - off;
    memset(buf, 0, sizeof buf);
    memcpy(buf, msg + off, rem);
    buf[rem] = 0x80;
    size_t tot = rem + 9 <= 64 ? 64 : 128;
    uint64_t bits = (uint64_t)len * 8;
    for (int i = 0; i < 8; ++i) buf[tot - 1 - i] = (uint8_t)(bits >> (8 * i));
    sha256_compress(h, buf);
    if (tot == 128) sha256_compress(h, buf + 64);
    for (int i = 0; i < 8; ++i) store_be32(out + 4 * i, h[i]);
}

EXPORT void oracle_sha256d_header(const uint8_t header[80], uint32_t nonce, uint8_t out[32]) {
    uint8_t h[80], d1[32];
    memcpy(h, header, 80);
    store_le32(h + 76, nonce);
    oracle_sha256(h, 80, d1);
    oracle_sha256(d1, 32, out);
}

/* ------------------------------------------------------------------ */
/* BLAKE-256 (SHA-3 finalist, 14 rounds) */
static const uint32_t BLAKE_C[16] = {
    0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0, 0x082EFA98, 0xEC4E6C89,
    0x452821E6, 0x38D01377, 0xBE5466CF, 0x34E90C6C, 0xC0AC29B7, 0xC97C50DD, 0x3F84D5B5, 0xB5470917};
static const uint8_t SIGMA[10][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15},
    {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4},
    {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13},
    {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11},
    {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5},
    {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};

static void blake256_compress(uint32_t h[8], const uint8_t block[64], uint64_t t, int rounds) {
    uint32_t m[16], v[16];
    for (int i = 0; i < 16; ++i) m[i] = load_be32(block + 4 * i);
    for (int i = 0; i < 8; ++i) v[i] = h[i];
    for (int i = 0; i < 4; ++i) v[8 + i] = BLAKE_C[i];          /* salt = 0 */
    uint32_t t0 = (uint32_t)t, t1 = (uint32_t)(t >> 32);
    v[12] = t0 ^ BLAKE_C[4]; v[13] = t0 ^ BLAKE_C[5];
    v[14] = t1 ^ BLAKE_C[6]; v[15] = t1 ^ BLAKE_C[7];
#define BG(a, b, c, d, i)                                               \
    do {                                                                \
        v[a] += v[b] + (m[s[2 * i]] ^ BLAKE_C[s[2 * i + 1]]);           \
        v[d] = rotr32(v[d] ^ v[a], 16);                                 \
        v[c] += v[d];                                                   \
        v[b] = rotr32(v[b] ^ v[c], 12);                                 \
        v[a] += v[b] + (m[s[2 * i + 1]] ^ BLAKE_C[s[2 * i]]);           \
        v[d] = rotr32(v[d] ^ v[a], 8);                                  \
        v[c] += v[d];                                                   \
        v[b] = rotr32(v[b] ^ v[c], 7);                                  \
    } while (0)
    for (int r = 0; r < rounds; ++r) {
        const uint8_t *s = SIGMA[r % 10];
        BG(0, 4, 8, 12, 0); BG(1, 5, 9, 13, 1); BG(2, 6, 10, 14, 2); BG(3, 7, 11, 15, 3);
        BG(0, 5, 10, 15, 4); BG(1, 6, 11, 12, 5); BG(2, 7, 8, 13, 6); BG(3, 4, 9, 14, 7);
    }
#undef BG
    for (int i = 0; i < 8; ++i) h[i] ^= v[i] ^ v[i + 8];
}

EXPORT void oracle_blake256(const uint8_t *msg, size_t len, uint8_t out[32]) {
    uint32_t h[8];
    memcpy(h, SHA_IV, sizeof h);   /* BLAKE-256 shares SHA-256's IV */
    uint64_t t = 0;
    size_t off = 0;
    for (; off + 64 <= len; off += 64) { t += 512; blake256_compress(h, msg + off, t, 14); }
    size_t rem = len - off;
    uint8_t buf[128];
    memset(buf, 0, sizeof buf);
    memcpy(buf, msg + off, rem);
    buf[rem] = 0x80;
    uint64_t bits = (uint64_t)len * 8;
    if (rem <= 55) {
        buf[55] |= 0x01;
        for (int i = 0; i < 8; ++i) buf[63 - i] = (uint8_t)(bits >> (8 * i));
        /* the counter counts message bits only: 0 for a block holding none */
        blake256_compress(h, buf, rem ? bits : 0, 14);
    } else {
        buf[119] |= 0x01;
        for (int i = 0; i < 8; ++i) buf[127 - i] = (uint8_t)(bits >> (8 * i));
        blake256_compress(h, buf, bits, 14);
        blake256_compress(h, buf + 64, 0, 14);
    }
    for (int i = 0; i < 8; ++i) store_be32(out + 4 * i, h[i]);
}

EXPORT void oracle_blake256_header(const uint8_t header[80], uint32_t nonce, uint8_t out[32]) {
    uint8_t h[80];
    memcpy(h, header, 80);
    store_le32(h + 76, nonce);
    oracle_blake256(h, 80, out);
}

/* ------------------------------------------------------------------ */
/* BLAKE2b (RFC 7693), unkeyed */
static const uint64_t B2B_IV[8] = {
    0x6a09e667f3bcc908ull, 0xbb67ae8584caa73bull, 0x3c6ef372fe94f82bull, 0xa54ff53a5f1d36f1ull,
    0x510e527fade682d1ull, 0x9b05688c2b3e6c1full, 0x1f83d9abfb41bd6bull, 0x5be0cd19137e2179ull};

static void blake2b_compress(uint64_t h[8], const uint8_t block[128], uint64_t t, int last) {
    uint64_t m[16], v[16];
    for (int i = 0; i < 16; ++i) m[i] = load_le64(block + 8 * i);
    for (int i = 0; i < 8; ++i) { v[i] = h[i]; v[8 + i] = B2B_IV[i]; }
    v[12] ^= t;
    if (last) v[14] = ~v[14];
#define G2(a, b, c, d, x, y)                    \
    do {                                        \
        v[a] = v[a] + v[b] + (x);               \
        v[d] = rotr64(v[d] ^ v[a], 32);         \
        v[c] = v[c] + v[d];                     \
        v[b] = rotr64(v[b] ^ v[c], 24);         \
        v[a] = v[a] + v[b] + (y);               \
        v[d] = rotr64(v[d] ^ v[a], 16);         \
        v[c] = v[c] + v[d];                     \
        v[b] = rotr64(v[b] ^ v[c], 63);         \
    } while (0)
    for (int r = 0; r < 12; ++r) {
        const uint8_t *s = SIGMA[r % 10];
        G2(0, 4, 8, 12, m[s[0]], m[s[1]]);   G2(1, 5, 9, 13, m[s[2]], m[s[3]]);
        G2(2, 6, 10, 14, m[s[4]], m[s[5]]);  G2(3, 7, 11, 15, m[s[6]], m[s[7]]);
        G2(0, 5, 10, 15, m[s[8]], m[s[9]]);  G2(1, 6, 11, 12, m[s[10]], m[s[11]]);
        G2(2, 7, 8, 13, m[s[12]], m[s[13]]); G2(3, 4, 9, 14, m[s[14]], m[s[15]]);
    }
#undef G2
    for (int i = 0; i < 8; ++i) h[i] ^= v[i] ^ v[i + 8];
}

EXPORT void oracle_blake2b(const uint8_t *msg, size_t len, uint8_t *out, size_t outlen) {
    uint64_t h[8];
    memcpy(h, B2B_IV, sizeof h);
    h[0] ^= 0x01010000ull ^ (uint64_t)outlen;
    size_t off = 0;
    uint8_t buf[128];
    while (len - off > 128) { off += 128; blake2b_compress(h, msg + off - 128, off, 0); }
    memset(buf, 0, sizeof buf);
    memcpy(buf, msg + off, len - off);
    blake2b_compress(h, buf, len, 1);
    uint8_t full[64];
    for (int i = 0; i < 8; ++i) store_le64(full + 8 * i, h[i]);
    memcpy(out, full, outlen);
}

EXPORT void oracle_sia_header(const uint8_t header[80], uint64_t nonce, uint8_t out[32]) {
    uint8_t h[80];
    memcpy(h, header, 80);
    store_le64(h + 32, nonce);
    oracle_blake2b(h, 80, out, 32);
}

/* ------------------------------------------------------------------ */
/* Keccak-f[1600] and a sponge with a selectable domain/pad byte */
static const uint64_t KECCAK_RC[24] = {
    0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808aull, 0x8000000080008000ull,
    0x000000000000808bull, 0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull,
    0x000000000000008aull, 0x0000000000000088ull, 0x0000000080008009ull, 0x000000008000000aull,
    0x000000008000808bull, 0x800000000000008bull, 0x8000000000008089ull, 0x8000000000008003ull,
    0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800aull, 0x800000008000000aull,
    0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull};
static const int KECCAK_ROT[25] = {0, 1, 62, 28, 27, 36, 44, 6, 55, 20, 3, 10, 43,
                                   25, 39, 41, 45, 15, 21, 8, 18, 2, 61, 56, 14};

static void keccak_f1600(uint64_t a[25]) {
    for (int r = 0; r < 24; ++r) {
        uint64_t c[5], b[25];
        for (int x = 0; x < 5; ++x) c[x] = a[x] ^ a[x + 5] ^ a[x + 10] ^ a[x + 15] ^ a[x + 20];
        for (int x = 0; x < 5; ++x) {
            uint64_t d = c[(x + 4) % 5] ^ rotl64(c[(x + 1) % 5], 1);
            for (int y = 0; y < 25; y += 5) a[y + x] ^= d;
        }
        /* rho + pi: B[y][2x+3y] = rot(A[x][y]) with lane index x + 5y */
        for (int x = 0; x < 5; ++x)
            for (int y = 0; y < 5; ++y) {
                int src = x + 5 * y;
                int dst = y + 5 * ((2 * x + 3 * y) % 5);
                int rot = KECCAK_ROT[src];
                b[dst] = rot ? rotl64(a[src], rot) : a[src];
            }
        for (int y = 0; y < 25; y += 5)
            for (int x = 0; x < 5; ++x) a[y + x] = b[y + x] ^ (~b[y + (x + 1) % 5] & b[y + (x + 2) % 5]);
        a[0] ^= KECCAK_RC[r];
    }
}

/* rate in bytes; pad = 0x01 (original Keccak) or 0x06 (NIST SHA-3) */
EXPORT void oracle_keccak(const uint8_t *msg, size_t len, size_t rate, uint8_t pad,
                          uint8_t *out, size_t outlen) {
    uint64_t a[25];
    uint8_t buf[200];
    memset(a, 0, sizeof a);
    size_t off = 0;
    for (; off + rate <= len; off += rate) {
        for (size_t i = 0; i < rate / 8; ++i) a[i] ^= load_le64(msg + off + 8 * i);
        keccak_f1600(a);
    }
    memset(buf, 0, sizeof buf);
    memcpy(buf, msg + off, len - off);
    buf[len - off] ^= pad;
    buf[rate - 1] ^= 0x80;
    for (size_t i = 0; i < rate / 8; ++i) a[i] ^= load_le64(buf + 8 * i);
    keccak_f1600(a);
    for (size_t i = 0; i < 25; ++i) store_le64(buf + 8 * i, a[i]);
    memcpy(out, buf, outlen);   /* outlen <= rate for every use here */
}

/* ------------------------------------------------------------------ */
/* ethash hashimoto over a supplied DAG of 128-byte items */
#define FNV_PRIME 0x01000193u
static inline uint32_t fnv(uint32_t a, uint32_t b) { return (a * FNV_PRIME) ^ b; }

EXPORT void oracle_ethash_hashimoto(const uint8_t *dag, uint32_t n_items, const uint8_t header_hash[32],
                                    uint64_t nonce, uint8_t mix_out[32], uint8_t result_out[32]) {
    uint8_t seed_in[40], s_bytes[64];
    memcpy(seed_in, header_hash, 32);
    store_le64(seed_in + 32, nonce);
    oracle_keccak(seed_in, 40, 72, 0x01, s_bytes, 64);
    uint32_t s[16], mix[32];
    for (int i = 0; i < 16; ++i) s[i] = load_le32(s_bytes + 4 * i);
    for (int i = 0; i < 32; ++i) mix[i] = s[i % 16];
    for (uint32_t i = 0; i < 64; ++i) {
        uint32_t p = fnv(i ^ s[0], mix[i % 32]) % n_items;
        const uint8_t *item = dag + (size_t)p * 128;
        for (int j = 0; j < 32; ++j) mix[j] = fnv(mix[j], load_le32(item + 4 * j));
    }
    uint8_t fin[96];
    memcpy(fin, s_bytes, 64);
    for (int i = 0; i < 8; ++i) {
        uint32_t c = fnv(fnv(fnv(mix[4 * i], mix[4 * i + 1]), mix[4 * i + 2]), mix[4 * i + 3]);
        store_le32(mix_out + 4 * i, c);
    }
    memcpy(fin + 64, mix_out, 32);
    oracle_keccak(fin, 96, 136, 0x01, result_out, 32);
}

/* ------------------------------------------------------------------ */
/* ethash light cache and DAG generation (public ethash specification, revision 23):
 *   cache:  o[0] = Keccak-512(seed), o[i] = Keccak-512(o[i-1]); then 3 rounds of
 *           o[i] = Keccak-512(o[(i-1+n) % n] xor o[o[i][0] % n])
 *   node i: mix = cache[i % n]; mix[0] ^= i; mix = Keccak-512(mix);
 *           256 times: mix = fnv(mix, cache[fnv(i ^ j, mix[j % 16]) % n]); node = Keccak-512(mix)
 * Nodes are 64 bytes; a 128-byte DAG item is two consecutive nodes. */
EXPORT void oracle_ethash_mkcache(const uint8_t seed[32], uint32_t n, uint8_t *cache) {
    oracle_keccak(seed, 32, 72, 0x01, cache, 64);
    for (uint32_t i = 1; i < n; ++i) oracle_keccak(cache + 64 * (size_t)(i - 1), 64, 72, 0x01, cache + 64 * (size_t)i, 64);
    for (int round = 0; round < 3; ++round)
        for (uint32_t i = 0; i < n; ++i) {
            uint32_t v = load_le32(cache + 64 * (size_t)i) % n;
            uint8_t x[64];
            const uint8_t *a = cache + 64 * (size_t)((i + n - 1) % n), *b = cache + 64 * (size_t)v;
            for (int k = 0; k < 64; ++k) x[k] = a[k] ^ b[k];
            oracle_keccak(x, 64, 72, 0x01, cache + 64 * (size_t)i, 64);
        }
}

EXPORT void oracle_ethash_dataset_node(const uint8_t *cache, uint32_t n, uint32_t i, uint8_t out[64]) {
    uint32_t mix[16];
    uint8_t buf[64];
    for (int k = 0; k < 16; ++k) mix[k] = load_le32(cache + 64 * (size_t)(i % n) + 4 * k);
    mix[0] ^= i;
    for (int k = 0; k < 16; ++k) store_le32(buf + 4 * k, mix[k]);
    oracle_keccak(buf, 64, 72, 0x01, buf, 64);
    for (int k = 0; k < 16; ++k) mix[k] = load_le32(buf + 4 * k);
    for (uint32_t j = 0; j < 256; ++j) {
        const uint32_t parent = fnv(i ^ j, mix[j % 16]) % n;
        for (int k = 0; k < 16; ++k) mix[k] = fnv(mix[k], load_le32(cache + 64 * (size_t)parent + 4 * k));
    }
    for (int k = 0; k < 16; ++k) store_le32(buf + 4 * k, mix[k]);
    oracle_keccak(buf, 64, 72, 0x01, out, 64);
}

EXPORT void oracle_ethash_dataset(const uint8_t *cache, uint32_t n, uint32_t first, uint32_t count, uint8_t *out) {
#pragma omp parallel for schedule(static)
    for (uint32_t k = 0; k < count; ++k) oracle_ethash_dataset_node(cache, n, first + k, out + 64 * (size_t)k);
}

/* ------------------------------------------------------------------ */
/* Nonce sweeps (OpenMP over nonces).  Hits come back sorted by nonce.
 * kind: 0 = BLAKE-256, 1 = SHA-256d, 2 = Sia BLAKE2b-256, 3 = ethash.
 * Returns the number of hits found; when that exceeds max_hits only an
 * arbitrary max_hits of them are stored, so callers size max_hits generously. */
static void sort_hits(uint64_t *nonces, uint8_t *mix, int n) {
    for (int i = 1; i < n; ++i) {
        uint64_t k = nonces[i];
        uint8_t km[32];
        if (mix) memcpy(km, mix + 32 * i, 32);
        int j = i - 1;
        while (j >= 0 && nonces[j] > k) {
            nonces[j + 1] = nonces[j];
            if (mix) memcpy(mix + 32 * (j + 1), mix + 32 * j, 32);
            --j;
        }
        nonces[j + 1] = k;
        if (mix) memcpy(mix + 32 * (j + 1), km, 32);
    }
}

EXPORT int oracle_search(int kind, const uint8_t *header, const uint8_t *dag, uint32_t n_items,
                         uint64_t start, uint64_t count, const uint8_t target[32],
                         uint64_t *hit_nonces, uint8_t *hit_mix, int max_hits, int threads) {
    int found = 0;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < count; ++i) {
        uint8_t d[32], mix[32];
        uint64_t nonce = start + i;
        switch (kind) {
        case 0: nonce = (uint32_t)nonce; oracle_blake256_header(header, (uint32_t)nonce, d); break;
        case 1: nonce = (uint32_t)nonce; oracle_sha256d_header(header, (uint32_t)nonce, d); break;
        case 2: oracle_sia_header(header, nonce, d); break;
        default: oracle_ethash_hashimoto(dag, n_items, header, nonce, mix, d); break;
        }
        if (memcmp(d, target, 32) < 0) {
#pragma omp critical
            {
                if (found < max_hits) {
                    hit_nonces[found] = nonce;
                    if (kind == 3 && hit_mix) memcpy(hit_mix + 32 * found, mix, 32);
                }
                ++found;
            }
        }
    }
    int stored = found < max_hits ? found : max_hits;
    sort_hits(hit_nonces, (kind == 3) ? hit_mix : NULL, stored);
    return found;
}

EXPORT int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
