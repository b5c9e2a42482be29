// Role bodies of the four nonce-search kernels.
//
// Reference kernels these replace (configs/crypto_kernels.yaml:1-32 of
// aoli-al/HFuse; signatures in scripts/data/ethminer_event.csv:2-27):
//   blake2b_gpu_hash ("Blake256")   -> Blake256Role   BLAKE-256, 14 rounds
//   sha256d_gpu_hash_shared         -> Sha256dRole    SHA-256(SHA-256(header))
//   sia_blake2b_gpu_hash            -> SiaRole        BLAKE2b-256, one block
//   ethash_search                   -> EthashRole     hashimoto over a DAG
// The reference kernels read header, target and DAG from __constant__
// symbols; here everything arrives in the kernel parameters.  Work that does
// not depend on the nonce (first-block midstates, constant message words) is
// done once on the host.
//
// All four are integer-ALU work on 32-bit lanes (ethash: plus random 128-byte
// DAG reads): rotations are funnel shifts or byte permutes, boolean
// functions collapse to LOP3; no tensor cores, nothing here is a contraction.
#pragma once
#include "common.cuh"
#include "../../include/hfuse_b200.h"

namespace hfuse {

// ---------------------------------------------------------------------------
// shared pieces
// ---------------------------------------------------------------------------
struct SearchCommon {
    unsigned long long start;   // first nonce
    unsigned long long count;   // nonces to sweep
    uint32_t target[8];         // big-endian words of the 256-bit target, most significant first
    hfuse_hits* hits;           // result record (device)
    uint8_t* out32;             // when non-null: write every digest here instead of searching (tests)
    uint8_t* mix32;             // ditto for ethash mix digests
    uint32_t one;               // the value 1, opaque to the compiler: see add_fma()
};

__device__ __forceinline__ uint32_t rotr32(uint32_t x, int n) { return __funnelshift_r(x, x, n); }
__device__ __forceinline__ uint32_t bswap32(uint32_t x) { return __byte_perm(x, 0, 0x0123); }

// a + b computed as a * one + b: an integer multiply-add, which issues to the FMA pipe.  The
// 32-bit hashes saturate the integer ALU pipe (adds, logic, shifts and permutes all go there)
// while the FMA pipe idles; moving a third of the adds over is worth 5-8 % (measured).  The
// multiplier comes from the kernel arguments so that it is not folded back into an add.
__device__ __forceinline__ uint32_t add_fma(uint32_t a, uint32_t one, uint32_t b) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(one), "r"(b));
    return d;
}

// digest words most-significant first; strict "<" on the 256-bit integer
__device__ __forceinline__ bool below_target(const uint32_t d[8], const uint32_t t[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (d[i] < t[i]) return true;
        if (d[i] > t[i]) return false;
    }
    return false;
}

__device__ __forceinline__ void record_hit(hfuse_hits* hits, unsigned long long nonce, const uint32_t* mix) {
    const uint32_t slot = atomicAdd(&hits->count, 1u);
    if (slot < HFUSE_MAX_HITS) {
        hits->nonce[slot] = nonce;
#pragma unroll
        for (int i = 0; i < 8; ++i) hits->mix[slot][i] = mix ? mix[i] : 0u;
    }
}

// digest words (most significant first) -> 32 bytes, big-endian words
__device__ __forceinline__ void write_digest_be(uint8_t* out, unsigned long long i, const uint32_t d[8]) {
    uint32_t* p = reinterpret_cast<uint32_t*>(out + 32 * i);
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] = bswap32(d[k]);
}

// ---------------------------------------------------------------------------
// SHA-256d
// ---------------------------------------------------------------------------
struct Sha256dArgs {
    SearchCommon c;
    uint32_t mid[8];     // state after the first 64 header bytes
    uint32_t w0, w1, w2; // header bytes 64..75 as big-endian words
};

// K as literals so that the fully unrolled rounds carry them as immediates
#define HFUSE_SHA_K(i) kShaKLit[i]
#define HFUSE_SHAK_INIT { \
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, \
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, \
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, \
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, \
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, \
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, \
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, \
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2}
static constexpr uint32_t kShaKLit[64] = HFUSE_SHAK_INIT;

__device__ __forceinline__ void sha256_rounds(uint32_t s[8], uint32_t w[16], uint32_t one) {
    constexpr uint32_t kShaKLit[64] = HFUSE_SHAK_INIT;   // local copy: folds into immediates
    uint32_t a = s[0], b = s[1], c = s[2], d = s[3], e = s[4], f = s[5], g = s[6], h = s[7];
#pragma unroll
    for (int i = 0; i < 64; ++i) {
        if (i >= 16) {
            const uint32_t x = w[(i + 1) & 15], y = w[(i + 14) & 15];
            const uint32_t s0 = rotr32(x, 7) ^ rotr32(x, 18) ^ (x >> 3);
            const uint32_t s1 = rotr32(y, 17) ^ rotr32(y, 19) ^ (y >> 10);
            w[i & 15] = add_fma(w[i & 15] + s0, one, w[(i + 9) & 15] + s1);
        }
        const uint32_t S1 = rotr32(e, 6) ^ rotr32(e, 11) ^ rotr32(e, 25);
        const uint32_t ch = (e & f) ^ (~e & g);
        const uint32_t t1 = add_fma(h + S1 + ch, one, HFUSE_SHA_K(i) + w[i & 15]);
        const uint32_t S0 = rotr32(a, 2) ^ rotr32(a, 13) ^ rotr32(a, 22);
        const uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
        h = g; g = f; f = e; e = add_fma(d, one, t1); d = c; c = b; b = a; a = add_fma(t1, one, S0 + mj);
    }
    s[0] += a; s[1] += b; s[2] += c; s[3] += d; s[4] += e; s[5] += f; s[6] += g; s[7] += h;
}

struct Sha256dRole {
    using Args = Sha256dArgs;
    static constexpr bool kCooperative = false;

    static __device__ __forceinline__ void hash(const Args& a, uint32_t nonce, uint32_t d[8]) {
        uint32_t w[16] = {a.w0, a.w1, a.w2, bswap32(nonce), 0x80000000u, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 640u};
        uint32_t s[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = a.mid[i];
        sha256_rounds(s, w, a.c.one);
        uint32_t w2[16] = {s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7], 0x80000000u, 0, 0, 0, 0, 0, 0, 256u};
        d[0] = 0x6a09e667u; d[1] = 0xbb67ae85u; d[2] = 0x3c6ef372u; d[3] = 0xa54ff53au;
        d[4] = 0x510e527fu; d[5] = 0x9b05688cu; d[6] = 0x1f83d9abu; d[7] = 0x5be0cd19u;
        sha256_rounds(d, w2, a.c.one);
    }
};

// ---------------------------------------------------------------------------
// BLAKE-256 (14 rounds)
// ---------------------------------------------------------------------------
struct Blake256Args {
    SearchCommon c;
    uint32_t mid[8];     // chain value after the first 64 header bytes (counter 512)
    uint32_t m0, m1, m2; // header bytes 64..75 as big-endian words
};

#define HFUSE_BLAKEC_INIT { \
    0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0, 0x082EFA98, 0xEC4E6C89, \
    0x452821E6, 0x38D01377, 0xBE5466CF, 0x34E90C6C, 0xC0AC29B7, 0xC97C50DD, 0x3F84D5B5, 0xB5470917}
static constexpr uint32_t kBlakeC[16] = HFUSE_BLAKEC_INIT;
#define HFUSE_SIGMA_INIT { \
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3}, \
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8}, \
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9}, \
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10}, \
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}}
static constexpr unsigned char kSigma[10][16] = HFUSE_SIGMA_INIT;

struct Blake256Role {
    using Args = Blake256Args;
    static constexpr bool kCooperative = false;

    static __device__ __forceinline__ void hash(const Args& a, uint32_t nonce, uint32_t d[8]) {
        constexpr uint32_t kBlakeC[16] = HFUSE_BLAKEC_INIT;
        constexpr unsigned char kSigma[10][16] = HFUSE_SIGMA_INIT;
        // second block: 16 header bytes, 0x80, zeros, 0x01 in byte 55, bit length 640
        const uint32_t m[16] = {a.m0, a.m1, a.m2, bswap32(nonce), 0x80000000u, 0, 0, 0, 0, 0, 0, 0, 0, 1u, 0, 640u};
        const uint32_t one = a.c.one;
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = a.mid[i];
        v[8] = kBlakeC[0]; v[9] = kBlakeC[1]; v[10] = kBlakeC[2]; v[11] = kBlakeC[3];
        v[12] = 640u ^ kBlakeC[4]; v[13] = 640u ^ kBlakeC[5]; v[14] = kBlakeC[6]; v[15] = kBlakeC[7];
#define HFUSE_BG(A, B, C, D, I)                                                      \
    v[A] = add_fma(v[A] + v[B], one, (m[kSigma[r % 10][2 * I]] ^ kBlakeC[kSigma[r % 10][2 * I + 1]]));  \
    v[D] = __byte_perm(v[D] ^ v[A], 0, 0x1032);                                      \
    v[C] = add_fma(v[C], one, v[D]);                                                 \
    v[B] = rotr32(v[B] ^ v[C], 12);                                                  \
    v[A] = add_fma(v[A] + v[B], one, (m[kSigma[r % 10][2 * I + 1]] ^ kBlakeC[kSigma[r % 10][2 * I]]));  \
    v[D] = __byte_perm(v[D] ^ v[A], 0, 0x0321);                                      \
    v[C] = add_fma(v[C], one, v[D]);                                                 \
    v[B] = rotr32(v[B] ^ v[C], 7);
#pragma unroll
        for (int r = 0; r < 14; ++r) {
            HFUSE_BG(0, 4, 8, 12, 0) HFUSE_BG(1, 5, 9, 13, 1) HFUSE_BG(2, 6, 10, 14, 2) HFUSE_BG(3, 7, 11, 15, 3)
            HFUSE_BG(0, 5, 10, 15, 4) HFUSE_BG(1, 6, 11, 12, 5) HFUSE_BG(2, 7, 8, 13, 6) HFUSE_BG(3, 4, 9, 14, 7)
        }
#undef HFUSE_BG
#pragma unroll
        for (int i = 0; i < 8; ++i) d[i] = a.mid[i] ^ v[i] ^ v[i + 8];
    }
};

// ---------------------------------------------------------------------------
// Sia: BLAKE2b-256 of an 80-byte header, 64-bit nonce = message word 4
// ---------------------------------------------------------------------------
struct SiaArgs {
    SearchCommon c;
    unsigned long long m[10];   // header as little-endian u64 words (m[4] is replaced by the nonce)
};

__device__ __forceinline__ unsigned long long ror64(unsigned long long x, int n) {
    uint32_t lo = (uint32_t)x, hi = (uint32_t)(x >> 32);
    uint32_t rl, rh;
    if (n == 32) { rl = hi; rh = lo; }
    else if (n == 24) { rl = __byte_perm(lo, hi, 0x6543); rh = __byte_perm(lo, hi, 0x2107); }
    else if (n == 16) { rl = __byte_perm(lo, hi, 0x5432); rh = __byte_perm(lo, hi, 0x1076); }
    else if (n < 32) { rl = __funnelshift_r(lo, hi, n); rh = __funnelshift_r(hi, lo, n); }
    else { rl = __funnelshift_r(hi, lo, n - 32); rh = __funnelshift_r(lo, hi, n - 32); }
    return ((unsigned long long)rh << 32) | rl;
}

#define HFUSE_B2BIV_INIT { \
    0x6a09e667f3bcc908ull, 0xbb67ae8584caa73bull, 0x3c6ef372fe94f82bull, 0xa54ff53a5f1d36f1ull, \
    0x510e527fade682d1ull, 0x9b05688c2b3e6c1full, 0x1f83d9abfb41bd6bull, 0x5be0cd19137e2179ull}
static constexpr unsigned long long kB2bIV[8] = HFUSE_B2BIV_INIT;

struct SiaRole {
    using Args = SiaArgs;
    static constexpr bool kCooperative = false;

    static __device__ __forceinline__ void hash(const Args& a, unsigned long long nonce, uint32_t d[8]) {
        constexpr unsigned long long kB2bIV[8] = HFUSE_B2BIV_INIT;
        constexpr unsigned char kSigma[10][16] = HFUSE_SIGMA_INIT;
        const unsigned long long m[16] = {a.m[0], a.m[1], a.m[2], a.m[3], nonce, a.m[5], a.m[6], a.m[7],
                                          a.m[8], a.m[9], 0, 0, 0, 0, 0, 0};
        unsigned long long v[16];
        const unsigned long long h0 = kB2bIV[0] ^ 0x01010020ull;
        v[0] = h0;
#pragma unroll
        for (int i = 1; i < 8; ++i) v[i] = kB2bIV[i];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[8 + i] = kB2bIV[i];
        v[12] ^= 80ull;          // byte counter
        v[14] = ~v[14];          // last block
#define HFUSE_G2(A, B, C, D, X, Y)             \
    v[A] = v[A] + v[B] + m[X];                 \
    v[D] = ror64(v[D] ^ v[A], 32);             \
    v[C] = v[C] + v[D];                        \
    v[B] = ror64(v[B] ^ v[C], 24);             \
    v[A] = v[A] + v[B] + m[Y];                 \
    v[D] = ror64(v[D] ^ v[A], 16);             \
    v[C] = v[C] + v[D];                        \
    v[B] = ror64(v[B] ^ v[C], 63);
#pragma unroll
        for (int r = 0; r < 12; ++r) {
            HFUSE_G2(0, 4, 8, 12, kSigma[r % 10][0], kSigma[r % 10][1])
            HFUSE_G2(1, 5, 9, 13, kSigma[r % 10][2], kSigma[r % 10][3])
            HFUSE_G2(2, 6, 10, 14, kSigma[r % 10][4], kSigma[r % 10][5])
            HFUSE_G2(3, 7, 11, 15, kSigma[r % 10][6], kSigma[r % 10][7])
            HFUSE_G2(0, 5, 10, 15, kSigma[r % 10][8], kSigma[r % 10][9])
            HFUSE_G2(1, 6, 11, 12, kSigma[r % 10][10], kSigma[r % 10][11])
            HFUSE_G2(2, 7, 8, 13, kSigma[r % 10][12], kSigma[r % 10][13])
            HFUSE_G2(3, 4, 9, 14, kSigma[r % 10][14], kSigma[r % 10][15])
        }
#undef HFUSE_G2
        // digest bytes are the little-endian words h0..h3; as a big-endian integer the
        // most significant 32 bits are the byte-swapped low half of h0
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned long long h = (i == 0 ? h0 : kB2bIV[i]) ^ v[i] ^ v[i + 8];
            d[2 * i] = bswap32((uint32_t)h);
            d[2 * i + 1] = bswap32((uint32_t)(h >> 32));
        }
    }
};

// ---------------------------------------------------------------------------
// ethash
// ---------------------------------------------------------------------------
struct EthashArgs {
    SearchCommon c;
    const uint4* dag;               // dag_items x 128 bytes
    uint32_t dag_items;
    uint32_t pow2_mask;             // dag_items - 1 when dag_items is a power of two (index = hash & mask), else 0
    unsigned long long mod_magic;   // floor(2^64 / dag_items) + 1, for the division-free modulo
    unsigned long long header[4];   // header hash as little-endian u64 words
};

__device__ __forceinline__ unsigned long long rol64(unsigned long long x, int n) { return ror64(x, 64 - n); }

#define HFUSE_KECCAKRC_INIT { \
    0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808aull, 0x8000000080008000ull, \
    0x000000000000808bull, 0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull, \
    0x000000000000008aull, 0x0000000000000088ull, 0x0000000080008009ull, 0x000000008000000aull, \
    0x000000008000808bull, 0x800000000000008bull, 0x8000000000008089ull, 0x8000000000008003ull, \
    0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800aull, 0x800000008000000aull, \
    0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull}
static constexpr unsigned long long kKeccakRC[24] = HFUSE_KECCAKRC_INIT;

// Round constants in constant memory: the round loop is NOT unrolled.  ethash is bound by
// DAG reads, and 2 x 24 unrolled rounds of 64-bit lane arithmetic overflow the instruction
// cache (measured: 517 MH/s unrolled, 626 MH/s as a loop on B200).
static __device__ __constant__ unsigned long long kKeccakRCc[24] = HFUSE_KECCAKRC_INIT;

// Keccak-f[1600], lanes s[x + 5y]
__device__ __forceinline__ void keccak_f1600(unsigned long long s[25]) {
#pragma unroll 1
    for (int r = 0; r < 24; ++r) {
        unsigned long long c[5], t;
#pragma unroll
        for (int x = 0; x < 5; ++x) c[x] = s[x] ^ s[x + 5] ^ s[x + 10] ^ s[x + 15] ^ s[x + 20];
#pragma unroll
        for (int x = 0; x < 5; ++x) {
            t = c[(x + 4) % 5] ^ rol64(c[(x + 1) % 5], 1);
#pragma unroll
            for (int y = 0; y < 25; y += 5) s[y + x] ^= t;
        }
        // rho and pi along the 24-lane cycle that starts at lane 1
        t = s[1];
        unsigned long long u;
#define HFUSE_RP(DST, ROT) u = s[DST]; s[DST] = rol64(t, ROT); t = u;
        HFUSE_RP(10, 1)  HFUSE_RP(7, 3)   HFUSE_RP(11, 6)  HFUSE_RP(17, 10) HFUSE_RP(18, 15) HFUSE_RP(3, 21)
        HFUSE_RP(5, 28)  HFUSE_RP(16, 36) HFUSE_RP(8, 45)  HFUSE_RP(21, 55) HFUSE_RP(24, 2)  HFUSE_RP(4, 14)
        HFUSE_RP(15, 27) HFUSE_RP(23, 41) HFUSE_RP(19, 56) HFUSE_RP(13, 8)  HFUSE_RP(12, 25) HFUSE_RP(2, 43)
        HFUSE_RP(20, 62) HFUSE_RP(14, 18) HFUSE_RP(22, 39) HFUSE_RP(9, 61)  HFUSE_RP(6, 20)  HFUSE_RP(1, 44)
#undef HFUSE_RP
#pragma unroll
        for (int y = 0; y < 25; y += 5) {
            const unsigned long long a0 = s[y], a1 = s[y + 1], a2 = s[y + 2], a3 = s[y + 3], a4 = s[y + 4];
            s[y] = a0 ^ (~a1 & a2); s[y + 1] = a1 ^ (~a2 & a3); s[y + 2] = a2 ^ (~a3 & a4);
            s[y + 3] = a3 ^ (~a4 & a0); s[y + 4] = a4 ^ (~a0 & a1);
        }
        s[0] ^= kKeccakRCc[r];
    }
}

__device__ __forceinline__ uint32_t fnv1(uint32_t a, uint32_t b) { return (a * 0x01000193u) ^ b; }

// x mod d without a divide: with M = floor(2^64/d)+1, x mod d = hi64((M*x mod 2^64) * d)
__device__ __forceinline__ uint32_t fastmod(uint32_t x, unsigned long long magic, uint32_t d) {
    return (uint32_t)__umul64hi(magic * x, (unsigned long long)d);
}

struct EthashRole {
    using Args = EthashArgs;
    static constexpr bool kCooperative = true;
    static constexpr int kLanes = 8;      // threads that share one 128-byte DAG item
    static constexpr int kParallel = 4;   // hashes one 8-lane group walks at the same time

    // Executed by whole warps.  Each thread owns one nonce; groups of eight
    // lanes walk the DAG for each other's nonces so that every DAG read is one
    // coalesced 128-byte line (16 bytes per lane).
    static __device__ __forceinline__ void hash(const Args& a, unsigned long long nonce, uint32_t d[8],
                                                uint32_t mix_out[8]) {
        // a power-of-two item count turns the index reduction into a mask (six instructions fewer
        // per DAG access; the walk's instructions are what the board's power goes to)
        if (a.pow2_mask) hash_impl<true>(a, nonce, d, mix_out);
        else hash_impl<false>(a, nonce, d, mix_out);
    }

    template <bool POW2>
    static __device__ __forceinline__ void hash_impl(const Args& a, unsigned long long nonce, uint32_t d[8],
                                                     uint32_t mix_out[8]) {
        unsigned long long st[25];
#pragma unroll
        for (int i = 0; i < 4; ++i) st[i] = a.header[i];
        st[4] = nonce;
        st[5] = 0x0000000000000001ull;
#pragma unroll
        for (int i = 6; i < 25; ++i) st[i] = 0;
        st[8] = 0x8000000000000000ull;
        keccak_f1600(st);                       // Keccak-512(header || nonce): st[0..7]

        const int g = threadIdx.x & (kLanes - 1);
        uint32_t seed[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) { seed[2 * i] = (uint32_t)st[i]; seed[2 * i + 1] = (uint32_t)(st[i] >> 32); }

#pragma unroll 1
        for (int p = 0; p < kLanes; p += kParallel) {
            uint4 mix[kParallel];
            uint32_t init0[kParallel];
#pragma unroll
            for (int i = 0; i < kParallel; ++i) {
                uint32_t sh[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) sh[j] = __shfl_sync(0xffffffffu, seed[j], p + i, kLanes);
                init0[i] = sh[0];
                // the 128-byte mix is the 64-byte seed twice; lane g holds words 4g..4g+3
                switch (g & 3) {
                case 0: mix[i] = make_uint4(sh[0], sh[1], sh[2], sh[3]); break;
                case 1: mix[i] = make_uint4(sh[4], sh[5], sh[6], sh[7]); break;
                case 2: mix[i] = make_uint4(sh[8], sh[9], sh[10], sh[11]); break;
                default: mix[i] = make_uint4(sh[12], sh[13], sh[14], sh[15]); break;
                }
            }
#pragma unroll 1
            for (uint32_t acc = 0; acc < 64; acc += 4) {
                const int owner = (acc >> 2) & (kLanes - 1);   // lane holding mix words acc..acc+3 (mod 32)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    uint32_t idx[kParallel];
#pragma unroll
                    for (int i = 0; i < kParallel; ++i) {
                        const uint32_t word = b == 0 ? mix[i].x : b == 1 ? mix[i].y : b == 2 ? mix[i].z : mix[i].w;
                        const uint32_t h = fnv1(init0[i] ^ (acc + b), word);
                        idx[i] = POW2 ? (h & a.pow2_mask) : fastmod(h, a.mod_magic, a.dag_items);
                        idx[i] = __shfl_sync(0xffffffffu, idx[i], owner, kLanes);
                    }
                    uint4 item[kParallel];
#pragma unroll
                    for (int i = 0; i < kParallel; ++i) item[i] = __ldg(a.dag + (size_t)idx[i] * 8 + g);
#pragma unroll
                    for (int i = 0; i < kParallel; ++i) {
                        mix[i].x = fnv1(mix[i].x, item[i].x); mix[i].y = fnv1(mix[i].y, item[i].y);
                        mix[i].z = fnv1(mix[i].z, item[i].z); mix[i].w = fnv1(mix[i].w, item[i].w);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kParallel; ++i) {
                const uint32_t folded = fnv1(fnv1(fnv1(mix[i].x, mix[i].y), mix[i].z), mix[i].w);
                uint32_t cm[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) cm[j] = __shfl_sync(0xffffffffu, folded, j, kLanes);
                if (g == p + i) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) mix_out[j] = cm[j];
                }
            }
        }
        // Keccak-256(seed || mix digest)
#pragma unroll
        for (int i = 0; i < 8; ++i) st[i] = ((unsigned long long)seed[2 * i + 1] << 32) | seed[2 * i];
#pragma unroll
        for (int i = 0; i < 4; ++i) st[8 + i] = ((unsigned long long)mix_out[2 * i + 1] << 32) | mix_out[2 * i];
        st[12] = 0x0000000000000001ull;
#pragma unroll
        for (int i = 13; i < 25; ++i) st[i] = 0;
        st[16] = 0x8000000000000000ull;
        keccak_f1600(st);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            d[2 * i] = bswap32((uint32_t)st[i]);
            d[2 * i + 1] = bswap32((uint32_t)(st[i] >> 32));
        }
    }
};

// ---------------------------------------------------------------------------
// The sweep every hash shares.
//   run()   : grid-stride loop over the nonce range (standalone kernels); the trip count is
//             uniform per block because ethash lanes must stay together.
//   drain() : work-queue form used by the fused pairs.  Warps take chunks of nonces from a
//             cursor kept in hfuse_hits::reserved (zeroed by hfuse_hits_reset) until the range is
//             used up.  A thread range first drains its own hash's queue and then the other
//             one's, so both ranges finish together whatever the cost ratio of the two hashes.
// ---------------------------------------------------------------------------
template <class H> struct NonceIs32 { static constexpr bool value = false; };
template <> struct NonceIs32<Sha256dRole> { static constexpr bool value = true; };
template <> struct NonceIs32<Blake256Role> { static constexpr bool value = true; };

template <class Hash>
struct SearchRole {
    using Args = typename Hash::Args;
    static int smem_bytes(const Args&, int) { return 0; }
    static int plan(Args&, int, int) { return 0; }

    // nonce number i of the sweep; every lane of a warp must call this together (ethash)
    static __device__ __forceinline__ void one(const Args& a, unsigned long long i, bool live) {
        const SearchCommon& c = a.c;
        unsigned long long nonce = c.start + (live ? i : 0);
        uint32_t d[8], mix[8];
        if constexpr (Hash::kCooperative) {
            Hash::hash(a, nonce, d, mix);
        } else {
            if (!live) return;
            if constexpr (NonceIs32<Hash>::value) { nonce = (uint32_t)nonce; Hash::hash(a, (uint32_t)nonce, d); }
            else Hash::hash(a, nonce, d);
        }
        if (!live) return;
        if (c.out32) {
            write_digest_be(c.out32, i, d);
            if (Hash::kCooperative && c.mix32) {
                uint32_t* p = reinterpret_cast<uint32_t*>(c.mix32 + 32 * i);
#pragma unroll
                for (int k = 0; k < 8; ++k) p[k] = mix[k];
            }
        } else if (d[0] <= c.target[0] && below_target(d, c.target)) {
            record_hit(c.hits, nonce, Hash::kCooperative ? mix : nullptr);
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        const unsigned long long stride = (unsigned long long)ctx.nblocks * T;
        for (unsigned long long base = (unsigned long long)ctx.block * T; base < a.c.count; base += stride) {
            const unsigned long long i = base + ctx.tid;
            one(a, i, i < a.c.count);
        }
    }

    static __device__ __forceinline__ void drain(const Args& a, unsigned chunk) {
        const unsigned lane = threadIdx.x & 31;
        const unsigned long long nchunks = (a.c.count + chunk - 1) / chunk;
        for (;;) {
            unsigned ci = 0;
            if (lane == 0) ci = atomicAdd(&a.c.hits->reserved, 1u);
            ci = __shfl_sync(0xffffffffu, ci, 0);
            if (ci >= nchunks) break;          // every warp overshoots the cursor once, then stops
            const unsigned long long lo = (unsigned long long)ci * chunk;
            const unsigned long long hi = lo + chunk < a.c.count ? lo + chunk : a.c.count;
            for (unsigned long long base = lo; base < hi; base += 32) {
                const unsigned long long i = base + lane;
                one(a, i, i < hi);
            }
        }
    }
};

}  // namespace hfuse
