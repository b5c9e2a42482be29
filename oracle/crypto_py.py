"""Second, independent pure-Python restatement of the crypto algorithms.

TEST INFRASTRUCTURE ONLY (see oracle/crypto_oracle.c for the scope note and
the "parity unpinned" status: the reference, aoli-al/HFuse, names these hashes
in configs/crypto_kernels.yaml:1-32 but ships neither their code nor any
known-answer vectors).  This file is written separately from the C oracle, in
a different style (table-driven, Python big integers), so that an error shared
by both is unlikely; the tests require the two to agree on random inputs and
require each to reproduce hashlib / specification digests where those exist.

Slow by design: use it on a handful of inputs only.
"""
from __future__ import annotations

import struct

M32 = 0xFFFFFFFF
M64 = 0xFFFFFFFFFFFFFFFF


def _rotr32(x, n):
    return ((x >> n) | (x << (32 - n))) & M32


def _rotl64(x, n):
    n %= 64
    return ((x << n) | (x >> (64 - n))) & M64 if n else x


# ---------------------------------------------------------------- xoshiro256**
def splitmix64_stream(seed):
    x = seed & M64
    while True:
        x = (x + 0x9E3779B97F4A7C15) & M64
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        yield z ^ (z >> 31)


def xoshiro256ss_bytes(seed: int, nbytes: int) -> bytes:
    """State = four splitmix64(seed) outputs; output = little-endian u64 stream."""
    sm = splitmix64_stream(seed)
    s = [next(sm) for _ in range(4)]
    out = bytearray()
    while len(out) < nbytes:
        r = (_rotl64((s[1] * 5) & M64, 7) * 9) & M64
        t = (s[1] << 17) & M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl64(s[3], 45)
        out += struct.pack("<Q", r)
    return bytes(out[:nbytes])


# ---------------------------------------------------------------- BLAKE-256
_PI = [0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0, 0x082EFA98, 0xEC4E6C89,
       0x452821E6, 0x38D01377, 0xBE5466CF, 0x34E90C6C, 0xC0AC29B7, 0xC97C50DD, 0x3F84D5B5, 0xB5470917]
_IV256 = [0x6A09E667, 0xBB67AE85, 0x3C6EF372, 0xA54FF53A, 0x510E527F, 0x9B05688C, 0x1F83D9AB, 0x5BE0CD19]
_SIGMA = [
    [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15],
    [14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3],
    [11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4],
    [7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8],
    [9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13],
    [2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9],
    [12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11],
    [13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10],
    [6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5],
    [10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0],
]
_QUADS = [(0, 4, 8, 12), (1, 5, 9, 13), (2, 6, 10, 14), (3, 7, 11, 15),
          (0, 5, 10, 15), (1, 6, 11, 12), (2, 7, 8, 13), (3, 4, 9, 14)]


def _blake256_block(h, block, t):
    m = struct.unpack(">16I", block)
    v = list(h) + _PI[:4] + [(t & M32) ^ _PI[4], (t & M32) ^ _PI[5], (t >> 32) ^ _PI[6], (t >> 32) ^ _PI[7]]
    for r in range(14):
        s = _SIGMA[r % 10]
        for i, (a, b, c, d) in enumerate(_QUADS):
            j, k = s[2 * i], s[2 * i + 1]
            v[a] = (v[a] + v[b] + (m[j] ^ _PI[k])) & M32
            v[d] = _rotr32(v[d] ^ v[a], 16)
            v[c] = (v[c] + v[d]) & M32
            v[b] = _rotr32(v[b] ^ v[c], 12)
            v[a] = (v[a] + v[b] + (m[k] ^ _PI[j])) & M32
            v[d] = _rotr32(v[d] ^ v[a], 8)
            v[c] = (v[c] + v[d]) & M32
            v[b] = _rotr32(v[b] ^ v[c], 7)
    return [h[i] ^ v[i] ^ v[i + 8] for i in range(8)]


def blake256(msg: bytes) -> bytes:
    bits = len(msg) * 8
    # pad to 447 mod 512 with 1 0*, then a single 1 bit, then the 64-bit length
    padded = bytearray(msg) + b"\x80"
    while len(padded) % 64 != 56:
        padded.append(0)
    padded[-1] |= 0x01
    padded += struct.pack(">Q", bits)
    h = list(_IV256)
    nblocks = len(padded) // 64
    for i in range(nblocks):
        # counter = message bits hashed up to and including this block; zero
        # for a block that carries padding only
        upto = min(bits, (i + 1) * 512)
        carries_msg = i * 512 < bits
        h = _blake256_block(h, bytes(padded[64 * i:64 * i + 64]), upto if carries_msg else 0)
    return struct.pack(">8I", *h)


# ---------------------------------------------------------------- Keccak
def _keccak_f(lanes):
    """lanes[x][y], 24 rounds; round constants from the LFSR, offsets from the
    (t+1)(t+2)/2 walk, as the Keccak reference describes them."""
    R = 1
    for _ in range(24):
        C = [lanes[x][0] ^ lanes[x][1] ^ lanes[x][2] ^ lanes[x][3] ^ lanes[x][4] for x in range(5)]
        D = [C[(x + 4) % 5] ^ _rotl64(C[(x + 1) % 5], 1) for x in range(5)]
        lanes = [[lanes[x][y] ^ D[x] for y in range(5)] for x in range(5)]
        (x, y) = (1, 0)
        cur = lanes[x][y]
        for t in range(24):
            (x, y) = (y, (2 * x + 3 * y) % 5)
            cur, lanes[x][y] = lanes[x][y], _rotl64(cur, (t + 1) * (t + 2) // 2)
        for y in range(5):
            T = [lanes[x][y] for x in range(5)]
            for x in range(5):
                lanes[x][y] = T[x] ^ ((~T[(x + 1) % 5]) & M64 & T[(x + 2) % 5])
        for j in range(7):
            R = ((R << 1) ^ ((R >> 7) * 0x71)) % 256
            if R & 2:
                lanes[0][0] ^= 1 << ((1 << j) - 1)
    return lanes


def keccak(msg: bytes, rate: int, pad: int, outlen: int) -> bytes:
    state = bytearray(200)
    padded = bytearray(msg)
    q = rate - (len(msg) % rate)
    padded += bytes([pad]) + bytes(q - 1)
    padded[-1] |= 0x80
    for off in range(0, len(padded), rate):
        for i in range(rate):
            state[i] ^= padded[off + i]
        lanes = [[struct.unpack_from("<Q", state, 8 * (x + 5 * y))[0] for y in range(5)] for x in range(5)]
        lanes = _keccak_f(lanes)
        for x in range(5):
            for y in range(5):
                struct.pack_into("<Q", state, 8 * (x + 5 * y), lanes[x][y])
    return bytes(state[:outlen])


def keccak256(msg):
    return keccak(msg, 136, 0x01, 32)


def keccak512(msg):
    return keccak(msg, 72, 0x01, 64)


# ---------------------------------------------------------------- ethash
def _fnv(a, b):
    return ((a * 0x01000193) & M32) ^ b


def hashimoto(dag: bytes, n_items: int, header_hash: bytes, nonce: int):
    """Returns (mix_digest, result).  dag = n_items x 128 bytes."""
    seed = keccak512(header_hash + struct.pack("<Q", nonce))
    s = struct.unpack("<16I", seed)
    mix = list(s) * 2
    for i in range(64):
        p = _fnv(i ^ s[0], mix[i % 32]) % n_items
        item = struct.unpack_from("<32I", dag, 128 * p)
        mix = [_fnv(a, b) for a, b in zip(mix, item)]
    cmix = []
    for i in range(0, 32, 4):
        cmix.append(_fnv(_fnv(_fnv(mix[i], mix[i + 1]), mix[i + 2]), mix[i + 3]))
    mix_digest = struct.pack("<8I", *cmix)
    return mix_digest, keccak256(seed + mix_digest)


def ethash_cache(seed: bytes, n: int) -> list:
    """Light cache as a list of n 64-byte strings (sequential by construction)."""
    o = [keccak512(seed)]
    for _ in range(1, n):
        o.append(keccak512(o[-1]))
    for _ in range(3):
        for i in range(n):
            v = struct.unpack_from("<I", o[i])[0] % n
            o[i] = keccak512(bytes(a ^ b for a, b in zip(o[(i - 1 + n) % n], o[v])))
    return o


def ethash_dataset_node(cache: list, i: int) -> bytes:
    n = len(cache)
    mix = list(struct.unpack("<16I", cache[i % n]))
    mix[0] ^= i
    mix = list(struct.unpack("<16I", keccak512(struct.pack("<16I", *mix))))
    for j in range(256):
        parent = struct.unpack("<16I", cache[_fnv(i ^ j, mix[j % 16]) % n])
        mix = [_fnv(a, b) for a, b in zip(mix, parent)]
    return keccak512(struct.pack("<16I", *mix))
