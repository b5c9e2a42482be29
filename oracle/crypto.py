"""ctypes front-end of the C crypto oracle (oracle/crypto_oracle.c).

TEST INFRASTRUCTURE ONLY.  Builds `liboracle_crypto.so` with the Makefile
beside it when the library is missing or older than its source.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle_crypto.so")
_SRC = os.path.join(_HERE, "crypto_oracle.c")

KIND_BLAKE256, KIND_SHA256D, KIND_SIA, KIND_ETHASH = 0, 1, 2, 3


def build(force: bool = False) -> str:
    stale = (not os.path.exists(_SO)) or (
        os.path.exists(_SRC) and os.path.getmtime(_SRC) > os.path.getmtime(_SO))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle_crypto.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        u8p, u64p = ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64)
        _lib.oracle_search.restype = ctypes.c_int
        _lib.oracle_search.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32,
                                       ctypes.c_uint64, ctypes.c_uint64, u8p, u64p, ctypes.c_void_p,
                                       ctypes.c_int, ctypes.c_int]
        _lib.oracle_xoshiro256ss_fill.argtypes = [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_size_t]
        _lib.oracle_keccak.argtypes = [u8p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_uint8,
                                       ctypes.c_void_p, ctypes.c_size_t]
        _lib.oracle_ethash_hashimoto.argtypes = [ctypes.c_void_p, ctypes.c_uint32, u8p, ctypes.c_uint64,
                                                 ctypes.c_void_p, ctypes.c_void_p]
        _lib.oracle_ethash_mkcache.argtypes = [u8p, ctypes.c_uint32, ctypes.c_void_p]
        _lib.oracle_ethash_dataset.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                               ctypes.c_void_p]
        _lib.oracle_blake2b.argtypes = [u8p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
        for name in ("oracle_sha256", "oracle_blake256"):
            getattr(_lib, name).argtypes = [u8p, ctypes.c_size_t, ctypes.c_void_p]
        for name in ("oracle_sha256d_header", "oracle_blake256_header"):
            getattr(_lib, name).argtypes = [u8p, ctypes.c_uint32, ctypes.c_void_p]
        _lib.oracle_sia_header.argtypes = [u8p, ctypes.c_uint64, ctypes.c_void_p]
    return _lib


def _out(n=32):
    return ctypes.create_string_buffer(n)


def xoshiro_bytes(seed: int, nbytes: int) -> np.ndarray:
    buf = np.empty(nbytes, dtype=np.uint8)
    lib().oracle_xoshiro256ss_fill(seed, buf.ctypes.data, nbytes)
    return buf


def sha256(msg: bytes) -> bytes:
    o = _out()
    lib().oracle_sha256(msg, len(msg), o)
    return o.raw


def blake256(msg: bytes) -> bytes:
    o = _out()
    lib().oracle_blake256(msg, len(msg), o)
    return o.raw


def blake2b(msg: bytes, outlen: int = 32) -> bytes:
    o = _out(outlen)
    lib().oracle_blake2b(msg, len(msg), o, outlen)
    return o.raw


def keccak(msg: bytes, rate: int, pad: int, outlen: int) -> bytes:
    o = _out(outlen)
    lib().oracle_keccak(msg, len(msg), rate, pad, o, outlen)
    return o.raw


def sha256d_header(header: bytes, nonce: int) -> bytes:
    o = _out()
    lib().oracle_sha256d_header(header, nonce & 0xFFFFFFFF, o)
    return o.raw


def blake256_header(header: bytes, nonce: int) -> bytes:
    o = _out()
    lib().oracle_blake256_header(header, nonce & 0xFFFFFFFF, o)
    return o.raw


def sia_header(header: bytes, nonce: int) -> bytes:
    o = _out()
    lib().oracle_sia_header(header, nonce, o)
    return o.raw


def hashimoto(dag: np.ndarray, header_hash: bytes, nonce: int):
    """dag: uint8 array of n_items*128 bytes.  Returns (mix_digest, result)."""
    assert dag.dtype == np.uint8 and dag.size % 128 == 0 and dag.flags.c_contiguous
    mix, res = _out(), _out()
    lib().oracle_ethash_hashimoto(dag.ctypes.data, dag.size // 128, header_hash, nonce, mix, res)
    return mix.raw, res.raw


def ethash_cache(seed: bytes, n_nodes: int) -> np.ndarray:
    """Light cache of n_nodes 64-byte nodes."""
    out = np.empty(64 * n_nodes, dtype=np.uint8)
    lib().oracle_ethash_mkcache(seed, n_nodes, out.ctypes.data)
    return out


def ethash_dataset(cache: np.ndarray, first: int, count: int) -> np.ndarray:
    """DAG nodes [first, first+count) of 64 bytes each."""
    out = np.empty(64 * count, dtype=np.uint8)
    lib().oracle_ethash_dataset(cache.ctypes.data, cache.size // 64, first, count, out.ctypes.data)
    return out


def search(kind: int, header: bytes, start: int, count: int, target: bytes,
           dag: np.ndarray | None = None, max_hits: int = 4096, threads: int = 0):
    """Sweep `count` nonces from `start`.  Returns (total_found, nonces[, mixes]) with the
    stored hits sorted by nonce.  kind 0/1 wrap the nonce to 32 bits."""
    nonces = (ctypes.c_uint64 * max_hits)()
    mixes = np.zeros((max_hits, 32), dtype=np.uint8)
    dag_ptr, n_items = (None, 0)
    if kind == KIND_ETHASH:
        assert dag is not None
        dag_ptr, n_items = dag.ctypes.data, dag.size // 128
    hdr = ctypes.create_string_buffer(bytes(header), len(header))
    found = lib().oracle_search(kind, ctypes.addressof(hdr), dag_ptr, n_items, start, count,
                                bytes(target), nonces, mixes.ctypes.data, max_hits, threads)
    n = min(found, max_hits)
    out_n = [int(nonces[i]) for i in range(n)]
    if kind == KIND_ETHASH:
        return found, out_n, [bytes(mixes[i]) for i in range(n)]
    return found, out_n


def num_threads() -> int:
    return lib().oracle_num_threads()
