"""Python call harness for the nonce searches and their fused pairs.

Plays the part of the reference's `build/fuse/fuser` binary (README.md:101 of
aoli-al/HFuse), which launches each hash kernel and each fused pair over a
block of nonces.  A search is described by a small object (`Blake256`,
`Sha256d`, `Sia`, `Ethash`) holding its header, nonce range, target and a
device-side result record; `run(s)` launches the standalone kernel,
`run_pair(a, b)` the fused pair named after the two halves (the six pairs of
the reference's configs/crypto_fusion.yaml).  Everything executes on the GPU
through the C ABI; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib

KIND = {"blake256": 0, "sha256d": 1, "sia": 2, "ethash": 3}


def target_from_difficulty_bits(bits: int) -> bytes:
    """The 32-byte big-endian target 2^256 / 2^bits."""
    return (1 << (256 - bits)).to_bytes(32, "big")


def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class _Search:
    key = ""
    nonce_bits = 64

    def __init__(self, header: bytes, start: int, count: int, target: bytes, device=None):
        if len(header) != self.header_len:
            raise ValueError(f"{self.key}: header must be {self.header_len} bytes")
        if len(target) != 32:
            raise ValueError("target must be 32 bytes (big-endian)")
        if count < 0 or start < 0:
            raise ValueError("start and count must be non-negative")
        if not torch.cuda.is_available():
            raise RuntimeError("hfuse_b200 has no CPU path: a CUDA device is required")
        self.header, self.start, self.count, self.target = bytes(header), int(start), int(count), bytes(target)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.hits = torch.zeros(C.sizeof(_lib.Hits), dtype=torch.uint8, device=self.device)

    def reset(self, stream=None):
        _lib.check(_lib.lib().hfuse_hits_reset(self.hits.data_ptr(), _stream_ptr(stream)), "hfuse_hits_reset")

    def c_args(self):
        return [self.header, self.start & (2 ** 64 - 1), self.count, self.target, self.hits.data_ptr()]

    def result(self):
        """(total hit count, sorted list of (nonce, mix digest bytes)).  Synchronises."""
        raw = self.hits.cpu().numpy().tobytes()
        h = _lib.Hits.from_buffer_copy(raw)
        n = min(h.count, _lib.HFUSE_MAX_HITS)
        out = sorted((int(h.nonce[i]), bytes(np.array(h.mix[i][:], dtype="<u4").tobytes())) for i in range(n))
        return h.count, out

    def nonces(self):
        return [n for n, _ in self.result()[1]]


class Blake256(_Search):
    """BLAKE-256 (14 rounds) over an 80-byte header, 32-bit LE nonce at bytes 76..79."""
    key, header_len, nonce_bits = "blake256", 80, 32


class Sha256d(_Search):
    """SHA-256(SHA-256(header80)), 32-bit LE nonce at bytes 76..79."""
    key, header_len, nonce_bits = "sha256d", 80, 32


class Sia(_Search):
    """BLAKE2b-256 over an 80-byte header, 64-bit LE nonce at bytes 32..39."""
    key, header_len, nonce_bits = "sia", 80, 64


class Ethash(_Search):
    """ethash hashimoto over a device-resident DAG of 128-byte items."""
    key, header_len, nonce_bits = "ethash", 32, 64

    def __init__(self, dag: torch.Tensor, header_hash: bytes, start: int, count: int, target: bytes):
        if not dag.is_cuda or dag.dtype != torch.uint8 or not dag.is_contiguous() or dag.numel() % 128:
            raise ValueError("dag must be a contiguous CUDA uint8 tensor of n*128 bytes")
        super().__init__(header_hash, start, count, target, dag.device)
        self.dag = dag

    def c_args(self):
        return [self.dag.data_ptr(), self.dag.numel() // 128, self.header, self.start & (2 ** 64 - 1),
                self.count, self.target, self.hits.data_ptr()]


def run(s: _Search, stream=None, reset=True):
    if reset:
        s.reset(stream)
    fn = getattr(_lib.lib(), _lib.CRYPTO_SOLO[s.key])
    _lib.check(fn(*s.c_args(), _stream_ptr(stream)), _lib.CRYPTO_SOLO[s.key])
    return s


def pair_name(a: _Search, b: _Search) -> str:
    name = f"{a.key}_{b.key}"
    if name not in _lib.CRYPTO_PAIRS:
        raise KeyError(f"no fused pair {name}; the pairs are {sorted(_lib.CRYPTO_PAIRS)}")
    return name


def run_pair(a: _Search, b: _Search, stream=None, reset=True):
    """Launch the fused pair (a, b) as ONE kernel."""
    name = pair_name(a, b)
    if reset:
        a.reset(stream)
        b.reset(stream)
    fn = getattr(_lib.lib(), f"hfuse_{name}_search")
    _lib.check(fn(*a.c_args(), *b.c_args(), _stream_ptr(stream)), f"hfuse_{name}_search")
    return a, b


def run_back_to_back(a: _Search, b: _Search, stream=None, reset=True):
    """The unfused baseline: both standalone kernels queued on one stream."""
    return run(a, stream, reset), run(b, stream, reset)


def hash_batch(kind: str, header: bytes, start: int, count: int, dag: torch.Tensor | None = None):
    """Digests (and ethash mix digests) of `count` consecutive nonces, computed on the GPU.
    Returns uint8 arrays [count,32] (digest) and [count,32] (mix, ethash only, else None)."""
    dev = dag.device if dag is not None else torch.device("cuda", torch.cuda.current_device())
    out = torch.empty((count, 32), dtype=torch.uint8, device=dev)
    mix = torch.empty((count, 32), dtype=torch.uint8, device=dev) if kind == "ethash" else None
    _lib.check(_lib.lib().hfuse_hash_batch(
        KIND[kind], bytes(header), dag.data_ptr() if dag is not None else None,
        dag.numel() // 128 if dag is not None else 0, start & (2 ** 64 - 1), count, out.data_ptr(),
        mix.data_ptr() if mix is not None else None, _stream_ptr()), "hfuse_hash_batch")
    return out.cpu().numpy(), (mix.cpu().numpy() if mix is not None else None)


def make_cache(seed: bytes, cache_nodes: int) -> np.ndarray:
    """ethash light cache (cache_nodes x 64 bytes), built on the host: it is a sequential chain."""
    if len(seed) != 32:
        raise ValueError("seed must be 32 bytes")
    out = np.empty(64 * cache_nodes, dtype=np.uint8)
    _lib.check(_lib.lib().hfuse_ethash_make_cache(bytes(seed), cache_nodes, out.ctypes.data), "hfuse_ethash_make_cache")
    return out


def generate_dag(cache: torch.Tensor, n_nodes: int, chunks: int = 1) -> torch.Tensor:
    """DAG of n_nodes 64-byte nodes from a device-resident cache, in `chunks` launches
    (the reference's binary uses 16).  Returns a uint8 tensor of n_nodes * 64 bytes."""
    if not cache.is_cuda or cache.dtype != torch.uint8 or cache.numel() % 64:
        raise ValueError("cache must be a CUDA uint8 tensor of n*64 bytes")
    dag = torch.empty(n_nodes * 64, dtype=torch.uint8, device=cache.device)
    per = (n_nodes + chunks - 1) // chunks
    for first in range(0, n_nodes, per):
        cnt = min(per, n_nodes - first)
        _lib.check(_lib.lib().hfuse_ethash_generate_dag(cache.data_ptr(), cache.numel() // 64, dag.data_ptr(), first,
                                                        cnt, _stream_ptr()), "hfuse_ethash_generate_dag")
    return dag
