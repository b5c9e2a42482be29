"""Seeded synthetic inputs for the five benchmark configurations.

The reference measures on arbitrary tensors and nonces (its harness is not
part of its tree), so these generators only fix shapes, distributions and
seeds.  Choices the configuration text leaves open are fixed here:
  - "N(0.5, 2.0)" is read as mean 0.5, standard deviation 2.0;
  - byte strings (headers, header hash, DAG) come from xoshiro256** whose
    state is four splitmix64 outputs of the seed, emitted as little-endian
    64-bit words (`hfuse_xoshiro256ss_fill`); a configuration draws its
    strings from ONE stream in the order listed in the function;
  - tensors come from `torch.manual_seed(seed)` on the CPU generator, drawn in
    the order listed, then (optionally) copied to the device.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib


def xoshiro_bytes(seed: int, nbytes: int) -> np.ndarray:
    buf = np.empty(nbytes, dtype=np.uint8)
    _lib.lib().hfuse_xoshiro256ss_fill(seed, buf.ctypes.data, nbytes)
    return buf


def _dev(t, device):
    return t.to(device) if device is not None else t


def config0(device=None, batch=16):
    """im2col [B,64,56,56] k3 p1 s1 d1  +  max-pool [B,64,112,112] k2 s2; U(-1,1); seed 0."""
    torch.manual_seed(0)
    im = torch.rand(batch, 64, 56, 56) * 2 - 1
    pool = torch.rand(batch, 64, 112, 112) * 2 - 1
    return {"im": _dev(im, device), "pool": _dev(pool, device),
            "im2col": dict(kernel_size=3, padding=1, stride=1, dilation=1),
            "maxpool": dict(kernel_size=2, stride=2),
            "bytes": batch * (64 * 56 * 56 * 4 * 10 + 64 * 112 * 112 * 4 + 64 * 56 * 56 * 12)}


def config1(device=None, bn_batch=32, up_batch=16, seed=1):
    """BN statistics [B1,256,28,28] ~ 0.5 + 2.0*randn, eps 1e-5  +  bilinear x2 [B2,128,56,56] U(0,1); seed 1.
    (Another seed gives another draw of the same distributions: the batch shards of a multi-GPU run.)"""
    torch.manual_seed(seed)
    bn = 0.5 + 2.0 * torch.randn(bn_batch, 256, 28, 28)
    up = torch.rand(up_batch, 128, 56, 56)
    return {"bn": _dev(bn, device), "up": _dev(up, device), "eps": 1e-5,
            "bytes": bn_batch * 256 * 784 * 4 + 2048 + up_batch * 128 * 56 * 56 * 4 * 5}


def config2(device=None, n_hist=1 << 24, batch=32):
    """histc over n_hist N(0,1) values, 256 bins on [-4,4]  +  im2col as config 0 with batch 32; seed 2."""
    torch.manual_seed(2)
    hist = torch.randn(n_hist)
    im = torch.rand(batch, 64, 56, 56) * 2 - 1
    return {"hist": _dev(hist, device), "im": _dev(im, device), "bins": 256, "lo": -4.0, "hi": 4.0,
            "im2col": dict(kernel_size=3, padding=1, stride=1, dilation=1),
            "bytes": n_hist * 4 + 1024 + batch * 64 * 56 * 56 * 4 * 10}


def config3(seed=3):
    """BLAKE-256 + SHA-256d: two 80-byte headers (BLAKE first), target 2^256/2^32, 2^32 nonces."""
    b = xoshiro_bytes(seed * 1000 + 3, 160).tobytes()
    return {"blake_header": b[:80], "sha_header": b[80:160], "target": (1 << 224).to_bytes(32, "big"),
            "start": 0, "count": 1 << 32}


def config4(device=None, dag_items=8_388_608, seed=3):
    """ethash + Sia: DAG = dag_items x 128 bytes of xoshiro256**(seed); then, from xoshiro256**(seed*1000+4):
    32-byte header hash, 80-byte Sia header.  Boundary 2^256/2^24, 2^30 nonces."""
    dag = torch.from_numpy(xoshiro_bytes(seed, dag_items * 128))
    b = xoshiro_bytes(seed * 1000 + 4, 112).tobytes()
    return {"dag": _dev(dag, device), "header_hash": b[:32], "sia_header": b[32:112],
            "target": (1 << 232).to_bytes(32, "big"), "start": 0, "count": 1 << 30}
