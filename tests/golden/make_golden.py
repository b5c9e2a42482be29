"""Regenerates the golden fixtures in this directory from the CPU oracle.

Run from the repository root:  python tests/golden/make_golden.py

The reference ships no golden vectors, so these fixtures pin the oracle
itself: once committed, both the oracle (CPU tests) and the CUDA kernels (GPU
tests) must keep reproducing them bit for bit.  Inputs are seeded here and
stored next to the outputs, so the fixtures do not depend on any generator.

  dl_small.npz      small-shape inputs and outputs of the five DL operators
                    (odd sizes, padding, dilation, ties, NaN, -inf planes, bin edges)
  crypto_kat.json   digests of fixed headers / nonces for the four hashes, a
                    4099-item DAG hashimoto table, and hit lists of short sweeps
"""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import crypto as OC  # noqa: E402
from oracle import dl  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

IM2COL_CASES = [(3, 3, 1, 1, 1, 1, 1, 1), (2, 3, 0, 2, 2, 1, 1, 2), (3, 2, 2, 1, 1, 3, 2, 1), (1, 1, 0, 0, 1, 1, 1, 1)]
POOL_CASES = [(2, 2, 2, 2, 0, 0, 1, 1), (3, 3, 2, 1, 1, 1, 1, 1), (2, 3, 1, 2, 1, 1, 2, 1)]
UP_CASES = [(14, 18, False), (14, 18, True), (10, 13, False), (5, 20, True)]
HIST_CASES = [(10, -1.0, 1.0), (100, -3.0, 2.5), (256, -4.0, 4.0)]


def make_dl():
    g = torch.Generator().manual_seed(1234)
    out = {}
    x = torch.rand(2, 3, 9, 12, generator=g) * 2 - 1
    out["im2col_x"] = x.numpy()
    for i, p in enumerate(IM2COL_CASES):
        out[f"im2col_{i}"] = dl.im2col_torch(x, *p).numpy()
    q = torch.randint(0, 4, (2, 3, 8, 12), generator=g).float()     # many ties
    q[0, 0, 2, 3] = float("nan")
    q[1, 2, 0, 0] = float("nan")
    q[1, 2, 0, 1] = float("nan")
    q[0, 1] = -float("inf")
    out["pool_x"] = q.numpy()
    for i, p in enumerate(POOL_CASES):
        v, ix = dl.maxpool_torch(q, *p)
        out[f"pool_v_{i}"], out[f"pool_i_{i}"] = v.numpy(), ix.numpy()
    b = torch.randn(6, 5, 7, 4, generator=g) * 3 + 10
    m, s = dl.bnstats_f64(b, 1e-5)
    out["bn_x"], out["bn_mean"], out["bn_invstd"] = b.numpy(), m.numpy(), s.numpy()
    u = torch.rand(2, 3, 7, 9, generator=g)
    out["up_x"] = u.numpy()
    for i, (oh, ow, ac) in enumerate(UP_CASES):
        out[f"up_{i}"] = dl.upsample_numpy(u.numpy(), oh, ow, ac)
    h = torch.randn(5003, generator=g)
    h[0], h[1], h[2], h[3] = 1.0, -1.0, 2.5, float("nan")
    out["hist_x"] = h.numpy()
    for i, (nb, lo, hi) in enumerate(HIST_CASES):
        out[f"hist_{i}"] = dl.histc_numpy(h.numpy(), nb, lo, hi)
    np.savez_compressed(os.path.join(HERE, "dl_small.npz"), **out)


def make_crypto():
    hdr = OC.xoshiro_bytes(42, 80).tobytes()
    hh = OC.xoshiro_bytes(43, 32).tobytes()
    dag = OC.xoshiro_bytes(44, 128 * 4099)
    nonces32 = [0, 1, 2, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFF, 0x12345678]
    nonces64 = nonces32 + [1 << 32, (1 << 40) + 99, (1 << 64) - 1]
    kat = {
        "header80": hdr.hex(), "header_hash32": hh.hex(), "dag_seed": 44, "dag_items": 4099,
        "xoshiro_seed3_first64": OC.xoshiro_bytes(3, 64).tobytes().hex(),
        "blake256_spec": {"00": OC.blake256(b"\0").hex(), "00x72": OC.blake256(bytes(72)).hex()},
        "keccak_empty": {"256": OC.keccak(b"", 136, 1, 32).hex(), "512": OC.keccak(b"", 72, 1, 64).hex()},
        "blake256": {str(n): OC.blake256_header(hdr, n).hex() for n in nonces32},
        "sha256d": {str(n): OC.sha256d_header(hdr, n).hex() for n in nonces32},
        "sia": {str(n): OC.sia_header(hdr, n).hex() for n in nonces64},
        "ethash": {str(n): [x.hex() for x in OC.hashimoto(dag, hh, n)] for n in nonces64},
    }
    easy = (1 << (256 - 10)).to_bytes(32, "big")
    kat["easy_target"] = easy.hex()
    sweeps = {}
    for kind, name, start, count in [(0, "blake256", 0xFFFFF000, 8192), (1, "sha256d", 1000, 8192),
                                     (2, "sia", (1 << 36) + 7, 8192)]:
        found, n = OC.search(kind, hdr, start, count, easy)
        sweeps[name] = {"start": start, "count": count, "nonces": n}
    found, n, mix = OC.search(3, hh, 5000, 4096, easy, dag=dag)
    sweeps["ethash"] = {"start": 5000, "count": 4096, "nonces": n, "mix": [m.hex() for m in mix]}
    kat["sweeps"] = sweeps
    with open(os.path.join(HERE, "crypto_kat.json"), "w") as f:
        json.dump(kat, f, indent=1)


if __name__ == "__main__":
    make_dl()
    make_crypto()
    print("fixtures written to", HERE)
