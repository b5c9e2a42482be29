"""The C++ host program over the C ABI (hfuse_b200/fuser, the counterpart of the reference's
`fuser` binary) finds the same nonces as the Python harness and the oracle."""
import json
import os
import subprocess

import pytest
import torch

from hfuse_b200 import build, crypto, workloads
from oracle import crypto as OC

pytestmark = pytest.mark.gpu


def test_fuser_binary_matches_python_harness_and_oracle(dev):
    exe = build.FUSER
    assert os.path.exists(exe), "build it with python -m hfuse_b200.build --fuser"
    nonces, dag_nodes, cache_nodes, bits = 1 << 16, 4096, 509, 10
    r = subprocess.run([exe, "--nonces", str(nonces), "--dag-nodes", str(dag_nodes), "--cache-nodes", str(cache_nodes),
                        "--bits", str(bits)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    rows = {}
    for line in r.stdout.splitlines():
        d = json.loads(line)
        rows[d.get("kernel", d.get("step"))] = d
    s = workloads.xoshiro_bytes(2024, 224).tobytes()
    seed, hh, hdr_a, hdr_b = s[:32], s[32:64], s[64:144], s[144:224]
    target = crypto.target_from_difficulty_bits(bits)
    cache = OC.ethash_cache(seed, cache_nodes)
    dag = OC.ethash_dataset(cache, 0, dag_nodes)
    eth = OC.search(3, hh, 0, nonces, target, dag=dag)[1]
    blake = OC.search(0, hdr_a, 0, nonces, target)[1]
    sha = OC.search(1, hdr_b, 0, nonces, target)[1]
    sia = OC.search(2, hdr_b, 0, nonces, target)[1]
    assert len(eth) and len(blake) and len(sha) and len(sia)
    assert rows["ethash_search"]["first"]["nonces"] == eth
    assert rows["blake256"]["first"]["nonces"] == blake
    assert rows["sha256d"]["first"]["nonces"] == sha
    assert rows["sia_blake2b"]["first"]["nonces"] == sia
    expect = {"ethash_blake256": (eth, blake), "sha256d_ethash": (sha, eth), "sia_ethash": (sia, eth),
              "blake256_sha256d": (blake, sha), "blake256_sia": (blake, sia), "sha256d_sia": (sha, sia)}
    for name, (a, b) in expect.items():
        assert rows[name]["first"]["nonces"] == a and rows[name]["second"]["nonces"] == b, name
