"""Pins the crypto oracle: hashlib where it has the algorithm, the digests the BLAKE
and Keccak specifications publish, an independent pure-Python restatement, and the
committed golden fixtures."""
import hashlib
import json
import os
import random

import pytest

from conftest import GOLDEN
from oracle import crypto as OC
from oracle import crypto_py as OP

LENGTHS = [0, 1, 3, 55, 56, 63, 64, 65, 80, 111, 112, 119, 120, 127, 128, 129, 200, 300]


def _msgs():
    rnd = random.Random(7)
    return [bytes(rnd.randrange(256) for _ in range(n)) for n in LENGTHS]


def test_sha256_and_blake2b_match_hashlib():
    for m in _msgs():
        assert OC.sha256(m) == hashlib.sha256(m).digest()
        assert OC.blake2b(m, 32) == hashlib.blake2b(m, digest_size=32).digest()
        assert OC.blake2b(m, 64) == hashlib.blake2b(m).digest()


def test_keccak_sponge_matches_sha3_with_nist_padding():
    for m in _msgs():
        assert OC.keccak(m, 136, 0x06, 32) == hashlib.sha3_256(m).digest()
        assert OC.keccak(m, 72, 0x06, 64) == hashlib.sha3_512(m).digest()
        assert OP.keccak(m, 136, 0x06, 32) == hashlib.sha3_256(m).digest()
        assert OP.keccak(m, 72, 0x06, 64) == hashlib.sha3_512(m).digest()


def test_published_digests():
    # BLAKE-256 specification: one zero byte, and 72 zero bytes
    assert OC.blake256(b"\0").hex() == "0ce8d4ef4dd7cd8d62dfded9d4edb0a774ae6a41929a74da23109e8f11139c87"
    assert OC.blake256(bytes(72)).hex() == "d419bad32d504fb7d44d460c42c5593fe544fa4c135dec31e21bd9abdcc22d41"
    # original-padding Keccak of the empty string
    assert OC.keccak(b"", 136, 0x01, 32).hex() == \
        "c5d2460186f7233c927e7db2dcc703c0e500b653ca82273b7bfad8045d85a470"
    assert OC.keccak(b"", 72, 0x01, 64).hex().startswith("0eab42de4c3ceb9235fc91acffe746b29c29a8c366b7c60e")


def test_c_and_python_restatements_agree():
    for m in _msgs():
        assert OC.blake256(m) == OP.blake256(m)
        assert OC.keccak(m, 136, 0x01, 32) == OP.keccak256(m)
        assert OC.keccak(m, 72, 0x01, 64) == OP.keccak512(m)
    assert OC.xoshiro_bytes(3, 1001).tobytes() == OP.xoshiro256ss_bytes(3, 1001)
    dag = OC.xoshiro_bytes(9, 128 * 257)
    hh = bytes(range(32))
    for nonce in (0, 1, 2 ** 40 + 5, 2 ** 64 - 1):
        assert OC.hashimoto(dag, hh, nonce) == OP.hashimoto(dag.tobytes(), 257, hh, nonce)


def test_header_helpers_place_the_nonce():
    hdr = bytes(range(80))
    n = 0xA1B2C3D4
    h32 = hdr[:76] + n.to_bytes(4, "little")
    assert OC.sha256d_header(hdr, n) == hashlib.sha256(hashlib.sha256(h32).digest()).digest()
    assert OC.blake256_header(hdr, n) == OP.blake256(h32)
    n64 = 0x0102030405060708
    h64 = hdr[:32] + n64.to_bytes(8, "little") + hdr[40:]
    assert OC.sia_header(hdr, n64) == hashlib.blake2b(h64, digest_size=32).digest()


@pytest.fixture(scope="module")
def kat():
    with open(os.path.join(GOLDEN, "crypto_kat.json")) as f:
        return json.load(f)


def test_golden_digests(kat):
    hdr, hh = bytes.fromhex(kat["header80"]), bytes.fromhex(kat["header_hash32"])
    assert OC.xoshiro_bytes(3, 64).tobytes().hex() == kat["xoshiro_seed3_first64"]
    for n, d in kat["blake256"].items():
        assert OC.blake256_header(hdr, int(n)).hex() == d
    for n, d in kat["sha256d"].items():
        assert OC.sha256d_header(hdr, int(n)).hex() == d
    for n, d in kat["sia"].items():
        assert OC.sia_header(hdr, int(n)).hex() == d
    dag = OC.xoshiro_bytes(kat["dag_seed"], 128 * kat["dag_items"])
    for n, (mix, res) in kat["ethash"].items():
        m, r = OC.hashimoto(dag, hh, int(n))
        assert (m.hex(), r.hex()) == (mix, res)


def test_golden_sweeps_and_target_rule(kat):
    hdr, hh = bytes.fromhex(kat["header80"]), bytes.fromhex(kat["header_hash32"])
    easy = bytes.fromhex(kat["easy_target"])
    for kind, name in ((0, "blake256"), (1, "sha256d"), (2, "sia")):
        sw = kat["sweeps"][name]
        found, nonces = OC.search(kind, hdr, sw["start"], sw["count"], easy)
        assert found == len(sw["nonces"]) and nonces == sw["nonces"]
        assert len(nonces) > 0
    # the 32-bit kinds wrap: the blake sweep starts 4096 below 2^32
    assert any(n < 4096 for n in kat["sweeps"]["blake256"]["nonces"])
    # hit rule: digest as a big-endian integer strictly below the target
    fn = OC.sha256d_header
    sw = kat["sweeps"]["sha256d"]
    brute = [n for n in range(sw["start"], sw["start"] + 512)
             if int.from_bytes(fn(hdr, n), "big") < int.from_bytes(easy, "big")]
    assert brute == [n for n in sw["nonces"] if n < sw["start"] + 512]
    dag = OC.xoshiro_bytes(kat["dag_seed"], 128 * kat["dag_items"])
    sw = kat["sweeps"]["ethash"]
    found, nonces, mix = OC.search(3, hh, sw["start"], sw["count"], easy, dag=dag)
    assert nonces == sw["nonces"] and [m.hex() for m in mix] == sw["mix"]


def test_dag_generation_restatements_agree():
    seed = bytes(range(32))
    c = OC.ethash_cache(seed, 67)
    pc = OP.ethash_cache(seed, 67)
    assert c.tobytes() == b"".join(pc)
    d = OC.ethash_dataset(c, 5, 12)
    for k in range(12):
        assert d[64 * k:64 * k + 64].tobytes() == OP.ethash_dataset_node(pc, 5 + k)
    # the library's host-side cache builder is a third implementation of the same chain
    from hfuse_b200 import crypto
    import numpy as np
    assert np.array_equal(crypto.make_cache(seed, 67), c)
