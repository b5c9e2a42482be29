"""GPU parity of the four hash searches and their six fused pairs through the C ABI."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from hfuse_b200 import _lib, crypto, sharding, workloads
from oracle import crypto as OC

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kat():
    with open(os.path.join(GOLDEN, "crypto_kat.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def small_dag(kat, dev):
    host = workloads.xoshiro_bytes(kat["dag_seed"], 128 * kat["dag_items"])
    return host, torch.from_numpy(host).to(dev)


def test_golden_digests(dev, kat, small_dag):
    hdr, hh = bytes.fromhex(kat["header80"]), bytes.fromhex(kat["header_hash32"])
    for kind in ("blake256", "sha256d", "sia"):
        for n, d in kat[kind].items():
            out, _ = crypto.hash_batch(kind, hdr, int(n), 1)
            assert out[0].tobytes().hex() == d, (kind, n)
    for n, (mix, res) in kat["ethash"].items():
        out, m = crypto.hash_batch("ethash", hh, int(n), 1, small_dag[1])
        assert (m[0].tobytes().hex(), out[0].tobytes().hex()) == (mix, res)


@pytest.mark.parametrize("kind,fn", [("blake256", OC.blake256_header), ("sha256d", OC.sha256d_header),
                                     ("sia", OC.sia_header)])
def test_digest_batches_against_oracle(dev, kind, fn):
    hdr = workloads.xoshiro_bytes(7, 80).tobytes()
    starts = [0, 0xFFFFFF00, 123456789] + ([(1 << 40) + 3, (1 << 64) - 300] if kind == "sia" else [])
    for start in starts:
        out, _ = crypto.hash_batch(kind, hdr, start, 700)
        for i in range(700):
            assert out[i].tobytes() == fn(hdr, (start + i) & (2 ** 64 - 1)), (kind, start, i)


def test_ethash_batch_against_oracle(dev, small_dag):
    host, dag = small_dag
    hh = workloads.xoshiro_bytes(8, 32).tobytes()
    for start in (0, (1 << 33) + 5):
        out, mix = crypto.hash_batch("ethash", hh, start, 333, dag)       # not a multiple of the 8-lane group
        for i in range(333):
            m, r = OC.hashimoto(host, hh, start + i)
            assert mix[i].tobytes() == m and out[i].tobytes() == r, (start, i)
    # power-of-two DAG as in the benchmark
    host2 = workloads.xoshiro_bytes(9, 128 * 1024)
    out, mix = crypto.hash_batch("ethash", hh, 77, 64, torch.from_numpy(host2).to(dev))
    for i in range(64):
        assert (mix[i].tobytes(), out[i].tobytes()) == OC.hashimoto(host2, hh, 77 + i)


def test_golden_sweeps(dev, kat, small_dag):
    hdr, hh = bytes.fromhex(kat["header80"]), bytes.fromhex(kat["header_hash32"])
    easy = bytes.fromhex(kat["easy_target"])
    for cls, name in ((crypto.Blake256, "blake256"), (crypto.Sha256d, "sha256d"), (crypto.Sia, "sia")):
        sw = kat["sweeps"][name]
        s = crypto.run(cls(hdr, sw["start"], sw["count"], easy))
        total, hits = s.result()
        assert total == len(sw["nonces"]) and [h[0] for h in hits] == sw["nonces"], name
    sw = kat["sweeps"]["ethash"]
    s = crypto.run(crypto.Ethash(small_dag[1], hh, sw["start"], sw["count"], easy))
    total, hits = s.result()
    assert [h[0] for h in hits] == sw["nonces"] and [h[1].hex() for h in hits] == sw["mix"]


def test_edge_cases(dev, kat):
    hdr = bytes.fromhex(kat["header80"])
    easy = bytes.fromhex(kat["easy_target"])
    # empty sweep; zero target (nothing is below it); all-ones target (everything but a digest of all ones hits)
    assert crypto.run(crypto.Sha256d(hdr, 0, 0, easy)).result() == (0, [])
    assert crypto.run(crypto.Sha256d(hdr, 0, 4096, bytes(32))).result()[0] == 0
    total, hits = crypto.run(crypto.Blake256(hdr, 0, 1000, b"\xff" * 32)).result()
    assert total == 1000 and len(hits) == _lib.HFUSE_MAX_HITS            # count keeps counting past the record
    # a sweep across the 32-bit wrap equals the oracle's wrapped sweep
    s = crypto.run(crypto.Sha256d(hdr, 0xFFFFFE00, 1024, easy))
    assert s.nonces() == OC.search(1, hdr, 0xFFFFFE00, 1024, easy)[1]
    with pytest.raises(_lib.HfuseError):
        crypto.run(crypto.Sha256d(hdr, 0, (1 << 32) + 1, easy))


def _mk(key, kat, dag, easy):
    hdr, hh = bytes.fromhex(kat["header80"]), bytes.fromhex(kat["header_hash32"])
    if key == "blake256":
        return crypto.Blake256(hdr, 0xFFFF0000, 1 << 17, easy)
    if key == "sha256d":
        return crypto.Sha256d(hdr, 5, 1 << 17, easy)
    if key == "sia":
        return crypto.Sia(hdr, 1 << 35, 1 << 17, easy)
    return crypto.Ethash(dag, hh, 99, (1 << 14) + 3, easy)


@pytest.mark.parametrize("pair", sorted(_lib.CRYPTO_PAIRS))
def test_fused_pairs_equal_standalone_for_every_variant(dev, kat, small_dag, pair):
    easy = bytes.fromhex(kat["easy_target"])
    ka, kb = _lib.CRYPTO_PAIRS[pair]
    ra = crypto.run(_mk(ka, kat, small_dag[1], easy)).result()
    rb = crypto.run(_mk(kb, kat, small_dag[1], easy)).result()
    assert ra[0] > 0 and rb[0] > 0
    try:
        for v in range(len(_lib.tune_variants(pair))):
            _lib.tune_set(pair, v, 0)
            a, b = _mk(ka, kat, small_dag[1], easy), _mk(kb, kat, small_dag[1], easy)
            crypto.run_pair(a, b)
            assert a.result() == ra and b.result() == rb, (pair, v)
    finally:
        _lib.tune_set(pair, -1, 0)


def test_standalone_searches_give_the_same_hits_in_every_block_shape_and_form(dev, kat, small_dag):
    """Grid-stride and work-queue forms of the four searches, every compiled block shape; a record
    whose cursor was left non-zero by an earlier call must not matter."""
    easy = bytes.fromhex(kat["easy_target"])
    for key in sorted(_lib.CRYPTO_SOLO):
        want = crypto.run(_mk(key, kat, small_dag[1], easy)).result()
        assert want[0] > 0
        descr = _lib.tune_variants(key)
        assert any(d.endswith(" queue") for d in descr)
        try:
            for v in range(len(descr)):
                _lib.tune_set(key, v, 0)
                s = _mk(key, kat, small_dag[1], easy)
                crypto.run(s)
                assert s.result() == want, (key, descr[v])
                crypto.run(s)                      # the same record again
                assert s.result() == want, (key, descr[v], "second run")
        finally:
            _lib.tune_set(key, -1, 0)


def test_standalone_results_match_oracle_sweeps(dev, kat, small_dag):
    easy = bytes.fromhex(kat["easy_target"])
    hdr, hh = bytes.fromhex(kat["header80"]), bytes.fromhex(kat["header_hash32"])
    assert crypto.run(_mk("blake256", kat, None, easy)).nonces() == OC.search(0, hdr, 0xFFFF0000, 1 << 17, easy)[1]
    assert crypto.run(_mk("sha256d", kat, None, easy)).nonces() == OC.search(1, hdr, 5, 1 << 17, easy)[1]
    assert crypto.run(_mk("sia", kat, None, easy)).nonces() == OC.search(2, hdr, 1 << 35, 1 << 17, easy)[1]
    found, nonces, mix = OC.search(3, hh, 99, (1 << 14) + 3, easy, dag=small_dag[0])
    total, hits = crypto.run(_mk("ethash", kat, small_dag[1], easy)).result()
    assert [h[0] for h in hits] == nonces and [h[1] for h in hits] == mix


def test_nonce_sharding_gives_the_same_hits(dev, kat):
    hdr = bytes.fromhex(kat["header80"])
    easy = bytes.fromhex(kat["easy_target"])
    whole = crypto.run(crypto.Sia(hdr, (1 << 40) - 1000, 1 << 16, easy)).result()[1]
    for world in (2, 8):
        parts = []
        for r in range(world):
            st, n = sharding.shard_nonces((1 << 40) - 1000, 1 << 16, r, world)
            parts.append(crypto.run(crypto.Sia(hdr, st, n, easy)).result()[1])
        assert sharding.merge_hits(parts) == whole


def test_full_nonce_space_sweep_config3(dev):
    """Configuration 3 at full size: both halves sweep all 2^32 nonces in one fused launch;
    every reported nonce is re-hashed by the oracle and must be below the target, and the
    fused result equals the two standalone sweeps."""
    c = workloads.config3()
    a = crypto.Blake256(c["blake_header"], c["start"], c["count"], c["target"])
    b = crypto.Sha256d(c["sha_header"], c["start"], c["count"], c["target"])
    crypto.run_pair(a, b)
    ra, rb = a.result(), b.result()
    for n, _ in ra[1]:
        assert OC.blake256_header(c["blake_header"], n) < c["target"]
    for n, _ in rb[1]:
        assert OC.sha256d_header(c["sha_header"], n) < c["target"]
    assert crypto.run(crypto.Blake256(c["blake_header"], 0, c["count"], c["target"])).result() == ra
    assert crypto.run(crypto.Sha256d(c["sha_header"], 0, c["count"], c["target"])).result() == rb
    # an easier target over the first 2^22 nonces agrees with the oracle's sweep exactly
    t = crypto.target_from_difficulty_bits(16)
    assert crypto.run(crypto.Blake256(c["blake_header"], 0, 1 << 22, t)).nonces() == \
        OC.search(0, c["blake_header"], 0, 1 << 22, t)[1]


def test_config4_on_the_full_dag(dev):
    """Configuration 4 on its real 1 GiB DAG (2^23 items of xoshiro256** bytes).  The first 2^18
    nonces with an easy target: hits, mix digests and Sia hits equal the oracle's sweep over the
    same DAG, fused and standalone.  Then the full 2^30 sweep of the benchmark in one fused launch:
    every reported hit is re-hashed by the oracle (mix digest equal, result below the boundary) and
    the hit count is what 2^30 draws at 2^-24 make plausible."""
    c = workloads.config4()
    host = c["dag"].numpy()
    dag = c["dag"].to(dev)
    assert dag.numel() == 1 << 30
    easy = crypto.target_from_difficulty_bits(12)
    n = 1 << 18
    found, nonces, mixes = OC.search(3, c["header_hash"], 0, n, easy, dag=host)
    sia_found, sia_nonces = OC.search(2, c["sia_header"], 0, n, easy)
    assert found > 30 and sia_found > 30
    s, e = crypto.Sia(c["sia_header"], 0, n, easy), crypto.Ethash(dag, c["header_hash"], 0, n, easy)
    crypto.run_pair(s, e)
    total, hits = e.result()
    assert total == found and [h[0] for h in hits] == nonces and [h[1] for h in hits] == mixes
    assert s.nonces() == sia_nonces
    assert crypto.run(crypto.Ethash(dag, c["header_hash"], 0, n, easy)).result() == (total, hits)
    # the benchmark's own sweep
    s, e = crypto.Sia(c["sia_header"], c["start"], c["count"], c["target"]), \
        crypto.Ethash(dag, c["header_hash"], c["start"], c["count"], c["target"])
    crypto.run_pair(s, e)
    total, hits = e.result()
    assert 20 <= total <= 130 and total == len(hits)              # expectation 64
    for nonce, mix in hits:
        m, r = OC.hashimoto(host, c["header_hash"], nonce)
        assert m == mix and r < c["target"]
    stotal, shits = s.result()
    assert 20 <= stotal <= 130
    for nonce, _ in shits:
        assert OC.sia_header(c["sia_header"], nonce) < c["target"]


def test_dag_generation_matches_oracle_and_feeds_the_search(dev):
    """Light cache on the host, DAG nodes on the GPU, then a search over the generated DAG."""
    seed = workloads.xoshiro_bytes(55, 32).tobytes()
    n_cache, n_nodes = 1021, 2 * 1543                       # odd sizes on purpose
    cache = crypto.make_cache(seed, n_cache)
    assert np.array_equal(cache, OC.ethash_cache(seed, n_cache))
    dag = crypto.generate_dag(torch.from_numpy(cache).to(dev), n_nodes, chunks=3)
    ref = OC.ethash_dataset(cache, 0, n_nodes)
    assert np.array_equal(dag.cpu().numpy(), ref)
    hh = workloads.xoshiro_bytes(56, 32).tobytes()
    out, mix = crypto.hash_batch("ethash", hh, 1000, 40, dag)
    for i in range(40):
        assert (mix[i].tobytes(), out[i].tobytes()) == OC.hashimoto(ref, hh, 1000 + i)


def test_fused_search_without_a_reset_still_sweeps_everything(dev, kat):
    """The fused kernels clear their own work-queue cursors: a second launch on records that were
    not reset finds every hit again (the counts simply keep adding up)."""
    hdr = bytes.fromhex(kat["header80"])
    easy = bytes.fromhex(kat["easy_target"])
    a, b = crypto.Blake256(hdr, 0, 1 << 15, easy), crypto.Sha256d(hdr, 0, 1 << 15, easy)
    crypto.run_pair(a, b)
    first = (a.result()[0], b.result()[0])
    assert first[0] > 0 and first[1] > 0
    crypto.run_pair(a, b, reset=False)
    assert (a.result()[0], b.result()[0]) == (2 * first[0], 2 * first[1])


def test_int32_probe_reports_its_operation_count_and_rejects_bad_arguments(dev):
    import ctypes
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    n = ctypes.c_uint64(0)
    L = _lib.lib()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    for mix, per in ((0, 2), (1, 3), (2, 3)):
        assert L.hfuse_int32_probe(mix, 64, sink.data_ptr(), ctypes.byref(n), None) == 0
        assert n.value == sms * 8 * 256 * 64 * 16 * per
    torch.cuda.synchronize()
    assert int(sink.item()) == 0
    assert L.hfuse_int32_probe(3, 64, sink.data_ptr(), ctypes.byref(n), None) == -1
    assert L.hfuse_int32_probe(0, 0, sink.data_ptr(), ctypes.byref(n), None) == -1
    assert L.hfuse_int32_probe(0, 64, None, ctypes.byref(n), None) == -1
