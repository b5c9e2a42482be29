"""Host-side multi-GPU logic on CPU: shard arithmetic, and the two reductions over a
world_size-2 gloo group (spawned processes)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hfuse_b200 import sharding
from oracle import dl


def test_shard_range_covers_everything_once():
    for total in (0, 1, 7, 16, 2 ** 32, 2 ** 30 + 3):
        for world in (1, 2, 3, 4, 8):
            parts = [sharding.shard_range(total, r, world) for r in range(world)]
            assert parts[0][0] == 0
            for (o1, n1), (o2, _) in zip(parts, parts[1:]):
                assert o1 + n1 == o2
            assert parts[-1][0] + parts[-1][1] == total
            assert max(n for _, n in parts) - min(n for _, n in parts) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def test_c_abi_shard_range_agrees_with_the_python_split():
    """hfuse_shard_range is host arithmetic: it runs without a GPU."""
    import ctypes
    from hfuse_b200 import _lib
    L = _lib.lib()
    off, n = ctypes.c_uint64(), ctypes.c_uint64()
    for total in (0, 1, 7, 16, 2 ** 32, 2 ** 30 + 3, 2 ** 63 + 5):
        for world in (1, 2, 3, 8):
            for r in range(world):
                assert L.hfuse_shard_range(total, r, world, ctypes.byref(off), ctypes.byref(n)) == 0
                assert (off.value, n.value) == sharding.shard_range(total, r, world)
    assert L.hfuse_shard_range(4, 2, 2, ctypes.byref(off), ctypes.byref(n)) == -1
    assert L.hfuse_shard_range(4, 0, 0, ctypes.byref(off), ctypes.byref(n)) == -1
    assert L.hfuse_shard_range(4, 0, 1, None, ctypes.byref(n)) == -1


def test_nonce_shards_keep_64_bit_counts():
    # a full 32-bit sweep starting near the top of the space
    start, count = 0xFFFFFF00, 1 << 32
    parts = [sharding.shard_nonces(start, count, r, 8) for r in range(8)]
    assert sum(n for _, n in parts) == count and parts[3][0] == start + 3 * (1 << 29)


def test_flat_shards_stay_aligned():
    x = torch.arange(1003, dtype=torch.float32)
    parts = [sharding.shard_flat(x, r, 4) for r in range(4)]
    assert torch.equal(torch.cat(parts), x)
    assert all(p.data_ptr() % 16 == 0 for p in parts)


def test_merge_hits_sorts():
    assert sharding.merge_hits([[5, 9], [], [1]]) == [1, 5, 9]
    assert sharding.merge_hits([[(7, b"a")], [(2, b"b")]]) == [(2, b"b"), (7, b"a")]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(5)
        x = 0.5 + 2.0 * torch.randn(6, 4, 5, 3)
        h = torch.randn(4001)
        mine = sharding.shard_batch(x, rank, world).double()
        n = mine.shape[0] * 15
        mom = torch.stack([torch.full((4,), float(n), dtype=torch.float64), mine.sum(dim=(0, 2, 3)),
                           (mine * mine).sum(dim=(0, 2, 3))], dim=1).contiguous()
        sharding.allreduce_moments(mom)
        mean, invstd = sharding.moments_to_stats(mom, 1e-5)
        mref, sref = dl.bnstats_f64(x, 1e-5)
        ok = torch.allclose(mean, mref, rtol=1e-10) and torch.allclose(invstd, sref, rtol=1e-10)
        counts = torch.from_numpy(dl.histc_numpy(sharding.shard_flat(h, rank, world).numpy(), 16, -4, 4)
                                  .astype(np.int32))
        sharding.allreduce_counts(counts)
        ok = ok and np.array_equal(counts.numpy().astype(np.uint32), dl.histc_numpy(h.numpy(), 16, -4, 4))
        hits = sharding.gather_hits([(10 * rank + 3, b"x")])
        ok = ok and [h[0] for h in hits] == [3, 13]
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_reductions_over_gloo_world_2():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret[0] and ret[1]


def _exchange_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hfuse_b200 import _lib
        from hfuse_b200.exchange import BnExchange
        try:
            BnExchange(8)
            ret[rank] = "no error"
        except _lib.HfuseError as e:
            ret[rank] = f"raised {e.code}"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.is_available(), reason="exercises the set-up failure path of a box without a GPU")
def test_exchange_setup_fails_on_all_ranks_together_without_hanging():
    """Without a GPU the exchange buffer cannot be created; both ranks must learn that and raise,
    instead of one of them waiting inside a gather for a peer that gave up."""
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_exchange_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret[0].startswith("raised") and ret[1].startswith("raised")
