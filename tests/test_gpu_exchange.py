"""The in-kernel cross-GPU sum of the batch-norm moments (hfuse_*_allreduce_f32).

With one GPU the exchange degenerates to the local buffer: the same device code runs (rows
delivered, counters bumped, the last block waits and folds), so slot rotation and counter
arithmetic are covered on any box.  The 2-rank test needs two GPUs and is skipped otherwise;
its ranks are child processes that talk over gloo only to swap the IPC handles.
"""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from hfuse_b200 import ops
from oracle import dl

pytestmark = pytest.mark.gpu


def test_world_of_one_matches_plain_kernels_over_many_calls(dev):
    from hfuse_b200.exchange import BnExchange
    g = torch.Generator().manual_seed(21)
    shapes = [(8, 32, 14, 14), (64, 4, 32, 32)]              # one slice per channel, and many slices per channel
    for shape in shapes:
        ex = BnExchange(shape[1])
        for it in range(10):                                  # more calls than slots: counters keep growing
            x = (0.5 + 2.0 * torch.randn(*shape, generator=g))
            op = ops.BnStats(x.to(dev), 1e-5, want_moments=True)
            ex.run(op)
            mr, sr = dl.bnstats_f64(x, 1e-5)
            np.testing.assert_allclose(op.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
            np.testing.assert_allclose(op.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
            n = x.numel() // x.shape[1]
            np.testing.assert_allclose(op.moments[:, 0].cpu().numpy(), n)
        up = torch.rand(2, 4, 12, 16, generator=g)
        a, b = ops.Upsample(up.to(dev), scale_factor=2), ops.BnStats(x.to(dev), 1e-5)
        ex.run_pair(a, b)
        assert np.array_equal(a.out.cpu().numpy(), dl.upsample_numpy(up.numpy(), 24, 32))
        np.testing.assert_allclose(b.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
        assert not ex.timed_out()
        ex.close()


def test_statistics_range_takes_over_any_share_of_the_upsample(dev):
    """The fused exchange kernel hands per-mille shares of the upsample to the statistics thread
    range (after it has sent its moments).  Every share, every thread split and all three upsample
    paths (x2 strips, 4-wide, scalar) must give the bits of the plain kernels."""
    from hfuse_b200 import _lib
    from hfuse_b200.exchange import BnExchange
    g = torch.Generator().manual_seed(77)
    x = 0.5 + 2.0 * torch.randn(6, 40, 9, 12, generator=g)
    mr, sr = dl.bnstats_f64(x, 1e-5)
    cases = [((3, 5, 12, 16), dict(scale_factor=2)),          # x2 strip path
             ((2, 3, 7, 8), dict(scale_factor=2)),
             ((2, 3, 9, 10), dict(size=(13, 24))),            # 4-wide path
             ((2, 3, 9, 10), dict(size=(11, 15)))]            # scalar path
    ex = BnExchange(40)
    try:
        for variant in (15, 3, 0, 11):
            for share in (0, 1, 250, 500, 999, 1000):
                _lib.tune_set("upsample_bnstats_allreduce", variant, 0)
                _lib.tune_set_share("upsample_bnstats_allreduce", share)
                for shape, kw in cases:
                    up = torch.rand(*shape, generator=g)
                    a, b = ops.Upsample(up.to(dev), **kw), ops.BnStats(x.to(dev), 1e-5)
                    ex.run_pair(a, b)
                    oh, ow = a.out.shape[-2:]
                    assert np.array_equal(a.out.cpu().numpy(), dl.upsample_numpy(up.numpy(), oh, ow)), (variant, share, shape)
                    np.testing.assert_allclose(b.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
                    np.testing.assert_allclose(b.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        assert not ex.timed_out()
    finally:
        _lib.tune_set("upsample_bnstats_allreduce", -1, 0)
        _lib.tune_set_share("upsample_bnstats_allreduce", -1)
        ex.close()
    # the cursor form: every warp of either range draws chunks of the upsample; same bits for every split.
    # Statistics input with rows long enough for the bulk-load path too, read both ways.
    x_long = 0.5 + 2.0 * torch.randn(5, 40, 16, 20, generator=g)
    stats_inputs = [(x, mr, sr, (0,)), (x_long, *dl.bnstats_f64(x_long, 1e-5), (0, 1))]
    ex = BnExchange(40)
    try:
        _lib.tune_option("exchange_pair_pool", 1)
        for variant in range(len(_lib.tune_variants("upsample_bnstats_allreduce"))):
            _lib.tune_set("upsample_bnstats_allreduce", variant, 0)
            for xs, mrs, srs, paths in stats_inputs:
                for path in paths:
                    _lib.tune_option("bnstats_load_path", path)
                    for shape, kw in cases:
                        up = torch.rand(*shape, generator=g)
                        a, b = ops.Upsample(up.to(dev), **kw), ops.BnStats(xs.to(dev), 1e-5)
                        a.out.fill_(float("nan"))
                        ex.run_pair(a, b)
                        oh, ow = a.out.shape[-2:]
                        assert np.array_equal(a.out.cpu().numpy(), dl.upsample_numpy(up.numpy(), oh, ow)), (variant, shape, path)
                        np.testing.assert_allclose(b.mean.cpu().double().numpy(), mrs.numpy(), rtol=1e-5, atol=1e-6)
                        np.testing.assert_allclose(b.invstd.cpu().double().numpy(), srs.numpy(), rtol=1e-5)
        assert not ex.timed_out()
    finally:
        _lib.tune_set("upsample_bnstats_allreduce", -1, 0)
        _lib.tune_option("exchange_pair_pool", -1)
        _lib.tune_option("bnstats_load_path", -1)
        ex.close()
    with pytest.raises(_lib.HfuseError):
        _lib.tune_set_share("upsample_bnstats", 100)          # only the exchange pair has a share
    with pytest.raises(_lib.HfuseError):
        _lib.tune_set_share("upsample_bnstats_allreduce", 1001)


def test_full_size_configuration_1_through_the_exchange_pair(dev):
    """Benchmark configuration 1 (256 channels: one channel per block, the deferred collect) through
    the exchange entry point, with the compiled defaults and with the many-rank defaults."""
    from hfuse_b200 import _lib, workloads
    from hfuse_b200.exchange import BnExchange
    w = workloads.config1()
    ref = dl.upsample_numpy(w["up"].numpy(), 112, 112)
    mr, sr = dl.bnstats_f64(w["bn"], w["eps"])
    ex = BnExchange(256)
    try:
        for variant, share in ((-1, -1), (21, 400), (15, 0)):
            _lib.tune_set("upsample_bnstats_allreduce", variant, 0)
            _lib.tune_set_share("upsample_bnstats_allreduce", share)
            for _ in range(3):
                a = ops.Upsample(w["up"].to(dev), scale_factor=2)
                b = ops.BnStats(w["bn"].to(dev), w["eps"])
                ex.run_pair(a, b)
                assert np.array_equal(a.out.cpu().numpy(), ref)
                np.testing.assert_allclose(b.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
                np.testing.assert_allclose(b.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        assert not ex.timed_out()
    finally:
        _lib.tune_set("upsample_bnstats_allreduce", -1, 0)
        _lib.tune_set_share("upsample_bnstats_allreduce", -1)
        ex.close()


def test_a_rank_that_never_arrives_ends_the_wait_with_a_status_and_the_late_rank_still_sums(dev):
    """Two ranks driven by this process on one GPU, launched one after the other.  Rank 0 runs
    alone: nothing ever writes rank 1's rows, so its bounded wait (20 ms here) runs out, the kernel
    returns, the status word is raised and the context stays usable.  Rank 1 then runs: rank 0's
    rows are already in its buffer, so it does not wait and reports the statistics of both batches."""
    from hfuse_b200.exchange import BnExchange
    g = torch.Generator().manual_seed(91)
    x = 0.5 + 2.0 * torch.randn(8, 24, 10, 10, generator=g)
    mr, sr = dl.bnstats_f64(x, 1e-5)
    ex0, ex1 = BnExchange.local_ranks(24, [dev, dev])
    try:
        for ex in (ex0, ex1):
            ex.set_timeout(0.02)
        b0 = ops.BnStats(x[:4].contiguous().to(dev), 1e-5)
        b1 = ops.BnStats(x[4:].contiguous().to(dev), 1e-5)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        ex0.run(b0)
        t1.record()
        torch.cuda.synchronize()
        assert ex0.timed_out() and not ex1.timed_out()
        assert 15.0 < t0.elapsed_time(t1) < 2000.0                       # gave up after the limit, not at once, not never
        ex1.run(b1)
        torch.cuda.synchronize()
        assert not ex1.timed_out()
        np.testing.assert_allclose(b1.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
        np.testing.assert_allclose(b1.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        # the device is still usable for ordinary work
        c = ops.BnStats(x.to(dev), 1e-5)
        ops.run(c)
        np.testing.assert_allclose(c.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
    finally:
        ex0.close()
        ex1.close()


def test_fused_exchange_pair_across_two_ranks_launched_one_after_the_other(dev):
    """The fused pair (upsample | statistics: send, share of the upsample, collect) with two ranks
    driven by this process on one GPU.  Rank 0 runs alone: its collect runs out of time (20 ms)
    and raises the status, but its upsample, including the share handed to the statistics thread
    range, is complete and bit-exact.  Rank 1 then finds rank 0's rows, does not wait, and reports
    the statistics of both batches.  The two launches never wait on each other at the same time."""
    from hfuse_b200 import _lib
    from hfuse_b200.exchange import BnExchange
    g = torch.Generator().manual_seed(92)
    for C, shape in ((24, (8, 24, 10, 10)), (256, (4, 256, 28, 28))):       # few channels; one channel per block
        x = 0.5 + 2.0 * torch.randn(*shape, generator=g)
        mr, sr = dl.bnstats_f64(x, 1e-5)
        half = shape[0] // 2
        up0, up1 = torch.rand(2, 5, 12, 16, generator=g), torch.rand(3, 4, 8, 8, generator=g)
        ex0, ex1 = BnExchange.local_ranks(C, [dev, dev])
        try:
            for variant, share in ((-1, -1), (21, 400), (0, 1000)):
                _lib.tune_set("upsample_bnstats_allreduce", variant, 0)
                _lib.tune_set_share("upsample_bnstats_allreduce", share)
                for ex in (ex0, ex1):
                    ex.set_timeout(0.02)
                    ex.clear_status()
                a0, b0 = ops.Upsample(up0.to(dev), scale_factor=2), ops.BnStats(x[:half].contiguous().to(dev), 1e-5)
                a1, b1 = ops.Upsample(up1.to(dev), scale_factor=2), ops.BnStats(x[half:].contiguous().to(dev), 1e-5)
                a0.out.fill_(float("nan"))
                a1.out.fill_(float("nan"))
                ex0.run_pair(a0, b0)
                torch.cuda.synchronize()
                assert ex0.timed_out() and not ex1.timed_out()
                assert np.array_equal(a0.out.cpu().numpy(), dl.upsample_numpy(up0.numpy(), 24, 32))
                ex1.run_pair(a1, b1)
                torch.cuda.synchronize()
                assert not ex1.timed_out()
                assert np.array_equal(a1.out.cpu().numpy(), dl.upsample_numpy(up1.numpy(), 16, 16))
                np.testing.assert_allclose(b1.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
                np.testing.assert_allclose(b1.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        finally:
            _lib.tune_set("upsample_bnstats_allreduce", -1, 0)
            _lib.tune_set_share("upsample_bnstats_allreduce", -1)
            ex0.close()
            ex1.close()


def test_calls_replayed_from_a_cuda_graph_move_on_to_the_next_slot_and_epoch(dev):
    """Slot and epoch of a call are counted on the device, so a captured call that is replayed
    does not meet the rows of its previous replay.  World of one: three replays of ONE captured
    call follow three different inputs.  Two ranks on one GPU, one captured call each, replayed
    one after the other: on every replay rank 0 (alone at that moment) must run out of time again
    instead of folding the row rank 1 left in the previous replay, and rank 1 must report the
    statistics of the inputs of THIS replay."""
    from hfuse_b200.exchange import BnExchange
    g = torch.Generator().manual_seed(93)
    shape = (8, 24, 10, 10)
    xs = [0.5 * k + (1.0 + k) * torch.randn(*shape, generator=g) for k in range(3)]
    side = torch.cuda.Stream(dev)
    # ---- world of one
    ex = BnExchange(24)
    try:
        buf = xs[0].to(dev)
        op = ops.BnStats(buf, 1e-5)
        up = torch.rand(2, 3, 8, 8, generator=g)
        a = ops.Upsample(up.to(dev), scale_factor=2)
        with torch.cuda.stream(side):
            ex.run_pair(a, op)                                   # warm-up outside the capture
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                ex.run_pair(a, op)
        for x in xs + xs:                                        # six replays: every slot is reused
            buf.copy_(x)
            graph.replay()
            torch.cuda.synchronize()
            mr, sr = dl.bnstats_f64(x, 1e-5)
            np.testing.assert_allclose(op.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
            np.testing.assert_allclose(op.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        assert not ex.timed_out()
        del graph
    finally:
        ex.close()
    # ---- two ranks, sequential
    ex0, ex1 = BnExchange.local_ranks(24, [dev, dev])
    try:
        for e in (ex0, ex1):
            e.set_timeout(0.02)
        buf0, buf1 = xs[0][:4].contiguous().to(dev), xs[0][4:].contiguous().to(dev)
        b0, b1 = ops.BnStats(buf0, 1e-5), ops.BnStats(buf1, 1e-5)
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                ex0.run(b0)
                ex1.run(b1)
        for x in xs + xs:
            buf0.copy_(x[:4])
            buf1.copy_(x[4:])
            ex0.clear_status()
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            assert ex0.timed_out()            # rank 1's row of THIS call was not there yet
            assert not ex1.timed_out()
            mr, sr = dl.bnstats_f64(x, 1e-5)
            np.testing.assert_allclose(b1.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
            np.testing.assert_allclose(b1.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        del graph
    finally:
        ex0.close()
        ex1.close()


def test_a_call_that_fails_on_the_host_does_not_put_the_rank_out_of_step(dev):
    """A call refused after its arguments were accepted (here: a sliced plan without scratch) never
    ran, so it must not count as a use of the exchange: the next good call of that rank has to meet
    its peer in the same slot with the same epoch."""
    from hfuse_b200 import _lib
    from hfuse_b200.exchange import BnExchange
    g = torch.Generator().manual_seed(94)
    x = 0.5 + 2.0 * torch.randn(64, 4, 32, 32, generator=g)         # few channels: cut into slices, needs scratch
    mr, sr = dl.bnstats_f64(x, 1e-5)
    ex0, ex1 = BnExchange.local_ranks(4, [dev, dev])
    try:
        for e in (ex0, ex1):
            e.set_timeout(0.02)
        bad = ops.BnStats(x[:32].contiguous().to(dev), 1e-5, workspace=torch.zeros(16, dtype=torch.uint8, device=dev))
        with pytest.raises(_lib.HfuseError) as err:
            ex0.run(bad)
        assert err.value.code == -4
        b0 = ops.BnStats(x[:32].contiguous().to(dev), 1e-5)
        b1 = ops.BnStats(x[32:].contiguous().to(dev), 1e-5, workspace=torch.zeros_like(b0.ws))
        ex0.run(b0)                            # alone: runs out of time, but its rows are delivered
        ex1.run(b1)
        torch.cuda.synchronize()
        assert not ex1.timed_out()
        np.testing.assert_allclose(b1.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
        np.testing.assert_allclose(b1.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        # the flag stays up until it is cleared
        assert ex0.timed_out()
        ex0.clear_status()
        assert not ex0.timed_out()
    finally:
        ex0.close()
        ex1.close()


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hfuse_b200 import _lib, sharding
        from hfuse_b200.exchange import BnExchange
        dev = torch.device("cuda", rank)
        ex = BnExchange(24)
        ok = True
        g = torch.Generator().manual_seed(33)
        for it in range(9):
            x = 0.5 + 2.0 * torch.randn(8, 24, 10, 10, generator=g)         # same tensor on every rank
            mine = sharding.shard_batch(x, rank, world).contiguous().to(dev)
            up = torch.rand(2, 3, 8, 8, generator=g)
            a, b = ops.Upsample(up.to(dev), scale_factor=2), ops.BnStats(mine, 1e-5)
            if it % 2:
                _lib.tune_set_share("upsample_bnstats_allreduce", (0, 400, 1000)[it % 3])
                ex.run_pair(a, b)
                ok &= np.array_equal(a.out.cpu().numpy(), dl.upsample_numpy(up.numpy(), 16, 16))
            else:
                ex.run(b)
            mr, sr = dl.bnstats_f64(x, 1e-5)                                  # statistics of the WHOLE batch
            ok &= np.allclose(b.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5, atol=0)
            ok &= np.allclose(b.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5, atol=0)
        ok &= not ex.timed_out()
        # all ranks hold identical bits
        mine_bits = b.mean.cpu()
        got = [None] * world
        dist.all_gather_object(got, mine_bits)
        ok &= all(torch.equal(got[0], t) for t in got)
        ret[rank] = bool(ok)
        dist.barrier()
        ex.close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_sum_over_nvlink(dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert ret[0] and ret[1]
