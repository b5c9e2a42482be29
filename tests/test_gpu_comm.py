"""The C-level multi-GPU entry points (NCCL communicator behind the C ABI, sharded searches).

With one GPU the communicator has a world of one: the same calls run, the reductions leave the
data as it is.  The two-rank test needs two GPUs and is skipped otherwise; its ranks are child
processes that use gloo only to pass the communicator id from rank 0 to rank 1.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from hfuse_b200 import _lib, crypto, ops, sharding, workloads
from oracle import crypto as OC
from oracle import dl

pytestmark = pytest.mark.gpu


def _comm(world, rank, ident):
    h = C.c_void_p()
    _lib.check(_lib.lib().hfuse_comm_create(world, rank, ident, C.byref(h)), "hfuse_comm_create")
    return h


def _new_id():
    buf = C.create_string_buffer(128)
    _lib.check(_lib.lib().hfuse_comm_unique_id(buf), "hfuse_comm_unique_id")
    return buf.raw


def test_world_of_one_reductions_and_broadcast(dev):
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    comm = _comm(1, 0, _new_id())
    try:
        g = torch.Generator().manual_seed(41)
        x = 0.5 + 2.0 * torch.randn(8, 16, 6, 6, generator=g)
        op = ops.BnStats(x.to(dev), 1e-5, want_moments=True)
        ops.run(op)
        mean, invstd = torch.empty(16, device=dev), torch.empty(16, device=dev)
        _lib.check(L.hfuse_bnstats_allreduce_nccl_f64(comm, op.moments.data_ptr(), 16, 1e-5, mean.data_ptr(),
                                                      invstd.data_ptr(), st), "hfuse_bnstats_allreduce_nccl_f64")
        mr, sr = dl.bnstats_f64(x, 1e-5)
        np.testing.assert_allclose(mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
        np.testing.assert_allclose(invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
        h = torch.randn(5000, generator=g)
        cnt = ops.histc(h.to(dev), 64, -3.0, 3.0)
        before = cnt.clone()
        _lib.check(L.hfuse_histc_allreduce_counts(comm, cnt.data_ptr(), 64, st), "hfuse_histc_allreduce_counts")
        assert torch.equal(cnt, before)
        dag = torch.from_numpy(workloads.xoshiro_bytes(5, 128 * 64)).to(dev)
        keep = dag.clone()
        _lib.check(L.hfuse_dag_broadcast(comm, dag.data_ptr(), dag.numel(), 0, st), "hfuse_dag_broadcast")
        assert torch.equal(dag, keep)
        assert L.hfuse_dag_broadcast(comm, dag.data_ptr(), dag.numel(), 1, st) == -1      # no such root
    finally:
        assert L.hfuse_comm_destroy(comm) == 0


def test_sharded_searches_cover_the_range_exactly_once(dev):
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    hdr_a, hdr_b = workloads.xoshiro_bytes(61, 80).tobytes(), workloads.xoshiro_bytes(62, 80).tobytes()
    easy = crypto.target_from_difficulty_bits(10)
    start, count = 0xFFFFF000, (1 << 15) + 5                     # crosses the 32-bit wrap, does not divide evenly
    want_a = OC.search(0, hdr_a, start, count, easy)[1]
    want_b = OC.search(1, hdr_b, start, count, easy)[1]
    host_dag = workloads.xoshiro_bytes(63, 128 * 1021)
    dag = torch.from_numpy(host_dag).to(dev)
    hh = workloads.xoshiro_bytes(64, 32).tobytes()
    want_s = OC.search(2, hdr_a, 1 << 40, count, easy)[1]
    _, want_e, want_mix = OC.search(3, hh, 7, count, easy, dag=host_dag)
    for world in (1, 3, 8):
        got_a, got_b, got_s, got_e = [], [], [], []
        for rank in range(world):
            a, b = crypto.Blake256(hdr_a, start, count, easy), crypto.Sha256d(hdr_b, start, count, easy)
            _lib.check(L.hfuse_blake256_sha256d_search_sharded(*a.c_args(), *b.c_args(), rank, world, st), "sharded cfg3")
            got_a.append(a.result()[1])
            got_b.append(b.result()[1])
            s, e = crypto.Sia(hdr_a, 1 << 40, count, easy), crypto.Ethash(dag, hh, 7, count, easy)
            _lib.check(L.hfuse_sia_ethash_search_sharded(*s.c_args(), *e.c_args(), rank, world, st), "sharded cfg4")
            got_s.append(s.result()[1])
            got_e.append(e.result()[1])
        assert [h[0] for h in sharding.merge_hits(got_a)] == sorted(want_a)
        assert [h[0] for h in sharding.merge_hits(got_b)] == sorted(want_b)
        assert [h[0] for h in sharding.merge_hits(got_s)] == want_s
        merged = sharding.merge_hits(got_e)
        assert [h[0] for h in merged] == want_e and [h[1] for h in merged] == want_mix
    a, b = crypto.Blake256(hdr_a, 0, 16, easy), crypto.Sha256d(hdr_b, 0, 16, easy)
    assert L.hfuse_blake256_sha256d_search_sharded(*a.c_args(), *b.c_args(), 3, 3, st) == -1    # rank out of range


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L = _lib.lib()
        dev = torch.device("cuda", rank)
        ident = [_new_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        comm = _comm(world, rank, ident[0])
        st = torch.cuda.current_stream().cuda_stream
        ok = True
        g = torch.Generator().manual_seed(43)
        x = 0.5 + 2.0 * torch.randn(8, 16, 6, 6, generator=g)            # same tensor on every rank
        op = ops.BnStats(sharding.shard_batch(x, rank, world).contiguous().to(dev), 1e-5, want_moments=True)
        ops.run(op)
        mean, invstd = torch.empty(16, device=dev), torch.empty(16, device=dev)
        ok &= L.hfuse_bnstats_allreduce_nccl_f64(comm, op.moments.data_ptr(), 16, 1e-5, mean.data_ptr(),
                                                 invstd.data_ptr(), st) == 0
        mr, sr = dl.bnstats_f64(x, 1e-5)
        ok &= np.allclose(mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5, atol=0)
        ok &= np.allclose(invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5, atol=0)
        h = torch.randn(50001, generator=g)
        cnt = ops.histc(sharding.shard_flat(h, rank, world).contiguous().to(dev), 64, -3.0, 3.0)
        ok &= L.hfuse_histc_allreduce_counts(comm, cnt.data_ptr(), 64, st) == 0
        ok &= np.array_equal(cnt.cpu().numpy().view(np.uint32), dl.histc_numpy(h.numpy(), 64, -3.0, 3.0))
        want = workloads.xoshiro_bytes(5, 128 * 4096)
        dag = torch.from_numpy(want).to(dev) if rank == 0 else torch.zeros(128 * 4096, dtype=torch.uint8, device=dev)
        ok &= L.hfuse_dag_broadcast(comm, dag.data_ptr(), dag.numel(), 0, st) == 0
        ok &= np.array_equal(dag.cpu().numpy(), want)
        torch.cuda.synchronize()
        ret[rank] = bool(ok)
        dist.barrier()
        L.hfuse_comm_destroy(comm)
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_nccl(dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29800 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert ret[0] and ret[1]
