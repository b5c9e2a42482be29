"""Fused pairs: every pair, through the C ABI, must give exactly the bytes of its two
standalone kernels (which test_gpu_dl.py checks against the oracle), for every compiled
split variant; the benchmark configurations are checked against the oracle directly."""
import numpy as np
import pytest
import torch

from hfuse_b200 import _lib, ops, workloads
from oracle import dl

pytestmark = pytest.mark.gpu


def _mk(key, dev, big=False):
    g = torch.Generator().manual_seed(100 + len(key))
    if key == "im2col":
        return ops.Im2col((torch.rand(3, 5, 20, 24, generator=g) * 2 - 1).to(dev), 3, 1, 1, 1)
    if key == "maxpool":
        return ops.MaxPool(torch.randint(0, 5, (3, 5, 24, 32), generator=g).float().to(dev), 2, 2)
    if key == "bnstats":
        return ops.BnStats((0.5 + 2 * torch.randn(9, 7, 12, 12, generator=g)).to(dev), 1e-5)
    if key == "upsample":
        return ops.Upsample(torch.rand(3, 5, 12, 16, generator=g).to(dev), scale_factor=2)
    if key == "histc":
        return ops.Histc(torch.randn(2_000_003, generator=g).to(dev), 64, -3.0, 3.0)    # several chunks per block on the bulk-load path
    raise KeyError(key)


def _snapshot(op):
    r = op.result()
    return [t.clone() for t in (r if isinstance(r, tuple) else (r,))]


def _same(a, b):
    return all(torch.equal(x.view(torch.int32) if x.dtype == torch.float32 else x,
                           y.view(torch.int32) if y.dtype == torch.float32 else y) for x, y in zip(a, b))


@pytest.mark.parametrize("pair", sorted(_lib.DL_PAIRS))
def test_fused_equals_standalone_for_every_variant(dev, pair):
    ka, kb = _lib.DL_PAIRS[pair]
    a, b = _mk(ka, dev), _mk(kb, dev)
    ops.run(a)
    ops.run(b)
    ra, rb = _snapshot(a), _snapshot(b)
    try:
        paths = [(ip, hp) for ip in ((0, 1) if "im2col" in pair else (None,))       # both store paths of the im2col role
                 for hp in ((0, 1) if "histc" in pair else (None,))]                # both load paths of the histogram role
        for path in paths:
            if path[0] is not None:
                _lib.tune_option("im2col_store_path", path[0])
            if path[1] is not None:
                _lib.tune_option("histc_load_path", path[1])
            for v in range(len(_lib.tune_variants(pair))):
                _lib.tune_set(pair, v, 0)
                for t in a.result() if isinstance(a.result(), tuple) else (a.result(),):
                    t.fill_(0) if t.dtype != torch.int64 else t.fill_(-1)
                for t in b.result() if isinstance(b.result(), tuple) else (b.result(),):
                    t.fill_(0) if t.dtype != torch.int64 else t.fill_(-1)
                ops.run_pair(a, b)
                if ka == "bnstats" or kb == "bnstats":
                    # the statistics role splits channels into slices by grid size, so its rounding may
                    # differ between launch shapes: compare within the specified tolerance instead
                    bn_res, bn_ref = (_snapshot(a), ra) if ka == "bnstats" else (_snapshot(b), rb)
                    for x, y in zip(bn_res, bn_ref):
                        np.testing.assert_allclose(x.cpu().numpy(), y.cpu().numpy(), rtol=2e-6)
                    other_res, other_ref = (_snapshot(b), rb) if ka == "bnstats" else (_snapshot(a), ra)
                    assert _same(other_res, other_ref), (pair, path, v)
                else:
                    assert _same(_snapshot(a), ra) and _same(_snapshot(b), rb), (pair, path, v)
    finally:
        _lib.tune_set(pair, -1, 0)
        _lib.tune_option("im2col_store_path", -1)
        _lib.tune_option("histc_load_path", -1)


def test_pair_config0_against_oracle(dev):
    w = workloads.config0()
    a = ops.Im2col(w["im"].to(dev), **w["im2col"])
    b = ops.MaxPool(w["pool"].to(dev), **w["maxpool"])
    ops.run_pair(a, b)
    assert torch.equal(a.out.cpu(), dl.im2col_torch(w["im"], 3, 3, 1, 1, 1, 1, 1, 1))
    vr, ir = dl.maxpool_torch(w["pool"], 2, 2, 2, 2, 0, 0, 1, 1)
    assert torch.equal(b.out.cpu(), vr) and torch.equal(b.idx.cpu(), ir)


def test_pair_config1_against_oracle(dev):
    w = workloads.config1()
    a = ops.Upsample(w["up"].to(dev), scale_factor=2)
    b = ops.BnStats(w["bn"].to(dev), w["eps"])
    ops.run_pair(a, b)
    ref = dl.upsample_torch(w["up"], 112, 112)
    assert ((a.out.cpu() - ref).abs() <= 1e-6 * ref.abs()).all()
    assert np.array_equal(a.out.cpu().numpy(), dl.upsample_numpy(w["up"].numpy(), 112, 112))
    mr, sr = dl.bnstats_f64(w["bn"], w["eps"])
    np.testing.assert_allclose(b.mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
    np.testing.assert_allclose(b.invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)


def test_pair_config2_at_full_size_against_oracle(dev):
    """Configuration 2 as the benchmark runs it: im2col of batch 32 fused with histc over 2^24 values."""
    w = workloads.config2()
    assert w["im"].shape[0] == 32 and w["hist"].numel() == 1 << 24
    a = ops.Im2col(w["im"].to(dev), **w["im2col"])
    b = ops.Histc(w["hist"].to(dev), w["bins"], w["lo"], w["hi"])
    b.counts.fill_(-3)                                 # the entry point clears the counts itself
    ops.run_pair(a, b)
    assert np.array_equal(b.counts.cpu().numpy().view(np.uint32), dl.histc_torch(w["hist"], 256, -4, 4))
    assert np.array_equal(b.counts.cpu().numpy().view(np.uint32), dl.histc_numpy(w["hist"].numpy(), 256, -4.0, 4.0))
    ref_col = dl.im2col_torch(w["im"], 3, 3, 1, 1, 1, 1, 1, 1)
    assert torch.equal(a.out.cpu(), ref_col)


def test_pair_config2_against_oracle_and_batch_sharding(dev):
    from hfuse_b200 import sharding
    w = workloads.config2(n_hist=1 << 22, batch=8)
    a = ops.Im2col(w["im"].to(dev), **w["im2col"])
    b = ops.Histc(w["hist"].to(dev), w["bins"], w["lo"], w["hi"])
    ops.run_pair(a, b)
    ref_col = dl.im2col_torch(w["im"], 3, 3, 1, 1, 1, 1, 1, 1)
    ref_cnt = dl.histc_torch(w["hist"], 256, -4, 4)
    assert torch.equal(a.out.cpu(), ref_col)
    assert np.array_equal(b.counts.cpu().numpy().view(np.uint32), ref_cnt)
    # the same work cut into 4 rank-shards: concatenated im2col slices and summed counts are identical
    cols, total = [], torch.zeros(256, dtype=torch.int32, device=dev)
    for r in range(4):
        ar = ops.Im2col(sharding.shard_batch(w["im"], r, 4).contiguous().to(dev), **w["im2col"])
        br = ops.Histc(sharding.shard_flat(w["hist"], r, 4).contiguous().to(dev), w["bins"], w["lo"], w["hi"])
        ops.run_pair(ar, br)
        cols.append(ar.out.cpu())
        total += br.counts
    assert torch.equal(torch.cat(cols), ref_col)
    assert np.array_equal(total.cpu().numpy().view(np.uint32), ref_cnt)
