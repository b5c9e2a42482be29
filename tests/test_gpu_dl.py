"""GPU parity of the five DL kernels through the C ABI: golden fixtures, the oracle on
seeded inputs, edge cases, and the benchmark configurations at full size."""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from hfuse_b200 import _lib, ops, workloads
from oracle import dl

sys.path.insert(0, GOLDEN)
from make_golden import HIST_CASES, IM2COL_CASES, POOL_CASES, UP_CASES  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLDEN, "dl_small.npz"))


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def test_golden_im2col(dev, gold):
    x = torch.from_numpy(gold["im2col_x"]).to(dev)
    for i, (kh, kw, ph, pw, sh, sw, dh, dw) in enumerate(IM2COL_CASES):
        out = ops.im2col(x, (kh, kw), (ph, pw), (sh, sw), (dh, dw))
        assert np.array_equal(out.cpu().numpy(), gold[f"im2col_{i}"])


def test_golden_maxpool(dev, gold):
    x = torch.from_numpy(gold["pool_x"]).to(dev)
    for i, (kh, kw, sh, sw, ph, pw, dh, dw) in enumerate(POOL_CASES):
        v, ix = ops.max_pool2d_with_indices(x, (kh, kw), (sh, sw), (ph, pw), (dh, dw))
        assert np.array_equal(v.cpu().numpy(), gold[f"pool_v_{i}"], equal_nan=True)
        assert np.array_equal(ix.cpu().numpy(), gold[f"pool_i_{i}"])


def test_golden_bnstats(dev, gold):
    m, s = ops.batch_norm_stats(torch.from_numpy(gold["bn_x"]).to(dev), 1e-5)
    np.testing.assert_allclose(m.cpu().numpy(), gold["bn_mean"], rtol=1e-5)      # tolerance of the benchmark spec
    np.testing.assert_allclose(s.cpu().numpy(), gold["bn_invstd"], rtol=1e-5)


def test_golden_upsample(dev, gold):
    x = torch.from_numpy(gold["up_x"]).to(dev)
    for i, (oh, ow, ac) in enumerate(UP_CASES):
        out = ops.upsample_bilinear2d(x, (oh, ow), align_corners=ac)
        assert np.array_equal(out.cpu().numpy(), gold[f"up_{i}"])                # same roundings as the restatement


def test_golden_histc(dev, gold):
    x = torch.from_numpy(gold["hist_x"]).to(dev)
    for i, (nb, lo, hi) in enumerate(HIST_CASES):
        assert np.array_equal(_u32(ops.histc(x, nb, lo, hi)), gold[f"hist_{i}"])


@pytest.mark.parametrize("shape,prm", [
    ((2, 3, 12, 16), (3, 3, 1, 1, 1, 1, 1, 1)),      # tile path, small
    ((1, 1, 3, 4), (3, 3, 1, 1, 1, 1, 1, 1)),        # tile path, single strip per row
    ((2, 2, 10, 8), (3, 3, 2, 2, 1, 1, 1, 1)),       # tile path with pad 2 (scalar loads)
    ((2, 2, 10, 10), (3, 3, 0, 0, 1, 1, 1, 1)),      # tile path without padding
    ((1, 2, 9, 11), (5, 2, 2, 1, 2, 3, 1, 2)),       # generic path
    ((3, 1, 1, 1), (1, 1, 0, 0, 1, 1, 1, 1)),        # 1x1
])
def test_im2col_shapes(dev, shape, prm):
    g = torch.Generator().manual_seed(11)
    x = torch.rand(*shape, generator=g) * 2 - 1
    kh, kw, ph, pw, sh, sw, dh, dw = prm
    out = ops.im2col(x.to(dev), (kh, kw), (ph, pw), (sh, sw), (dh, dw))
    assert torch.equal(out.cpu(), dl.im2col_torch(x, *prm))


@pytest.mark.parametrize("shape,prm", [
    ((2, 3, 8, 16), (2, 2, 2, 2, 0, 0, 1, 1)),       # 2x2/2 path
    ((1, 1, 2, 8), (2, 2, 2, 2, 0, 0, 1, 1)),        # 2x2/2 path, one output row
    ((2, 3, 9, 10), (2, 2, 2, 2, 0, 0, 1, 1)),       # generic (odd sizes, last row/col dropped)
    ((2, 3, 9, 10), (3, 3, 2, 1, 1, 1, 1, 1)),
    ((1, 2, 7, 7), (3, 2, 1, 2, 1, 1, 2, 2)),
])
def test_maxpool_shapes_with_ties_and_nan(dev, shape, prm):
    g = torch.Generator().manual_seed(12)
    x = torch.randint(0, 3, shape, generator=g).float()       # plenty of exact ties
    x.view(-1)[5] = float("nan")
    x[0, 0, 0] = -float("inf")
    kh, kw, sh, sw, ph, pw, dh, dw = prm
    v, ix = ops.max_pool2d_with_indices(x.to(dev), (kh, kw), (sh, sw), (ph, pw), (dh, dw))
    vr, ir = dl.maxpool_torch(x, *prm)
    assert np.array_equal(v.cpu().numpy(), vr.numpy(), equal_nan=True)
    assert torch.equal(ix.cpu(), ir)


@pytest.mark.parametrize("shape", [(3, 5, 7, 9), (1, 4, 1, 1), (64, 3, 5, 4), (5, 2, 3, 3), (2, 3, 128, 128),
                                   (1, 1, 1, 2), (7, 300, 2, 2)])
def test_bnstats_shapes(dev, shape):
    g = torch.Generator().manual_seed(13)
    x = torch.randn(*shape, generator=g) * 3 + 10           # mean far from zero: cancellation would show
    m, s = ops.batch_norm_stats(x.to(dev), 1e-5)
    mr, sr = dl.bnstats_f64(x, 1e-5)
    np.testing.assert_allclose(m.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
    np.testing.assert_allclose(s.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
    # calling again with the same workspace gives the same answer (the scratch cleans itself)
    m2, s2 = ops.batch_norm_stats(x.to(dev), 1e-5)
    assert torch.equal(m, m2) and torch.equal(s, s2)


def test_bnstats_moments_sum_like_the_allreduce(dev):
    from hfuse_b200 import sharding
    g = torch.Generator().manual_seed(14)
    x = 0.5 + 2.0 * torch.randn(8, 16, 6, 6, generator=g)
    parts = []
    for r in range(4):
        op = ops.BnStats(sharding.shard_batch(x, r, 4).contiguous().to(dev), 1e-5, want_moments=True)
        ops.run(op)
        parts.append(op.moments)
    total = torch.stack(parts).sum(0).contiguous()
    mean, invstd = ops.bn_finalize(total, 1e-5)
    mr, sr = dl.bnstats_f64(x, 1e-5)
    np.testing.assert_allclose(mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
    np.testing.assert_allclose(invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)


@pytest.mark.parametrize("H,W,oh,ow,ac", [(7, 9, 14, 18, False), (7, 9, 14, 18, True), (7, 9, 10, 13, False),
                                          (7, 9, 5, 20, True), (4, 4, 8, 8, False), (1, 4, 2, 8, False),
                                          (6, 8, 12, 16, False), (5, 12, 10, 24, False), (3, 8, 3, 8, False)])
def test_upsample_shapes(dev, H, W, oh, ow, ac):
    g = torch.Generator().manual_seed(15)
    x = torch.rand(2, 3, H, W, generator=g)
    out = ops.upsample_bilinear2d(x.to(dev), (oh, ow), align_corners=ac).cpu().numpy()
    assert np.array_equal(out, dl.upsample_numpy(x.numpy(), oh, ow, ac))
    np.testing.assert_allclose(out, dl.upsample_torch(x, oh, ow, ac).numpy(), rtol=1e-5, atol=1e-6)


def test_upsample_x2_strip_path_equals_generic_formula_with_nonfinite(dev):
    # inf / nan must propagate exactly as in the per-output formula (0 * inf = nan)
    x = torch.rand(1, 2, 6, 8)
    x[0, 0, 1, 1] = float("inf")
    x[0, 1, 0, 1] = float("nan")
    x[0, 1, 5, 7] = -float("inf")
    out = ops.upsample_bilinear2d(x.to(dev), scale_factor=2).cpu().numpy()
    with np.errstate(invalid="ignore"):
        ref = dl.upsample_numpy(x.numpy(), 12, 16)
    assert np.array_equal(out, ref, equal_nan=True)


@pytest.mark.parametrize("n,nb,lo,hi", [(1000, 10, -1.0, 1.0), (12345, 100, -3.0, 2.5), (7, 5, 0.0, 1.0),
                                        (100003, 5000, -2.0, 2.0), (4096, 1, -10.0, 10.0), (0, 8, 0.0, 1.0),
                                        (3, 4, 0.0, 1.0), (50001, 20000, -1.0, 1.0)])
def test_histc_shapes(dev, n, nb, lo, hi):
    g = torch.Generator().manual_seed(16)
    x = torch.randn(n, generator=g)
    if n >= 3:
        x[0], x[1], x[2] = hi, lo, float("nan")
    got = _u32(ops.histc(x.to(dev), nb, lo, hi)) if n else _u32(ops.run(ops.Histc(torch.empty(0, device=dev), nb, lo, hi)))
    assert np.array_equal(got, dl.histc_numpy(x.numpy(), nb, lo, hi))


def test_histc_edge_values_ragged_sizes_and_dirty_counts_for_every_variant(dev):
    """Values at and next to both bounds, infinities and NaN; sizes around the boundaries of the
    sweep's unchecked main loop (one group = 4 items x threads x blocks); and a counts buffer that
    holds garbage before every call (the entry point clears it on the stream, with a kernel the
    histogram kernel only waits for before its flush)."""
    g = torch.Generator().manual_seed(160)
    f32 = np.float32
    group = 148 * 1024 * 4 * 4
    for nb, lo, hi in ((256, -4.0, 4.0), (100, -3.0, 2.5), (7, 0.1, 0.7), (1000, -1.0, 3.0)):
        edges = [lo, hi, np.nextafter(f32(lo), f32(-np.inf)), np.nextafter(f32(lo), f32(np.inf)),
                 np.nextafter(f32(hi), f32(-np.inf)), np.nextafter(f32(hi), f32(np.inf)),
                 float("inf"), -float("inf"), float("nan"), -0.0, 0.0]
        for n in (11, 4 * 1024 + 1, 8 * 768 * 148 + 5, group - 4, group, group + 7, 2 * group + 4 * 77 + 3):
            x = torch.randn(n, generator=g) * 1.5
            x[:len(edges)] = torch.tensor([float(e) for e in edges])
            want = dl.histc_numpy(x.numpy(), nb, lo, hi)
            xd = x.to(dev)
            op = ops.Histc(xd, nb, lo, hi)
            for path in (0, 1):         # 16-byte loads into registers; bulk copies into a shared-memory ring (up to 256 bins)
                for v in range(len(_lib.tune_variants("histc"))):
                    _lib.tune_set("histc", v, 0)
                    _lib.tune_option("histc_load_path", path)
                    try:
                        op.counts.fill_(-7)
                        assert np.array_equal(_u32(ops.run(op)), want), (nb, lo, hi, n, v, path)
                    finally:
                        _lib.tune_set("histc", -1, 0)
                        _lib.tune_option("histc_load_path", -1)
            # two calls in a row into the same buffer: the second must not see the first's counts
            ops.run(op)
            assert np.array_equal(_u32(ops.run(op)), want)


def test_full_size_configurations(dev):
    w = workloads.config0()
    col = ops.im2col(w["im"].to(dev), **w["im2col"])
    assert torch.equal(col.cpu(), dl.im2col_torch(w["im"], 3, 3, 1, 1, 1, 1, 1, 1))
    v, ix = ops.max_pool2d_with_indices(w["pool"].to(dev), **w["maxpool"])
    vr, ir = dl.maxpool_torch(w["pool"], 2, 2, 2, 2, 0, 0, 1, 1)
    assert torch.equal(v.cpu(), vr) and torch.equal(ix.cpu(), ir)
    del col
    w = workloads.config1()
    m, s = ops.batch_norm_stats(w["bn"].to(dev), w["eps"])
    mr, sr = dl.bnstats_f64(w["bn"], w["eps"])
    np.testing.assert_allclose(m.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
    np.testing.assert_allclose(s.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
    up = ops.upsample_bilinear2d(w["up"].to(dev), scale_factor=2).cpu()
    ref = dl.upsample_torch(w["up"], 112, 112)
    assert ((up - ref).abs() <= 1e-6 * ref.abs()).all()                       # 1e-6 relative, as specified
    w = workloads.config2()
    cnt = ops.histc(w["hist"].to(dev), w["bins"], w["lo"], w["hi"])
    ref = dl.histc_torch(w["hist"], 256, -4, 4)
    assert np.array_equal(_u32(cnt), ref)
    assert int(ref.sum()) + int(((w["hist"] < -4) | (w["hist"] > 4)).sum()) == w["hist"].numel()


def test_every_standalone_variant_gives_the_same_bytes(dev):
    g = torch.Generator().manual_seed(17)
    x = (torch.rand(2, 4, 16, 16, generator=g) * 2 - 1).to(dev)
    base = ops.im2col(x, 3, 1, 1, 1)
    for v in range(len(_lib.tune_variants("im2col"))):
        _lib.tune_set("im2col", v, 0)
        try:
            assert torch.equal(ops.im2col(x, 3, 1, 1, 1), base)
        finally:
            _lib.tune_set("im2col", -1, 0)


def test_im2col_through_shared_memory_and_bulk_stores_gives_the_same_bytes(dev):
    """The alternative store path (option im2col_store_path = 1): 3x3 / stride 1 / pad 1 shapes go
    through a shared-memory tile and bulk copies; every other shape must keep its usual path."""
    g = torch.Generator().manual_seed(19)
    cases = [((2, 3, 12, 16), (3, 3, 1, 1, 1, 1, 1, 1)),     # one band per plane
             ((1, 2, 64, 56), (3, 3, 1, 1, 1, 1, 1, 1)),     # several bands, ragged last band
             ((3, 1, 1, 4), (3, 3, 1, 1, 1, 1, 1, 1)),       # a single row
             ((1, 1, 5, 2048), (3, 3, 1, 1, 1, 1, 1, 1)),    # rows too wide for the tile: usual path
             ((2, 2, 10, 8), (3, 3, 2, 2, 1, 1, 1, 1)),      # pad 2: usual path
             ((1, 2, 9, 11), (5, 2, 2, 1, 2, 3, 1, 2))]      # generic path
    try:
        for path in (0, 1):                                  # both paths, whatever the compiled choice is
            _lib.tune_option("im2col_store_path", path)
            for shape, prm in cases:
                x = torch.rand(*shape, generator=g) * 2 - 1
                kh, kw, ph, pw, sh, sw, dh, dw = prm
                want = dl.im2col_torch(x, *prm)
                for v in range(len(_lib.tune_variants("im2col"))):
                    _lib.tune_set("im2col", v, 0)
                    out = ops.im2col(x.to(dev), (kh, kw), (ph, pw), (sh, sw), (dh, dw))
                    assert torch.equal(out.cpu(), want), (path, shape, prm, v)
                _lib.tune_set("im2col", -1, 0)
        # the benchmark shape, alone and fused with max-pool (another role beside it in the block)
        w = workloads.config0(batch=4)
        a = ops.Im2col(w["im"].to(dev), **w["im2col"])
        b = ops.MaxPool(w["pool"].to(dev), **w["maxpool"])
        want = dl.im2col_torch(w["im"], 3, 3, 1, 1, 1, 1, 1, 1)
        ops.run(a)
        assert torch.equal(a.out.cpu(), want)
        a.out.zero_()
        ops.run_pair(a, b)
        assert torch.equal(a.out.cpu(), want)
        vr, ir = dl.maxpool_torch(w["pool"], 2, 2, 2, 2, 0, 0, 1, 1)
        assert torch.equal(b.out.cpu(), vr) and torch.equal(b.idx.cpu(), ir)
        h = ops.Histc(torch.randn(100000, generator=g).to(dev), 256, -4.0, 4.0)      # 32 KB more shared memory
        a.out.zero_()
        ops.run_pair(a, h)
        assert torch.equal(a.out.cpu(), want)
    finally:
        _lib.tune_option("im2col_store_path", -1)
        _lib.tune_set("im2col", -1, 0)
    with pytest.raises(_lib.HfuseError):
        _lib.tune_option("no_such_option", 1)


def test_bnstats_through_bulk_loads_into_shared_memory(dev):
    """The alternative load path (option bnstats_load_path = 1): channels whose image rows are 1 to
    25 KB long come into shared memory through bulk copies counted on an mbarrier; every block
    shape, alone and beside another role; shapes outside that range keep the register path."""
    g = torch.Generator().manual_seed(23)
    cases = [(32, 20, 28, 28),       # the benchmark's rows (3,136 B), four equal buffer fills
             (5, 3, 16, 16),         # a single, short fill per channel (1,024 B rows)
             (19, 7, 20, 20),        # ragged last fill
             (3, 700, 16, 20),       # more channels than blocks: several units per block
             (2, 4, 80, 80),         # 25,600 B rows: one row per buffer
             (4, 5, 81, 80),         # rows too long: register path
             (6, 9, 6, 6)]           # rows too short: register path
    try:
        for path in (1, 0):
            _lib.tune_option("bnstats_load_path", path)
            for shape in cases:
                x = (0.5 + 2.0 * torch.randn(*shape, generator=g))
                mr, sr = dl.bnstats_f64(x, 1e-5)
                xd = x.to(dev)
                for v in range(len(_lib.tune_variants("bnstats"))):
                    _lib.tune_set("bnstats", v, 0)
                    op = ops.BnStats(xd, 1e-5, want_moments=True)
                    ops.run(op)
                    mean, invstd = op.result()
                    np.testing.assert_allclose(mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5, atol=1e-6, err_msg=str((path, shape, v)))
                    np.testing.assert_allclose(invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5, err_msg=str((path, shape, v)))
                    m2, s2 = ops.bn_finalize(op.moments, 1e-5)
                    np.testing.assert_allclose(m2.cpu().double().numpy(), mr.numpy(), rtol=1e-5, atol=1e-6)
                    np.testing.assert_allclose(s2.cpu().double().numpy(), sr.numpy(), rtol=1e-5)
                _lib.tune_set("bnstats", -1, 0)
            # beside another role in the block, every split (the partner's shared memory lies in front)
            x = (0.5 + 2.0 * torch.randn(8, 40, 28, 28, generator=g))
            mr, sr = dl.bnstats_f64(x, 1e-5)
            up_in = torch.rand(2, 6, 12, 16, generator=g)
            want_up = dl.upsample_numpy(up_in.numpy(), 24, 32, False)
            hv = torch.randn(50000, generator=g)
            want_h = torch.histc(hv, 256, -4.0, 4.0)
            for name, mk in (("upsample_bnstats", lambda: ops.Upsample(up_in.to(dev), scale_factor=2)),
                             ("histc_bnstats", lambda: ops.Histc(hv.to(dev), 256, -4.0, 4.0))):
                for v in range(len(_lib.tune_variants(name))):
                    _lib.tune_set(name, v, 0)
                    a, b = mk(), ops.BnStats(x.to(dev), 1e-5)
                    ops.run_pair(a, b)
                    mean, invstd = b.result()
                    np.testing.assert_allclose(mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5, atol=1e-6, err_msg=str((path, name, v)))
                    np.testing.assert_allclose(invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5, err_msg=str((path, name, v)))
                    if name == "upsample_bnstats":
                        assert np.array_equal(a.out.cpu().numpy(), want_up), (path, v)
                    else:
                        assert torch.equal(a.result().cpu().float(), want_h), (path, v)
                _lib.tune_set(name, -1, 0)
    finally:
        _lib.tune_option("bnstats_load_path", -1)
        for name in ("bnstats", "upsample_bnstats", "histc_bnstats"):
            _lib.tune_set(name, -1, 0)


def test_error_codes_on_device_buffers(dev):
    x = torch.zeros(1, 1, 4, 4, device=dev)
    with pytest.raises(ValueError):
        ops.im2col(x, 9, 0)
    with pytest.raises(_lib.HfuseError) as e:
        op = ops.BnStats(torch.zeros(64, 4, 64, 64, device=dev), workspace=torch.zeros(16, dtype=torch.uint8, device=dev))
        ops.run(op)
    assert e.value.code == -4
    with pytest.raises(ValueError):
        ops.Histc(x, 4, 2.0, 1.0)


def _offset16(shape, dtype, dev):
    """A tensor whose storage starts 16 bytes past a 32-byte boundary (allowed by the ABI)."""
    n = int(np.prod(shape))
    step = 16 // torch.empty(0, dtype=dtype).element_size()
    base = torch.empty(n + 2 * step, dtype=dtype, device=dev)
    off = step if base.data_ptr() % 32 == 0 else 0
    t = base[off:off + n].view(*shape)
    assert t.data_ptr() % 32 == 16
    return t


def test_outputs_that_are_only_16_byte_aligned_take_the_narrow_store_paths(dev):
    g = torch.Generator().manual_seed(18)
    x = torch.rand(2, 3, 8, 16, generator=g) * 2 - 1
    col = _offset16((2, 27, 128), torch.float32, dev)
    ops.run(ops.Im2col(x.to(dev), 3, 1, 1, 1, out=col))
    assert torch.equal(col.cpu(), dl.im2col_torch(x, 3, 3, 1, 1, 1, 1, 1, 1))
    up = _offset16((2, 3, 16, 32), torch.float32, dev)
    u = torch.rand(2, 3, 8, 16, generator=g)
    ops.run(ops.Upsample(u.to(dev), scale_factor=2, out=up))
    assert np.array_equal(up.cpu().numpy(), dl.upsample_numpy(u.numpy(), 16, 32))
    idx = _offset16((2, 3, 4, 8), torch.int64, dev)
    p = torch.randint(0, 3, (2, 3, 8, 16), generator=g).float()
    op = ops.MaxPool(p.to(dev), 2, 2, indices=idx)
    ops.run(op)
    vr, ir = dl.maxpool_torch(p, 2, 2, 2, 2, 0, 0, 1, 1)
    assert torch.equal(op.out.cpu(), vr) and torch.equal(idx.cpu(), ir)


def test_hbm_probe_copies_what_it_reads_and_rejects_bad_arguments(dev):
    from hfuse_b200 import _lib
    L = _lib.lib()
    src = torch.randn(4 * 1000, device=dev)
    dst = torch.zeros(8 * 3000, device=dev)
    assert L.hfuse_hbm_probe(src.data_ptr(), src.numel() * 4, dst.data_ptr(), dst.numel() * 4, None) == 0
    got = dst.cpu().view(3000, 2, 4)
    want = src.cpu().view(1000, 4)
    assert torch.equal(got[:1000, 0], want) and torch.equal(got[:1000, 1], want)
    assert torch.equal(got[1000:], torch.tensor([1., 2., 3., 4.]).expand(2000, 2, 4))
    assert L.hfuse_hbm_probe(None, 0, dst.data_ptr(), dst.numel() * 4, None) == 0             # write only
    assert L.hfuse_hbm_probe(src.data_ptr(), 16, dst.data_ptr(), 0, None) == -1
    assert L.hfuse_hbm_probe(src.data_ptr(), 64, dst.data_ptr(), 64, None) == -1              # more loads than stores
    assert L.hfuse_hbm_probe(src.data_ptr(), 16, dst.data_ptr() + 16, 32, None) == -2         # alignment
    # the bulk-store form: 8 KB chunks, the read part of every chunk first, the rest the same constant
    out = torch.zeros(3 * 2048, device=dev)                      # three chunks of 2048 floats
    inp = torch.randn(4 * 600, device=dev)                       # 600 16-byte loads: 200 per chunk
    assert L.hfuse_hbm_probe_bulk(inp.data_ptr(), inp.numel() * 4, out.data_ptr(), out.numel() * 4, None) == 0
    got, want = out.cpu().view(3, 512, 4), inp.cpu().view(3, 200, 4)
    assert torch.equal(got[:, :200], want)
    assert torch.equal(got[:, 200:], torch.tensor([1., 2., 3., 4.]).expand(3, 312, 4))
    assert L.hfuse_hbm_probe_bulk(None, 0, out.data_ptr(), out.numel() * 4, None) == 0        # write only
    assert L.hfuse_hbm_probe_bulk(None, 0, out.data_ptr(), 4096, None) == -1                  # not whole chunks
