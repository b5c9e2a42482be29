"""Seeded random shapes and parameters for every DL kernel against the oracle (bit-exact where
the specification says so), so that every code path (tile, strip, wide-store, generic, ragged
tails, multi-slice statistics) meets shapes nobody hand-picked."""
import numpy as np
import pytest
import torch

from hfuse_b200 import ops
from oracle import dl

pytestmark = pytest.mark.gpu


def _rng(seed):
    return np.random.default_rng(seed), torch.Generator().manual_seed(seed)


def test_im2col_random(dev):
    rng, g = _rng(101)
    for case in range(40):
        fast = case % 2 == 0
        N, C = int(rng.integers(1, 4)), int(rng.integers(1, 5))
        if fast:   # 3x3 stride 1: tile paths (Wc % 4 == 0, sometimes % 8 == 0)
            H, W = int(rng.integers(1, 20)), int(rng.integers(1, 9)) * 4
            prm = (3, 3, 1, 1, 1, 1, 1, 1) if case % 4 == 0 else (3, 3, int(rng.integers(1, 3)), 1, 1, 1, 1, 1)
        else:
            H, W = int(rng.integers(3, 18)), int(rng.integers(3, 18))
            kh, kw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
            dh, dw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
            prm = (kh, kw, int(rng.integers(0, 3)), int(rng.integers(0, 3)), int(rng.integers(1, 3)),
                   int(rng.integers(1, 3)), dh, dw)
        kh, kw, ph, pw, sh, sw, dh, dw = prm
        if H + 2 * ph < dh * (kh - 1) + 1 or W + 2 * pw < dw * (kw - 1) + 1:
            continue
        x = torch.rand(N, C, H, W, generator=g) * 2 - 1
        got = ops.im2col(x.to(dev), (kh, kw), (ph, pw), (sh, sw), (dh, dw)).cpu()
        assert torch.equal(got, dl.im2col_torch(x, *prm)), (x.shape, prm)


def test_maxpool_random(dev):
    rng, g = _rng(102)
    for case in range(40):
        N, C = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        if case % 2 == 0:
            H, W = int(rng.integers(1, 10)) * 2, int(rng.integers(1, 6)) * 8
            prm = (2, 2, 2, 2, 0, 0, 1, 1)
        else:
            kh, kw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
            prm = (kh, kw, int(rng.integers(1, 4)), int(rng.integers(1, 4)), int(rng.integers(0, kh // 2 + 1)),
                   int(rng.integers(0, kw // 2 + 1)), int(rng.integers(1, 3)), int(rng.integers(1, 3)))
            H, W = int(rng.integers(6, 20)), int(rng.integers(6, 20))
        kh, kw, sh, sw, ph, pw, dh, dw = prm
        x = torch.randint(-2, 3, (N, C, H, W), generator=g).float()        # ties everywhere
        if case % 5 == 0:
            x.view(-1)[int(rng.integers(0, x.numel()))] = float("nan")
        v, ix = ops.max_pool2d_with_indices(x.to(dev), (kh, kw), (sh, sw), (ph, pw), (dh, dw))
        vr, ir = dl.maxpool_torch(x, *prm)
        assert np.array_equal(v.cpu().numpy(), vr.numpy(), equal_nan=True), (x.shape, prm)
        assert torch.equal(ix.cpu(), ir), (x.shape, prm)


def test_upsample_random(dev):
    rng, g = _rng(103)
    for case in range(40):
        N, C = int(rng.integers(1, 3)), int(rng.integers(1, 4))
        H, W = int(rng.integers(1, 12)), int(rng.integers(1, 12))
        if case % 3 == 0:
            W = int(rng.integers(1, 5)) * 4
            oh, ow, ac = 2 * H, 2 * W, False                                 # strip path
        else:
            oh, ow, ac = int(rng.integers(1, 30)), int(rng.integers(1, 30)), bool(rng.integers(0, 2))
        x = torch.rand(N, C, H, W, generator=g)
        got = ops.upsample_bilinear2d(x.to(dev), (oh, ow), align_corners=ac).cpu().numpy()
        assert np.array_equal(got, dl.upsample_numpy(x.numpy(), oh, ow, ac)), (x.shape, oh, ow, ac)


def test_bnstats_random(dev):
    rng, g = _rng(104)
    for case in range(30):
        N, C = int(rng.integers(1, 40)), int(rng.integers(1, 40))
        hw = int(rng.integers(1, 400))
        x = torch.randn(N, C, hw, generator=g) * float(rng.uniform(0.1, 5)) + float(rng.uniform(-20, 20))
        m, s = ops.batch_norm_stats(x.to(dev), 1e-5)
        mr, sr = dl.bnstats_f64(x, 1e-5)
        np.testing.assert_allclose(m.cpu().double().numpy(), mr.numpy(), rtol=1e-5, atol=1e-6, err_msg=str(x.shape))
        np.testing.assert_allclose(s.cpu().double().numpy(), sr.numpy(), rtol=1e-5, err_msg=str(x.shape))


def test_histc_random(dev):
    rng, g = _rng(105)
    for case in range(30):
        n = int(rng.integers(0, 200000))
        nb = int(rng.choice([1, 2, 7, 64, 256, 257, 1000, 5000]))
        lo = float(np.float32(rng.uniform(-5, 0)))
        hi = float(np.float32(lo + rng.uniform(0.5, 8)))
        x = torch.randn(n, generator=g) * 2
        op = ops.Histc(x.to(dev) if n else torch.empty(0, device=dev), nb, lo, hi)
        got = ops.run(op).cpu().numpy().view(np.uint32)
        assert np.array_equal(got, dl.histc_numpy(x.numpy(), nb, lo, hi)), (n, nb, lo, hi)
