"""Pins the DL oracle: the PyTorch CPU operator and the explicit NumPy restatement of
each kernel must agree, and both must reproduce the committed fixtures."""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import dl

sys.path.insert(0, GOLDEN)
from make_golden import HIST_CASES, IM2COL_CASES, POOL_CASES, UP_CASES  # noqa: E402


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLDEN, "dl_small.npz"))


def test_im2col(gold):
    x = gold["im2col_x"]
    for i, p in enumerate(IM2COL_CASES):
        assert np.array_equal(dl.im2col_numpy(x, *p), gold[f"im2col_{i}"])
        assert np.array_equal(dl.im2col_torch(torch.from_numpy(x), *p).numpy(), gold[f"im2col_{i}"])


def test_maxpool_ties_nan_and_minus_inf(gold):
    x = gold["pool_x"]
    for i, p in enumerate(POOL_CASES):
        v, ix = dl.maxpool_numpy(x, *p)
        assert np.array_equal(v, gold[f"pool_v_{i}"], equal_nan=True)
        assert np.array_equal(ix, gold[f"pool_i_{i}"])
        vt, it = dl.maxpool_torch(torch.from_numpy(x), *p)
        assert np.array_equal(vt.numpy(), v, equal_nan=True) and np.array_equal(it.numpy(), ix)
    # first maximum wins on a tie
    t = np.zeros((1, 1, 2, 2), dtype=np.float32)
    v, ix = dl.maxpool_numpy(t, 2, 2, 2, 2, 0, 0, 1, 1)
    assert ix.item() == 0


def test_bnstats(gold):
    m, s = dl.bnstats_f64(torch.from_numpy(gold["bn_x"]), 1e-5)
    assert np.array_equal(m.numpy(), gold["bn_mean"]) and np.array_equal(s.numpy(), gold["bn_invstd"])
    x = gold["bn_x"].astype(np.float64)
    mean = x.mean(axis=(0, 2, 3))
    var = x.var(axis=(0, 2, 3))
    np.testing.assert_allclose(m.numpy(), mean, rtol=1e-12)
    np.testing.assert_allclose(s.numpy(), 1 / np.sqrt(var + 1e-5), rtol=1e-12)


def test_upsample(gold):
    x = gold["up_x"]
    for i, (oh, ow, ac) in enumerate(UP_CASES):
        mine = dl.upsample_numpy(x, oh, ow, ac)
        assert np.array_equal(mine, gold[f"up_{i}"])
        ref = dl.upsample_torch(torch.from_numpy(x), oh, ow, ac).numpy()
        np.testing.assert_allclose(mine, ref, rtol=1e-5, atol=1e-6)
    # the exact x2 case of the benchmark agrees with torch to 1e-6 relative
    y = np.random.default_rng(0).random((1, 2, 8, 8), dtype=np.float32)
    np.testing.assert_allclose(dl.upsample_numpy(y, 16, 16), dl.upsample_torch(torch.from_numpy(y), 16, 16).numpy(),
                               rtol=1e-6)


def test_histc(gold):
    x = gold["hist_x"]
    for i, (nb, lo, hi) in enumerate(HIST_CASES):
        assert np.array_equal(dl.histc_numpy(x, nb, lo, hi), gold[f"hist_{i}"])
    # power-of-two range: torch's CPU operator gives the same counts
    xs = x[~np.isnan(x)]
    assert np.array_equal(dl.histc_numpy(xs, 256, -4, 4), dl.histc_torch(torch.from_numpy(xs), 256, -4, 4))
    # edges: hi joins the last bin, lo the first, outside and NaN are dropped
    e = np.array([0.0, 1.0, -0.1, 1.1, np.nan, 0.5], dtype=np.float32)
    assert dl.histc_numpy(e, 2, 0.0, 1.0).tolist() == [1, 2]
