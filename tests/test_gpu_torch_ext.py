"""torch.ops.hfuse_b200.*: the PyTorch extension gives the bytes of the ctypes harness and of the oracle."""
import numpy as np
import pytest
import torch

from hfuse_b200 import ops
from oracle import dl

pytestmark = pytest.mark.gpu


def test_extension_pairs_match_harness_and_oracle(dev):
    from hfuse_b200 import torch_ops  # noqa: F401
    T = torch.ops.hfuse_b200
    g = torch.Generator().manual_seed(41)
    x = (torch.rand(2, 3, 12, 16, generator=g) * 2 - 1)
    y = torch.randint(0, 4, (2, 3, 8, 16), generator=g).float()
    col, out, idx = T.im2col_maxpool(x.to(dev), [3, 3], [1, 1], [1, 1], [1, 1], y.to(dev), [2, 2], [2, 2], [0, 0], [1, 1])
    assert torch.equal(col.cpu(), dl.im2col_torch(x, 3, 3, 1, 1, 1, 1, 1, 1))
    vr, ir = dl.maxpool_torch(y, 2, 2, 2, 2, 0, 0, 1, 1)
    assert torch.equal(out.cpu(), vr) and torch.equal(idx.cpu(), ir)

    u = torch.rand(2, 3, 6, 8, generator=g)
    b = 0.5 + 2 * torch.randn(5, 7, 4, 4, generator=g)
    up, mean, invstd = T.upsample_bnstats(u.to(dev), [12, 16], False, b.to(dev), 1e-5)
    assert np.array_equal(up.cpu().numpy(), dl.upsample_numpy(u.numpy(), 12, 16))
    mr, sr = dl.bnstats_f64(b, 1e-5)
    np.testing.assert_allclose(mean.cpu().double().numpy(), mr.numpy(), rtol=1e-5)
    np.testing.assert_allclose(invstd.cpu().double().numpy(), sr.numpy(), rtol=1e-5)

    h = torch.randn(10007, generator=g)
    col2, counts = T.im2col_histc(x.to(dev), [3, 3], [1, 1], [1, 1], [1, 1], h.to(dev), 64, -3.0, 3.0)
    assert torch.equal(col2, col)
    assert np.array_equal(counts.cpu().numpy().view(np.uint32), dl.histc_numpy(h.numpy(), 64, -3, 3))

    # standalone operators agree with the ctypes harness bit for bit
    assert torch.equal(T.im2col(x.to(dev), [3, 3], [1, 1], [1, 1], [1, 1]), ops.im2col(x.to(dev), 3, 1, 1, 1))
    assert torch.equal(T.upsample_bilinear2d(u.to(dev), [12, 16], False), ops.upsample_bilinear2d(u.to(dev), (12, 16)))
    c1 = T.histc(h.to(dev), 64, -3.0, 3.0)
    assert torch.equal(c1, ops.histc(h.to(dev), 64, -3.0, 3.0))
    with pytest.raises(RuntimeError):
        T.im2col(x.to(dev), [9, 99], [0, 0], [1, 1], [1, 1])
