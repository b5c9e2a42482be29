"""The two backward kernels (standalone and as a fused pair) against PyTorch's CPU operators."""
import numpy as np
import pytest
import torch

from hfuse_b200 import ops
from oracle import dl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,prm", [((2, 3, 8, 16), (2, 2, 2, 2, 0, 0, 1, 1)), ((2, 2, 9, 10), (3, 3, 2, 1, 1, 1, 1, 1)),
                                       ((1, 2, 7, 7), (3, 2, 1, 2, 1, 1, 2, 2)), ((3, 1, 5, 5), (3, 3, 1, 1, 1, 1, 1, 1))])
def test_maxpool_backward(dev, shape, prm):
    g = torch.Generator().manual_seed(61)
    x = torch.randint(0, 4, shape, generator=g).float()                       # ties: the index decides
    kh, kw, sh, sw, ph, pw, dh, dw = prm
    fwd = ops.MaxPool(x.to(dev), (kh, kw), (sh, sw), (ph, pw), (dh, dw))
    ops.run(fwd)
    go = torch.randint(-8, 9, tuple(fwd.out.shape), generator=g).float()      # small integers: sums are exact
    got = ops.max_pool2d_backward(fwd, go.to(dev)).cpu()
    vr, ir = dl.maxpool_torch(x, *prm)
    ref = dl.maxpool_backward_torch(x, go, ir, *prm)
    assert torch.equal(got, ref)
    go2 = torch.randn(tuple(fwd.out.shape), generator=g)
    got2 = ops.max_pool2d_backward(fwd, go2.to(dev)).cpu()
    np.testing.assert_allclose(got2.numpy(), dl.maxpool_backward_torch(x, go2, ir, *prm).numpy(), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("shape,with_weight", [((8, 16, 6, 6), True), ((5, 3, 7, 3), False), ((32, 64, 14, 14), True)])
def test_bn_backward(dev, shape, with_weight):
    g = torch.Generator().manual_seed(62)
    x = 0.5 + 2.0 * torch.randn(*shape, generator=g)
    dy = torch.randn(*shape, generator=g)
    w = (torch.rand(shape[1], generator=g) + 0.5) if with_weight else None
    mean, invstd = ops.batch_norm_stats(x.to(dev), 1e-5)
    dx, gw, gb = ops.batch_norm_backward(x.to(dev), dy.to(dev), mean, invstd, w.to(dev) if w is not None else None)
    rdx, rgw, rgb = dl.bn_backward_f64(x, dy, w, 1e-5)
    scale = rdx.abs().max().item()
    np.testing.assert_allclose(dx.cpu().double().numpy(), rdx.numpy(), rtol=1e-4, atol=2e-5 * scale)
    np.testing.assert_allclose(gw.cpu().double().numpy(), rgw.numpy(), rtol=1e-4, atol=1e-4 * rgw.abs().max().item())
    np.testing.assert_allclose(gb.cpu().double().numpy(), rgb.numpy(), rtol=1e-4, atol=1e-4 * rgb.abs().max().item())


def test_fused_backward_pair_equals_standalone(dev):
    g = torch.Generator().manual_seed(63)
    p = torch.rand(4, 8, 16, 16, generator=g)
    fwd = ops.MaxPool(p.to(dev), 2, 2)
    ops.run(fwd)
    go = torch.randn(tuple(fwd.out.shape), generator=g).to(dev)
    x = (0.5 + 2.0 * torch.randn(6, 12, 10, 10, generator=g)).to(dev)
    dy = torch.randn(6, 12, 10, 10, generator=g).to(dev)
    mean, invstd = ops.batch_norm_stats(x, 1e-5)
    ref_gi = ops.max_pool2d_backward(fwd, go)
    ref_dx, ref_gw, ref_gb = ops.batch_norm_backward(x, dy, mean, invstd)
    mp, bn = ops.MaxPoolBackward(fwd, go), ops.BnBackward(x, dy, mean, invstd)
    gi, (dx, gw, gb) = ops.run_backward_pair(mp, bn)
    assert torch.equal(gi, ref_gi)
    np.testing.assert_allclose(dx.cpu().numpy(), ref_dx.cpu().numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(gw.cpu().numpy(), ref_gw.cpu().numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gb.cpu().numpy(), ref_gb.cpu().numpy(), rtol=1e-5, atol=1e-5)
