"""Index arithmetic beyond 2^31 elements: the 64-bit paths of the generic kernels.

Inputs are created on the GPU (they are several GB); the checks use properties that need no
CPU copy of the whole tensor: a 1x1 im2col is the identity, and single output pixels of the
upsample are recomputed from the per-output formula."""
import numpy as np
import pytest
import torch

from hfuse_b200 import ops

pytestmark = pytest.mark.gpu


def _room(dev, gib):
    free, _ = torch.cuda.mem_get_info(dev)
    return free > gib * (1 << 30)


def test_im2col_identity_over_more_than_2_31_outputs(dev):
    if not _room(dev, 20):
        pytest.skip("needs 20 GiB of free device memory")
    g = torch.Generator(device=dev).manual_seed(71)
    x = torch.rand(2, 1025, 1024, 1024, device=dev, generator=g)        # 2,149,580,800 elements
    assert x.numel() > 2 ** 31
    col = ops.im2col(x, 1, 0, 1, 1)
    assert col.shape == (2, 1025, 1024 * 1024)
    assert torch.equal(col.view(-1), x.view(-1))


def test_upsample_scalar_path_over_more_than_2_31_outputs(dev):
    if not _room(dev, 14):
        pytest.skip("needs 14 GiB of free device memory")
    H = W = 5793
    g = torch.Generator(device=dev).manual_seed(72)
    x = torch.rand(4, 4, H, W, device=dev, generator=g)
    out = ops.upsample_bilinear2d(x, (2 * H, 2 * W))                     # 2,147,766,336 outputs, outW % 4 == 2
    assert out.numel() > 2 ** 31
    f32 = np.float32

    def ref(n, c, h2, w2):
        def src(d, n):
            s = max(f32(0), f32(0.5) * (f32(d) + f32(0.5)) - f32(0.5))
            i = int(s)
            return i, (1 if i < n - 1 else 0), f32(1) - (f32(s) - f32(i)), f32(s) - f32(i)
        h1, h1p, h0l, h1l = src(h2, H)
        w1, w1p, w0l, w1l = src(w2, W)
        a, b = f32(x[n, c, h1, w1].item()), f32(x[n, c, h1, w1 + w1p].item())
        cc, d = f32(x[n, c, h1 + h1p, w1].item()), f32(x[n, c, h1 + h1p, w1 + w1p].item())
        return f32(f32(h0l * f32(f32(w0l * a) + f32(w1l * b))) + f32(h1l * f32(f32(w0l * cc) + f32(w1l * d))))

    rng = np.random.default_rng(73)
    pts = [(0, 0, 0, 0), (3, 3, 2 * H - 1, 2 * W - 1), (3, 3, 2 * H - 1, 0), (3, 3, 11585, 11584), (2, 1, 7000, 123)]
    pts += [(int(rng.integers(0, 4)), int(rng.integers(0, 4)), int(rng.integers(0, 2 * H)), int(rng.integers(0, 2 * W)))
            for _ in range(40)]
    for n, c, h2, w2 in pts:
        assert f32(out[n, c, h2, w2].item()) == ref(n, c, h2, w2), (n, c, h2, w2)
