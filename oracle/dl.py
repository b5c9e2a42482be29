"""CPU oracle for the five deep-learning operators on the fused hot path.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
CPU-baseline leg of the benchmark, never by the shipped package.

Parity status: "parity unpinned" by the reference.  aoli-al/HFuse names these
kernels (configs/ml_kernels.yaml:1-45) and records their signatures in its
profiler traces (scripts/data/ml-event.csv:5,14,17,32,33) but ships neither
their source (they live in the un-vendored aoli-al/TorchKernel and
aoli-al/pytorch repositories, scripts/docker/Dockerfile:30-35) nor any golden
outputs.  Each operator is therefore stated twice here: through the PyTorch
CPU operator that descends from the same kernel family (`*_torch`), and as an
explicit NumPy restatement of the kernel's arithmetic (`*_numpy`); the tests
require both to agree and commit fixtures generated from them.

Semantics fixed here (and in the CUDA code):
  im2col   col[n, (c*kh+i)*kw+j, h*Wc+w] = im[n, c, h*sh-ph+i*dh, w*sw-pw+j*dw], 0 outside
  maxpool  scan the window in (h, w) order from -inf; a value replaces the
           maximum when it is strictly greater or is NaN; index = h*W + w of
           the kept element inside its (n, c) plane, int64; an untouched
           window reports its first in-range corner
  bnstats  biased variance over (N, HW) per channel, invstd = 1/sqrt(var+eps)
  upsample src = max(0, r*(dst+0.5)-0.5) (or r*dst when align_corners),
           r = in/out (or (in-1)/(out-1)); i1 = int(src), lambda1 = src-i1,
           out = h0*(w0*a + w1*b) + h1*(w0*c + w1*d)
  histc    bin = int((v-lo)*nbins/(hi-lo)) in fp32, v == hi joins the last
           bin, values outside [lo, hi] and NaN are dropped
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ im2col
def im2col_out_hw(H, W, kh, kw, ph, pw, sh, sw, dh, dw):
    Hc = (H + 2 * ph - (dh * (kh - 1) + 1)) // sh + 1
    Wc = (W + 2 * pw - (dw * (kw - 1) + 1)) // sw + 1
    return Hc, Wc


def im2col_torch(x: torch.Tensor, kh, kw, ph, pw, sh, sw, dh, dw) -> torch.Tensor:
    return F.unfold(x, (kh, kw), dilation=(dh, dw), padding=(ph, pw), stride=(sh, sw))


def im2col_numpy(x: np.ndarray, kh, kw, ph, pw, sh, sw, dh, dw) -> np.ndarray:
    N, C, H, W = x.shape
    Hc, Wc = im2col_out_hw(H, W, kh, kw, ph, pw, sh, sw, dh, dw)
    out = np.zeros((N, C * kh * kw, Hc * Wc), dtype=x.dtype)
    hs = np.arange(Hc)[:, None] * sh - ph
    ws = np.arange(Wc)[None, :] * sw - pw
    for i in range(kh):
        for j in range(kw):
            hi, wi = hs + i * dh, ws + j * dw
            ok = (hi >= 0) & (hi < H) & (wi >= 0) & (wi < W)
            g = x[:, :, np.clip(hi, 0, H - 1), np.clip(wi, 0, W - 1)] * ok
            out[:, (np.arange(C) * kh + i) * kw + j, :] = g.reshape(N, C, Hc * Wc)
    return out


# ------------------------------------------------------------------ max pool
def pool_out(n, k, s, p, d):
    return (n + 2 * p - d * (k - 1) - 1) // s + 1


def maxpool_torch(x: torch.Tensor, kh, kw, sh, sw, ph, pw, dh, dw):
    return F.max_pool2d(x, (kh, kw), (sh, sw), (ph, pw), (dh, dw), return_indices=True)


def maxpool_numpy(x: np.ndarray, kh, kw, sh, sw, ph, pw, dh, dw):
    """Explicit scan (small inputs only)."""
    N, C, H, W = x.shape
    pH, pW = pool_out(H, kh, sh, ph, dh), pool_out(W, kw, sw, pw, dw)
    val = np.empty((N, C, pH, pW), dtype=x.dtype)
    idx = np.empty((N, C, pH, pW), dtype=np.int64)
    for oh in range(pH):
        hstart = oh * sh - ph
        hend = min(hstart + (kh - 1) * dh + 1, H)
        while hstart < 0:
            hstart += dh
        for ow in range(pW):
            wstart = ow * sw - pw
            wend = min(wstart + (kw - 1) * dw + 1, W)
            while wstart < 0:
                wstart += dw
            best = np.full((N, C), -np.inf, dtype=x.dtype)
            bidx = np.full((N, C), hstart * W + wstart, dtype=np.int64)
            for h in range(hstart, hend, dh):
                for w in range(wstart, wend, dw):
                    v = x[:, :, h, w]
                    take = (v > best) | np.isnan(v)
                    best = np.where(take, v, best)
                    bidx = np.where(take, h * W + w, bidx)
            val[:, :, oh, ow] = best
            idx[:, :, oh, ow] = bidx
    return val, idx


# ------------------------------------------------------------------ batch-norm statistics
def bnstats_f64(x: torch.Tensor, eps: float):
    """x: [N, C, *].  Returns (mean, invstd) as float64 tensors."""
    xd = x.double().reshape(x.shape[0], x.shape[1], -1)
    var, mean = torch.var_mean(xd, dim=(0, 2), unbiased=False)
    return mean, 1.0 / torch.sqrt(var + eps)


def bnstats_f32_torch(x: torch.Tensor, eps: float):
    """fp32 CPU path, used only to time the CPU baseline."""
    xr = x.reshape(x.shape[0], x.shape[1], -1)
    var, mean = torch.var_mean(xr, dim=(0, 2), unbiased=False)
    return mean, torch.rsqrt(var + eps)


# ------------------------------------------------------------------ bilinear upsample
def upsample_torch(x: torch.Tensor, outH, outW, align_corners=False) -> torch.Tensor:
    return F.interpolate(x, size=(outH, outW), mode="bilinear", align_corners=align_corners)


def _src_index(out_n, in_n, align_corners):
    dst = np.arange(out_n, dtype=np.float32)
    if align_corners:
        r = np.float32((in_n - 1) / (out_n - 1)) if out_n > 1 else np.float32(0)
        src = r * dst
    else:
        r = np.float32(in_n / out_n)
        src = np.maximum(np.float32(0), r * (dst + np.float32(0.5)) - np.float32(0.5))
    src = src.astype(np.float32)
    i1 = src.astype(np.int32)
    i1p = (i1 < in_n - 1).astype(np.int32)
    lam1 = (src - i1.astype(np.float32)).astype(np.float32)
    lam0 = (np.float32(1) - lam1).astype(np.float32)
    return i1, i1p, lam0, lam1


def upsample_numpy(x: np.ndarray, outH, outW, align_corners=False) -> np.ndarray:
    """fp32 restatement with every product and sum rounded separately (no FMA)."""
    N, C, H, W = x.shape
    h1, h1p, h0l, h1l = _src_index(outH, H, align_corners)
    w1, w1p, w0l, w1l = _src_index(outW, W, align_corners)
    a = x[:, :, h1][:, :, :, w1]
    b = x[:, :, h1][:, :, :, w1 + w1p]
    c = x[:, :, h1 + h1p][:, :, :, w1]
    d = x[:, :, h1 + h1p][:, :, :, w1 + w1p]
    w0l, w1l = w0l[None, None, None, :], w1l[None, None, None, :]
    h0l, h1l = h0l[None, None, :, None], h1l[None, None, :, None]
    top = (w0l * a).astype(np.float32) + (w1l * b).astype(np.float32)
    bot = (w0l * c).astype(np.float32) + (w1l * d).astype(np.float32)
    return ((h0l * top).astype(np.float32) + (h1l * bot).astype(np.float32)).astype(np.float32)


# ------------------------------------------------------------------ histogram
def histc_torch(x: torch.Tensor, nbins, lo, hi) -> np.ndarray:
    return torch.histc(x.reshape(-1), nbins, lo, hi).to(torch.int64).numpy().astype(np.uint32)


def histc_numpy(x: np.ndarray, nbins, lo, hi) -> np.ndarray:
    v = x.reshape(-1).astype(np.float32)
    lo32, hi32 = np.float32(lo), np.float32(hi)
    keep = (v >= lo32) & (v <= hi32)
    v = v[keep]
    with np.errstate(invalid="ignore"):
        b = (((v - lo32) * np.float32(nbins)) / (hi32 - lo32)).astype(np.int32)
    b = np.where(b == nbins, nbins - 1, b)
    return np.bincount(b, minlength=nbins).astype(np.uint32)


# ------------------------------------------------------------------ backward kernels
def maxpool_backward_torch(x: torch.Tensor, grad_out: torch.Tensor, idx: torch.Tensor, kh, kw, sh, sw, ph, pw, dh, dw):
    return torch.ops.aten.max_pool2d_with_indices_backward(grad_out, x, [kh, kw], [sh, sw], [ph, pw], [dh, dw], False, idx)


def bn_backward_f64(x: torch.Tensor, grad_out: torch.Tensor, weight, eps: float):
    """Training-mode batch-norm backward in float64: (grad_in, grad_weight, grad_bias)."""
    xd, gd = x.double(), grad_out.double()
    dims = [0] + list(range(2, x.dim()))
    mean = xd.mean(dims)
    invstd = 1.0 / torch.sqrt(xd.var(dims, unbiased=False) + eps)
    wd = weight.double() if weight is not None else None
    return torch.ops.aten.native_batch_norm_backward(gd, xd, wd, None, None, mean, invstd, True, eps, [True, True, True])
