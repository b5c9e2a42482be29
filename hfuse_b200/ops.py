"""Python call harness for the deep-learning kernels and their fused pairs.

Plays the part of the reference's `TorchKernel/call_{1080,v100}.py` harness
(README.md:84-95 of aoli-al/HFuse): it hands CUDA tensors to the fused entry
points.  PyTorch only supplies device memory and the current stream; every
operator below runs a hand-written sm_100a kernel through the C ABI, and
raises if the tensors are not on a CUDA device — there is no CPU path.

An operator is described by a small object (`Im2col`, `MaxPool`, `BnStats`,
`Upsample`, `Histc`) that owns its output buffers; `run(op)` launches the
standalone kernel, `run_pair(a, b)` launches the fused pair named after the
two halves (the ten pairs of the reference's configs/ml_fusion.yaml).
"""
from __future__ import annotations

import torch

from . import _lib


def _check_input(x: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: hfuse_b200 has no CPU path")
    if x.dtype != torch.float32:
        raise TypeError(f"{name} must be float32, got {x.dtype}")
    if not x.is_contiguous():
        raise ValueError(f"{name} must be contiguous (NCHW)")
    return x


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class Im2col:
    """unfold: x [N,C,H,W] -> col [N, C*kh*kw, Hc*Wc]"""
    key = "im2col"

    def __init__(self, x, kernel_size, padding=0, stride=1, dilation=1, out=None):
        self.x = _check_input(x, "im2col input")
        if x.dim() != 4:
            raise ValueError("im2col input must be 4-D")
        (self.kh, self.kw), (self.ph, self.pw) = _pair(kernel_size), _pair(padding)
        (self.sh, self.sw), (self.dh, self.dw) = _pair(stride), _pair(dilation)
        N, C, H, W = x.shape
        Hc = (H + 2 * self.ph - (self.dh * (self.kh - 1) + 1)) // self.sh + 1
        Wc = (W + 2 * self.pw - (self.dw * (self.kw - 1) + 1)) // self.sw + 1
        if Hc <= 0 or Wc <= 0:
            raise ValueError("im2col: kernel does not fit the padded input")
        self.Hc, self.Wc = Hc, Wc
        self.out = out if out is not None else torch.empty(
            (N, C * self.kh * self.kw, Hc * Wc), dtype=torch.float32, device=x.device)

    def c_args(self):
        N, C, H, W = self.x.shape
        return [self.x.data_ptr(), N, C, H, W, self.kh, self.kw, self.ph, self.pw, self.sh, self.sw,
                self.dh, self.dw, self.out.data_ptr()]

    def result(self):
        return self.out


class MaxPool:
    """max_pool2d_with_indices: x [N,C,H,W] -> (values, int64 indices) [N,C,pH,pW]"""
    key = "maxpool"

    def __init__(self, x, kernel_size, stride=None, padding=0, dilation=1, out=None, indices=None):
        self.x = _check_input(x, "max_pool input")
        if x.dim() != 4:
            raise ValueError("max_pool input must be 4-D")
        (self.kh, self.kw) = _pair(kernel_size)
        (self.sh, self.sw) = _pair(stride) if stride is not None else (self.kh, self.kw)
        (self.ph, self.pw), (self.dh, self.dw) = _pair(padding), _pair(dilation)
        N, C, H, W = x.shape
        self.pH = (H + 2 * self.ph - self.dh * (self.kh - 1) - 1) // self.sh + 1
        self.pW = (W + 2 * self.pw - self.dw * (self.kw - 1) - 1) // self.sw + 1
        if self.pH <= 0 or self.pW <= 0:
            raise ValueError("max_pool: window does not fit the padded input")
        shape = (N, C, self.pH, self.pW)
        self.out = out if out is not None else torch.empty(shape, dtype=torch.float32, device=x.device)
        self.idx = indices if indices is not None else torch.empty(shape, dtype=torch.int64, device=x.device)

    def c_args(self):
        N, C, H, W = self.x.shape
        return [self.x.data_ptr(), N, C, H, W, self.pH, self.pW, self.kh, self.kw, self.sh, self.sw,
                self.ph, self.pw, self.dh, self.dw, self.out.data_ptr(), self.idx.data_ptr()]

    def result(self):
        return self.out, self.idx


_workspaces: dict = {}


def bn_workspace(C: int, device) -> torch.Tensor:
    """Zero-initialised scratch for the statistics kernel, one per (device, stream, C)."""
    key = (str(device), torch.cuda.current_stream(device).cuda_stream, C)
    ws = _workspaces.get(key)
    if ws is None:
        nbytes = _lib.lib().hfuse_bnstats_workspace_bytes(1, C, 1)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


class BnStats:
    """batch_norm_collect_statistics: x [N,C,...] -> (mean[C], invstd[C]); optional fp64 moments [C,3]"""
    key = "bnstats"

    def __init__(self, x, eps=1e-5, want_moments=False, workspace=None):
        self.x = _check_input(x, "batch_norm input")
        if x.dim() < 2:
            raise ValueError("batch_norm input must have at least 2 dimensions")
        self.N, self.C = x.shape[0], x.shape[1]
        self.HW = x.numel() // (self.N * self.C) if self.N * self.C else 0
        self.eps = float(eps)
        self.mean = torch.empty(self.C, dtype=torch.float32, device=x.device)
        self.invstd = torch.empty(self.C, dtype=torch.float32, device=x.device)
        self.moments = torch.empty((self.C, 3), dtype=torch.float64, device=x.device) if want_moments else None
        self.ws = workspace if workspace is not None else bn_workspace(self.C, x.device)

    def c_args(self):
        return [self.x.data_ptr(), self.N, self.C, self.HW, self.eps, self.mean.data_ptr(),
                self.invstd.data_ptr(), self.moments.data_ptr() if self.moments is not None else None,
                self.ws.data_ptr(), self.ws.numel()]

    def result(self):
        return self.mean, self.invstd


class Upsample:
    """upsample_bilinear2d: x [N,C,H,W] -> [N,C,outH,outW]"""
    key = "upsample"

    def __init__(self, x, size=None, scale_factor=None, align_corners=False, out=None):
        self.x = _check_input(x, "upsample input")
        if x.dim() != 4:
            raise ValueError("upsample input must be 4-D")
        N, C, H, W = x.shape
        if size is None:
            if scale_factor is None:
                raise ValueError("give size or scale_factor")
            sh, sw = (scale_factor, scale_factor) if not isinstance(scale_factor, (tuple, list)) else scale_factor
            size = (int(H * sh), int(W * sw))
        self.outH, self.outW = _pair(size)
        if self.outH <= 0 or self.outW <= 0:
            raise ValueError("upsample: output size must be positive")
        self.align = bool(align_corners)
        self.out = out if out is not None else torch.empty((N, C, self.outH, self.outW), dtype=torch.float32,
                                                           device=x.device)

    def c_args(self):
        N, C, H, W = self.x.shape
        return [self.x.data_ptr(), N, C, H, W, self.outH, self.outW, int(self.align), self.out.data_ptr()]

    def result(self):
        return self.out


class Histc:
    """histc: all elements of x -> uint32 counts[bins] over [min, max] (stored as int32 bits in torch)"""
    key = "histc"

    def __init__(self, x, bins=100, min=0.0, max=0.0, out=None):
        self.x = _check_input(x, "histc input")
        if bins <= 0:
            raise ValueError("histc: bins must be positive")
        if float(min) == float(max):
            # same rule as torch.histc: derive the range from the data
            if x.numel():
                lo, hi = float(x.min()), float(x.max())
            else:
                lo, hi = 0.0, 0.0
            if lo == hi:
                lo, hi = lo - 1.0, hi + 1.0
            min, max = lo, hi
        if not float(min) < float(max):
            raise ValueError("histc: max must be larger than min")
        self.bins, self.lo, self.hi = int(bins), float(min), float(max)
        self.counts = out if out is not None else torch.empty(self.bins, dtype=torch.int32, device=x.device)

    def c_args(self):
        return [self.x.data_ptr(), self.x.numel(), self.bins, self.lo, self.hi, self.counts.data_ptr()]

    def result(self):
        return self.counts


def run(op, stream=None):
    """Launch the standalone kernel of one operator on the current (or given) stream."""
    fn = getattr(_lib.lib(), _lib.DL_SOLO[op.key])
    _lib.check(fn(*op.c_args(), _stream_ptr(stream)), _lib.DL_SOLO[op.key])
    return op.result()


def pair_name(a, b) -> str:
    name = f"{a.key}_{b.key}"
    if name not in _lib.DL_PAIRS:
        raise KeyError(f"no fused pair {name}; the pairs are {sorted(_lib.DL_PAIRS)}")
    return name


def run_pair(a, b, stream=None):
    """Launch the fused pair (a, b) as ONE kernel."""
    name = pair_name(a, b)
    fn = getattr(_lib.lib(), f"hfuse_{name}_f32")
    _lib.check(fn(*a.c_args(), *b.c_args(), _stream_ptr(stream)), f"hfuse_{name}_f32")
    return a.result(), b.result()


def run_back_to_back(a, b, stream=None):
    """The unfused baseline: the two standalone kernels queued on one stream with no
    host synchronisation in between (the reference's "ST" measurement,
    scripts/analyze_nvprof.py:264-284)."""
    return run(a, stream), run(b, stream)


# ---- functional conveniences, named after the torch operators they stand in for --------
def im2col(x, kernel_size, padding=0, stride=1, dilation=1):
    return run(Im2col(x, kernel_size, padding, stride, dilation))


def max_pool2d_with_indices(x, kernel_size, stride=None, padding=0, dilation=1):
    return run(MaxPool(x, kernel_size, stride, padding, dilation))


def batch_norm_stats(x, eps=1e-5):
    return run(BnStats(x, eps))


def upsample_bilinear2d(x, size=None, scale_factor=None, align_corners=False):
    return run(Upsample(x, size, scale_factor, align_corners))


def histc(x, bins=100, min=0.0, max=0.0):
    return run(Histc(x, bins, min, max))


def bn_finalize(moments: torch.Tensor, eps: float):
    """mean / invstd from fp64 moments [C,3] that were summed over GPUs."""
    if not moments.is_cuda or moments.dtype != torch.float64 or not moments.is_contiguous():
        raise ValueError("moments must be a contiguous CUDA float64 tensor [C,3]")
    Cn = moments.shape[0]
    mean = torch.empty(Cn, dtype=torch.float32, device=moments.device)
    invstd = torch.empty(Cn, dtype=torch.float32, device=moments.device)
    _lib.check(_lib.lib().hfuse_bnstats_finalize_f64(moments.data_ptr(), Cn, float(eps), mean.data_ptr(),
                                                     invstd.data_ptr(), _stream_ptr()),
               "hfuse_bnstats_finalize_f64")
    return mean, invstd


# ---- backward kernels (listed by the reference next to the forward ones, never fused there) ------
class MaxPoolBackward:
    """grad_in of max_pool2d from grad_out and the indices a MaxPool operator wrote."""

    def __init__(self, fwd: MaxPool, grad_out: torch.Tensor):
        self.fwd = fwd
        self.grad_out = _check_input(grad_out, "max_pool grad_out")
        if tuple(grad_out.shape) != tuple(fwd.out.shape):
            raise ValueError("grad_out must have the shape of the pooled output")
        self.grad_in = torch.empty_like(fwd.x)

    def c_args(self):
        f = self.fwd
        N, C, H, W = f.x.shape
        return [self.grad_out.data_ptr(), f.idx.data_ptr(), N, C, H, W, f.pH, f.pW, f.kh, f.kw, f.sh, f.sw, f.ph, f.pw,
                f.dh, f.dw, self.grad_in.data_ptr()]


class BnBackward:
    """Training-mode batch-norm backward from the saved mean / invstd of the statistics kernel."""

    def __init__(self, x, grad_out, mean, invstd, weight=None):
        self.x, self.dy = _check_input(x, "batch_norm input"), _check_input(grad_out, "batch_norm grad_out")
        if x.shape != grad_out.shape:
            raise ValueError("grad_out must have the shape of the input")
        self.N, self.C = x.shape[0], x.shape[1]
        self.HW = x.numel() // (self.N * self.C)
        self.mean, self.invstd, self.weight = mean, invstd, weight
        self.dx = torch.empty_like(x)
        self.grad_weight = torch.empty(self.C, dtype=torch.float32, device=x.device)
        self.grad_bias = torch.empty(self.C, dtype=torch.float32, device=x.device)

    def c_args(self):
        return [self.x.data_ptr(), self.dy.data_ptr(), self.N, self.C, self.HW,
                self.weight.data_ptr() if self.weight is not None else None, self.mean.data_ptr(),
                self.invstd.data_ptr(), self.dx.data_ptr(), self.grad_weight.data_ptr(), self.grad_bias.data_ptr()]


def max_pool2d_backward(fwd: MaxPool, grad_out, stream=None):
    op = MaxPoolBackward(fwd, grad_out)
    _lib.check(_lib.lib().hfuse_maxpool2d_backward_f32(*op.c_args(), _stream_ptr(stream)), "hfuse_maxpool2d_backward_f32")
    return op.grad_in


def batch_norm_backward(x, grad_out, mean, invstd, weight=None, stream=None):
    op = BnBackward(x, grad_out, mean, invstd, weight)
    _lib.check(_lib.lib().hfuse_bn_backward_f32(*op.c_args(), _stream_ptr(stream)), "hfuse_bn_backward_f32")
    return op.dx, op.grad_weight, op.grad_bias


def run_backward_pair(mp: MaxPoolBackward, bn: BnBackward, stream=None):
    """max-pool backward and batch-norm backward in ONE fused launch."""
    _lib.check(_lib.lib().hfuse_maxpool_backward_bn_backward_f32(*mp.c_args(), *bn.c_args(), _stream_ptr(stream)),
               "hfuse_maxpool_backward_bn_backward_f32")
    return mp.grad_in, (bn.dx, bn.grad_weight, bn.grad_bias)
