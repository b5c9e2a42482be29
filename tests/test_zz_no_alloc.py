"""The no-allocation batch-norm statistics entry point (hfuse_bnstats_noalloc_f32).

Collected last on purpose: should it fail, a run that stops at the first failure has
already run every other test.  It calls the entry point through the C ABI twice in a row
and compares with hfuse_bnstats_f32, which takes its scratch from the caller.  The
entry point is for callers that cannot allocate device memory when they call (memory
planning phases, plugin interfaces with fixed buffers, threads kept out of the
allocator), so the test also checks that PyTorch's allocator sees no new memory
during the calls.
"""
import numpy as np
import pytest
import torch

from hfuse_b200 import _lib, ops
from oracle import dl

pytestmark = pytest.mark.gpu


def _noalloc(x, eps, mean, invstd):
    N, C = x.shape[0], x.shape[1]
    HW = x.numel() // (N * C)
    rc = _lib.lib().hfuse_bnstats_noalloc_f32(x.data_ptr(), N, C, HW, eps, mean.data_ptr(), invstd.data_ptr(), None,
                                              torch.cuda.current_stream().cuda_stream)
    return rc


def test_two_calls_in_a_row_match_the_workspace_entry_point(dev):
    g = torch.Generator().manual_seed(99)
    # few channels and many values per channel: every channel is cut into slices, so the
    # built-in scratch (tickets and slice moments) is really used; then a many-channel call
    shapes = [(64, 4, 64, 64), (9, 300, 5, 4)]
    xs = [(0.5 + 2.0 * torch.randn(*s, generator=g)).to(dev) for s in shapes]
    refs = [ops.batch_norm_stats(x, 1e-5) for x in xs]
    outs = [(torch.empty(x.shape[1], device=dev), torch.empty(x.shape[1], device=dev)) for x in xs]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    free_after_first = None
    for round_ in range(2):                      # two calls in a row per shape, sharing the array
        for x, (m, s) in zip(xs, outs):
            m.fill_(float("nan"))
            s.fill_(float("nan"))
            assert _noalloc(x, 1e-5, m, s) == 0
        torch.cuda.synchronize()
        if round_ == 0:
            # the first call on a device may make the runtime load the library's device code (that is
            # when the driver places the array); from then on the device's free memory must not move,
            # which PyTorch's own counter could not show (it only sees PyTorch's allocator)
            free_after_first = torch.cuda.mem_get_info(dev)[0]
    assert torch.cuda.memory_allocated(dev) == before
    assert torch.cuda.mem_get_info(dev)[0] == free_after_first
    for x, (m, s), (mr, sr) in zip(xs, outs, refs):
        # same kernel, same launch shape: the tolerance is the one the other BN tests use
        np.testing.assert_allclose(m.cpu().numpy(), mr.cpu().numpy(), rtol=1e-5)
        np.testing.assert_allclose(s.cpu().numpy(), sr.cpu().numpy(), rtol=1e-5)
        m64, s64 = dl.bnstats_f64(x.cpu(), 1e-5)
        np.testing.assert_allclose(m.cpu().double().numpy(), m64.numpy(), rtol=1e-5)
        np.testing.assert_allclose(s.cpu().double().numpy(), s64.numpy(), rtol=1e-5)


def test_sizes_beyond_the_built_in_scratch_are_refused(dev):
    C = _lib.HFUSE_NOALLOC_MAX_CHANNELS + 1
    x = torch.zeros(2, C, 2, 2, device=dev)
    m, s = torch.empty(C, device=dev), torch.empty(C, device=dev)
    rc = _noalloc(x, 1e-5, m, s)
    assert rc == -8
    assert "HFUSE_NOALLOC_MAX_CHANNELS" in _lib.error_string(rc)
