"""mc_morpho_backward_noalloc, the backward pass for hosts that cannot allocate device memory, against
mc_morpho_backward with a caller workspace. Collected last (file name) so that a failure here cannot
hide another test. Two calls in a row, the second smaller than the first, so the scratch array still
holds the first call's winners when the second one starts."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_pair(C, op, merge, shape, k, seed):
    B, Ci, Co, H, W = shape
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((B, Ci, H, W), generator=g).cuda()
    w = (0.3 * torch.randn((Co, Ci, k, k), generator=g)).cuda()
    gy = torch.randn((B, Co, H, W), generator=g).cuda()
    want_gx, want_gw = C.morpho_backward(op, x, w, gy, merge, "replicate", idx=None)   # winners recomputed into a torch workspace
    d = C.make_desc(op, x, w, merge, "replicate")
    gx, gw = torch.full_like(x, 7.0), torch.full_like(w, 7.0)
    rc = C.lib.mc_morpho_backward_noalloc(ctypes.byref(d), C.ptr(x), C.ptr(w), C.ptr(gy), C.ptr(gx), C.ptr(gw), C.stream())
    C.check(rc)
    torch.cuda.synchronize()
    # same kernels; only the atomic summation order differs between two runs
    np.testing.assert_allclose(gx.cpu().numpy(), want_gx.cpu().numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gw.cpu().numpy(), want_gw.cpu().numpy(), rtol=1e-4, atol=1e-3)
    assert gx.abs().sum().item() > 0


def test_noalloc_matches_workspace_entry_point_twice():
    import _cabi as C
    run_pair(C, "dilation", "max", (3, 4, 6, 45, 83), 5, seed=1)
    run_pair(C, "erosion", "min", (2, 3, 5, 20, 31), 3, seed=2)     # smaller: stale winners remain beyond it
    run_pair(C, "erosion", "sum", (2, 3, 5, 20, 31), 3, seed=3)     # a merge that needs no scratch


def test_noalloc_rejects_oversized_calls():
    import _cabi as C
    x = torch.zeros(1, 1, 8, 8, device="cuda")
    w = torch.zeros(1, 1, 3, 3, device="cuda")
    d = C.make_desc("dilation", x, w, "max")
    d.B, d.Co, d.H, d.W = 64, 64, 64, 64      # 16.8 M output pixels > 4 194 304; rejected before any pointer is read
    rc = C.lib.mc_morpho_backward_noalloc(ctypes.byref(d), C.ptr(x), C.ptr(w), C.ptr(x), C.ptr(x), C.ptr(w), C.stream())
    assert rc == -2
    assert b"built-in scratch" in C.lib.mc_last_error()
