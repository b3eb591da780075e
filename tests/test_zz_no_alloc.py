"""fs_apply_mat_static: the one entry point for callers that are not allowed to allocate.

Some users of the library run where no scratch buffer can be created for it: inside another
framework's operator callback (its allocator must not be re-entered), in loops whose memory was
fixed at start-up, or as a plug-in that only receives its input and output buffers. For them
`fs_apply_mat_static` keeps its scratch in a static device array inside the library. This file
checks, through the C ABI, that it returns what the ordinary entry point (caller-provided
workspace) returns, on two calls in a row that share the static array, and that it refuses sizes
beyond the array. It is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from flash_sinkhorn_b200 import _lib

STATIC_MAX_ROWS = 65536
TOL = 2e-4  # the suite's budget for the CUDA-core fp32 engine (both entry points run that engine)


def _problem(seed, n, m, d, dv):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, d, generator=g) / d**0.5
    y = 0.2 + torch.randn(m, d, generator=g) / d**0.5
    f_hat = -0.5 * (x**2).sum(1) + 0.05 * torch.randn(n, generator=g)
    g_hat = -0.5 * (y**2).sum(1) + 0.05 * torch.randn(m, generator=g)
    a = torch.softmax(torch.randn(n, generator=g), 0)
    b = torch.softmax(torch.randn(m, generator=g), 0)
    mat_m = torch.randn(m, dv, generator=g)
    mat_n = torch.randn(n, dv, generator=g)
    scale = torch.randn(m, generator=g)
    return [t.cuda().contiguous() for t in (x, y, f_hat, g_hat, a.log(), b.log(), mat_m, mat_n, scale)]


def _with_workspace(x, y, fh, gh, la, lb, mat, scale, axis, eps, cs):
    n, d = x.shape
    m = y.shape[0]
    dv = mat.shape[1]
    dev = x.device
    out = torch.empty((n if axis == 1 else m, dv), device=dev)
    ws = _lib.workspace(_lib.OP_APPLY_MAT, n, m, d, _lib.PREC_SIMT, dev)
    _lib.call("fs_apply_mat", dev, x.data_ptr(), y.data_ptr(), n, m, d, fh.data_ptr(), gh.data_ptr(), la.data_ptr(),
              lb.data_ptr(), mat.data_ptr(), dv, None if scale is None else scale.data_ptr(), out.data_ptr(),
              eps, axis, cs, _lib.PREC_SIMT, ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev))
    return out


def _static(x, y, fh, gh, la, lb, mat, scale, axis, eps, cs):
    n, d = x.shape
    m = y.shape[0]
    dv = mat.shape[1]
    dev = x.device
    out = torch.empty((n if axis == 1 else m, dv), device=dev)
    _lib.call("fs_apply_mat_static", dev, x.data_ptr(), y.data_ptr(), n, m, d, fh.data_ptr(), gh.data_ptr(),
              la.data_ptr(), lb.data_ptr(), mat.data_ptr(), dv, None if scale is None else scale.data_ptr(),
              out.data_ptr(), eps, axis, cs, _lib.stream_ptr(dev))
    return out


def _close(got, want):
    err = (got - want).abs().max().item()
    return err <= TOL * max(want.abs().max().item(), 1e-30)


@pytest.mark.gpu
def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    eps, cs = 0.3, 0.5
    # first call: larger problem, axis 1 with a per-row scale of the matrix
    x, y, fh, gh, la, lb, mat_m, mat_n, scale = _problem(101, 1500, 1100, 24, 24)
    got1 = _static(x, y, fh, gh, la, lb, mat_m, scale, 1, eps, cs)
    want1 = _with_workspace(x, y, fh, gh, la, lb, mat_m, scale, 1, eps, cs)
    # second call straight after, smaller and transposed: it finds the first call's values in the
    # shared array and must not be affected by them
    x2, y2, fh2, gh2, la2, lb2, mat_m2, mat_n2, _ = _problem(202, 333, 450, 7, 5)
    got2 = _static(x2, y2, fh2, gh2, la2, lb2, mat_n2, None, 0, eps, cs)
    want2 = _with_workspace(x2, y2, fh2, gh2, la2, lb2, mat_n2, None, 0, eps, cs)
    torch.cuda.synchronize()
    assert torch.isfinite(got1).all() and torch.isfinite(got2).all()
    assert want1.abs().max().item() > 0 and want2.abs().max().item() > 0
    assert _close(got1, want1)
    assert _close(got2, want2)
    # and the first problem again: same answer as before (nothing leaked from call two)
    got1b = _static(x, y, fh, gh, la, lb, mat_m, scale, 1, eps, cs)
    torch.cuda.synchronize()
    assert torch.equal(got1b, got1)


@pytest.mark.gpu
def test_static_scratch_entry_at_its_row_limit_and_against_the_oracle():
    """Exactly 65,536 output rows (the last 64-row block of the kernel ends at the end of the static array): the
    static entry and the workspace entry run the same kernels in the same order, so their outputs are equal bit
    for bit. A second, small problem is also compared with the dense fp64 oracle, and the launch counter of the
    library must see the two streaming passes of a static call."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from oracle import dense_sinkhorn as O
    eps, cs = 0.4, 1.0
    x, y, fh, gh, la, lb, mat_m, mat_n, scale = _problem(303, STATIC_MAX_ROWS, 200, 8, 3)
    lib = _lib.load()
    before = lib.fs_launch_count()
    got = _static(x, y, fh, gh, la, lb, mat_m, None, 1, eps, cs)
    assert lib.fs_launch_count() - before == 2
    want = _with_workspace(x, y, fh, gh, la, lb, mat_m, None, 1, eps, cs)
    torch.cuda.synchronize()
    assert got.shape == (STATIC_MAX_ROWS, 3) and torch.isfinite(got).all()
    assert torch.equal(got, want)
    xs, ys, fs_, gs, las, lbs, mm, mn, sc = _problem(404, 257, 190, 5, 4)
    got_s = _static(xs, ys, fs_, gs, las, lbs, mm, sc, 1, eps, cs)
    ref = O.apply_mat(*(t.double().cpu().numpy() for t in (xs, ys, fs_, gs, las, lbs, mm)), eps, 1, cost_scale=cs,
                      scale=sc.double().cpu().numpy())
    err = np.abs(got_s.double().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= TOL


def test_static_scratch_entry_rejects_sizes_beyond_its_array():
    """Runs without a GPU: the size check comes before any device work."""
    import os
    if not os.path.exists(_lib.library_path()):
        pytest.skip("the CUDA library has not been built")
    lib = _lib.load()
    dummy = ctypes.c_void_p(256)  # never dereferenced: the call must fail on the size alone
    rc = lib.fs_apply_mat_static(dummy, dummy, STATIC_MAX_ROWS + 1, 10, 4, dummy, dummy, dummy, dummy, dummy, 4,
                                 None, dummy, 0.1, 1, 1.0, None)
    assert rc == 1  # FS_ERR_BAD_ARG
    assert b"static scratch" in lib.fs_last_error()
    rc = lib.fs_apply_mat_static(dummy, dummy, 10, STATIC_MAX_ROWS + 1, 4, dummy, dummy, dummy, dummy, dummy, 4,
                                 None, dummy, 0.1, 0, 1.0, None)
    assert rc == 1
