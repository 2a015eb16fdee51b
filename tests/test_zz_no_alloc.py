"""The allocation-free RMSNorm backward entry point, checked against the regular one and
against the CPU oracle.

Collected last on purpose: the entry point shares one fixed device array between all calls,
so this file runs after every other GPU test and must also pass alone in a fresh process.
`test_this_file_is_collected_last` checks the position instead of trusting the file name."""

import ctypes as C

import numpy as np
import pytest

from oracle import kernels as ok

pytestmark = pytest.mark.gpu


def _run(ctx, name, x, w, g, want_gw=True):
    """Calls ft_rms_norm_backward or its no-alloc twin through the C ABI on device copies."""
    from ferrotensor_b200._lib import call
    from ferrotensor_b200.engine import UnifiedTensor
    rows, size = x.shape
    X, W, G = (UnifiedTensor.new(ctx, a, list(a.shape)) for a in (x, w, g))
    gx = UnifiedTensor.empty(ctx, [rows, size])
    gw = UnifiedTensor.empty(ctx, [size]) if want_gw else None
    call(name, ctx.handle, X.ptr, W.ptr, G.ptr, gx.ptr, gw.ptr if gw is not None else None,
         rows, size, C.c_float(1e-5))
    return gx.to_vec(ctx), (gw.to_vec(ctx) if gw is not None else None)


@pytest.mark.parametrize("shapes", [[(16, 2048), (5, 576)], [(300, 960), (300, 960)]])
def test_noalloc_matches_regular_entry_point_twice_in_a_row(cuda_ctx, shapes):
    """Two calls in a row (the second sees the first call's leftovers in the fixed array):
    both must agree with ft_rms_norm_backward within the kernel tests' tolerance."""
    rng = np.random.default_rng(42)
    for rows, size in shapes:
        x = rng.standard_normal((rows, size), dtype=np.float32)
        w = (1 + 0.25 * rng.standard_normal(size)).astype(np.float32)
        g = rng.standard_normal((rows, size), dtype=np.float32)
        ref_gx, ref_gw = _run(cuda_ctx, "ft_rms_norm_backward", x, w, g)
        gx, gw = _run(cuda_ctx, "ft_rms_norm_backward_noalloc", x, w, g)
        assert np.all(np.abs(gx - ref_gx) <= 1e-5 + 1e-4 * np.abs(ref_gx))
        assert np.all(np.abs(gw - ref_gw) <= 1e-4 + 1e-4 * np.abs(ref_gw))
        # and with the oracle, at the tolerance the kernel tests use for this operator
        exp_gx, exp_gw = ok.rms_norm_backward(x, w, g, 1e-5)
        exp_gx = exp_gx.reshape(gx.shape)
        assert np.all(np.abs(gx - exp_gx) <= 1e-5 + 1e-4 * np.abs(exp_gx))
        assert np.all(np.abs(gw - exp_gw) <= 1e-4 + 1e-4 * np.abs(exp_gw))
        gx2, none = _run(cuda_ctx, "ft_rms_norm_backward_noalloc", x, w, g, want_gw=False)
        assert none is None and np.array_equal(gx2, gx)


def test_noalloc_rejects_shapes_beyond_the_fixed_scratch(cuda_ctx):
    from ferrotensor_b200._lib import FtError
    rows, size = 64, 600_000           # 64 + 600000 floats > 524288
    x = np.zeros((rows, size), dtype=np.float32)
    with pytest.raises(FtError, match="exceeds the fixed scratch"):
        _run(cuda_ctx, "ft_rms_norm_backward_noalloc", x, np.ones(size, np.float32), x)


def test_this_file_is_collected_last(request):
    """A run that stops at the first failure must already have run every other test file."""
    files = []
    for item in request.session.items:
        f = item.nodeid.split("::")[0]
        if not files or files[-1] != f:
            files.append(f)
    if len(files) > 1:   # run as part of the suite
        assert files[-1].endswith("test_zz_no_alloc.py"), files[-3:]
