"""Decode-time kernels against the oracle: matrix-vector products through the matmul entry
points (m = 1), single-query attention through ft_flash_attention_v2, argmax_rows (bit-exact)."""

import numpy as np
import pytest
import torch

from oracle import kernels as ok

pytestmark = pytest.mark.gpu


def _ut(ctx, arr):
    from ferrotensor_b200.engine import UnifiedTensor
    arr = np.ascontiguousarray(arr, dtype=np.float32)
    return UnifiedTensor.new(ctx, arr, list(arr.shape))


def _empty(ctx, shape):
    from ferrotensor_b200.engine import UnifiedTensor
    return UnifiedTensor.empty(ctx, list(shape))


def _close(got, exp, atol, rtol, what):
    got, exp = np.asarray(got, np.float64).ravel(), np.asarray(exp, np.float64).ravel()
    err = np.abs(got - exp)
    tol = atol + rtol * np.abs(exp)
    assert (err <= tol).all(), f"{what}: worst {err.max():.3e} (tolerance {tol[err.argmax()]:.3e})"


@pytest.fixture
def eng(cuda_ctx):
    from ferrotensor_b200.engine import ComputeEngine
    return ComputeEngine(cuda_ctx)


@pytest.mark.parametrize("k,n", [(64, 32), (576, 1536), (2048, 6144), (8192, 2048), (100, 7), (1, 300), (515, 1003)])
def test_matvec_f32_and_f16(cuda_ctx, eng, k, n):
    from ferrotensor_b200.engine import UnifiedTensor
    rng = np.random.default_rng(k + n)
    x = rng.standard_normal((1, k), dtype=np.float32)
    w = (rng.standard_normal((k, n), dtype=np.float32) * 0.05).astype(np.float32)
    out = _empty(cuda_ctx, (1, n))
    eng.matmul(cuda_ctx, _ut(cuda_ctx, x), _ut(cuda_ctx, w), out)
    exp = x.astype(np.float64) @ w.astype(np.float64)
    _close(out.to_vec(cuda_ctx), exp, 1e-4, 1e-3, "matvec f32")
    w16 = w.astype(np.float16).astype(np.float32)
    out2 = _empty(cuda_ctx, (1, n))
    eng.matmul_f16b(cuda_ctx, _ut(cuda_ctx, x), UnifiedTensor.from_f32_as_f16(cuda_ctx, w, [k, n]), out2)
    _close(out2.to_vec(cuda_ctx), x.astype(np.float64) @ w16.astype(np.float64), 1e-4, 1e-3, "matvec f16 weights")
    # twice: same bits (fixed summation order)
    out3 = _empty(cuda_ctx, (1, n))
    eng.matmul(cuda_ctx, _ut(cuda_ctx, x), _ut(cuda_ctx, w), out3)
    assert np.array_equal(out.to_vec(cuda_ctx).view(np.uint32), out3.to_vec(cuda_ctx).view(np.uint32))


@pytest.mark.parametrize("b,sk,h,hkv,d,causal,offset,window", [
    (1, 1, 2, 2, 8, True, 0, 0), (2, 37, 4, 2, 16, True, 36, 0), (1, 300, 9, 3, 64, True, 299, 0),
    (2, 1024, 32, 32, 64, True, 1023, 0), (1, 5000, 14, 2, 64, True, 4999, 0), (1, 200, 4, 4, 128, False, 50, 0),
    (1, 200, 4, 1, 32, True, 120, 16), (1, 64, 2, 2, 24, True, 10, 0), (1, 40, 2, 2, 8, False, 5, 3),
])
def test_attention_decode(cuda_ctx, eng, b, sk, h, hkv, d, causal, offset, window):
    from ferrotensor_b200.engine import AttentionOptions
    rng = np.random.default_rng(sk * 7 + h)
    q = rng.standard_normal((b, 1, h, d), dtype=np.float32)
    k = rng.standard_normal((b, sk, hkv, d), dtype=np.float32)
    v = rng.standard_normal((b, sk, hkv, d), dtype=np.float32)
    out = _empty(cuda_ctx, (b, 1, h, d))
    opts = AttentionOptions(causal=causal, causal_offset=offset, window=window)
    eng.flash_attention_v2_with(cuda_ctx, _ut(cuda_ctx, q), _ut(cuda_ctx, k), _ut(cuda_ctx, v), out, opts)
    exp = ok.attention_decode(q, k, v, b, sk, h, hkv, d, causal, offset, window)
    _close(out.to_vec(cuda_ctx), exp, 1e-5, 1e-3, "decode attention")
    # the many-query kernel (taken when stats are asked for) agrees
    stats = _empty(cuda_ctx, (b * h * 2,))
    out2 = _empty(cuda_ctx, (b, 1, h, d))
    eng.flash_attention_v2_with_stats(cuda_ctx, _ut(cuda_ctx, q), _ut(cuda_ctx, k), _ut(cuda_ctx, v), out2, stats, opts)
    _close(out2.to_vec(cuda_ctx), exp, 1e-5, 1e-3, "one-query attention with stats")


def test_argmax_rows_bit_exact(cuda_ctx, eng):
    from ferrotensor_b200.engine import DType, UnifiedTensor
    rng = np.random.default_rng(3)
    cases = [rng.standard_normal((5, 49152), dtype=np.float32), rng.standard_normal((64, 1000), dtype=np.float32),
             rng.standard_normal((3, 1), dtype=np.float32), rng.standard_normal((2, 255), dtype=np.float32)]
    special = np.array([[1.0, 3.0, 3.0, -2.0, 3.0, 0.0], [np.nan, 1.0, 2.0, 0.0, np.inf, 5.0],
                        [-0.0, 0.0, -1.0, 0.0, -0.0, -3.0], [-np.inf, -5.0, -np.inf, -6.0, -5.0, -7.0]], dtype=np.float32)
    neg_nan = special.copy()
    neg_nan.view(np.uint32)[3, 0] = 0xFFC00000      # -NaN: the lowest of all in total_cmp
    ties = np.zeros((2, 70000), dtype=np.float32)    # every element equal: the last index wins
    for x in cases + [special, neg_nan, ties]:
        rows = x.shape[0]
        out = UnifiedTensor.empty_with_dtype(cuda_ctx, [rows], DType.U32)
        eng.argmax_rows(cuda_ctx, _ut(cuda_ctx, x), out)
        assert np.array_equal(out.to_vec(cuda_ctx), ok.argmax_rows(x)), x.shape
    assert ok.argmax_rows(ties).tolist() == [69999, 69999]
