"""Per-kernel parity on a B200: every operator of the C ABI against the CPU oracle, at the
shapes and tolerances the reference's own kernel tests use
(ferrotensor-backend/tests/gpu_kernels.rs)."""

import numpy as np
import pytest
import torch

from oracle import kernels as ok

pytestmark = pytest.mark.gpu


def _close(got, exp, atol, rtol, what=""):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    exp = np.asarray(exp, dtype=np.float64).reshape(-1)
    assert got.shape == exp.shape, (what, got.shape, exp.shape)
    err = np.abs(got - exp)
    bad = err > atol + rtol * np.abs(exp)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} off, worst {err.max():.3e}"


@pytest.fixture(scope="module")
def eng(cuda_ctx):
    from ferrotensor_b200.engine import ComputeEngine
    return ComputeEngine(cuda_ctx)


def _ut(ctx, a):
    from ferrotensor_b200.engine import UnifiedTensor
    a = np.asarray(a, dtype=np.float32)
    return UnifiedTensor.new(ctx, a, list(a.shape))


def _empty(ctx, shape):
    from ferrotensor_b200.engine import UnifiedTensor
    return UnifiedTensor.empty(ctx, list(shape))


# matmul: gpu_kernels.rs:234-246 shapes, tolerance 1e-4 + 1e-4*|w|
@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (4, 8, 4), (64, 64, 64), (127, 129, 65),
                                   (33, 300, 17), (256, 2048, 96), (16, 4096, 512)])
def test_matmul_variants(cuda_ctx, eng, m, k, n):
    rng = np.random.default_rng(m * 1000 + k + n)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    out = _empty(cuda_ctx, (m, n))
    eng.matmul(cuda_ctx, _ut(cuda_ctx, a), _ut(cuda_ctx, b), out)
    exp = ok.matmul(a, b, torch.float64)
    _close(out.to_vec(cuda_ctx), exp, 1e-4, 1e-4, "matmul")
    eng.matmul_bt(cuda_ctx, _ut(cuda_ctx, a), _ut(cuda_ctx, b.T.copy()), out)
    _close(out.to_vec(cuda_ctx), exp, 1e-4, 1e-4, "matmul_bt")
    eng.matmul_at(cuda_ctx, _ut(cuda_ctx, a.T.copy()), _ut(cuda_ctx, b), out)
    _close(out.to_vec(cuda_ctx), exp, 1e-4, 1e-4, "matmul_at")


@pytest.mark.parametrize("m,k,n", [(5, 32, 64), (127, 129, 66), (64, 576, 192)])
def test_matmul_f16_weights(cuda_ctx, eng, m, k, n):
    from ferrotensor_b200.engine import DType, UnifiedTensor
    rng = np.random.default_rng(7)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    b16 = UnifiedTensor.from_f32_as_f16(cuda_ctx, b, [k, n])
    assert b16.dtype is DType.FP16
    # the device copy holds exactly the oracle's packed words
    words = b16.storage[: ((k * n + 1) // 2) * 4].cpu().numpy().view(np.uint32)
    assert np.array_equal(words, ok.pack_f16(b))
    out = _empty(cuda_ctx, (m, n))
    eng.matmul_f16b(cuda_ctx, _ut(cuda_ctx, a), b16, out)
    exp = ok.matmul(a, ok.f16_round(b), torch.float64)
    _close(out.to_vec(cuda_ctx), exp, 1e-4, 1e-4, "matmul_f16b")
    bt16 = UnifiedTensor.from_f32_transposed(cuda_ctx, b, [k, n], DType.FP16)   # holds [n, k]
    assert bt16.shape == [n, k]
    eng.matmul_bt_f16b(cuda_ctx, _ut(cuda_ctx, a), bt16, out)
    _close(out.to_vec(cuda_ctx), exp, 1e-4, 1e-4, "matmul_bt_f16b")


def test_f16_upload_rounding_edge_cases(cuda_ctx):
    # tensor.rs:565-608: ties to even, overflow to inf, subnormals, signed zero
    from ferrotensor_b200.engine import UnifiedTensor
    vals = np.array([1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 65504.0, 65520.0, 1e-8, 6e-8, -0.0,
                     -2.5, 3.0e-5], dtype=np.float32)
    t = UnifiedTensor.from_f32_as_f16(cuda_ctx, vals, [vals.size])
    got = t.to_vec(cuda_ctx)
    exp = vals.astype(np.float16).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


@pytest.mark.parametrize("rows,size", [(1, 1), (3, 7), (4, 64), (5, 576), (16, 2048), (2, 4099)])
def test_rms_norm_forward_backward(cuda_ctx, eng, rows, size):
    rng = np.random.default_rng(rows * 31 + size)
    x = rng.standard_normal((rows, size), dtype=np.float32)
    w = (1 + 0.25 * rng.standard_normal(size)).astype(np.float32)
    g = rng.standard_normal((rows, size), dtype=np.float32)
    out = _empty(cuda_ctx, (rows, size))
    eng.rms_norm_eps(cuda_ctx, _ut(cuda_ctx, x), _ut(cuda_ctx, w), out, 1e-5)
    _close(out.to_vec(cuda_ctx), ok.rms_norm(x, w, 1e-5), 1e-5, 1e-4, "rms_norm")
    gx, gw = _empty(cuda_ctx, (rows, size)), _empty(cuda_ctx, (size,))
    eng.rms_norm_backward(cuda_ctx, _ut(cuda_ctx, x), _ut(cuda_ctx, w), _ut(cuda_ctx, g), gx, gw, 1e-5)
    egx, egw = ok.rms_norm_backward(x, w, g, 1e-5)
    _close(gx.to_vec(cuda_ctx), egx, 1e-5, 1e-4, "rms gx")
    _close(gw.to_vec(cuda_ctx), egw, 1e-4, 1e-4, "rms gw")
    eng.rms_norm_backward(cuda_ctx, _ut(cuda_ctx, x), _ut(cuda_ctx, w), _ut(cuda_ctx, g), gx, None, 1e-5)
    _close(gx.to_vec(cuda_ctx), egx, 1e-5, 1e-4, "rms gx (frozen norm)")


@pytest.mark.parametrize("b,s,heads,d,pos,theta", [(1, 5, 1, 4, 0, 10000.0), (2, 9, 3, 8, 0, 500.0),
                                                   (2, 33, 4, 64, 7, 130000.0),
                                                   (1, 1024, 2, 64, 0, 1e6)])
def test_rope_and_inverse(cuda_ctx, eng, b, s, heads, d, pos, theta):
    from ferrotensor_b200.engine import UnifiedTensor
    rng = np.random.default_rng(s)
    x = rng.standard_normal((b, s, heads * d), dtype=np.float32)
    t = UnifiedTensor.new(cuda_ctx, x, [b, s, heads * d])
    eng.rope_theta(cuda_ctx, t, d, pos, theta)
    exp = ok.rope(x.reshape(-1), d, s, heads, pos, theta)
    # long positions: one ulp of the f32 angle is ~6e-5 rad at position 1023
    _close(t.to_vec(cuda_ctx), exp, 2e-4 if s > 512 else 1e-5, 1e-4, "rope")
    eng.rope_theta_inverse(cuda_ctx, t, d, pos, theta)
    _close(t.to_vec(cuda_ctx), x, 2e-4 if s > 512 else 2e-5, 1e-4, "rope inverse")


@pytest.mark.parametrize("n", [1, 5, 1024, 4096 * 3 + 17, 1 << 20])
def test_elementwise(cuda_ctx, eng, n):
    rng = np.random.default_rng(n)
    a = (rng.standard_normal(n) * 3).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    A, B, G = _ut(cuda_ctx, a), _ut(cuda_ctx, b), _ut(cuda_ctx, g)
    out = _empty(cuda_ctx, (n,))
    eng.add(cuda_ctx, A, B, out)
    assert np.array_equal(out.to_vec(cuda_ctx), a + b)
    ga, gb = _empty(cuda_ctx, (n,)), _empty(cuda_ctx, (n,))
    eng.add_backward(cuda_ctx, G, ga, gb)
    assert np.array_equal(ga.to_vec(cuda_ctx), g) and np.array_equal(gb.to_vec(cuda_ctx), g)
    eng.silu_gate_fused(cuda_ctx, A, B, out)
    _close(out.to_vec(cuda_ctx), ok.silu_gate(a, b), 1e-6, 1e-5, "silu_gate")
    eng.silu_gate_backward(cuda_ctx, A, B, G, ga, gb)
    ea, eb = ok.silu_gate_backward(a, b, g)
    _close(ga.to_vec(cuda_ctx), ea, 1e-6, 1e-5, "silu bwd first")
    _close(gb.to_vec(cuda_ctx), eb, 1e-6, 1e-5, "silu bwd second")
    eng.gradient_scale(cuda_ctx, G, 0.125)
    assert np.array_equal(G.to_vec(cuda_ctx), g * np.float32(0.125))
    eng.clip_grad_by_norm(cuda_ctx, G, 2.0)
    assert np.array_equal(G.to_vec(cuda_ctx), g * np.float32(0.25))
    dst = _empty(cuda_ctx, (n + 4,))
    eng.copy_tensor(cuda_ctx, A, dst, 16)
    assert np.array_equal(dst.to_vec(cuda_ctx)[4:], a)


ATTN_SHAPES = [  # (b, sq, sk, h, hkv, d, causal)   gpu_kernels.rs:1639-1646 and the model shapes
    (1, 1, 1, 1, 1, 8, True), (2, 16, 16, 4, 2, 8, True), (2, 37, 37, 4, 2, 64, True),
    (1, 130, 130, 2, 2, 128, True), (1, 33, 33, 2, 1, 16, False), (1, 96, 96, 6, 2, 32, True),
    (1, 64, 64, 3, 3, 12, True),
]


@pytest.mark.parametrize("b,sq,sk,h,hkv,d,causal", ATTN_SHAPES)
def test_attention_forward_backward(cuda_ctx, eng, b, sq, sk, h, hkv, d, causal):
    from ferrotensor_b200.engine import AttentionOptions, UnifiedTensor
    rng = np.random.default_rng(sq * 7 + d)
    q = rng.standard_normal((b, sq, h, d), dtype=np.float32)
    k = rng.standard_normal((b, sk, hkv, d), dtype=np.float32)
    v = rng.standard_normal((b, sk, hkv, d), dtype=np.float32)
    do = rng.standard_normal((b, sq, h, d), dtype=np.float32)
    Q, K, V, DO = (UnifiedTensor.new(cuda_ctx, t, list(t.shape)) for t in (q, k, v, do))
    out = _empty(cuda_ctx, (b, sq, h, d))
    stats = _empty(cuda_ctx, (b, h, sq, 2))
    opts = AttentionOptions(causal=causal)
    eng.flash_attention_v2_with_stats(cuda_ctx, Q, K, V, out, stats, opts)
    eo, elses, _ = ok.attention(q, k, v, b, sq, sk, h, hkv, d, causal, torch.float64)
    _close(out.to_vec(cuda_ctx), eo, 1e-5, 1e-3, "attention out")
    _close(stats.to_vec(cuda_ctx).reshape(-1, 2)[:, 1], elses, 1e-5, 1e-4, "attention lse")
    out2 = _empty(cuda_ctx, (b, sq, h, d))
    eng.flash_attention_v2_with(cuda_ctx, Q, K, V, out2, opts)
    assert np.array_equal(out2.to_vec(cuda_ctx), out.to_vec(cuda_ctx))
    dq, dk, dv = _empty(cuda_ctx, q.shape), _empty(cuda_ctx, k.shape), _empty(cuda_ctx, v.shape)
    eng.flash_attention_v2_backward_with_stats(cuda_ctx, Q, K, V, out, DO, dq, dk, dv, stats, opts)
    edq, edk, edv = ok.attention_backward(q, k, v, do, b, sq, sk, h, hkv, d, causal, torch.float64)
    _close(dq.to_vec(cuda_ctx), edq, 1e-4, 1e-3, "dq")
    _close(dk.to_vec(cuda_ctx), edk, 1e-4, 1e-3, "dk")
    _close(dv.to_vec(cuda_ctx), edv, 1e-4, 1e-3, "dv")
    # without saved stats the backward pass recomputes the log-sum-exp: same result
    dq2, dk2, dv2 = _empty(cuda_ctx, q.shape), _empty(cuda_ctx, k.shape), _empty(cuda_ctx, v.shape)
    eng.flash_attention_v2_backward_with(cuda_ctx, Q, K, V, out, DO, dq2, dk2, dv2, opts)
    _close(dq2.to_vec(cuda_ctx), edq, 1e-4, 1e-3, "dq (lse recomputed)")
    _close(dk2.to_vec(cuda_ctx), edk, 1e-4, 1e-3, "dk (lse recomputed)")
    # run twice: no atomics, so bit-identical
    eng.flash_attention_v2_backward_with_stats(cuda_ctx, Q, K, V, out, DO, dq2, dk2, dv2, stats, opts)
    assert np.array_equal(dk2.to_vec(cuda_ctx), dk.to_vec(cuda_ctx))


def test_attention_rejects_a_mask_of_another_shape(cuda_ctx, eng):
    from ferrotensor_b200.engine import AttentionOptions
    q = _ut(cuda_ctx, np.zeros((1, 4, 1, 8), dtype=np.float32))
    with pytest.raises(Exception, match="attention mask"):
        eng.flash_attention_v2_with(cuda_ctx, q, q, q, _empty(cuda_ctx, (1, 4, 1, 8)),
                                    AttentionOptions(causal=True), mask=q)


# masked CE: gpu_kernels.rs:1375-1436 incl. (3, 49152); loss 1e-4/1e-4, grad 1e-6 + 1e-3
@pytest.mark.parametrize("rows,vocab", [(1, 2), (4, 33), (6, 256), (3, 49152), (2, 151936)])
def test_masked_cross_entropy(cuda_ctx, eng, rows, vocab):
    from ferrotensor_b200.engine import MASKED_CE_SKIP, UnifiedTensor
    rng = np.random.default_rng(vocab)
    z = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    tg = rng.integers(0, vocab, rows).astype(np.uint32)
    if rows > 1:
        tg[1] = MASKED_CE_SKIP
    w = (1.0 / rng.integers(1, 9, rows)).astype(np.float32)
    T = UnifiedTensor.from_bytes(cuda_ctx, tg.tobytes(), [rows])
    grad, loss = _empty(cuda_ctx, (rows, vocab)), _empty(cuda_ctx, (rows,))
    eng.masked_cross_entropy_weighted(cuda_ctx, _ut(cuda_ctx, z), T, _ut(cuda_ctx, w), grad, loss)
    el, eg = ok.masked_cross_entropy_weighted(z, tg, w)
    _close(loss.to_vec(cuda_ctx), el, 1e-4, 1e-4, "ce loss")
    _close(grad.to_vec(cuda_ctx), eg, 1e-6, 1e-3, "ce grad")
    if rows > 1:
        assert loss.to_vec(cuda_ctx)[1] == 0.0 and not grad.to_vec(cuda_ctx).reshape(rows, vocab)[1].any()


@pytest.mark.parametrize("n", [1, 4096, 4097, 50000])
def test_sum_squares_and_adamw(cuda_ctx, eng, n):
    from ferrotensor_b200.engine import AdamParams
    rng = np.random.default_rng(n)
    g = rng.standard_normal(n).astype(np.float32)
    chunks = -(-n // 4096)
    out = _empty(cuda_ctx, (chunks + 2,))
    assert eng.sum_squares_partial(cuda_ctx, _ut(cuda_ctx, g), out, 2) == chunks
    _close(out.to_vec(cuda_ctx)[2:], ok.sum_squares_partial(g), 1e-3, 1e-5, "sum squares")
    # AdamW: gpu_kernels.rs:2193-2231, tolerance 1e-5 + 1e-4
    w = rng.standard_normal(n).astype(np.float32)
    m = (rng.standard_normal(n) * 0.1).astype(np.float32)
    v = (rng.random(n) * 0.01).astype(np.float32)
    W, M, V = _ut(cuda_ctx, w), _ut(cuda_ctx, m), _ut(cuda_ctx, v)
    hp = AdamParams(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, t=3.0)
    eng.adamw_update(cuda_ctx, W, _ut(cuda_ctx, g), M, V, hp)
    ew, em, ev = ok.adamw(w, g, m, v, 1e-2, 0.9, 0.999, 1e-8, 0.01, 3.0)
    _close(W.to_vec(cuda_ctx), ew, 1e-5, 1e-4, "adamw w")
    _close(M.to_vec(cuda_ctx), em, 1e-6, 1e-5, "adamw m")
    _close(V.to_vec(cuda_ctx), ev, 1e-7, 1e-5, "adamw v")


def test_embedding_gather_is_bit_exact(cuda_ctx, eng):
    from ferrotensor_b200.engine import UnifiedTensor
    rng = np.random.default_rng(0)
    table = rng.standard_normal((50, 36), dtype=np.float32)
    ids = np.array([0, 49, 7, 50, 4000000000, 7], dtype=np.uint32)   # two out-of-range ids
    out = _empty(cuda_ctx, (ids.size, 36))
    eng.embedding_gather(cuda_ctx, _ut(cuda_ctx, table), UnifiedTensor.from_bytes(
        cuda_ctx, ids.tobytes(), [ids.size]), out)
    exp = ok.embedding(table, ids)
    assert np.array_equal(out.to_vec(cuda_ctx).view(np.uint32), exp.reshape(-1).view(np.uint32))


def test_shape_errors_raise_instead_of_launching(cuda_ctx, eng):
    from ferrotensor_b200._lib import FtError
    a = _ut(cuda_ctx, np.zeros((4, 5), dtype=np.float32))
    b = _ut(cuda_ctx, np.zeros((6, 3), dtype=np.float32))
    with pytest.raises(FtError):
        eng.matmul(cuda_ctx, a, b, _empty(cuda_ctx, (4, 3)))
    with pytest.raises(FtError):
        eng.matmul_f16b(cuda_ctx, a, b, _empty(cuda_ctx, (4, 3)))   # b is not FP16


# Tensor-core attention (tcgen05): q, k, v are rounded to f16 (11 significant bits) and the
# probabilities to f16 before P.V; accumulation and softmax are f32.  Stated tolerance against
# the f64 oracle: 2e-3 absolute + 1e-2 relative on outputs of O(1) inputs.
@pytest.mark.parametrize("b,s,h,hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 1024, 3, 3),
                                       (2, 200, 2, 1), (1, 77, 2, 2), (1, 640, 14, 2),
                                       # more tiles than resident blocks (each walks several),
                                       # and Qwen2's 7:1 head sharing at 4096 positions
                                       (4, 1024, 12, 4), (1, 4096, 7, 1)])
def test_attention_forward_on_tensor_cores(cuda_ctx, eng, b, s, h, hkv):
    from ferrotensor_b200.engine import AttentionOptions, GemmMode, UnifiedTensor
    d = 64
    rng = np.random.default_rng(s + h)
    q = rng.standard_normal((b, s, h, d), dtype=np.float32)
    k = rng.standard_normal((b, s, hkv, d), dtype=np.float32)
    v = rng.standard_normal((b, s, hkv, d), dtype=np.float32)
    Q, K, V = (UnifiedTensor.new(cuda_ctx, t, list(t.shape)) for t in (q, k, v))
    out = _empty(cuda_ctx, (b, s, h, d))
    stats = UnifiedTensor.zeros(cuda_ctx, [b, h, s, 2])
    cuda_ctx.set_gemm_mode(GemmMode.F16)
    try:
        eng.flash_attention_v2_with_stats(cuda_ctx, Q, K, V, out, stats, AttentionOptions(causal=True))
        got, lse = out.to_vec(cuda_ctx), stats.to_vec(cuda_ctx).reshape(-1, 2)[:, 1]
    finally:
        cuda_ctx.set_gemm_mode(GemmMode.F32)
    eo, elses, _ = ok.attention(q, k, v, b, s, s, h, hkv, d, True, torch.float64)
    _close(got, eo, 2e-3, 1e-2, "tc attention out")
    _close(lse, elses, 2e-3, 1e-3, "tc attention lse")


# Tensor-core attention backward: operands in f16 (the output gradient after a power-of-two
# scale), P and dS rounded to f16 before the second products, f32 accumulation.  Stated
# tolerance against the f64 oracle: 2e-3 of the tensor's largest magnitude + 1e-2 relative.
@pytest.mark.parametrize("b,s,h,hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 1024, 3, 3),
                                       (2, 200, 2, 1), (1, 77, 2, 2), (1, 640, 14, 2),
                                       # more tiles than resident blocks (each walks several),
                                       # and Qwen2's 7:1 head sharing at 4096 positions
                                       (4, 1024, 12, 4), (1, 4096, 7, 1)])
def test_attention_backward_on_tensor_cores(cuda_ctx, eng, b, s, h, hkv):
    from ferrotensor_b200.engine import AttentionOptions, GemmMode, UnifiedTensor
    d = 64
    rng = np.random.default_rng(s * 3 + h)
    q = rng.standard_normal((b, s, h, d), dtype=np.float32)
    k = rng.standard_normal((b, s, hkv, d), dtype=np.float32)
    v = rng.standard_normal((b, s, hkv, d), dtype=np.float32)
    do = (rng.standard_normal((b, s, h, d)) * 1e-4).astype(np.float32)   # gradient-sized values
    Q, K, V, DO = (UnifiedTensor.new(cuda_ctx, t, list(t.shape)) for t in (q, k, v, do))
    out = _empty(cuda_ctx, (b, s, h, d))
    stats = UnifiedTensor.zeros(cuda_ctx, [b, h, s, 2])
    dq, dk, dv = _empty(cuda_ctx, q.shape), _empty(cuda_ctx, k.shape), _empty(cuda_ctx, v.shape)
    opts = AttentionOptions(causal=True)
    cuda_ctx.set_gemm_mode(GemmMode.F16)
    try:
        eng.flash_attention_v2_with_stats(cuda_ctx, Q, K, V, out, stats, opts)
        eng.flash_attention_v2_backward_with_stats(cuda_ctx, Q, K, V, out, DO, dq, dk, dv, stats, opts)
        got = [t.to_vec(cuda_ctx) for t in (dq, dk, dv)]
        eng.flash_attention_v2_backward_with_stats(cuda_ctx, Q, K, V, out, DO, dq, dk, dv, stats, opts)
        again = [t.to_vec(cuda_ctx) for t in (dq, dk, dv)]
    finally:
        cuda_ctx.set_gemm_mode(GemmMode.F32)
    exp = ok.attention_backward(q, k, v, do, b, s, s, h, hkv, d, True, torch.float64)
    for name, g, e, a in zip(("dq", "dk", "dv"), got, exp, again):
        _close(g, e, 2e-3 * np.abs(e).max(), 1e-2, f"tc {name}")
        assert np.array_equal(g, a), f"{name}: two runs differ"


# tcgen05 GEMM through ft_matmul_bt_f16b in F16 mode: activations with 8 significant bits times
# f16 weights give exact products, so only f32 accumulation order separates the result from
# the f64 product.  Both output tile heights and CTA pairs (512), ragged M/N/K tails.
@pytest.mark.parametrize("tile_m", [128, 256, 512])
@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (256, 256, 128), (384, 320, 192), (1000, 1000, 520),
                                   (2048, 768, 4096), (777, 2048, 264)])
def test_tensor_core_gemm_shapes(cuda_ctx, eng, tile_m, m, n, k):
    from ferrotensor_b200._lib import call
    from ferrotensor_b200.engine import GemmMode, UnifiedTensor
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).float()
    b = (torch.randn(n, k, generator=g) * 0.1).to(torch.float16).float()
    out = _empty(cuda_ctx, (m, n))
    cuda_ctx.set_gemm_mode(GemmMode.F16)
    call("ft_ctx_set_gemm_tile_m", cuda_ctx.handle, tile_m)
    try:
        eng.matmul_bt_f16b(cuda_ctx, _ut(cuda_ctx, a.numpy()),
                           UnifiedTensor.from_f32_as_f16(cuda_ctx, b.numpy(), [n, k]), out)
        got = out.to_vec(cuda_ctx)
    finally:
        call("ft_ctx_set_gemm_tile_m", cuda_ctx.handle, 0)
        cuda_ctx.set_gemm_mode(GemmMode.F32)
    exp = (a.double() @ b.double().T).numpy()
    _close(got, exp, 1e-4 * max(1.0, np.abs(exp).max()), 1e-4, "tcgen05 gemm")
