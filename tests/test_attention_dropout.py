"""Attention with an additive mask and dropout: the reference's tests
(ferrotensor-backend/tests/gpu_kernels.rs:1735-1762, :1960-2056, :2316-2476 and
ferrotensor-graph/src/dropout.rs:43-87) restated against the oracle."""

import numpy as np
import pytest

from ferrotensor_b200.dropout import derive_seed, layer_seed
from oracle import kernels as ok


def test_seeds_are_deterministic_and_differ_by_step_layer_and_run():
    assert derive_seed([42, 0, 7, 1]) == derive_seed([42, 0, 7, 1]) and layer_seed(9, 3) == layer_seed(9, 3)
    base = derive_seed([42, 0, 7, 0])
    others = [derive_seed([43, 0, 7, 0]), derive_seed([42, 1, 7, 0]), derive_seed([42, 0, 8, 0]),
              derive_seed([42, 0, 7, 1]), derive_seed([42, 0, 7])]
    assert all(o != base for o in others) and layer_seed(base, 0) != layer_seed(base, 1)
    assert 0 <= base < 1 << 64

    def far(a, b):
        return min((a - b) & 0xFFFFFFFF, (b - a) & 0xFFFFFFFF) > 1 << 12
    for step in range(64):
        a, b = derive_seed([0, 0, step, 0]) & 0xFFFFFFFF, derive_seed([0, 0, step + 1, 0]) & 0xFFFFFFFF
        assert far(a, b), step
        for layer in range(8):
            assert far(layer_seed(a, layer) & 0xFFFFFFFF, layer_seed(a, layer + 1) & 0xFFFFFFFF), (step, layer)


def _agree(x, y):
    return float((x == y).mean())


def test_oracle_masks_of_nearby_seeds_are_unrelated():
    sq, sk, prob, seed = 64, 32, 0.5, 1000
    qi, kj = np.arange(sq)[:, None], np.arange(sk)[None, :]
    a = ok.dropout_keep(prob, seed, 0, qi, kj)
    assert abs(a.mean() - 0.5) < 0.1
    b = ok.dropout_keep(prob, seed + 1, 0, qi, kj)
    assert abs(_agree(a[:, 1:], b[:, :-1]) - 0.5) < 0.1 and abs(_agree(a, b) - 0.5) < 0.1
    assert abs(_agree(a, ok.dropout_keep(prob, seed + (1 << 32), 0, qi, kj)) - 0.5) < 0.1
    assert abs(_agree(a, ok.dropout_keep(prob, seed, 1, qi, kj)) - 0.5) < 0.1
    assert ok.dropout_keep(0.0, seed, 0, qi, kj).all()
    # scalar evaluation with Python integers agrees with the vectorised form
    def keep(bh, q, k):
        m = 0xFFFFFFFF
        def fmix(h):
            h ^= h >> 16; h = h * 0x85EBCA6B & m; h ^= h >> 13; h = h * 0xC2B2AE35 & m
            return h ^ (h >> 16)
        key = fmix((seed & m) ^ fmix((seed >> 32) ^ 0x9E3779B9))
        x, y, z = ((t * 1664525 + 1013904223) & m for t in (bh ^ key, q, k))
        x = (x + y * z) & m; y = (y + z * x) & m; z = (z + x * y) & m
        x ^= x >> 16; y ^= y >> 16; z ^= z >> 16
        return np.float32((x + y + z) & m) * np.float32(2.3283064365386963e-10) >= np.float32(prob)
    for q in (0, 5, 63):
        for k in (0, 7, 31):
            assert keep(0, q, k) == a[q, k]


# ---- on the device ----------------------------------------------------------------------------
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


def _device_mask(ctx, eng, prob, seed, sq, sk):
    """The keep mask the forward kernel draws, read back through the output: zero scores give
    uniform weights and one-hot values (head_dim == seq_k) put weight j of row i in out[i, j]."""
    q, k, v = np.zeros((1, sq, 1, sk), np.float32), np.zeros((1, sk, 1, sk), np.float32), np.eye(sk, dtype=np.float32)
    out = _empty(ctx, (1, sq, 1, sk))
    eng.flash_attention_v2(ctx, _ut(ctx, q), _ut(ctx, k), _ut(ctx, v.reshape(1, sk, 1, sk)), out, False, prob, seed)
    return out.to_vec(ctx).reshape(sq, sk) > 0


@pytest.mark.gpu
def test_device_mask_is_the_oracle_mask_bit_for_bit(cuda_ctx, eng):
    sq, sk, prob = 64, 32, 0.5
    qi, kj = np.arange(sq)[:, None], np.arange(sk)[None, :]
    for seed in (1000, 1001, 1000 + (1 << 32), 0x123456789ABCDEF0, 0):
        got = _device_mask(cuda_ctx, eng, prob, seed, sq, sk)
        assert np.array_equal(got, ok.dropout_keep(prob, seed, 0, qi, kj)), hex(seed)
    for prob in (0.1, 0.25, 0.9):
        got = _device_mask(cuda_ctx, eng, prob, 77, 128, 64)
        assert np.array_equal(got, ok.dropout_keep(prob, 77, 0, np.arange(128)[:, None], np.arange(64)[None, :]))


@pytest.mark.gpu
def test_dropout_keeps_expected_fraction(cuda_ctx, eng):
    b, s, h, d = 1, 256, 2, 16
    rng = np.random.default_rng(22)
    q, k = rng.standard_normal((b, s, h, d), dtype=np.float32), rng.standard_normal((b, s, h, d), dtype=np.float32)
    out = _empty(cuda_ctx, (b, s, h, d))
    eng.flash_attention_v2(cuda_ctx, _ut(cuda_ctx, q), _ut(cuda_ctx, k), _ut(cuda_ctx, np.ones((b, s, h, d), np.float32)),
                           out, False, 0.25, 1234)
    got = out.to_vec(cuda_ctx)
    assert abs(got.mean() - 1.0) < 0.05 and (np.abs(got - 1.0) > 1e-3).any()


@pytest.mark.gpu
@pytest.mark.parametrize("b,sq,sk,h,hkv,d,causal,offset,window,prob,seed,mask_kind", [
    (2, 21, 21, 4, 2, 32, True, 0, 0, 0.2, 0x9E3779B90000004D, "pad"),      # the reference's case
    (2, 45, 45, 4, 2, 64, True, 0, 20, 0.2, 0x123456789ABCDEF0, "pad"),
    (1, 70, 70, 3, 1, 16, False, 0, 0, 0.5, 5, None),
    (2, 33, 50, 2, 2, 8, True, 17, 0, 0.1, 1 << 40, "full"),
    (1, 40, 40, 2, 2, 128, True, 0, 0, 0.0, 0, "rows"),                     # mask only, some rows all hidden
    (1, 1, 37, 4, 2, 32, True, 36, 0, 0.3, 9, "pad"),                       # one query: hashed with q = 0
])
def test_mask_and_dropout_forward_backward_match_oracle(cuda_ctx, eng, b, sq, sk, h, hkv, d, causal, offset, window,
                                                        prob, seed, mask_kind):
    from ferrotensor_b200.engine import AttentionOptions
    rng = np.random.default_rng(sq * 31 + d)
    q = rng.standard_normal((b, sq, h, d), dtype=np.float32)
    k = rng.standard_normal((b, sk, hkv, d), dtype=np.float32)
    v = rng.standard_normal((b, sk, hkv, d), dtype=np.float32)
    dout = rng.standard_normal((b, sq, h, d), dtype=np.float32)
    mask = None
    if mask_kind == "pad":        # [batch, 1, 1, seq_k]: the last batch hides its last keys
        mask = np.zeros((b, 1, 1, sk), np.float32)
        mask[-1, 0, 0, sk - max(sk // 6, 1):] = -1e9
    elif mask_kind == "full":
        mask = (rng.standard_normal((b, h, sq, sk)) * 0.5).astype(np.float32)
        mask[rng.random((b, h, sq, sk)) < 0.1] = -2e30
    elif mask_kind == "rows":     # [1, 1, seq_q, seq_k]: rows 3 and 4 see nothing
        mask = np.zeros((1, 1, sq, sk), np.float32)
        mask[0, 0, 3:5, :] = -1e31
    opts = AttentionOptions(causal=causal, causal_offset=offset, window=window, dropout_prob=prob, seed=seed)
    exp = ok.attention_general(q, k, v, b, sq, sk, h, hkv, d, causal, offset, window, mask, prob, seed, dout)
    tq, tk, tv, tdo = (_ut(cuda_ctx, x) for x in (q, k, v, dout))
    tmask = _ut(cuda_ctx, mask) if mask is not None else None
    out, stats = _empty(cuda_ctx, (b, sq, h, d)), _empty(cuda_ctx, (b * h * sq * 2,))
    eng.flash_attention_v2_with_stats(cuda_ctx, tq, tk, tv, out, stats, opts, tmask)
    plain = _empty(cuda_ctx, (b, sq, h, d))
    eng.flash_attention_v2_with(cuda_ctx, tq, tk, tv, plain, opts, tmask)
    assert np.array_equal(out.to_vec(cuda_ctx), plain.to_vec(cuda_ctx)), "saving stats changed the output"
    _close(out.to_vec(cuda_ctx), exp[0], 1e-5, 1e-3, "forward")
    _close(stats.to_vec(cuda_ctx)[1::2], exp[1], 1e-5, 1e-5, "log-sum-exp")
    grads = {}
    for saved in (True, False):
        gq, gk, gv = _empty(cuda_ctx, (b, sq, h, d)), _empty(cuda_ctx, (b, sk, hkv, d)), _empty(cuda_ctx, (b, sk, hkv, d))
        if saved:
            eng.flash_attention_v2_backward_with_stats(cuda_ctx, tq, tk, tv, out, tdo, gq, gk, gv, stats, opts, tmask)
        else:
            eng.flash_attention_v2_backward_with(cuda_ctx, tq, tk, tv, out, tdo, gq, gk, gv, opts, tmask)
        grads[saved] = [g.to_vec(cuda_ctx) for g in (gq, gk, gv)]
        for got, want, name in zip(grads[saved], exp[2:], ("dq", "dk", "dv")):
            _close(got, want, 1e-4, 1e-3, f"{name} (saved stats: {saved})")
    for a, c, name in zip(grads[True], grads[False], ("dq", "dk", "dv")):
        _close(a, c, 1e-5, 1e-4, f"{name} saved vs recomputed")


@pytest.mark.gpu
def test_masks_and_dropout_take_the_exact_kernels_in_every_gemm_mode(cuda_ctx, eng):
    """A shape the tensor-core kernels would take (head_dim 64, causal, square) still honours the
    mask and the dropout when the context computes in f16."""
    from ferrotensor_b200.engine import AttentionOptions, GemmMode
    b, s, h, hkv, d = 1, 128, 2, 2, 64
    rng = np.random.default_rng(4)
    q, k, v = (rng.standard_normal((b, s, n, d), dtype=np.float32) for n in (h, hkv, hkv))
    opts = AttentionOptions(causal=True, dropout_prob=0.3, seed=11)
    exp = ok.attention_general(q, k, v, b, s, s, h, hkv, d, True, 0, 0, None, 0.3, 11)
    cuda_ctx.set_gemm_mode(GemmMode.F16)
    try:
        out = _empty(cuda_ctx, (b, s, h, d))
        eng.flash_attention_v2_with(cuda_ctx, _ut(cuda_ctx, q), _ut(cuda_ctx, k), _ut(cuda_ctx, v), out, opts)
        _close(out.to_vec(cuda_ctx), exp[0], 1e-5, 1e-3, "forward in f16 mode")
    finally:
        cuda_ctx.set_gemm_mode(GemmMode.F32)
    with pytest.raises(Exception, match="dropout_prob"):
        eng.flash_attention_v2_with(cuda_ctx, _ut(cuda_ctx, q), _ut(cuda_ctx, k), _ut(cuda_ctx, v), out,
                                    AttentionOptions(causal=True, dropout_prob=1.0))


def test_oracle_seed_derivation_agrees_with_the_host_module():
    from oracle import lora_step as ol
    for parts in ([1, 2], [42, 0, 7, 1], [0], [(1 << 64) - 1, 5]):
        assert ol.derive_seed(parts) == derive_seed(parts)


@pytest.mark.gpu
@pytest.mark.parametrize("mode_name,checkpoint", [("F32", False), ("F32", True), ("F16", False)])
def test_training_step_with_attention_dropout_matches_oracle(cuda_ctx, mode_name, checkpoint):
    """A model whose config asks for attention dropout: the step's loss and adapter gradients
    against the oracle under the same per-pass seed (run seed, rank, optimizer step, position in
    the accumulation window), in the exact mode, with block replay, and in the f16 mode (whose
    attention then stays on the exact kernels); evaluation drops nothing."""
    import copy
    from oracle import lora_step as ol
    from ferrotensor_b200.config import ALL7, WORKLOADS, LoRaConfig, init_adapters, init_weights, synthetic_batch
    from ferrotensor_b200.dropout import attention_dropout_seed
    from ferrotensor_b200.engine import GemmMode
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    from tests.test_step_gpu import _oracle_cfg, _oracle_params
    f16 = mode_name == "F16"
    if f16:
        w = copy.deepcopy(WORKLOADS["smollm2-135m"])
        w.model.layers, w.model.vocab, w.seq_len, w.global_batch = 2, 2048, 64, 2
        w.lora = LoRaConfig(8, 16.0, ALL7)
    else:
        w = copy.deepcopy(WORKLOADS["tiny"])
    w.model.attention_dropout = 0.25
    weights = init_weights(w.model, 21, f16_base=f16, norm_jitter=0.25)
    adapters = init_adapters(w.model, w.lora, 21, b_std=0.02)
    cuda_ctx.set_gemm_mode(GemmMode[mode_name])
    try:
        model = LoraModel(cuda_ctx, w.model, w.lora, weights, adapters, f16_base=f16, checkpoint_blocks=checkpoint)
        ids, tg, mk = synthetic_batch(w, 2)
        tr = Trainer(model, AdamW(0.0)).with_grad_accum_steps(4).with_dropout_seed(99)
        tr.optimizer_step_count, tr.step_in_accum = 3, 2       # a pass in the middle of a run
        pass_seed = attention_dropout_seed(99, 0, 3, 2)
        assert tr.attention_dropout_seed() == pass_seed
        model.zero_grad()
        tr._run_chunk(ids, tg, mk)
        stats = tr._collect()
        ocfg = _oracle_cfg(w.model, w.lora, f16_base=f16)
        p = _oracle_params(w.model, weights, adapters, f16)
        r = ol.forward_backward(ocfg, p, ids.astype(np.int64), tg.astype(np.int64), mk, seed_scale=0.25,
                                dropout_seed=pass_seed)
        plain = ol.forward_backward(ocfg, p, ids.astype(np.int64), tg.astype(np.int64), mk, seed_scale=0.25)
        rel, atol = (2e-3, 0.0) if f16 else (1e-3, 1e-4)
        for s_, (el, et), (pl, _) in zip(stats, r.per_sequence, plain.per_sequence):
            assert s_.tokens == et and abs(s_.loss - el) <= atol + rel * abs(el)
        differs = 0.0
        for name, g in model.named_grads().items():
            got, exp = g.cpu().numpy().astype(np.float64), r.grads[name].numpy().astype(np.float64)
            differs = max(differs, np.linalg.norm(exp - plain.grads[name].numpy()) / max(np.linalg.norm(exp), 1e-30))
            if f16:
                err = np.linalg.norm(got - exp) / max(np.linalg.norm(exp), 1e-30)
                assert err < 5e-3, f"{name}: relative L2 error {err:.2e}"
            else:
                assert (np.abs(got - exp) <= 1e-4 + 1e-3 * np.abs(exp)).all(), name
        assert differs > 0.1, "the dropout case does not differ from the plain one"
        # evaluation: no dropout
        import torch
        from ferrotensor_b200.trainer import batch_targets_weights
        row_tgt, row_w, tokens = batch_targets_weights(tg, mk, w.model.vocab)
        dev = cuda_ctx.device
        n, s = ids.shape
        row_loss = torch.empty(n * s, device=dev)
        model.forward_loss(torch.from_numpy(ids.reshape(-1).view(np.int32)).to(dev),
                           torch.from_numpy(row_tgt.reshape(-1).view(np.int32)).to(dev),
                           torch.from_numpy(row_w.reshape(-1)).to(dev), n, s, row_loss)
        per_seq = row_loss.cpu().numpy().reshape(n, s).astype(np.float64).sum(axis=1) / tokens
        for got, (pl, _) in zip(per_seq, plain.per_sequence):
            assert abs(got - pl) <= atol + rel * abs(pl)
        model.close()
    finally:
        cuda_ctx.set_gemm_mode(GemmMode.F32)
