"""Whole-step parity on a B200: the fused step driver against the reference's golden
vectors and against the CPU oracle on the benchmark workloads' shapes."""

import numpy as np
import pytest
import torch

from oracle import lora_step as ol
from oracle import reference_rng as rr
from tests.golden_io import load_gradient_parity, load_qwen2_family, to_torch, within

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-4, 1e-3   # the reference's gradient-parity rule (gradient_parity.rs:48-49)


def _oracle_cfg(cfg, lora, f16_base=False, lora_head=False):
    targets = tuple(lora.target_modules) + (("lm_head",) if lora_head else ())
    return ol.OracleConfig(vocab=cfg.vocab, hidden=cfg.hidden, layers=cfg.layers, heads=cfg.heads,
                           kv_heads=cfg.kv_heads, ffn=cfg.ffn, eps=cfg.eps, theta=cfg.theta,
                           head_dim=cfg.head_dim, tied=cfg.tied, qkv_bias=cfg.qkv_bias,
                           lora_rank=lora.rank, lora_alpha=lora.alpha, lora_targets=targets,
                           f16_base=f16_base, attention_dropout=getattr(cfg, "attention_dropout", 0.0))


def _oracle_params(cfg, weights, adapters, f16_base):
    from ferrotensor_b200.config import head_weight
    p = {k: v.detach().cpu().to(torch.float32).clone() for k, v in {**weights, **adapters}.items()}
    p["lm_head.weight"] = head_weight(cfg, weights, f16_base).cpu().clone()
    return p


def _run(trainer, ids, tgt, msk):
    return trainer.train_arrays(np.asarray(ids, dtype=np.uint32), np.asarray(tgt, dtype=np.uint32),
                                np.asarray(msk, dtype=np.uint8))


def _check(got, exp, what, atol=ATOL, rtol=RTOL):
    good, worst = within(got, exp, atol, rtol)
    assert good, f"{what}: worst abs error {worst:.3e}"


@pytest.mark.parametrize("case", ["single", "batch", "masked"])
def test_reference_gradient_parity_fixture(cuda_ctx, case):
    """The reference's own fixture (30 adapter gradients, logits, loss) through the CUDA step."""
    from ferrotensor_b200.config import LoRaConfig, ModelConfig
    from ferrotensor_b200.engine import GemmMode
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    cj, weights, adapters, cases, expected = load_gradient_parity()
    cfg = ModelConfig(vocab=cj["vocab_size"], hidden=cj["hidden_size"], layers=cj["num_hidden_layers"],
                      heads=cj["num_attention_heads"], kv_heads=cj["num_key_value_heads"],
                      ffn=cj["intermediate_size"], eps=cj["rms_norm_eps"], theta=cj["rope_theta"])
    lora = LoRaConfig(cases["lora_rank"], cases["lora_alpha"], ("proj",))
    cuda_ctx.set_gemm_mode(GemmMode.F32)
    model = LoraModel(cuda_ctx, cfg, lora, to_torch(weights), to_torch(adapters), f16_base=False,
                      lora_head=True)
    spec = cases["cases"][case]
    n = len(spec["rows"])
    tr = Trainer(model, AdamW(0.0, weight_decay=0.0)).with_grad_accum_steps(1)
    tr.keep_logits, tr.length_bucket = True, 8
    # the fixture's loss is the SUM of per-sequence means: seed 1 for every sequence
    model.zero_grad()
    tr.grad_accum_steps = 1
    ids, tg, mk = (np.asarray(spec[k]) for k in ("rows", "targets", "masks"))
    tr._run_chunk(ids.astype(np.uint32), tg.astype(np.uint32), mk.astype(np.uint8))
    stats = tr._collect()
    loss = sum(s.loss for s in stats)
    assert abs(loss - spec["loss"]) <= ATOL + RTOL * abs(spec["loss"])
    _check(tr.last_logits.cpu().numpy(), expected[f"logits.{case}"], "logits")
    grads = model.named_grads()
    assert len(grads) == 30
    for name, g in grads.items():
        _check(g.cpu().numpy(), expected[f"grad.{case}.{name}"], f"{case}/{name}")
    assert sum(s.tokens for s in stats) == int(np.asarray(spec["masks"]).sum())
    model.close()


def test_qwen2_bias_tied_head_against_transformers_fixture(cuda_ctx):
    """q/k/v bias, tied head, theta 1e6: logits against Hugging Face's Qwen2ForCausalLM, and
    dB of zero-initialised adapters through the identity dB = (alpha/r) A^T dW
    (ferrotensor-trainer/tests/qwen2_family.rs:250-328)."""
    from ferrotensor_b200.config import LoRaConfig, ModelConfig, init_adapters
    from ferrotensor_b200.engine import GemmMode
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    cj, weights, cases, expected = load_qwen2_family()
    cfg = ModelConfig(vocab=cj["vocab_size"], hidden=cj["hidden_size"], layers=cj["num_hidden_layers"],
                      heads=cj["num_attention_heads"], kv_heads=cj["num_key_value_heads"],
                      ffn=cj["intermediate_size"], eps=cj["rms_norm_eps"], theta=cj["rope_theta"],
                      tied=True, qkv_bias=True)
    lora = LoRaConfig(4, 8.0, ("proj",))
    adapters = init_adapters(cfg, lora, seed=3)          # B = 0
    cuda_ctx.set_gemm_mode(GemmMode.F32)
    model = LoraModel(cuda_ctx, cfg, lora, to_torch(weights), adapters, f16_base=False)
    tr = Trainer(model, AdamW(0.0))
    tr.keep_logits, tr.length_bucket = True, 1
    n = len(cases["ids"])
    model.zero_grad()
    tr._run_chunk(np.array([cases["ids"]], dtype=np.uint32), np.array([cases["targets"]], dtype=np.uint32),
                  np.ones((1, n), dtype=np.uint8))
    stats = tr._collect()
    assert abs(stats[0].loss - cases["loss"]) <= ATOL + RTOL * abs(cases["loss"])
    _check(tr.last_logits.cpu().numpy(), expected["logits"], "qwen2 logits")
    for name, g in model.named_grads().items():
        prefix, kind = name.rsplit(".", 1)
        if kind == "lora_a":
            assert not g.any(), f"{name}: dA must vanish while B = 0"
        else:
            dw_in_out = torch.tensor(expected[f"grad.{prefix}.weight"]).T      # [in, out]
            exp = lora.scale * adapters[f"{prefix}.lora_a"].T @ dw_in_out
            _check(g.cpu().numpy(), exp.numpy(), name)
    model.close()


def _tiny_setup(cuda_ctx, name="tiny", f16_base=None, mode=None, checkpoint=False, layers=None,
                seq_len=None, n_seq=None, b_std=None):
    from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights
    from ferrotensor_b200.engine import GemmMode
    from ferrotensor_b200.model import LoraModel
    import copy
    w = copy.deepcopy(WORKLOADS[name])
    if layers:
        w.model.layers = layers
    if seq_len:
        w.seq_len = seq_len
    if n_seq:
        w.global_batch = n_seq
    if f16_base is not None:
        w.f16_base = f16_base
    weights = init_weights(w.model, w.seed, f16_base=w.f16_base, norm_jitter=0.25)
    adapters = init_adapters(w.model, w.lora, w.seed, b_std=w.adapter_b_std if b_std is None else b_std)
    cuda_ctx.set_gemm_mode(mode if mode is not None else GemmMode.F32)
    model = LoraModel(cuda_ctx, w.model, w.lora, weights, adapters, f16_base=w.f16_base,
                      checkpoint_blocks=checkpoint)
    return w, weights, adapters, model


def test_tiny_workload_full_step_with_adamw(cuda_ctx):
    """Workload 1: 2 x 16 tokens, f32 base, rank-4 adapters on all seven linears, one
    forward/backward and one AdamW step; loss, logits, 28 gradients, 28 updated tensors and
    both moments against the oracle."""
    from ferrotensor_b200.config import synthetic_batch
    from ferrotensor_b200.trainer import AdamW, Trainer
    w, weights, adapters, model = _tiny_setup(cuda_ctx)
    ids, tg, mk = synthetic_batch(w, w.global_batch)
    tr = Trainer(model, AdamW(w.lr, weight_decay=w.weight_decay)).with_grad_accum_steps(w.global_batch)
    tr.keep_logits, tr.length_bucket = True, 16
    stats = _run(tr, ids, tg, mk)
    ocfg = _oracle_cfg(w.model, w.lora)
    p = _oracle_params(w.model, weights, adapters, False)
    hp = ol.AdamParams(lr=w.lr, weight_decay=w.weight_decay)
    res, pre_clip, norm, scale, skipped, state = ol.lora_step(
        ocfg, p, [[(ids.astype(np.int64), tg.astype(np.int64), mk)]], hp)
    assert len(model.adapter_names()) == 28 and not skipped
    _check(tr.last_logits.cpu().numpy(), res[0].logits.numpy(), "logits")
    for s, (el, et) in zip(stats, res[0].per_sequence):
        assert s.tokens == et and abs(s.loss - el) <= ATOL + RTOL * abs(el)
    assert stats[-1].optimizer_step and abs(stats[-1].grad_norm - norm) <= 1e-5 + 1e-3 * norm
    for name, g in model.named_grads().items():
        _check(g.cpu().numpy(), pre_clip[name].numpy(), f"grad {name}")
    ms, vs = model.named_moments()
    for name, t in model.named_lora_params().items():
        _check(t.cpu().numpy(), p[name].numpy(), f"param {name}", 1e-5, 1e-4)
        _check(ms[name].cpu().numpy(), state[name]["m"].numpy(), f"m {name}", 1e-6, 1e-3)
        _check(vs[name].cpu().numpy(), state[name]["v"].numpy(), f"v {name}", 1e-9, 1e-3)
    model.close()


def test_accumulation_clipping_and_ragged_batch(cuda_ctx):
    """Ragged sequences through `train_batch` (padding with the last token, bucket 32),
    two micro-batches per window, clipping at a norm the step exceeds."""
    from ferrotensor_b200.trainer import AdamW, Batch, Trainer
    w, weights, adapters, model = _tiny_setup(cuda_ctx, b_std=0.3)
    rng = np.random.default_rng(5)
    lens = [40, 17, 64, 33]
    longest = max(lens)
    rows, tgts, attn, lms = [], [], [], []
    for n in lens:
        seq = rng.integers(0, w.model.vocab, n + 1)
        pad = longest - n
        rows.append(seq[:-1].tolist() + [0] * pad)
        tgts.append(seq[1:].tolist() + [0] * pad)
        attn.append([1] * n + [0] * pad)
        lms.append((rng.random(n) < 0.7).astype(int).tolist() + [0] * pad)
    batch = Batch(rows, tgts, attn, lms)
    clip = 0.05
    tr = Trainer(model, AdamW(1e-2)).with_grad_accum_steps(4).with_clip_grad_norm(clip)
    tr.max_chunk = 2
    stats = tr.train_batch(batch)
    assert len(stats) == 4 and stats[-1].optimizer_step
    ocfg = _oracle_cfg(w.model, w.lora)
    p = _oracle_params(w.model, weights, adapters, False)
    chunks = []
    for c in (0, 2):
        tri = [(rows[i][:lens[i]], tgts[i][:lens[i]], lms[i][:lens[i]]) for i in (c, c + 1)]
        chunks.append(ol.pad_chunk(tri, 32))
    hp = ol.AdamParams(lr=1e-2)
    res, pre_clip, norm, scale, skipped, state = ol.lora_step(ocfg, p, [chunks], hp, clip_grad_norm=clip)
    assert scale is not None and norm > clip
    assert abs(stats[-1].grad_norm - norm) <= 1e-5 + 1e-3 * norm
    flat = [x for r in res for x in r.per_sequence]
    for s, (el, et) in zip(stats, flat):
        assert s.tokens == et and abs(s.loss - el) <= ATOL + RTOL * abs(el)
    for name, t in model.named_lora_params().items():
        _check(t.cpu().numpy(), p[name].numpy(), f"param {name}", 1e-5, 1e-3)
    model.close()


def test_block_checkpointing_gives_the_same_gradients(cuda_ctx):
    """block_checkpointing.rs:166-199: gradients within 1e-6 + 1e-4*|y| with and without."""
    from ferrotensor_b200.config import synthetic_batch
    from ferrotensor_b200.trainer import AdamW, Trainer
    grads = []
    for ckpt in (False, True):
        w, _, _, model = _tiny_setup(cuda_ctx, checkpoint=ckpt)
        ids, tg, mk = synthetic_batch(w, 2)
        tr = Trainer(model, AdamW(0.0)).with_grad_accum_steps(2)
        tr.length_bucket = 16
        model.zero_grad()
        tr._run_chunk(ids, tg, mk)
        cuda_ctx.synchronize()
        grads.append({k: v.cpu().numpy().copy() for k, v in model.named_grads().items()})
        tr._collect()
        model.close()
    for k in grads[0]:
        _check(grads[1][k], grads[0][k], k, 1e-6, 1e-4)


def test_nonfinite_gradients_skip_the_step(cuda_ctx):
    """lib.rs:330-335: a non-finite norm leaves parameters and moments untouched."""
    from ferrotensor_b200.config import synthetic_batch
    from ferrotensor_b200.trainer import AdamW, StepStats, Trainer, WarmupCosineScheduler
    w, _, _, model = _tiny_setup(cuda_ctx)
    tr = Trainer(model, AdamW(1e-2)).with_lr_scheduler(WarmupCosineScheduler(1e-2, 1e-3, 2, 10))
    before = model.params.clone()
    model.grads.fill_(1.0)
    model.grads[3] = float("nan")
    s = StepStats()
    tr.apply_gradients(s)
    assert not s.optimizer_step and not np.isfinite(s.grad_norm)
    assert torch.equal(model.params, before) and not model.adam_m.any()
    assert tr.optimizer.t == 0.0
    # the schedule does not advance on a skipped step and no learning rate is reported
    assert tr.lr_scheduler.current_step() == tr.optimizer_step_count == 0
    assert s.lr is None and tr.optimizer.lr == 1e-2
    # the next good step is step 1 of the schedule
    model.grads.fill_(1.0)
    s = StepStats()
    tr.apply_gradients(s)
    assert s.optimizer_step and tr.lr_scheduler.current_step() == tr.optimizer_step_count == 1
    assert abs(s.lr - 5e-3) < 1e-9
    model.close()


def test_forty_step_trajectory_of_the_reference_example(cuda_ctx):
    """lora_finetune_tiny.rs:12-29 prints these losses (tied head, norms = 1, rank 4 on
    q/k/v/o, AdamW lr 1e-2 wd 0.01, no clipping, one 15-token sequence padded to 16)."""
    from ferrotensor_b200.config import LoRaConfig, ModelConfig
    from ferrotensor_b200.engine import GemmMode
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    V, H, HEADS, KV, L, F, R = 64, 32, 4, 2, 2, 64, 4
    weights = to_torch(rr.tiny_llama_weights(V, H, HEADS, KV, L, F, norm_scale=0.0, lm_head=False))
    cfg = ModelConfig(vocab=V, hidden=H, layers=L, heads=HEADS, kv_heads=KV, ffn=F, eps=1e-5,
                      theta=10000.0, tied=True)
    lora = LoRaConfig(R, 8.0, ("q_proj", "k_proj", "v_proj", "o_proj"))
    adapters = {}
    for l in range(L):
        for m, (o, i) in cfg.linear_shapes().items():
            if lora.targeted(m):
                pre = f"model.layers.{l}.{m}"
                adapters[f"{pre}.lora_a"] = torch.tensor(rr.lora_a_seeded(i, o, R, l + 1))
                adapters[f"{pre}.lora_b"] = torch.zeros(R, o)
    cuda_ctx.set_gemm_mode(GemmMode.F32)
    model = LoraModel(cuda_ctx, cfg, lora, weights, adapters, f16_base=False)
    assert model.trainable == 1792
    seq = [(i * 7 + 3) % V for i in range(16)]
    tr = Trainer(model, AdamW(1e-2))
    tr.length_bucket = 16
    printed = {0: 5.9385, 10: 2.5799, 20: 0.9200, 30: 0.4844, 39: 0.2989}
    for step in range(40):
        stats = tr.train_chunk([(seq[:-1], seq[1:], [1] * 15)])
        assert stats[-1].optimizer_step
        if step in printed:
            assert abs(stats[-1].loss - printed[step]) < 3e-4, (step, stats[-1].loss)
    model.close()


# ---- tensor-core path -----------------------------------------------------------------
# Operand rounding of the tcgen05 path, stated: activations (as they are) and activation
# gradients (after a power-of-two scale) are rounded to f16 - 11 significant bits, relative
# rounding error up to 2^-12 - before each dense product with a frozen weight; weights are
# f16 exactly as stored; products are exact and accumulate in f32.  Against the f32 oracle,
# through a stack of such products, tensors are compared with
#     |got - exp| <= TC_ATOL_REL * max|exp| + TC_RTOL * |exp|
# and, in the split mode (two f16 halves, 22 significant bits, two passes), with the
# reference's own f32 rule 1e-4 + 1e-3*|exp|.
TC_ATOL_REL, TC_RTOL = 2e-3, 1e-2


def _tc_check(got, exp, what):
    exp = np.asarray(exp, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    tol = TC_ATOL_REL * np.abs(exp).max() + TC_RTOL * np.abs(exp)
    err = np.abs(got - exp)
    denom = np.linalg.norm(exp)
    rel = np.linalg.norm(got - exp) / denom if denom > 0 else 0.0
    print(f"  {what}: rel L2 {rel:.2e}, worst abs {err.max():.2e} of scale {np.abs(exp).max():.2e}")
    assert (err <= tol).all(), f"{what}: worst {err.max():.3e} vs scale {np.abs(exp).max():.3e}"
    assert rel < 2e-3, f"{what}: relative L2 error {rel:.2e} too large"


@pytest.mark.parametrize("mode_name", ["F16", "F16X2"])
def test_tensor_core_step_matches_oracle(cuda_ctx, mode_name):
    """SmolLM2-135M-shaped blocks (hidden 576, 9/3 heads of 64, ffn 1536, f16 base) cut to
    2 layers and a 4096-token vocabulary... sized so the CPU oracle finishes in seconds."""
    import copy
    from ferrotensor_b200.config import (WORKLOADS, LoRaConfig, init_adapters, init_weights,
                                         synthetic_batch, ALL7)
    from ferrotensor_b200.engine import GemmMode
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    w = copy.deepcopy(WORKLOADS["smollm2-135m"])
    w.model.layers, w.model.vocab, w.seq_len, w.global_batch = 2, 4096, 128, 2
    w.lora = LoRaConfig(8, 16.0, ALL7)
    weights = init_weights(w.model, 11, f16_base=True, norm_jitter=0.25)
    adapters = init_adapters(w.model, w.lora, 11, b_std=0.02)
    mode = GemmMode[mode_name]
    cuda_ctx.set_gemm_mode(mode)
    model = LoraModel(cuda_ctx, w.model, w.lora, weights, adapters, f16_base=True)
    ids, tg, mk = synthetic_batch(w, 2)
    tr = Trainer(model, AdamW(0.0)).with_grad_accum_steps(2)
    tr.keep_logits = True
    model.zero_grad()
    tr._run_chunk(ids, tg, mk)
    stats = tr._collect()
    ocfg = _oracle_cfg(w.model, w.lora, f16_base=True)
    p = _oracle_params(w.model, weights, adapters, True)
    r = ol.forward_backward(ocfg, p, ids.astype(np.int64), tg.astype(np.int64), mk, seed_scale=0.5)
    check = _check if mode is GemmMode.F16X2 else _tc_check
    check(tr.last_logits.cpu().numpy(), r.logits.numpy(), "logits")
    for s, (el, et) in zip(stats, r.per_sequence):
        assert s.tokens == et
        assert abs(s.loss - el) <= (1e-4 + 1e-3 * abs(el) if mode is GemmMode.F16X2 else 2e-3 * abs(el))
    for name, g in model.named_grads().items():
        check(g.cpu().numpy(), r.grads[name].numpy(), f"{mode_name} grad {name}")
    cuda_ctx.set_gemm_mode(GemmMode.F32)
    model.close()


def test_data_parallel_two_ranks_emulated_on_one_gpu(cuda_ctx):
    """Two ranks' shards run one after the other on one device; their summed gradient
    buffers times 1/world must equal the single-rank gradient of the whole batch scaled the
    reference's way (each rank seeds with 1/(its own sequences), then the mean over ranks)."""
    from ferrotensor_b200.config import synthetic_batch
    from ferrotensor_b200.trainer import AdamW, Trainer, shard_indices
    w, weights, adapters, model = _tiny_setup(cuda_ctx, n_seq=4)
    ids, tg, mk = synthetic_batch(w, 4)
    tr = Trainer(model, AdamW(0.0)).with_grad_accum_steps(4)
    tr.length_bucket = 16
    model.zero_grad()
    tr._run_chunk(ids, tg, mk)
    tr._collect()
    whole = model.grads.clone()
    total = torch.zeros_like(whole)
    for rank in range(2):
        idx = shard_indices(4, 2, rank)
        tr2 = Trainer(model, AdamW(0.0)).with_grad_accum_steps(len(idx))
        tr2.length_bucket = 16
        model.zero_grad()
        tr2._run_chunk(ids[idx], tg[idx], mk[idx])
        tr2._collect()
        total += model.grads
    _check((total * 0.5).cpu().numpy(), whole.cpu().numpy(), "mean over ranks", 1e-6, 1e-4)
    # and against the oracle's two-rank step
    ocfg = _oracle_cfg(w.model, w.lora)
    p = _oracle_params(w.model, weights, adapters, False)
    mbs = [[(ids[shard_indices(4, 2, r)].astype(np.int64), tg[shard_indices(4, 2, r)].astype(np.int64),
             mk[shard_indices(4, 2, r)])] for r in range(2)]
    _, pre_clip, *_ = ol.lora_step(ocfg, p, mbs, ol.AdamParams(lr=0.0, weight_decay=0.0), world=2)
    got = (total * 0.5)
    for name in model.adapter_names():
        off, rows, cols = model._slices[name]
        _check(got[off:off + rows * cols].view(rows, cols).cpu().numpy(), pre_clip[name].numpy(), name)
    model.close()
