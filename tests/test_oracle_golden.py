"""Pins the CPU oracle to the reference's own golden vectors (runs without a GPU)."""

import numpy as np
import pytest
import torch

from oracle import kernels as ok
from oracle import lora_step as ol
from oracle import reference_rng as rr
from tests.golden_io import load_gradient_parity, load_qwen2_family, to_torch, within


def _tiny_cfg(cfg_json, rank, alpha, targets):
    return ol.OracleConfig(
        vocab=cfg_json["vocab_size"], hidden=cfg_json["hidden_size"],
        layers=cfg_json["num_hidden_layers"], heads=cfg_json["num_attention_heads"],
        kv_heads=cfg_json["num_key_value_heads"], ffn=cfg_json["intermediate_size"],
        eps=cfg_json["rms_norm_eps"], theta=cfg_json["rope_theta"],
        tied=cfg_json.get("tie_word_embeddings", False),
        lora_rank=rank, lora_alpha=alpha, lora_targets=targets)


def test_weight_generator_is_bit_exact():
    # ferrotensor-graph/tests/common/mod.rs:66-161 vs the committed model.safetensors
    cfg, weights, _, _, _ = load_gradient_parity()
    mine = rr.tiny_llama_weights(cfg["vocab_size"], cfg["hidden_size"], cfg["num_attention_heads"],
                                 cfg["num_key_value_heads"], cfg["num_hidden_layers"],
                                 cfg["intermediate_size"])
    assert set(mine) == set(weights)
    for n in weights:
        assert np.array_equal(mine[n], weights[n]), n


def test_lora_seed_known_answers():
    # ferrotensor-graph/src/model_builder.rs:869-876
    assert rr.lora_seed(1, "q_proj") == 0x5F28D61921D3DDB3
    assert rr.lora_seed(1, "o_proj") == 0xFABFD7977F143D7C
    assert rr.lora_seed(2, "q_proj") == 0x4BAE9242648E2FC1
    assert rr.lora_seed(0, "lm_head") == 0x6D1A1DFFACC30DEF


@pytest.mark.parametrize("case", ["single", "batch", "masked", "full"])
def test_gradient_parity_cases(case):
    """Loss, logits and every gradient tensor of the reference's fixture
    (ferrotensor-trainer/tests/gradient_parity.rs:48-49: 1e-4 + 1e-3*|e|)."""
    cfg_json, weights, adapters, cases, expected = load_gradient_parity()
    cfg = _tiny_cfg(cfg_json, cases["lora_rank"], cases["lora_alpha"], ("proj", "lm_head"))
    spec = cases["cases"][case]
    p = to_torch({**weights, **adapters})
    train = sorted(adapters)
    if spec["trainable_base"]:
        train += [n for n in weights if n != "model.embed_tokens.weight"]
    r = ol.forward_backward(cfg, p, spec["rows"], spec["targets"], spec["masks"], train=train)
    assert abs(r.loss - spec["loss"]) <= 1e-4 + 1e-3 * abs(spec["loss"])
    good, worst = within(r.logits.numpy(), expected[f"logits.{case}"])
    assert good, f"logits off by {worst}"
    n_checked = 0
    for n in train:
        g = r.grads[n]
        if n.endswith(".weight") and g.dim() == 2:
            g = g.T  # fixture stores linear weights [in, out]
        good, worst = within(g.numpy(), expected[f"grad.{case}.{n}"])
        assert good, f"{case}/{n} off by {worst}"
        n_checked += 1
    assert n_checked == (50 if spec["trainable_base"] else 30)


def test_base_logits_without_adapters():
    cfg_json, weights, adapters, cases, expected = load_gradient_parity()
    cfg = _tiny_cfg(cfg_json, 0, 0.0, ())
    p = to_torch(weights)
    logits = ol.forward(cfg, p, torch.tensor([cases["cases"]["single"]["rows"][0]]))
    good, worst = within(logits.numpy(), expected["logits.base"])
    assert good, worst


def test_qwen2_family_bias_tied_theta():
    """HF Qwen2ForCausalLM logits and base-weight gradients
    (scripts/gen_qwen2_fixture.py; q/k/v bias, tied head, theta 1e6, eps 1e-6)."""
    cfg_json, weights, cases, expected = load_qwen2_family()
    cfg = _tiny_cfg(cfg_json, 0, 0.0, ())
    cfg.qkv_bias = True
    p = to_torch(weights)
    p["lm_head.weight"] = p["model.embed_tokens.weight"]
    train = [n for n in expected if n.startswith("grad.")]
    train = [n[len("grad."):] for n in train]
    ids, tg = [cases["ids"]], [cases["targets"]]
    r = ol.forward_backward(cfg, p, ids, tg, [[1] * len(cases["ids"])], train=train)
    assert abs(r.loss - cases["loss"]) <= 1e-4 + 1e-3 * abs(cases["loss"])
    good, worst = within(r.logits.numpy(), expected["logits"])
    assert good, worst
    for n in train:
        good, worst = within(r.grads[n].numpy(), expected[f"grad.{n}"])
        assert good, f"{n}: {worst}"


def test_tiny_finetune_trajectory():
    """40 AdamW steps of the reference's lora_finetune_tiny example
    (ferrotensor-trainer/examples/lora_finetune_tiny.rs:12-29 prints these losses; they
    were produced with per-layer adapter seeds, i.e. before adapter seeds started to
    depend on the projection name)."""
    V, H, HEADS, KV, L, F, SEQ, R, ALPHA = 64, 32, 4, 2, 2, 64, 16, 4, 8.0
    w = rr.tiny_llama_weights(V, H, HEADS, KV, L, F, norm_scale=0.0, lm_head=False)
    p = to_torch(w)
    p["lm_head.weight"] = p["model.embed_tokens.weight"]
    cfg = ol.OracleConfig(vocab=V, hidden=H, layers=L, heads=HEADS, kv_heads=KV, ffn=F, eps=1e-5,
                          theta=10000.0, tied=True, lora_rank=R, lora_alpha=ALPHA,
                          lora_targets=("q_proj", "k_proj", "v_proj", "o_proj"))
    shapes = cfg.linear_shapes()
    for l in range(L):
        for m in ("q_proj", "k_proj", "v_proj", "o_proj"):
            out_dim, in_dim = shapes[f"self_attn.{m}"]
            pre = f"model.layers.{l}.self_attn.{m}"
            p[f"{pre}.lora_a"] = torch.tensor(rr.lora_a_seeded(in_dim, out_dim, R, l + 1))
            p[f"{pre}.lora_b"] = torch.zeros(R, out_dim)
    assert sum(p[n].numel() for n in ol.trainable_names(p)) == 1792
    seq = [(i * 7 + 3) % V for i in range(SEQ)]
    ids, tg, mk = ol.pad_chunk([(seq[:-1], seq[1:], [1] * 15)], bucket=16)
    assert ids[0][-1] == seq[-2] and mk[0] == [1] * 15 + [0]
    hp = ol.AdamParams(lr=1e-2, weight_decay=0.01)
    state = {}
    printed = {0: 5.9385, 10: 2.5799, 20: 0.9200, 30: 0.4844, 39: 0.2989}
    for step in range(40):
        res, _, norm, _, skipped, state = ol.lora_step(cfg, p, [[(ids, tg, mk)]], hp, state)
        assert not skipped
        if step in printed:
            assert abs(res[0].loss - printed[step]) < 2e-4, (step, res[0].loss)
    with torch.no_grad():
        lg = ol.forward(cfg, p, torch.tensor([seq[:-1]]))
        final = torch.nn.functional.cross_entropy(lg[0], torch.tensor(seq[1:])).item()
    assert abs(final - 0.2841) < 2e-4, final


def test_lr_schedule_known_answers():
    # ferrotensor-autograd/src/lib.rs:1926-1938
    lrs = [ol.warmup_cosine_lr(i, 1.0, 0.1, 4, 14) for i in range(15)]
    assert lrs[:5] == [0.0, 0.25, 0.5, 0.75, 1.0]
    assert abs(lrs[9] - 0.55) < 1e-6
    assert lrs[14] == pytest.approx(0.1)


def test_batch_targets_and_padding_rules():
    # ferrotensor-trainer/src/lib.rs:689-716 and :431-450
    tg, w, tokens = ol.batch_targets_weights([1, 2, 99, 3, 4, 5], [1, 0, 1, 1, 1, 1], 2, vocab=10)
    assert tg.tolist() == [1, ol.MASKED_CE_SKIP, ol.MASKED_CE_SKIP, 3, 4, 5]
    assert tokens == [1, 3]
    assert w.tolist() == [1.0, 0.0, 0.0, np.float32(1 / 3), np.float32(1 / 3), np.float32(1 / 3)]
    ids, tgt, msk = ol.pad_chunk([([5, 6, 7], [6, 7, 8], [1, 1, 1]), ([1], [2], [1])], bucket=4)
    assert ids == [[5, 6, 7, 7], [1, 1, 1, 1]]
    assert tgt == [[6, 7, 8, 7], [2, 1, 1, 1]]
    assert msk == [[1, 1, 1, 0], [1, 0, 0, 0]]
    assert ol.shard_indices(7, 3, 1) == [1, 4]


def test_kernel_oracles_agree_with_step_oracle():
    """The per-kernel loops and the autograd restatement are two statements of the same
    math: check attention fwd/bwd, RMSNorm bwd and CE against torch autograd."""
    g = torch.Generator().manual_seed(3)
    b, s, h, hkv, d = 2, 37, 4, 2, 16
    q = torch.randn(b, s, h, d, generator=g, requires_grad=True)
    k = torch.randn(b, s, hkv, d, generator=g, requires_grad=True)
    v = torch.randn(b, s, hkv, d, generator=g, requires_grad=True)
    cfg = ol.OracleConfig(vocab=8, hidden=h * d, layers=1, heads=h, kv_heads=hkv, ffn=8)
    out = ol.attention(cfg, q.view(b, s, -1), k.view(b, s, -1), v.view(b, s, -1))
    do = torch.randn(out.shape, generator=g)
    out.backward(do)
    o2, lse, _ = ok.attention(q.detach().numpy(), k.detach().numpy(), v.detach().numpy(),
                              b, s, s, h, hkv, d)
    assert np.allclose(o2.reshape(b, s, -1), out.detach().numpy(), atol=1e-5)
    dq, dk, dv = ok.attention_backward(q.detach().numpy(), k.detach().numpy(), v.detach().numpy(),
                                       do.numpy(), b, s, s, h, hkv, d)
    assert np.allclose(dq, q.grad.numpy(), atol=2e-5)
    assert np.allclose(dk, k.grad.numpy(), atol=2e-5)
    assert np.allclose(dv, v.grad.numpy(), atol=2e-5)

    x = torch.randn(5, 48, generator=g, requires_grad=True)
    w = torch.randn(48, generator=g, requires_grad=True)
    gy = torch.randn(5, 48, generator=g)
    ol.rms_norm(x, w, 1e-5).backward(gy)
    gx, gw = ok.rms_norm_backward(x.detach().numpy(), w.detach().numpy(), gy.numpy(), 1e-5)
    assert np.allclose(gx, x.grad.numpy(), atol=1e-5) and np.allclose(gw, w.grad.numpy(), atol=1e-5)

    z = torch.randn(6, 33, generator=g, requires_grad=True)
    tg = [3, 32, 0, 7, 9, 1]
    mk = [1, 1, 0, 1, 1, 1]
    t, wts, _ = ol.batch_targets_weights(tg, mk, 2, vocab=33)
    loss = ol.loss_fn(z.view(2, 3, 33), torch.tensor(tg).view(2, 3), torch.tensor(mk).view(2, 3))
    loss.backward()
    rl, gz = ok.masked_cross_entropy_weighted(z.detach().numpy(), t, wts)
    assert np.allclose(gz, z.grad.numpy(), atol=1e-6)
    assert abs(float((rl * wts).sum()) - float(loss.detach())) < 1e-5

    # rope: kernel formula (flat buffer, position from token index) == model formula
    xr = torch.randn(2, 9, 3 * 8, generator=g)
    a = ol.rope(xr, 3, 8, 500.0).numpy().reshape(-1)
    bb = ok.rope(xr.numpy().reshape(-1), 8, 9, 3, 0, 500.0)
    assert np.allclose(a, bb, atol=1e-6)
    back = ok.rope(bb, 8, 9, 3, 0, 500.0, inverse=True)
    assert np.allclose(back, xr.numpy().reshape(-1), atol=1e-5)


def test_f16_packing_layout():
    # ferrotensor-backend/src/tensor.rs:625-680: element 2i in the low half of word i
    words = ok.pack_f16([1.0, -2.0, 0.5])
    assert words.tolist() == [0x3C00 | (0xC000 << 16), 0x3800]
    # round to nearest even at the f16 grid
    assert ok.f16_round([1.0 + 2.0 ** -11])[0] == 1.0
    assert ok.f16_round([1.0 + 3 * 2.0 ** -11])[0] == np.float32(1.0 + 2.0 ** -9)


def test_dropout_hash_building_blocks_against_published_algorithms():
    """The attention-dropout hash (flash_attention_v2.wgsl:68-104, CPU copy in
    backend/tests/gpu_kernels.rs:2261-2287) is made of two published pieces; the reference holds
    no output vector of it, so the oracle's restatement is pinned piece by piece instead:
    * `fmix32` is MurmurHash3's 32-bit finaliser.  MurmurHash3_x86_32 of an EMPTY key is
      fmix32(seed), so scikit-learn's independent implementation gives known answers.
    * the three steps `v * 1664525 + 1013904223` are the Numerical Recipes generator, whose
      sequence from 0 is published.
    * the cross-multiplication round is checked against exact integer arithmetic reduced mod
      2^32 (guards the wrap-around of the numpy form)."""
    from sklearn.utils import murmurhash3_32
    seeds = [0, 1, 2, 0x9E3779B9, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFF, 123456789, 0xDEADBEEF]
    for s_ in seeds:
        assert int(ok._fmix32(np.uint32(s_))) == murmurhash3_32(b"", seed=s_, positive=True), hex(s_)
    assert int(ok._fmix32(np.uint32(1))) == 0x514E28B7 and int(ok._fmix32(np.uint32(0xFFFFFFFF))) == 0x81F16F39
    # Numerical Recipes LCG from 0
    x, seq = 0, []
    for _ in range(4):
        x = (x * 1664525 + 1013904223) % (1 << 32)
        seq.append(x)
    assert seq == [1013904223, 1196435762, 3519870697, 2868466484]

    def hash3_exact(x, y, z):
        m = 1 << 32
        a, b, c = ((v * 1664525 + 1013904223) % m for v in (x, y, z))
        a = (a + b * c) % m
        b = (b + c * a) % m
        c = (c + a * b) % m
        a, b, c = (v ^ (v >> 16) for v in (a, b, c))
        return np.float32((a + b + c) % m) * np.float32(2.3283064365386963e-10)

    rng = np.random.default_rng(7)
    for x, y, z in rng.integers(0, 1 << 32, size=(200, 3), dtype=np.uint64):
        got = ok._hash3(np.uint32(x), np.uint32(y), np.uint32(z))
        assert np.float32(got) == hash3_exact(int(x), int(y), int(z)), (x, y, z)
    # the keep decision: key = fmix32(lo ^ fmix32(hi ^ golden ratio)), hash3(bh ^ key, q, k) >= p
    seed = 0x0123456789ABCDEF
    key = murmurhash3_32(b"", seed=(seed & 0xFFFFFFFF) ^ murmurhash3_32(
        b"", seed=(seed >> 32) ^ 0x9E3779B9, positive=True), positive=True)
    for bh, q, k in [(0, 0, 0), (3, 17, 5), (31, 1023, 4095)]:
        expect = hash3_exact(bh ^ key, q, k) >= np.float32(0.3)
        assert bool(ok.dropout_keep(0.3, seed, bh, q, k)) == bool(expect)
