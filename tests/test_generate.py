"""Generation: the sampler's rules and the cache bookkeeping on the CPU
(ferrotensor-loader/src/tokenizer.rs:498-583, ferrotensor-cli/src/main.rs:1309-1361,
tests :2746-2763 restated), and on the GPU greedy KV-cache decoding against the oracle's
full-sequence forward."""

import copy

import numpy as np
import pytest

from ferrotensor_b200 import generate as gen


def test_sampler_rules():
    logits = np.array([0.1, 2.0, -1.0, 2.0, np.nan], dtype=np.float32)
    assert gen.Sampler(0.0).is_greedy() and gen.Sampler(0.7, top_k=1).is_greedy() and not gen.Sampler(0.7).is_greedy()
    assert gen.Sampler(0.0).sample(logits) == gen.argmax(logits) == 4      # NaN is the largest in total order
    assert gen.argmax(np.array([1.0, 3.0, 3.0], np.float32)) == 2          # the last maximum wins
    assert gen.Sampler(0.0).sample(np.array([], np.float32)) == 0
    z = np.array([5.0, 4.0, 1.0, 0.0, -3.0], dtype=np.float32)
    picks = {gen.Sampler(1.0, top_k=2, top_p=1.0, seed=s).sample(z) for s in range(50)}
    assert picks == {0, 1}
    picks = {gen.Sampler(1.0, top_k=0, top_p=0.5, seed=s).sample(z) for s in range(50)}
    assert picks == {0}                                                   # the first candidate alone reaches 0.5
    counts = np.bincount([gen.Sampler(1.0, 0, 1.0, seed=s).sample(z) for s in range(400)], minlength=5)
    p = np.exp(z - z.max()); p /= p.sum()
    assert np.abs(counts / 400 - p).max() < 0.08
    a = [gen.Sampler(0.8, 0, 0.9, seed=7).sample(z) for _ in range(3)]
    assert a == [gen.Sampler(0.8, 0, 0.9, seed=7).sample(z) for _ in range(3)]


def test_new_tokens_are_clipped_to_the_context():
    assert gen.new_tokens_within(2048, 2000, 100) == 48
    assert gen.new_tokens_within(2048, 10, 100) == 100
    assert gen.new_tokens_within(2048, 2048, 100) == 0
    assert gen.new_tokens_within(2048, 2049, 100) is None


class _FakeModel:
    """Stands in for the device model: records what the cache asks it to run."""

    class _T:
        def __init__(self, shape):
            self.shape = shape

    def __init__(self):
        self.calls = []
        self.ctx = self.engine = None

    def new_kv_cache(self, capacity):
        return [[self._T([1, capacity, 8]), self._T([1, capacity, 8])]]

    def forward(self, ids, pos, cache):
        self.calls.append((list(ids), pos))
        return None


def test_cache_keeps_the_common_prefix_and_leaves_the_last_prompt_token():
    m = _FakeModel()
    c = gen.DecodeCache(m, 32)
    assert c.reuse([1, 2, 3], 10) == 0
    c.feed([1, 2, 3])
    c.feed([9])
    assert c.ids == [1, 2, 3, 9] and m.calls == [([1, 2, 3], 0), ([9], 3)]
    assert c.reuse([1, 2, 3, 9, 4], 12) == 4 and c.ids == [1, 2, 3, 9]
    assert c.reuse([1, 2, 7], 12) == 2 and c.ids == [1, 2]
    assert c.reuse([1, 2], 12) == 1 and c.ids == [1]         # the last prompt token runs for its logits
    assert c.reuse([5], 12) == 0 and c.ids == []


def test_prompt_stop_tokens():
    class Tok:
        eos_token_id, vocab, hf_tokenizer = 2, {"<|im_end|>": 7}, None
    assert gen.Prompt.raw(Tok, {"eos_token_id": [2, 11]}, [1]).stop == [2, 2, 11]
    assert gen.Prompt.chatml(Tok, {"eos_token_id": 5}, [1]).stop == [2, 5, 7]
    assert gen.Prompt.raw(Tok, {}, [1, 2]).ids == [1, 2]
    d = gen.Decoded([1], 1, 0, 0.1, 0, 0.0)
    assert d.decode_tokens_per_second() is None
    assert gen.Decoded([1, 2, 3], 3, 0, 0.5, 2, 0.25).decode_tokens_per_second() == 8.0


# ---- on the device ----------------------------------------------------------------------------
def _model(cuda_ctx, name, f16, bias=False, tied=False):
    from ferrotensor_b200.config import ALL7, WORKLOADS, LoRaConfig, init_adapters, init_weights
    w = copy.deepcopy(WORKLOADS[name])
    if name != "tiny":
        w.model.layers, w.model.vocab = 2, 1024
        w.lora = LoRaConfig(8, 16.0, ALL7)
    w.model.qkv_bias, w.model.tied = bias, tied
    weights = init_weights(w.model, 13, f16_base=f16, norm_jitter=0.25)
    if tied:
        weights.pop("lm_head.weight", None)
    adapters = init_adapters(w.model, w.lora, 13, b_std=0.05)
    return w, weights, adapters


@pytest.mark.gpu
@pytest.mark.parametrize("name,f16,bias,tied", [("tiny", False, False, False), ("tiny", False, True, True),
                                                 ("smollm2-135m", True, False, True)])
def test_greedy_decoding_matches_the_oracle_forward(cuda_ctx, name, f16, bias, tied):
    """Prefill + one-token passes through the KV cache give the logits the oracle computes by
    running the whole sequence again, and therefore the same greedy tokens."""
    import torch
    from oracle import lora_step as ol
    from tests.test_step_gpu import _oracle_cfg, _oracle_params
    w, weights, adapters = _model(cuda_ctx, name, f16, bias, tied)
    model = gen.InferenceModel(cuda_ctx, w.model, weights, w.lora, adapters, f16_base=f16)
    ocfg = _oracle_cfg(w.model, w.lora, f16_base=f16)
    p = _oracle_params(w.model, weights, adapters, f16)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, w.model.vocab, 11).tolist()
    cache = gen.DecodeCache(model, 16)                     # grows once during the run
    out = gen.generate_tokens(model, gen.Prompt(prompt, stop=[]), 12, gen.Sampler(0.0), cache)
    assert out.new_tokens == 12 and out.decode_steps == 11 and out.cached_tokens == 0 and cache.capacity >= 23
    seq = list(prompt)
    for step, tok in enumerate(out.tokens):
        logits = ol.forward(ocfg, p, torch.tensor([seq]))[0, -1].double().numpy()
        top2 = np.sort(logits)[-2:]
        if top2[1] - top2[0] > 1e-3 * max(1.0, abs(top2[1])):
            assert int(np.argmax(logits)) == tok, f"step {step}"
        seq.append(tok)
    # the logits themselves, for a fresh prefill and for a pass that reuses the cached prefix
    cache2 = gen.DecodeCache(model, 64)
    got = cache2.feed(seq[:9]).to_vec(cuda_ctx)
    exp = ol.forward(ocfg, p, torch.tensor([seq[:9]]))[0, -1].numpy()
    tol = (2e-2, 2e-2) if f16 else (1e-4, 1e-3)
    assert (np.abs(got - exp) <= tol[0] + tol[1] * np.abs(exp)).all()
    assert cache2.reuse(seq[:12], 20) == 9
    got = cache2.feed(seq[9:12]).to_vec(cuda_ctx)
    exp = ol.forward(ocfg, p, torch.tensor([seq[:12]]))[0, -1].numpy()
    assert (np.abs(got - exp) <= tol[0] + tol[1] * np.abs(exp)).all()
    # a second run on the same prompt takes every prompt token but the last from the cache
    again = gen.generate_tokens(model, gen.Prompt(prompt, stop=[]), 12, gen.Sampler(0.0), cache)
    assert again.cached_tokens == len(prompt) - 1 and again.tokens == out.tokens
    # a stop token ends the reply before it is emitted
    stopped = gen.generate_tokens(model, gen.Prompt(prompt, stop=[out.tokens[3]]), 12, gen.Sampler(0.0))
    assert stopped.tokens == out.tokens[:out.tokens.index(out.tokens[3])]


def test_chacha_block_against_published_vectors():
    """The block function behind the sampler's generator (`std_rng.chacha_block`) against
    published known answers: the ChaCha20 block of RFC 7539 section 2.3.2 (key 00..1f, counter 1,
    nonce 00:00:00:09:00:00:00:4a:00:00:00:00) and the all-zero-key keystreams of ChaCha20,
    ChaCha12 and ChaCha8 (test case 1 of the ChaCha test-vector Internet-Draft).  The 12-round
    case is the variant `StdRng` of rand 0.8 runs."""
    from ferrotensor_b200.std_rng import chacha_block
    key = [int.from_bytes(bytes(range(32))[4 * i:4 * i + 4], "little") for i in range(8)]
    assert chacha_block(key, [1, 0x09000000, 0x4a000000, 0], 20) == [
        0xe4e7f110, 0x15593bd1, 0x1fdd0f50, 0xc47120a3, 0xc7f4d1c7, 0x0368c033, 0x9aaa2204, 0x4e6cd4c3,
        0x466482d2, 0x09aa9f07, 0x05d7c214, 0xa2028bd9, 0xd19c12b5, 0xb94e16de, 0xe883d0cb, 0x4e3c50a2]

    def stream(rounds):
        return b"".join(w.to_bytes(4, "little") for w in chacha_block([0] * 8, [0, 0, 0, 0], rounds)).hex()

    assert stream(20).startswith("76b8e0ada0f13d90405d6ae55386bd28bdd219b8a08ded1aa836efcc8b770dc7")
    assert stream(12) == ("9bf49a6a0755f953811fce125f2683d50429c3bb49e074147e0089a52eae155f"
                          "0564f879d27ae3c02ce82834acfa8c793a629f2ca0de6919610be82f411326be")
    assert stream(8).startswith("3e00ef2f895f40d67f5bb8e81f09a5a12c840ec3ce9a7f3b181be188ef711a1e")


def test_std_rng_stream_properties():
    """`StdRng.seed_from_u64`: the same seed gives the same stream, nearby seeds unrelated ones;
    draws lie in [0, 1) on a 2^-24 grid and are uniform; the block counter advances every 16
    words (restated mechanics: no reference-held vector exists for them)."""
    from ferrotensor_b200.std_rng import StdRng, seed_from_u64
    a, b, c = StdRng.seed_from_u64(7), StdRng.seed_from_u64(7), StdRng.seed_from_u64(8)
    xa = [a.gen_f32() for _ in range(64)]
    assert xa == [b.gen_f32() for _ in range(64)]
    xc = [c.gen_f32() for _ in range(64)]
    assert sum(x == y for x, y in zip(xa, xc)) == 0
    assert all(0.0 <= x < 1.0 and (x * (1 << 24)) == int(x * (1 << 24)) for x in xa)
    assert a.counter == 4 and len(seed_from_u64(0)) == 32 and seed_from_u64(0) != seed_from_u64(1)
    big = StdRng.seed_from_u64(123)
    draws = np.array([big.gen_f32() for _ in range(4000)])
    assert abs(draws.mean() - 0.5) < 0.02 and abs(np.mean(draws < 0.25) - 0.25) < 0.03
