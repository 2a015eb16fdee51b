"""Generation on the device: KV-cache decoding through the engine's per-op calls.

The counterpart of `generate_tokens`, `DecodeCache`, `Prompt` and `sample_last_row`
(ferrotensor-cli/src/main.rs:1313-1507), of the cache branch of `Attention::forward`
(ferrotensor-graph/src/lib.rs:416-448) and of `Sampler` (ferrotensor-loader/src/tokenizer.rs:498-583).
One forward pass over `n` new tokens at position `pos` is the reference's op sequence per block:
RMSNorm, q/k/v projections (+ adapters, + bias), RoPE at `pos`, the new keys and values copied
into the cache at `pos`, attention of the `n` queries over the whole cache with
`causal_offset = pos` (slots not written yet are hidden by causality), output projection,
residual, RMSNorm, SwiGLU MLP, residual.  With one new token the projections are matrix-vector
products and the attention is the split-key decode kernel; greedy decoding takes the argmax on
the device and reads back one token id per step.

A sampler with temperature > 0 follows the reference's filtering rules (top-k, then nucleus) but
draws from numpy's generator: its random stream is not the reference's.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .config import LINEARS, LoRaConfig, ModelConfig
from .engine import AttentionOptions, ComputeEngine, CudaContext, DType, UnifiedTensor


class Sampler:
    """Next-token sampler: temperature <= 0 (or top_k == 1) is greedy; top_k == 0 and
    top_p >= 1 switch those filters off."""

    def __init__(self, temperature: float = 0.7, top_k: int = 0, top_p: float = 0.9, seed: Optional[int] = None):
        import os
        from .std_rng import StdRng
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        # the reference's generator: StdRng::seed_from_u64(seed), or seeded from the OS
        # (tokenizer.rs:519-526); one `gen::<f32>()` per sampled token
        self.rng = StdRng.seed_from_u64(int(seed)) if seed is not None else StdRng(os.urandom(32))

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def sample(self, logits: np.ndarray) -> int:
        logits = np.asarray(logits, dtype=np.float32)
        if logits.size == 0:
            return 0
        if self.is_greedy():
            return int(argmax(logits))
        # candidates by logit, highest first, NaNs last
        order = np.argsort(-np.where(np.isnan(logits), -np.inf, logits), kind="stable")
        if self.top_k > 0:
            order = order[:self.top_k]
        f = np.float32
        probs = np.exp((logits[order] - logits[order[0]]) / f(self.temperature)).astype(f)
        # f32 sums in index order, as `iter().sum()` adds them (np.cumsum accumulates sequentially)
        probs = probs / np.cumsum(probs, dtype=f)[-1]
        if self.top_p < 1.0:
            reach = np.nonzero(np.cumsum(probs, dtype=f) >= f(self.top_p))[0]
            keep = int(reach[0]) + 1 if reach.size else len(probs)
            order, probs = order[:keep], probs[:keep]
        r = f(self.rng.gen_f32()) * np.cumsum(probs, dtype=f)[-1]
        for idx, p in zip(order, probs):
            if r < p:
                return int(idx)
            r = f(r - p)
        return int(order[-1])


def argmax(logits: np.ndarray) -> int:
    """Index of the largest logit in f32 total order, the last winning ties
    (`Iterator::max_by` keeps the last maximum)."""
    bits = np.ascontiguousarray(logits, dtype=np.float32).view(np.uint32)
    key = np.where(bits & np.uint32(0x80000000), ~bits, bits | np.uint32(0x80000000))
    best = key.max()
    return int(np.nonzero(key == best)[0][-1])


class _Linear:
    def __init__(self, w: UnifiedTensor, bias=None, a=None, b=None):
        self.w, self.bias, self.a, self.b = w, bias, a, b


class InferenceModel:
    """Device copies of a Llama-style model's weights in the reference's layout ([in, out],
    f16 or f32) and an optional set of LoRA adapters, run through the engine's per-op calls."""

    def __init__(self, ctx: CudaContext, cfg: ModelConfig, weights: Dict[str, torch.Tensor],
                 lora: Optional[LoRaConfig] = None, adapters: Optional[Dict[str, torch.Tensor]] = None,
                 f16_base: bool = True):
        self.ctx, self.cfg, self.engine = ctx, cfg, ComputeEngine(ctx)
        self.f16_base = f16_base
        self.scale = float(np.float32(lora.scale)) if lora is not None and lora.rank > 0 else 0.0
        dt = DType.FP16 if f16_base else DType.F32

        def host(t) -> np.ndarray:
            return t.detach().to(device="cpu", dtype=torch.float32).contiguous().numpy()

        def f32(name) -> UnifiedTensor:
            arr = host(weights[name])
            return UnifiedTensor.new(ctx, arr, list(arr.shape))

        def linear(prefix: str) -> _Linear:
            w = host(weights[f"{prefix}.weight"])                  # Hugging Face [out, in]
            lin = _Linear(UnifiedTensor.from_f32_transposed(ctx, w, list(w.shape), dt))
            if f"{prefix}.bias" in weights:
                lin.bias = f32(f"{prefix}.bias").reshaped([1, w.shape[0]])
            if adapters is not None and f"{prefix}.lora_a" in adapters:
                a, b = host(adapters[f"{prefix}.lora_a"]), host(adapters[f"{prefix}.lora_b"])
                lin.a, lin.b = UnifiedTensor.new(ctx, a, list(a.shape)), UnifiedTensor.new(ctx, b, list(b.shape))
            return lin

        self.embed = f32("model.embed_tokens.weight")
        self.final_norm = f32("model.norm.weight")
        head = host(weights["lm_head.weight"] if "lm_head.weight" in weights else weights["model.embed_tokens.weight"])
        self.head = _Linear(UnifiedTensor.from_f32_transposed(ctx, head, list(head.shape), dt))
        self.layers = []
        for l in range(cfg.layers):
            pre = f"model.layers.{l}"
            self.layers.append({
                "norm1": f32(f"{pre}.input_layernorm.weight"),
                "norm2": f32(f"{pre}.post_attention_layernorm.weight"),
                **{name.split(".")[-1]: linear(f"{pre}.{name}") for name in LINEARS},
            })
        self._ones: Dict[int, UnifiedTensor] = {}

    # ---- building blocks ----------------------------------------------------------------------
    def _project(self, x: UnifiedTensor, lin: _Linear, n: int) -> UnifiedTensor:
        """Y = X W + (alpha/r) (X A) B + 1 bias  (ferrotensor-graph/src/lib.rs:112-142)."""
        ctx, eng = self.ctx, self.engine
        out = UnifiedTensor.empty(ctx, [n, lin.w.shape[1]])
        (eng.matmul_f16b if lin.w.dtype is DType.FP16 else eng.matmul)(ctx, x, lin.w, out)
        if lin.a is not None:
            xa = UnifiedTensor.empty(ctx, [n, lin.a.shape[1]])
            eng.matmul(ctx, x, lin.a, xa)
            delta = UnifiedTensor.empty(ctx, [n, lin.b.shape[1]])
            eng.matmul(ctx, xa, lin.b, delta)
            eng.gradient_scale(ctx, delta, self.scale)
            eng.add(ctx, out, delta, out)
        if lin.bias is not None:
            if n not in self._ones:
                self._ones[n] = UnifiedTensor.new(ctx, np.ones((n, 1), np.float32), [n, 1])
            rows = UnifiedTensor.empty(ctx, [n, lin.bias.shape[1]])
            eng.matmul(ctx, self._ones[n], lin.bias, rows)
            eng.add(ctx, out, rows, out)
        return out

    def new_kv_cache(self, capacity: int) -> List[List[UnifiedTensor]]:
        """Per layer [key, value], each `[1, capacity, kv_heads * head_dim]` of zeros."""
        width = self.cfg.kv_heads * self.cfg.head_dim
        return [[UnifiedTensor.zeros(self.ctx, [1, capacity, width]) for _ in range(2)] for _ in self.layers]

    def forward(self, ids: Sequence[int], pos: int, cache: List[List[UnifiedTensor]]) -> UnifiedTensor:
        """Logits `[1, vocab]` of the last of `ids`, which sit at positions pos .. pos + n - 1;
        their keys and values join `cache`."""
        ctx, eng, c = self.ctx, self.engine, self.cfg
        n, d = len(ids), c.head_dim
        assert n >= 1 and pos + n <= cache[0][0].shape[1], "the KV cache is too small for these positions"
        ids_t = UnifiedTensor.from_bytes(ctx, np.asarray(ids, dtype=np.uint32).tobytes(), [n])
        x = UnifiedTensor.empty(ctx, [n, c.hidden])
        eng.embedding_gather(ctx, self.embed, ids_t, x)
        opts = AttentionOptions(causal=True, causal_offset=pos)
        for ly, (key, value) in zip(self.layers, cache):
            h1 = UnifiedTensor.empty(ctx, [n, c.hidden])
            eng.rms_norm_eps(ctx, x, ly["norm1"], h1, c.eps)
            q, k, v = (self._project(h1, ly[name], n) for name in ("q_proj", "k_proj", "v_proj"))
            eng.rope_theta(ctx, q.reshaped([1, n, c.heads * d]), d, pos, c.theta)
            eng.rope_theta(ctx, k.reshaped([1, n, c.kv_heads * d]), d, pos, c.theta)
            offset = pos * c.kv_heads * d * 4
            eng.copy_tensor(ctx, k, key, offset)
            eng.copy_tensor(ctx, v, value, offset)
            cap = key.shape[1]
            attn = UnifiedTensor.empty(ctx, [1, n, c.heads, d])
            eng.flash_attention_v2_with(ctx, q.reshaped([1, n, c.heads, d]), key.reshaped([1, cap, c.kv_heads, d]),
                                        value.reshaped([1, cap, c.kv_heads, d]), attn, opts)
            o = self._project(attn.reshaped([n, c.heads * d]), ly["o_proj"], n)
            eng.add(ctx, x, o, o)
            h2 = UnifiedTensor.empty(ctx, [n, c.hidden])
            eng.rms_norm_eps(ctx, o, ly["norm2"], h2, c.eps)
            gate, up = self._project(h2, ly["gate_proj"], n), self._project(h2, ly["up_proj"], n)
            f = UnifiedTensor.empty(ctx, [n, c.ffn])
            eng.silu_gate_fused(ctx, gate, up, f)          # the first operand goes through SiLU
            down = self._project(f, ly["down_proj"], n)
            eng.add(ctx, o, down, down)
            x = down
        # only the last row is sampled from: its norm and its logits
        row_bytes = c.hidden * 4
        last = UnifiedTensor(x.storage[(n - 1) * row_bytes:n * row_bytes], [1, c.hidden], DType.F32)
        hn = UnifiedTensor.empty(ctx, [1, c.hidden])
        eng.rms_norm_eps(ctx, last, self.final_norm, hn, c.eps)
        return self._project(hn, self.head, 1)


class DecodeCache:
    """A KV cache and the token ids whose keys and values it holds, at positions 0..len(ids)."""

    def __init__(self, model: InferenceModel, capacity: int, max_positions: Optional[int] = None):
        self.model, self.capacity, self.max_positions = model, int(capacity), max_positions
        self.kv = model.new_kv_cache(self.capacity)
        self.ids: List[int] = []

    def reuse(self, prompt: Sequence[int], length: int) -> int:
        """Keep the cached ids `prompt` starts with (leaving at least its last token to run for
        its logits) and make room for `length` positions; returns how many prompt tokens the
        cache holds.  Keys and values at a position depend only on the tokens up to it."""
        common = 0
        for a, b in zip(self.ids, prompt):
            if a != b:
                break
            common += 1
        keep = min(common, max(len(prompt) - 1, 0))
        del self.ids[keep:]
        if length > self.capacity:
            doubled = 2 * self.capacity
            capacity = max(min(doubled, self.max_positions) if self.max_positions else doubled, length)
            ctx, eng = self.model.ctx, self.model.engine
            for pair in self.kv:
                for i, old in enumerate(pair):
                    new = UnifiedTensor.zeros(ctx, [1, capacity, old.shape[2]])
                    eng.copy_tensor(ctx, old, new, 0)
                    pair[i] = new
            self.capacity = capacity
        return keep

    def feed(self, ids: Sequence[int]) -> UnifiedTensor:
        logits = self.model.forward(ids, len(self.ids), self.kv)
        self.ids.extend(int(t) for t in ids)
        return logits


@dataclass
class Prompt:
    """Prompt token ids and the token ids that end the reply."""
    ids: List[int]
    stop: List[int] = field(default_factory=list)

    @staticmethod
    def raw(tokenizer, config: dict, ids: Sequence[int]) -> "Prompt":
        stop = [tokenizer.eos_token_id]
        eos = config.get("eos_token_id")
        stop += [int(e) for e in (eos if isinstance(eos, list) else [eos] if eos is not None else [])]
        if tokenizer.hf_tokenizer is not None:
            end = tokenizer.hf_tokenizer.token_to_id("<|endoftext|>")
            if end is not None:
                stop.append(int(end))
        return Prompt(list(ids), stop)

    @staticmethod
    def chatml(tokenizer, config: dict, ids: Sequence[int]) -> "Prompt":
        p = Prompt.raw(tokenizer, config, ids)
        if "<|im_end|>" in tokenizer.vocab:
            p.stop.append(tokenizer.vocab["<|im_end|>"])
        return p


@dataclass
class Decoded:
    tokens: List[int]
    new_tokens: int
    cached_tokens: int
    prefill_seconds: float
    decode_steps: int
    decode_seconds: float

    def decode_tokens_per_second(self) -> Optional[float]:
        """Speed of the one-token passes alone; None without one."""
        if self.decode_steps == 0 or self.decode_seconds <= 0:
            return None
        return self.decode_steps / self.decode_seconds


def new_tokens_within(limit: int, prompt_len: int, max_new: int) -> Optional[int]:
    """How many new tokens fit a context of `limit` positions; None when the prompt alone is longer."""
    return None if prompt_len > limit else min(limit - prompt_len, max_new)


def sample_last_row(model: InferenceModel, sampler: Sampler, logits: UnifiedTensor) -> int:
    ctx = model.ctx
    if sampler.is_greedy():
        rows = logits.numel() // model.cfg.vocab
        picks = UnifiedTensor.empty_with_dtype(ctx, [rows], DType.U32)
        model.engine.argmax_rows(ctx, logits.reshaped([rows, model.cfg.vocab]), picks)
        return int(picks.to_vec(ctx)[-1])
    host = logits.to_vec(ctx)
    return sampler.sample(host[-model.cfg.vocab:])


def generate_tokens(model: InferenceModel, prompt: Prompt, max_new: int, sampler: Sampler,
                    cache: Optional[DecodeCache] = None, decode: Optional[Callable[[List[int]], str]] = None,
                    emit: Optional[Callable[[str], None]] = None) -> Decoded:
    """Sample up to `max_new` tokens after `prompt`; with `decode` and `emit`, stream the text
    that each new token adds.  Only the prompt tokens the cache does not hold are run."""
    if not prompt.ids:
        raise ValueError("the prompt encodes to no tokens")
    if cache is None:
        cache = DecodeCache(model, len(prompt.ids) + max_new)
    generated: List[int] = []
    printed = ""
    start = time.perf_counter()
    cached = cache.reuse(prompt.ids, len(prompt.ids) + max_new)
    nxt = sample_last_row(model, sampler, cache.feed(prompt.ids[cached:]))
    prefill = time.perf_counter() - start
    decode_start = time.perf_counter()
    steps = 0
    while len(generated) < max_new:
        if nxt in prompt.stop:
            break
        generated.append(nxt)
        if decode is not None and emit is not None:
            text = decode(generated)
            if text.startswith(printed):
                emit(text[len(printed):])
                printed = text
        if len(generated) == max_new:       # nothing would sample from the logits after the last token
            break
        nxt = sample_last_row(model, sampler, cache.feed([nxt]))
        steps += 1
    return Decoded(generated, len(generated), cached, prefill, steps, time.perf_counter() - decode_start)
