"""Model / adapter configuration, the five benchmark workloads, and their seeded
synthetic weights and token batches.

The checkpoints and datasets the reference was measured on are not available offline, so
every workload uses random-init weights of the named architecture and synthetic token
ids with the stated distribution.  Weight names and layouts are Hugging Face's
(`model.layers.N.self_attn.q_proj.weight` `[out, in]`), adapters are the reference's
(`<prefix>.lora_a [in, rank]`, `<prefix>.lora_b [rank, out]`;
ferrotensor-graph/src/lib.rs:28-54,191-202).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

LINEARS = (
    "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
    "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj",
)


@dataclass
class ModelConfig:
    """The fields of a Hugging Face config.json the step depends on
    (ferrotensor-loader/src/lib.rs:74-146)."""
    vocab: int
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    ffn: int
    eps: float = 1e-5
    theta: float = 10000.0
    head_dim: Optional[int] = None
    tied: bool = False
    qkv_bias: bool = False
    attention_dropout: float = 0.0   # applied to attention weights in training passes only

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden // self.heads

    def linear_shapes(self) -> Dict[str, Tuple[int, int]]:
        """name -> (out, in)"""
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        return {
            "self_attn.q_proj": (q, self.hidden), "self_attn.k_proj": (kv, self.hidden),
            "self_attn.v_proj": (kv, self.hidden), "self_attn.o_proj": (self.hidden, q),
            "mlp.gate_proj": (self.ffn, self.hidden), "mlp.up_proj": (self.ffn, self.hidden),
            "mlp.down_proj": (self.hidden, self.ffn),
        }

    def base_parameters(self) -> int:
        per_layer = sum(o * i for o, i in self.linear_shapes().values())
        return self.layers * per_layer + self.vocab * self.hidden * (1 if self.tied else 2)


@dataclass
class LoRaConfig:
    """ferrotensor-graph/src/model_builder.rs:111-135.  A linear carries an adapter when its
    name contains one of `target_modules` (model_builder.rs:426-446)."""
    rank: int = 0
    alpha: float = 0.0
    target_modules: Tuple[str, ...] = ()

    def targeted(self, name: str) -> bool:
        return self.rank > 0 and any(t in name for t in self.target_modules)

    @property
    def scale(self) -> float:
        return self.alpha / self.rank if self.rank else 0.0


QKVO = ("q_proj", "k_proj", "v_proj", "o_proj")
ALL7 = QKVO + ("gate_proj", "up_proj", "down_proj")


@dataclass
class Workload:
    name: str
    model: ModelConfig
    lora: LoRaConfig
    seq_len: int
    global_batch: int
    f16_base: bool
    checkpoint_blocks: bool = False
    ids: str = "zipf"            # "zipf" (s = 1.1) or "uniform"
    mask: str = "full"           # "full" | "bernoulli0.8" | "prefix10-40"
    adapter_b_std: float = 0.0   # B ~ N(0, std); 0 = the reference's zero init
    lr: float = 1e-3
    weight_decay: float = 0.01
    clip: Optional[float] = 1.0
    seed: int = 1234


WORKLOADS: Dict[str, Workload] = {
    # gradient-parity shape, runnable on a CPU: everything f32
    "tiny": Workload(
        "tiny", ModelConfig(vocab=256, hidden=32, layers=2, heads=4, kv_heads=2, ffn=64,
                            eps=1e-5, theta=10000.0, tied=False),
        LoRaConfig(4, 8.0, ALL7), seq_len=16, global_batch=2, f16_base=False, ids="uniform",
        mask="bernoulli0.8", adapter_b_std=0.01, clip=None),
    "smollm2-135m": Workload(
        "smollm2-135m", ModelConfig(vocab=49152, hidden=576, layers=30, heads=9, kv_heads=3,
                                    ffn=1536, eps=1e-5, theta=10000.0, tied=True),
        LoRaConfig(8, 16.0, QKVO), seq_len=256, global_batch=8, f16_base=True),
    "smollm2-360m": Workload(
        "smollm2-360m", ModelConfig(vocab=49152, hidden=960, layers=32, heads=15, kv_heads=5,
                                    ffn=2560, eps=1e-5, theta=10000.0, tied=True),
        LoRaConfig(8, 16.0, ALL7), seq_len=512, global_batch=32, f16_base=True,
        checkpoint_blocks=True, mask="prefix10-40"),
    # headline
    "smollm2-1.7b": Workload(
        "smollm2-1.7b", ModelConfig(vocab=49152, hidden=2048, layers=24, heads=32, kv_heads=32,
                                    ffn=8192, eps=1e-5, theta=130000.0, tied=True),
        LoRaConfig(16, 32.0, ALL7), seq_len=1024, global_batch=64, f16_base=True),
    "qwen2-0.5b": Workload(
        "qwen2-0.5b", ModelConfig(vocab=151936, hidden=896, layers=24, heads=14, kv_heads=2,
                                  ffn=4864, eps=1e-6, theta=1e6, tied=True, qkv_bias=True),
        LoRaConfig(8, 16.0, QKVO), seq_len=4096, global_batch=16, f16_base=True),
}


# ---------------------------------------------------------------------------------------
# seeded synthetic weights
# ---------------------------------------------------------------------------------------

def init_weights(cfg: ModelConfig, seed: int, device="cpu", f16_base=False,
                 norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    """Base weights ~ N(0, 0.02) in Hugging Face layout, f32.  With `f16_base` the linear
    weights already hold binary16-representable values, so that the f16 device copy and an
    f32 consumer of this dict see identical numbers.  Norm weights are 1 (+ U(+-jitter))."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)

    def normal(shape):
        w = torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * 0.02
        return w.to(torch.float16).to(torch.float32) if f16_base else w

    def norm(n):
        w = torch.ones(n, device=dev)
        if norm_jitter:
            w = w + (torch.rand(n, generator=g, device=dev) * 2 - 1) * norm_jitter
        return w

    out: Dict[str, torch.Tensor] = {}
    out["model.embed_tokens.weight"] = torch.randn(
        (cfg.vocab, cfg.hidden), generator=g, device=dev, dtype=torch.float32) * 0.02
    for l in range(cfg.layers):
        pre = f"model.layers.{l}"
        for name, (o, i) in cfg.linear_shapes().items():
            out[f"{pre}.{name}.weight"] = normal((o, i))
            if cfg.qkv_bias and name in LINEARS[:3]:
                out[f"{pre}.{name}.bias"] = torch.randn(
                    o, generator=g, device=dev, dtype=torch.float32) * 0.02
        out[f"{pre}.input_layernorm.weight"] = norm(cfg.hidden)
        out[f"{pre}.post_attention_layernorm.weight"] = norm(cfg.hidden)
    out["model.norm.weight"] = norm(cfg.hidden)
    if not cfg.tied:
        out["lm_head.weight"] = normal((cfg.vocab, cfg.hidden))
    return out


def head_weight(cfg: ModelConfig, weights: Dict[str, torch.Tensor], f16_base: bool) -> torch.Tensor:
    """[vocab, hidden] matrix the logits are computed with.  A tied head is a separate copy of
    the embedding, rounded to f16 on its own when the base is stored as f16
    (ferrotensor-graph/src/model_builder.rs:653-689)."""
    if not cfg.tied:
        return weights["lm_head.weight"]
    w = weights["model.embed_tokens.weight"]
    return w.to(torch.float16).to(torch.float32) if f16_base else w


def init_adapters(cfg: ModelConfig, lora: LoRaConfig, seed: int, device="cpu",
                  b_std: float = 0.0) -> Dict[str, torch.Tensor]:
    """A ~ N(0, 1/sqrt(in)), B ~ N(0, b_std) (zeros when b_std == 0)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed + 7919)
    out: Dict[str, torch.Tensor] = {}
    for l in range(cfg.layers):
        for name, (o, i) in cfg.linear_shapes().items():
            if not lora.targeted(name):
                continue
            pre = f"model.layers.{l}.{name}"
            out[f"{pre}.lora_a"] = torch.randn((i, lora.rank), generator=g, device=dev) / math.sqrt(i)
            b = torch.randn((lora.rank, o), generator=g, device=dev) * b_std if b_std else \
                torch.zeros((lora.rank, o), device=dev)
            out[f"{pre}.lora_b"] = b
    return out


# ---------------------------------------------------------------------------------------
# seeded synthetic batches
# ---------------------------------------------------------------------------------------

def _zipf_sampler(vocab: int, seed: int):
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    p = ranks ** -1.1
    cdf = np.cumsum(p / p.sum())
    perm = np.random.default_rng(seed ^ 0x5EED).permutation(vocab)  # rank -> token id

    def draw(rng, n):
        r = np.searchsorted(cdf, rng.random(n), side="left").clip(0, vocab - 1)
        return perm[r]
    return draw


def synthetic_batch(w: Workload, sequences: int, seed: Optional[int] = None, first: int = 0):
    """`sequences` rows of the workload's token stream, starting at global row `first`:
    ids [n, S] and targets [n, S] (ids shifted by one, last target drawn) as uint32,
    loss mask [n, S] uint8.  Row i depends only on (seed, first + i), so data-parallel
    ranks can draw their own rows."""
    seed = w.seed if seed is None else seed
    s, v = w.seq_len, w.model.vocab
    ids = np.empty((sequences, s), dtype=np.uint32)
    tgt = np.empty((sequences, s), dtype=np.uint32)
    msk = np.ones((sequences, s), dtype=np.uint8)
    zipf = _zipf_sampler(v, seed) if w.ids == "zipf" else None
    for r in range(sequences):
        rng = np.random.default_rng([seed, first + r])
        row = zipf(rng, s + 1) if zipf else rng.integers(0, v, s + 1)
        ids[r], tgt[r] = row[:-1], row[1:]
        if w.mask == "bernoulli0.8":
            m = (rng.random(s) < 0.8).astype(np.uint8)
            if not m.any():
                m[-1] = 1
            msk[r] = m
        elif w.mask == "prefix10-40":
            msk[r, : int(s * rng.uniform(0.10, 0.40))] = 0
    return ids, tgt, msk


def gemm_flops(w: Workload, tokens: int) -> float:
    """The dense-contraction part of `step_flops`: frozen projections and head (forward +
    input gradient) and the adapter products (forward + two gradients); no attention."""
    c, lo = w.model, w.lora
    p_layer = sum(o * i for o, i in c.linear_shapes().values())
    base = 2 * 2 * (c.layers * p_layer + c.hidden * c.vocab)
    lora = 6 * lo.rank * sum(o + i for n, (o, i) in c.linear_shapes().items() if lo.targeted(n)) * c.layers
    return float(tokens) * (base + lora)


def step_flops(w: Workload, tokens: int) -> float:
    """Algorithmic FLOPs of one step over `tokens` positions, in the reference's
    conventions (matmul 2MNK; causal attention forward 2 S^2 D per head and sequence,
    backward 2.5x): frozen base forward + input gradient, adapters forward + 2 gradients."""
    c, lo = w.model, w.lora
    p_layer = sum(o * i for o, i in c.linear_shapes().values())
    base = 2 * 2 * (c.layers * p_layer + c.hidden * c.vocab)
    lora = 6 * lo.rank * sum(o + i for n, (o, i) in c.linear_shapes().items() if lo.targeted(n)) * c.layers
    attn = 7 * w.seq_len * c.heads * c.head_dim * c.layers
    return float(tokens) * (base + lora + attn)
