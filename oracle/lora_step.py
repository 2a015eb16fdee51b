"""Whole-step CPU oracle (TEST INFRASTRUCTURE - never imported by the product).

A parametrised restatement, in plain PyTorch on the CPU, of the reference's
LoRA training step for Llama-style decoders.  Weight names and layouts are the
reference's: base linears in Hugging Face layout `[out, in]`, LoRA factors
`<prefix>.lora_a [in, rank]`, `<prefix>.lora_b [rank, out]`.

Reference lines followed, function by function:
  rms_norm, linear, rope, attention, forward, loss_fn
      scripts/gen_gradient_fixtures.py:131-195
      (= ferrotensor-graph/src/lib.rs:112-142,367-414,504-510,
         ferrotensor-graph/src/lfm.rs:116-139,597-623)
  q/k/v bias                     ferrotensor-graph/src/lib.rs:128-139
  tied head as an f16 copy       ferrotensor-graph/src/model_builder.rs:653-689
  f16 storage of frozen linears  ferrotensor-backend/src/tensor.rs:261-269
  batch_targets_weights          ferrotensor-trainer/src/lib.rs:676-716
  pad_chunk                      ferrotensor-trainer/src/lib.rs:426-450
  global_grad_norm               ferrotensor-trainer/src/lib.rs:507-534
  clip scale                     ferrotensor-trainer/src/lib.rs:336-343
  adamw_update                   ferrotensor-backend/src/shaders/kernels.wgsl:355-387
  WarmupCosine                   ferrotensor-autograd/src/lib.rs:1789-1805
  mean over ranks                ferrotensor-trainer/src/distributed.rs:135-172
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

MASKED_CE_SKIP = 0xFFFFFFFF  # ferrotensor-backend/src/engine/training.rs:7
SUM_SQUARES_CHUNK = 4096  # ferrotensor-backend/src/engine/training.rs:11

LINEARS = (
    "self_attn.q_proj",
    "self_attn.k_proj",
    "self_attn.v_proj",
    "self_attn.o_proj",
    "mlp.gate_proj",
    "mlp.up_proj",
    "mlp.down_proj",
)


@dataclass
class OracleConfig:
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
    lora_rank: int = 0
    lora_alpha: float = 0.0
    # substrings matched against the linear's name, as
    # ferrotensor-graph/src/model_builder.rs:426-446 does
    lora_targets: Tuple[str, ...] = ()
    f16_base: bool = False  # frozen linears (and the head) rounded to f16
    attention_dropout: float = 0.0  # config.json attention_dropout (model_builder.rs:541)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden // self.heads

    @property
    def scale(self) -> float:
        return self.lora_alpha / self.lora_rank if self.lora_rank else 0.0

    def linear_shapes(self) -> Dict[str, Tuple[int, int]]:
        """name -> (out, in) of one block's linears."""
        q = self.heads * self.head_dim
        kv = self.kv_heads * self.head_dim
        return {
            "self_attn.q_proj": (q, self.hidden),
            "self_attn.k_proj": (kv, self.hidden),
            "self_attn.v_proj": (kv, self.hidden),
            "self_attn.o_proj": (self.hidden, q),
            "mlp.gate_proj": (self.ffn, self.hidden),
            "mlp.up_proj": (self.ffn, self.hidden),
            "mlp.down_proj": (self.hidden, self.ffn),
        }

    def targeted(self, name: str) -> bool:
        return self.lora_rank > 0 and any(t in name for t in self.lora_targets)


# ---------------------------------------------------------------------------
# model
# ---------------------------------------------------------------------------


def f16_round(w: torch.Tensor) -> torch.Tensor:
    """IEEE round-to-nearest-even to binary16 and back (what the f16 upload stores)."""
    return w.to(torch.float16).to(w.dtype)


def rms_norm(x, g, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g


def linear(cfg: OracleConfig, p, prefix: str, x):
    w = p[f"{prefix}.weight"]
    out = x @ w.T
    a = p.get(f"{prefix}.lora_a")
    if a is not None:
        # the reference scales (x A) before multiplying by B
        out = out + ((x @ a) * cfg.scale) @ p[f"{prefix}.lora_b"]
    b = p.get(f"{prefix}.bias")
    if b is not None:
        out = out + b
    return out


def rope_tables(seq: int, head_dim: int, theta: float, dtype=torch.float32):
    """cos/sin [seq, head_dim/2]: angle = f32(pos) * theta^(-2i/d) evaluated in f32."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    freq = torch.tensor(theta, dtype=torch.float32).pow(-2.0 * i / head_dim)
    angle = torch.arange(seq, dtype=torch.float32)[:, None] * freq[None, :]
    return angle.cos().to(dtype), angle.sin().to(dtype)


def rope(x, heads: int, head_dim: int, theta: float):
    b, s, _ = x.shape
    x = x.view(b, s, heads, head_dim)
    half = head_dim // 2
    cos, sin = rope_tables(s, head_dim, theta, x.dtype)
    cos, sin = cos[None, :, None, :], sin[None, :, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).view(b, s, heads * head_dim)


def _mix64(z: int) -> int:
    m = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def derive_seed(parts: Sequence[int]) -> int:
    """ferrotensor-graph/src/dropout.rs:25-32: fold of SplitMix64 finalisers over the list."""
    acc = _mix64(len(parts))
    for part in parts:
        acc = _mix64(acc ^ _mix64(part & ((1 << 64) - 1)))
    return acc


def attention(cfg: OracleConfig, q, k, v, dropout_seed: Optional[int] = None):
    """`dropout_seed` (the layer's seed) multiplies the softmax weights by the keep mask of
    flash_attention_v2.wgsl:94-104 scaled by 1/(1-p); None = evaluation, no dropout."""
    b, s, _ = q.shape
    h, hk, d = cfg.heads, cfg.kv_heads, cfg.head_dim
    q = q.view(b, s, h, d).transpose(1, 2)
    k = k.view(b, s, hk, d).transpose(1, 2).repeat_interleave(h // hk, dim=1)
    v = v.view(b, s, hk, d).transpose(1, 2).repeat_interleave(h // hk, dim=1)
    scores = q @ k.transpose(-1, -2) / math.sqrt(d)
    causal = torch.ones(s, s, dtype=torch.bool).tril()
    scores = scores.masked_fill(~causal, float("-inf"))
    weights = scores.softmax(-1)
    if dropout_seed is not None and cfg.attention_dropout > 0.0:
        import numpy as np
        from .kernels import dropout_keep
        bh = (np.arange(b)[:, None] * h + np.arange(h)[None, :])[:, :, None, None]
        keep = dropout_keep(cfg.attention_dropout, dropout_seed, bh, np.arange(s)[None, None, :, None],
                            np.arange(s)[None, None, None, :])
        scale = 1.0 / (1.0 - float(np.float32(cfg.attention_dropout)))
        weights = weights * torch.as_tensor(keep.astype(np.float64) * scale, dtype=weights.dtype)
    out = weights @ v
    return out.transpose(1, 2).reshape(b, s, h * d)


def forward(cfg: OracleConfig, p, ids: torch.Tensor, return_hidden: bool = False,
            dropout_seed: Optional[int] = None):
    """ids [B, S] int64 -> logits [B, S, V].  Out-of-range ids embed as zero rows
    (ferrotensor-autograd/src/lib.rs:1163-1168).  `dropout_seed` is the forward pass's seed;
    layer l draws its masks from derive_seed([dropout_seed, l]) (lfm.rs:568)."""
    emb = p["model.embed_tokens.weight"]
    in_range = ids < cfg.vocab
    x = emb[ids.clamp(max=cfg.vocab - 1)] * in_range[..., None].to(emb.dtype)
    for l in range(cfg.layers):
        pre = f"model.layers.{l}"
        h = rms_norm(x, p[f"{pre}.input_layernorm.weight"], cfg.eps)
        q = rope(linear(cfg, p, f"{pre}.self_attn.q_proj", h), cfg.heads, cfg.head_dim, cfg.theta)
        k = rope(linear(cfg, p, f"{pre}.self_attn.k_proj", h), cfg.kv_heads, cfg.head_dim, cfg.theta)
        v = linear(cfg, p, f"{pre}.self_attn.v_proj", h)
        layer_seed = None if dropout_seed is None else derive_seed([dropout_seed, l])
        x = x + linear(cfg, p, f"{pre}.self_attn.o_proj", attention(cfg, q, k, v, layer_seed))
        h = rms_norm(x, p[f"{pre}.post_attention_layernorm.weight"], cfg.eps)
        gate = linear(cfg, p, f"{pre}.mlp.gate_proj", h)
        up = linear(cfg, p, f"{pre}.mlp.up_proj", h)
        x = x + linear(cfg, p, f"{pre}.mlp.down_proj", torch.nn.functional.silu(gate) * up)
    hidden = rms_norm(x, p["model.norm.weight"], cfg.eps)
    logits = linear(cfg, p, "lm_head", hidden)
    return (logits, hidden) if return_hidden else logits


def loss_fn(logits, targets, masks):
    """Sum over sequences of the mean CE over each sequence's supervised positions.

    `targets` may hold ids >= vocab: those positions are unsupervised
    (ferrotensor-trainer/src/lib.rs:689-694)."""
    vocab = logits.shape[-1]
    ok = masks.to(torch.bool) & (targets < vocab)
    per_pos = torch.nn.functional.cross_entropy(
        logits.reshape(-1, vocab), targets.clamp(max=vocab - 1).reshape(-1), reduction="none"
    ).view(targets.shape)
    m = ok.to(logits.dtype)
    tokens = m.sum(-1)
    per_seq = (per_pos * m).sum(-1) / tokens.clamp(min=1.0)
    return per_seq.sum()


# ---------------------------------------------------------------------------
# host-side integer logic
# ---------------------------------------------------------------------------


def batch_targets_weights(target_ids: Sequence[int], loss_mask: Sequence[int], sequences: int,
                          vocab: int):
    """Row targets (u32, MASKED_CE_SKIP when unsupervised) and row weights
    1/tokens(sequence) as the trainer builds them for the CE kernel."""
    rows = len(target_ids)
    assert rows % sequences == 0
    seq_len = rows // sequences
    sup = [loss_mask[r] != 0 and target_ids[r] < vocab for r in range(rows)]
    tokens = [sum(sup[s * seq_len:(s + 1) * seq_len]) for s in range(sequences)]
    targets = np.empty(rows, dtype=np.uint32)
    weights = np.empty(rows, dtype=np.float32)
    for r in range(rows):
        if sup[r]:
            targets[r] = target_ids[r]
            weights[r] = np.float32(1.0) / np.float32(tokens[r // seq_len])
        else:
            targets[r] = MASKED_CE_SKIP
            weights[r] = 0.0
    return targets, weights, tokens


def pad_chunk(chunk: Sequence[Tuple[Sequence[int], Sequence[int], Sequence[int]]], bucket: int = 32):
    """Right-pad (input_ids, target_ids, loss_mask) triples to a common multiple of
    `bucket`: inputs and targets with the sequence's own last input id, masks with 0."""
    longest = max(min(len(i), len(t)) for i, t, _ in chunk)
    padded = -(-longest // bucket) * bucket
    ids, tgt, msk = [], [], []
    for i, t, m in chunk:
        n = min(len(i), len(t))
        pad = i[n - 1] if n else 0
        ids.append(list(i[:n]) + [pad] * (padded - n))
        tgt.append(list(t[:n]) + [pad] * (padded - n))
        msk.append([m[j] if j < len(m) else 0 for j in range(n)] + [0] * (padded - n))
    return ids, tgt, msk


def shard_indices(n: int, world: int, rank: int) -> List[int]:
    """ferrotensor-trainer/src/distributed.rs:222-227: round-robin sharding."""
    return [i for i in range(n) if i % world == rank]


# ---------------------------------------------------------------------------
# optimizer side
# ---------------------------------------------------------------------------


def global_grad_norm(grads: Sequence[torch.Tensor]) -> float:
    """f32 chunk partials of 4096 elements summed in f64, sqrt, cast to f32."""
    total = 0.0
    for g in grads:
        flat = g.detach().reshape(-1).to(torch.float32)
        for start in range(0, flat.numel(), SUM_SQUARES_CHUNK):
            c = flat[start:start + SUM_SQUARES_CHUNK]
            total += float((c * c).sum(dtype=torch.float32))
    return float(np.float32(math.sqrt(total)))


def clip_scale(norm: float, max_norm: Optional[float]) -> Optional[float]:
    if max_norm is None or not norm > max_norm:
        return None
    return float(np.float32(max_norm) / (np.float32(norm) + np.float32(1e-6)))


@dataclass
class AdamParams:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    t: float = 0.0


def adamw_update(w, g, m, v, hp: AdamParams):
    """In place on f32 tensors; every scalar is f32 as in the shader."""
    f = np.float32
    b1, b2 = f(hp.beta1), f(hp.beta2)
    m.mul_(float(b1)).add_(g, alpha=float(f(1.0) - b1))
    v.mul_(float(b2)).addcmul_(g, g, value=float(f(1.0) - b2))
    c1 = f(1.0) - np.power(b1, f(hp.t), dtype=f)
    c2 = f(1.0) - np.power(b2, f(hp.t), dtype=f)
    m_hat = m / float(c1)
    v_hat = v / float(c2)
    w.sub_(float(f(hp.lr)) * (m_hat / (v_hat.sqrt() + float(f(hp.eps))) + float(f(hp.weight_decay)) * w))


def warmup_cosine_lr(current: int, peak: float, min_lr: float, warmup: int, total: int) -> float:
    f = np.float32
    if current < warmup:
        return float(f(peak) * (f(current) / f(warmup)))
    if current >= total:
        return float(f(min_lr))
    progress = f(current - warmup) / f(total - warmup)
    cosine = (f(1.0) + np.cos(f(np.pi) * progress, dtype=f)) / f(2.0)
    return float(f(min_lr) + (f(peak) - f(min_lr)) * cosine)


# ---------------------------------------------------------------------------
# the step
# ---------------------------------------------------------------------------


def trainable_names(p) -> List[str]:
    return sorted(n for n in p if n.endswith(".lora_a") or n.endswith(".lora_b"))


@dataclass
class StepResult:
    loss: float
    per_sequence: List[Tuple[float, int]]
    logits: torch.Tensor
    grads: Dict[str, torch.Tensor]
    grad_norm: float = 0.0
    clip: Optional[float] = None
    skipped: bool = False


def forward_backward(cfg: OracleConfig, p, ids, targets, masks, seed_scale: float = 1.0,
                     train: Optional[Sequence[str]] = None, dtype=torch.float32,
                     dropout_seed: Optional[int] = None) -> StepResult:
    """One micro-batch: forward, loss, autograd backward seeded with `seed_scale`
    (the trainer's 1/grad_accum_steps).  Returns grads of the LoRA factors (or `train`)."""
    q = {n: t.detach().to(dtype).clone() for n, t in p.items()}
    names = list(train) if train is not None else trainable_names(q)
    for n in names:
        q[n].requires_grad_(True)
    ids = torch.as_tensor(ids, dtype=torch.long)
    targets = torch.as_tensor(targets, dtype=torch.long)
    masks = torch.as_tensor(masks, dtype=torch.long)
    logits = forward(cfg, q, ids, dropout_seed=dropout_seed)
    loss = loss_fn(logits, targets, masks)
    (loss * seed_scale).backward()
    vocab = logits.shape[-1]
    ok = masks.to(torch.bool) & (targets < vocab)
    per_pos = torch.nn.functional.cross_entropy(
        logits.detach().reshape(-1, vocab), targets.clamp(max=vocab - 1).reshape(-1),
        reduction="none").view(targets.shape)
    per_seq = []
    for s in range(ids.shape[0]):
        t = int(ok[s].sum())
        per_seq.append((float((per_pos[s] * ok[s]).sum(dtype=torch.float64) / max(t, 1)), t))
    grads = {n: (q[n].grad if q[n].grad is not None else torch.zeros_like(q[n])).detach()
             for n in names}
    return StepResult(float(loss.detach()), per_seq, logits.detach(), grads)


def apply_gradients(p, grads: Dict[str, torch.Tensor], state: Dict[str, Dict[str, torch.Tensor]],
                    hp: AdamParams, clip_grad_norm: Optional[float] = None):
    """Norm -> skip if non-finite -> clip -> AdamW (t incremented first), in place on `p`.
    `grads` are already averaged over ranks.  Returns (norm, clip_scale or None, skipped)."""
    names = sorted(grads)
    norm = global_grad_norm([grads[n] for n in names])
    if not math.isfinite(norm):
        return norm, None, True
    scale = clip_scale(norm, clip_grad_norm)
    if scale is not None:
        for n in names:
            grads[n] = grads[n] * scale
    hp.t += 1.0
    for n in names:
        st = state.setdefault(n, {"m": torch.zeros_like(p[n]), "v": torch.zeros_like(p[n])})
        adamw_update(p[n], grads[n].to(p[n].dtype), st["m"], st["v"], hp)
    return norm, scale, False


def lora_step(cfg: OracleConfig, p, micro_batches, hp: AdamParams,
              state: Optional[Dict] = None, clip_grad_norm: Optional[float] = None,
              world: int = 1, dtype=torch.float32):
    """A full optimizer step.

    `micro_batches` is a list over ranks of lists of (ids, targets, masks) micro-batches.
    Every rank seeds backward with 1/(its own sequence count) and the rank gradients are
    averaged (ferrotensor-trainer/src/lib.rs:474, distributed.rs:135-172).  With world == 1
    pass `[[mb0, mb1, ...]]`."""
    if state is None:
        state = {}
    assert len(micro_batches) == world
    rank_grads = []
    results = []
    for mbs in micro_batches:
        accum = sum(len(mb[0]) for mb in mbs)
        acc: Dict[str, torch.Tensor] = {}
        for ids, tg, mk in mbs:
            r = forward_backward(cfg, p, ids, tg, mk, seed_scale=1.0 / accum, dtype=dtype)
            results.append(r)
            for n, g in r.grads.items():
                acc[n] = g if n not in acc else acc[n] + g
        rank_grads.append(acc)
    grads = {n: sum(rg[n] for rg in rank_grads) / world for n in rank_grads[0]}
    pre_clip = {n: g.clone() for n, g in grads.items()}
    norm, scale, skipped = apply_gradients(p, grads, state, hp, clip_grad_norm)
    return results, pre_clip, norm, scale, skipped, state
