"""Bit-exact restatements of the reference's deterministic generators
(TEST INFRASTRUCTURE - never imported by the product).

  pseudo_random        ferrotensor-graph/tests/common/mod.rs:66-78  (xorshift64*)
  tiny_llama_weights   ferrotensor-graph/tests/common/mod.rs:82-161
  lora_seed            ferrotensor-graph/src/model_builder.rs:746-759 (FNV-1a + splitmix64)
  lora_a_seeded        ferrotensor-graph/src/lib.rs:59-92 (`LoRAAdapter::new_seeded`)
"""

import numpy as np

M64 = (1 << 64) - 1


def _xorshift_units(n: int, state: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    s = state
    for i in range(n):
        s ^= s >> 12
        s ^= (s << 25) & M64
        s ^= s >> 27
        out[i] = np.float32(((s * 0x2545F4914F6CDD1D) & M64) >> 40)
    return out / np.float32(1 << 24)


def pseudo_random(n: int, seed: int, scale: float) -> np.ndarray:
    """Deterministic f32 values in [-scale, scale)."""
    state = ((seed * 0x9E3779B97F4A7C15) & M64) | 1
    u = _xorshift_units(n, state)
    return (u * np.float32(2.0) - np.float32(1.0)) * np.float32(scale)


def tiny_llama_weights(vocab, hidden, heads, kv_heads, layers, ffn, norm_scale=0.25,
                       lm_head=True):
    """name -> f32 array in Hugging Face layout, generated in the reference's order.
    `norm_scale == 0` gives all-ones norm weights (the examples' variant)."""
    head_dim = hidden // heads
    q, kv = heads * head_dim, kv_heads * head_dim
    weights = {}
    seed = [1]

    def add(name, shape, scale, offset):
        seed[0] += 1
        n = int(np.prod(shape))
        if scale == 0.0:
            vals = np.full(n, np.float32(offset), dtype=np.float32)
        else:
            vals = pseudo_random(n, seed[0], scale) + np.float32(offset)
        weights[name] = vals.astype(np.float32).reshape(shape)

    add("model.embed_tokens.weight", [vocab, hidden], 0.5, 0.0)
    for l in range(layers):
        p = f"model.layers.{l}"
        add(f"{p}.self_attn.q_proj.weight", [q, hidden], 0.2, 0.0)
        add(f"{p}.self_attn.k_proj.weight", [kv, hidden], 0.2, 0.0)
        add(f"{p}.self_attn.v_proj.weight", [kv, hidden], 0.2, 0.0)
        add(f"{p}.self_attn.o_proj.weight", [hidden, q], 0.2, 0.0)
        add(f"{p}.mlp.gate_proj.weight", [ffn, hidden], 0.2, 0.0)
        add(f"{p}.mlp.up_proj.weight", [ffn, hidden], 0.2, 0.0)
        add(f"{p}.mlp.down_proj.weight", [hidden, ffn], 0.2, 0.0)
        add(f"{p}.input_layernorm.weight", [hidden], norm_scale, 1.0)
        add(f"{p}.post_attention_layernorm.weight", [hidden], norm_scale, 1.0)
    add("model.norm.weight", [hidden], norm_scale, 1.0)
    if lm_head:
        add("lm_head.weight", [vocab, hidden], 0.2, 0.0)
    return weights


def lora_seed(layer_seed: int, module_name: str) -> int:
    h = 0xCBF29CE484222325
    for b in list(module_name.encode()) + list(layer_seed.to_bytes(8, "little")):
        h ^= b
        h = (h * 0x100000001B3) & M64
    h ^= h >> 30
    h = (h * 0xBF58476D1CE4E5B9) & M64
    h ^= h >> 27
    h = (h * 0x94D049BB133111EB) & M64
    return h ^ (h >> 31)


def lora_a_seeded(in_dim: int, out_dim: int, rank: int, seed: int) -> np.ndarray:
    """Initial A [in, rank], uniform in (-1/sqrt(in), 1/sqrt(in)); B starts at zero."""
    bound = np.float32(1.0) / np.sqrt(np.float32(max(in_dim, 1)))
    state = ((seed * 0x9E3779B97F4A7C15) & M64) + ((in_dim << 32) | (out_dim << 8) | rank)
    state = (state & M64) | 1
    u = _xorshift_units(in_dim * rank, state)
    return ((u * np.float32(2.0) - np.float32(1.0)) * bound).reshape(in_dim, rank)
