"""Hugging Face checkpoint directories -> the weight dict `LoraModel` takes.

Mirrors ferrotensor-loader/src/lib.rs:74-146 (config.json fields, defaults and aliases),
:394-503 (`WeightsContext`: sharded files through `model.safetensors.index.json`, else
`model.safetensors`, else `consolidated.safetensors`; shard names must stay inside the
directory) and ferrotensor-graph/src/model_builder.rs:187-223 (`check_supported`, same
messages), :505-548 (head_dim, KV heads, RoPE base), :623-690 (final norm, tied head).
Tensors are returned as f32 in the Hugging Face `[out, in]` layout; `LoraModel` transposes
to the reference's `[in, out]` and rounds to f16 on upload, as the reference's builder does.
"""

from __future__ import annotations

import json
from pathlib import Path, PurePosixPath
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .checkpoint import CheckpointError, read_safetensors
from .config import LINEARS, ModelConfig

MAX_JSON_FILE_BYTES = 64 * 1024 * 1024
MAX_HIDDEN_SIZE = 1 << 20
MAX_INTERMEDIATE_SIZE = 1 << 22
MAX_VOCAB_SIZE = 1 << 24
MAX_ATTENTION_HEADS = 1 << 16
MAX_HIDDEN_LAYERS = 1 << 14


class LoaderError(RuntimeError):
    pass


class BuildError(RuntimeError):
    pass


def _read_json(path: Path) -> dict:
    if not path.is_file():
        raise LoaderError(f"{path}: not a regular file")
    if path.stat().st_size > MAX_JSON_FILE_BYTES:
        raise LoaderError(f"{path}: file is {path.stat().st_size} bytes, more than the "
                          f"{MAX_JSON_FILE_BYTES} byte limit")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise LoaderError(f"{path}: {e}") from e


def _rope_kind(rope: dict) -> Optional[str]:
    return rope.get("rope_type") or rope.get("type")


def check_supported(config: dict) -> None:
    """model_builder.rs:187-223.  Raises BuildError naming the field and its value."""
    act = config.get("hidden_act")
    if act is not None and act not in ("silu", "swish"):
        raise BuildError(f'hidden_act "{act}" is not supported: the MLP computes SiLU (silu) only')
    for fld in ("rope_scaling", "rope_parameters"):
        rope = config.get(fld)
        if rope is None:
            continue
        kind = _rope_kind(rope)
        if kind is None:
            kind = "default" if rope.get("factor") is None else "unnamed"
        if kind != "default":
            raise BuildError(f'{fld} type "{kind}" is not supported: RoPE runs unscaled')
    if config.get("use_sliding_window") is True:
        w = config.get("sliding_window")
        raise BuildError(f"sliding_window {'unset' if w is None else w} is not supported: "
                         "attention always covers the whole sequence")


def model_config_from_json(config: dict) -> ModelConfig:
    """The fields the step depends on, with the reference's defaults and aliases."""
    try:
        hidden, ffn = int(config["hidden_size"]), int(config["intermediate_size"])
        heads, layers = int(config["num_attention_heads"]), int(config["num_hidden_layers"])
        vocab = int(config["vocab_size"])
    except KeyError as e:
        raise LoaderError(f"config.json: missing field {e}") from e
    for name, v, top in (("hidden_size", hidden, MAX_HIDDEN_SIZE), ("intermediate_size", ffn, MAX_INTERMEDIATE_SIZE),
                         ("vocab_size", vocab, MAX_VOCAB_SIZE), ("num_attention_heads", heads, MAX_ATTENTION_HEADS),
                         ("num_hidden_layers", layers, MAX_HIDDEN_LAYERS)):
        if v <= 0 or v > top:
            raise LoaderError(f"config.json: {name} {v} is out of range (1..={top})")
    eps = config.get("norm_eps", config.get("rms_norm_eps"))
    kv = config.get("num_key_value_heads") or heads
    theta = config.get("rope_theta")
    if theta is None and config.get("rope_parameters"):
        theta = config["rope_parameters"].get("rope_theta")
    head_dim = config.get("head_dim") or hidden // heads
    if head_dim % 2 or head_dim > 128:
        raise BuildError(f"head_dim {head_dim} is not supported (RoPE needs an even size, and the "
                         "attention kernel handles at most 128)")
    return ModelConfig(vocab=vocab, hidden=hidden, layers=layers, heads=heads, kv_heads=int(kv), ffn=ffn,
                       eps=float(np.float32(1e-5 if eps is None else eps)),
                       theta=float(np.float32(10000.0 if theta is None else theta)), head_dim=int(head_dim),
                       tied=bool(config.get("tie_word_embeddings") or False),
                       attention_dropout=float(config.get("attention_dropout") or 0.0))


class WeightsContext:
    """loader/lib.rs:394-560: the tensors of one or more safetensors files by name."""

    def __init__(self):
        self._files: Dict[str, Dict[str, Tuple[List[int], np.ndarray]]] = {}
        self.weight_map: Dict[str, str] = {}

    def load_file(self, path) -> None:
        path = Path(path)
        try:
            tensors, _ = read_safetensors(path)
        except CheckpointError as e:
            raise LoaderError(str(e)) from e
        self._files[path.name] = tensors
        for name in tensors:
            self.weight_map[name] = path.name

    def load_model_dir(self, model_dir) -> None:
        model_dir = Path(model_dir)
        index_path = model_dir / "model.safetensors.index.json"
        if index_path.exists():
            index = _read_json(index_path)
            wm = index.get("weight_map")
            if not isinstance(wm, dict):
                raise LoaderError(f"{index_path}: missing field `weight_map`")
            shards = sorted(set(wm.values()))
            if not shards:
                raise LoaderError(f"{index_path}: weight_map lists no weights")
            for shard in shards:
                parts = PurePosixPath(shard).parts
                inside = bool(parts) and not PurePosixPath(shard).is_absolute() and \
                    all(p not in ("..", ".", "/") and "\\" not in p for p in parts)
                if not inside:
                    raise LoaderError(f'{index_path}: shard path "{shard}" is not a relative path inside '
                                      "the model directory")
            for shard in shards:
                self.load_file(model_dir / shard)
            return
        for name in ("model.safetensors", "consolidated.safetensors"):
            if (model_dir / name).exists():
                self.load_file(model_dir / name)
                return
        raise LoaderError("no model.safetensors, consolidated.safetensors, or model.safetensors.index.json found")

    def tensor_names(self):
        return self.weight_map.keys()

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def get_tensor_info(self, name: str) -> Optional[List[int]]:
        f = self.weight_map.get(name)
        return None if f is None else list(self._files[f][name][0])

    def read(self, name: str) -> np.ndarray:
        f = self.weight_map.get(name)
        if f is None:
            raise LoaderError(f"missing weight {name}")
        return self._files[f][name][1]


def load_model_dir(model_dir) -> Tuple[ModelConfig, Dict[str, torch.Tensor], dict]:
    """config.json + safetensors of a Llama-style checkpoint -> (ModelConfig, weights, raw config).
    `weights` holds f32 tensors under Hugging Face names in `[out, in]` layout; a checkpoint
    without `lm_head.weight` is tied (the head is the embedding table, model_builder.rs:652-686);
    q/k/v biases are taken when present (Qwen2)."""
    model_dir = Path(model_dir)
    raw = _read_json(model_dir / "config.json")
    check_supported(raw)
    cfg = model_config_from_json(raw)
    ctx = WeightsContext()
    ctx.load_model_dir(model_dir)
    if ctx.has("model.layers.0.self_attn.q_layernorm.weight"):
        raise BuildError("LFM2 per-head q/k layernorm is not supported yet")
    if not ctx.has("model.norm.weight"):
        raise BuildError("no final norm (model.norm.weight or model.embedding_norm.weight)")
    cfg.tied = not ctx.has("lm_head.weight")
    cfg.qkv_bias = ctx.has("model.layers.0.self_attn.q_proj.bias")
    shapes = cfg.linear_shapes()
    out: Dict[str, torch.Tensor] = {}

    def take(name: str, shape: Optional[Tuple[int, ...]] = None) -> None:
        arr = ctx.read(name)
        if shape is not None and tuple(arr.shape) != tuple(shape):
            raise BuildError(f"{name} has shape {list(arr.shape)}, the config implies {list(shape)}")
        out[name] = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32))

    take("model.embed_tokens.weight", (cfg.vocab, cfg.hidden))
    take("model.norm.weight", (cfg.hidden,))
    if not cfg.tied:
        take("lm_head.weight", (cfg.vocab, cfg.hidden))
    for l in range(cfg.layers):
        pre = f"model.layers.{l}"
        take(f"{pre}.input_layernorm.weight", (cfg.hidden,))
        take(f"{pre}.post_attention_layernorm.weight", (cfg.hidden,))
        for name in LINEARS:
            take(f"{pre}.{name}.weight", shapes[name])
            if cfg.qkv_bias and name in LINEARS[:3]:
                take(f"{pre}.{name}.bias", (shapes[name][0],))
    return cfg, out, raw
