"""Adapter and training-state files in the reference's formats.

Mirrors ferrotensor-trainer/src/checkpoint.rs: adapters are F32 safetensors with the LoRA
settings in the header metadata (checkpoint.rs:42-163), read back as F32 from F32/F16/BF16
(:168-212) and applied all-or-nothing (:214-297); the training state is pretty JSON
(:312-412) and the optimizer moments sit beside it in `x.state.safetensors` under `m/<name>`
and `v/<name>` with the step recorded, so a torn save is detected (:414-612).  Tensor names are
the reference's (`model.layers.N.self_attn.q_proj.lora_A.weight` `[in, r]`, `...lora_B.weight`
`[r, out]`, graph/lib.rs:191-202), so its `eval`, `merge` and `export-adapter` commands can
read what this library trained, and this library can resume from what the reference saved.

The safetensors container is written and parsed here (8-byte little-endian header length, JSON
header padded with spaces to a multiple of 8, raw little-endian data), not through a package.
"""

from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np

_DTYPES = {"F32": (np.dtype("<f4"), 4), "F16": (np.dtype("<f2"), 2), "BF16": (None, 2)}


class CheckpointError(RuntimeError):
    pass


# ---- safetensors container -----------------------------------------------------------------
def write_safetensors(path, tensors: Dict[str, np.ndarray], metadata: Optional[Dict[str, str]] = None,
                      tmp_suffix: str = ".tmp") -> None:
    """F32 tensors in name order; the file appears under its final name only when complete."""
    path = Path(path)
    header: Dict[str, object] = {}
    if metadata is not None:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        arr = np.ascontiguousarray(tensors[name], dtype="<f4")
        blob = arr.tobytes()
        header[name] = {"dtype": "F32", "shape": [int(d) for d in arr.shape],
                        "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path.with_name(path.name + tmp_suffix)
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for blob in blobs:
            f.write(blob)
    os.replace(tmp, path)


def _bf16_to_f32(raw: bytes) -> np.ndarray:
    half = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
    return half.view(np.float32)


def read_safetensors(path) -> Tuple[Dict[str, Tuple[List[int], np.ndarray]], Optional[Dict[str, str]]]:
    """name -> (shape, f32 values); F16 and BF16 are widened (checkpoint.rs:183-207)."""
    path = Path(path)
    try:
        data = path.read_bytes()
    except OSError as e:
        raise CheckpointError(f"cannot read {path}: {e}") from e
    if len(data) < 8:
        raise CheckpointError(f"{path} is not a safetensors file: too short")
    (n,) = struct.unpack("<Q", data[:8])
    if n > len(data) - 8:
        raise CheckpointError(f"{path} is not a safetensors file: header length {n}")
    try:
        header = json.loads(data[8:8 + n].decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise CheckpointError(f"{path} is not a safetensors file: {e}") from e
    metadata = header.pop("__metadata__", None)
    body = memoryview(data)[8 + n:]
    out: Dict[str, Tuple[List[int], np.ndarray]] = {}
    for name, info in header.items():
        dtype, shape = info["dtype"], [int(d) for d in info["shape"]]
        b, e = info["data_offsets"]
        if dtype not in _DTYPES:
            raise CheckpointError(f"tensor {name} has unsupported dtype {dtype}")
        count = int(np.prod(shape)) if shape else 1
        if e - b != count * _DTYPES[dtype][1] or e > len(body):
            raise CheckpointError(f"tensor {name}: data range does not match its shape")
        raw = bytes(body[b:e])
        if dtype == "BF16":
            vals = _bf16_to_f32(raw)
        else:
            vals = np.frombuffer(raw, dtype=_DTYPES[dtype][0]).astype(np.float32)
        out[name] = (shape, vals.reshape(shape) if shape else vals.reshape(()))
    return out, metadata


def _rust_f32(x: float) -> str:
    """How Rust's `f32::to_string` prints (shortest round-trip digits, no exponent, no `.0`)."""
    v = np.float32(x)
    if np.isnan(v):
        return "NaN"
    if np.isinf(v):
        return "inf" if v > 0 else "-inf"
    s = np.format_float_positional(v, unique=True, trim="-")
    return s


# ---- adapter files -------------------------------------------------------------------------
@dataclass
class LoraMetadata:
    """checkpoint.rs:42-103"""
    rank: int
    alpha: float
    target_modules: List[str] = field(default_factory=list)
    trained_modules: Optional[str] = None

    @staticmethod
    def trained_weights(trained_modules: str) -> "LoraMetadata":
        return LoraMetadata(0, 0.0, [], trained_modules)

    def to_map(self) -> Dict[str, str]:
        m = {"format": "ferrotensor-weights" if self.trained_modules is not None else "ferrotensor-lora",
             "rank": str(int(self.rank)), "alpha": _rust_f32(self.alpha),
             "target_modules": ",".join(self.target_modules)}
        if self.trained_modules is not None:
            m["trained_modules"] = self.trained_modules
        return m

    @staticmethod
    def from_map(m: Dict[str, str]) -> Optional["LoraMetadata"]:
        try:
            rank = int(m["rank"])
            alpha = float(m["alpha"])
            targets = [s for s in m["target_modules"].split(",") if s]
        except (KeyError, ValueError):
            return None
        if rank < 0:
            return None
        trained = m.get("trained_modules") or None
        return LoraMetadata(rank, alpha, targets, trained)


@dataclass
class LoraCheckpoint:
    """checkpoint.rs:105-123"""
    tensors: Dict[str, Tuple[List[int], np.ndarray]]
    metadata: Optional[LoraMetadata]

    def __len__(self) -> int:
        return len(self.tensors)

    def is_empty(self) -> bool:
        return not self.tensors


def save_lora_checkpoint(path, tensors: Dict[str, np.ndarray], metadata: Optional[LoraMetadata]) -> None:
    """checkpoint.rs:125-163.  Every tensor must be f32."""
    for name, t in tensors.items():
        if np.asarray(t).dtype != np.float32:
            raise CheckpointError(f"tensor {name} is stored as {np.asarray(t).dtype}; only f32 tensors can be saved")
    path = Path(path)
    # `path.with_extension("safetensors.tmp")` in the reference: x.safetensors -> x.safetensors.tmp
    write_safetensors(path, {k: np.asarray(v) for k, v in tensors.items()},
                      metadata.to_map() if metadata is not None else None)


def load_lora_checkpoint(path) -> LoraCheckpoint:
    """checkpoint.rs:165-212"""
    tensors, meta = read_safetensors(path)
    return LoraCheckpoint(tensors, LoraMetadata.from_map(meta) if meta else None)


_LLAMA_RENAMES = ((".input_layernorm.", ".operator_norm."),
                  (".post_attention_layernorm.", ".ffn_norm."),
                  (".mlp.", ".feed_forward."))


def legacy_llama_name(name: str) -> Optional[str]:
    """graph/lfm.rs:231-255: the name a Llama-block parameter had in older files."""
    if not name.startswith("model.layers."):
        return None
    for new, old in _LLAMA_RENAMES:
        if new in name:
            return name.replace(new, old, 1)
    return None


def resolve_checkpoint(checkpoint: LoraCheckpoint, expected: Dict[str, List[int]]) -> Dict[str, str]:
    """The all-or-nothing matching of checkpoint.rs:229-282: model name -> checkpoint key.
    `expected` maps every tensor the model wants to its shape."""
    sources: Dict[str, str] = {}
    for name in sorted(expected):
        old = legacy_llama_name(name)
        legacy = old if old is not None and old in checkpoint.tensors else None
        has = name in checkpoint.tensors
        if has and legacy is not None:
            raise CheckpointError(f"checkpoint has both {name} and its old name {legacy}")
        if has:
            key = name
        elif legacy is not None:
            key = legacy
        else:
            raise CheckpointError(f"checkpoint has no tensor {name}")
        shape = checkpoint.tensors[key][0]
        if list(shape) != list(expected[name]):
            raise CheckpointError(f"tensor {key}: checkpoint has shape {list(shape)}, model expects {list(expected[name])}")
        sources[name] = key
    used = set(sources.values())
    unused = sorted(k for k in checkpoint.tensors if k not in used)
    if unused:
        raise CheckpointError(f"checkpoint has {len(unused)} tensor(s) the model does not have, e.g. {unused[0]} "
                              "(a different rank, LoRA targets or --train-modules?)")
    return sources


# ---- training state ------------------------------------------------------------------------
@dataclass
class TrainingState:
    """checkpoint.rs:312-451 (also what `training_state.json` holds)."""
    step: int = 0
    total_steps: int = 0
    best_loss: Optional[float] = None
    lr: float = 0.0
    epoch: int = 0
    batch_size: int = 1
    grad_accum_steps: int = 1
    sequence_length: int = 128
    fp16: bool = False
    train_modules: str = "lora"
    task: str = "sft"
    model_path: str = ""
    dataset_path: str = ""
    seed: int = 0
    q4_weights: Optional[dict] = None

    @staticmethod
    def new(total_steps: int) -> "TrainingState":
        return TrainingState(total_steps=total_steps)

    def to_json_obj(self) -> dict:
        d = {"step": self.step, "total_steps": self.total_steps, "best_loss": self.best_loss,
             "lr": self.lr, "epoch": self.epoch, "batch_size": self.batch_size,
             "grad_accum_steps": self.grad_accum_steps, "sequence_length": self.sequence_length,
             "fp16": self.fp16, "train_modules": self.train_modules, "task": self.task,
             "model_path": self.model_path, "dataset_path": self.dataset_path, "seed": self.seed}
        if self.q4_weights is not None:   # skip_serializing_if = "Option::is_none"
            d["q4_weights"] = self.q4_weights
        return d

    @staticmethod
    def from_json_obj(d: dict) -> "TrainingState":
        try:
            return TrainingState(
                step=int(d["step"]), total_steps=int(d["total_steps"]), best_loss=d["best_loss"],
                lr=float(d["lr"]), epoch=int(d["epoch"]), batch_size=int(d["batch_size"]),
                grad_accum_steps=int(d["grad_accum_steps"]), sequence_length=int(d["sequence_length"]),
                fp16=bool(d["fp16"]), train_modules=str(d["train_modules"]),
                task=str(d.get("task", "sft")), model_path=str(d.get("model_path", "")),
                dataset_path=str(d.get("dataset_path", "")), seed=int(d.get("seed", 0)),
                q4_weights=d.get("q4_weights"))
        except KeyError as e:
            raise CheckpointError(f"training state lacks field {e}") from e

    def save(self, path) -> None:
        Path(path).write_text(json.dumps(self.to_json_obj(), indent=2))

    @staticmethod
    def load(path) -> "TrainingState":
        return TrainingState.from_json_obj(json.loads(Path(path).read_text()))

    def validate_resume(self, train_modules: str, task: str, sequence_length: int, model_path: str) -> None:
        """checkpoint.rs:414-449; raises with the reference's message."""
        if self.train_modules and self.train_modules != train_modules:
            raise CheckpointError(f"checkpoint train_modules `{self.train_modules}` != requested `{train_modules}`")
        if self.task and self.task != task:
            raise CheckpointError(f"checkpoint task `{self.task}` != requested `{task}`")
        if self.sequence_length != 0 and self.sequence_length != sequence_length:
            raise CheckpointError(f"checkpoint sequence_length `{self.sequence_length}` != requested `{sequence_length}`")
        if self.model_path and self.model_path != model_path:
            raise CheckpointError(f"checkpoint model_path `{self.model_path}` != requested `{model_path}`")


@dataclass
class OptimizerTensorState:
    """autograd/lib.rs:1444-1451"""
    shape: List[int]
    data: np.ndarray   # f32, row-major; empty when the values live in the moments file


@dataclass
class AdamWCheckpoint:
    """autograd/lib.rs:1453-1472"""
    lr: float
    beta1: float
    beta2: float
    eps: float
    weight_decay: float
    t: float
    m_states: Dict[str, OptimizerTensorState] = field(default_factory=dict)
    v_states: Dict[str, OptimizerTensorState] = field(default_factory=dict)


@dataclass
class GradScalerCheckpoint:
    """trainer/scaler.rs:54-70"""
    scale: float
    growth_factor: float
    backoff_factor: float
    growth_interval: int
    consecutive_good_steps: int
    found_overflow: bool
    enabled: bool


MOMENTS_FORMAT = "ferrotensor-adamw-moments"


def moments_path(path) -> Path:
    """checkpoint.rs:498-503: `x.state.json` -> `x.state.safetensors`."""
    return Path(path).with_suffix(".safetensors")


def _f32_json(x: float) -> float:
    """A Python float that prints like the f32 it came from (serde_json prints the shortest
    digits that round-trip the f32: 1e-4f32 is 0.0001, not 0.00009999999747378752)."""
    return float(np.format_float_positional(np.float32(x), unique=True, trim="0")) if np.isfinite(x) else x


def _states_json(states: Dict[str, OptimizerTensorState], with_data: bool) -> dict:
    return {n: {"shape": [int(d) for d in s.shape],
                "data": [_f32_json(v) for v in np.asarray(s.data, np.float32).ravel()] if with_data else []}
            for n, s in states.items()}


@dataclass
class TrainingCheckpoint:
    """checkpoint.rs:453-496"""
    training_state: TrainingState
    optimizer_state: Optional[AdamWCheckpoint] = None
    grad_scaler_state: Optional[GradScalerCheckpoint] = None

    def _json_obj(self, inline_moments: bool) -> dict:
        opt = None
        if self.optimizer_state is not None:
            a = self.optimizer_state
            opt = {"AdamW": {"lr": _f32_json(a.lr), "beta1": _f32_json(a.beta1), "beta2": _f32_json(a.beta2),
                             "eps": _f32_json(a.eps), "weight_decay": _f32_json(a.weight_decay),
                             "t": _f32_json(a.t),
                             "m_states": _states_json(a.m_states, inline_moments),
                             "v_states": _states_json(a.v_states, inline_moments)}}
        gs = None
        if self.grad_scaler_state is not None:
            g = self.grad_scaler_state
            gs = {"scale": _f32_json(g.scale), "growth_factor": _f32_json(g.growth_factor),
                  "backoff_factor": _f32_json(g.backoff_factor), "growth_interval": int(g.growth_interval),
                  "consecutive_good_steps": int(g.consecutive_good_steps),
                  "found_overflow": bool(g.found_overflow), "enabled": bool(g.enabled)}
        return {"training_state": self.training_state.to_json_obj(), "optimizer_state": opt,
                "grad_scaler_state": gs}

    def save(self, path) -> None:
        """Moments first (they record the step), then the JSON; each through a temporary name."""
        path = Path(path)
        a = self.optimizer_state
        if a is not None and (a.m_states or a.v_states):
            entries = {}
            for prefix, states in (("m/", a.m_states), ("v/", a.v_states)):
                for name, s in states.items():
                    entries[prefix + name] = np.asarray(s.data, np.float32).reshape(s.shape)
            meta = {"format": MOMENTS_FORMAT, "step": str(int(self.training_state.step)), "t": _rust_f32(a.t)}
            write_safetensors(moments_path(path), entries, meta)
        tmp = path.with_name(path.name + ".tmp")
        tmp.write_text(json.dumps(self._json_obj(False), indent=2))
        os.replace(tmp, path)

    @staticmethod
    def load(path) -> "TrainingCheckpoint":
        path = Path(path)
        d = json.loads(path.read_text())
        ts = TrainingState.from_json_obj(d["training_state"])
        opt = None
        if d.get("optimizer_state") is not None:
            o = d["optimizer_state"]["AdamW"]

            def states(m):
                return {n: OptimizerTensorState([int(x) for x in s["shape"]], np.asarray(s["data"], np.float32))
                        for n, s in m.items()}
            opt = AdamWCheckpoint(float(o["lr"]), float(o["beta1"]), float(o["beta2"]), float(o["eps"]),
                                  float(o["weight_decay"]), float(o["t"]), states(o["m_states"]),
                                  states(o["v_states"]))
            missing = any(s.data.size == 0 and int(np.prod(s.shape)) > 0
                          for s in list(opt.m_states.values()) + list(opt.v_states.values()))
            if missing:
                _read_moments(moments_path(path), opt, ts.step)
        gs = None
        if d.get("grad_scaler_state") is not None:
            g = d["grad_scaler_state"]
            gs = GradScalerCheckpoint(float(g["scale"]), float(g["growth_factor"]), float(g["backoff_factor"]),
                                      int(g["growth_interval"]), int(g["consecutive_good_steps"]),
                                      bool(g["found_overflow"]), bool(g["enabled"]))
        return TrainingCheckpoint(ts, opt, gs)


def _read_moments(path: Path, adam: AdamWCheckpoint, step: int) -> None:
    """checkpoint.rs:568-612"""
    try:
        tensors, meta = read_safetensors(path)
    except CheckpointError as e:
        raise CheckpointError(f"cannot read optimizer moments {path}: {e}") from e
    meta = meta or {}
    if meta.get("format") != MOMENTS_FORMAT:
        raise CheckpointError(f"{path} is not an optimizer moments file")
    try:
        saved_step = int(meta.get("step", ""))
    except ValueError:
        saved_step = -1
    try:
        saved_t = np.float32(float(meta.get("t", "nan")))
    except ValueError:
        saved_t = np.float32("nan")
    if saved_step != step or not (saved_t == np.float32(adam.t)):
        raise CheckpointError(f"optimizer moments in {path} are from step {saved_step}, but the checkpoint is at "
                              f"step {step}; the run was probably interrupted while saving")
    for prefix, states in (("m/", adam.m_states), ("v/", adam.v_states)):
        for name, s in states.items():
            key = prefix + name
            if key not in tensors:
                raise CheckpointError(f"{path} has no tensor {key}")
            shape, vals = tensors[key]
            if list(shape) != list(s.shape):
                raise CheckpointError(f"{key} in {path} has shape {list(shape)}, expected {list(s.shape)}")
            s.data = np.ascontiguousarray(vals, np.float32).ravel()


# ---- names ---------------------------------------------------------------------------------
def reference_tensor_name(host_name: str) -> str:
    """`model.layers.0.self_attn.q_proj.lora_a` (the gradient-fixture names the host model uses)
    -> `model.layers.0.self_attn.q_proj.lora_A.weight` (graph/lib.rs:191-202)."""
    if host_name.endswith(".lora_a"):
        return host_name[:-len(".lora_a")] + ".lora_A.weight"
    if host_name.endswith(".lora_b"):
        return host_name[:-len(".lora_b")] + ".lora_B.weight"
    return host_name


def host_tensor_name(ref_name: str) -> str:
    if ref_name.endswith(".lora_A.weight"):
        return ref_name[:-len(".lora_A.weight")] + ".lora_a"
    if ref_name.endswith(".lora_B.weight"):
        return ref_name[:-len(".lora_B.weight")] + ".lora_b"
    return ref_name


def upgrade_optimizer_names(adam, param_names) -> int:
    """Moments stored under old Llama-block names move to the names in `param_names` (reference
    names), so a run started before the rename resumes with its moments
    (ferrotensor-trainer/src/checkpoint.rs:283-307).  Returns how many were renamed."""
    renamed = 0
    for states in (adam.m_states, adam.v_states):
        for name in param_names:
            if name in states:
                continue
            old = legacy_llama_name(name)
            if old is not None and old in states:
                states[name] = states.pop(old)
                renamed += 1
    return renamed


@dataclass
class OptimizerLoad:
    """What `match_moments` found (ferrotensor-autograd/src/lib.rs OptimizerLoad)."""
    matched: int = 0
    missing: int = 0      # parameters without both saved moments
    unused: int = 0       # saved names that took no part


def match_moments(shapes: Dict[str, Tuple[int, ...]], adam) -> Tuple[List[str], OptimizerLoad]:
    """Which saved moments belong to which parameters, without touching a device
    (ferrotensor-autograd/src/lib.rs:1668-1703).  `shapes` maps reference parameter names to
    shapes.  A parameter takes its saved state when BOTH moments are stored under its name; a
    moment whose shape or value count differs from the parameter's is an error."""
    saved = sorted(set(adam.m_states) | set(adam.v_states))
    matched: List[str] = []
    for name in saved:
        shape = shapes.get(name)
        m, v = adam.m_states.get(name), adam.v_states.get(name)
        if shape is None or m is None or v is None:
            continue
        want = 1
        for d in shape:
            want *= int(d)
        for kind, moment in (("first", m), ("second", v)):
            count = int(np.asarray(moment.data).size)
            if tuple(moment.shape) != tuple(shape) or count != want:
                raise CheckpointError(
                    f"saved {kind} moment of {name} has shape {list(moment.shape)} ({count} values), "
                    f"the parameter has shape {list(shape)}")
        matched.append(name)
    return matched, OptimizerLoad(matched=len(matched), missing=len(shapes) - len(matched),
                                  unused=len(saved) - len(matched))
