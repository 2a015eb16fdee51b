"""Llama-style decoder with LoRA adapters on the `cuda` device: weight preparation and the
handle of the fused step driver.

Counterpart of `Lfm2ModelBuilder::build` + `Lfm2Model`
(ferrotensor-graph/src/model_builder.rs:328-339,415-446,623-709; lfm.rs:532-623,714-770):
every Hugging Face `[out, in]` linear is transposed to `[in, out]` and stored as f16 (or
f32), the tied head is a separate transposed copy of the embedding, adapters attach to
linears whose name contains a target string.  All trainable tensors live in ONE flat f32
buffer (with matching gradient / Adam moment buffers) so that the cross-rank sum, the
norm and the optimizer each touch one contiguous range.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib
from ._lib import FtAdamParams, FtModelConfig, call
from .config import LINEARS, LoRaConfig, ModelConfig
from .engine import CudaContext


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(None)


class LoraModel:
    def __init__(self, ctx: CudaContext, cfg: ModelConfig, lora: LoRaConfig,
                 weights: Dict[str, torch.Tensor], adapters: Optional[Dict[str, torch.Tensor]] = None,
                 f16_base: bool = True, checkpoint_blocks: bool = False,
                 lora_head: bool = False):
        self.ctx, self.cfg, self.lora = ctx, cfg, lora
        self.f16_base = f16_base
        dev = ctx.device
        mask = 0
        for i, name in enumerate(LINEARS):
            if lora.targeted(name):
                mask |= 1 << i
        self.lora_mask = mask
        c = FtModelConfig(cfg.vocab, cfg.hidden, cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim,
                          cfg.ffn, cfg.eps, cfg.theta, int(cfg.qkv_bias), lora.rank, lora.alpha,
                          mask, int(lora_head and lora.rank > 0), int(f16_base),
                          int(checkpoint_blocks), float(cfg.attention_dropout))
        handle = C.c_void_p()
        call("ft_model_create", ctx.handle, C.byref(c), C.byref(handle))
        self.handle = handle
        self._keep: List[torch.Tensor] = []   # device tensors the library borrows

        # ---- frozen weights -------------------------------------------------------------
        def f32(name):
            t = weights[name].to(device=dev, dtype=torch.float32).contiguous()
            self._keep.append(t)
            return t

        def linear_in_out(w_out_in: torch.Tensor) -> torch.Tensor:
            """HF [out, in] -> device [in, out], f16 (RNE) or f32, through the library."""
            src = w_out_in.to(device=dev, dtype=torch.float32).contiguous()
            o, i = src.shape
            dst = torch.empty((i, o), device=dev, dtype=torch.float16 if f16_base else torch.float32)
            call("ft_transpose_f32", ctx.handle, _ptr(src), _ptr(dst), o, i, int(f16_base))
            self._keep.append(dst)
            return dst

        self.embed = f32("model.embed_tokens.weight")
        self.final_norm = f32("model.norm.weight")
        head_src = weights["model.embed_tokens.weight"] if cfg.tied else weights["lm_head.weight"]
        self.head = linear_in_out(head_src)
        call("ft_model_set_embedding", handle, _ptr(self.embed), _ptr(self.final_norm),
             _ptr(self.head))
        self.layer_weights = []
        for l in range(cfg.layers):
            pre = f"model.layers.{l}"
            n1 = f32(f"{pre}.input_layernorm.weight")
            n2 = f32(f"{pre}.post_attention_layernorm.weight")
            lins = [linear_in_out(weights[f"{pre}.{name}.weight"]) for name in LINEARS]
            arr = (C.c_void_p * _lib.FT_LINEARS)(*[t.data_ptr() for t in lins])
            if cfg.qkv_bias:
                bs = [f32(f"{pre}.{name}.bias") for name in LINEARS[:3]]
                barr = (C.c_void_p * 3)(*[t.data_ptr() for t in bs])
            else:
                barr = None
            call("ft_model_set_layer", handle, l, _ptr(n1), _ptr(n2), arr, barr)
            self.layer_weights.append(lins)
        ctx.synchronize()  # the f32 staging copies made above may now be released

        # ---- trainable state --------------------------------------------------------------
        n = C.c_size_t()
        call("ft_model_trainable_count", handle, C.byref(n))
        self.trainable = n.value
        size = max(self.trainable, 1)
        self.params = torch.zeros(size, device=dev, dtype=torch.float32)
        self.grads = torch.zeros(size, device=dev, dtype=torch.float32)
        self.adam_m = torch.zeros(size, device=dev, dtype=torch.float32)
        self.adam_v = torch.zeros(size, device=dev, dtype=torch.float32)
        call("ft_model_set_state", handle, _ptr(self.params), _ptr(self.grads), _ptr(self.adam_m),
             _ptr(self.adam_v))
        self._slices: Dict[str, Tuple[int, int, int]] = {}
        for l in range(cfg.layers):
            for i, name in enumerate(LINEARS):
                if (mask >> i) & 1:
                    self._register(f"model.layers.{l}.{name}", l, i)
        if lora_head and lora.rank > 0:
            self._register("lm_head", -1, 0)
        if adapters:
            self.load_adapters(adapters)
        call("ft_model_prepare", handle)
        self.norm_out = torch.zeros(4, device=dev, dtype=torch.float32)
        self._workspace: Optional[torch.Tensor] = None
        self._ws_key = None

    # ---- adapters -------------------------------------------------------------------------
    def _register(self, prefix: str, layer: int, linear: int) -> None:
        for which, suffix in ((0, "lora_a"), (1, "lora_b")):
            off, rows, cols = C.c_size_t(), C.c_int(), C.c_int()
            call("ft_model_adapter_offset", self.handle, layer, linear, which, C.byref(off),
                 C.byref(rows), C.byref(cols))
            self._slices[f"{prefix}.{suffix}"] = (off.value, rows.value, cols.value)

    def _view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        off, rows, cols = self._slices[name]
        return flat[off:off + rows * cols].view(rows, cols)

    def adapter_names(self) -> List[str]:
        return sorted(self._slices)

    def load_adapters(self, adapters: Dict[str, torch.Tensor]) -> None:
        for name in self._slices:
            self._view(self.params, name).copy_(adapters[name].to(self.params.device, torch.float32))
        call("ft_model_params_changed", self.handle)

    def named_lora_params(self) -> Dict[str, torch.Tensor]:
        """name -> view into the flat parameter buffer (lfm.rs:744-770)."""
        return {n: self._view(self.params, n) for n in self.adapter_names()}

    def named_grads(self) -> Dict[str, torch.Tensor]:
        return {n: self._view(self.grads, n) for n in self.adapter_names()}

    def named_moments(self) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
        return ({n: self._view(self.adam_m, n) for n in self.adapter_names()},
                {n: self._view(self.adam_v, n) for n in self.adapter_names()})

    # ---- the step ---------------------------------------------------------------------------
    def workspace_bytes(self, sequences: int, seq_len: int) -> int:
        n = C.c_size_t()
        call("ft_model_workspace_bytes", self.handle, sequences, seq_len, C.byref(n))
        return n.value

    def _ensure_workspace(self, sequences: int, seq_len: int) -> None:
        key = (sequences, seq_len, int(self.ctx.gemm_mode))  # the layout depends on the mode
        if self._ws_key == key:
            return
        need = self.workspace_bytes(sequences, seq_len)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = None
            self._workspace = torch.empty(need, device=self.ctx.device, dtype=torch.uint8)
        call("ft_model_set_workspace", self.handle, _ptr(self._workspace), self._workspace.numel())
        self._ws_key = key

    def zero_grad(self) -> None:
        call("ft_model_zero_grad", self.handle)

    def forward_backward(self, ids: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor,
                         sequences: int, seq_len: int, seed: float, row_loss: torch.Tensor,
                         logits: Optional[torch.Tensor] = None) -> None:
        """One micro-batch on device tensors (ids/targets int32 bit patterns of u32, weights
        f32, row_loss f32 [rows]); LoRA gradients are added into `self.grads`."""
        self._ensure_workspace(sequences, seq_len)
        call("ft_model_forward_backward", self.handle, _ptr(ids), _ptr(targets), _ptr(weights),
             sequences, seq_len, float(seed), _ptr(row_loss), _ptr(logits))

    def set_dropout_seed(self, step_seed: int) -> None:
        """Seed of the next training pass's attention-dropout masks (no effect at dropout 0)."""
        call("ft_model_set_dropout_seed", self.handle, C.c_uint64(step_seed & 0xFFFFFFFFFFFFFFFF))

    def forward_loss(self, ids: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor,
                     sequences: int, seq_len: int, row_loss: torch.Tensor,
                     logits: Optional[torch.Tensor] = None) -> None:
        """The forward half only: row losses (and logits), gradients untouched."""
        self._ensure_workspace(sequences, seq_len)
        call("ft_model_forward_loss", self.handle, _ptr(ids), _ptr(targets), _ptr(weights),
             sequences, seq_len, _ptr(row_loss), _ptr(logits))

    def apply_gradients(self, grad_scale: float, max_norm: Optional[float], adam: FtAdamParams) -> None:
        call("ft_model_apply_gradients", self.handle, float(grad_scale),
             float(max_norm) if max_norm else 0.0, C.byref(adam), _ptr(self.norm_out))

    def allreduce_apply_gradients(self, comm, max_norm: Optional[float], adam: FtAdamParams) -> None:
        """Sum of the gradient buffer over the communicator's ranks, then the same update with
        1/world folded in (`comm` None = a single rank)."""
        call("ft_model_allreduce_apply_gradients", self.handle,
             comm.handle if comm is not None else C.c_void_p(None),
             float(max_norm) if max_norm else 0.0, C.byref(adam), _ptr(self.norm_out))

    def close(self) -> None:
        if self.handle:
            call("ft_model_destroy", self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
